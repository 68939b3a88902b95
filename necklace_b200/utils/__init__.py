"""Small host-side utilities: CLI flags, IP discovery, hook / wrapper bases, timers."""
