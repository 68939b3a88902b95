"""Trainer operators (per-worker) and services (scheduler / worker state machines)."""
