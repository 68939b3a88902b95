"""Framework layer (PyTorch)."""
