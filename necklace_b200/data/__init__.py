"""Samplers, datasets and multi-process data loaders."""
