"""PyTorch framework layer: parameter / gradient traffic, tensor-parallel layers,
ZeRO helpers, model-part wrappers, flat-memory manager, utilities."""
