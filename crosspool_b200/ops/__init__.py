"""Operators backed by the in-tree sm_100a kernels (no eager fallback on CUDA tensors)."""
