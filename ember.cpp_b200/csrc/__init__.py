"""CUDA sources, their build and the Python side of the kernels."""
