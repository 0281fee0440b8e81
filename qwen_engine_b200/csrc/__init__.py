"""CUDA sources of the kernels and the script that builds them in-tree."""
