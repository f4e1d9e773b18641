"""CUDA sources of the kernels and the code that builds and loads them."""
