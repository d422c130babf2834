"""CUDA sources of the kernel library and the script that builds them."""
