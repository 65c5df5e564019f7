"""CUDA kernels for sm_100a: sources in ../csrc, built on first use."""
