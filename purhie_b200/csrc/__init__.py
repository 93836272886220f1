"""Hand-written CUDA kernels for sm_100a, compiled on first use and called through ctypes."""
