"""B200-native backend for the Inferred-Thoughts hybrid-MoE token loop.

`libitb.so` (hand-written CUDA for sm_100a behind a C ABI, include/itb.h) is the product; this package
holds its build recipe and a thin ctypes host layer that mirrors the reference's backend interface.
"""
__all__ = ["build", "host", "configs"]
