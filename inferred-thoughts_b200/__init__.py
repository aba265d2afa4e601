"""B200-native backend for the Inferred-Thoughts hybrid-MoE token loop.

`libitb.so` (hand-written CUDA for sm_100a behind a C ABI, include/itb.h) is the product; this directory holds its
sources (csrc/), its build recipe (build.py) and a thin ctypes host layer that mirrors the reference's backend
interface (host.py). Import it as `inferred_thoughts_b200`.
"""
