"""Convert the reference's own binary test fixtures for this path into .npz golden vectors.

Run once in a checkout that has the reference tree; the .npz outputs are committed so the tests
never need the reference at run time.

    python tests/golden/make_golden.py /path/to/reference

Formats (little-endian), as the reference's loaders read them:
  ITDP (tests/kquant_dots.rs:57-109): magic, u32 version, u32 ggml type, u64 n, u64 rows,
       u32 name_len, name, u64 w_len, weights, n x f32 activation, u64 q_len, ggml's quantised
       activation bytes, rows x f32 generic dots, rows x f32 dispatch dots.
  ITFX (tests/dequantize.rs:32-67): magic, u32 version, u32 type, u64 n, u64 raw_len,
       u32 name_len, name, raw bytes, n x f32 reference values.
"""
import struct
import sys
from pathlib import Path

import numpy as np


def read_itdp(p):
    b = p.read_bytes()
    assert b[:4] == b"ITDP"
    ver, ty, n, rows, name_len = struct.unpack_from("<IIQQI", b, 4)
    assert ver == 1
    o = 4 + 28
    name = b[o:o + name_len].decode(); o += name_len
    (w_len,) = struct.unpack_from("<Q", b, o); o += 8
    w = np.frombuffer(b, np.uint8, w_len, o); o += w_len
    act = np.frombuffer(b, "<f4", n, o); o += 4 * n
    (q_len,) = struct.unpack_from("<Q", b, o); o += 8
    q = np.frombuffer(b, np.uint8, q_len, o); o += q_len
    generic = np.frombuffer(b, "<f4", rows, o); o += 4 * rows
    dispatch = np.frombuffer(b, "<f4", rows, o); o += 4 * rows
    assert o == len(b)
    return dict(ty=ty, n=n, rows=rows, name=name, weights=w, activation=act, qact=q, generic=generic,
                dispatch=dispatch)


def read_itfx(p):
    b = p.read_bytes()
    assert b[:4] == b"ITFX"
    ver, ty, n, raw_len, name_len = struct.unpack_from("<IIQQI", b, 4)
    assert ver == 1
    o = 4 + 28
    name = b[o:o + name_len].decode(); o += name_len
    raw = np.frombuffer(b, np.uint8, raw_len, o); o += raw_len
    ref = np.frombuffer(b, "<f4", n, o); o += 4 * n
    assert o == len(b)
    return dict(ty=ty, n=n, name=name, raw=raw, reference=ref)


def main():
    fx = Path(sys.argv[1]) / "tests" / "fixtures"
    out = Path(__file__).parent
    d = read_itdp(fx / "dot_nvfp4_Qwen3.6-35B-A3B-NVFP4-Q8_0.gguf.itdp")
    np.savez_compressed(out / "dot_nvfp4_q8_0.npz", **d)
    for src, dst in [("q8_0_Qwen3-0.6B-Q8_0.gguf.itfx", "dequant_q8_0_a.npz"),
                     ("q8_0_Qwen_Qwen3.6-35B-A3B-IQ4_XS.gguf.itfx", "dequant_q8_0_b.npz"),
                     ("f16_edge_cases.itfx", "dequant_f16_edges.npz"),
                     ("f32_Qwen3-0.6B-Q8_0.gguf.itfx", "dequant_f32_a.npz"),
                     ("f32_Qwen_Qwen3.6-35B-A3B-IQ4_XS.gguf.itfx", "dequant_f32_b.npz")]:
        np.savez_compressed(out / dst, **read_itfx(fx / src))
    print("wrote", sorted(p.name for p in out.glob("*.npz")))


if __name__ == "__main__":
    main()
