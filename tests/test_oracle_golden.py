"""The CPU oracle against the reference's own golden vectors and restated known-answer tests.

Pins: NVFP4 x Q8_0 dots and the Q8_0 activation quantiser (tests/kquant_dots.rs:274-326 of the
reference), Q8_0 / F16 / F32 dequantisation (tests/dequantize.rs), the format KATs of
src/quant/mod.rs:549-631 and the op KATs of src/ops/naive.rs:889-1284, routing tie tables of
tests/cuda_ops.rs:1273-1390.
"""
import math
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle_py as O

G = Path(__file__).parent / "golden"
L = O.lib()


def test_nvfp4_q8_0_dots_reproduce_ggml_bit_for_bit():
    d = np.load(G / "dot_nvfp4_q8_0.npz")
    n, rows = int(d["n"]), int(d["rows"])
    assert int(d["ty"]) == 40 and n == 2048 and rows == 64
    w = np.ascontiguousarray(d["weights"]).reshape(rows, n // 64 * 36)
    x = np.ascontiguousarray(d["activation"])
    got = np.array([L.orc_vec_dot_nvfp4_q8_0(np.ascontiguousarray(w[r]), x, n) for r in range(rows)], np.float32)
    assert got.view(np.uint32).tolist() == d["generic"].view(np.uint32).tolist()
    assert got.view(np.uint32).tolist() == d["dispatch"].view(np.uint32).tolist()


def test_q8_0_activation_matches_ggml_byte_for_byte():
    d = np.load(G / "dot_nvfp4_q8_0.npz")
    x = np.ascontiguousarray(d["activation"])
    out = np.zeros(x.size // 32 * 34, np.uint8)
    L.orc_q8_0_blocks(x, x.size, out)
    assert out.tobytes() == d["qact"].tobytes()


@pytest.mark.parametrize("name", ["dequant_q8_0_a", "dequant_q8_0_b", "dequant_f16_edges", "dequant_f32_a",
                                  "dequant_f32_b"])
def test_dequantize_is_bit_exact(name):
    d = np.load(G / f"{name}.npz")
    n = int(d["n"])
    out = np.zeros(n, np.float32)
    L.orc_dequantize(int(d["ty"]), np.ascontiguousarray(d["raw"]), out, n)
    ref = d["reference"]
    same = (out.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(out) & np.isnan(ref))
    assert same.all()


def test_f16_round_trip_exhaustive():
    # src/quant/half.rs:153-233: every non-NaN half survives f16 -> f32 -> f16.
    for h in range(0x10000):
        f = L.orc_f16_to_f32(h)
        if math.isnan(f):
            continue
        assert L.orc_f32_to_f16(f) == h
    assert L.orc_f32_to_f16(65520.0) == 0x7c00          # overflow rounds to infinity
    assert L.orc_f32_to_f16(2.0 ** -25) == 0            # half the smallest subnormal ties to even (0)
    assert L.orc_f32_to_f16(1.0 + 2.0 ** -11) == 0x3c00  # tie to even


def test_nvfp4_is_e2m1_times_e4m3_with_split_nibbles():
    e2m1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, 0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    blk = np.zeros(36, np.uint8)
    blk[0], blk[1] = 0x38, 0x40
    for j in range(8):
        blk[4 + j] = j | ((15 - j) << 4)
        blk[12 + j] = j
    got = np.zeros(64, np.float32)
    L.orc_dequantize(40, blk, got, 64)
    for j in range(8):
        assert got[j] == e2m1[j] and got[j + 8] == e2m1[15 - j] and got[16 + j] == 2.0 * e2m1[j]
    assert (got[32:] == 0).all()


def test_ue4m3_decodes_every_code():
    for x in range(256):
        if x == 0xff:
            assert L.orc_ue4m3_to_f32(x) == 240.0
            continue
        c = x & 0x7f
        e, m = c >> 3, c & 7
        want = 0.0 if c in (0, 0x7f) else (m * 2.0 ** -9 * 0.5 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7) * 0.5)
        assert L.orc_ue4m3_to_f32(x) == want, hex(x)
    assert L.orc_ue4m3_to_f32(0x7e) == 224.0


def test_fp32_to_ue4m3_rounds_to_nearest_even_and_saturates():
    value = lambda c: 2.0 * L.orc_ue4m3_to_f32(c)
    for c in range(1, 0x7f):
        assert L.orc_fp32_to_ue4m3_rn(value(c)) == c
    for c in range(1, 0x7e):
        mid = (value(c) + value(c + 1)) / 2
        assert L.orc_fp32_to_ue4m3_rn(mid) == (c if c % 2 == 0 else c + 1)
    assert L.orc_fp32_to_ue4m3_rn(2.0 ** -10) == 0
    assert L.orc_fp32_to_ue4m3_rn(448.0) == 0x7e and L.orc_fp32_to_ue4m3_rn(1e6) == 0x7e
    assert L.orc_fp32_to_ue4m3_rn(0.0) == 0 and L.orc_fp32_to_ue4m3_rn(-1.0) == 0
    assert L.orc_fp32_to_ue4m3_rn(float("nan")) == 0


def test_fp4_activation_recovers_an_exact_block():
    x = np.array([9.0, -6.0, 4.5, -3.0, 2.25, -1.5, 0.75, 0.0, -0.0, 9.0, -9.0, 6.0, 0.75, -0.75, 1.5, 3.0], np.float32)
    sc, codes = np.zeros(1, np.uint8), np.zeros(16, np.uint8)
    L.orc_fp4_activation(x, 16, sc, codes)
    assert sc[0] == 0x3c
    assert codes.tolist() == [7, 8 | 6, 5, 8 | 4, 3, 8 | 2, 1, 0, 0, 7, 8 | 7, 6, 1, 8 | 1, 2, 4]


def test_fp4_dot_equals_dequantised_product():
    # src/quant/mod.rs:683-719: with both sides exactly representable the FP4 dot is the plain product sum.
    rng = np.random.default_rng(5)
    n = 256
    d = np.load(G / "dot_nvfp4_q8_0.npz")
    w = np.ascontiguousarray(d["weights"][: n // 64 * 36])
    wf = np.zeros(n, np.float32)
    L.orc_dequantize(40, w, wf, n)
    mags = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float32)
    x = (mags[rng.integers(0, 8, n)] * rng.choice([-1.0, 1.0], n)).astype(np.float32)
    x[::16] = 6.0  # pin every block's amax so the scale is exactly 1.0
    got = L.orc_vec_dot_nvfp4_fp4(w, x, n)
    want = float(np.dot(wf.astype(np.float64), x.astype(np.float64)))
    assert abs(got - want) <= 1e-5 * max(1.0, abs(want))


def test_rope_kats():
    x = np.array([1, 0, 0, 0], np.float32)
    L.orc_rope_neox(x, 4, 1, 4, 4, 1, 10000.0)
    assert abs(x[0] - math.cos(1.0)) < 1e-6 and abs(x[2] - math.sin(1.0)) < 1e-6 and x[1] == 0.0
    y = np.array([.3, -1.2, 2.0, .7], np.float32); y0 = y.copy()
    L.orc_rope_neox(y, 4, 0, 4, 4, 1, 10000.0)
    assert np.allclose(y, y0, atol=1e-6)
    two = np.array([1, 2, 3, 4, 1, 2, 3, 4], np.float32)
    L.orc_rope_neox(two, 8, 5, 4, 4, 2, 10000.0)
    assert (two[:4] == two[4:]).all()
    # partial rotation leaves the tail untouched
    p = np.arange(8, dtype=np.float32) + 1; p0 = p.copy()
    L.orc_rope_neox(p, 8, 3, 8, 4, 1, 1e7)
    assert (p[4:] == p0[4:]).all() and not (p[:4] == p0[:4]).all()


def test_norm_kats():
    x = np.array([3.0, 4.0], np.float32); w = np.ones(2, np.float32); out = np.zeros(2, np.float32)
    L.orc_rms_norm(x, 2, w, 2, 0.0, out)
    rms = math.sqrt(12.5)
    assert abs(out[0] - 3 / rms) < 1e-6 and abs(out[1] - 4 / rms) < 1e-6
    L.orc_rms_norm(x, 2, np.zeros(2, np.float32), 2, 1e-6, out)
    assert (out == 0).all()
    v = np.array([3.0, 4.0], np.float32)
    L.orc_l2_norm_heads(v, 2, 2, 1e-6)
    assert abs(v[0] - .6) < 1e-6 and abs(v[1] - .8) < 1e-6
    t = np.array([1e-6, 0.0], np.float32)
    L.orc_l2_norm_heads(t, 2, 2, 1e-3)
    assert abs(t[0] - 1e-3) < 1e-9


def test_ssm_conv_is_depthwise_and_reads_oldest_first():
    state = np.array([1, 2, 0, 0], np.float32); x = np.array([3, 0], np.float32)
    w = np.array([100, 10, 1, 100, 10, 1], np.float32); out = np.zeros(2, np.float32)
    L.orc_ssm_conv(state, x, 2, w, 6, 3, out)
    assert abs(out[0] - 123.0 / (1 + math.exp(-123.0))) < 1e-3 and out[1] == 0.0
    assert state.tolist() == [2, 3, 0, 0]


def _delta(q, k, v, alpha, beta, ssm_a, dt, hk, hv, nk, nv, state):
    f = lambda a: np.ascontiguousarray(a, np.float32)
    out = np.zeros(nv * hv, np.float32)
    L.orc_delta_rule(f(q), f(k), f(v), f(alpha), f(beta), f(ssm_a), f(dt), 1, hk, hv, nk, nv, state, out)
    return out


def test_delta_rule_kats():
    k = [.5] * 4; v = [1, 2, 3, 4]
    st = np.zeros(16, np.float32)
    out = _delta(k, k, v, [0], [40], [0], [0], 4, 4, 1, 1, st)
    assert np.allclose(out, np.array(v) * .5, atol=1e-4)           # writes a value it can read back
    again = _delta(k, k, v, [0], [40], [0], [0], 4, 4, 1, 1, st)
    assert np.allclose(out, again, atol=1e-4)                       # corrects rather than accumulates
    dec = _delta(k, k, [0] * 4, [0], [-40], [-1], [0], 4, 4, 1, 1, st)
    assert np.allclose(dec, out * .5, atol=1e-3)                    # forgets at the gate's rate
    q = [1, 0, 0, 1]; vv = [1, 0] * 4
    o = _delta(q, q, vv, [0] * 4, [40] * 4, [0] * 4, [0] * 4, 2, 2, 2, 4, np.zeros(16, np.float32))
    assert o[2] > 0 and abs(o[0] - o[2]) < 1e-6                     # value heads map to key heads by modulo


def test_softmax_and_silu():
    x = np.array([1, 2, 3], np.float32); L.orc_softmax(x, 3, 3)
    assert abs(x.sum() - 1) < 1e-6 and x[2] > x[1] > x[0]
    big = np.array([1000, 1001, 1002], np.float32); L.orc_softmax(big, 3, 3)
    assert np.isfinite(big).all() and abs(big.sum() - 1) < 1e-6
    g = np.array([1, -1], np.float32); L.orc_silu_mul(g, np.array([2, 2], np.float32), 2)
    silu = lambda z: z / (1 + math.exp(-z))
    assert abs(g[0] - silu(1) * 2) < 1e-6 and abs(g[1] - silu(-1) * 2) < 1e-6


def _host_topk(p, n_expert, n_used):
    """The routing rule as written in tests/cuda_ops.rs:1204-1230 of the reference, in numpy f32."""
    ids, ws = [], []
    for row in p.reshape(-1, n_expert):
        pick = []
        for _ in range(n_used):
            best = -1
            for e in range(n_expert):
                if e in pick:
                    continue
                if best < 0 or row[e] > row[best]:
                    best = e
            pick.append(best)
        s = np.float32(0)
        for e in pick:
            s = np.float32(s + row[e])
        denom = max(s, np.float32(6.103515625e-5))
        ids += pick; ws += [np.float32(row[e] / denom) for e in pick]
    return np.array(ids, np.int32), np.array(ws, np.float32)


def routing_tables():
    t = {}
    t["all_equal"] = np.full(256, 1 / 256, np.float32)
    tie = np.full(256, 1e-4, np.float32); tie[[3, 17, 40, 41, 99, 100, 101, 200, 201, 255]] = .05
    t["ten_way_tie_for_8"] = tie
    spike = np.full(256, 1e-42, np.float32); spike[7] = 1.0
    t["spike_denormal_tail"] = spike
    t["below_clamp"] = np.full(256, 1e-7, np.float32)
    t["ascending"] = (np.arange(256, dtype=np.float32) + 1) / np.float32(32896)
    t["descending"] = t["ascending"][::-1].copy()
    return t


@pytest.mark.parametrize("name", list(routing_tables()))
def test_route_tables(name):
    p = routing_tables()[name]
    ids, w = np.zeros(8, np.int32), np.zeros(8, np.float32)
    L.orc_route(p, 256, 256, 8, ids, w)
    wi, ww = _host_topk(p, 256, 8)
    assert ids.tolist() == wi.tolist()
    assert w.view(np.uint32).tolist() == ww.view(np.uint32).tolist()
    if name == "all_equal":
        assert ids.tolist() == list(range(8))
    if name == "ten_way_tie_for_8":
        assert ids.tolist() == [3, 17, 40, 41, 99, 100, 101, 200]


def test_route_top10_of_512_with_12_way_tie():
    p = np.full(512, 1e-5, np.float32); tied = list(range(5, 500, 45))[:12]; p[tied] = .01
    ids, w = np.zeros(10, np.int32), np.zeros(10, np.float32)
    L.orc_route(p, 512, 512, 10, ids, w)
    assert ids.tolist() == tied[:10]


def test_matmul_q8_0_semantics_and_row_selection():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(64).astype(np.float32)
    wf = rng.standard_normal((3, 64)).astype(np.float32)
    blocks = np.zeros((3, 2 * 34), np.uint8)
    for r in range(3):
        L.orc_q8_0_blocks(np.ascontiguousarray(wf[r]), 64, blocks[r])
    out = np.zeros(3, np.float32)
    L.orc_matmul(8, blocks.reshape(-1), 64, 3, x, 64, out, 0)
    exact = wf @ x
    rel = np.abs(out - exact).max() / np.abs(exact).max()
    assert 1e-7 < rel < 0.05          # quantised, and only by quantisation error
    for r in range(3):
        assert out[r] == L.orc_vec_dot_q8_0(np.ascontiguousarray(blocks[r]), x, 64)


def test_moe_finish_order_and_kv_write():
    rows = np.array([[1, 2], [10, 20]], np.float32).reshape(-1)
    out = np.zeros(4, np.float32)
    L.orc_moe_finish(out, 2, 2, rows, np.array([0, 1], np.int32), np.array([.25, .75], np.float32), 2, 2,
                     np.array([4, 8], np.float32), np.array([0.0], np.float32), 0)
    assert out.tolist() == [0, 0, .25 * 1 + .75 * 10 + 4 * .5, .25 * 2 + .75 * 20 + 8 * .5]
    slab = np.zeros(8, np.uint16)
    L.orc_kv_write(slab, 2, np.array([1.0, -2.0, 65520.0], np.float32), 3, 0)
    assert slab.tolist() == [0, 0, 0x3c00, 0xc000, 0x7c00, 0, 0, 0]
    L.orc_kv_write(slab, 0, np.array([1.0, 3.140625], np.float32), 2, 1)
    assert slab[:2].tolist() == [0x3f80, 0x4049]


def test_restated_expf_equals_the_c_library():
    """The kernels' exp is the C library's expf algorithm restated (table-driven exp2 with a cubic polynomial in double), because
    that is what the reference CPU path calls (Rust's f32::exp). The host build of the same code against libm: a few million
    inputs over the whole range, at most a handful of last-bit differences (measured: about 1 in 10^8)."""
    import ctypes as C
    from inferred_thoughts_b200 import host
    L = host.lib()
    L.itb_expf_host.restype = C.c_float
    L.itb_expf_host.argtypes = [C.c_float]
    rng = np.random.default_rng(7)
    x = np.concatenate([rng.uniform(-104, 89, 300_000), rng.uniform(-12, 12, 300_000), rng.normal(0, 1, 100_000),
                        [0.0, -0.0, 88.0, 88.72, 88.73, -87.3, -87.4, -103.9, -104.0, np.inf, -np.inf, 1e-30, -1e-30]]).astype(np.float32)
    want = np.zeros_like(x)
    O.lib().orc_libm(0, x, x.size, want)
    got = np.array([L.itb_expf_host(float(v)) for v in x], np.float32)
    bad = int((want.view(np.uint32) != got.view(np.uint32)).sum())
    assert bad <= 2, f"{bad} of {x.size} differ"
    assert np.isnan(L.itb_expf_host(float("nan")))
