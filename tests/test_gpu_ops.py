"""Op-level parity on the GPU: every seam op through the C ABI against the CPU oracle on the same seeded inputs.

Classes (the reference's discipline, src/ops/cuda/ops/mod.rs:7-30 there): EXACT = equal to the bit (integer
work, quantised matmuls, norms, routing, copies); CLOSE = a derived tolerance (anything through exp(), and the
attention reduction whose summation order differs).
"""
import numpy as np
import pytest

from oracle import oracle_py as O
from tests.util import noise

pytestmark = pytest.mark.gpu
L = O.lib()
EPS = np.finfo(np.float32).eps


@pytest.fixture(scope="module")
def ops():
    from inferred_thoughts_b200 import host
    o = host.B200Ops(0)
    yield o
    o.check()
    o.close()


# Host addresses are the library's handles (weights, KV slabs): an array that has been passed in must stay alive,
# or a later allocation can reuse its address and meet the stale device copy. Same rule as the reference's mmap.
KEEP = []


def keep(a):
    KEEP.append(a)
    return a


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def exact(got, want, what=""):
    bad = np.flatnonzero(bits(got) != bits(want))
    assert bad.size == 0, f"{what}: {bad.size} of {got.size} differ, first at {bad[:4]}: {got.flat[bad[:4]]} vs {want.flat[bad[:4]]}"


def close(got, want, tol, what=""):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    lim = tol * np.maximum(1.0, np.abs(want))
    assert (err <= lim).all(), f"{what}: max err {err.max():.3e} (limit {lim[err.argmax()]:.3e})"


def q8_weights(n_out, n_in, seed):
    w = noise(n_out * n_in, seed, 0.02)
    out = np.zeros(n_out * n_in // 32 * 34, np.uint8)
    L.orc_q8_0_blocks(w, w.size, out)
    return keep(out)


def nvfp4_weights(n_expert, n_out, n_in, seed):
    """Random but valid NVFP4 blocks: scale codes in the normal range, uniform nibbles; plus second scales."""
    rng = np.random.default_rng(seed)
    nb = n_expert * n_out * n_in // 64
    blk = np.zeros((nb, 36), np.uint8)
    blk[:, :4] = rng.integers(0x20, 0x50, (nb, 4))
    blk[:, 4:] = rng.integers(0, 256, (nb, 32))
    scale = (rng.random(n_expert).astype(np.float32) + 0.5) * 1e-3
    return keep(blk.reshape(-1)), keep(scale)


@pytest.mark.parametrize("n_in,n_out,n_tok", [(2048, 96, 1), (4096, 40, 1), (512, 64, 3), (256, 33, 2), (128, 7, 1), (3072, 16, 1), (768, 24, 1),
                                              (2048, 300, 33), (4096, 130, 70), (512, 17, 5), (3072, 144, 32)])
def test_matmul_q8_0_exact(ops, n_in, n_out, n_tok):
    from inferred_thoughts_b200 import host
    wb = q8_weights(n_out, n_in, 10 + n_in)
    x = noise(n_tok * n_in, 11); out = np.zeros(n_tok * n_out, np.float32); want = np.zeros_like(out)
    ops.begin_pass(n_tok)
    ops.matmul(host.Weights(wb, host.Q8_0, n_in, n_out), x, out); ops.host_needs(out); ops.check()
    L.orc_matmul(8, wb, n_in, n_out, x, x.size, want, 0)
    exact(out, want, "Q8_0 matmul")


@pytest.mark.parametrize("n_in,n_out,n_tok", [(512, 256, 150), (2048, 384, 700), (256, 128, 64), (4096, 128, 257)])
def test_matmul_q8_0_as_f16_tensor_core_gemm(n_in, n_out, n_tok):
    """opts dense=f16tc: a many-row Q8_0 matmul as one tcgen05 kind::f16 GEMM over operands dequantised to f16 (weights and the
    Q8_0-quantised activation rows: int8 * block scale, rounded to nearest). Against the oracle's Q8_0 matmul: every operand
    carries a relative rounding of at most 2^-12, so a product at most 2^-11, and the sum of n_in such errors with random signs stays
    within a few times 2^-11 * sqrt(n_in) * the typical product. Checked as: the worst output error against the oracle is below
    0.3 % of the outputs' root mean square (measured 0.12 %; bf16 operands measured 1 %) (an indexing mistake -- a K block, a row group or a token tile in the wrong place -- moves
    outputs by their full size), over ragged token counts (a last tile of 150, 188, 64 and 1 rows) and 1 to 3 row tiles."""
    from inferred_thoughts_b200 import host
    o2 = host.B200Ops(0, "exact=1,dense=f16tc")
    wb = q8_weights(n_out, n_in, 20 + n_in)
    x = noise(n_tok * n_in, 21); out = np.zeros(n_tok * n_out, np.float32); want = np.zeros_like(out)
    o2.begin_pass(n_tok)
    o2.matmul(host.Weights(wb, host.Q8_0, n_in, n_out), x, out); o2.host_needs(out); o2.check()
    L.orc_matmul(8, wb, n_in, n_out, x, x.size, want, 0)
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    err = float(np.abs(out - want).max())
    print(f"f16 GEMM {n_out} x {n_tok} x {n_in}: worst error {err:.3e}, output rms {rms:.3e}")
    assert err <= 0.003 * rms, (err, rms)
    o2.close()


@pytest.mark.parametrize("n_in,n_out,n_tok", [(2048, 64, 1), (512, 48, 2), (256, 16, 1), (128, 9, 3), (768, 8, 1), (2048, 200, 40), (512, 130, 33)])
def test_matmul_nvfp4_dense_exact(ops, n_in, n_out, n_tok):
    from inferred_thoughts_b200 import host
    wb, _ = nvfp4_weights(1, n_out, n_in, 20 + n_in)
    x = noise(n_tok * n_in, 21); out = np.zeros(n_tok * n_out, np.float32); want = np.zeros_like(out)
    ops.begin_pass(n_tok)
    ops.matmul(host.Weights(wb, host.NVFP4, n_in, n_out), x, out); ops.host_needs(out); ops.check()
    L.orc_matmul(40, wb, n_in, n_out, x, x.size, want, 0)
    exact(out, want, "NVFP4 matmul")


def test_matmul_nvfp4_golden_rows(ops):
    """The reference's own fixture rows (real checkpoint bytes) through the GPU kernel."""
    from pathlib import Path
    from inferred_thoughts_b200 import host
    d = np.load(Path(__file__).parent / "golden" / "dot_nvfp4_q8_0.npz")
    wb = keep(np.ascontiguousarray(d["weights"])); x = np.ascontiguousarray(d["activation"])
    out = np.zeros(64, np.float32)
    ops.begin_pass(1)
    ops.matmul(host.Weights(wb, host.NVFP4, 2048, 64), x, out); ops.host_needs(out); ops.check()
    exact(out, d["generic"], "NVFP4 fixture dots")


@pytest.mark.parametrize("n_in,n_out,n_tok", [(2048, 256, 1), (2048, 1, 2), (256, 40, 3)])
def test_matmul_f32_exact_serial(ops, n_in, n_out, n_tok):
    from inferred_thoughts_b200 import host
    w = keep(noise(n_out * n_in, 30, 0.02))
    x = noise(n_tok * n_in, 31); out = np.zeros(n_tok * n_out, np.float32); want = np.zeros_like(out)
    ops.begin_pass(n_tok)
    ops.matmul(host.Weights(w, host.F32, n_in, n_out), x, out); ops.host_needs(out); ops.check()
    L.orc_matmul(0, w.view(np.uint8), n_in, n_out, x, x.size, want, 0)
    exact(out, want, "F32 matmul")


def test_matmul_pair_and_f16(ops):
    from inferred_thoughts_b200 import host
    n_in = 256
    wa = keep(noise(32 * n_in, 40, 0.02)); wb16 = keep(noise(3 * n_in, 41, 0.02).astype(np.float16))
    x = noise(2 * n_in, 42); oa = np.zeros(64, np.float32); ob = np.zeros(6, np.float32)
    ops.begin_pass(2)
    ops.matmul_pair(host.Weights(wa, host.F32, n_in, 32), host.Weights(wb16, host.F16, n_in, 3), x, oa, ob)
    ops.host_needs(oa); ops.host_needs(ob); ops.check()
    wa_ = np.zeros(64, np.float32); wb_ = np.zeros(6, np.float32)
    L.orc_matmul(0, wa.view(np.uint8), n_in, 32, x, x.size, wa_, 0)
    L.orc_matmul(1, wb16.view(np.uint8), n_in, 3, x, x.size, wb_, 0)
    exact(oa, wa_, "pair a"); exact(ob, wb_, "pair b (F16)")


def test_norms_exact(ops):
    x = noise(3 * 2048, 50); w = 1 + noise(2048, 51, 0.02); out = np.zeros_like(x); want = np.zeros_like(x)
    ops.begin_pass(3)
    ops.rms_norm(x, w, 1e-6, out); ops.host_needs(out)
    L.orc_rms_norm(x, x.size, w, 2048, 1e-6, want)
    exact(out, want, "rms_norm")
    h = noise(5 * 4 * 64, 52); hw = 1 + noise(64, 53, 0.02); h2 = h.copy()
    ops.rms_norm_heads(h, hw, 64, 1e-6); ops.host_needs(h)
    L.orc_rms_norm_heads(h2, h2.size, hw, 64, 1e-6)
    exact(h, h2, "rms_norm_heads")
    v = noise(6 * 128, 54); v2 = v.copy()
    ops.l2_norm_heads(v, 128, 1e-6); ops.host_needs(v)
    L.orc_l2_norm_heads(v2, v2.size, 128, 1e-6)
    exact(v, v2, "l2_norm_heads")
    ops.check()


def test_rope_close(ops):
    x = noise(3 * 4 * 64, 60); x2 = x.copy()
    ops.begin_pass(3)
    ops.rope_neox(x, 1234, 64, 16, 4, 1e7); ops.host_needs(x); ops.check()
    L.orc_rope_neox(x2, x2.size, 1234, 64, 16, 4, 1e7)
    close(x, x2, 2 * EPS, "rope")
    assert (bits(x) == bits(x2)).mean() > 0.99


def test_elementwise(ops):
    n = 1000
    a = noise(n, 70); b = noise(n, 71); lg = noise(1, 72)
    ops.begin_pass(1)
    g = a.copy(); g2 = a.copy(); ops.silu_mul(g, b); ops.host_needs(g); L.orc_silu_mul(g2, b, n); close(g, g2, 4 * EPS, "silu_mul")
    s = a.copy(); s2 = a.copy(); ops.sigmoid_mul(s, b); ops.host_needs(s); L.orc_sigmoid_mul(s2, b, n); close(s, s2, 4 * EPS, "sigmoid_mul")
    c = a.copy(); c2 = a.copy(); ops.scale(c, 0.37); ops.host_needs(c); L.orc_scale(c2, n, 0.37); exact(c, c2, "scale")
    d = a.copy(); d2 = a.copy(); ops.add_assign(d, b); ops.host_needs(d); L.orc_add_assign(d2, b, n); exact(d, d2, "add_assign")
    e = a.copy(); e2 = a.copy(); ops.add_scaled(e, b, -1.7); ops.host_needs(e); L.orc_add_scaled(e2, b, n, -1.7); exact(e, e2, "add_scaled")
    f = a.copy(); f2 = a.copy(); ops.add_scaled_sigmoid(f, b, lg); ops.host_needs(f); L.orc_add_scaled_sigmoid(f2, b, n, lg); close(f, f2, 4 * EPS, "add_scaled_sigmoid")
    rows = noise(8 * 256, 73); sc = noise(8, 74); acc = np.zeros(256, np.float32); acc2 = np.zeros(256, np.float32)
    ops.add_scaled_rows(acc, rows, sc); ops.host_needs(acc); L.orc_add_scaled_rows(acc2, 256, rows, sc, 8); exact(acc, acc2, "add_scaled_rows")
    sm = noise(4 * 256, 75, 3.0); sm2 = sm.copy(); ops.softmax(sm, 256); ops.host_needs(sm); L.orc_softmax(sm2, sm2.size, 256); close(sm, sm2, 8 * EPS, "softmax")
    ops.check()


def test_gather_scatter_kv_write(ops):
    src = noise(4 * 96, 80); out = np.zeros(4 * 32, np.float32); want = np.zeros_like(out)
    ops.begin_pass(4)
    ops.gather_chunks(src, 32, 96, 64, out); ops.host_needs(out); L.orc_gather_chunks(src, 32, 96, 64, want, want.size); exact(out, want, "gather")
    dst = noise(4 * 96, 81); dst2 = dst.copy()
    ops.scatter_chunks(out, 32, 96, 5, dst); ops.host_needs(dst); L.orc_scatter_chunks(out, out.size, 32, 96, 5, dst2); exact(dst, dst2, "scatter")
    slab = keep(np.zeros(64 * 8, np.uint16)); slab2 = slab.copy(); kv = noise(3 * 64, 82, 50.0)
    ops.kv_write(slab, 2 * 64, kv); ops.read_kv(slab); L.orc_kv_write(slab2, 2 * 64, kv, kv.size, 0)
    assert (slab == slab2).all()
    ops.check()


def test_bad_shapes_set_the_sticky_error_and_nothing_runs(ops):
    x = noise(100, 90); out = np.zeros(100, np.float32)
    ops.gather_chunks(x, 32, 96, 64, out)           # out is not whole chunks
    assert "gather_chunks" in ops.take_error()
    assert ops.take_error() is None                  # cleared by the take


def test_ssm_conv_and_state(ops):
    nc, kern, nt = 512, 4, 5
    st = keep(noise(nc * 3, 100)); st2 = st.copy(); x = noise(nt * nc, 101); w = noise(nc * kern, 102, 0.5)
    out = np.zeros_like(x); want = np.zeros_like(x)
    ops.begin_pass(nt)
    ops.ssm_conv(st, x, w, kern, out); ops.host_needs(out); ops.read_state(st); ops.check()
    L.orc_ssm_conv(st2, x, x.size, w, w.size, kern, want)
    close(out, want, 4 * EPS, "ssm_conv")
    exact(st, st2, "conv window left behind")
    ops.forget_state()


@pytest.mark.parametrize("sk,nk,nv,nt", [(128, 16, 32, 1), (64, 2, 4, 6), (128, 16, 48, 2)])
def test_delta_rule_and_state(ops, sk, nk, nv, nt):
    q = noise(nt * nk * sk, 110, 0.1); k = noise(nt * nk * sk, 111, 0.1); v = noise(nt * nv * sk, 112)
    al = noise(nt * nv, 113); be = noise(nt * nv, 114); sa = -np.abs(noise(nv, 115)); dt = noise(nv, 116, 0.02)
    st = keep(noise(nv * sk * sk, 117, 0.1)); st2 = st.copy()
    out = np.zeros(nt * nv * sk, np.float32); want = np.zeros_like(out)
    ops.begin_pass(nt)
    ops.delta_rule(q, k, v, al, be, sa, dt, sk, sk, nk, nv, st, out); ops.host_needs(out); ops.read_state(st); ops.check()
    L.orc_delta_rule(q, k, v, al, be, sa, dt, nt, sk, sk, nk, nv, st2, want)
    # the reference holds its device kernel to 40 eps including the state left behind (tests/cuda_ops.rs:863-950 there)
    scale = max(1.0, float(np.abs(want).max()))
    assert np.abs(out - want).max() <= 40 * EPS * scale
    assert np.abs(st - st2).max() <= 40 * EPS * max(1.0, float(np.abs(st2).max()))
    ops.forget_state()


def test_route_exact_including_tie_tables(ops):
    from tests.test_oracle_golden import routing_tables
    tables = list(routing_tables().values())
    rng = np.random.default_rng(120)
    for _ in range(6):
        lg = rng.standard_normal(256).astype(np.float32) * 3; e = np.exp(lg - lg.max()); tables.append((e / e.sum()).astype(np.float32))
    probs = np.concatenate(tables).astype(np.float32)
    ops.begin_pass(len(tables))
    r = ops.route(probs, 256, 8); ids, w = ops.read_route(r); ops.check()
    wi = np.zeros(len(tables) * 8, np.int32); ww = np.zeros(len(tables) * 8, np.float32)
    L.orc_route(probs, probs.size, 256, 8, wi, ww)
    assert ids.tolist() == wi.tolist()
    exact(w, ww, "route weights")
    p512 = np.full(512, 1e-5, np.float32); tied = list(range(5, 500, 45))[:12]; p512[tied] = .01
    r = ops.route(p512, 512, 10); ids, _ = ops.read_route(r)
    assert ids.tolist() == tied[:10]


def _zipf_logits(n_tok, n_expert, seed, s=1.1):
    """Router logits whose softmax is Zipf(s) over a per-token random ranking of the experts (BASELINE config 2's skew)."""
    rng = np.random.default_rng(seed)
    base = (-s * np.log(np.arange(1, n_expert + 1))).astype(np.float32)
    return keep(np.concatenate([base[rng.permutation(n_expert)] for _ in range(n_tok)]).astype(np.float32))


@pytest.fixture(scope="module")
def cfg2_experts():
    """BASELINE config 2's stack: hidden 2048, expert FFN 512, 256 experts, top-8."""
    H, ff, E = 2048, 512, 256
    g = nvfp4_weights(E, ff, H, 140); u = nvfp4_weights(E, ff, H, 141); d = nvfp4_weights(E, H, ff, 142)
    for _, sc in (g, u, d):
        sc *= 300
    return H, ff, E, 8, g, u, d


@pytest.mark.parametrize("n_tok", [1, 8, 32, 200])
def test_grouped_expert_matmuls_config2_exact(ops, cfg2_experts, n_tok):
    """gate/up/SiLU and down over Zipf-skewed routing at the microbenchmark's shapes: 1 and 8 tokens take the per-pair
    dequant-and-dot kernels, 32 and 200 the expert-grouped int8-MMA tiles (8- and 16-token tiles); routing ids bit-exact,
    the down matmul bit-exact on the same inputs, gate/up within the exp tolerance."""
    from inferred_thoughts_b200 import host
    H, ff, E, K, (gb, gs), (ub, us), (db, ds) = cfg2_experts
    x = noise(n_tok * H, 143)
    probs = _zipf_logits(n_tok, E, 2).copy(); L.orc_softmax(probs, probs.size, E)
    want_ids = np.zeros(n_tok * K, np.int32); want_w = np.zeros(n_tok * K, np.float32)
    L.orc_route(probs.copy(), probs.size, E, K, want_ids, want_w)
    ops.begin_pass(n_tok)
    route = ops.route(probs, E, K); ids, wts = ops.read_route(route)
    assert ids.tolist() == want_ids.tolist()
    h = keep(np.zeros(n_tok * K * ff, np.float32)); scratch = keep(np.zeros_like(h)); o = keep(np.zeros(n_tok * K * H, np.float32))
    G, U, D = host.Experts(gb, host.NVFP4, H, ff, E, gs), host.Experts(ub, host.NVFP4, H, ff, E, us), host.Experts(db, host.NVFP4, ff, H, E, ds)
    ops.moe_glu(G, U, route, x, h, scratch)
    ops.matmul_experts(D, route, h, o)
    ops.host_needs(h); ops.host_needs(o); ops.check()
    h_want = np.zeros_like(h); o_want = np.zeros_like(o)
    L.orc_moe_glu(gb, gs.ctypes.data, ub, us.ctypes.data, H, ff, E, ids, ids.size, K, x, x.size, h_want, 0)
    close(h, h_want, 8 * EPS, "moe_glu (through silu)")
    L.orc_matmul_experts(db, ff, H, E, ds.ctypes.data, ids, ids.size, K, h, h.size, o_want, 0)
    exact(o, o_want, "matmul_experts(down)")


def test_grouped_expert_matmuls_at_8192_tokens_repeat_the_small_case(ops, cfg2_experts):
    """At the microbenchmark's largest size the CPU check is too slow; instead 8,192 tokens made of 16 copies of 512 distinct
    ones must give 16 copies of the 512-token result (the tiles are 64 tokens wide there, 16 wide at 512 tokens)."""
    from inferred_thoughts_b200 import host
    H, ff, E, K, (gb, gs), (ub, us), (db, ds) = cfg2_experts
    G, U, D = host.Experts(gb, host.NVFP4, H, ff, E, gs), host.Experts(ub, host.NVFP4, H, ff, E, us), host.Experts(db, host.NVFP4, ff, H, E, ds)
    outs = []
    for reps in (1, 16):
        n_tok = 512 * reps
        x = keep(np.tile(noise(512 * H, 144), reps)); probs = keep(np.tile(_zipf_logits(512, E, 3), reps)); L.orc_softmax(probs, probs.size, E)
        ops.begin_pass(n_tok)
        route = ops.route(probs, E, K)
        h = keep(np.zeros(n_tok * K * ff, np.float32)); scratch = keep(np.zeros_like(h)); o = keep(np.zeros(n_tok * K * H, np.float32))
        ops.moe_glu(G, U, route, x, h, scratch)
        ops.matmul_experts(D, route, h, o)
        ops.host_needs(o); ops.check()
        outs.append(o)
    small = outs[0].view(np.uint32)
    for i, part in enumerate(outs[1].view(np.uint32).reshape(16, -1)):
        assert (part == small).all(), f"copy {i} differs from the 512-token result"


@pytest.mark.parametrize("n_tok", [1, 3])
def test_routed_experts_exact(ops, n_tok):
    from inferred_thoughts_b200 import host
    H, ff, E, K = 256, 128, 16, 4
    gb, gs = nvfp4_weights(E, ff, H, 130); ub, us = nvfp4_weights(E, ff, H, 131); db, ds = nvfp4_weights(E, H, ff, 132)
    gs *= 300; us *= 300; ds *= 300
    x = noise(n_tok * H, 133)
    lg = noise(n_tok * E, 134, 2.0); probs = lg.copy(); L.orc_softmax(probs, probs.size, E)
    ops.begin_pass(n_tok)
    route = ops.route(probs, E, K); ids, wts = ops.read_route(route)
    h = np.zeros(n_tok * K * ff, np.float32); scratch = np.zeros_like(h); o = np.zeros(n_tok * K * H, np.float32)
    G, U, D = host.Experts(gb, host.NVFP4, H, ff, E, gs), host.Experts(ub, host.NVFP4, H, ff, E, us), host.Experts(db, host.NVFP4, ff, H, E, ds)
    ops.moe_glu(G, U, route, x, h, scratch)
    ops.matmul_experts(D, route, h, o)
    shared = noise(n_tok * H, 135); logit = noise(n_tok, 136); out = noise(2 * H + n_tok * H, 137); out2 = out.copy()
    ops.moe_finish(out, 2 * H, H, o, route, shared, logit, 0)
    ops.host_needs(h); ops.host_needs(o); ops.host_needs(out); ops.check()
    gp, up_, dp = (a.ctypes.data for a in (gs, us, ds))
    h_want = np.zeros_like(h); o_want = np.zeros_like(o)
    L.orc_moe_glu(gb, gp, ub, up_, H, ff, E, ids, ids.size, K, x, x.size, h_want, 0)
    close(h, h_want, 8 * EPS, "moe_glu (through silu)")
    L.orc_matmul_experts(db, ff, H, E, dp, ids, ids.size, K, h, h.size, o_want, 0)   # on the GPU's h: isolates the down matmul
    exact(o, o_want, "matmul_experts(down)")
    L.orc_moe_finish(out2, 2 * H, H, o, ids, wts, ids.size, K, shared, logit, 0)
    close(out, out2, 4 * EPS, "moe_finish")
    # a host-built route must be honoured too (src/ops/cuda/ops/moe.rs:878-921 there)
    hr = host.Route.host(ids[::-1].astype(np.uint64), None, K)
    o2 = np.zeros_like(o); ops.matmul_experts(D, hr, h, o2); ops.host_needs(o2); ops.check()
    o2_want = np.zeros_like(o); rid = np.ascontiguousarray(ids[::-1])
    L.orc_matmul_experts(db, ff, H, E, dp, rid, rid.size, K, h, h.size, o2_want, 0)
    exact(o2, o2_want, "host route")


@pytest.mark.parametrize("hd,nh,nkv,n_pos,n_q", [(256, 16, 2, 700, 1), (64, 4, 1, 40, 1), (64, 4, 1, 33, 7), (128, 8, 2, 300, 3), (256, 16, 2, 5000, 1)])
def test_attend_close(ops, hd, nh, nkv, n_pos, n_q):
    kvd = hd * nkv; n_ctx = n_pos + 8
    q = noise(n_q * nh * hd, 140)
    kf = noise(n_ctx * kvd, 141); vf = noise(n_ctx * kvd, 142)
    ks = keep(np.zeros(n_ctx * kvd, np.uint16)); vs = keep(np.zeros_like(ks))
    L.orc_kv_write(ks, 0, kf, kf.size, 0); L.orc_kv_write(vs, 0, vf, vf.size, 0)
    out = np.zeros(n_q * nh * hd, np.float32); want = np.zeros_like(out)
    scale = 1.0 / np.sqrt(hd)
    ops.begin_pass(n_q)
    ops.attend(q, ks, vs, kvd, n_pos, hd, nh, nkv, scale, out); ops.host_needs(out); ops.check()
    L.orc_attend(q, q.size, ks, vs, kvd, n_pos, hd, nh, nkv, scale, 0, want)
    # derived bound in the style of the reference's attend_tolerance (tests/cuda_ops.rs:178-183 there):
    # a handful of roundings per merge step times the largest value
    tol = (7 + 64 + 4 + np.log2(n_pos)) * EPS * float(np.abs(vf).max()) * 4
    assert np.abs(out - want).max() <= tol, (np.abs(out - want).max(), tol)


def test_synth_generator_matches_cpu_bit_for_bit(ops):
    key = L.orc_tensor_key(3, b"blk.7.ffn_gate_exps.weight")
    for dist, sd in ((0, 0.02), (1, 0.02), (2, 1.0)):
        got = ops.synth_values(key, 12345, 4096, dist, sd)
        want = np.array([L.orc_synth_value(key, 12345 + i, dist, sd) for i in range(4096)], np.float32)
        exact(got, want, f"synth dist {dist}")
    assert abs(float(np.std(ops.synth_values(key, 0, 1 << 16, 0, 1.0))) - 1.0) < 0.02


def test_exp_and_log_follow_the_c_library():
    """exp and log as every kernel computes them against the C library the CPU path calls: exp by the restated library algorithm,
    log by the correction table built from the host's logf (softplus asks for log(1 + e^a), a <= 20: arguments in [1, 4.9e8))."""
    import ctypes as C
    from inferred_thoughts_b200 import host
    from oracle import oracle_py as O
    ops = host.B200Ops(0)
    L = host.lib()
    rng = np.random.default_rng(8)
    a = np.concatenate([rng.uniform(-30, 20, 2_000_000), rng.normal(0, 2, 2_000_000)]).astype(np.float32)
    want_e = np.zeros_like(a); got_e = np.zeros_like(a)
    O.lib().orc_libm(0, a, a.size, want_e)
    assert L.itb_eval_unary(ops.h, 0, C.c_void_p(a.ctypes.data), C.c_size_t(a.size), C.c_void_p(got_e.ctypes.data)) == 0
    bad = int((want_e.view(np.uint32) != got_e.view(np.uint32)).sum())
    assert bad <= 2, f"exp: {bad} of {a.size} differ"
    x = (np.float32(1.0) + want_e).astype(np.float32)
    x = x[x < np.float32(2.0 ** 29)]
    want_l = np.zeros_like(x); got_l = np.zeros_like(x)
    O.lib().orc_libm(1, x, x.size, want_l)
    assert L.itb_eval_unary(ops.h, 1, C.c_void_p(x.ctypes.data), C.c_size_t(x.size), C.c_void_p(got_l.ctypes.data)) == 0
    bad = int((want_l.view(np.uint32) != got_l.view(np.uint32)).sum())
    assert bad <= 2, f"log: {bad} of {x.size} differ"
    ops.check(); ops.close()


@pytest.mark.parametrize("hd,nh,nkv,n_pos,n_q", [(256, 16, 2, 700, 1), (64, 4, 1, 100, 3), (128, 6, 2, 333, 2), (256, 32, 4, 1500, 1)])
def test_attend_in_exact_mode_equals_the_cpu_path_bit_for_bit(hd, nh, nkv, n_pos, n_q):
    """exact=1: scores, softmax and weighted values in the CPU path's own order (src/ops/naive.rs:420-466 there)."""
    from inferred_thoughts_b200 import host
    from oracle import oracle_py as O
    ops = host.B200Ops(0, "exact=1")
    kvd = hd * nkv
    q = noise(n_q * nh * hd, 70)
    ks = noise(n_pos * kvd, 71).astype(np.float16).view(np.uint16)
    vs = noise(n_pos * kvd, 72).astype(np.float16).view(np.uint16)
    scale = np.float32(1.0 / np.sqrt(hd))
    want = np.zeros(n_q * nh * hd, np.float32); got = np.zeros_like(want)
    O.lib().orc_attend(q, q.size, ks, vs, kvd, n_pos, hd, nh, nkv, scale, 0, want)
    ops.begin_pass(n_q)
    ops.attend(q, ks, vs, kvd, n_pos, hd, nh, nkv, float(scale), got); ops.host_needs(got); ops.check()
    assert got.view(np.uint32).tolist() == want.view(np.uint32).tolist(), float(np.abs(got - want).max())
    ops.close()


def test_fp4_tensor_core_ceiling_runs_and_verifies_its_accumulators():
    """tcgen05.mma kind::mxf4nvf4 with unchanging operands (every value 1.0, every scale 1.0): each accumulator must end at
    64 * iters exactly; the rate is the denominator of the expert GEMMs' roofline fraction."""
    from inferred_thoughts_b200 import host
    ops = host.B200Ops(0)
    for n in (128, 256):
        tflops, status, cycles = ops.fp4_ceiling(n=n, iters=2000, reps=3)
        print(f"FP4 ceiling N={n}: {tflops:.0f} TFLOP/s dense, {cycles:.1f} cycles per MMA")
        assert status == 0, status
        assert tflops > 500.0
    ops.check(); ops.close()


def test_fp4_activation_quantiser_equals_the_cpu_record_bit_for_bit(ops):
    """The tensor-core path's activation quantiser against Fp4Row::from_f32 as the oracle restates it: scale codes and
    element codes equal, over ordinary rows, tiny and huge magnitudes, zeros, ties and a saturating block."""
    rng = np.random.default_rng(7)
    parts = [noise(16 * 4096, 150), noise(16 * 512, 151, 1e-4), noise(16 * 512, 152, 300.0), np.zeros(64, np.float32),
             np.tile(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0], np.float32), 8),
             (rng.standard_normal(16 * 256) * 10.0 ** rng.uniform(-6, 4, 16 * 256)).astype(np.float32),
             np.full(32, 5000.0, np.float32)]
    x = np.ascontiguousarray(np.concatenate(parts), np.float32)
    sc, q = ops.fp4_quantize(x)
    want_sc = np.zeros(x.size // 16, np.uint8); want_q = np.zeros(x.size, np.uint8)
    L.orc_fp4_activation(x, x.size, want_sc, want_q)
    bad = np.flatnonzero(sc != want_sc)
    assert bad.size == 0, f"{bad.size} scale codes differ, first block {bad[:4]}: {sc[bad[:4]]} vs {want_sc[bad[:4]]}"
    bad = np.flatnonzero(q != want_q)
    assert bad.size == 0, f"{bad.size} element codes differ, first at {bad[:4]}: {q[bad[:4]]} vs {want_q[bad[:4]]}"


def _fp4tc_case(tc, H, ff, E, K, n_tok, seed, x=None, zipf=False):
    """moe_glu + down through experts=fp4tc against the oracle with FP4 activations. Returns (h, h_want, o, o_want)."""
    from inferred_thoughts_b200 import host
    (gb, gs), (ub, us), (db, ds) = nvfp4_weights(E, ff, H, seed), nvfp4_weights(E, ff, H, seed + 1), nvfp4_weights(E, H, ff, seed + 2)
    for s in (gs, us, ds):
        s *= 300
    x = keep(noise(n_tok * H, seed + 3) if x is None else np.ascontiguousarray(x, np.float32))
    probs = _zipf_logits(n_tok, E, seed) if zipf else keep(noise(n_tok * E, seed + 4, 2.0))
    probs = keep(probs.copy()); L.orc_softmax(probs, probs.size, E)
    tc.begin_pass(n_tok)
    route = tc.route(probs, E, K); ids, _ = tc.read_route(route)
    h = keep(np.zeros(n_tok * K * ff, np.float32)); scratch = keep(np.zeros_like(h)); o = keep(np.zeros(n_tok * K * H, np.float32))
    G, U, D = host.Experts(gb, host.NVFP4, H, ff, E, gs), host.Experts(ub, host.NVFP4, H, ff, E, us), host.Experts(db, host.NVFP4, ff, H, E, ds)
    tc.moe_glu(G, U, route, x, h, scratch)
    tc.matmul_experts(D, route, h, o)
    tc.host_needs(h); tc.host_needs(o); tc.check()
    h_want = np.zeros_like(h); o_want = np.zeros_like(o)
    L.orc_moe_glu(gb, gs.ctypes.data, ub, us.ctypes.data, H, ff, E, ids, ids.size, K, x, x.size, h_want, 1)
    L.orc_matmul_experts(db, ff, H, E, ds.ctypes.data, ids, ids.size, K, h, h.size, o_want, 1)   # on the GPU's h: isolates the down matmul
    return h.reshape(n_tok * K, ff), h_want.reshape(n_tok * K, ff), o.reshape(n_tok * K, H), o_want.reshape(n_tok * K, H)


def _rel_err(got, want):
    """Largest error of a row relative to that row's largest magnitude (accumulation-order class)."""
    scale = np.maximum(np.abs(want).max(axis=1, keepdims=True), 1e-20)
    return float((np.abs(got.astype(np.float64) - want) / scale).max())


FP4TC_TOL = 2e-5     # f32 accumulation in another order over <= 2048 products of like magnitude


@pytest.mark.parametrize("H,ff,E,K,n_tok,zipf", [(256, 256, 4, 2, 5, False), (512, 256, 16, 4, 40, False), (2048, 512, 256, 8, 200, True),
                                                   (2048, 512, 8, 2, 700, False)])
def test_routed_experts_on_the_fp4_tensor_cores(H, ff, E, K, n_tok, zipf):
    """experts=fp4tc: FP4 activations (bit-identical quantiser) times FP4 weights by tcgen05.mma kind::mxf4nvf4 against the
    CPU statement of the same arithmetic (dot_nvfp4_fp4): the products are exact in both, only the f32 summation order inside
    the tensor core differs. Cases: one ragged tile per expert, several experts, the microbenchmark's stack with Zipf routing,
    and experts whose pairs span several 128-token tiles."""
    from inferred_thoughts_b200 import host
    tc = host.B200Ops(0, "experts=fp4tc")
    h, h_want, o, o_want = _fp4tc_case(tc, H, ff, E, K, n_tok, 160 + n_tok, zipf=zipf)
    eh, eo = _rel_err(h, h_want), _rel_err(o, o_want)
    print(f"fp4tc H={H} ff={ff} E={E} n_tok={n_tok}: gate/up rel err {eh:.2e}, down rel err {eo:.2e}")
    assert eh <= 4 * FP4TC_TOL, eh          # through silu(gate) * up: both factors carry the order error
    assert eo <= FP4TC_TOL, eo
    tc.check(); tc.close()


@pytest.mark.parametrize("nk,nv,nt,corr", [(2, 4, 64, 0.0), (2, 4, 150, 0.0), (16, 32, 200, 0.0), (2, 4, 150, 0.8), (2, 2, 33, 0.8)])
def test_chunk_parallel_delta_rule_against_the_serial_order(nk, nv, nt, corr):
    """gdn=chunk: the delta rule as chunk-parallel matrix products against the CPU path's token-by-token recurrence, outputs and
    the state left behind. Same f32 arithmetic, another association: held to 2e-4 of the largest magnitude (the recurrence
    compounds rounding over the tokens of a call). Cases: one full chunk, ragged last chunks, the benchmark's head counts, and
    keys that are strongly correlated inside a chunk (corr: the weight of a shared direction; the model's keys pass through
    SiLU and are mostly positive), normalised like the model's."""
    from inferred_thoughts_b200 import host
    sk = 128
    ops = host.B200Ops(0, "gdn=chunk")
    rng = np.random.default_rng(900 + nt)

    def unit(x):
        x = x.reshape(-1, sk)
        return np.ascontiguousarray(x / np.maximum(np.linalg.norm(x, axis=1, keepdims=True), 1e-6), np.float32).reshape(-1)
    shared = rng.standard_normal(sk).astype(np.float32)
    q = unit(noise(nt * nk * sk, 310, 1.0).reshape(-1, sk) + 3 * corr * shared)
    k = unit(noise(nt * nk * sk, 311, 1.0).reshape(-1, sk) + 3 * corr * shared)
    v = noise(nt * nv * sk, 312)
    al = noise(nt * nv, 313); be = noise(nt * nv, 314); sa = -np.abs(noise(nv, 315)); dt = noise(nv, 316, 0.02)
    st = keep(noise(nv * sk * sk, 317, 0.1)); st2 = st.copy()
    out = np.zeros(nt * nv * sk, np.float32); want = np.zeros_like(out)
    ops.begin_pass(nt)
    ops.delta_rule(q, k, v, al, be, sa, dt, sk, sk, nk, nv, st, out); ops.host_needs(out); ops.read_state(st); ops.check()
    L.orc_delta_rule(q, k, v, al, be, sa, dt, nt, sk, sk, nk, nv, st2, want)
    eo = float(np.abs(out - want).max()) / max(1.0, float(np.abs(want).max()))
    es = float(np.abs(st - st2).max()) / max(1.0, float(np.abs(st2).max()))
    print(f"chunked delta rule nk={nk} nv={nv} nt={nt} corr={corr}: output err {eo:.2e}, state err {es:.2e}")
    assert eo <= 2e-4 and es <= 2e-4
    ops.forget_state(); ops.close()


@pytest.mark.parametrize("hd,nh,nkv,n_pos,n_q,kv", [(256, 16, 2, 700, 150, "f16"), (256, 16, 2, 700, 150, "bf16"), (64, 4, 1, 200, 200, "f16"),
                                                    (128, 8, 2, 333, 77, "f16"), (256, 32, 4, 130, 16, "bf16")])
def test_tensor_core_attention_against_the_cpu_order(hd, nh, nkv, n_pos, n_q, kv):
    """attn=mma at op level: n_q consecutive query rows deep in a cache of n_pos positions (row i sees n_pos - n_q + 1 + i of
    them) through the many-token kernel, against the CPU path. q and the softmax weights are rounded to the cache's 16-bit
    type (2^-11 relative for f16, 2^-8 for bf16) before their matrix products, so the bound is that rounding times the
    largest value, with head room for the sums' association; ragged last tiles in tokens and positions, 4 and 8 heads per
    KV head, every head_dim."""
    from inferred_thoughts_b200 import host
    bf = kv == "bf16"
    ops = host.B200Ops(0, "attn=mma" + (",kv=bf16" if bf else ""))
    kvd = hd * nkv; n_ctx = n_pos + 8
    q = noise(n_q * nh * hd, 440)
    kf = noise(n_ctx * kvd, 441); vf = noise(n_ctx * kvd, 442)
    ks = keep(np.zeros(n_ctx * kvd, np.uint16)); vs = keep(np.zeros_like(ks))
    L.orc_kv_write(ks, 0, kf, kf.size, int(bf)); L.orc_kv_write(vs, 0, vf, vf.size, int(bf))
    out = np.zeros(n_q * nh * hd, np.float32); want = np.zeros_like(out)
    scale = 1.0 / np.sqrt(hd)
    ops.begin_pass(n_q)
    ops.attend(q, ks, vs, kvd, n_pos, hd, nh, nkv, scale, out); ops.host_needs(out); ops.check()
    L.orc_attend(q, q.size, ks, vs, kvd, n_pos, hd, nh, nkv, scale, int(bf), want)
    err = float(np.abs(out - want).max()); tol = (2.0 ** -8 if bf else 2.0 ** -11) * 4 * float(np.abs(vf).max())
    print(f"attn=mma hd={hd} heads {nh}/{nkv} n_pos={n_pos} n_q={n_q} kv={kv}: max err {err:.2e} (bound {tol:.2e})")
    assert err <= tol
    ops.close()
