"""Model-level parity on the GPU: the tiny synthetic hybrid MoE (BASELINE config 1) through the fused engine
against the CPU oracle on identical seeded weights.

Checks, in the reference's order of strength (tests/cuda_ops.rs:544-626 there): routing ids bit-exact per
layer per token, logits within max-abs 2e-2 / cosine >= 0.999 under TEACHER FORCING (the oracle's tokens are
fed to both sides, never each side's own argmax), greedy tokens equal, recurrent state left behind.
"""
import numpy as np
import pytest

from oracle import oracle_py as O
from tests.util import MID, ODD, TINY, cosine, host_dims, oracle_dims, prompt_ids

pytestmark = pytest.mark.gpu
SEED = 0


@pytest.fixture(scope="module")
def oracle():
    m = O.OracleModel(oracle_dims(TINY)); m.synth(SEED, threads=8)
    return m


@pytest.fixture(scope="module")
def gpu():
    from inferred_thoughts_b200 import host
    ops = host.B200Ops(0, "exact=1")
    model = host.Model(ops, host_dims(TINY)); model.synth(SEED)
    yield ops, model
    ops.check()


def test_device_generator_equals_cpu_generator(oracle, gpu):
    _, model = gpu
    for name in ("blk.0.attn_qkv.weight", "blk.3.attn_q.weight", "blk.1.ffn_gate_exps.weight", "blk.2.ffn_down_exps.weight",
                 "blk.0.ssm_a", "output_norm.weight", "token_embd.weight", "blk.3.ffn_gate_inp.weight"):
        spec = next(s for s in oracle.specs if s["name"] == name)
        want, wsc = oracle.tensor(name)
        got, gsc = model.synth_read(SEED, name, spec["bytes"], spec["n_expert"] if spec["has_scale"] else 0)
        assert got.tobytes() == want.tobytes(), name
        if wsc is not None:
            assert gsc.tobytes() == wsc.tobytes(), name + " second scales"


def _teacher_forced(oracle, eng, prompt, n_new):
    """Prefill + n_new decode steps with the ORACLE's greedy tokens fed to both sides."""
    oracle.begin(128, log_routes=True)
    eng.reset()
    o_logits = [oracle.forward(prompt)]
    g_logits = [eng.prefill(prompt)]
    toks = []
    L = TINY["n_layer"]; K = TINY["n_expert_used"]
    o_routes = oracle.route_log().reshape(L, len(prompt), K)   # prefill pass: [layer][token][k]
    g_routes_last = eng.read_routes(L, K)[:, 0, :]
    assert g_routes_last.tolist() == o_routes[:, -1, :].tolist(), "routing of the last prompt token"
    for _ in range(n_new):
        t = int(np.argmax(o_logits[-1]))          # np.argmax returns the first maximum, like the reference's scan
        toks.append(t)
        oracle.clear_route_log()
        o_logits.append(oracle.forward([t]))
        lg, _ = eng.decode([t])
        g_logits.append(lg[0])
        assert eng.read_routes(L, K)[:, 0, :].tolist() == oracle.route_log().reshape(L, K).tolist(), f"routing at step {len(toks)}"
    return np.array(o_logits), np.array(g_logits), toks


def test_tiny_model_teacher_forced_logits_and_routing(oracle, gpu):
    from inferred_thoughts_b200 import host
    ops, model = gpu
    eng = host.Engine(model, 128, 1)
    prompt = prompt_ids(1, 64, TINY["n_vocab"])
    o, g, _ = _teacher_forced(oracle, eng, prompt, 32)
    err = np.abs(o - g).max()
    cos = min(cosine(a, b) for a, b in zip(o, g))
    print(f"tiny teacher-forced: max-abs {err:.3e}, min cosine {cos:.8f}, exact logits {(o == g).mean():.3f}")
    assert err <= 2e-2 and cos >= 0.999
    assert (np.argmax(o, 1) == np.argmax(g, 1)).all()
    # recurrent state left behind
    for il in range(3):
        so, sg = oracle.ssm_state(il), eng.read_ssm_state(il)
        assert np.abs(so - sg).max() <= 1e-4 * max(1.0, float(np.abs(so).max())), il
    eng.close()


def test_tiny_model_greedy_tokens_match(oracle, gpu):
    from inferred_thoughts_b200 import host
    ops, model = gpu
    eng = host.Engine(model, 128, 1)
    prompt = prompt_ids(1, 64, TINY["n_vocab"])
    oracle.begin(128)
    want, margins = oracle.generate(prompt, 32)
    got = eng.generate(prompt, 32)
    first_div = next((i for i in range(len(want)) if want[i] != got[i]), None)
    assert first_div is None, f"first divergence at {first_div}, oracle top-2 margin there {margins[first_div]:.3e}"
    # the device-resident loop produces the same tokens
    eng.reset(); eng.prefill(prompt)
    loop = eng.decode_loop([want[0]], 31)
    assert loop[:, 0].tolist() == want[1:].tolist()
    eng.close()


def test_loaded_tensors_equal_generated_tensors(oracle, gpu):
    """set_tensor (host bytes, the drop-in path) and the device generator give the same engine outputs."""
    from inferred_thoughts_b200 import host
    ops, model = gpu
    m2 = host.Model(ops, host_dims(TINY))
    for s in oracle.specs:
        data, sc = oracle.tensor(s["name"])
        m2.set_tensor(s["name"], s["ty"], data, sc)
    prompt = prompt_ids(2, 16, TINY["n_vocab"])
    e1, e2 = host.Engine(model, 64, 1), host.Engine(m2, 64, 1)
    a, b = e1.prefill(prompt), e2.prefill(prompt)
    assert a.view(np.uint32).tolist() == b.view(np.uint32).tolist()
    e1.close(); e2.close(); m2.close()


def test_batch_of_sequences_equals_single_sequences(oracle, gpu):
    """Three sequences in one engine (multi-row passes: int8-MMA matmuls, per-sequence state and KV) give the bits the
    same sequences give alone, through prefill and through decode steps."""
    from inferred_thoughts_b200 import host
    ops, model = gpu
    prompts = np.stack([prompt_ids(10 + i, 12, TINY["n_vocab"]) for i in range(3)])
    eb = host.Engine(model, 64, 3)
    logits_b = eb.prefill(prompts)
    ops.check()
    singles = [host.Engine(model, 64, 1) for _ in range(3)]
    for i in range(3):
        l1 = singles[i].prefill(prompts[i])
        assert l1.view(np.uint32).tolist() == logits_b[i].view(np.uint32).tolist(), i
    toks = np.argmax(logits_b, 1).astype(np.uint32)
    for step in range(4):
        lb, nb = eb.decode(toks)
        for i in range(3):
            l1, n1 = singles[i].decode([toks[i]])
            assert l1[0].view(np.uint32).tolist() == lb[i].view(np.uint32).tolist(), (step, i)
            assert n1[0] == nb[i]
        toks = nb
    for i in range(3):
        singles[i].close()
    eb.close()


def test_multi_row_prefill_equals_token_by_token(oracle, gpu):
    """Prefill in multi-row passes == the same tokens fed one at a time, to the bit: logits, recurrent state, and the
    decode steps that follow (the reference's own invariant, tests/qwen35.rs:94-139 there), and both equal the oracle."""
    import os
    from inferred_thoughts_b200 import host
    ops, model = gpu
    prompt = prompt_ids(3, 80, TINY["n_vocab"])   # 80 rows: the grouped MMA expert kernels; the 21/59 split below: the few-rows ones
    e1, e2 = host.Engine(model, 128, 1), host.Engine(model, 128, 1)
    a = e1.prefill(prompt)
    os.environ["ITB_PREFILL_STEPWISE"] = "1"
    try:
        b = e2.prefill(prompt)
    finally:
        del os.environ["ITB_PREFILL_STEPWISE"]
    assert a.view(np.uint32).tolist() == b.view(np.uint32).tolist()
    for il in range(3):
        assert e1.read_ssm_state(il).view(np.uint32).tolist() == e2.read_ssm_state(il).view(np.uint32).tolist(), il
    oracle.begin(128)
    want = oracle.forward(prompt)
    assert np.abs(want - a).max() <= 2e-2
    t = int(np.argmax(a))
    la, _ = e1.decode([t]); lb, _ = e2.decode([t])
    assert la.view(np.uint32).tolist() == lb.view(np.uint32).tolist()
    # a second chunk appended after the first (split prefill == single prefill, tests/kv_cache.rs:109-133 there)
    e3 = host.Engine(model, 128, 1)
    e3.prefill(prompt[:21]); c = e3.prefill(prompt[21:])
    assert c.view(np.uint32).tolist() == a.view(np.uint32).tolist()
    e1.close(); e2.close(); e3.close()


@pytest.fixture(scope="module")
def mid():
    """A shape with every k a multiple of 256: the pipelined (cp.async ring) multi-row kernels run, not the direct ones."""
    from inferred_thoughts_b200 import host
    om = O.OracleModel(oracle_dims(MID)); om.synth(5, threads=8)
    ops = host.B200Ops(0, "exact=1")
    model = host.Model(ops, host_dims(MID)); model.synth(5)
    yield om, ops, model
    ops.check()


@pytest.mark.parametrize("n_tok", [70, 200, 300, 640])
def test_pipelined_rows_prefill_equals_token_by_token_and_oracle(mid, n_tok):
    """One pass of n_tok rows: 70, 200, 300 and 640 rows give the routed experts about 5, 13, 19 and 40 rows each, i.e. the 8-, 16-,
    32- and 64-token expert tiles; the dense tiles are 64 tokens wide with a ragged last tile in every case."""
    import os
    from inferred_thoughts_b200 import host
    om, ops, model = mid
    prompt = prompt_ids(4, n_tok, MID["n_vocab"])
    os.environ["ITB_ROWS"] = "640"
    try:
        e1, e2 = host.Engine(model, 768, 1), host.Engine(model, 768, 1)
    finally:
        del os.environ["ITB_ROWS"]
    a = e1.prefill(prompt)
    os.environ["ITB_PREFILL_STEPWISE"] = "1"
    try:
        b = e2.prefill(prompt)
    finally:
        del os.environ["ITB_PREFILL_STEPWISE"]
    ops.check()
    assert a.view(np.uint32).tolist() == b.view(np.uint32).tolist()
    L, K = MID["n_layer"], MID["n_expert_used"]
    assert e1.read_routes(L, K).tolist() == e2.read_routes(L, K).tolist()
    for il in range(3):
        assert e1.read_ssm_state(il).view(np.uint32).tolist() == e2.read_ssm_state(il).view(np.uint32).tolist(), il
    om.begin(768, log_routes=True)
    want = om.forward(prompt)
    assert om.route_log().reshape(L, len(prompt), K)[:, -1, :].tolist() == e1.read_routes(L, K)[:, 0, :].tolist()
    err = np.abs(want - a).max()
    print(f"mid prefill vs oracle: max-abs {err:.3e}, exact {(want == a).mean():.3f}")
    assert err <= 2e-2 and cosine(want, a) >= 0.999 and int(np.argmax(want)) == int(np.argmax(a))
    e1.close(); e2.close()


@pytest.mark.parametrize("n_seq", [5, 33])
def test_pipelined_rows_batched_decode_equals_single_sequences(mid, n_seq):
    """n_seq <= 32 runs the 32-token tiles, 33 the 64-token ones; both must give each sequence the bits it gets alone."""
    from inferred_thoughts_b200 import host
    om, ops, model = mid
    prompts = np.stack([prompt_ids(20 + i, 9, MID["n_vocab"]) for i in range(n_seq)])
    eb = host.Engine(model, 64, n_seq)
    logits_b = eb.prefill(prompts)
    ops.check()
    probe = sorted({0, n_seq // 2, n_seq - 1})
    singles = {i: host.Engine(model, 64, 1) for i in probe}
    for i in probe:
        l1 = singles[i].prefill(prompts[i])
        assert l1.view(np.uint32).tolist() == logits_b[i].view(np.uint32).tolist(), i
    toks = np.argmax(logits_b, 1).astype(np.uint32)
    for step in range(3):
        lb, nb = eb.decode(toks)
        for i in probe:
            l1, n1 = singles[i].decode([toks[i]])
            assert l1[0].view(np.uint32).tolist() == lb[i].view(np.uint32).tolist(), (step, i)
            assert n1[0] == nb[i]
        toks = nb
    for i in probe:
        singles[i].close()
    eb.close()


def test_tree_mode_rows_equal_single_rows():
    """exact=0 (F32 dots by a shuffle tree, the benchmark's mode): the multi-row F32 kernel keeps the one-token kernel's
    summation order, so batched decode and multi-row prefill still give each row the bits it gets alone."""
    import os
    from inferred_thoughts_b200 import host
    ops = host.B200Ops(0, "exact=0")
    model = host.Model(ops, host_dims(MID)); model.synth(5)
    prompts = np.stack([prompt_ids(40 + i, 11, MID["n_vocab"]) for i in range(5)])
    eb = host.Engine(model, 64, 5)
    lb = eb.prefill(prompts)
    singles = [host.Engine(model, 64, 1) for _ in range(5)]
    os.environ["ITB_PREFILL_STEPWISE"] = "1"
    try:
        ls = [e.prefill(p) for e, p in zip(singles, prompts)]     # token by token through the fused one-token kernels
    finally:
        del os.environ["ITB_PREFILL_STEPWISE"]
    for i in range(5):
        assert ls[i].view(np.uint32).tolist() == lb[i].view(np.uint32).tolist(), i
    toks = np.argmax(lb, 1).astype(np.uint32)
    for step in range(3):
        l2, nb = eb.decode(toks)
        for i in range(5):
            l1, n1 = singles[i].decode([toks[i]])
            assert l1[0].view(np.uint32).tolist() == l2[i].view(np.uint32).tolist(), (step, i)
        toks = nb
    ops.check()
    for e in singles:
        e.close()
    eb.close(); model.close(); ops.close()


def test_phase_timeline_records_every_structured_launch(oracle, gpu):
    """itb_timeline_arm/read: one decode step of the tiny model (3 GDN layers + 1 attention layer) fills one slot per structured
    launch, phase stamps ascending inside a launch and launches in order; disarmed, nothing is written."""
    import ctypes as C
    from inferred_thoughts_b200 import host
    ops, model = gpu
    eng = host.Engine(model, 64, 1)
    eng.prefill(prompt_ids(9, 8, TINY["n_vocab"]))
    eng.decode([1])
    L = eng.L
    L.itb_timeline_read.restype = C.c_long
    slots = 64
    assert L.itb_timeline_arm(eng.h, slots) == 0
    eng.decode([2])
    words = np.zeros(slots * 16, np.uint64)
    assert L.itb_timeline_read(eng.h, C.c_void_p(words.ctypes.data), slots) == slots
    w = words.reshape(slots, 16)
    used = [i for i in range(slots) if w[i].any()]
    # per layer: in_proj, core|prep, out_proj, ffn in_proj, glu, down = 6 structured launches, plus the LM head
    assert used == list(range(4 * 6 + 1))
    kinds = [int(w[i][w[i] != 0][0]) & 255 for i in used]
    assert kinds[:6] == [2, 3, 4, 2, 8, 9] and kinds[18:24] == [2, 5, 4, 2, 8, 9] and kinds[24] == 2
    first = []
    for i in used:
        ts = [int(v) >> 8 for v in w[i] if v]
        assert ts == sorted(ts) or kinds[used.index(i)] == 8, i     # moe_glu's shared-expert blocks return before phase 2
        first.append(min(ts))
    assert first == sorted(first)
    assert L.itb_timeline_arm(eng.h, 0) == 0
    eng.decode([3]); ops.check()
    eng.close()


def test_odd_shape_matches_oracle_through_every_path():
    """The ~177B model's ratios in small (configs.ODD: 24- and 6-block rows, 10 picks of 48 experts, 3 query heads per kv
    head, 6 value heads on 3 key heads): fused one-token steps, a multi-row prefill and a batch of sequences all give the
    oracle's routing and logits, and each other's bits."""
    import os
    from inferred_thoughts_b200 import host
    om = O.OracleModel(oracle_dims(ODD)); om.synth(6, threads=8)
    ops = host.B200Ops(0, "exact=1")
    model = host.Model(ops, host_dims(ODD)); model.synth(6)
    L, K = ODD["n_layer"], ODD["n_expert_used"]
    prompt = prompt_ids(31, 70, ODD["n_vocab"])
    om.begin(128, log_routes=True)
    want = om.forward(prompt)
    want_routes = om.route_log().reshape(L, len(prompt), K)[:, -1, :]
    e_rows, e_step = host.Engine(model, 128, 1), host.Engine(model, 128, 1)
    a = e_rows.prefill(prompt)
    os.environ["ITB_PREFILL_STEPWISE"] = "1"
    try:
        b = e_step.prefill(prompt)
    finally:
        del os.environ["ITB_PREFILL_STEPWISE"]
    ops.check()
    for name, got, eng in (("multi-row", a, e_rows), ("one token at a time", b, e_step)):
        err = np.abs(want - got).max()
        assert err <= 2e-2 and cosine(want, got) >= 0.999 and int(np.argmax(want)) == int(np.argmax(got)), (name, err)
        assert eng.read_routes(L, K)[:, 0, :].tolist() == want_routes.tolist(), name
    assert a.view(np.uint32).tolist() == b.view(np.uint32).tolist()
    print(f"odd shape: max-abs vs oracle {np.abs(want - a).max():.3e}, exact {(want == a).mean():.3f}")
    # decode: the oracle's greedy tokens fed to the fused step and to a 3-sequence batch
    eb = host.Engine(model, 128, 3)
    lb = eb.prefill(np.stack([prompt, prompt, prompt]))
    assert lb[1].view(np.uint32).tolist() == a.view(np.uint32).tolist()
    t = int(np.argmax(want))
    for _ in range(6):
        w = om.forward([t])
        g1, _ = e_step.decode([t]); g3, _ = eb.decode([t, t, t])
        assert np.abs(w - g1[0]).max() <= 2e-2 and int(np.argmax(w)) == int(np.argmax(g1[0]))
        assert g3[2].view(np.uint32).tolist() == g1[0].view(np.uint32).tolist()
        t = int(np.argmax(w))
    ops.check()
    e_rows.close(); e_step.close(); eb.close(); model.close(); ops.close()


def test_benchmark_mode_bf16_kv_and_tree_dots_stays_within_tolerance(oracle):
    """kv=bf16 (BASELINE config 3) with exact=0 (tree-summed F32 dots; many-token passes on the tensor-core attention kernel)
    against the oracle with the reference's f16 cache and serial dots: the difference must stay inside the logits tolerance,
    for the multi-row pass and for the same prompt token by token (the two no longer share their attention kernel, so they
    agree with each other to the same tolerance, not to the bit; exact=1 keeps them bit-identical, see the tests above)."""
    import os
    from inferred_thoughts_b200 import host
    ops = host.B200Ops(0, "kv=bf16,exact=0")
    model = host.Model(ops, host_dims(TINY)); model.synth(SEED)
    prompt = prompt_ids(1, 64, TINY["n_vocab"])
    oracle.begin(128)
    want = oracle.forward(prompt)
    e1, e2 = host.Engine(model, 128, 1), host.Engine(model, 128, 1)
    a = e1.prefill(prompt)
    os.environ["ITB_PREFILL_STEPWISE"] = "1"
    try:
        b = e2.prefill(prompt)
    finally:
        del os.environ["ITB_PREFILL_STEPWISE"]
    for what, g in (("multi-row pass", a), ("token by token", b)):
        err, cos = float(np.abs(want - g).max()), cosine(want, g)
        print(f"bf16 kv, tree dots, {what} vs oracle: max-abs {err:.3e}, cosine {cos:.7f}")
        assert err <= 2e-2 and cos >= 0.999
    assert float(np.abs(a - b).max()) <= 2e-2
    ops.check()
    e1.close(); e2.close(); model.close(); ops.close()


def test_checkpoint_restore_replays_the_same_tokens(oracle, gpu):
    """Engine::checkpoint / restore (src/engine/mod.rs:255-294 there): save after the prompt, decode, go back, decode again:
    same logits bit for bit; a checkpoint of another shape is refused."""
    from inferred_thoughts_b200 import host
    ops, model = gpu
    eng = host.Engine(model, 128, 2)
    prompts = np.stack([prompt_ids(50 + i, 20, TINY["n_vocab"]) for i in range(2)])
    first = np.argmax(eng.prefill(prompts), 1).astype(np.uint32)
    ck = eng.checkpoint()
    run1, t = [], first
    for _ in range(5):
        lg, t = eng.decode(t); run1.append(lg.copy())
    assert eng.pos(0) == 25
    eng.restore(ck)
    assert eng.pos(0) == 20 and eng.pos(1) == 20
    t = first
    for i in range(5):
        lg, t = eng.decode(t)
        assert lg.view(np.uint32).tolist() == run1[i].view(np.uint32).tolist(), i
    other = host.Engine(model, 128, 1)
    with pytest.raises(RuntimeError):
        other.restore(ck)
    other.close(); eng.close()


def test_context_overflow_is_refused_before_any_write(oracle, gpu):
    from inferred_thoughts_b200 import host
    ops, model = gpu
    eng = host.Engine(model, 8, 1)
    eng.prefill(prompt_ids(1, 6, TINY["n_vocab"]))
    with pytest.raises(RuntimeError, match="context overflow"):
        eng.prefill([1, 2, 3])
    assert eng.pos() == 6
    eng.close()


def test_token_ids_outside_the_vocabulary_are_refused_before_any_launch(oracle, gpu):
    """TokenOutOfRange (src/model/qwen35.rs:866 there): decode, the device-resident loop, the profiled step and prefill all
    refuse on the host; nothing is copied or launched, and the engine goes on working."""
    from inferred_thoughts_b200 import host
    ops, model = gpu
    eng = host.Engine(model, 32, 1)
    eng.prefill(prompt_ids(1, 4, TINY["n_vocab"]))
    ops.check()
    before = ops.launch_count()
    for bad in (TINY["n_vocab"], 0xFFFFFFFF):
        with pytest.raises(RuntimeError, match="out of range"):
            eng.decode([bad])
        with pytest.raises(RuntimeError, match="out of range"):
            eng.decode_loop([bad], 2)
        with pytest.raises(RuntimeError, match="out of range"):
            eng.prefill([1, bad])
    assert ops.launch_count() == before and eng.pos() == 4
    lg, _ = eng.decode([3])
    assert np.isfinite(lg).all()
    # a host-built route naming an expert the stack does not have is refused the same way (src/ops/mod.rs:176-218 there)
    gate, gs = oracle.tensor("blk.0.ffn_gate_exps.weight")
    G = host.Experts(gate, host.NVFP4, TINY["n_embd"], TINY["expert_ff"], TINY["n_expert"], gs)
    x = np.zeros(TINY["n_embd"], np.float32); out = np.zeros(TINY["n_expert_used"] * TINY["expert_ff"], np.float32)
    ops.begin_pass(1)
    ops.matmul_experts(G, host.Route.host([0, 1, 2, TINY["n_expert"]], None, TINY["n_expert_used"]), x, out)
    assert "expert id out of range" in (ops.take_error() or "")
    eng.close()


def test_seam_ops_drive_a_whole_layer_like_the_reference_model_does(oracle, gpu):
    """Qwen35::gated_delta + moe_batch (src/model/qwen35.rs:1232-1328, :1587-1699 there) written against the op-level
    seam with host buffers as handles, exactly as the reference's model code calls its backend; compared with the
    oracle's first-layer output through the embedding of one token."""
    from inferred_thoughts_b200 import host
    ops, _ = gpu
    c = TINY; H = c["n_embd"]
    T = lambda n: oracle.tensor(n)
    def W(n, ty, n_in, n_out): return host.Weights(T(n)[0], ty, n_in, n_out)
    def V(n): return np.ascontiguousarray(T(n)[0]).view(np.float32)
    def E(n, n_in, n_out): d, s = T(n); return host.Experts(d, host.NVFP4, n_in, n_out, c["n_expert"], s)
    key_dim = c["ssm_d_state"] * c["ssm_n_group"]; vd = c["ssm_d_inner"]; cd = 2 * key_dim + vd; nv = c["ssm_dt_rank"]; sk = c["ssm_d_state"]
    tok = 17
    x = V("token_embd.weight")[tok * H:(tok + 1) * H].copy()
    f = lambda n: np.zeros(n, np.float32)
    normed, qkv, z, alpha, beta, conv, qp, kp, vp, core, mixed = f(H), f(cd), f(vd), f(nv), f(nv), f(cd), f(key_dim), f(key_dim), f(vd), f(vd), f(H)
    conv_state, ssm_state = f(cd * 3), f(nv * sk * sk)
    P = "blk.0."
    ops.begin_pass(1); ops.host_wrote(x)
    ops.rms_norm(x, V(P + "attn_norm.weight"), c["rms_eps"], normed)
    ops.matmul(W(P + "attn_qkv.weight", host.Q8_0, H, cd), normed, qkv)
    ops.matmul(W(P + "attn_gate.weight", host.Q8_0, H, vd), normed, z)
    ops.matmul_pair(W(P + "ssm_alpha.weight", host.F32, H, nv), W(P + "ssm_beta.weight", host.F32, H, nv), normed, alpha, beta)
    ops.ssm_conv(conv_state, qkv, V(P + "ssm_conv1d.weight"), 4, conv)
    ops.gather_chunks(conv, key_dim, cd, 0, qp); ops.gather_chunks(conv, key_dim, cd, key_dim, kp); ops.gather_chunks(conv, vd, cd, 2 * key_dim, vp)
    ops.l2_norm_heads(qp, sk, c["rms_eps"]); ops.l2_norm_heads(kp, sk, c["rms_eps"])
    ops.delta_rule(qp, kp, vp, alpha, beta, V(P + "ssm_a"), V(P + "ssm_dt.bias"), sk, sk, c["ssm_n_group"], nv, ssm_state, core)
    ops.rms_norm_heads(core, V(P + "ssm_norm.weight"), sk, c["rms_eps"])
    ops.silu_mul(z, core)
    ops.matmul(W(P + "ssm_out.weight", host.Q8_0, vd, H), z, mixed)
    ops.add_assign(x, mixed)
    # routed FFN
    e_in, router, logit = f(H), f(c["n_expert"]), f(1)
    ff, K = c["expert_ff"], c["n_expert_used"]
    g_all, u_all, o_all, e_gate, e_up, e_out, ffn_out = f(K * ff), f(K * ff), f(K * H), f(c["shared_ff"]), f(c["shared_ff"]), f(H), f(H)
    ops.rms_norm(x, V(P + "post_attention_norm.weight"), c["rms_eps"], normed)
    ops.gather_chunks(normed, H, H, 0, e_in)
    ops.matmul_pair(W(P + "ffn_gate_inp.weight", host.F32, H, c["n_expert"]), W(P + "ffn_gate_inp_shexp.weight", host.F32, H, 1), e_in, router, logit)
    ops.softmax(router, c["n_expert"])
    route = ops.route(router, c["n_expert"], K)
    ops.moe_glu(E(P + "ffn_gate_exps.weight", H, ff), E(P + "ffn_up_exps.weight", H, ff), route, e_in, g_all, u_all)
    ops.matmul_experts(E(P + "ffn_down_exps.weight", ff, H), route, g_all, o_all)
    ops.matmul(W(P + "ffn_gate_shexp.weight", host.Q8_0, H, c["shared_ff"]), e_in, e_gate)
    ops.matmul(W(P + "ffn_up_shexp.weight", host.Q8_0, H, c["shared_ff"]), e_in, e_up)
    ops.silu_mul(e_gate, e_up)
    ops.matmul(W(P + "ffn_down_shexp.weight", host.Q8_0, c["shared_ff"], H), e_gate, e_out)
    ops.moe_finish(ffn_out, 0, H, o_all, route, e_out, logit, 0)
    ops.add_assign(x, ffn_out)
    ops.end_pass(); ops.host_needs(x); ops.check()
    ids, _ = ops.read_route(route)
    # the oracle, one layer only: a model with the same tensors but n_layer = 1
    one = dict(TINY); one["n_layer"] = 1
    om = O.OracleModel(oracle_dims(one))
    for s in om.specs:
        d, sc = oracle.tensor(s["name"]); om.set_tensor(s["name"], d, sc)
    om.begin(8, log_routes=True)
    om.forward([tok])
    assert ids.tolist() == om.route_log().tolist()
    # x after the layer is not exposed by the oracle's forward; compare through its recurrent state instead
    ops.read_state(ssm_state)
    so = om.ssm_state(0)
    assert np.abs(ssm_state - so).max() <= 1e-5 * max(1.0, float(np.abs(so).max()))
    ops.forget_state()


def test_l2_hints_leave_the_step_bit_identical():
    """ITB_L2_HINT=1: every kernel of the one-token step asks for what the kernels after it will stream to be brought into L2
    (`cp.async.bulk.prefetch.L2`). Hints move no results: the smoke run (prefill against the oracle, routing ids, 8 greedy
    tokens) must pass unchanged with them on. A child process, because the library reads the variable once per process."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, ITB_L2_HINT="1")
    p = subprocess.run([sys.executable, "-c", "import __graft_entry__ as g; g.smoke()"], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "smoke ok" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]
