"""Model-level parity at the BENCHMARKED shapes: the 35B-A3B shape (BASELINE configs 3 and 4) and the ~177B shape
(config 5), cut to their first four layers (GDN, GDN, GDN, full attention) with the full vocabulary, against the CPU
oracle on identical weights.

The kernels the benchmark times are specialised by shape -- 256 or 512 experts with top-8 / top-10, head_dim 256 with
eight query heads per KV head, 128-wide delta-rule heads -- so the small shapes of the other model tests do not reach
them. Checks, as there: routing ids bit-exact per layer and token, logits within max-abs 2e-2 / cosine >= 0.999 under
teacher forcing (tests/cuda_ops.rs:544-626 in the reference), greedy tokens equal, the recurrent state left behind;
through the fused one-token step, a multi-row prefill pass and a three-sequence batch.

The weights are generated on the device and copied to the oracle (the device generator equals the CPU generator byte for
byte, tests/test_gpu_model.py::test_device_generator_equals_cpu_generator; generating 4 GB on the CPU would take minutes).
"""
import numpy as np
import pytest

from oracle import oracle_py as O
from tests.util import L177B, M35B, cosine, host_dims, oracle_dims, prompt_ids
from inferred_thoughts_b200 import configs

pytestmark = pytest.mark.gpu

SHAPES = {"m35b": (configs.with_layers(M35B, 4), configs.SEEDS["m35b"]),
          "l177b": (configs.with_layers(L177B, 4), configs.SEEDS["l177b"])}
N_CTX = 96


@pytest.fixture(scope="module", params=["m35b", "l177b"])
def pair(request):
    """(dims, oracle model, ops, device model) for one shape; exact arithmetic (serial-k F32 dots, f16 KV) on the device."""
    from inferred_thoughts_b200 import host
    dims, seed = SHAPES[request.param]
    ops = host.B200Ops(0, "exact=1")
    model = host.Model(ops, host_dims(dims)); model.synth(seed)
    om = O.OracleModel(oracle_dims(dims))
    for s in om.specs:
        data, sc = model.synth_read(seed, s["name"], s["bytes"], s["n_expert"] if s["has_scale"] else 0)
        om.set_tensor(s["name"], data, sc)
    O.lib().orc_set_threads(max(1, O.lib().orc_hw_threads()))
    yield dims, om, ops, model
    ops.check()
    model.close(); ops.close()


def _check_logits(o, g, what):
    err = float(np.abs(o - g).max())
    cos = cosine(o, g)
    assert err <= 2e-2 and cos >= 0.999, f"{what}: max-abs {err:.3e}, cosine {cos:.6f}"
    assert int(np.argmax(o)) == int(np.argmax(g)), f"{what}: argmax differs"
    return err


def test_fused_step_and_prefill_pass_against_the_oracle(pair):
    """A 12-token prompt in ONE multi-row pass, then 6 teacher-forced decode steps through the fused one-token step."""
    from inferred_thoughts_b200 import host
    dims, om, ops, model = pair
    L, K = dims["n_layer"], dims["n_expert_used"]
    prompt = prompt_ids(21, 12, dims["n_vocab"])
    eng = host.Engine(model, N_CTX, 1)
    om.begin(N_CTX, log_routes=True)
    o = om.forward(prompt)
    g = eng.prefill(prompt)
    worst = _check_logits(o, g, "prefill pass")
    o_routes = om.route_log().reshape(L, len(prompt), K)
    assert eng.read_routes(L, K)[:, 0, :].tolist() == o_routes[:, -1, :].tolist(), "routing of the last prompt token"
    exact = [bool((o == g).all())]
    for step in range(6):
        t = int(np.argmax(o))
        om.clear_route_log()
        o = om.forward([t])
        lg, _ = eng.decode([t])
        g = lg[0]
        assert eng.read_routes(L, K)[:, 0, :].tolist() == om.route_log().reshape(L, K).tolist(), f"routing at decode step {step}"
        worst = max(worst, _check_logits(o, g, f"decode step {step}"))
        exact.append(bool((o == g).all()))
    print(f"{dims['n_embd']}-wide: worst max-abs {worst:.3e}; logits bit-identical in {sum(exact)}/{len(exact)} passes")
    for il in range(3):   # the three GDN layers' delta-rule state left behind
        so, sg = om.ssm_state(il), eng.read_ssm_state(il)
        assert np.abs(so - sg).max() <= 1e-4 * max(1.0, float(np.abs(so).max())), il
    ops.check(); eng.close()


def test_token_by_token_prefill_and_greedy_tokens(pair):
    """The same prompt one token at a time (every prompt token through the fused step), then 8 greedy tokens."""
    import os
    from inferred_thoughts_b200 import host
    dims, om, ops, model = pair
    prompt = prompt_ids(22, 10, dims["n_vocab"])
    eng = host.Engine(model, N_CTX, 1)
    om.begin(N_CTX)
    want, margins = om.generate(prompt, 8)
    os.environ["ITB_PREFILL_STEPWISE"] = "1"
    try:
        got = eng.generate(prompt, 8)
    finally:
        del os.environ["ITB_PREFILL_STEPWISE"]
    first_div = next((i for i in range(len(want)) if want[i] != got[i]), None)
    assert first_div is None, f"first divergence at {first_div}, oracle top-2 margin there {margins[first_div]:.3e}"
    eng.reset()
    assert eng.generate(prompt, 8).tolist() == want.tolist(), "multi-row prefill, then greedy tokens"
    ops.check(); eng.close()


def test_three_sequences_against_the_oracle(pair):
    """Three sequences in one engine (multi-row passes for prefill and decode) against the oracle run on each alone."""
    from inferred_thoughts_b200 import host
    dims, om, ops, model = pair
    L, K = dims["n_layer"], dims["n_expert_used"]
    prompts = np.stack([prompt_ids(30 + i, 9, dims["n_vocab"]) for i in range(3)])
    eng = host.Engine(model, N_CTX, 3)
    g0 = eng.prefill(prompts)
    toks = []
    for i in range(3):
        om.begin(N_CTX, log_routes=True)
        o = om.forward(prompts[i])
        _check_logits(o, g0[i], f"sequence {i} prefill")
        toks.append(int(np.argmax(o)))
    lg, nxt = eng.decode(np.array(toks, np.uint32))
    routes = eng.read_routes(L, K)
    for i in range(3):
        om.begin(N_CTX, log_routes=True)
        om.forward(prompts[i]); om.clear_route_log()
        o = om.forward([toks[i]])
        _check_logits(o, lg[i], f"sequence {i} decode")
        assert routes[:, i, :].tolist() == om.route_log().reshape(L, K).tolist(), f"sequence {i} routing"
        assert int(nxt[i]) == int(np.argmax(o))
    ops.check(); eng.close()


def test_prefill_pass_with_fp4_tensor_core_experts_against_the_oracle_with_fp4_activations():
    """experts=fp4tc at the 35B-A3B shape: a 160-token prompt in one pass, the routed experts as FP4 x FP4 tensor-core GEMMs,
    against the oracle run with FP4 activations (the reference's default device arithmetic and its CPU statement,
    src/ops/naive.rs:755-837). Same quantiser bit for bit; the tensor core's summation order is its own, so the logits are
    held to the north-star tolerance and the routing ids may differ only where the router's margin is at rounding level."""
    from inferred_thoughts_b200 import host
    dims, seed = SHAPES["m35b"]
    ops = host.B200Ops(0, "exact=1,experts=fp4tc")
    model = host.Model(ops, host_dims(dims)); model.synth(seed)
    om = O.OracleModel(oracle_dims(dims))
    for s in om.specs:
        data, sc = model.synth_read(seed, s["name"], s["bytes"], s["n_expert"] if s["has_scale"] else 0)
        om.set_tensor(s["name"], data, sc)
    O.lib().orc_set_threads(max(1, O.lib().orc_hw_threads()))
    L, K = dims["n_layer"], dims["n_expert_used"]
    prompt = prompt_ids(41, 160, dims["n_vocab"])
    eng = host.Engine(model, 256, 1)
    om.begin(256, fp4act=True, log_routes=True)
    o = om.forward(prompt)
    g = eng.prefill(prompt)
    err = _check_logits(o, g, "prefill pass, FP4 tensor-core experts")
    mism = int((eng.read_routes(L, K)[:, 0, :] != om.route_log().reshape(L, len(prompt), K)[:, -1, :]).sum())
    print(f"fp4tc prefill: logits max-abs {err:.3e}, routing ids differing on the last token {mism}/{L * K}")
    assert mism <= 2
    ops.check(); eng.close(); model.close(); ops.close()


@pytest.mark.parametrize("shape,kv,fast", [("mid", "f16", "attn=mma"), ("m35b", "f16", "attn=mma"), ("m35b", "bf16", "attn=mma"),
                                           ("m35b", "f16", "gdn=chunk"), ("m35b", "bf16", "attn=mma,gdn=chunk"),
                                           ("mid", "f16", "dense=f16tc"), ("m35b", "f16", "dense=f16tc")])
def test_prefill_with_the_many_token_kernels_against_the_oracle(shape, kv, fast):
    """The kernels many-token passes may use in place of the CPU-order ones, each selectable under exact=1 so that it is the
    only difference from the oracle:
      attn=mma   causal attention as 16-bit matrix products over (token, head) tiles with a running softmax (q and the
                 probabilities rounded to the cache's type, sums reassociated);
      gdn=chunk  the delta rule chunk-parallel (64-token chunks; everything off the state for all chunks at once);
      dense=f16tc  the dense Q8_0 matmuls as f16 tcgen05 GEMMs over dequantised operands (int8 * scale rounded to f16).
    All reassociate sums: tolerance class. A 150-token prompt in one pass (several K/V tiles and chunks, ragged last ones), 70
    more tokens in a second pass (queries deep in the cache, a state carried over), then two teacher-forced single-token steps
    over the cache and state the passes left.

    What bound holds depends on the model, not on the kernel: each kernel alone matches the CPU order to rounding level
    (tests/test_gpu_ops.py: the chunked delta rule to 1e-6, tensor-core attention to its 16-bit operand rounding), but every
    layer re-quantises its activations to int8 and picks 8 of 256 experts, and on the 35B-shape synthetic model (random
    weights, nearly flat router) a 1e-6 difference in one layer's output flips such a rounding or pick somewhere in a
    150-token pass and moves a logit by 0.03-0.14, and by up to 0.7 two teacher-forced steps later (measured). So the small
    model is held to the north-star bound (max-abs 2e-2, cosine 0.999) and the 35B shape only to a sanity bound (cosine
    0.98, max-abs 1.0: an indexing mistake gives cosine near 0); the 2e-2 bar at that shape is met by the bit-exact kernels
    only (the other tests of this file).

    dense=f16tc perturbs every dense output by ~3e-4 of the outputs' root mean square (tests/test_gpu_ops.py holds the GEMM itself
    to that), a thousand times the reassociation level of the other two. On these random-weight models that is past the
    router's margins: picks of the last prompt token differ from the oracle's in several (layer, pick) places on the small
    model too (printed below), and a swapped expert moves a logit by tenths -- bf16 operands (eight times the rounding) gave
    the same 0.35 / cosine 0.973 as f16, i.e. the error is the flipped picks, not the rounding. So this option is held to
    the sanity bound on both shapes (cosine 0.95, max-abs 1.5) and its precision claim rests on the op-level test."""
    from inferred_thoughts_b200 import host
    dims, seed = (configs.MID, configs.SEEDS["mid"]) if shape == "mid" else SHAPES["m35b"]
    ops = host.B200Ops(0, "exact=1," + fast + (",kv=bf16" if kv == "bf16" else ""))
    model = host.Model(ops, host_dims(dims)); model.synth(seed)
    om = O.OracleModel(oracle_dims(dims))
    for s in om.specs:
        data, sc = model.synth_read(seed, s["name"], s["bytes"], s["n_expert"] if s["has_scale"] else 0)
        om.set_tensor(s["name"], data, sc)
    O.lib().orc_set_threads(max(1, O.lib().orc_hw_threads()))
    prompt = prompt_ids(51, 220, dims["n_vocab"])
    eng = host.Engine(model, 256, 1)
    om.begin(256, kv_bf16=(kv == "bf16"), log_routes=True)
    bound, cos_min = (2e-2, 0.999) if shape == "mid" else (1.0, 0.98)
    if "f16tc" in fast: bound, cos_min = 1.5, 0.95

    def check(o, g, what):
        err, cos = float(np.abs(o - g).max()), cosine(o, g)
        assert err <= bound and cos >= cos_min, f"{what}: max-abs {err:.3e}, cosine {cos:.6f}"
        return err
    o = om.forward(prompt[:150]); g = eng.prefill(prompt[:150])
    worst = check(o, g, "first pass")
    L, K = dims["n_layer"], dims["n_expert_used"]
    mism = int((eng.read_routes(L, K)[:, 0, :] != om.route_log().reshape(L, 150, K)[:, -1, :]).sum())
    print(f"{fast} {shape}: routing ids of the last prompt token differing from the oracle's: {mism}/{L * K}")
    o = om.forward(prompt[150:]); g = eng.prefill(prompt[150:])
    worst = max(worst, check(o, g, "second pass"))
    for step in range(2):
        t = int(np.argmax(o))
        o = om.forward([t]); lg, _ = eng.decode([t]); g = lg[0]
        worst = max(worst, check(o, g, f"decode step {step}"))
    print(f"{fast} {shape} kv={kv}: worst logits max-abs {worst:.3e}")
    for il in range(3):
        so, sg = om.ssm_state(il), eng.read_ssm_state(il)
        assert np.abs(so - sg).max() <= 0.2 * max(1.0, float(np.abs(so).max())), il
    ops.check(); eng.close(); model.close(); ops.close()


def test_three_sequences_with_tensor_core_attention():
    """Three sequences of 40 tokens in one pass (query tiles never straddle sequences), each against the oracle alone."""
    from inferred_thoughts_b200 import host
    dims, seed = SHAPES["m35b"]
    ops = host.B200Ops(0, "exact=1,attn=mma")
    model = host.Model(ops, host_dims(dims)); model.synth(seed)
    om = O.OracleModel(oracle_dims(dims))
    for s in om.specs:
        data, sc = model.synth_read(seed, s["name"], s["bytes"], s["n_expert"] if s["has_scale"] else 0)
        om.set_tensor(s["name"], data, sc)
    O.lib().orc_set_threads(max(1, O.lib().orc_hw_threads()))
    prompts = np.stack([prompt_ids(60 + i, 40, dims["n_vocab"]) for i in range(3)])
    eng = host.Engine(model, N_CTX, 3)
    g0 = eng.prefill(prompts)
    for i in range(3):
        om.begin(N_CTX)
        o = om.forward(prompts[i])
        err, cos = float(np.abs(o - g0[i]).max()), cosine(o, g0[i])
        assert err <= 1.0 and cos >= 0.98, f"sequence {i}: max-abs {err:.3e}, cosine {cos:.6f}"
    ops.check(); eng.close(); model.close(); ops.close()


@pytest.mark.parametrize("shape", ["mid", "m35b", "l177b"])
def test_dense_q8_0_matmuls_on_the_int8_tensor_cores_are_bit_identical(shape):
    """dense=q8tc: many-row passes run every dense Q8_0 matmul as tcgen05 int8 MMAs (one per 32-element block, s32 accumulators
    in tensor memory), the block scales and the sum applied afterwards in the CPU path's order and rounding. Nothing is
    reassociated, so under exact=1 the logits of a 200-token prompt pass (a ragged second token tile), of 70 more tokens and
    of a decode step must equal the oracle's bit for bit."""
    from inferred_thoughts_b200 import host
    dims, seed = (configs.MID, configs.SEEDS["mid"]) if shape == "mid" else SHAPES[shape]
    ops = host.B200Ops(0, "exact=1,dense=q8tc")
    model = host.Model(ops, host_dims(dims)); model.synth(seed)
    om = O.OracleModel(oracle_dims(dims))
    for s in om.specs:
        data, sc = model.synth_read(seed, s["name"], s["bytes"], s["n_expert"] if s["has_scale"] else 0)
        om.set_tensor(s["name"], data, sc)
    O.lib().orc_set_threads(max(1, O.lib().orc_hw_threads()))
    prompt = prompt_ids(71, 270, dims["n_vocab"])
    eng = host.Engine(model, 288, 1)
    om.begin(288)
    o = om.forward(prompt[:200]); g = eng.prefill(prompt[:200])
    assert (o.view(np.uint32) == g.view(np.uint32)).all(), f"first pass: max-abs {np.abs(o - g).max():.3e}"
    o = om.forward(prompt[200:]); g = eng.prefill(prompt[200:])
    assert (o.view(np.uint32) == g.view(np.uint32)).all(), f"second pass: max-abs {np.abs(o - g).max():.3e}"
    t = int(np.argmax(o))
    o = om.forward([t]); lg, _ = eng.decode([t])
    assert (o.view(np.uint32) == lg[0].view(np.uint32)).all(), "decode step"
    ops.check(); eng.close(); model.close(); ops.close()
