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


@pytest.mark.parametrize("shape,kv", [("mid", "f16"), ("m35b", "f16"), ("m35b", "bf16")])
def test_prefill_with_tensor_core_attention_against_the_oracle(shape, kv):
    """attn=mma: many-token passes run causal attention as 16-bit matrix products over (token, head) tiles with a running
    softmax -- q and the probabilities rounded to the cache's type, sums reassociated -- so the logits are held to the
    north-star tolerance, not to the bit. A 150-token prompt in one pass (several K/V tiles, a ragged last query tile), 70 more
    tokens in a second pass (queries that start deep in the cache), then two teacher-forced single-token steps (the split-K
    path over the cache the tensor-core pass wrote), for head_dim 64 with 4 heads per KV head and head_dim 256 with 8."""
    from inferred_thoughts_b200 import host
    dims, seed = (configs.MID, configs.SEEDS["mid"]) if shape == "mid" else SHAPES["m35b"]
    ops = host.B200Ops(0, "exact=1,attn=mma" + (",kv=bf16" if kv == "bf16" else ""))
    model = host.Model(ops, host_dims(dims)); model.synth(seed)
    om = O.OracleModel(oracle_dims(dims))
    for s in om.specs:
        data, sc = model.synth_read(seed, s["name"], s["bytes"], s["n_expert"] if s["has_scale"] else 0)
        om.set_tensor(s["name"], data, sc)
    O.lib().orc_set_threads(max(1, O.lib().orc_hw_threads()))
    prompt = prompt_ids(51, 220, dims["n_vocab"])
    eng = host.Engine(model, 256, 1)
    om.begin(256, kv_bf16=(kv == "bf16"))
    o = om.forward(prompt[:150]); g = eng.prefill(prompt[:150])
    worst = _check_logits(o, g, "first pass")
    o = om.forward(prompt[150:]); g = eng.prefill(prompt[150:])
    worst = max(worst, _check_logits(o, g, "second pass"))
    for step in range(2):
        t = int(np.argmax(o))
        o = om.forward([t]); lg, _ = eng.decode([t]); g = lg[0]
        worst = max(worst, _check_logits(o, g, f"decode step {step}"))
    print(f"attn=mma {shape} kv={kv}: worst logits max-abs {worst:.3e}")
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
        _check_logits(om.forward(prompts[i]), g0[i], f"sequence {i}")
    ops.check(); eng.close(); model.close(); ops.close()
