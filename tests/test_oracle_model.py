"""Model-level self-consistency of the CPU oracle on the tiny synthetic hybrid MoE.

Whole-model parity with the reference is unpinned (its model tests need checkpoint files), so the
oracle's model level is held by the invariants the reference asserts of its own CPU backend:
batched prefill == token-by-token to the bit (tests/qwen35.rs:94-139,348-395), split prefill ==
single prefill (tests/kv_cache.rs:109-133), overflow leaves the cache untouched (:161-172),
position advances (tests/qwen35.rs:41-74).
"""
import numpy as np
import pytest

from oracle import oracle_py as O
from tests.util import TINY, oracle_dims, prompt_ids


@pytest.fixture(scope="module")
def model():
    m = O.OracleModel(oracle_dims(TINY))
    m.synth(0, threads=8)
    return m


def test_tensor_inventory(model):
    names = [s["name"] for s in model.specs]
    assert "blk.3.attn_q.weight" in names and "blk.0.attn_qkv.weight" in names
    assert "blk.3.attn_qkv.weight" not in names          # layer 3 is the full-attention layer
    exps = next(s for s in model.specs if s["name"] == "blk.1.ffn_down_exps.weight")
    assert (exps["n_in"], exps["n_out"], exps["n_expert"], exps["ty"]) == (128, 256, 16, 40)


def test_batched_prefill_equals_token_by_token(model):
    ids = prompt_ids(1, 24, TINY["n_vocab"])
    model.begin(64)
    batched = model.forward(ids)
    st_b = [model.ssm_state(i).copy() for i in range(3)]
    model.begin(64)
    for t in ids:
        one = model.forward([t])
    assert batched.view(np.uint32).tolist() == one.view(np.uint32).tolist()
    for i in range(3):
        assert (st_b[i].view(np.uint32) == model.ssm_state(i).view(np.uint32)).all()
    assert model.pos() == 24


def test_split_prefill_equals_single_prefill(model):
    ids = prompt_ids(1, 20, TINY["n_vocab"])
    model.begin(32); a = model.forward(ids)
    model.begin(32); model.forward(ids[:7]); b = model.forward(ids[7:])
    assert a.view(np.uint32).tolist() == b.view(np.uint32).tolist()


def test_overflow_leaves_the_cache_untouched(model):
    model.begin(8)
    model.forward(prompt_ids(1, 6, TINY["n_vocab"]))
    with pytest.raises(RuntimeError):
        model.forward([1, 2, 3])
    assert model.pos() == 6


def test_greedy_generation_is_deterministic_and_logs_routes(model):
    ids = prompt_ids(1, 16, TINY["n_vocab"])
    model.begin(64, log_routes=True)
    a, margins = model.generate(ids, 8)
    routes = model.route_log()
    # prefill 16 tokens + 7 decode steps, 4 layers, top-4
    assert routes.size == (16 + 7) * 4 * 4 and routes.min() >= 0 and routes.max() < 16
    model.begin(64)
    b, _ = model.generate(ids, 8)
    assert a.tolist() == b.tolist() and len(a) == 8 and (margins >= 0).all()


def test_nvfp4_shared_expert_and_lm_head_scales_are_applied_to_the_matmul_results():
    """An NVFP4 file's shared expert and LM head (src/model/mod.rs:351-361; src/model/qwen35.rs:1668-1682, :1117-1120): the oracle
    tells the storage type by byte count and multiplies each matmul's result by the tensor's `.scale`. Checked against the
    same model with the scale folded in by hand: a power-of-two `output.scale` must scale the logits exactly, and the batched
    == token-by-token invariant must survive the other storage type."""
    m = O.OracleModel(oracle_dims(TINY)); m.synth(0, threads=8)
    rng = np.random.default_rng(5)

    def fp4(n_in, n_out):
        nb = n_out * n_in // 64
        blk = np.zeros((nb, 36), np.uint8)
        blk[:, :4] = rng.integers(0x20, 0x50, (nb, 4)); blk[:, 4:] = rng.integers(0, 256, (nb, 32))
        return blk.reshape(-1)
    m.set_tensor("output.weight", fp4(TINY["n_embd"], TINY["n_vocab"]))
    for il in range(TINY["n_layer"]):
        m.set_tensor(f"blk.{il}.ffn_gate_shexp.weight", fp4(TINY["n_embd"], TINY["shared_ff"]))
        m.set_tensor(f"blk.{il}.ffn_up_shexp.weight", fp4(TINY["n_embd"], TINY["shared_ff"]))
        m.set_tensor(f"blk.{il}.ffn_down_shexp.weight", fp4(TINY["shared_ff"], TINY["n_embd"]))
        m.set_tensor(f"blk.{il}.ffn_gate_shexp.scale", np.array([0.05], np.float32))
        m.set_tensor(f"blk.{il}.ffn_down_shexp.scale", np.array([0.03], np.float32))
    ids = prompt_ids(3, 12, TINY["n_vocab"])
    m.begin(32); plain = m.forward(ids).copy()
    m.set_tensor("output.scale", np.array([0.25], np.float32))
    m.begin(32); scaled = m.forward(ids).copy()
    assert (scaled.view(np.uint32) == (plain * np.float32(0.25)).view(np.uint32)).all()
    m.begin(32)
    for t in ids:
        one = m.forward([t])
    assert one.view(np.uint32).tolist() == scaled.view(np.uint32).tolist()
    assert np.isfinite(scaled).all() and float(np.abs(scaled).max()) > 0
