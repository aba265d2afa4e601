"""GGUF loader: failure paths on CPU (they are decided before any device call), the round trip on the GPU."""
import ctypes as C
import struct

import numpy as np
import pytest

from tests import gguf_writer as W
from tests.util import TINY, host_dims, oracle_dims, prompt_ids


def _load_err(path):
    from inferred_thoughts_b200 import host
    L = host.lib()
    h = C.c_void_p()
    err = C.create_string_buffer(512)
    rc = L.itb_model_load_gguf(None, str(path).encode(), C.byref(h), err, C.c_size_t(512))
    return rc, err.value.decode()


def test_rejects_what_is_not_gguf(tmp_path):
    p = tmp_path / "x.gguf"
    p.write_bytes(b"FUGG" + b"\0" * 64)
    rc, msg = _load_err(p)
    assert rc != 0 and "magic" in msg
    p.write_bytes(b"GGUF" + struct.pack("<IQQ", 2, 0, 0) + b"\0" * 32)
    rc, msg = _load_err(p)
    assert rc != 0 and "version" in msg
    rc, msg = _load_err(tmp_path / "absent.gguf")
    assert rc != 0 and "open" in msg


def test_truncated_and_incomplete_files_fail_with_a_message(tmp_path):
    kv = W.metadata(dict(TINY))
    p = tmp_path / "t.gguf"
    W.write(p, kv, [])
    whole = p.read_bytes()
    p.write_bytes(whole[: len(whole) // 2])                    # cut inside the metadata
    rc, msg = _load_err(p)
    assert rc != 0 and ("truncated" in msg or "malformed" in msg)
    W.write(p, [x for x in kv if not x[0].endswith("expert_count")], [])
    rc, msg = _load_err(p)
    assert rc != 0 and "qwen35moe.expert_count" in msg
    W.write(p, [("general.architecture", 8, "llama")], [])
    rc, msg = _load_err(p)
    assert rc != 0 and "architecture" in msg


@pytest.mark.gpu
def test_loaded_file_equals_generated_model(tmp_path):
    """Oracle tensors -> GGUF file -> itb_model_load_gguf gives the engine outputs of the generated model, bit for bit."""
    from inferred_thoughts_b200 import host
    from oracle import oracle_py as O
    om = O.OracleModel(oracle_dims(TINY)); om.synth(0, threads=8)
    path = tmp_path / "tiny.gguf"
    W.from_oracle(path, dict(TINY), om)
    ops = host.B200Ops(0, "exact=1")
    gen = host.Model(ops, host_dims(TINY)); gen.synth(0)
    loaded = host.Model.from_gguf(ops, path)
    assert loaded.dims.n_vocab == TINY["n_vocab"] and loaded.dims.n_expert == TINY["n_expert"]
    prompt = prompt_ids(7, 24, TINY["n_vocab"])
    e1, e2 = host.Engine(gen, 64, 1), host.Engine(loaded, 64, 1)
    a, b = e1.prefill(prompt), e2.prefill(prompt)
    assert a.view(np.uint32).tolist() == b.view(np.uint32).tolist()
    ops.check()
    e1.close(); e2.close(); loaded.close(); gen.close(); ops.close()


@pytest.mark.gpu
def test_nvfp4_shared_expert_and_lm_head_with_their_scales_against_the_oracle(tmp_path):
    """An NVFP4 file stores the shared expert's three matrices and the LM head as NVFP4 too, each with a one-element second
    scale applied to the matmul's result (`<weight>.scale`, src/model/mod.rs:351-361; src/model/qwen35.rs:1668-1682 and
    :1117-1120 for `output.scale`). The tiny model with those four kinds of tensors replaced -- in the oracle by name, in the
    library both by `itb_model_set_tensor` and through a GGUF file -- must give the oracle's logits and routing ids bit for
    bit through a multi-row prefill pass and teacher-forced decode steps (such a model's steps run the multi-row kernels)."""
    from inferred_thoughts_b200 import host
    from oracle import oracle_py as O
    dims = dict(TINY)
    om = O.OracleModel(oracle_dims(dims)); om.synth(0, threads=8)
    ops = host.B200Ops(0, "exact=1")
    model = host.Model(ops, host_dims(dims)); model.synth(0)
    rng = np.random.default_rng(77)
    override = {}

    def fp4(n_in, n_out):
        nb = n_out * n_in // 64
        blk = np.zeros((nb, 36), np.uint8)
        blk[:, :4] = rng.integers(0x20, 0x50, (nb, 4)); blk[:, 4:] = rng.integers(0, 256, (nb, 32))
        return blk.reshape(-1)
    names = [("output.weight", dims["n_embd"], dims["n_vocab"], 0.004)]
    for il in range(dims["n_layer"]):
        names += [(f"blk.{il}.ffn_gate_shexp.weight", dims["n_embd"], dims["shared_ff"], 0.05), (f"blk.{il}.ffn_up_shexp.weight", dims["n_embd"], dims["shared_ff"], 0.04),
                  (f"blk.{il}.ffn_down_shexp.weight", dims["shared_ff"], dims["n_embd"], 0.03)]
    for i, (name, n_in, n_out, sc) in enumerate(names):
        data = fp4(n_in, n_out)
        scale = None if i % 4 == 3 else np.float32(sc * (1 + 0.1 * i))      # every fourth matrix without a scale: it is optional
        override[name] = (W.GGML["NVFP4"], data, scale)
        om.set_tensor(name, data)
        model.set_tensor(name, host.NVFP4, data)
        if scale is not None:
            om.set_tensor(name.replace(".weight", ".scale"), np.array([scale], np.float32))
            model.set_tensor(name.replace(".weight", ".scale"), host.F32, np.array([scale], np.float32))
    path = tmp_path / "tiny_fp4_dense.gguf"
    W.from_oracle(path, dims, om, override=override)
    loaded = host.Model.from_gguf(ops, path)
    L, K = dims["n_layer"], dims["n_expert_used"]
    prompt = prompt_ids(9, 40, dims["n_vocab"])
    for what, mdl in (("set_tensor", model), ("gguf", loaded)):
        eng = host.Engine(mdl, 64, 1)
        om.begin(64, log_routes=True)
        o = om.forward(prompt); g = eng.prefill(prompt)
        assert o.view(np.uint32).tolist() == g.view(np.uint32).tolist(), f"{what}: prompt logits, max-abs {np.abs(o - g).max():.3e}"
        for step in range(4):
            t = int(np.argmax(o))
            om.clear_route_log()
            o = om.forward([t]); lg, _ = eng.decode([t])
            assert o.view(np.uint32).tolist() == lg[0].view(np.uint32).tolist(), f"{what}: decode step {step}"
            assert eng.read_routes(L, K)[:, 0, :].tolist() == om.route_log().reshape(L, K).tolist()
        eng.close()
    with pytest.raises(RuntimeError):
        model.set_tensor("blk.0.attn_norm.scale", host.F32, np.array([1.0], np.float32))      # no weight takes such a scalar
    ops.take_error()
    ops.check()
    loaded.close(); model.close(); ops.close()
