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
