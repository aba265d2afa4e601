"""A minimal GGUF v3 writer for tests: metadata of a qwen35moe model plus tensors given as raw block bytes.
Layout as the reference reads it (src/gguf/mod.rs:143-296 there)."""
import struct

import numpy as np

GGML = {"F32": 0, "F16": 1, "Q8_0": 8, "NVFP4": 40}
_U32, _F32, _STR, _ARR = 4, 6, 8, 9


def _s(b):
    b = b.encode() if isinstance(b, str) else b
    return struct.pack("<Q", len(b)) + b


def _kv(key, ty, val):
    out = _s(key) + struct.pack("<I", ty)
    if ty == _U32:
        return out + struct.pack("<I", val)
    if ty == _F32:
        return out + struct.pack("<f", val)
    if ty == _STR:
        return out + _s(val)
    if ty == _ARR:      # (element type, values): u32 arrays only
        return out + struct.pack("<IQ", _U32, len(val)) + b"".join(struct.pack("<I", v) for v in val)
    raise ValueError(ty)


def metadata(dims, arch="qwen35moe", alignment=32):
    a = arch + "."
    kv = [("general.architecture", _STR, arch), ("general.alignment", _U32, alignment),
          (a + "block_count", _U32, dims["n_layer"]), (a + "embedding_length", _U32, dims["n_embd"]),
          (a + "attention.head_count", _U32, dims["n_head"]), (a + "attention.head_count_kv", _U32, dims["n_head_kv"]),
          (a + "attention.key_length", _U32, dims["head_dim"]), (a + "attention.value_length", _U32, dims["head_dim"]),
          (a + "rope.freq_base", _F32, dims["rope_theta"]), (a + "attention.layer_norm_rms_epsilon", _F32, dims["rms_eps"]),
          (a + "rope.dimension_count", _U32, dims["n_rot"]), (a + "rope.dimension_sections", _ARR, [dims["n_rot"] // 2, 0, 0, 0]),
          (a + "ssm.conv_kernel", _U32, dims["ssm_d_conv"]), (a + "ssm.inner_size", _U32, dims["ssm_d_inner"]),
          (a + "ssm.state_size", _U32, dims["ssm_d_state"]), (a + "ssm.time_step_rank", _U32, dims["ssm_dt_rank"]),
          (a + "ssm.group_count", _U32, dims["ssm_n_group"]), (a + "full_attention_interval", _U32, dims["full_attention_interval"]),
          (a + "expert_count", _U32, dims["n_expert"]), (a + "expert_used_count", _U32, dims["n_expert_used"]),
          (a + "expert_feed_forward_length", _U32, dims["expert_ff"]),
          (a + "expert_shared_feed_forward_length", _U32, dims["shared_ff"])]
    return kv


def write(path, kv, tensors, alignment=32):
    """tensors: list of (name, ggml type id, dims with the fastest first, bytes)."""
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kv)) + b"".join(_kv(*x) for x in kv)
    infos, blobs, off = b"", [], 0
    for name, ty, dims, data in tensors:
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ty, off)
        data = bytes(data)
        pad = (-len(data)) % alignment
        blobs.append(data + b"\0" * pad)
        off += len(data) + pad
    head += infos
    head += b"\0" * ((-len(head)) % alignment)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)


def from_oracle(path, dims, oracle, override=None):
    """Every tensor of an oracle model (its specs: name, type id, shape, block bytes) into a GGUF file. override: name ->
    (ggml type id, bytes, second scale or None) for tensors written in another storage type than the spec's (an NVFP4
    shared expert or LM head with its one-element `.scale`)."""
    tensors = []
    for s in oracle.specs:
        if override and s["name"] in override:
            ty, data, sc = override[s["name"]]
            shape = [s["n_in"], s["n_out"]]
            tensors.append((s["name"], ty, shape, np.asarray(data).tobytes()))
            if sc is not None:
                tensors.append((s["name"].replace(".weight", ".scale"), GGML["F32"], [1], np.asarray([sc], np.float32).tobytes()))
            continue
        data, sc = oracle.tensor(s["name"])
        if s["n_expert"] > 1 or s["has_scale"]:
            shape = [s["n_in"], s["n_out"], s["n_expert"]]
        elif s["n_out"] > 1 or s["name"].endswith("_inp_shexp.weight"):
            shape = [s["n_in"], s["n_out"]]
        else:
            shape = [s["n_in"]]
        tensors.append((s["name"], s["ty"], shape, np.asarray(data).tobytes()))
        if sc is not None:
            tensors.append((s["name"].replace(".weight", ".scale"), GGML["F32"], [len(sc)], np.asarray(sc, np.float32).tobytes()))
    write(path, metadata(dims), tensors)
