"""Host side of the C ABI in Python: the reference's backend interface (`trait Ops`, src/ops/mod.rs:489-1426)
with the same method names, argument meaning and error behaviour, over ctypes.

Buffers are numpy arrays whose host ADDRESSES are the handles, exactly as the reference's device backend
keys its mirrors (src/ops/cuda/ops/residency.rs:23-57): keep an array alive and pass the same array (not a
slice or a copy) for the same logical buffer. Methods return nothing; failures are sticky and surface
through `take_error()` / `check()`.
"""
import ctypes as C
from pathlib import Path

import numpy as np

from . import build as _build

SZ = C.c_size_t
F32, F16, Q8_0, NVFP4 = 0, 1, 8, 40


class _Weights(C.Structure):
    _fields_ = [("data", C.c_void_p), ("bytes", SZ), ("ggml_type", C.c_uint32), ("n_in", SZ), ("n_out", SZ), ("pooled", C.c_int)]


class _Experts(C.Structure):
    _fields_ = [("data", C.c_void_p), ("bytes", SZ), ("ggml_type", C.c_uint32), ("n_in", SZ), ("n_out", SZ),
                ("n_expert", SZ), ("scale", C.c_void_p), ("scale_bytes", SZ)]


class _Route(C.Structure):
    _fields_ = [("on_device", C.c_int), ("n_used", SZ), ("n_tok", SZ), ("ids", C.c_void_p), ("weights", C.c_void_p)]


class _Attn(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_len", SZ), ("k", C.c_void_p), ("v", C.c_void_p), ("slab_len", SZ), ("kv_dim", SZ),
                ("n_pos", SZ), ("head_dim", SZ), ("n_head", SZ), ("n_head_kv", SZ), ("scale", C.c_float)]


class _Delta(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("q", "k", "v", "alpha", "beta", "ssm_a", "dt_bias")] + \
               [(n, SZ) for n in ("n_tokens", "head_k_dim", "head_v_dim", "n_k_heads", "n_v_heads")]


class ModelDims(C.Structure):
    """itb_model_dims: src/model/qwen35.rs:193-249 `Config` + `Moe`."""
    _fields_ = [(n, C.c_uint32) for n in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_vocab")] + \
               [("rope_theta", C.c_float), ("rms_eps", C.c_float)] + \
               [(n, C.c_uint32) for n in ("n_rot", "ssm_d_conv", "ssm_d_inner", "ssm_d_state", "ssm_dt_rank",
                                          "ssm_n_group", "full_attention_interval", "n_expert", "n_expert_used",
                                          "expert_ff", "shared_ff")]


_LIB = None


def lib():
    """Load libitb.so (building it if stale). Raises if it cannot be built or loaded: there is no fallback."""
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(str(_build.build()))
        L = _LIB
        L.itb_take_error.restype = C.c_char_p
        L.itb_last_create_error.restype = C.c_char_p
        L.itb_launch_count.restype = C.c_uint64
        L.itb_model_decode_bytes.restype = C.c_uint64
        L.itb_engine_pos.restype = C.c_uint32
        L.itb_engine_last_ms.restype = C.c_float
        L.itb_engine_launches_per_step.restype = C.c_uint64
        L.itb_engine_generate.restype = C.c_long
        L.itb_gclock_create.restype = C.c_void_p
    return _LIB


def _p(a):
    return C.c_void_p(a.ctypes.data) if a is not None else C.c_void_p(None)


class Weights:
    """Borrowed weight bytes in the file's block layout (src/ops/mod.rs:62-92)."""

    def __init__(self, data, ty, n_in, n_out):
        self.data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        self.ty, self.n_in, self.n_out = ty, n_in, n_out
        self.c = _Weights(self.data.ctypes.data, self.data.size, ty, n_in, n_out, 0)


class Experts:
    """A stack of n_expert matrices with an optional per-expert second scale (src/ops/mod.rs:107-152)."""

    def __init__(self, data, ty, n_in, n_out, n_expert, scale=None):
        self.data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        self.scale = None if scale is None else np.ascontiguousarray(scale, np.float32)
        self.ty, self.n_in, self.n_out, self.n_expert = ty, n_in, n_out, n_expert
        self.c = _Experts(self.data.ctypes.data, self.data.size, ty, n_in, n_out, n_expert,
                          None if self.scale is None else self.scale.ctypes.data, 0 if self.scale is None else self.scale.size * 4)


class Route:
    """src/ops/mod.rs:176-218. `Route.host(ids, weights, n_used)` or the device route `B200Ops.route` returns."""

    def __init__(self, c, keep=()):
        self.c, self._keep = c, keep

    @staticmethod
    def host(ids, weights, n_used):
        ids = np.ascontiguousarray(ids, np.uint64)
        weights = None if weights is None else np.ascontiguousarray(weights, np.float32)
        return Route(_Route(0, n_used, ids.size // n_used, ids.ctypes.data, None if weights is None else weights.ctypes.data),
                     (ids, weights))

    @property
    def n_used(self):
        return self.c.n_used

    @property
    def n_tok(self):
        return self.c.n_tok


class B200Ops:
    """The backend object: one CUDA context-equivalent on one device, single-threaded."""

    def __init__(self, device=0, opts=""):
        self.L = lib()
        h = C.c_void_p()
        rc = self.L.itb_create(device, opts.encode(), C.byref(h))
        if rc:
            raise RuntimeError(f"itb_create failed ({rc}): {(self.L.itb_last_create_error() or b'').decode()}")
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.L.itb_destroy(self.h); self.h = None

    def __del__(self):
        self.close()

    # -- errors (src/ops/cuda/ops/mod.rs:91-110)
    def take_error(self):
        e = self.L.itb_take_error(self.h)
        return None if e is None else e.decode()

    def check(self):
        e = self.take_error()
        if e:
            raise RuntimeError(e)

    # -- residency protocol
    def begin_pass(self, n_tokens): self.L.itb_begin_pass(self.h, SZ(n_tokens))
    def end_pass(self): self.L.itb_end_pass(self.h)
    def host_wrote(self, buf): self.L.itb_host_wrote(self.h, _p(buf), SZ(buf.size))
    def host_needs(self, buf): self.L.itb_host_needs(self.h, _p(buf), SZ(buf.size))
    def forget_state(self): self.L.itb_forget_state(self.h)
    def read_state(self, host): self.L.itb_read_state(self.h, _p(host), SZ(host.size))
    def read_kv(self, slab): self.L.itb_read_kv(self.h, _p(slab), SZ(slab.size))
    def launch_count(self): return self.L.itb_launch_count(self.h)

    def fp4_ceiling(self, n=256, iters=4000, reps=5):
        """Measured dense TFLOP/s of tcgen05.mma kind::mxf4nvf4 (M128 x N n x K64), accumulators verified: (tflops, status, cycles per MMA)."""
        t, st, cy = C.c_double(), C.c_int(), C.c_double()
        if self.L.itb_fp4_ceiling(self.h, n, iters, reps, C.byref(t), C.byref(st), C.byref(cy)):
            self.check(); raise RuntimeError("fp4_ceiling failed")
        return t.value, st.value, cy.value

    def fp4_quantize(self, x):
        """FP4 activation record of x (length a multiple of 16): (UE4M3 scale codes [n/16], E2M1 codes [n]) as the tensor-core path makes them."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        sc = np.zeros(x.size // 16, np.uint8); q = np.zeros(x.size, np.uint8)
        if self.L.itb_fp4_quantize(self.h, _p(x), SZ(x.size), _p(sc), _p(q)):
            self.check(); raise RuntimeError("fp4_quantize failed")
        return sc, q

    def config_report(self):
        b = C.create_string_buffer(512)
        self.L.itb_config_report(self.h, b, SZ(512))
        return b.value.decode()

    # -- ops
    def rms_norm(self, x, weight, eps, out):
        self.L.itb_rms_norm(self.h, _p(x), SZ(x.size), _p(weight), SZ(weight.size), C.c_float(eps), _p(out))

    def rms_norm_heads(self, x, weight, head_dim, eps):
        self.L.itb_rms_norm_heads(self.h, _p(x), SZ(x.size), _p(weight), SZ(head_dim), C.c_float(eps))

    def matmul(self, w, x, out):
        self.L.itb_matmul(self.h, C.byref(w.c), _p(x), SZ(x.size), _p(out), SZ(out.size))

    def matmul_pair(self, a, b, x, out_a, out_b):
        self.L.itb_matmul_pair(self.h, C.byref(a.c), C.byref(b.c), _p(x), SZ(x.size), _p(out_a), SZ(out_a.size), _p(out_b), SZ(out_b.size))

    def rope_neox(self, x, pos, head_dim, n_rot, n_heads, theta):
        self.L.itb_rope_neox(self.h, _p(x), SZ(x.size), SZ(pos), SZ(head_dim), SZ(n_rot), SZ(n_heads), C.c_float(theta))

    def softmax(self, x, row): self.L.itb_softmax(self.h, _p(x), SZ(x.size), SZ(row))

    def attend(self, q, k_slab, v_slab, kv_dim, n_pos, head_dim, n_head, n_head_kv, scale, out):
        a = _Attn(q.ctypes.data, q.size, k_slab.ctypes.data, v_slab.ctypes.data, k_slab.size, kv_dim, n_pos, head_dim,
                  n_head, n_head_kv, scale)
        self.L.itb_attend(self.h, C.byref(a), _p(out), SZ(out.size))

    def kv_write(self, slab, offset, src):
        self.L.itb_kv_write(self.h, _p(slab), SZ(slab.size), SZ(offset), _p(src), SZ(src.size))

    def silu_mul(self, gate, up): self.L.itb_silu_mul(self.h, _p(gate), _p(up), SZ(gate.size))
    def sigmoid_mul(self, x, g): self.L.itb_sigmoid_mul(self.h, _p(x), _p(g), SZ(x.size))
    def scale(self, buf, s): self.L.itb_scale(self.h, _p(buf), SZ(buf.size), C.c_float(s))
    def add_assign(self, a, b): self.L.itb_add_assign(self.h, _p(a), _p(b), SZ(a.size))
    def add_scaled(self, a, b, s): self.L.itb_add_scaled(self.h, _p(a), _p(b), SZ(a.size), C.c_float(s))

    def add_scaled_rows(self, acc, rows, scales):
        self.L.itb_add_scaled_rows(self.h, _p(acc), SZ(acc.size), _p(rows), _p(scales), SZ(scales.size))

    def add_scaled_sigmoid(self, acc, b, logit): self.L.itb_add_scaled_sigmoid(self.h, _p(acc), _p(b), SZ(acc.size), _p(logit))

    def gather_chunks(self, src, chunk, stride, offset, out):
        self.L.itb_gather_chunks(self.h, _p(src), SZ(src.size), SZ(chunk), SZ(stride), SZ(offset), _p(out), SZ(out.size))

    def scatter_chunks(self, src, chunk, stride, offset, dst):
        self.L.itb_scatter_chunks(self.h, _p(src), SZ(src.size), SZ(chunk), SZ(stride), SZ(offset), _p(dst), SZ(dst.size))

    def l2_norm_heads(self, x, head_dim, eps): self.L.itb_l2_norm_heads(self.h, _p(x), SZ(x.size), SZ(head_dim), C.c_float(eps))

    def ssm_conv(self, state, x, weight, kernel, out):
        self.L.itb_ssm_conv(self.h, _p(state), SZ(state.size), _p(x), SZ(x.size), _p(weight), SZ(weight.size), SZ(kernel), _p(out))

    def delta_rule(self, q, k, v, alpha, beta, ssm_a, dt_bias, head_k_dim, head_v_dim, n_k_heads, n_v_heads, state, out):
        n_tok = v.size // (n_v_heads * head_v_dim)
        d = _Delta(q.ctypes.data, k.ctypes.data, v.ctypes.data, alpha.ctypes.data, beta.ctypes.data, ssm_a.ctypes.data,
                   dt_bias.ctypes.data, n_tok, head_k_dim, head_v_dim, n_k_heads, n_v_heads)
        self.L.itb_delta_rule(self.h, C.byref(d), _p(state), SZ(state.size), _p(out), SZ(out.size))

    def route(self, probs, n_expert, n_used):
        r = _Route()
        self.L.itb_route(self.h, _p(probs), SZ(probs.size), SZ(n_expert), SZ(n_used), C.byref(r))
        return Route(r)

    def read_route(self, route):
        n = route.n_tok * route.n_used
        ids, w = np.zeros(n, np.int32), np.zeros(n, np.float32)
        self.L.itb_read_route(self.h, _p(ids), _p(w), SZ(n))
        return ids, w

    def matmul_experts(self, w, route, x, out):
        self.L.itb_matmul_experts(self.h, C.byref(w.c), C.byref(route.c), _p(x), SZ(x.size), _p(out), SZ(out.size))

    def moe_glu(self, gate, up, route, x, out, scratch):
        self.L.itb_moe_glu(self.h, C.byref(gate.c), C.byref(up.c), C.byref(route.c), _p(x), SZ(x.size), _p(out), SZ(out.size), _p(scratch))

    def moe_finish(self, out, at, n, rows, route, shared, logit, logit_at):
        self.L.itb_moe_finish(self.h, _p(out), SZ(out.size), SZ(at), SZ(n), _p(rows), SZ(rows.size), C.byref(route.c),
                              _p(shared), _p(logit), SZ(logit_at))

    def synth_values(self, key, first, n, dist, std):
        out = np.zeros(n, np.float32)
        rc = self.L.itb_synth_values(self.h, C.c_uint64(key), C.c_uint64(first), SZ(n), dist, C.c_float(std), _p(out))
        if rc:
            self.check()
        return out


class Model:
    """A model resident on the device: tensors by GGUF name, loaded from host bytes or generated in place."""

    def __init__(self, ops: B200Ops, dims: ModelDims):
        self.ops, self.dims, self.L = ops, dims, ops.L
        h = C.c_void_p()
        if self.L.itb_model_create(ops.h, C.byref(dims), C.byref(h)):
            ops.check(); raise RuntimeError("itb_model_create failed")
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.L.itb_model_destroy(self.h); self.h = None

    def __del__(self):
        self.close()

    def set_tensor(self, name, ty, data, scale=None):
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        sc = None if scale is None else np.ascontiguousarray(scale, np.float32)
        if self.L.itb_model_set_tensor(self.h, name.encode(), ty, _p(data), SZ(data.size), _p(sc), SZ(0 if sc is None else sc.size)):
            self.ops.check(); raise RuntimeError(f"set_tensor({name}) failed")

    @classmethod
    def from_gguf(cls, ops, path):
        """Load a qwen35moe GGUF file (src/gguf/mod.rs, src/model/qwen35.rs:333-486): dims from its metadata, tensors from the mapping."""
        h = C.c_void_p()
        err = C.create_string_buffer(512)
        if ops.L.itb_model_load_gguf(ops.h, str(path).encode(), C.byref(h), err, SZ(512)):
            raise RuntimeError("gguf: " + err.value.decode(errors="replace"))
        self = cls.__new__(cls)
        self.ops, self.L, self.h = ops, ops.L, h
        d = ModelDims()
        ops.L.itb_model_dims_of(h, C.byref(d))
        self.dims = d
        return self

    def offload_experts(self):
        """Move the routed experts to pinned host memory; only tiered engines (Engine(tier_capacity=...)) can run the model after."""
        if self.L.itb_model_offload_experts(self.h):
            self.ops.check(); raise RuntimeError("offload_experts failed")

    def synth(self, seed, expert_lo=0, expert_hi=0):
        if self.L.itb_model_synth(self.h, C.c_uint64(seed), expert_lo, expert_hi):
            self.ops.check(); raise RuntimeError("model synth failed")

    def synth_read(self, seed, name, nbytes, n_scale=0):
        out = np.zeros(nbytes, np.uint8)
        sc = np.zeros(n_scale, np.float32) if n_scale else None
        if self.L.itb_model_synth_read(self.h, C.c_uint64(seed), name.encode(), _p(out), SZ(nbytes), _p(sc)):
            self.ops.check(); raise RuntimeError(f"synth_read({name}) failed")
        return out, sc

    def decode_bytes(self, n_seq, n_pos, distinct_experts):
        return self.L.itb_model_decode_bytes(self.h, n_seq, n_pos, distinct_experts)


def expert_range(rank, world, n_expert):
    """The contiguous range of routed experts rank `rank` of `world` stores (src/ops/mod.rs:1024-1048: placement by range)."""
    if world < 1 or not 0 <= rank < world or n_expert % world:
        raise ValueError("world must divide n_expert and 0 <= rank < world")
    per = n_expert // world
    return per * rank, per * (rank + 1)


def ep_a2a_plan(cnt, rank):
    """cnt[s][d] = pairs rank s sends to rank d -> (send_off[world + 1], recv_off[world + 1], n_recv) of rank `rank`."""
    cnt = np.ascontiguousarray(cnt, np.int32)
    world = cnt.shape[0]
    so, ro, n = np.zeros(world + 1, np.int32), np.zeros(world + 1, np.int32), C.c_int()
    if lib().itb_ep_a2a_plan(_p(cnt), world, rank, _p(so), _p(ro), C.byref(n)):
        raise ValueError("bad count matrix or rank")
    return so, ro, n.value


def ep_unique_id(lib_=None):
    """128 bytes that name a new NCCL communicator; rank 0 makes them, every rank passes the same bytes to Engine(ep=...)."""
    L = lib_ or lib()
    out = np.zeros(128, np.uint8)
    if L.itb_ep_unique_id(_p(out)):
        raise RuntimeError("NCCL is not loadable in this process")
    return out.tobytes()


def share_unique_id(rank, lib_=None, group=None):
    """Rank 0's unique id handed to every rank of an initialised torch.distributed group (any backend)."""
    import torch
    import torch.distributed as dist
    t = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        t = torch.frombuffer(bytearray(ep_unique_id(lib_)), dtype=torch.uint8).clone()
    if dist.get_backend(group) == "nccl":
        t = t.cuda(); dist.broadcast(t, 0, group=group); t = t.cpu()
    else:
        dist.broadcast(t, 0, group=group)
    return t.numpy().tobytes()


class Engine:
    """Engine::{prefill, decode, generate} (src/engine/mod.rs:352-437) over n_seq independent sequences."""

    def __init__(self, model: Model, n_ctx, n_seq=1, ep=None, tier_capacity=None):
        """ep = (rank, world, unique_id bytes): an expert-parallel engine over a model that holds this rank's expert range
        (`expert_range`); every rank must then make the same calls with the same shapes (each on its own sequences)."""
        self.model, self.L, self.n_seq = model, model.L, n_seq
        h = C.c_void_p()
        if tier_capacity is not None:
            # experts in pinned host memory (Model.offload_experts), `tier_capacity` (layer, expert) entries cached in HBM
            rc = self.L.itb_engine_create_tiered(model.h, n_ctx, n_seq, int(tier_capacity), C.byref(h))
        elif ep is None:
            rc = self.L.itb_engine_create(model.h, n_ctx, n_seq, C.byref(h))
        else:
            rank, world, uid = ep
            uid = np.frombuffer(bytes(uid), np.uint8).copy()
            assert uid.size == 128
            rc = self.L.itb_engine_create_ep(model.h, n_ctx, n_seq, _p(uid), int(rank), int(world), C.byref(h))
        if rc:
            model.ops.check(); raise RuntimeError("itb_engine_create failed")
        self.h = h
        self.n_vocab = model.dims.n_vocab

    def close(self):
        if getattr(self, "h", None):
            self.L.itb_engine_destroy(self.h); self.h = None

    def __del__(self):
        self.close()

    def _chk(self, rc, what):
        if rc:
            self.model.ops.check(); raise RuntimeError(f"{what} failed ({rc})")

    def checkpoint(self):
        """Positions + recurrent state as bytes (src/engine/mod.rs:255-270); the KV cache needs no copy."""
        self.L.itb_engine_checkpoint_bytes.restype = C.c_size_t
        n = self.L.itb_engine_checkpoint_bytes(self.h)
        buf = np.zeros(n, np.uint8)
        self._chk(self.L.itb_engine_checkpoint(self.h, _p(buf), SZ(n)), "checkpoint")
        return buf

    def restore(self, ckpt):
        buf = np.ascontiguousarray(ckpt, np.uint8)
        self._chk(self.L.itb_engine_restore(self.h, _p(buf), SZ(buf.size)), "restore")

    def tier_stats(self):
        out = (C.c_uint64 * 4)()
        self.L.itb_engine_tier_stats(self.h, out)
        return dict(hits=out[0], misses=out[1], evictions=out[2], bytes_moved=out[3])

    def ep_step_transport(self):
        """How an expert-parallel engine's one-token step moves rows between ranks: 'peer-memory', 'nccl', or 'none' (not expert parallel)."""
        return {0: "none", 1: "nccl", 2: "peer-memory"}[self.L.itb_engine_ep_transport(self.h)]

    def tier_counters(self):
        """The reference's TierCounters as far as they exist here (see itb.h), as a dict."""
        names = ("fetched fetch_bytes picks_wait_us prefetch_reads prefetch_used lookups host_reads slot_bytes slots pool_bytes "
                 "vram_free vram_total mirrors mirror_bytes weight_bytes kv_bytes resident_bytes").split()
        out = (C.c_uint64 * len(names))()
        if self.L.itb_tier_counters(self.h, out):
            raise RuntimeError("tier_counters failed")
        return dict(zip(names, (int(v) for v in out)))

    def reset(self): self.L.itb_engine_reset(self.h)
    def pos(self, seq=0): return self.L.itb_engine_pos(self.h, seq)

    def prefill(self, tokens, want_logits=True):
        """tokens: [n_seq][n] (or [n] for one sequence); returns the last token's logits, [n_seq][n_vocab] (or [n_vocab])."""
        tokens = np.ascontiguousarray(tokens, np.uint32).reshape(self.n_seq, -1)
        logits = np.zeros((self.n_seq, self.n_vocab), np.float32) if want_logits else None
        self._chk(self.L.itb_engine_prefill(self.h, _p(tokens), SZ(tokens.shape[1]), _p(logits)), "prefill")
        if logits is None:
            return None
        return logits[0] if self.n_seq == 1 else logits

    def decode(self, tokens, want_logits=True):
        tokens = np.ascontiguousarray(tokens, np.uint32).reshape(-1)
        assert tokens.size == self.n_seq
        logits = np.zeros((self.n_seq, self.n_vocab), np.float32) if want_logits else None
        nxt = np.zeros(self.n_seq, np.uint32)
        self._chk(self.L.itb_engine_decode(self.h, _p(tokens), _p(logits), _p(nxt)), "decode")
        return logits, nxt

    def decode_loop(self, first_tokens, steps):
        first = np.ascontiguousarray(first_tokens, np.uint32).reshape(-1)
        out = np.zeros((steps, self.n_seq), np.uint32)
        self._chk(self.L.itb_engine_decode_loop(self.h, _p(first), steps, _p(out)), "decode_loop")
        return out

    def generate(self, prompt, max_new):
        prompt = np.ascontiguousarray(prompt, np.uint32)
        out = np.zeros(max_new, np.uint32)
        n = self.L.itb_engine_generate(self.h, _p(prompt), SZ(prompt.size), SZ(max_new), _p(out))
        if n < 0:
            self._chk(1, "generate")
        return out[:n]

    def read_routes(self, n_moe_layers, n_used):
        ids = np.zeros(n_moe_layers * self.n_seq * n_used, np.int32)
        self._chk(self.L.itb_engine_read_routes(self.h, _p(ids), SZ(ids.size)), "read_routes")
        return ids.reshape(n_moe_layers, self.n_seq, n_used)

    def read_ssm_state(self, il, seq=0):
        d = self.model.dims
        n = d.ssm_d_state * d.ssm_d_inner
        out = np.zeros(n, np.float32)
        self._chk(self.L.itb_engine_read_ssm_state(self.h, seq, il, _p(out), SZ(n)), "read_ssm_state")
        return out

    def decode_path(self):
        """(1, text) when single-token steps run as the one persistent kernel, else (0, why not)."""
        why = C.create_string_buffer(256)
        return self.L.itb_engine_decode_path(self.h, why, SZ(256)), why.value.decode()

    def last_ms(self): return self.L.itb_engine_last_ms(self.h)
    def launches_per_step(self): return self.L.itb_engine_launches_per_step(self.h)
