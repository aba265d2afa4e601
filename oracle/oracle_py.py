"""ctypes binding of the CPU oracle (liboracle.so). TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg import this module;
the product never does.
"""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB = None

F32P = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
U8P = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
U16P = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
I32P = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
U32P = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
SZ = C.c_size_t


class ModelDims(C.Structure):
    """Mirror of synth::ModelDims (csrc/synth_model.h)."""
    _fields_ = [(n, C.c_uint32) for n in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_vocab")] + \
               [("rope_theta", C.c_float), ("rms_eps", C.c_float)] + \
               [(n, C.c_uint32) for n in ("n_rot", "ssm_d_conv", "ssm_d_inner", "ssm_d_state", "ssm_dt_rank",
                                          "ssm_n_group", "full_attention_interval", "n_expert", "n_expert_used",
                                          "expert_ff", "shared_ff")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


def build(force=False):
    so = _DIR / "liboracle.so"
    srcs = [_DIR / f for f in ("oracle_ops.cpp", "oracle_model.cpp", "oracle_capi.cpp", "oracle.h")]
    srcs += [_DIR.parent / "inferred-thoughts_b200" / "csrc" / f for f in ("synth.h", "synth_model.h")]
    if force or not so.exists() or any(s.stat().st_mtime > so.stat().st_mtime for s in srcs if s.exists()):
        subprocess.check_call(["make", "-C", str(_DIR), "liboracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    L = C.CDLL(str(build()))

    def sig(name, res, *args):
        f = getattr(L, name); f.restype = res; f.argtypes = list(args)
    sig("orc_f16_to_f32", C.c_float, C.c_uint16)
    sig("orc_f32_to_f16", C.c_uint16, C.c_float)
    sig("orc_f32_to_bf16", C.c_uint16, C.c_float)
    sig("orc_ue4m3_to_f32", C.c_float, C.c_uint8)
    sig("orc_fp32_to_ue4m3_rn", C.c_uint8, C.c_float)
    sig("orc_e2m1_code", C.c_uint8, C.c_float, C.c_float)
    sig("orc_dequantize", None, C.c_uint32, U8P, F32P, SZ)
    sig("orc_q8_0_blocks", None, F32P, SZ, U8P)
    sig("orc_fp4_activation", None, F32P, SZ, U8P, U8P)
    sig("orc_vec_dot_nvfp4_q8_0", C.c_float, U8P, F32P, SZ)
    sig("orc_vec_dot_nvfp4_fp4", C.c_float, U8P, F32P, SZ)
    sig("orc_vec_dot_q8_0", C.c_float, U8P, F32P, SZ)
    sig("orc_set_threads", None, C.c_int)
    sig("orc_hw_threads", C.c_int)
    sig("orc_rms_norm", None, F32P, SZ, F32P, SZ, C.c_float, F32P)
    sig("orc_rms_norm_heads", None, F32P, SZ, F32P, SZ, C.c_float)
    sig("orc_matmul", None, C.c_uint32, U8P, SZ, SZ, F32P, SZ, F32P, C.c_int)
    sig("orc_rope_neox", None, F32P, SZ, SZ, SZ, SZ, SZ, C.c_float)
    sig("orc_softmax", None, F32P, SZ, SZ)
    sig("orc_attend", None, F32P, SZ, U16P, U16P, SZ, SZ, SZ, SZ, SZ, C.c_float, C.c_int, F32P)
    sig("orc_silu_mul", None, F32P, F32P, SZ)
    sig("orc_sigmoid_mul", None, F32P, F32P, SZ)
    sig("orc_scale", None, F32P, SZ, C.c_float)
    sig("orc_add_assign", None, F32P, F32P, SZ)
    sig("orc_add_scaled", None, F32P, F32P, SZ, C.c_float)
    sig("orc_add_scaled_rows", None, F32P, SZ, F32P, F32P, SZ)
    sig("orc_add_scaled_sigmoid", None, F32P, F32P, SZ, F32P)
    sig("orc_l2_norm_heads", None, F32P, SZ, SZ, C.c_float)
    sig("orc_ssm_conv", None, F32P, F32P, SZ, F32P, SZ, SZ, F32P)
    sig("orc_gather_chunks", None, F32P, SZ, SZ, SZ, F32P, SZ)
    sig("orc_scatter_chunks", None, F32P, SZ, SZ, SZ, SZ, F32P)
    sig("orc_delta_rule", None, F32P, F32P, F32P, F32P, F32P, F32P, F32P, SZ, SZ, SZ, SZ, SZ, F32P, F32P)
    sig("orc_kv_write", None, U16P, SZ, F32P, SZ, C.c_int)
    sig("orc_route", None, F32P, SZ, SZ, SZ, I32P, F32P)
    sig("orc_matmul_experts", None, U8P, SZ, SZ, SZ, C.c_void_p, I32P, SZ, SZ, F32P, SZ, F32P, C.c_int)
    sig("orc_moe_glu", None, U8P, C.c_void_p, U8P, C.c_void_p, SZ, SZ, SZ, I32P, SZ, SZ, F32P, SZ, F32P, C.c_int)
    sig("orc_moe_finish", None, F32P, SZ, SZ, F32P, I32P, F32P, SZ, SZ, F32P, F32P, SZ)
    sig("orc_argmax", C.c_uint32, F32P, SZ, C.POINTER(C.c_uint32))
    sig("orc_libm", None, C.c_int, F32P, SZ, F32P)
    sig("orc_tensor_key", C.c_uint64, C.c_uint64, C.c_char_p)
    sig("orc_synth_value", C.c_float, C.c_uint64, C.c_uint64, C.c_int, C.c_float)
    sig("orc_model_create", C.c_void_p, C.POINTER(ModelDims))
    sig("orc_model_destroy", None, C.c_void_p)
    sig("orc_model_n_tensors", SZ, C.c_void_p)
    sig("orc_model_tensor_info", SZ, C.c_void_p, SZ, C.c_char_p, SZ, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64),
        C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_int))
    sig("orc_model_synth", None, C.c_void_p, C.c_uint64, C.c_int)
    sig("orc_model_set_tensor", C.c_int, C.c_void_p, C.c_char_p, C.c_void_p, SZ, C.c_void_p, SZ)
    sig("orc_model_tensor_data", C.c_void_p, C.c_void_p, C.c_char_p)
    sig("orc_model_tensor_scale", C.c_void_p, C.c_void_p, C.c_char_p)
    sig("orc_model_begin", None, C.c_void_p, SZ, C.c_int, C.c_int)
    sig("orc_model_log_routes", None, C.c_void_p, C.c_int)
    sig("orc_model_pos", SZ, C.c_void_p)
    sig("orc_model_forward", C.c_int, C.c_void_p, U32P, SZ, F32P)
    sig("orc_model_route_log", SZ, C.c_void_p, C.c_void_p, SZ)
    sig("orc_model_clear_route_log", None, C.c_void_p)
    sig("orc_model_ssm_state", C.c_void_p, C.c_void_p, SZ)
    sig("orc_model_conv_state", C.c_void_p, C.c_void_p, SZ)
    sig("orc_model_k_slab", C.c_void_p, C.c_void_p, SZ)
    sig("orc_model_v_slab", C.c_void_p, C.c_void_p, SZ)
    sig("orc_model_generate", SZ, C.c_void_p, U32P, SZ, SZ, SZ, U32P, C.c_void_p)
    _LIB = L
    return L


def _fptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class OracleModel:
    """A synthetic model held by the oracle: CPU-generated (or externally supplied) weights, KV cache,
    recurrent state and the forward pass of src/model/qwen35.rs restated on the CPU."""

    def __init__(self, dims: ModelDims):
        self.L = lib()
        self.dims = dims
        self.h = self.L.orc_model_create(C.byref(dims))
        self.specs = []
        for i in range(self.L.orc_model_n_tensors(self.h)):
            name = C.create_string_buffer(128)
            ty, n_in, n_out, n_exp, hs = C.c_uint32(), C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_int()
            nbytes = self.L.orc_model_tensor_info(self.h, i, name, 128, C.byref(ty), C.byref(n_in), C.byref(n_out),
                                                  C.byref(n_exp), C.byref(hs))
            self.specs.append(dict(name=name.value.decode(), ty=ty.value, n_in=n_in.value, n_out=n_out.value,
                                   n_expert=n_exp.value, has_scale=bool(hs.value), bytes=nbytes))

    def __del__(self):
        if getattr(self, "h", None):
            self.L.orc_model_destroy(self.h); self.h = None

    def synth(self, seed, threads=8):
        self.L.orc_model_synth(self.h, seed, threads)

    def set_tensor(self, name, data: np.ndarray, scale=None):
        data = np.ascontiguousarray(data).view(np.uint8)
        self.L.orc_model_set_tensor(self.h, name.encode(), data.ctypes.data_as(C.c_void_p), data.size,
                                    _fptr(scale), 0 if scale is None else scale.size)

    def tensor(self, name):
        spec = next(s for s in self.specs if s["name"] == name)
        p = self.L.orc_model_tensor_data(self.h, name.encode())
        data = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(spec["bytes"],))
        sc = None
        if spec["has_scale"]:
            ps = self.L.orc_model_tensor_scale(self.h, name.encode())
            sc = np.ctypeslib.as_array(C.cast(ps, C.POINTER(C.c_float)), shape=(spec["n_expert"],))
        return data, sc

    def begin(self, n_ctx, kv_bf16=False, fp4act=False, log_routes=False):
        self.L.orc_model_begin(self.h, n_ctx, int(kv_bf16), int(fp4act))
        self.L.orc_model_log_routes(self.h, int(log_routes))

    def forward(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.uint32)
        logits = np.empty(self.dims.n_vocab, np.float32)
        rc = self.L.orc_model_forward(self.h, tokens, tokens.size, logits)
        if rc:
            raise RuntimeError(f"oracle forward failed: {rc}")
        return logits

    def generate(self, prompt, max_new, max_batch=512):
        prompt = np.ascontiguousarray(prompt, np.uint32)
        out = np.zeros(max_new, np.uint32)
        margins = np.zeros(max_new, np.float32)
        n = self.L.orc_model_generate(self.h, prompt, prompt.size, max_new, max_batch, out, _fptr(margins))
        return out[:n], margins[:n]

    def route_log(self):
        n = self.L.orc_model_route_log(self.h, None, 0)
        out = np.zeros(n, np.int32)
        self.L.orc_model_route_log(self.h, _fptr(out), n)
        return out

    def clear_route_log(self):
        self.L.orc_model_clear_route_log(self.h)

    def pos(self):
        return self.L.orc_model_pos(self.h)

    def ssm_state(self, il):
        d = self.dims
        n = d.ssm_d_state * (d.ssm_d_inner // d.ssm_dt_rank) * d.ssm_dt_rank
        return np.ctypeslib.as_array(C.cast(self.L.orc_model_ssm_state(self.h, il), C.POINTER(C.c_float)), shape=(n,))

    def conv_state(self, il):
        d = self.dims
        n = (d.ssm_d_conv - 1) * (2 * d.ssm_d_state * d.ssm_n_group + d.ssm_d_inner)
        return np.ctypeslib.as_array(C.cast(self.L.orc_model_conv_state(self.h, il), C.POINTER(C.c_float)), shape=(n,))
