"""The allocation-free decode-attention entry point against the ordinary one.

`itb_attend_decode_noalloc` exists for callers that may not allocate device memory while serving (an allocation
synchronises the whole device; some hosts also fix the backend's memory budget at start-up). It takes device
pointers the caller already owns and keeps its split-K partials in an array built into the library. This test
calls it through the C ABI twice in a row -- the second call reuses the scratch the first one left behind, at a
different length -- and checks both results against `itb_attend`, the entry point every other attention test uses.
It sits in a file of its own that pytest collects last.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
EPS = np.finfo(np.float32).eps


def test_no_alloc_attention_matches_the_ordinary_entry_point_twice_in_a_row():
    import torch
    from inferred_thoughts_b200 import host
    from tests.util import noise
    L = host.lib()
    L.itb_attend_decode_noalloc.restype = C.c_int
    ops = host.B200Ops(0)
    hd, nh, nkv = 256, 16, 2
    kvd = hd * nkv
    scale = 1.0 / np.sqrt(hd)
    keep = []
    for call, n_pos in enumerate((1500, 333)):
        n_ctx = n_pos + 4
        q = noise(nh * hd, 900 + call)
        ks = (noise(n_ctx * kvd, 910 + call)).astype(np.float16).view(np.uint16)
        vs = (noise(n_ctx * kvd, 920 + call)).astype(np.float16).view(np.uint16)
        keep += [q, ks, vs]
        want = np.zeros(nh * hd, np.float32)
        ops.begin_pass(1)
        ops.attend(q, ks, vs, kvd, n_pos, hd, nh, nkv, scale, want); ops.host_needs(want); ops.check()
        # device buffers owned by the caller (torch stands in for that caller's allocator)
        qd = torch.from_numpy(q).cuda()
        kd = torch.from_numpy(ks.view(np.int16)).cuda()
        vd = torch.from_numpy(vs.view(np.int16)).cuda()
        od = torch.full((nh * hd,), float("nan"), device="cuda")
        err = C.create_string_buffer(256)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = L.itb_attend_decode_noalloc(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.c_void_p(qd.data_ptr()),
                                         C.c_void_p(kd.data_ptr()), C.c_void_p(vd.data_ptr()), C.c_size_t(kvd), C.c_size_t(n_pos),
                                         C.c_size_t(hd), C.c_size_t(nh), C.c_size_t(nkv), C.c_float(scale), 0, C.c_void_p(od.data_ptr()),
                                         err, C.c_size_t(256))
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        if call == 1:   # the first call may load the module image; later calls must leave free memory alone
            assert torch.cuda.mem_get_info()[0] == free_before
        got = od.cpu().numpy()
        # both paths are the same split-K algorithm with different split counts: the attention tests' bound
        tol = (7 + 64 + 4 + np.log2(n_pos)) * EPS * 4 * 4.0
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= tol, (call, float(np.abs(got - want).max()), tol)
    # sizes beyond the built-in scratch are refused with a message, and nothing runs
    err = C.create_string_buffer(256)
    rc = L.itb_attend_decode_noalloc(None, C.c_void_p(qd.data_ptr()), C.c_void_p(kd.data_ptr()), C.c_void_p(vd.data_ptr()), C.c_size_t(kvd),
                                     C.c_size_t(10), C.c_size_t(hd), C.c_size_t(128), C.c_size_t(16), C.c_float(scale), 0,
                                     C.c_void_p(od.data_ptr()), err, C.c_size_t(256))
    assert rc == 1 and b"exceeds the built-in scratch" in err.value
    # so are a row stride or a slab address the kernel's vector loads could not take
    for kv_dim_bad, k_off, want_msg in ((kvd + 4, 0, b"multiple of head_dim/32"), (kvd, 2, b"aligned")):
        err = C.create_string_buffer(256)
        rc = L.itb_attend_decode_noalloc(None, C.c_void_p(qd.data_ptr()), C.c_void_p(kd.data_ptr() + k_off), C.c_void_p(vd.data_ptr()),
                                         C.c_size_t(kv_dim_bad), C.c_size_t(10), C.c_size_t(hd), C.c_size_t(nh), C.c_size_t(nkv), C.c_float(scale), 0,
                                         C.c_void_p(od.data_ptr()), err, C.c_size_t(256))
        assert rc == 1 and want_msg in err.value, err.value
    ops.check(); ops.close()
