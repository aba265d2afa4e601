"""One multi-row pass of the engine inside a CUDA profiler range, for `ncu --profile-from-start off`.

    python -m inferred_thoughts_b200.probe decode  <n_seq>  [n_layer]   one batched decode step of n_seq sequences
    python -m inferred_thoughts_b200.probe prefill <n_tok>  [n_layer]   one prefill pass of n_tok rows of one sequence
    python -m inferred_thoughts_b200.probe timeline <n_pos> [n_layer]   phase timeline of one fused one-token step at n_pos

The model is the 35B-A3B shape with n_layer layers (default 8: about 5 GB on the device, small enough for a
multi-pass capture). Prints the pass's device time.
"""
import sys

import numpy as np


def main(argv):
    import torch
    from . import configs, host
    mode, n = argv[0], int(argv[1])
    dims = configs.with_layers(dict(configs.M35B), int(argv[2]) if len(argv) > 2 else 8)
    ops = host.B200Ops(0, "kv=bf16,exact=0")
    model = host.Model(ops, host.ModelDims(**dims)); model.synth(configs.SEEDS["m35b"])
    rng = np.random.default_rng(3)
    if mode == "decode":
        eng = host.Engine(model, 2048, n)
        eng.prefill(rng.integers(0, dims["n_vocab"], (n, 64)).astype(np.uint32), want_logits=False)
        t = eng.decode_loop(np.zeros(n, np.uint32), 2)[-1]
        torch.cuda.synchronize(); torch.cuda.profiler.start()
        eng.decode_loop(t, 1)
        torch.cuda.synchronize(); torch.cuda.profiler.stop()
    elif mode == "prefill":
        eng = host.Engine(model, 2048, 1)
        pr = rng.integers(0, dims["n_vocab"], n).astype(np.uint32)
        eng.prefill(pr[:32], want_logits=False); eng.reset()
        torch.cuda.synchronize(); torch.cuda.profiler.start()
        eng.prefill(pr, want_logits=False)
        torch.cuda.synchronize(); torch.cuda.profiler.stop()
    elif mode == "timeline":
        timeline(host, model, dims, n)
        model.close(); ops.close()
        return
    else:
        raise SystemExit(__doc__)
    print(f"{mode} {n}: {eng.last_ms():.3f} ms")
    eng.close(); model.close(); ops.close()


KERNELS = {2: "k_in_proj", 3: "k_gdn_core", 4: "k_out_proj", 5: "k_attn_prep", 8: "k_moe_glu", 9: "k_moe_down"}


def timeline(host, model, dims, n_pos):
    """itb_timeline_arm / itb_timeline_read around one step replayed from the CUDA graph: per structured launch, the time from
    one phase mark to the next on block 0 (us), and from the previous launch's last mark to this one's first mark after its
    dependency wait (the gap)."""
    import collections
    import ctypes as C
    eng = host.Engine(model, max(2048, n_pos + 64), 1)
    eng.prefill((np.arange(n_pos, dtype=np.uint32) * 7919) % dims["n_vocab"], want_logits=False)
    t = eng.decode_loop([1], 8)[-1]
    L = eng.L
    L.itb_timeline_read.restype = C.c_long
    slots = 8 * dims["n_layer"] + 8
    assert L.itb_timeline_arm(eng.h, slots) == 0
    eng.decode_loop(t, 1)
    words = np.zeros(slots * 16, np.uint64)
    L.itb_timeline_read(eng.h, C.c_void_p(words.ctypes.data), slots)
    L.itb_timeline_arm(eng.h, 0)
    agg = collections.OrderedDict()
    prev_last = None
    for w in words.reshape(slots, 16):
        marks = {i: int(v) >> 8 for i, v in enumerate(w) if v}
        if not marks:
            continue
        name = KERNELS.get(int(w[w != 0][0]) & 255, "?")
        order = sorted(marks.items(), key=lambda x: x[1])
        for (i, a), (j, b) in zip(order, order[1:]):
            agg.setdefault((name, f"phase {i}->{j}"), []).append((b - a) / 1e3)
        if prev_last is not None and 1 in marks:
            agg.setdefault((name, "gap before"), []).append((marks[1] - prev_last) / 1e3)
        prev_last = max(marks.values())
    for (name, what), v in sorted(agg.items()):
        print(f"{name:12s} {what:14s} n={len(v):3d} mean {np.mean(v):6.2f} us  min {np.min(v):6.2f}  max {np.max(v):6.2f}")
    eng.close()


if __name__ == "__main__":
    main(sys.argv[1:])
