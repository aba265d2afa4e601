"""One multi-row pass of the engine inside a CUDA profiler range, for `ncu --profile-from-start off`.

    python -m inferred_thoughts_b200.probe decode  <n_seq>  [n_layer]   one batched decode step of n_seq sequences
    python -m inferred_thoughts_b200.probe prefill <n_tok>  [n_layer]   one prefill pass of n_tok rows of one sequence

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
    else:
        raise SystemExit(__doc__)
    print(f"{mode} {n}: {eng.last_ms():.3f} ms")
    eng.close(); model.close(); ops.close()


if __name__ == "__main__":
    main(sys.argv[1:])
