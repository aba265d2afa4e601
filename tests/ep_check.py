"""Expert-parallel parity check, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
        -m tests.ep_check

Each rank builds (a) the whole `configs.MID` model and a single-GPU engine and (b) its expert shard and an
expert-parallel engine, runs the same prompts and decode steps through both on ITS OWN sequences, and requires the
logits to be bit-identical. Then one rank alone is handed a token id outside the vocabulary: every rank must get an
error back (the ranks agree before anything is enqueued) and the engines must still work afterwards.
Exit code 0 and one line "ep_check ok" per rank on success.
"""
import os
import sys

import numpy as np


def main():
    import torch
    import torch.distributed as dist
    from inferred_thoughts_b200 import configs, host
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo")          # host-side rendezvous only; the data path is the library's own NCCL communicator
    dims = dict(configs.MID)
    seed = configs.SEEDS["mid"]
    ops = host.B200Ops(dev, "exact=1")
    full = host.Model(ops, host.ModelDims(**dims)); full.synth(seed)
    lo, hi = host.expert_range(rank, world, dims["n_expert"])
    shard = host.Model(ops, host.ModelDims(**dims)); shard.synth(seed, lo, hi)
    ok = True
    rng = np.random.default_rng(100 + rank)                 # every rank its own sequences
    for n_seq in (3, 1):                                     # 3: the multi-row passes and steps; 1: the fused one-token step
        prompts = rng.integers(0, dims["n_vocab"], (n_seq, 40)).astype(np.uint32)
        e1 = host.Engine(full, 128, n_seq)
        e2 = host.Engine(shard, 128, n_seq, ep=(rank, world, host.share_unique_id(rank)))
        # steps of one sequence (fused one-token kernels) and of several (multi-row kernels) both exchange through peer memory
        want = "nccl" if os.environ.get("ITB_EP_P2P") == "0" else "peer-memory"
        ok = ok and e2.ep_step_transport() == want
        a, b = e1.prefill(prompts), e2.prefill(prompts)
        a, b = np.atleast_2d(a), np.atleast_2d(b)
        ok = ok and a.view(np.uint32).tolist() == b.view(np.uint32).tolist()
        toks = np.argmax(a, 1).astype(np.uint32)
        for _ in range(6):
            (la, na), (lb, nb) = e1.decode(toks), e2.decode(toks)
            ok = ok and la.view(np.uint32).tolist() == lb.view(np.uint32).tolist() and na.tolist() == nb.tolist()
            toks = na
        L, K = dims["n_layer"], dims["n_expert_used"]
        ok = ok and e1.read_routes(L, K).tolist() == e2.read_routes(L, K).tolist()
        ops.check()
        if n_seq == 1:
            # a failure on ONE rank: rank 0 passes a bad token; no rank may enter the layer's collectives alone
            bad = np.array([dims["n_vocab"] + 5], np.uint32) if rank == 0 else toks
            refused = False
            try:
                e2.decode(bad)
            except RuntimeError as ex:
                refused = True
                msg = str(ex)
                ok = ok and (("out of range" in msg) if rank == 0 else ("refused this call" in msg))
            ok = ok and refused
            (la, na), (lb, nb) = e1.decode(toks), e2.decode(toks)      # and the next step is in step again on every rank
            ok = ok and la.view(np.uint32).tolist() == lb.view(np.uint32).tolist()
        e2.close(); e1.close()
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    shard.close(); full.close(); ops.close()
    dist.destroy_process_group()
    if not ok:
        print(f"ep_check FAILED on rank {rank}", flush=True)
        sys.exit(1)
    print(f"ep_check ok rank {rank}/{world} experts [{lo},{hi})", flush=True)
    sys.exit(0 if int(flag) else 1)


if __name__ == "__main__":
    main()
