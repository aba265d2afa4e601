"""Host side of expert parallelism on CPU: the expert ranges, and the communicator id reaching every rank of a
world_size-2 gloo group (the id itself comes from a stand-in library: NCCL needs a GPU)."""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch.multiprocessing as mp

from inferred_thoughts_b200 import host


def test_expert_ranges_tile_the_experts():
    for world in (1, 2, 4, 8):
        got = [host.expert_range(r, world, 256) for r in range(world)]
        assert got[0][0] == 0 and got[-1][1] == 256
        assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
        assert len({hi - lo for lo, hi in got}) == 1
    with pytest.raises(ValueError):
        host.expert_range(0, 3, 256)
    with pytest.raises(ValueError):
        host.expert_range(2, 2, 256)


class _FakeLib:
    """itb_ep_unique_id of a library that needs no GPU: 128 recognisable bytes."""
    def itb_ep_unique_id(self, out):
        C.memmove(out, bytes(range(128)), 128)
        return 0


def _rank(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    uid = host.share_unique_id(rank, lib_=_FakeLib() if rank == 0 else None)
    q.put((rank, uid))
    dist.destroy_process_group()


def test_unique_id_reaches_every_rank_over_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = dict(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(60); assert p.exitcode == 0
    assert got[0] == got[1] == bytes(range(128))


def _a2a_rank(rank, world, port, q):
    """One rank of the packed all-to-all on CPU: route random pairs, exchange the counts, plan, dispatch the pairs' tags with
    point-to-point messages sized by the plan, "serve" them (tag -> tag * 3 + 1), combine back, unsort."""
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n_expert, rows, k = 64, 37, 4
    lo, hi = host.expert_range(rank, world, n_expert)
    rng = np.random.default_rng(7 + rank)
    ids = rng.integers(0, n_expert, rows * k).astype(np.int64)
    if rank == 1:
        ids[:] = ids % (n_expert // world)                      # rank 1 sends everything to rank 0: an empty message one way
    owner = ids // (n_expert // world)
    order = np.argsort(owner, kind="stable")                    # owner order, pair order inside an owner: what the device sort gives
    tags = (rank * 100000 + np.arange(rows * k)).astype(np.int64)
    mine = torch.tensor(np.bincount(owner, minlength=world).astype(np.int32))
    allc = [torch.zeros(world, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(allc, mine)
    cnt = np.stack([c.numpy() for c in allc])
    so, ro, n_recv = host.ep_a2a_plan(cnt, rank)
    assert so[-1] == rows * k and n_recv == int(cnt[:, rank].sum())
    send_tags, send_ids = torch.tensor(tags[order]), torch.tensor(ids[order])
    recv_tags, recv_ids = torch.zeros(n_recv, dtype=torch.int64), torch.zeros(n_recv, dtype=torch.int64)
    reqs = []
    for r in range(world):
        if r == rank:
            recv_tags[ro[r]:ro[r + 1]] = send_tags[so[r]:so[r + 1]]; recv_ids[ro[r]:ro[r + 1]] = send_ids[so[r]:so[r + 1]]
            continue
        if so[r + 1] > so[r]:
            reqs += [dist.isend(send_tags[so[r]:so[r + 1]].clone(), r, tag=1), dist.isend(send_ids[so[r]:so[r + 1]].clone(), r, tag=2)]
        if ro[r + 1] > ro[r]:
            reqs += [dist.irecv(recv_tags[ro[r]:ro[r + 1]], r, tag=1), dist.irecv(recv_ids[ro[r]:ro[r + 1]], r, tag=2)]
    for w in reqs:
        w.wait()
    assert ((recv_ids >= lo) & (recv_ids < hi)).all(), "a received pair names an expert stored elsewhere"
    served = recv_tags * 3 + 1
    back = torch.zeros(rows * k, dtype=torch.int64)
    reqs = []
    for r in range(world):
        if r == rank:
            back[so[r]:so[r + 1]] = served[ro[r]:ro[r + 1]]
            continue
        if ro[r + 1] > ro[r]:
            reqs.append(dist.isend(served[ro[r]:ro[r + 1]].clone(), r, tag=3))
        if so[r + 1] > so[r]:
            reqs.append(dist.irecv(back[so[r]:so[r + 1]], r, tag=3))
    for w in reqs:
        w.wait()
    out = np.zeros(rows * k, np.int64)
    out[order] = back.numpy()
    q.put((rank, bool((out == tags * 3 + 1).all())))
    dist.destroy_process_group()


def test_packed_all_to_all_plan_round_trip_over_gloo():
    """The dispatch/combine of expert-parallel many-row passes, host side: counts -> plan -> messages of exactly the planned
    sizes (one direction empty) -> every pair's result back in its own place, on a world_size-2 gloo group."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_a2a_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = dict(q.get(timeout=180) for _ in ps)
    for p in ps:
        p.join(60); assert p.exitcode == 0
    assert got == {0: True, 1: True}


def test_all_to_all_plan_refuses_bad_input():
    with pytest.raises(ValueError):
        host.ep_a2a_plan(np.array([[1, -1], [0, 2]]), 0)
    with pytest.raises(ValueError):
        host.ep_a2a_plan(np.array([[1, 1], [0, 2]]), 2)
    so, ro, n = host.ep_a2a_plan(np.array([[3, 1, 0], [2, 0, 5], [0, 4, 1]]), 1)
    assert so.tolist() == [0, 2, 2, 7] and ro.tolist() == [0, 1, 1, 5] and n == 5
