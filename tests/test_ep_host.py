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
