"""Expert tiering: the GCLOCK policy on CPU (no device), the tiered engine against the plain one on the GPU."""
import ctypes as C

import numpy as np
import pytest

from tests.util import TINY, host_dims, prompt_ids


class Clock:
    def __init__(self, capacity, n_keys):
        from inferred_thoughts_b200 import host
        self.L = host.lib()
        self.g = C.c_void_p(self.L.itb_gclock_create(capacity, n_keys))

    def touch(self, key):
        hit, ev = C.c_int(0), C.c_int64(-1)
        slot = self.L.itb_gclock_touch(self.g, C.c_int64(key), C.byref(hit), C.byref(ev))
        return slot, bool(hit.value), ev.value

    def next_pass(self): self.L.itb_gclock_next_pass(self.g)
    def close(self): self.L.itb_gclock_destroy(self.g)


def test_gclock_fills_hits_and_evicts_the_coldest():
    g = Clock(3, 10)
    assert [g.touch(k)[:2] for k in (0, 1, 2)] == [(0, False), (1, False), (2, False)]       # empty slots first, in hand order
    g.next_pass()
    assert g.touch(0) == (0, True, -1) and g.touch(0) == (0, True, -1)                        # counter of key 0 goes to 3
    g.next_pass()
    # the sweep passes 0 (count 3 -> 2), 1 (1 -> 0), 2 (1 -> 0), 0 (2 -> 1), then takes key 1's slot
    assert g.touch(3) == (1, False, 1)
    assert g.touch(1) == (2, False, 2)                                                        # 3 is leased; 2 is at zero
    g.next_pass()
    assert g.touch(0)[1] and g.touch(3)[1] and g.touch(1)[1]
    assert g.touch(99)[0] == -2                                                               # key out of range
    g.close()


def test_gclock_never_evicts_what_the_pass_uses():
    g = Clock(2, 8)
    assert g.touch(5)[1] is False and g.touch(6)[1] is False
    assert g.touch(7)[0] == -1                 # both slots leased by this pass: the caller must cut the pass
    g.next_pass()
    slot, hit, ev = g.touch(7)
    assert slot >= 0 and not hit and ev in (5, 6)
    g.close()


@pytest.mark.gpu
@pytest.mark.parametrize("capacity", [8, 20, 64])
def test_tiered_engine_equals_plain_engine(capacity):
    """TINY has 4 layers x 16 experts = 64 (layer, expert) entries, 4 picks per token: a pool of 8 holds two rows' picks and
    evicts constantly, 20 evicts sometimes, 64 holds everything. Logits must equal the plain engine's, bit for bit."""
    from inferred_thoughts_b200 import host
    ops = host.B200Ops(0, "exact=1")
    plain = host.Model(ops, host_dims(TINY)); plain.synth(0)
    cold = host.Model(ops, host_dims(TINY)); cold.synth(0); cold.offload_experts()
    with pytest.raises(RuntimeError):
        host.Engine(cold, 64, 1)               # a plain engine cannot run a model whose experts left the device
    e1, e2 = host.Engine(plain, 64, 1), host.Engine(cold, 64, 1, tier_capacity=capacity)
    prompt = prompt_ids(11, 30, TINY["n_vocab"])
    a, b = e1.prefill(prompt), e2.prefill(prompt)
    assert a.view(np.uint32).tolist() == b.view(np.uint32).tolist()
    t = int(np.argmax(a))
    for _ in range(8):
        (la, na), (lb, nb) = e1.decode([t]), e2.decode([t])
        assert la.view(np.uint32).tolist() == lb.view(np.uint32).tolist() and na[0] == nb[0]
        t = int(na[0])
    st = e2.tier_stats()
    print(capacity, st)
    assert st["hits"] > 0 and st["misses"] > 0 and st["bytes_moved"] > 0
    if capacity == 64:
        assert st["evictions"] == 0 and st["misses"] <= 64
    if capacity == 8:
        assert st["evictions"] > st["misses"] // 2
    ops.check()
    e1.close(); e2.close(); cold.close(); plain.close(); ops.close()
