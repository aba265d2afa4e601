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


@pytest.mark.gpu
@pytest.mark.parametrize("prefetch", [0, 8])
def test_tiered_engine_against_the_oracle_with_and_without_the_prefetch_hint(prefetch):
    """The tiered engine against the CPU oracle (not against another engine): prompt logits, teacher-forced decode logits and
    routing ids bit for bit on the tiny model with a pool of 24 of its 64 (layer, expert) entries. With the prefetch hint on
    (8 guesses per row for the next layer, copied on a second stream) nothing the model computes may change; the counters
    must show the guesses being made and some of them being used, and must add up."""
    import os
    from inferred_thoughts_b200 import host
    from oracle import oracle_py as O
    from tests.util import oracle_dims
    ops = host.B200Ops(0, "exact=1")
    cold = host.Model(ops, host_dims(TINY)); cold.synth(0)
    om = O.OracleModel(oracle_dims(TINY))
    for sp in om.specs:
        data, sc = cold.synth_read(0, sp["name"], sp["bytes"], sp["n_expert"] if sp["has_scale"] else 0)
        om.set_tensor(sp["name"], data, sc)
    cold.offload_experts()
    if prefetch:
        os.environ["ITB_TIER_PREFETCH"] = str(prefetch)
    try:
        eng = host.Engine(cold, 64, 1, tier_capacity=24)
    finally:
        os.environ.pop("ITB_TIER_PREFETCH", None)
    L, K = TINY["n_layer"], TINY["n_expert_used"]
    prompt = prompt_ids(12, 30, TINY["n_vocab"])
    om.begin(64, log_routes=True)
    o = om.forward(prompt); g = eng.prefill(prompt)
    assert o.view(np.uint32).tolist() == g.view(np.uint32).tolist(), "prompt logits"
    for step in range(10):
        t = int(np.argmax(o))
        om.clear_route_log()
        o = om.forward([t]); lg, _ = eng.decode([t])
        assert o.view(np.uint32).tolist() == lg[0].view(np.uint32).tolist(), f"decode step {step}"
        assert eng.read_routes(L, K)[:, 0, :].tolist() == om.route_log().reshape(L, K).tolist(), f"routing at step {step}"
    c, st = eng.tier_counters(), eng.tier_stats()
    print(prefetch, c)
    assert c["lookups"] == st["hits"] + st["misses"] and c["host_reads"] == st["misses"]
    assert c["fetch_bytes"] == st["bytes_moved"] and c["fetched"] * c["slot_bytes"] == c["fetch_bytes"]
    assert c["slots"] == 24 and c["pool_bytes"] == 24 * c["slot_bytes"] and c["vram_total"] > c["vram_free"] > 0
    assert c["resident_bytes"] >= c["weight_bytes"] + c["kv_bytes"] + c["pool_bytes"] and c["kv_bytes"] > 0
    if prefetch:
        assert c["prefetch_reads"] > 0 and 0 < c["prefetch_used"] <= c["prefetch_reads"]
        assert c["fetched"] == c["host_reads"] + c["prefetch_reads"]
    else:
        assert c["prefetch_reads"] == 0 and c["prefetch_used"] == 0 and c["fetched"] == c["host_reads"]
    ops.check()
    eng.close(); cold.close(); ops.close()
