// GCLOCK residency policy for routed experts kept in pinned host memory with a cache of slots in HBM (the reference's
// expert tiers: src/cache GCLOCK, src/ops/cuda/experts.rs:2179-2234 there). Host-only, no CUDA: every key is a
// (layer, expert) number, every slot holds one key. A touch either finds the key (its counter goes up, capped) or
// takes a victim: the hand sweeps the slots, decrementing counters, and stops at the first slot that is empty or at
// zero and not leased. Keys touched in the current pass are leased until the pass ends, so a pass never evicts what
// it is about to use.
#pragma once
#include <cstdint>
#include <vector>

struct GClock {
    static constexpr uint8_t MAX_COUNT = 3;
    struct Slot { int64_t key = -1; uint8_t count = 0; uint64_t lease = 0; };
    std::vector<Slot> slots;
    std::vector<int32_t> slot_of;      // key -> slot or -1
    size_t hand = 0;
    uint64_t pass = 1;                 // current lease epoch
    uint64_t hits = 0, misses = 0, evictions = 0;

    GClock(size_t capacity, size_t n_keys) : slots(capacity), slot_of(n_keys, -1) {}
    void next_pass() { ++pass; }
    // Returns the key's slot (>= 0) and sets *hit; *evicted = the key that lost the slot or -1. Returns -1 when every
    // slot is leased by this pass (the pass needs more distinct keys than there are slots).
    int touch(int64_t key, bool* hit, int64_t* evicted) {
        *evicted = -1;
        int s = slot_of[(size_t)key];
        if (s >= 0) {
            Slot& sl = slots[(size_t)s];
            if (sl.count < MAX_COUNT) ++sl.count;
            sl.lease = pass; *hit = true; ++hits;
            return s;
        }
        *hit = false;
        const size_t n = slots.size();
        for (size_t tries = 0; tries < (size_t)(MAX_COUNT + 2) * n; ++tries) {
            Slot& sl = slots[hand];
            const size_t at = hand;
            hand = (hand + 1) % n;
            if (sl.lease == pass) continue;
            if (sl.key >= 0 && sl.count > 0) { --sl.count; continue; }
            if (sl.key >= 0) { slot_of[(size_t)sl.key] = -1; *evicted = sl.key; ++evictions; }
            sl.key = key; sl.count = 1; sl.lease = pass;
            slot_of[(size_t)key] = (int32_t)at;
            ++misses;
            return (int)at;
        }
        return -1;
    }
    // A guess, not a use: bring `key` in if it is absent and a slot can be had without touching this pass's leases. The
    // entry starts at count 0 (the first to go if the guess was wrong) and is leased like any other until the pass ends,
    // so the copy in flight is not overwritten. Returns the slot to fill, or -1 (already resident, or no slot). Hits and
    // misses are not counted: a guess is neither.
    int prefetch(int64_t key, int64_t* evicted) {
        *evicted = -1;
        if (slot_of[(size_t)key] >= 0) return -1;
        const size_t n = slots.size();
        for (size_t tries = 0; tries < 2 * n; ++tries) {
            Slot& sl = slots[hand];
            const size_t at = hand;
            hand = (hand + 1) % n;
            if (sl.lease == pass) continue;
            if (sl.key >= 0 && sl.count > 0) { --sl.count; continue; }
            if (sl.key >= 0) { slot_of[(size_t)sl.key] = -1; *evicted = sl.key; ++evictions; }
            sl.key = key; sl.count = 0; sl.lease = pass;
            slot_of[(size_t)key] = (int32_t)at;
            return (int)at;
        }
        return -1;
    }
};
