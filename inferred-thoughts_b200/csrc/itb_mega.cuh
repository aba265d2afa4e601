// One decode step as ONE persistent kernel: a block per SM walks the step's stages (the same dependent stages the fused
// kernels of itb_fused.cuh run as separate launches) with a grid barrier between them, while a producer warp per block
// streams the block's share of every stage's weights through a shared-memory ring with bulk asynchronous copies
// (cp.async.bulk, completed on mbarriers). Weights do not depend on activations, so the ring runs ahead of the dependency
// chain: while the consumer warps wait at a barrier or run a prologue, HBM keeps streaming the next stages' rows.
// Routed-expert rows, whose addresses depend on this token's routing, go through a second ring that starts the moment
// the ids exist.
//
// Arithmetic is that of the fused kernels, value for value: integer dots per quantisation block, f32 terms folded in
// ascending order by one lane per row (src/ops/naive.rs:691-734), f64 sums where the CPU path has them.
//
// Every wait in this file is bounded: mbarrier polls and grid-barrier polls give up after the wait limit, record a status
// word (stage << 8 | reason) that the host turns into an error, tell the rest of the block and of the grid, wait (bounded
// again) for the block's own copies in flight, and return. A consumer thread whose wait failed does not leave its stage: it
// skips the work that needed the data and keeps the stage's control flow, so the block's named barriers stay matched; the
// decision to stop is taken by thread 0 at the next grid barrier and read by everyone after that barrier's own sync.
#pragma once
#include "itb_fused.cuh"

namespace {

constexpr int MG_NW = 16;                    // consumer warps per block
constexpr int MG_CT = MG_NW * 32;            // consumer threads
constexpr int MG_THREADS = MG_CT + 64;       // + one producer warp per ring
constexpr int MG_MAX_SLOTS = 8;
constexpr unsigned long long MG_WAIT_NS = 2000000000ull;   // default limit of a wait, 2 s: far beyond any legitimate wait inside a step
constexpr int MG_ATTN_MIN_SPLIT = 32;        // positions per attention split at least
constexpr int MG_MAX_LOCAL_HEADS = 8;        // delta-rule heads one block's rows may touch

enum { MS_EMBED = 1, MS_ROWS, MS_GDN, MS_OUT, MS_ATTN_PREP, MS_ATTN_PART, MS_ATTN_COMB, MS_GLU, MS_DOWN, MS_ADVANCE };
enum { MGE_FULL_WAIT = 1, MGE_EMPTY_WAIT, MGE_GRID_WAIT, MGE_IDS_WAIT, MGE_DRAIN_WAIT, MGE_SHAPE };
enum { MSF_ARGMAX = 1, MSF_OUT_ATTN = 2 };

struct MStage {
    int type, flags;
    const float* norm_w;
    int nq, nf;
    DevQ8 q[3]; float* qout[3];
    DevF32 f[2]; float* fout[2];
    const float* conv_w; float* conv_state;                          // MS_ROWS of a recurrent layer
    const float *ssm_a, *dt_bias, *ssm_norm; float* state;           // MS_GDN, MS_OUT (recurrent flavour)
    DevQ8 w;                                                         // MS_OUT: the output projection
    const float *q_norm, *k_norm; uint16_t *kslab, *vslab;           // attention stages
    DevFp4 gate, up, down; DevQ8 shared_down;                        // MS_GLU, MS_DOWN
    int32_t* ids_out; float* w_out;
};

struct MegaParams {
    const MStage* stages; int n_stages;
    int H, n_vocab, cd, vd, key_dim, sk, n_k, n_v, conv_kernel, qd, kvd, hd, n_head, n_head_kv, n_rot, n_expert, n_used, ff, sff, n_ctx;
    float eps, theta; int exact, kv_bf16;
    const float* tok_embd;
    float *x, *qkvc, *z, *alpha, *beta, *core, *qg, *kbuf, *vbuf, *qn, *gate, *part_acc, *part_ml, *router, *shlogit, *sg, *su, *logits;
    int8_t *aq, *hq, *sq; float *as, *hs, *ss;
    int32_t* tokens; int* pos; int32_t* next; int32_t* history; int history_cap; int* step_counter;
    float* arg_v; int* arg_i;
    unsigned* bar; unsigned* done; int* err;
    int n_split;                                                     // attention splits (partials are [n_head][n_split])
    unsigned long long wait_ns;                                      // limit of every wait
    int test_stall;                                                  // tests of the bounded waits: the first layer's picks are never published
    int off_act, off_terms, off_ring_a, off_ring_b, ns_a, ns_b, slot_a, slot_b, tw_floats;   // dynamic shared-memory layout
};

// ------------------------------------------------------------------------------------------------ primitives
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t a, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t a, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t a) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint32_t a, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    return ok != 0;
}
// Bulk asynchronous copy global -> this block's shared memory (no multicast); completes `bytes` on the mbarrier.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ unsigned long long gtimer() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;" ::"n"(MG_CT) : "memory"); }   // the consumer warps only
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) { unsigned v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void red_release(unsigned* p, unsigned v) { asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
// activations written by other blocks of this launch: read around the (incoherent) L1
__device__ __forceinline__ float ldg_f(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float4 ldg_f4(const float* p) { return __ldcg((const float4*)p); }

// Block-wide control words in static shared memory.
struct MegaCtl {
    volatile int abort_;             // set by whoever gave up; every wait loop of the block looks at it
    int go;                          // thread 0's reading of !abort_ at the last grid barrier: the consumers' uniform decision to go on
    int ids[16];                     // this token's picks, for the expert ring's producer
    unsigned long long bars[2 * MG_MAX_SLOTS * 2 + 2];   // ring A full/empty, ring B full/empty, ids-ready, ids-taken
};

struct Ring {
    uint32_t base, full, empty;      // shared-space addresses
    int ns, slot_bytes;
    uint32_t n;                      // chunks produced / consumed so far on this side
    __device__ __forceinline__ uint32_t slot() const { return n % (uint32_t)ns; }
    __device__ __forceinline__ uint32_t phase() const { return (n / (uint32_t)ns) & 1u; }
    __device__ __forceinline__ uint32_t slot_addr() const { return base + slot() * (uint32_t)slot_bytes; }
    __device__ __forceinline__ uint32_t full_bar() const { return full + slot() * 8u; }
    __device__ __forceinline__ uint32_t empty_bar() const { return empty + slot() * 8u; }
};

__device__ __noinline__ void mg_fail(const MegaParams& p, MegaCtl* ctl, int stage, int reason) {
    atomicCAS(p.err, 0, (stage << 8) | reason);
    ctl->abort_ = 1;
    __threadfence();
}
// Wait for an mbarrier phase. false: gave up (time limit, or somebody else of the block or grid did).
__device__ __forceinline__ bool mg_wait(const MegaParams& p, MegaCtl* ctl, uint32_t bar, uint32_t parity, int stage, int reason) {
    if (mbar_try(bar, parity)) return true;
    const unsigned long long t0 = gtimer();
    for (unsigned it = 1;; ++it) {
        if (mbar_try(bar, parity)) return true;
        if (ctl->abort_) return false;
        if ((it & 255u) == 0) {
            if (*(volatile int*)p.err) { ctl->abort_ = 1; return false; }
            if (gtimer() - t0 > p.wait_ns) { mg_fail(p, ctl, stage, reason); return false; }
        }
    }
}

// The same for a whole (converged) warp: lane 0 polls, the other lanes wait at the shuffle and issue nothing meanwhile.
__device__ __forceinline__ bool mg_wait_warp(const MegaParams& p, MegaCtl* ctl, uint32_t bar, uint32_t parity, int stage, int reason) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mg_wait(p, ctl, bar, parity, stage, reason) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Grid barrier k (0-based) of this launch, consumer warps only: arrive once per block, poll until every block has.
__device__ __forceinline__ bool mg_grid_barrier(const MegaParams& p, MegaCtl* ctl, unsigned k, int stage) {
    csync();
    if (threadIdx.x == 0) {
        __threadfence();
        red_release(p.bar, 1u);
        const unsigned target = (k + 1u) * gridDim.x;
        if (ld_acquire(p.bar) < target) {
            const unsigned long long t0 = gtimer();
            for (unsigned it = 1; ld_acquire(p.bar) < target; ++it) {
                if (ctl->abort_) break;
                if ((it & 63u) == 0) {
                    if (*(volatile int*)p.err) { ctl->abort_ = 1; break; }
                    if (gtimer() - t0 > p.wait_ns) { mg_fail(p, ctl, stage, MGE_GRID_WAIT); break; }
                }
            }
        }
        __threadfence();
        ctl->go = !ctl->abort_;
    }
    csync();
    return ctl->go != 0;
}

// ------------------------------------------------------------------------------------------------ row plans
// Rows [r0, r1) of a matrix belong to this block; they travel in chunks of `rc` rows: plane A rows (ra bytes each) then
// plane B rows (rb bytes each) in one ring slot. Producer and consumers derive the same plan from the same numbers.
struct RowPlan { int r0, r1, rc, nchunks; uint32_t ra, rb; };
__device__ __forceinline__ RowPlan row_plan(int n_out, uint32_t ra, uint32_t rb, int slot_bytes) {
    RowPlan pl;
    share(n_out, gridDim.x, blockIdx.x, pl.r0, pl.r1);
    pl.ra = ra; pl.rb = rb;
    pl.rc = max(1, min(2 * MG_NW, slot_bytes / (int)(ra + rb)));
    pl.nchunks = (pl.r1 - pl.r0 + pl.rc - 1) / pl.rc;
    return pl;
}
__device__ __forceinline__ RowPlan q8_plan(const DevQ8& w, int slot_bytes) { return row_plan(w.n_out, (uint32_t)w.n_in, (uint32_t)w.n_in / 16, slot_bytes); }
__device__ __forceinline__ RowPlan f32_plan(const DevF32& w, int slot_bytes) { return row_plan(w.n_out, (uint32_t)w.n_in * 4, 0, slot_bytes); }

// Units of the gated expert half: unit u = (pick, 32 h-rows); after them one unit per 32 elements of the shared
// expert's activation. Units are dealt round-robin to the blocks.
__device__ __forceinline__ int glu_units(const MegaParams& p) { return p.n_used * (p.ff / 32); }
// Down projection: this block's output rows [o0, o1), `pc` picks per chunk.
struct DownPlan { int o0, o1, nr, pc, nchunks; uint32_t ra, rb; };
__device__ __forceinline__ DownPlan down_plan(const MegaParams& p) {
    DownPlan d;
    share(p.H, gridDim.x, blockIdx.x, d.o0, d.o1);
    d.nr = d.o1 - d.o0;
    d.ra = (uint32_t)p.ff / 2; d.rb = (uint32_t)p.ff / 16;
    d.pc = d.nr ? max(1, min(p.n_used, p.slot_b / (int)(d.nr * (d.ra + d.rb)))) : p.n_used;
    d.nchunks = d.nr ? (p.n_used + d.pc - 1) / d.pc : 0;
    return d;
}

// ------------------------------------------------------------------------------------------------ producers
__device__ __forceinline__ bool prod_begin(const MegaParams& p, MegaCtl* ctl, Ring& r, uint32_t bytes, int stage) {
    if (!mg_wait(p, ctl, r.empty_bar(), r.phase() ^ 1u, stage, MGE_EMPTY_WAIT)) return false;
    mbar_expect_tx(r.full_bar(), bytes);
    return true;
}
__device__ __forceinline__ bool prod_rows(const MegaParams& p, MegaCtl* ctl, Ring& r, const RowPlan& pl, const uint8_t* a, const uint8_t* b, int stage) {
    for (int c = 0; c < pl.nchunks; ++c) {
        const int c0 = pl.r0 + c * pl.rc, nr = min(pl.rc, pl.r1 - c0);
        const uint32_t ab = (uint32_t)nr * pl.ra, bb = (uint32_t)nr * pl.rb;
        if (c == 0) tl_mark_any(stage, 0, 7);
        if (!prod_begin(p, ctl, r, ab + bb, stage)) return false;
        if (c == 0) tl_mark_any(stage, 0, 8);
        bulk_g2s(r.slot_addr(), a + (size_t)c0 * pl.ra, ab, r.full_bar());
        if (bb) bulk_g2s(r.slot_addr() + ab, b + (size_t)c0 * pl.rb, bb, r.full_bar());
        r.n++;
    }
    return true;
}
// Both producers are whole warps: lane 0 issues the copies; all lanes fetch the NEXT stage's descriptor into registers while
// it does, and store it to the warp's shared-memory double buffer afterwards, so a descriptor costs no round trip.
struct StageFeed {
    MStage* buf; const MStage* table; int n_stages; uint32_t regs[(sizeof(MStage) / 4 + 31) / 32];
    __device__ __forceinline__ void load(int s) {
        const int lane = threadIdx.x & 31, words = (int)(sizeof(MStage) / 4);
        if (s < n_stages)
#pragma unroll
            for (int j = 0; j < (int)(sizeof(regs) / 4); ++j) if (lane + 32 * j < words) regs[j] = __ldg((const uint32_t*)(table + s) + lane + 32 * j);
    }
    __device__ __forceinline__ void store(int s) {
        const int lane = threadIdx.x & 31, words = (int)(sizeof(MStage) / 4);
        if (s < n_stages)
#pragma unroll
            for (int j = 0; j < (int)(sizeof(regs) / 4); ++j) if (lane + 32 * j < words) ((uint32_t*)(buf + (s & 1)))[lane + 32 * j] = regs[j];
        __syncwarp();
    }
};
// on a failure: the copies already issued must land before the block's shared memory goes away
__device__ __forceinline__ void prod_drain(const MegaParams& p, Ring& r) {
    const uint32_t issued = r.n;
    for (uint32_t k = issued > (uint32_t)r.ns ? issued - r.ns : 0; k < issued; ++k) {
        r.n = k;
        const unsigned long long t0 = gtimer();
        while (!mbar_try(r.full_bar(), r.phase())) if (gtimer() - t0 > p.wait_ns / 4) { atomicCAS(p.err, 0, MGE_DRAIN_WAIT); break; }
    }
}
// Ring A: everything whose address is known before the step starts.
__device__ __noinline__ void mg_producer_static(const MegaParams& p, MegaCtl* ctl, Ring r, MStage* buf) {
    const int lane = threadIdx.x & 31;
    StageFeed feed{buf, p.stages, p.n_stages, {}};
    feed.load(0); feed.store(0);
    for (int s = 0; s < p.n_stages; ++s) {
        feed.load(s + 1);
        if (lane == 0) {
            const MStage* st = buf + (s & 1);
            const int type = st->type;
            bool ok = true;
            if (type == MS_ROWS) {
                const int nq = st->nq, nf = st->nf;
                for (int m = 0; m < nq && ok; ++m) { const DevQ8 w = st->q[m]; ok = prod_rows(p, ctl, r, q8_plan(w, r.slot_bytes), (const uint8_t*)w.q, (const uint8_t*)w.s, s); }
                for (int m = 0; m < nf && ok; ++m) { const DevF32 w = st->f[m]; ok = prod_rows(p, ctl, r, f32_plan(w, r.slot_bytes), (const uint8_t*)w.w, nullptr, s); }
            } else if (type == MS_GDN) {
                ok = prod_rows(p, ctl, r, row_plan(p.n_v * p.sk, (uint32_t)p.sk * 4, 0, r.slot_bytes), (const uint8_t*)st->state, nullptr, s);
            } else if (type == MS_OUT) {
                const DevQ8 w = st->w; ok = prod_rows(p, ctl, r, q8_plan(w, r.slot_bytes), (const uint8_t*)w.q, (const uint8_t*)w.s, s);
            } else if (type == MS_DOWN) {
                const DevQ8 w = st->shared_down; ok = prod_rows(p, ctl, r, q8_plan(w, r.slot_bytes), (const uint8_t*)w.q, (const uint8_t*)w.s, s);
            }
        }
        __syncwarp();
        if (ctl->abort_) break;
        feed.store(s + 1);
    }
    if (lane == 0 && ctl->abort_) prod_drain(p, r);
}
// Ring B: routed-expert rows, issued when the consumers have published this layer's picks.
__device__ __noinline__ void mg_producer_experts(const MegaParams& p, MegaCtl* ctl, Ring r, MStage* buf, uint32_t ids_ready, uint32_t ids_taken) {
    const int lane = threadIdx.x & 31;
    StageFeed feed{buf, p.stages, p.n_stages, {}};
    feed.load(0); feed.store(0);
    uint32_t layer = 0;
    for (int s = 0; s < p.n_stages; ++s) {
        feed.load(s + 1);
        const MStage* st = buf + (s & 1);
        const int type = st->type;
        if (lane == 0 && type == MS_GLU) {
            if (mg_wait(p, ctl, ids_ready, layer & 1u, s, MGE_IDS_WAIT)) {
                const DevFp4 g = st->gate, u = st->up;
                const int n = p.H, nsb = n / 16, upp = p.ff / 32, n_units = glu_units(p);
                bool ok = true;
                for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
                    const int pick = unit / upp, row0 = (unit % upp) * 32, el = ctl->ids[pick];      // kept within [0, n_expert) by the consumers
                    const size_t ro = (size_t)el * p.ff + row0;
                    for (int half = 0; half < 2 && ok; ++half) {
                        const DevFp4& w = half ? u : g;
                        const uint32_t ab = 32u * (uint32_t)(n / 2), bb = 32u * (uint32_t)nsb;
                        if (!(ok = prod_begin(p, ctl, r, ab + bb, s))) break;
                        bulk_g2s(r.slot_addr(), w.nib + ro * (n / 2), ab, r.full_bar());
                        bulk_g2s(r.slot_addr() + ab, w.sc + ro * nsb, bb, r.full_bar());
                        r.n++;
                    }
                }
            }
        } else if (lane == 0 && type == MS_DOWN) {
            const DevFp4 w = st->down;
            const DownPlan d = down_plan(p);
            bool ok = true;
            for (int c = 0; c < d.nchunks && ok; ++c) {
                const int k0 = c * d.pc, nk = min(d.pc, p.n_used - k0);
                const uint32_t ab = (uint32_t)d.nr * d.ra, bb = (uint32_t)d.nr * d.rb;
                if (!(ok = prod_begin(p, ctl, r, (uint32_t)nk * (ab + bb), s))) break;
                for (int k = 0; k < nk; ++k) {
                    const size_t ro = (size_t)ctl->ids[k0 + k] * p.H + d.o0;
                    const uint32_t dst = r.slot_addr() + (uint32_t)k * (ab + bb);
                    bulk_g2s(dst, w.nib + ro * d.ra, ab, r.full_bar());
                    bulk_g2s(dst + ab, w.sc + ro * d.rb, bb, r.full_bar());
                }
                r.n++;
            }
            mbar_arrive(ids_taken);     // the picks have been read for the last time: the next layer may overwrite them
        }
        if (type == MS_DOWN) layer++;
        __syncwarp();
        if (ctl->abort_) break;
        feed.store(s + 1);
    }
    if (lane == 0 && ctl->abort_) prod_drain(p, r);
}

// ------------------------------------------------------------------------------------------------ row dots from shared memory
// One row's f32 terms, the whole warp on one row. Q8_0: lane pairs share a 32-block (16 quants each, integer halves added
// by one shuffle: exact); NVFP4: a lane owns 32 elements = two 16-blocks. Terms go to t[] in block order.
__device__ __forceinline__ void q8_row_terms(const uint8_t* wa, const uint8_t* wb, int n_in, const int8_t* xq, const float* xs, float* t) {
    const int lane = threadIdx.x & 31, np = n_in >> 4;
#pragma unroll 2
    for (int i = 0, pp = lane; pp - lane < np; pp += 32, ++i) {
        int s = 0;
        const bool in = pp < np;
        if (in) {
            const uint4 w = *(const uint4*)(wa + pp * 16), x = *(const uint4*)(xq + pp * 16);
            s = __dp4a((int)w.x, (int)x.x, s); s = __dp4a((int)w.y, (int)x.y, s);
            s = __dp4a((int)w.z, (int)x.z, s); s = __dp4a((int)w.w, (int)x.w, s);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        if (in && (lane & 1) == (i & 1)) {
            const int b = pp >> 1;
            t[b] = i2f_small(s) * (f16_bits_to_f32(((const uint16_t*)wb)[b]) * xs[b]);           // src/ops/naive.rs:701
        }
    }
}
__device__ __forceinline__ void fp4_row_terms(const uint8_t* wa, const uint8_t* wb, int n_in, const int8_t* xq, const float* xs, float* t) {
    const int lane = threadIdx.x & 31, np = n_in >> 5;
#pragma unroll 2
    for (int pp = lane; pp < np; pp += 32) {
        const uint4 w = *(const uint4*)(wa + pp * 16);
        const uint4 xa = *(const uint4*)(xq + pp * 32), xb = *(const uint4*)(xq + pp * 32 + 16);
        const int s0 = fp4_dot8(w.x, xa.x, xa.y) + fp4_dot8(w.y, xa.z, xa.w);
        const int s1 = fp4_dot8(w.z, xb.x, xb.y) + fp4_dot8(w.w, xb.z, xb.w);
        float d0, d1;
        ue4m3x2_half(((const uint16_t*)wb)[pp], d0, d1);
        const float dx = xs[pp];
        t[2 * pp] = dx * d0 * i2f_small(s0);                                                      // src/ops/naive.rs:730
        t[2 * pp + 1] = dx * d1 * i2f_small(s1);
    }
}

// A warp's pending rows: terms collected row after row, folded together (one lane per row) when the buffer is full.
struct Pending {
    float* tw; int stride, cap, n; int my_row;
    __device__ __forceinline__ void init(float* tw_, int nt, int tw_floats) { tw = tw_; stride = nt + 1; cap = min(32, tw_floats / stride); n = 0; my_row = 0; }
    __device__ __forceinline__ float* next(int row) { if ((int)(threadIdx.x & 31) == n) my_row = row; return tw + (n++) * stride; }
    template <class Epi> __device__ __forceinline__ void flush(Epi epi) {
        __syncwarp();
        const int lane = threadIdx.x & 31;
        if (lane < n) epi(my_row, fold_terms(tw + lane * stride, stride - 1));
        __syncwarp();
        n = 0;
    }
};

// Consume a RowPlan's chunks of a quantised matrix from ring `r`: warp w takes rows w, w + MG_NW, ... of every chunk.
// `claim(row)` runs on the lane that will fold `row`, when the row is taken (prefetch of epilogue operands).
template <int KIND, class Claim, class Epi>
__device__ __forceinline__ void consume_rows(const MegaParams& p, MegaCtl* ctl, Ring& r, const RowPlan& pl, int n_in, const int8_t* xq, const float* xs,
                                             Pending& pd, int stage, Claim claim, Epi epi) {
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c = 0; c < pl.nchunks; ++c) {
        const int c0 = pl.r0 + c * pl.rc, nr = min(pl.rc, pl.r1 - c0);
        if (c == 0) tl_mark(stage, 0, 5);
        const bool have = mg_wait_warp(p, ctl, r.full_bar(), r.phase(), stage, MGE_FULL_WAIT);
        if (c == 0) tl_mark(stage, 0, 6);
        const uint8_t* slot = (const uint8_t*)__cvta_shared_to_generic(r.slot_addr());
        const uint8_t* pb = slot + (size_t)nr * pl.ra;
        for (int i = wid; have && i < nr; i += MG_NW) {
            if (pd.n == pd.cap) pd.flush(epi);
            if (lane == pd.n) claim(c0 + i);
            float* t = pd.next(c0 + i);
            if (KIND == MK_Q8) q8_row_terms(slot + (size_t)i * pl.ra, pb + (size_t)i * pl.rb, n_in, xq, xs, t);
            else fp4_row_terms(slot + (size_t)i * pl.ra, pb + (size_t)i * pl.rb, n_in, xq, xs, t);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(r.empty_bar());
        r.n++;
    }
}

// ------------------------------------------------------------------------------------------------ prologues
// RMSNorm + Q8_0 quantisation of the residual row, as block_rms_norm's vector path with MG_CT threads (same sums, same order).
__device__ __noinline__ void mg_norm_quant(const float* x, const float* w, int n, float eps, float* xn, double* red, int8_t* xq, float* xs) {
    const int tid = threadIdx.x, wid = tid >> 5;
    float4 xv[4], wv[4];
    const int nv = n >> 2;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = tid + j * MG_CT;
        if (i < nv) { xv[j] = ldg_f4(x + 4 * i); wv[j] = __ldg((const float4*)w + i); }
    }
    double acc = 0.0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (tid + j * MG_CT < nv)
            acc += (double)(xv[j].x * xv[j].x) + (double)(xv[j].y * xv[j].y) + (double)(xv[j].z * xv[j].z) + (double)(xv[j].w * xv[j].w);
    acc = warp_sum_d(acc);
    if ((tid & 31) == 0) red[wid] = acc;
    csync();
    double tot = 0.0;
    for (int i = 0; i < MG_NW; ++i) tot += red[i];
    const float mean = (float)(tot / (double)n);
    const float sc = 1.0f / sqrtf(mean + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = tid + j * MG_CT;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < nv) { o = make_float4(xv[j].x * sc * wv[j].x, xv[j].y * sc * wv[j].y, xv[j].z * sc * wv[j].z, xv[j].w * sc * wv[j].w); ((float4*)xn)[i] = o; }
        if (j * MG_CT < nv) {
            float amax = fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w)));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const float d = amax / 127.0f, id = d != 0.0f ? 1.0f / d : 0.0f;
            if (i < nv) {
                char4 q;
                q.x = (signed char)fminf(127.0f, fmaxf(-128.0f, roundf(o.x * id))); q.y = (signed char)fminf(127.0f, fmaxf(-128.0f, roundf(o.y * id)));
                q.z = (signed char)fminf(127.0f, fmaxf(-128.0f, roundf(o.z * id))); q.w = (signed char)fminf(127.0f, fmaxf(-128.0f, roundf(o.w * id)));
                ((char4*)xq)[i] = q;
                if ((i & 7) == 0) xs[i >> 3] = __half2float(__float2half_rn(d));
            }
        }
    }
    csync();
}

// ------------------------------------------------------------------------------------------------ stages
// Shared-memory views of one block.
struct Smem {
    int8_t* xq; float* xs; float* xn;        // activation region: quantised row, its scales, the f32 normed row
    float* terms;                            // MG_NW * tw_floats
    double* red;                             // 32 doubles
};

// MS_ROWS: norm + quantise, then the block's rows of up to three Q8_0 and two F32 matrices against that row
// (src/model/qwen35.rs:1010, :1167-1179, :1262-1273, :1626). conv_w: rows of q[0] go through the depthwise causal conv
// (src/ops/naive.rs:275-315), pre-activation sum stored. MSF_ARGMAX: the block's best (value, row) of q[0] is kept.
__device__ __forceinline__ void mg_stage_rows(const MegaParams& p, MegaCtl* ctl, const MStage& st, const Smem& sm, Ring& ra, int s) {
    const int n = p.H, wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    mg_norm_quant(p.x, st.norm_w, n, p.eps, sm.xn, sm.red, sm.xq, sm.xs);
    tl_mark(s, 16 + MS_ROWS, 3);
    Pending pd;
    pd.init(sm.terms + wid * p.tw_floats, n / 32, p.tw_floats);
    float best_v = -INFINITY; int best_i = 0x7fffffff;
    for (int m = 0; m < st.nq; ++m) {
        const DevQ8 w = st.q[m];
        const RowPlan pl = q8_plan(w, ra.slot_bytes);
        float* o = st.qout[m];
        if (m == 0 && st.conv_w) {
            const int keep = p.conv_kernel - 1;
            float* cs = st.conv_state; const float* cw = st.conv_w;
            float past[7], taps[8];                 // the claiming lane's window and taps (conv width <= 8), fetched when the row is taken
            auto claim = [&](int row) {
#pragma unroll
                for (int k = 0; k < 7; ++k) if (k < keep) past[k] = cs[(size_t)row * keep + k];
#pragma unroll
                for (int k = 0; k < 8; ++k) if (k <= keep) taps[k] = __ldg(cw + (size_t)row * (keep + 1) + k);
            };
            auto epi = [&](int row, float v) {
                float sum = 0.0f, last = 0.0f;
#pragma unroll
                for (int k = 0; k < 7; ++k) if (k < keep) sum += past[k] * taps[k];
#pragma unroll
                for (int k = 0; k < 8; ++k) if (k == keep) last = taps[k];
                sum += v * last;
                o[row] = sum;
                float* pst = cs + (size_t)row * keep;
#pragma unroll
                for (int k = 0; k < 6; ++k) if (k + 1 < keep) pst[k] = past[k + 1];
                pst[keep - 1] = v;
            };
            consume_rows<MK_Q8>(p, ctl, ra, pl, n, sm.xq, sm.xs, pd, s, claim, epi);
            pd.flush(epi);
        } else if (st.flags & MSF_ARGMAX) {
            auto epi = [&](int row, float v) { o[row] = v; if (best_i == 0x7fffffff || v > best_v || (v == best_v && row < best_i)) { best_v = v; best_i = row; } };
            consume_rows<MK_Q8>(p, ctl, ra, pl, n, sm.xq, sm.xs, pd, s, [](int) {}, epi);
            pd.flush(epi);
        } else {
            auto epi = [&](int row, float v) { o[row] = v; };
            consume_rows<MK_Q8>(p, ctl, ra, pl, n, sm.xq, sm.xs, pd, s, [](int) {}, epi);
            pd.flush(epi);
        }
    }
    tl_mark(s, 16 + MS_ROWS, 4);
    // F32 rows: one row per warp at a time. Serial-k mode keeps the CPU's left fold (src/ops/naive.rs:845-849): one lane
    // walks the row; otherwise lane-strided partial sums and a shuffle tree.
    for (int m = 0; m < st.nf; ++m) {
        const DevF32 w = st.f[m];
        const RowPlan pl = f32_plan(w, ra.slot_bytes);
        float* o = st.fout[m];
        for (int c = 0; c < pl.nchunks; ++c) {
            const int c0 = pl.r0 + c * pl.rc, nr = min(pl.rc, pl.r1 - c0);
            const bool have = mg_wait_warp(p, ctl, ra.full_bar(), ra.phase(), s, MGE_FULL_WAIT);
            const float* slot = (const float*)__cvta_shared_to_generic(ra.slot_addr());
            for (int i = wid; have && i < nr; i += MG_NW) {
                const float* row = slot + (size_t)i * n;
                if (p.exact) {
                    if (lane == 0) {
                        float sum = 0.0f;
#pragma unroll 4
                        for (int k = 0; k < n; k += 4) {
                            const float4 a = *(const float4*)(row + k), b = *(const float4*)(sm.xn + k);
                            sum += a.x * b.x; sum += a.y * b.y; sum += a.z * b.z; sum += a.w * b.w;
                        }
                        o[c0 + i] = sum;
                    }
                } else {
                    float sacc = 0.0f;
#pragma unroll 1
                    for (int k0 = lane * 4; k0 < n; k0 += 128 * 8) {
                        float4 v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) if (k0 + 128 * j < n) v[j] = *(const float4*)(row + k0 + 128 * j);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int k = k0 + 128 * j;
                            if (k < n) sacc += v[j].x * sm.xn[k] + v[j].y * sm.xn[k + 1] + v[j].z * sm.xn[k + 2] + v[j].w * sm.xn[k + 3];
                        }
                    }
                    sacc = warp_sum(sacc);
                    if (lane == 0) o[c0 + i] = sacc;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(ra.empty_bar());
            ra.n++;
        }
    }
    if (st.flags & MSF_ARGMAX) {
        // block's best of its rows: strict '>' with the lowest index winning ties (src/profile.rs:192-213)
        for (int o = 16; o > 0; o >>= 1) argmax_merge(best_v, best_i, __shfl_xor_sync(0xffffffffu, best_v, o), __shfl_xor_sync(0xffffffffu, best_i, o));
        float* sv = (float*)sm.red; int* si = (int*)(sv + MG_NW);
        csync();
        if (lane == 0) { sv[wid] = best_v; si[wid] = best_i; }
        csync();
        if (threadIdx.x == 0) {
            for (int w2 = 1; w2 < MG_NW; ++w2) argmax_merge(best_v, best_i, sv[w2], si[w2]);
            p.arg_v[blockIdx.x] = best_v; p.arg_i[blockIdx.x] = best_i;
        }
    }
}

// MS_GDN: the gated delta rule over the block's rows of the [n_v][sv][sk] state (src/ops/naive.rs:86-135), with the SiLU of
// the conv sums and the l2-norm of q and k (src/model/qwen35.rs:1280-1310) done for the heads those rows belong to.
// One thread per state row, keys walked serially in the CPU's order; the row stays in shared memory (padded).
__device__ __forceinline__ void mg_stage_gdn(const MegaParams& p, MegaCtl* ctl, const MStage& st, const Smem& sm, Ring& ra, int s) {
    const int sk = p.sk, sv = p.sk, tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const RowPlan pl = row_plan(p.n_v * sv, (uint32_t)sk * 4, 0, ra.slot_bytes);
    const int nrows = pl.r1 - pl.r0;
    if (nrows == 0) return;
    const int h0 = pl.r0 / sv, h1 = (pl.r1 - 1) / sv, nh = h1 - h0 + 1;
    float* S = sm.terms;                                   // [nrows][sk + 1]
    float* kq = S + (size_t)nrows * (sk + 1);              // [nh][2 * sk]: k | q
    float* gb = kq + (size_t)nh * 2 * sk;                  // [nh][2]: g, beta
    // per local head: warp 2*hi normalises k, warp 2*hi + 1 normalises q (f64 tree sum, narrowing before the root)
    if (wid < 2 * nh) {
        const int hi = wid >> 1, h = h0 + hi, kh = h % p.n_k, isq = wid & 1;
        float* dst = kq + (size_t)hi * 2 * sk + isq * sk;
        const float* src = p.qkvc + (isq ? 0 : p.key_dim) + kh * sk;
        float v[4];
        double acc = 0.0;
#pragma unroll
        for (int j = 0; j < 4; ++j) if (lane + 32 * j < sk) v[j] = ldg_f(src + lane + 32 * j);
#pragma unroll
        for (int j = 0; j < 4; ++j) if (lane + 32 * j < sk) { v[j] = silu_f(v[j]); acc += (double)(v[j] * v[j]); }
        acc = warp_sum_d(acc);
        const float sc = 1.0f / fmaxf(sqrtf((float)acc), p.eps);
        const float qs = 1.0f / sqrtf((float)sk);
#pragma unroll
        for (int j = 0; j < 4; ++j) if (lane + 32 * j < sk) { const float t = v[j] * sc; dst[lane + 32 * j] = isq ? t * qs : t; }
        if (isq && lane == 0) {
            const float a = ldg_f(p.alpha + h) + __ldg(st.dt_bias + h);
            const float sp = a > 20.0f ? a : log_f(1.0f + exp_f(a));
            gb[hi * 2] = exp_f(sp * __ldg(st.ssm_a + h));
            gb[hi * 2 + 1] = sigmoid_f(ldg_f(p.beta + h));
        }
    }
    float vj = 0.0f;
    if (tid < nrows) vj = silu_f(ldg_f(p.qkvc + 2 * p.key_dim + pl.r0 + tid));
    // the state rows: chunks of the ring into the padded layout
    int done = 0;
    for (int c = 0; c < pl.nchunks; ++c) {
        const int nr = min(pl.rc, nrows - done);
        const bool have = mg_wait_warp(p, ctl, ra.full_bar(), ra.phase(), s, MGE_FULL_WAIT);
        const float* slot = (const float*)__cvta_shared_to_generic(ra.slot_addr());
        for (int idx = tid; have && idx < nr * sk; idx += MG_CT) S[(size_t)(done + idx / sk) * (sk + 1) + idx % sk] = slot[idx];
        __syncwarp();
        if (lane == 0) mbar_arrive(ra.empty_bar());
        ra.n++;
        done += nr;
    }
    csync();
    if (tid < nrows) {
        const int hi = (pl.r0 + tid) / sv - h0;
        const float* kk = kq + (size_t)hi * 2 * sk; const float* qq = kk + sk;
        const float g = gb[hi * 2], bt = gb[hi * 2 + 1];
        float* row = S + (size_t)tid * (sk + 1);
        float pred = 0.0f;                                                     // src/ops/naive.rs:109-132: decay, predict, update, read out
#pragma unroll 8
        for (int i = 0; i < sk; ++i) { const float r = row[i] * g; pred += r * kk[i]; }
        const float d = bt * (vj - pred);
        float acc = 0.0f;
#pragma unroll 8
        for (int i = 0; i < sk; ++i) { float r = row[i] * g; r = r + kk[i] * d; row[i] = r; acc += r * qq[i]; }
        p.core[pl.r0 + tid] = acc;
    }
    csync();
    float* sg = st.state + (size_t)pl.r0 * sk;
    if (!ctl->abort_)      // a state that never arrived is not written back
        for (int idx = tid; idx < nrows * sk; idx += MG_CT) sg[idx] = S[(size_t)(idx / sk) * (sk + 1) + idx % sk];
}

// MS_OUT: x += W . a with the activation's prologue fused. Recurrent flavour: gated RMSNorm of the delta rule's output per
// head, times SiLU(z), quantised (src/model/qwen35.rs:1319-1325); attention flavour: the quantised activation written
// by MS_ATTN_COMB is loaded.
__device__ __forceinline__ void mg_stage_out(const MegaParams& p, MegaCtl* ctl, const MStage& st, const Smem& sm, Ring& ra, int s) {
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const DevQ8 w = st.w;
    const int n = w.n_in, nb = n / 32;
    if (st.flags & MSF_OUT_ATTN) {
        for (int i = tid; i < n / 16; i += MG_CT) ((uint4*)sm.xq)[i] = __ldcg((const uint4*)p.aq + i);
        for (int i = tid; i < nb; i += MG_CT) sm.xs[i] = ldg_f(p.as + i);
    } else {
        const int sv = p.sk, per = sv / 32;
        for (int h = wid; h < p.n_v; h += MG_NW) {
            float o[4], zz[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) if (j < per) { o[j] = ldg_f(p.core + h * sv + 32 * j + lane); zz[j] = ldg_f(p.z + h * sv + 32 * j + lane); }
            double tot = 0.0;
#pragma unroll
            for (int j = 0; j < 4; ++j) if (j < per) tot += warp_sum_d((double)(o[j] * o[j]));
            const float mean = (float)(tot / (double)sv);
            const float sc = 1.0f / sqrtf(mean + p.eps);
#pragma unroll
            for (int j = 0; j < 4; ++j) if (j < per) {
                const float core = o[j] * sc * __ldg(st.ssm_norm + 32 * j + lane);
                const float val = silu_f(zz[j]) * core;
                float dq;
                const int8_t q = warp_quant_q8(val, &dq);
                sm.xq[h * sv + 32 * j + lane] = q;
                if (lane == 0) sm.xs[(h * sv + 32 * j) / 32] = dq;
            }
        }
    }
    csync();
    Pending pd;
    pd.init(sm.terms + wid * p.tw_floats, nb, p.tw_floats);
    float* x = p.x;
    auto epi = [&](int row, float v) { x[row] += v; };
    consume_rows<MK_Q8>(p, ctl, ra, q8_plan(w, ra.slot_bytes), n, sm.xq, sm.xs, pd, s, [](int) {}, epi);
    pd.flush(epi);
}

// MS_ATTN_PREP: per head, de-interleave q|gate, QK RMSNorm, partial NEOX RoPE at the sequence's position, KV write
// (src/model/qwen35.rs:1175-1198). One head per block at a time, a thread per dimension.
__device__ __forceinline__ void mg_stage_attn_prep(const MegaParams& p, const MStage& st, const Smem& sm) {
    const int hd = p.hd, d = threadIdx.x, jobs = p.n_head + 2 * p.n_head_kv;
    float* val = sm.terms;
    const int pos = *(volatile int*)p.pos;
    for (int job = blockIdx.x; job < jobs; job += gridDim.x) {
        const bool is_q = job < p.n_head, is_k = !is_q && job < p.n_head + p.n_head_kv;
        const int hk = is_q ? job : is_k ? job - p.n_head : job - p.n_head - p.n_head_kv;
        float v = 0.0f;
        if (d < hd) {
            if (is_q) {
                v = ldg_f(p.qg + (size_t)hk * 2 * hd + d);
                p.gate[(size_t)hk * hd + d] = ldg_f(p.qg + (size_t)hk * 2 * hd + hd + d);
            } else v = ldg_f((is_k ? p.kbuf : p.vbuf) + hk * hd + d);
        }
        if (is_q || is_k) {
            double acc = warp_sum_d(d < hd ? (double)(v * v) : 0.0);
            if ((d & 31) == 0) sm.red[d >> 5] = acc;
            csync();
            double tot = 0.0;
            for (int w = 0; w < hd / 32; ++w) tot += sm.red[w];
            const float mean = (float)(tot / (double)hd);
            const float sc = 1.0f / sqrtf(mean + p.eps);
            if (d < hd) { v = v * sc * __ldg((is_q ? st.q_norm : st.k_norm) + d); val[d] = v; }
            csync();
            const int half = p.n_rot / 2;
            if (d < half) {
                const double freq = pow((double)p.theta, -2.0 * (double)d / (double)p.n_rot);
                const double th = (double)pos * freq;
                const float sn = (float)sin(th), cs = (float)cos(th);
                const float x0 = val[d], x1 = val[d + half];
                val[d] = x0 * cs - x1 * sn;
                val[d + half] = x0 * sn + x1 * cs;
            }
            csync();
            if (d < hd) v = val[d];
        }
        if (d < hd) {
            if (is_q) p.qn[(size_t)hk * hd + d] = v;
            else {
                uint16_t* slab = (is_k ? st.kslab : st.vslab) + (size_t)pos * p.kvd + hk * hd + d;
                *slab = p.kv_bf16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v);
            }
        }
        csync();
    }
}

// MS_ATTN_PART: split-K decode attention (tolerance class, like the reference's device kernels: kernels/attention.cuh:61-195
// there). Block = (kv head, split of the positions); a warp = (query head of the group, part of the split's positions);
// a lane owns hd/32 contiguous dims. Partials m, l, acc[hd] per (head, split).
template <int HD>
__device__ __forceinline__ void mg_attn_part_body(const MegaParams& p, const MStage& st, const Smem& sm) {
    constexpr int DPL = HD / 32;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int group = p.n_head / p.n_head_kv, parts = MG_NW / group;
    const int n_pos = *(volatile int*)p.pos + 1;
    const int per = max(MG_ATTN_MIN_SPLIT, (n_pos + p.n_split - 1) / p.n_split);
    const float scale = 1.0f / sqrtf((float)HD);
    float* s_ml = sm.terms;                         // [group][parts][2]
    float* s_acc = s_ml + group * parts * 2;        // [group][parts][HD]
    for (int job = blockIdx.x; job < p.n_head_kv * p.n_split; job += gridDim.x) {
        const int hk = job % p.n_head_kv, sp = job / p.n_head_kv;
        const int p0 = sp * per, p1 = min(n_pos, p0 + per);
        if (p0 >= p1) continue;                     // the combine reads the splits that hold positions only
        const int g = wid % group, part = wid / group;
        float m = -INFINITY, l = 0.0f, acc[DPL], qr[DPL];
#pragma unroll
        for (int d = 0; d < DPL; ++d) { acc[d] = 0.0f; qr[d] = 0.0f; }
        if (part < parts) {
#pragma unroll
            for (int d = 0; d < DPL; ++d) qr[d] = ldg_f(p.qn + (size_t)(hk * group + g) * HD + lane * DPL + d);
            for (int pp = p0 + part; pp < p1; pp += parts) {
                const uint16_t* kr = st.kslab + (size_t)pp * p.kvd + hk * HD + lane * DPL;
                const uint16_t* vr = st.vslab + (size_t)pp * p.kvd + hk * HD + lane * DPL;
                uint32_t kw[DPL / 2], vw[DPL / 2];          // two 16-bit elements per word
                if (DPL == 8) { const uint4 a = *(const uint4*)kr, b = *(const uint4*)vr; kw[0] = a.x; kw[1] = a.y; kw[DPL / 2 - 2] = a.z; kw[DPL / 2 - 1] = a.w; vw[0] = b.x; vw[1] = b.y; vw[DPL / 2 - 2] = b.z; vw[DPL / 2 - 1] = b.w; }
                else if (DPL == 4) { const uint2 a = *(const uint2*)kr, b = *(const uint2*)vr; kw[0] = a.x; kw[DPL / 2 - 1] = a.y; vw[0] = b.x; vw[DPL / 2 - 1] = b.y; }
                else { kw[0] = *(const uint32_t*)kr; vw[0] = *(const uint32_t*)vr; }
                auto elem = [&](const uint32_t* w, int d) { const uint16_t h = (uint16_t)(w[d >> 1] >> ((d & 1) * 16)); return p.kv_bf16 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h); };
                float sdot = 0.0f;
#pragma unroll
                for (int d = 0; d < DPL; ++d) sdot += qr[d] * elem(kw, d);
                sdot = warp_sum(sdot) * scale;
                const float mn = fmaxf(m, sdot);
                const float corr = __expf(m - mn), pw = __expf(sdot - mn);
                l = l * corr + pw;
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[d] = acc[d] * corr + pw * elem(vw, d);
                m = mn;
            }
            if (lane == 0) { s_ml[(g * parts + part) * 2] = m; s_ml[(g * parts + part) * 2 + 1] = l; }
#pragma unroll
            for (int d = 0; d < DPL; ++d) s_acc[(size_t)(g * parts + part) * HD + lane * DPL + d] = acc[d];
        }
        csync();
        for (int idx = tid; idx < group * HD; idx += MG_CT) {
            const int gg = idx / HD, d = idx % HD;
            float M = -INFINITY;
            for (int w = 0; w < parts; ++w) M = fmaxf(M, s_ml[(gg * parts + w) * 2]);
            float L = 0.0f, A = 0.0f;
            for (int w = 0; w < parts; ++w) {
                const float mw = s_ml[(gg * parts + w) * 2];
                const float c = mw == -INFINITY ? 0.0f : __expf(mw - M);
                L += s_ml[(gg * parts + w) * 2 + 1] * c;
                A += s_acc[(size_t)(gg * parts + w) * HD + d] * c;
            }
            const size_t o = (size_t)(hk * group + gg) * p.n_split + sp;
            p.part_acc[o * HD + d] = A;
            if (d == 0) { p.part_ml[o * 2] = M; p.part_ml[o * 2 + 1] = L; }
        }
        csync();
    }
}
__device__ __forceinline__ void mg_stage_attn_part(const MegaParams& p, const MStage& st, const Smem& sm) {
    if (p.hd == 256) mg_attn_part_body<256>(p, st, sm);
    else if (p.hd == 128) mg_attn_part_body<128>(p, st, sm);
    else mg_attn_part_body<64>(p, st, sm);
}

// MS_ATTN_COMB: combine of the splits per query head, the sigmoid output gate (src/model/qwen35.rs:1216-1218) and the Q8_0
// quantisation the output projection would apply. One head per block at a time, a thread per dimension.
__device__ __forceinline__ void mg_stage_attn_comb(const MegaParams& p) {
    const int hd = p.hd, d = threadIdx.x;
    const int n_pos = *(volatile int*)p.pos + 1;
    const int per = max(MG_ATTN_MIN_SPLIT, (n_pos + p.n_split - 1) / p.n_split), n_act = (n_pos + per - 1) / per;
    for (int th = blockIdx.x; th < p.n_head; th += gridDim.x) {
        if (d >= hd) continue;
        const float gt = ldg_f(p.gate + (size_t)th * hd + d);
        float M = -INFINITY;
        for (int sp = 0; sp < n_act; ++sp) M = fmaxf(M, ldg_f(p.part_ml + ((size_t)th * p.n_split + sp) * 2));
        float L = 0.0f, A = 0.0f;
        for (int s0 = 0; s0 < n_act; s0 += 8) {
            float mv[8], lv[8], av[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool in = s0 + j < n_act;
                const size_t o = (size_t)th * p.n_split + s0 + j;
                mv[j] = in ? ldg_f(p.part_ml + o * 2) : -INFINITY;
                lv[j] = in ? ldg_f(p.part_ml + o * 2 + 1) : 0.0f;
                av[j] = in ? ldg_f(p.part_acc + o * hd + d) : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < n_act) {
                    const float c = mv[j] == -INFINITY ? 0.0f : __expf(mv[j] - M);
                    L += lv[j] * c; A += av[j] * c;
                }
        }
        float v = A / L;
        v *= sigmoid_f(gt);
        float dq;
        const int8_t q = warp_quant_q8(v, &dq);
        p.aq[(size_t)th * hd + d] = q;
        if ((d & 31) == 0) p.as[((size_t)th * hd + d) / 32] = dq;
    }
}

// MS_GLU: norm + quantise again (the row MS_ROWS of the FFN saw), routing -- softmax over all experts, top-k by counting,
// weights (src/model/qwen35.rs:1626-1638, src/ops/mod.rs:1191-1216) -- published at once to the expert ring's producer; then
// per unit h = silu(gate_e . x * s_g) * (up_e . x * s_u) (src/ops/mod.rs:1105-1117) quantised to Q8_0. Units past the
// routed ones quantise 32 elements of the shared expert's silu(gate) * up (src/model/qwen35.rs:1669-1678).
__device__ __forceinline__ void mg_stage_glu(const MegaParams& p, MegaCtl* ctl, const MStage& st, const Smem& sm, Ring& rb, int s,
                                          uint32_t ids_ready, uint32_t ids_taken, uint32_t layer) {
    __shared__ float s_wts[16];
    __shared__ float s_gu[64];
    __shared__ float s_sum;
    const int n = p.H, tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int ne = p.n_expert, nu = p.n_used, ne32 = (ne + 31) & ~31;
    // the previous layer's picks must have been read by the producer before they are overwritten
    if (layer > 0) mg_wait_warp(p, ctl, ids_taken, (layer - 1) & 1u, s, MGE_IDS_WAIT);
    float* probs = sm.terms;                       // [ne32]
    float* cand_p = probs + ne32;                  // [MOE_CAND]
    int* cand_i = (int*)(cand_p + MOE_CAND);       // [MOE_CAND]
    {
        float mx = -INFINITY;
        for (int i = lane; i < ne; i += 32) mx = fmaxf(mx, ldg_f(p.router + i));
        mx = warp_max(mx);
        for (int i = tid; i < ne32; i += MG_CT) probs[i] = i < ne ? exp_f(ldg_f(p.router + i) - mx) : 0.0f;
    }
    csync();
    if (tid == 0) {                                // softmax denominator: serial sum in index order (src/ops/naive.rs:362-376)
        float sum = 0.0f;
#pragma unroll 1
        for (int i0 = 0; i0 < ne; i0 += 32) {
            float4 q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = *(const float4*)(probs + i0 + 4 * j);
            const int lim = ne - i0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (4 * j < lim) sum += q[j].x;
                if (4 * j + 1 < lim) sum += q[j].y;
                if (4 * j + 2 < lim) sum += q[j].z;
                if (4 * j + 3 < lim) sum += q[j].w;
            }
        }
        s_sum = sum;
    }
    csync();
    {
        const float sum = s_sum;
        for (int i = tid; i < ne; i += MG_CT) probs[i] /= sum;
    }
    csync();
    {
        // top-k in two stages of counting (an expert's place = how many beat it: greater, or equal with a lower id)
        const int ng = (ne + 31) >> 5;
        for (int g = wid; g < ng; g += MG_NW) {
            const int t = g * 32 + lane;
            const float v = t < ne ? probs[t] : -1.0f;
            int rank = 0;
#pragma unroll 8
            for (int j = 0; j < 32; ++j) {
                const float q = __shfl_sync(0xffffffffu, v, j);
                rank += (int)(q > v) | ((int)(q == v) & (int)(j < lane));
            }
            if (rank < nu) { cand_p[g * nu + rank] = v; cand_i[g * nu + rank] = t < ne ? t : -1; }
        }
        csync();
        const int cnt = ng * nu;
        for (int c = tid; c < cnt; c += MG_CT) {
            const float v = cand_p[c];
            const int id = cand_i[c];
            if (id < 0) continue;
            int rank = 0;
#pragma unroll 8
            for (int j = 0; j < cnt; ++j) {
                const float q = cand_p[j];
                const int qi = cand_i[j];
                rank += (int)(qi >= 0) & ((int)(q > v) | ((int)(q == v) & (int)(qi < id)));
            }
            if (rank < nu) { ctl->ids[rank] = min(max(id, 0), ne - 1); s_wts[rank] = v; }   // in range whatever the logits were (a NaN ranks first everywhere)
        }
    }
    csync();
    if (tid == 0) {
        if (!(p.test_stall && layer == 0)) mbar_arrive(ids_ready);   // the picks are final: the producer may fetch their rows
        float sum = 0.0f;
        for (int r = 0; r < nu; ++r) sum += s_wts[r];                           // summed in pick order (src/ops/mod.rs:1211)
        const float denom = fmaxf(sum, 6.103515625e-5f);
        for (int r = 0; r < nu; ++r) {
            const float w = s_wts[r] / denom;
            if (blockIdx.x == 0) { st.ids_out[r] = ctl->ids[r]; st.w_out[r] = w; }
        }
    }
    mg_norm_quant(p.x, st.norm_w, n, p.eps, sm.xn, sm.red, sm.xq, sm.xs);       // also orders the routing scratch before the terms reuse it
    const int ff = p.ff, upp = ff / 32, n_units = glu_units(p), n_all = n_units + p.sff / 32, nsb = n / 16;
    const bool has_g = st.gate.scale2 != nullptr, has_u = st.up.scale2 != nullptr;
    Pending pd;
    pd.init(sm.terms + wid * p.tw_floats, nsb, p.tw_floats);
    for (int unit = blockIdx.x; unit < n_all; unit += gridDim.x) {
        if (unit >= n_units) {
            if (wid == 0) {
                const int k = (unit - n_units) * 32 + lane;
                const float v = silu_f(ldg_f(p.sg + k)) * ldg_f(p.su + k);
                float dq;
                const int8_t q = warp_quant_q8(v, &dq);
                p.sq[k] = q;
                if (lane == 0) p.ss[unit - n_units] = dq;
            }
            continue;
        }
        const int pick = unit / upp, row0 = (unit % upp) * 32, el = ctl->ids[pick];
        float sg2 = 1.0f, su2 = 1.0f;
        if (wid == 0) { if (has_g) sg2 = __ldg(st.gate.scale2 + el); if (has_u) su2 = __ldg(st.up.scale2 + el); }
        for (int half = 0; half < 2; ++half) {
            const bool have = mg_wait_warp(p, ctl, rb.full_bar(), rb.phase(), s, MGE_FULL_WAIT);
            const uint8_t* slot = (const uint8_t*)__cvta_shared_to_generic(rb.slot_addr());
            const uint8_t* pb = slot + (size_t)32 * (n / 2);
            auto epi = [&](int k, float v) { s_gu[k] = v; };
            for (int i = wid; have && i < 32; i += MG_NW) {
                if (pd.n == pd.cap) pd.flush(epi);
                float* t = pd.next(half * 32 + i);
                fp4_row_terms(slot + (size_t)i * (n / 2), pb + (size_t)i * nsb, n, sm.xq, sm.xs, t);
            }
            pd.flush(epi);
            __syncwarp();
            if (lane == 0) mbar_arrive(rb.empty_bar());
            rb.n++;
        }
        csync();
        if (wid == 0) {
            float g = s_gu[lane], u = s_gu[32 + lane];
            if (has_g) g = g * sg2;
            if (has_u) u = u * su2;
            const float v = silu_f(g) * u;
            float dq;
            const int8_t q = warp_quant_q8(v, &dq);
            p.hq[(size_t)pick * ff + row0 + lane] = q;
            if (lane == 0) p.hs[pick * upp + unit % upp] = dq;
        }
        csync();
    }
}

// MS_DOWN: the FFN tail for the block's output rows: down projections of the picks (expert ring) and of the shared expert
// (static ring), the weighted sum in pick order, the sigmoid-gated shared term and the residual add
// (src/model/qwen35.rs:1659-1699, src/ops/mod.rs:1134-1171, src/model/qwen35.rs:1090).
__device__ __forceinline__ void mg_stage_down(const MegaParams& p, MegaCtl* ctl, const MStage& st, const Smem& sm, Ring& ra, Ring& rb, int s) {
    __shared__ float s_wt[16], s_s2[16];
    __shared__ float s_g;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int ff = p.ff, sff = p.sff, K = p.n_used, nbf = ff / 32, nbs = sff / 32;
    const DownPlan d = down_plan(p);
    // activations: the picks' quantised h, the shared expert's quantised activation
    int8_t* hq = sm.xq;                                    // [K][ff]
    float* hs = (float*)(hq + (size_t)K * ff);             // [K][nbf]
    int8_t* sq = (int8_t*)(hs + K * nbf);                  // [sff]
    float* ss = (float*)(sq + sff);                        // [nbs]
    float* outv = ss + nbs;                                // [nr][K + 1]
    for (int i = tid; i < K * ff / 16; i += MG_CT) ((uint4*)hq)[i] = __ldcg((const uint4*)p.hq + i);
    for (int i = tid; i < K * nbf; i += MG_CT) hs[i] = ldg_f(p.hs + i);
    for (int i = tid; i < sff / 16; i += MG_CT) ((uint4*)sq)[i] = __ldcg((const uint4*)p.sq + i);
    for (int i = tid; i < nbs; i += MG_CT) ss[i] = ldg_f(p.ss + i);
    if (tid < K) {
        s_wt[tid] = ldg_f(st.w_out + tid);
        s_s2[tid] = st.down.scale2 ? __ldg(st.down.scale2 + ctl->ids[tid]) : 1.0f;
    }
    if (tid == 32) s_g = sigmoid_f(ldg_f(p.shlogit));
    csync();
    Pending pd;
    pd.init(sm.terms + wid * p.tw_floats, ff / 16, p.tw_floats);
    auto epi = [&](int item, float v) { outv[item] = v; };
    // routed picks: item (row r, pick k) -> outv[r * (K + 1) + k]
    for (int c = 0; c < d.nchunks; ++c) {
        const int k0 = c * d.pc, nk = min(d.pc, K - k0);
        const bool have = mg_wait_warp(p, ctl, rb.full_bar(), rb.phase(), s, MGE_FULL_WAIT);
        const uint8_t* slot = (const uint8_t*)__cvta_shared_to_generic(rb.slot_addr());
        const uint32_t ab = (uint32_t)d.nr * d.ra, bb = (uint32_t)d.nr * d.rb;
        for (int it = wid; have && it < nk * d.nr; it += MG_NW) {
            const int k = it / d.nr, r = it % d.nr;
            const uint8_t* base = slot + (size_t)k * (ab + bb);
            if (pd.n == pd.cap) pd.flush(epi);
            float* t = pd.next(r * (K + 1) + k0 + k);
            fp4_row_terms(base + (size_t)r * d.ra, base + ab + (size_t)r * d.rb, ff, hq + (size_t)(k0 + k) * ff, hs + (k0 + k) * nbf, t);
        }
        pd.flush(epi);
        __syncwarp();
        if (lane == 0) mbar_arrive(rb.empty_bar());
        rb.n++;
    }
    // shared expert's down projection: item (row r) -> outv[r * (K + 1) + K]
    {
        const DevQ8 w = st.shared_down;
        const RowPlan pl = q8_plan(w, ra.slot_bytes);
        pd.init(sm.terms + wid * p.tw_floats, nbs, p.tw_floats);
        const int o0 = d.o0;
        auto epi_s = [&](int row, float v) { outv[(row - o0) * (K + 1) + K] = v; };
        consume_rows<MK_Q8>(p, ctl, ra, pl, sff, sq, ss, pd, s, [](int) {}, epi_s);
        pd.flush(epi_s);
    }
    csync();
    if (tid < d.nr) {
        const float* ov = outv + tid * (K + 1);
        float acc = 0.0f;                                   // experts in pick order from zero, shared last
        for (int k = 0; k < K; ++k) {
            const float v = st.down.scale2 ? ov[k] * s_s2[k] : ov[k];
            acc += s_wt[k] * v;
        }
        acc += ov[K] * s_g;
        p.x[d.o0 + tid] += acc;
    }
}

// ------------------------------------------------------------------------------------------------ the kernel
__global__ void __launch_bounds__(MG_THREADS, 1) k_mega(const __grid_constant__ MegaParams p) {
    extern __shared__ __align__(16) unsigned char smem[];   // the runtime places dynamic shared memory on a 1 KB boundary when static use allows; offsets below keep 128-byte steps
    __shared__ MegaCtl ctl;
    __shared__ __align__(16) double s_red[32];
    __shared__ MStage s_pstage[2][2];          // the producers' descriptor double buffers
    const int tid = threadIdx.x;
    // barriers: ring A full[ns_a], empty[ns_a]; ring B full[ns_b], empty[ns_b]; ids-ready; ids-taken
    const uint32_t bars = smem_u32(ctl.bars);
    const uint32_t a_full = bars, a_empty = bars + 8u * MG_MAX_SLOTS, b_full = bars + 16u * MG_MAX_SLOTS, b_empty = bars + 24u * MG_MAX_SLOTS;
    const uint32_t ids_ready = bars + 32u * MG_MAX_SLOTS, ids_taken = ids_ready + 8u;
    if (tid < 16) ctl.ids[tid] = 0;
    if (tid == 0) {
        ctl.abort_ = 0;
        for (int i = 0; i < p.ns_a; ++i) { mbar_init(a_full + 8u * i, 1); mbar_init(a_empty + 8u * i, MG_NW); }
        for (int i = 0; i < p.ns_b; ++i) { mbar_init(b_full + 8u * i, 1); mbar_init(b_empty + 8u * i, MG_NW); }
        mbar_init(ids_ready, 1); mbar_init(ids_taken, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    Ring ra{smem_u32(smem + p.off_ring_a), a_full, a_empty, p.ns_a, p.slot_a, 0};
    Ring rb{smem_u32(smem + p.off_ring_b), b_full, b_empty, p.ns_b, p.slot_b, 0};
    if (tid >= MG_CT) {
        // producers: warp MG_NW feeds ring A, warp MG_NW + 1 feeds ring B
        if (tid < MG_CT + 32) mg_producer_static(p, &ctl, ra, s_pstage[0]);
        else mg_producer_experts(p, &ctl, rb, s_pstage[1], ids_ready, ids_taken);
        return;
    }
    Smem sm;
    sm.xq = (int8_t*)(smem + p.off_act);
    {
        const int nmax = max(p.H, max(p.vd, p.qd));
        sm.xs = (float*)(sm.xq + nmax);
        sm.xn = sm.xs + nmax / 32;
    }
    sm.terms = (float*)(smem + p.off_terms);
    sm.red = s_red;
    __shared__ MStage s_stage[2];
    // stage descriptors are staged one ahead: stage s + 1's words are requested when stage s starts and stored when it ends
    const int words = (int)(sizeof(MStage) / 4);
    if (tid < words) ((uint32_t*)&s_stage[0])[tid] = __ldg((const uint32_t*)p.stages + tid);
    csync();
    unsigned nbar = 0;
    uint32_t layer = 0;
    bool ok = true;
    for (int s = 0; s < p.n_stages && ok; ++s) {
        const MStage& st = s_stage[s & 1];
        uint32_t nxt = 0;
        if (tid < words && s + 1 < p.n_stages) nxt = __ldg((const uint32_t*)(p.stages + s + 1) + tid);
        tl_mark(s, 16 + st.type, 0);
        switch (st.type) {
            case MS_EMBED: {
                const float* row = p.tok_embd + (size_t)(*(volatile int32_t*)p.tokens) * p.H;
                int lo, hi;
                share(p.H, gridDim.x, blockIdx.x, lo, hi);
                for (int i = lo + tid; i < hi; i += MG_CT) p.x[i] = __ldg(row + i);
            } break;
            case MS_ROWS: mg_stage_rows(p, &ctl, st, sm, ra, s); break;
            case MS_GDN: mg_stage_gdn(p, &ctl, st, sm, ra, s); break;
            case MS_OUT: mg_stage_out(p, &ctl, st, sm, ra, s); break;
            case MS_ATTN_PREP: mg_stage_attn_prep(p, st, sm); break;
            case MS_ATTN_PART: mg_stage_attn_part(p, st, sm); break;
            case MS_ATTN_COMB: mg_stage_attn_comb(p); break;
            case MS_GLU: mg_stage_glu(p, &ctl, st, sm, rb, s, ids_ready, ids_taken, layer); break;
            case MS_DOWN: mg_stage_down(p, &ctl, st, sm, ra, rb, s); layer++; break;
            case MS_ADVANCE: {
                // merge of the blocks' argmax partials, the token fed back, the position advanced (as k_argmax_advance)
                if (blockIdx.x == 0 && tid < 32) {
                    float bv = -INFINITY; int bi = 0x7fffffff;
                    for (int i = tid; i < (int)gridDim.x; i += 32) argmax_merge(bv, bi, ldg_f(p.arg_v + i), __ldcg(p.arg_i + i));
                    for (int o = 16; o > 0; o >>= 1) argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
                    if (tid == 0) {
                        p.tokens[0] = bi; p.next[0] = bi; p.pos[0] += 1;
                        const int sc = p.step_counter[0];
                        if (p.history && sc < p.history_cap) p.history[sc] = bi;
                        p.step_counter[0] = sc + 1;
                    }
                }
            } break;
            default: break;
        }
        tl_mark(s, 16 + st.type, 1);
        if (tid < words && s + 1 < p.n_stages) ((uint32_t*)&s_stage[(s + 1) & 1])[tid] = nxt;
        if (s + 1 < p.n_stages) ok = mg_grid_barrier(p, &ctl, nbar++, s);
        tl_mark(s, 16 + st.type, 2);
    }
    // the last block out puts the grid barrier's counter back to zero for the next launch
    csync();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(p.done, 1u) == gridDim.x - 1) { *p.bar = 0; *p.done = 0; __threadfence(); }
    }
}

}  // namespace
