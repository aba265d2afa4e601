// The 5th-generation tensor-core path: tcgen05.mma kind::mxf4nvf4 (E2M1 values with one UE4M3 scale per 16 elements on BOTH
// operands, f32 accumulators in tensor memory), operands in shared memory behind matrix descriptors, scale factors copied
// into tensor memory by tcgen05.cp, completion through an mbarrier (tcgen05.commit), accumulators read back by tcgen05.ld.
//
// This file holds the measured ceiling of that instruction -- the denominator of every "fraction of the FP4 tensor peak" --
// by the reference's own method for its sm_120 instructions (tests/cuda_ops.rs:5899-5925 there): back-to-back MMAs on operands
// that never change, nothing but the MMA in the loop, accumulators verified afterwards.
//
// Every wait is bounded; a kernel that gives up frees its tensor memory and reports through its status word.
#include "itb_internal.cuh"

namespace {

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// Bounded wait on an mbarrier phase: polls (the try_wait itself suspends for a short, hardware-chosen time) and gives up after
// `limit_cycles` of this SM's clock (the cheap clock: reading the global timer in the polling loop costs microseconds).
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity, unsigned long long limit_cycles) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
            if (ok) return true;
        }
        if ((unsigned long long)(clock64() - t0) > limit_cycles) return false;
    }
}
// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; `lbo` = bytes between the two 16-byte
// K chunks of a row, `sbo` = bytes between 8-row groups; version 1 (this architecture) in bits 46-47.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr >> 4) & 0x3fff) | ((uint64_t)((lbo >> 4) & 0x3fff) << 16) | ((uint64_t)((sbo >> 4) & 0x3fff) << 32) | (1ull << 46);
}
// Instruction descriptor of kind::mxf4nvf4: E2M1 x E2M1 (format code 1), UE4M3 scales (0), both operands K-major, M x N.
__host__ __device__ constexpr uint32_t tc_idesc_fp4(int m, int n) { return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }

__device__ __forceinline__ void tc_mma_fp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p; }\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}

// N = 128 or 256 accumulator columns; operands: every E2M1 code 1.0 (0x2), every scale 1.0 (0x38): each accumulator ends at
// 64 * iters exactly.
template <int N>
__global__ void __launch_bounds__(128) k_fp4_ceiling(int iters, int* status, unsigned long long* cycles) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ unsigned long long s_bar;
    __shared__ uint32_t s_tmem;
    unsigned char* a = smem;                      // 128 x 64 e2m1: 4096 B
    unsigned char* b = a + 4096;                  // N x 64 e2m1
    unsigned char* sfa = b + N * 32;              // 128 rows x 4 scales: 512 B
    unsigned char* sfb = sfa + 512;               // N rows x 4 scales
    const int tid = threadIdx.x, wid = tid >> 5;
    for (int i = tid; i < (4096 + N * 32) / 4; i += 128) ((uint32_t*)a)[i] = 0x22222222u;
    for (int i = tid; i < (512 + N * 4) / 4; i += 128) ((uint32_t*)sfa)[i] = 0x38383838u;
    const uint32_t bar = tc_smem(&s_bar);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the generic-proxy fills above, before the tensor core reads them
    __syncthreads();
    if (wid == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(tc_smem(&s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tm = s_tmem, d_tm = tm, sfa_tm = tm + 256, sfb_tm = tm + 264;
    bool ok = true;
    unsigned long long c0 = 0, c1 = 0;
    if (tid == 0) {
        // scale factors into tensor memory: 32 rows x 16 bytes per copy, replicated to the four lane quarters
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(sfa_tm), "l"(tc_desc(tc_smem(sfa), 128, 128)) : "memory");
        for (int k = 0; k < N / 128; ++k)
            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(sfb_tm + 4 * k), "l"(tc_desc(tc_smem(sfb) + 512 * k, 128, 128)) : "memory");
        const uint64_t da = tc_desc(tc_smem(a), 2048, 128), db = tc_desc(tc_smem(b), N * 16, 128);
        const uint32_t idesc = tc_idesc_fp4(128, N);
        c0 = clock64();
        for (int i = 0; i < iters; ++i) tc_mma_fp4(d_tm, da, db, idesc, sfa_tm, sfb_tm, i ? 1u : 0u);
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    }
    ok = __all_sync(0xffffffffu, tc_mbar_wait(bar, 0, 2000000000ull));
    c1 = clock64();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        // verify: lane (row) 32 * warp + lane of this warp, all N columns
        const float want = 64.0f * (float)iters;
        for (int c = 0; c < N && ok; c += 8) {
            uint32_t r[8];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                         : "r"(d_tm + ((uint32_t)(wid * 32) << 16) + (uint32_t)c) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 8; ++j) if (__uint_as_float(r[j]) != want) ok = false;
        }
        if (!ok) atomicCAS(status, 0, 2);          // accumulators are not 64 * iters
    } else atomicCAS(status, 0, 1);                // the MMAs never completed
    if (tid == 0 && cycles) cycles[blockIdx.x] = c1 - c0;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (wid == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tm) : "memory");
}

}  // namespace

// Measured ceiling of tcgen05.mma kind::mxf4nvf4 (M 128, N `n` = 128 or 256, K 64 per instruction) with one block per SM:
// `iters` accumulating MMAs per block, timed with CUDA events over `reps` launches (best taken). tflops_out: dense FP4
// TFLOP/s (2 * M * N * K per MMA); status_out: 0 accumulators verified, 1 a wait ran out, 2 accumulators wrong.
extern "C" int itb_fp4_ceiling(itb_ctx* c, int n, int iters, int reps, double* tflops_out, int* status_out, double* mma_cycles_out) {
    if ((n != 128 && n != 256) || iters < 1 || iters > 200000 || reps < 1) { itb_fail_msg(c, "fp4_ceiling: n must be 128 or 256, 1 <= iters <= 200000"); return 1; }
    int* status = nullptr; unsigned long long* cyc = nullptr;
    const int blocks = c->sm_count;
    if (cudaMalloc(&status, 4) != cudaSuccess || cudaMalloc(&cyc, (size_t)blocks * 8) != cudaSuccess) { cudaFree(status); itb_fail_msg(c, "fp4_ceiling: out of device memory"); return 1; }
    cudaMemsetAsync(status, 0, 4, c->stream);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    const size_t smem = 4096 + (size_t)n * 32 + 512 + (size_t)n * 4 + 128;
    float best = 1e30f;
    for (int r = 0; r < reps + 1; ++r) {           // the first launch warms up
        cudaEventRecord(e0, c->stream);
        if (n == 256) k_fp4_ceiling<256><<<blocks, 128, smem, c->stream>>>(iters, status, cyc);
        else k_fp4_ceiling<128><<<blocks, 128, smem, c->stream>>>(iters, status, cyc);
        cudaEventRecord(e1, c->stream);
        ITB_LAUNCHED(c);
        if (cudaEventSynchronize(e1) != cudaSuccess) break;
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (r > 0 && ms < best) best = ms;
    }
    int st = -1;
    std::vector<unsigned long long> hc(blocks, 0);
    cudaError_t err = cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
    if (err == cudaSuccess) err = cudaMemcpy(hc.data(), cyc, (size_t)blocks * 8, cudaMemcpyDeviceToHost);
    cudaFree(status); cudaFree(cyc);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (err != cudaSuccess) { itb_fail(c, "fp4_ceiling", err); return 1; }
    unsigned long long worst = 0;
    for (auto v : hc) worst = std::max(worst, v);
    if (status_out) *status_out = st;
    if (tflops_out) *tflops_out = 2.0 * 128.0 * n * 64.0 * (double)iters * blocks / ((double)best * 1e-3) / 1e12;
    if (mma_cycles_out) *mma_cycles_out = (double)worst / iters;
    return 0;
}

// =====================================================================================================
// Routed experts on the FP4 tensor cores (many tokens per pass: prefill and large batches)
// =====================================================================================================
// The reference's default device path quantises the activations to FP4 too and multiplies FP4 x FP4 on its tensor cores
// (kernels/nvfp4.cuh:232, :344, :434 there; CPU statement: Fp4Row::from_f32 and dot_nvfp4_fp4, src/ops/naive.rs:755-837).
// Here: the same activation quantiser, bit for bit, writing straight into tensor-core operand tiles; the expert weights
// re-tiled once into the same form; one block-scaled tcgen05 GEMM per (expert, 128 weight rows, up to 128 tokens) with
// operands fetched by bulk asynchronous copies (whole tiles are contiguous in HBM) and accumulators in tensor memory.
// Results are tolerance class against dot_nvfp4_fp4 (the tensor core's accumulation order inside a 64-wide step is its
// own), exactly as the reference holds its own FP4 path (src/ops/cuda/mod.rs:239-248 there).
//
// Operand tile ("K64 block"): rows x 64 E2M1 values = rows x 32 bytes, stored as [2 chunks of 16 bytes][rows / 8][8 rows][16 B]
// (K-major, no swizzle: 8-row x 16-byte core matrices; descriptor: leading offset = rows * 16, stride offset = 128).
// Scale tile: 128 rows x 4 scales per K64 block = 512 B at (row % 32) * 16 + (row / 32) * 4 + scale (the layout
// tcgen05.cp 32x128b.warpx4 spreads over the four lane quarters of tensor memory).
namespace {

constexpr int TC_M = 128;          // weight rows per tile
constexpr int TC_NMAX = 128;       // tokens per tile at most
constexpr int TC_KS = 4;           // K64 blocks per pipeline stage
constexpr int TC_STAGES = 4;         // pipeline stages of the down form (33 KB each)
constexpr int TC_STAGES_GLU = 3;     // of the gate+up form (50 KB each): three stages and the 64 KB staging tile fill shared memory

// ---- E2M1 / UE4M3 helpers (src/ops/naive.rs:794-806, src/quant/mod.rs:265-336) ----
__device__ __forceinline__ float ue4m3_half(uint32_t c) { return ue4m3_half_dev(c & 0x7f); }
// Round to nearest even onto the UE4M3 grid, saturating at 0x7e (448); non-positive and NaN give 0.
__device__ __forceinline__ int f32_to_ue4m3_rn(float x) {
    if (!(x > 0.0f)) return 0;
    if (x >= 448.0f) return 0x7e;
    // codes are monotone in value: binary search on 2 * ue4m3_half(code), then the tie rule on the code's parity
    int lo = 0, hi = 0x7e;
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (2.0f * ue4m3_half((uint32_t)mid) <= x) lo = mid; else hi = mid; }
    const double v = (double)x, below = v - 2.0 * (double)ue4m3_half((uint32_t)lo), above = 2.0 * (double)ue4m3_half((uint32_t)hi) - v;
    return (below < above || (below == above && (lo & 1) == 0)) ? lo : hi;
}
// Nearest of {0, .5, 1, 1.5, 2, 3, 4, 6} to |x| * inv, the lower one on ties; sign in bit 3.
__device__ __forceinline__ uint32_t e2m1_of(float x, float inv) {
    const float ax = fabsf(x) * inv;
    const uint32_t m = (uint32_t)(ax > 0.25f) + (uint32_t)(ax > 0.75f) + (uint32_t)(ax > 1.25f) + (uint32_t)(ax > 1.75f) + (uint32_t)(ax > 2.5f) +
                       (uint32_t)(ax > 3.5f) + (uint32_t)(ax > 5.0f);
    return m | (x < 0.0f ? 8u : 0u);
}
// One 16-element block: the scale code of least squared error among the seed and its four neighbours, then the codes.
__device__ __forceinline__ void fp4_quant_block(const float* blk, uint32_t* scale_code, uint32_t* codes_lo, uint32_t* codes_hi) {
    float v[16];
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) { v[j] = blk[j]; amax = fmaxf(amax, fabsf(v[j])); }
    const int seed = f32_to_ue4m3_rn(amax / 6.0f);
    const int offs[5] = {0, -1, 1, -2, 2};
    float best_err = 3.40282347e+38f, best_scale = 0.0f;
    int best_code = 0;
#pragma unroll 1
    for (int o = 0; o < 5; ++o) {
        const int code = seed + offs[o];
        if (code < 0 || code > 0x7e) continue;
        const float sc = ue4m3_half((uint32_t)code);
        const float inv = sc > 0.0f ? 0.5f / sc : 0.0f;
        float err = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            // the code's doubled magnitude {0,1,2,3,4,6,8,12} built by the same comparisons that pick the code (no table look-up)
            const float ax = fabsf(v[j]) * inv;
            const float mag = (ax > 0.25f ? 1.0f : 0.0f) + (ax > 0.75f ? 1.0f : 0.0f) + (ax > 1.25f ? 1.0f : 0.0f) + (ax > 1.75f ? 1.0f : 0.0f) +
                              (ax > 2.5f ? 2.0f : 0.0f) + (ax > 3.5f ? 2.0f : 0.0f) + (ax > 5.0f ? 4.0f : 0.0f);
            const float d = fabsf(v[j]) - mag * sc;
            err = __fmaf_rn(d, d, err);
        }
        if (err < best_err) { best_err = err; best_code = code; best_scale = sc; }
    }
    const float inv = best_scale > 0.0f ? 0.5f / best_scale : 0.0f;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { lo |= e2m1_of(v[j], inv) << (4 * j); hi |= e2m1_of(v[8 + j], inv) << (4 * j); }
    *scale_code = (uint32_t)best_code; *codes_lo = lo; *codes_hi = hi;
}

// Plain form (tests): codes one per byte, scales one per 16 elements, like the oracle's record.
__global__ void k_fp4_quant_plain(const float* x, size_t n_blocks, uint8_t* scales, uint8_t* codes) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint32_t sc, lo, hi;
    fp4_quant_block(x + b * 16, &sc, &lo, &hi);
    scales[b] = (uint8_t)sc;
    for (int j = 0; j < 8; ++j) { codes[b * 16 + j] = (lo >> (4 * j)) & 15; codes[b * 16 + 8 + j] = (hi >> (4 * j)) & 15; }
}

// ---- tiles of one pass ----
// A tile = up to TC_NMAX pairs of one expert (slots [n0, n0 + cnt) of the expert-sorted pair list), padded to a multiple of 16.
struct TcTile { int expert, n0, cnt, npad; unsigned b_off, sf_off; };   // offsets in padded rows / in 512-byte scale tiles
// pair_off[e .. e+1): the expert's slots. One block; a thread per expert counts its tiles, a block-wide scan places them
// (tiles in expert order, so the blocks that share an expert's weights run next to each other).
__global__ void __launch_bounds__(1024) k_tc_build_tiles(const int* pair_off, int n_expert, int expert_lo, int expert_cnt, TcTile* tiles, int* n_tiles_out, int max_tiles, int k_blocks) {
    __shared__ int s_tiles[1024], s_rows[1024];
    const int e = threadIdx.x;
    int a = 0, z = 0;
    if (e < n_expert && e >= expert_lo && e < expert_lo + expert_cnt) { a = pair_off[e]; z = pair_off[e + 1]; }
    const int cnt = z - a, nt = (cnt + TC_NMAX - 1) / TC_NMAX;
    // padded rows of this expert's tiles: full tiles are 128, the last one is rounded up to 16
    const int rows = nt ? (nt - 1) * TC_NMAX + ((cnt - (nt - 1) * TC_NMAX + 15) & ~15) : 0;
    s_tiles[e] = nt; s_rows[e] = rows;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {                  // inclusive scans of both counts
        const int t1 = e >= d ? s_tiles[e - d] : 0, r1 = e >= d ? s_rows[e - d] : 0;
        __syncthreads();
        s_tiles[e] += t1; s_rows[e] += r1;
        __syncthreads();
    }
    int ti = s_tiles[e] - nt; unsigned boff = (unsigned)(s_rows[e] - rows);
    for (int n0 = a; n0 < z; n0 += TC_NMAX, ++ti) {
        const int c = min(TC_NMAX, z - n0), npad = (c + 15) & ~15;
        if (ti < max_tiles) tiles[ti] = TcTile{e, n0, c, npad, boff, (unsigned)ti * (unsigned)k_blocks};
        boff += (unsigned)npad;
    }
    if (e == 1023) *n_tiles_out = min(s_tiles[1023], max_tiles);
}

// Activation rows -> FP4 records, each row once: codes [row][n_in / 2] (element order, low nibble first), scale codes
// [row][n_in / 16]. One thread per 16-element block.
__global__ void k_tc_quant_rows(const float* x, size_t n_blocks, uint8_t* codes, uint8_t* scales) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint32_t sc, lo, hi;
    fp4_quant_block(x + b * 16, &sc, &lo, &hi);
    *(uint2*)(codes + b * 8) = make_uint2(lo, hi);
    scales[b] = (uint8_t)sc;
}
// FP4 records -> the operand tiles of one pass. grid (tiles, row eighths); a thread moves 16 bytes (32 elements) of one slot's row
// and, for every other chunk, the 4 scale codes of its K64 block. Source row of a slot: pair_list[slot] / rows_div (rows_div =
// n_used when the rows are tokens shared by a token's picks, 1 when there is a row per pair). Padding rows are written as zeros.
__global__ void k_tc_gather_tiles(const uint8_t* codes, const uint8_t* scales, int n_in, const int* pair_list, int rows_div, const TcTile* tiles,
                                  const int* n_tiles, uint8_t* b_img, uint8_t* sf_img) {
    if ((int)blockIdx.x >= *n_tiles) return;
    const TcTile t = tiles[blockIdx.x];
    const int cpr = n_in / 32;                              // 16-byte chunks per row
    uint8_t* img = b_img + (size_t)t.b_off * (n_in / 2);
    uint8_t* sf = sf_img + (size_t)t.sf_off * 512;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < t.npad * cpr; i += gridDim.y * blockDim.x) {
        const int n = i / cpr, ch = i % cpr, kb = ch >> 1, half = ch & 1;
        uint4 v = make_uint4(0, 0, 0, 0);
        uint32_t s4 = 0;
        if (n < t.cnt) {
            const size_t row = (size_t)(pair_list[t.n0 + n] / rows_div);
            v = *(const uint4*)(codes + row * (n_in / 2) + (size_t)ch * 16);
            if (!half) s4 = *(const uint32_t*)(scales + row * (n_in / 16) + kb * 4);
        }
        *(uint4*)(img + (size_t)kb * (t.npad * 32) + half * (t.npad * 16) + (n >> 3) * 128 + (n & 7) * 16) = v;
        if (!half) *(uint32_t*)(sf + (size_t)kb * 512 + (n & 31) * 16 + (n >> 5) * 4) = s4;
    }
    // the rest of every 512-byte scale tile (rows npad .. 127): zeros, so a tile never holds codes of an earlier pass
    const int kbs = n_in / 64, rest = 128 - t.npad;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < rest * kbs; i += gridDim.y * blockDim.x) {
        const int n = t.npad + i / kbs, kb = i % kbs;
        *(uint32_t*)(sf + (size_t)kb * 512 + (n & 31) * 16 + (n >> 5) * 4) = 0u;
    }
}

// Expert weights -> operand tiles, once per stack. One thread per (expert, row, K64 block).
// out: [expert][row tile][K64 block][4096 B]; scales: [expert][row tile][K64 block][512 B].
__global__ void k_tc_tile_weights(const uint8_t* nib, const uint8_t* sc, int n_expert, int n_out, int n_in, uint8_t* w_img, uint8_t* sf_img) {
    const int kbs = n_in / 64;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_expert * n_out * kbs) return;
    const int kb = (int)(idx % kbs); const size_t er = idx / kbs;
    const int row = (int)(er % n_out); const int e = (int)(er / n_out);
    const int mt = row / TC_M, r = row % TC_M;
    const uint4* src = (const uint4*)(nib + ((size_t)e * n_out + row) * (n_in / 2) + kb * 32);
    uint8_t* blk = w_img + (((size_t)e * (n_out / TC_M) + mt) * kbs + kb) * 4096;
    *(uint4*)(blk + (r >> 3) * 128 + (r & 7) * 16) = src[0];
    *(uint4*)(blk + 2048 + (r >> 3) * 128 + (r & 7) * 16) = src[1];
    const uint32_t s4 = *(const uint32_t*)(sc + ((size_t)e * n_out + row) * (n_in / 16) + kb * 4);
    *(uint32_t*)(sf_img + (((size_t)e * (n_out / TC_M) + mt) * kbs + kb) * 512 + (r & 31) * 16 + (r >> 5) * 4) = s4;
}

// ---- the GEMM ----
struct TcGemm {
    const uint8_t *wg_img, *wg_sf, *wu_img, *wu_sf;      // weights of the (gate, up) pair, or of the one matrix (wu_* null)
    const float *s2g, *s2u;                              // per-expert second scales (or null)
    int expert_lo;
    const uint8_t *b_img, *b_sf;                         // this pass's activation tiles
    const TcTile* tiles; const int* n_tiles; const int* pair_list;
    int n_out, n_in;                                     // rows of one matrix, K
    float* out; int out_stride;                          // out[pair][n_out]
    int* status;
    long long* prof;                                     // optional: 8 clock64 stamps per block (ITB_TC_PROF=1)
};
__device__ __forceinline__ void tc_bulk(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Persistent: grid = one block per SM; block b takes work items b, b + grid, ... of the (tile, row tile) list, row tile fastest, so
// the blocks running at one time share activation tiles and an expert's weights in L2. Block 320: warps 0-7 epilogue (tensor-
// memory lane quarter = warp % 4, column half = warp / 4), warp 8 producer, warp 9 MMA. The three roles run as a pipeline over
// the block's items: the producer's stage ring runs on into the next item; the epilogue warps read an item's accumulators into
// registers, hand tensor memory back (s_free), and do their arithmetic and stores while the next item's MMAs run.
// EXACT_SILU is a template parameter, not a flag read in the loop: the library-exact exponential is some hundred instructions, and
// both forms inside the 64-times unrolled epilogue overflow the instruction cache (measured: 14,900 cycles per tile against 5,300 for
// the same stores without the activation).
template <bool GLU, bool EXACT_SILU>
__global__ void __launch_bounds__(320, 1) k_tc_gemm(TcGemm p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int NST = GLU ? TC_STAGES_GLU : TC_STAGES;
    __shared__ unsigned long long s_full[NST], s_empty[NST], s_acc, s_free;
    __shared__ uint32_t s_tmem;
    __shared__ int s_pair[TC_NMAX];
    __shared__ int s_bad;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int n_mt = p.n_out / TC_M, n_work = *p.n_tiles * n_mt;
    if ((int)blockIdx.x >= n_work) return;
    const int kbs = p.n_in / 64, n_stage = kbs / TC_KS;
    const uint32_t a_bytes = TC_KS * 4096, sf_bytes = TC_KS * 512;
    // stage layout: A_g | A_u | B | SFA_g | SFA_u | SFB
    const uint32_t o_au = a_bytes, o_b = a_bytes * (GLU ? 2 : 1), o_sfg = o_b + TC_NMAX * 32 * TC_KS, o_sfu = o_sfg + sf_bytes, o_sfb = o_sfu + (GLU ? sf_bytes : 0);
    const uint32_t stage_bytes = o_sfb + sf_bytes;
    const uint32_t sbase = tc_smem(smem);
    float* stg = (float*)(smem + (size_t)NST * stage_bytes);      // the epilogue's staging tile: [token column][128 weight rows]
    if (tid == 0) {
        s_bad = 0;
        for (int s = 0; s < NST; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&s_full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&s_empty[s])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&s_acc)) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;" ::"r"(tc_smem(&s_free)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (wid == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(tc_smem(&s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tm = s_tmem;
    // optional stamps of this block: [0] start, [1] MMA thread's cycles waiting for operands, [2] waiting for tensor memory to be
    // handed back, [3] epilogue warp 0 waiting for accumulators, [4] its arithmetic and stores, [5] end, [6] items, [7] columns
    long long* pf = p.prof ? p.prof + (size_t)blockIdx.x * 8 : nullptr;
    if (pf && tid == 0) pf[0] = clock64();
    // tensor memory: D_g at 0, D_u at 128, scale factors from 256: per stage slot 48 columns (SFA_g 16, SFA_u 16, SFB 16)
    const uint32_t d_g = tm, d_u = tm + 128, sf0 = tm + 256;
    const unsigned long long limit = 2000000000ull;
    bool ok = true;
    if (wid == 8 && lane == 0) {
        int it = 0;                                           // stages issued so far, over all items
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
            const TcTile t = p.tiles[w / n_mt];
            const int mt = w % n_mt;
            const size_t w_tile = ((size_t)(t.expert - p.expert_lo) * n_mt + mt) * kbs;
            const uint32_t b_bytes = (uint32_t)t.npad * 32 * TC_KS;
            const uint32_t total = a_bytes * (GLU ? 2 : 1) + b_bytes + sf_bytes * (GLU ? 3 : 2);
            for (int st = 0; st < n_stage; ++st, ++it) {
                const int s = it % NST;
                if (it >= NST) ok = tc_mbar_wait(tc_smem(&s_empty[s]), ((it / NST) - 1) & 1, limit);
                if (!ok) break;
                const uint32_t full = tc_smem(&s_full[s]), dst = sbase + s * stage_bytes;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"(total) : "memory");
                const size_t kb0 = (size_t)st * TC_KS;
                tc_bulk(dst, p.wg_img + (w_tile + kb0) * 4096, a_bytes, full);
                tc_bulk(dst + o_sfg, p.wg_sf + (w_tile + kb0) * 512, sf_bytes, full);
                if (GLU) {
                    tc_bulk(dst + o_au, p.wu_img + (w_tile + kb0) * 4096, a_bytes, full);
                    tc_bulk(dst + o_sfu, p.wu_sf + (w_tile + kb0) * 512, sf_bytes, full);
                }
                tc_bulk(dst + o_b, p.b_img + (size_t)t.b_off * (p.n_in / 2) + kb0 * (t.npad * 32), b_bytes, full);
                tc_bulk(dst + o_sfb, p.b_sf + ((size_t)t.sf_off + kb0) * 512, sf_bytes, full);
            }
        }
        if (!ok) atomicCAS(p.status, 0, 3);
    } else if (wid == 9 && lane == 0) {
        // descriptors of stage slot 0; a slot or K block further on only moves the 14-bit start-address field (address >> 4), which
        // cannot carry out of it (shared memory ends below 256 KB), so the low words are advanced by plain adds
        const uint64_t dA = tc_desc(sbase, 2048, 128), dAu = tc_desc(sbase + o_au, 2048, 128);
        const uint64_t dSg = tc_desc(sbase + o_sfg, 128, 128), dSu = tc_desc(sbase + o_sfu, 128, 128), dSb = tc_desc(sbase + o_sfb, 128, 128);
        int it = 0, item = 0;
        long long t_load = 0, t_free = 0;
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++item) {
            const TcTile t = p.tiles[w / n_mt];
            const uint32_t idesc = tc_idesc_fp4(TC_M, t.npad);
            const uint64_t dB = tc_desc(sbase + o_b, (uint32_t)t.npad * 16, 128);
            const uint32_t b_step = (uint32_t)(t.npad * 32) >> 4;
            if (item) {                                       // the epilogue warps have read the previous item's accumulators
                const long long c0 = pf ? clock64() : 0;
                ok = tc_mbar_wait(tc_smem(&s_free), (item - 1) & 1, limit);
                if (pf) t_free += clock64() - c0;
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            for (int st = 0; st < n_stage; ++st, ++it) {
                const int s = it % NST;
                const long long c0 = pf ? clock64() : 0;
                ok = tc_mbar_wait(tc_smem(&s_full[s]), (it / NST) & 1, limit);
                if (pf) t_load += clock64() - c0;
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t so = (uint32_t)s * (stage_bytes >> 4), sft = sf0 + s * 48;
#pragma unroll
                for (int k = 0; k < TC_KS; ++k) {
                    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(sft + 4 * k), "l"(dSg + so + 32u * k) : "memory");
                    if (GLU) asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(sft + 16 + 4 * k), "l"(dSu + so + 32u * k) : "memory");
                    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(sft + 32 + 4 * k), "l"(dSb + so + 32u * k) : "memory");
                }
#pragma unroll
                for (int k = 0; k < TC_KS; ++k) {
                    const uint64_t db = dB + so + b_step * k;
                    const uint32_t acc = (st | k) ? 1u : 0u;
                    tc_mma_fp4(d_g, dA + so + 256u * k, db, idesc, sft + 4 * k, sft + 32 + 4 * k, acc);
                    if (GLU) tc_mma_fp4(d_u, dAu + so + 256u * k, db, idesc, sft + 16 + 4 * k, sft + 32 + 4 * k, acc);
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&s_empty[s])) : "memory");
            }
            if (!ok) break;
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&s_acc)) : "memory");
        }
        if (!ok) atomicCAS(p.status, 0, 4);
        if (pf) { pf[1] = t_load; pf[2] = t_free; }
    } else if (wid < 8) {
        // epilogue: lane quarter `wid % 4` of tensor memory = weight rows 32 * (wid % 4) .. of the tile; the tile's token columns are
        // split between the two warps of a quarter. All of a warp's accumulator reads are issued before the one wait; the values
        // (after SiLU * up for the gated form) go to the staging tile, column-major, and from there each warp writes whole
        // 512-byte pieces of output rows (one 16-byte store per lane) instead of 128-byte pieces per quarter.
        // The eight warps meet at two named barriers per item; none leaves the loop except after the first of them and on a
        // decision all of them read there, so no warp is ever left waiting at a barrier.
        const int quarter = wid & 3, half = wid >> 2;
        int item = 0;
        long long t_wait = 0, t_work = 0, cols = 0;
        for (int w = blockIdx.x; w < n_work; w += gridDim.x, ++item) {
            const TcTile t = p.tiles[w / n_mt];
            const int mt = w % n_mt, el = t.expert - p.expert_lo;
            const int split = ((t.npad / 16 + 1) / 2) * 16;          // npad is a multiple of 16
            const int c0 = half ? split : 0, nchunk = ((half ? t.npad : split) - c0) / 16;      // up to 4 chunks of 16 columns
            // where each column goes (read before the wait, so the latency hides behind the MMAs)
            if (tid < TC_NMAX) s_pair[tid] = tid < t.cnt ? p.pair_list[t.n0 + tid] : -1;
            const float sg = p.s2g ? p.s2g[el] : 1.0f, su = (GLU && p.s2u) ? p.s2u[el] : 1.0f;
            const long long k0 = pf ? clock64() : 0;
            ok = __all_sync(0xffffffffu, tc_mbar_wait(tc_smem(&s_acc), item & 1, limit));      // one answer per warp: the loads below are warp-wide
            if (!ok && lane == 0) atomicCAS(p.status, 0, 5);                                    // the accumulators never came
            ok = ok && __shfl_sync(0xffffffffu, *(volatile int*)p.status, 0) == 0;
            const long long k1 = pf ? clock64() : 0;
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t g[64], u[64];
                const uint32_t ta = ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    if (ch < nchunk) {
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                     : "=r"(g[16 * ch]), "=r"(g[16 * ch + 1]), "=r"(g[16 * ch + 2]), "=r"(g[16 * ch + 3]), "=r"(g[16 * ch + 4]), "=r"(g[16 * ch + 5]),
                                       "=r"(g[16 * ch + 6]), "=r"(g[16 * ch + 7]), "=r"(g[16 * ch + 8]), "=r"(g[16 * ch + 9]), "=r"(g[16 * ch + 10]), "=r"(g[16 * ch + 11]),
                                       "=r"(g[16 * ch + 12]), "=r"(g[16 * ch + 13]), "=r"(g[16 * ch + 14]), "=r"(g[16 * ch + 15]) : "r"(d_g + ta + 16u * ch) : "memory");
                        if (GLU)
                            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                         : "=r"(u[16 * ch]), "=r"(u[16 * ch + 1]), "=r"(u[16 * ch + 2]), "=r"(u[16 * ch + 3]), "=r"(u[16 * ch + 4]), "=r"(u[16 * ch + 5]),
                                           "=r"(u[16 * ch + 6]), "=r"(u[16 * ch + 7]), "=r"(u[16 * ch + 8]), "=r"(u[16 * ch + 9]), "=r"(u[16 * ch + 10]), "=r"(u[16 * ch + 11]),
                                           "=r"(u[16 * ch + 12]), "=r"(u[16 * ch + 13]), "=r"(u[16 * ch + 14]), "=r"(u[16 * ch + 15]) : "r"(d_u + ta + 16u * ch) : "memory");
                    }
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                // the accumulators are in registers: tensor memory goes back to the MMA warp for the next item
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(&s_free)) : "memory");
                float* srow = stg + (size_t)c0 * TC_M + quarter * 32 + lane;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    if (ch < nchunk) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            float v = __uint_as_float(g[16 * ch + j]);
                            if (p.s2g) v = v * sg;
                            if (GLU) {
                                // SiLU(gate) * up (src/ops/mod.rs:1105-1117). exact=0: the fast exponential (this path is tolerance class
                                // through the tensor core's summation order anyway); exact=1: the library-exact one, on the f64 unit
                                float x = __uint_as_float(u[16 * ch + j]); if (p.s2u) x = x * su;
                                v = (EXACT_SILU ? silu_f(v) : __fdividef(v, 1.0f + __expf(-v))) * x;
                            }
                            srow[(16 * ch + j) * TC_M] = v;
                        }
                    }
                }
            } else s_bad = 1;
            asm volatile("bar.sync 1, 256;" ::: "memory");        // the tile is staged (or some warp gave up: every warp reads that here)
            if (s_bad) break;
            const size_t obase = (size_t)mt * TC_M + lane * 4;
            for (int col = wid; col < t.npad; col += 8) {
                const int pair = s_pair[col];
                if (pair >= 0) *(float4*)(p.out + (size_t)pair * p.out_stride + obase) = *(const float4*)(stg + (size_t)col * TC_M + lane * 4);
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");        // the staging tile and the pair list are free for the next item
            if (pf) { t_wait += k1 - k0; t_work += clock64() - k1; cols += t.npad; }
        }
        if (pf && tid == 0) { pf[3] = t_wait; pf[4] = t_work; pf[6] = item; pf[7] = cols; }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (wid == 9) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tm) : "memory");
    if (pf && tid == 0) pf[5] = clock64();
}
inline size_t tc_gemm_smem(bool glu) {
    const size_t a = TC_KS * 4096, b = (size_t)TC_NMAX * 32 * TC_KS, sf = TC_KS * 512;
    return (glu ? TC_STAGES_GLU : TC_STAGES) * (a * (glu ? 2 : 1) + b + sf * (glu ? 3 : 2)) + (size_t)TC_NMAX * TC_M * 4 + 128;
}

}  // namespace

bool itb_tc_shape_ok(const DevFp4& w) { return w.n_in % (64 * TC_KS) == 0 && w.n_out % TC_M == 0 && !w.slot_map && w.expert_lo + w.n_expert <= 1024; }
void itb_tc_free(itb_ctx* c) {
    for (auto& kv : c->tc_weights) { cudaFree(kv.second.img); cudaFree(kv.second.sf); }
    c->tc_weights.clear();
    cudaFree(c->tc_tiles); cudaFree(c->tc_n_tiles); cudaFree(c->tc_slot_tile); cudaFree(c->tc_b_img); cudaFree(c->tc_b_sf); cudaFree(c->tc_status); cudaFree(c->tc_codes); cudaFree(c->tc_scales); cudaFree(c->tc_q8_b); cudaFree(c->tc_q8_sx); cudaFree(c->tc_hf_b);
    c->tc_hf_b = nullptr; c->tc_cap_hfb = 0; c->tc_hf_src = nullptr;
    c->tc_q8_b = nullptr; c->tc_q8_sx = nullptr; c->tc_cap_q8b = c->tc_cap_q8sx = 0; c->tc_q8_src = nullptr;
    c->tc_tiles = nullptr; c->tc_n_tiles = nullptr; c->tc_slot_tile = nullptr; c->tc_b_img = nullptr; c->tc_b_sf = nullptr; c->tc_status = nullptr; c->tc_codes = nullptr; c->tc_scales = nullptr; c->tc_cap_codes = c->tc_cap_scales = 0;
    c->tc_cap_tiles = c->tc_cap_slots = c->tc_cap_b = c->tc_cap_sf = 0;
}
static const itb_ctx::TcWeights* tc_weights_of(itb_ctx* c, cudaStream_t st, const DevFp4& w) {
    auto it = c->tc_weights.find(w.nib);
    if (it != c->tc_weights.end()) return &it->second;
    itb_ctx::TcWeights t;
    const size_t kbs = w.n_in / 64, tiles = (size_t)w.n_expert * (w.n_out / TC_M) * kbs;
    if (cudaMalloc(&t.img, tiles * 4096) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (cudaMalloc(&t.sf, tiles * 512) != cudaSuccess) { cudaFree(t.img); cudaGetLastError(); return nullptr; }
    t.bytes = tiles * (4096 + 512);
    const size_t n = (size_t)w.n_expert * w.n_out * kbs;
    k_tc_tile_weights<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(w.nib, w.sc, w.n_expert, w.n_out, w.n_in, t.img, t.sf);
    c->launches++;
    return &c->tc_weights.emplace(w.nib, t).first->second;
}
template <class T>
static bool tc_grow(T** p, size_t* cap, size_t need, cudaStream_t st) {
    if (*cap >= need) return true;
    cudaStreamSynchronize(st);
    cudaFree(*p); *p = nullptr; *cap = 0;
    if (cudaMalloc((void**)p, need * sizeof(T)) != cudaSuccess) { cudaGetLastError(); return false; }
    *cap = need;
    return true;
}
bool itb_tc_experts(itb_ctx* c, cudaStream_t st, const DevFp4& wg, const DevFp4* wu, const float* x, int rows_div, const int* pair_off,
                    const int* pair_list, int n_pairs, float* out) {
    if (!itb_tc_shape_ok(wg) || (wu && (!itb_tc_shape_ok(*wu) || wu->n_in != wg.n_in || wu->n_out != wg.n_out)) || n_pairs <= 0) return false;
    const itb_ctx::TcWeights* tg = tc_weights_of(c, st, wg);
    const itb_ctx::TcWeights* tu = wu ? tc_weights_of(c, st, *wu) : nullptr;
    if (!tg || (wu && !tu)) return itb_fail_msg(c, "FP4 tensor path: out of device memory for the tiled expert weights");
    const size_t kbs = wg.n_in / 64, max_tiles = (size_t)wg.n_expert + (size_t)n_pairs / TC_NMAX + 1;
    const size_t b_rows = (size_t)n_pairs + 16 * max_tiles;
    TcTile* tiles = (TcTile*)c->tc_tiles;
    size_t cap_t = c->tc_cap_tiles;
    bool ok = tc_grow(&tiles, &cap_t, max_tiles, st);
    c->tc_tiles = tiles; c->tc_cap_tiles = cap_t;
    size_t cap1 = c->tc_n_tiles ? 1 : 0, cap2 = c->tc_status ? 1 : 0;
    ok = ok && tc_grow(&c->tc_n_tiles, &cap1, 1, st) && tc_grow(&c->tc_status, &cap2, 1, st) &&
         tc_grow(&c->tc_b_img, &c->tc_cap_b, b_rows * (wg.n_in / 2), st) && tc_grow(&c->tc_b_sf, &c->tc_cap_sf, max_tiles * kbs * 512, st) &&
         tc_grow(&c->tc_codes, &c->tc_cap_codes, (size_t)n_pairs * (wg.n_in / 2), st) && tc_grow(&c->tc_scales, &c->tc_cap_scales, (size_t)n_pairs * (wg.n_in / 16), st);
    if (!ok) return itb_fail_msg(c, "FP4 tensor path: out of device memory for the pass");
    cudaMemsetAsync(c->tc_status, 0, 4, st);
    k_tc_build_tiles<<<1, 1024, 0, st>>>(pair_off, wg.expert_lo + wg.n_expert, wg.expert_lo, wg.n_expert, tiles, c->tc_n_tiles, (int)max_tiles, (int)kbs);
    const size_t x_rows = rows_div == 1 ? (size_t)n_pairs : rows_div >= n_pairs ? 1 : ((size_t)n_pairs + rows_div - 1) / rows_div;
    const size_t nq = x_rows * (wg.n_in / 16);
    k_tc_quant_rows<<<(unsigned)((nq + 255) / 256), 256, 0, st>>>(x, nq, c->tc_codes, c->tc_scales);
    // scale tiles of a pass are whole 512-byte tiles: rows past npad of a tile's scale tile are never read by a matrix of npad rows
    k_tc_gather_tiles<<<dim3((unsigned)max_tiles, 4), 256, 0, st>>>(c->tc_codes, c->tc_scales, wg.n_in, pair_list, rows_div, tiles, c->tc_n_tiles, c->tc_b_img, c->tc_b_sf);
    TcGemm g{};
    g.wg_img = tg->img; g.wg_sf = tg->sf; g.wu_img = tu ? tu->img : nullptr; g.wu_sf = tu ? tu->sf : nullptr;
    g.s2g = wg.scale2; g.s2u = wu ? wu->scale2 : nullptr; g.expert_lo = wg.expert_lo;
    g.b_img = c->tc_b_img; g.b_sf = c->tc_b_sf; g.tiles = tiles; g.n_tiles = c->tc_n_tiles; g.pair_list = pair_list;
    g.n_out = wg.n_out; g.n_in = wg.n_in; g.out = out; g.out_stride = wg.n_out; g.status = c->tc_status;
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(k_tc_gemm<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_gemm_smem(true));
        cudaFuncSetAttribute(k_tc_gemm<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_gemm_smem(true));
        cudaFuncSetAttribute(k_tc_gemm<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_gemm_smem(false));
        attr = true;
    }
    const size_t n_blocks = std::min<size_t>((size_t)c->sm_count, max_tiles * (size_t)(wg.n_out / TC_M));
    const dim3 grid((unsigned)n_blocks);
    static const bool prof_on = getenv("ITB_TC_PROF") != nullptr;
    if (prof_on) { cudaMalloc(&g.prof, n_blocks * 64); cudaMemsetAsync(g.prof, 0, n_blocks * 64, st); }
    if (wu && c->exact) k_tc_gemm<true, true><<<grid, 320, tc_gemm_smem(true), st>>>(g);
    else if (wu) k_tc_gemm<true, false><<<grid, 320, tc_gemm_smem(true), st>>>(g);
    else k_tc_gemm<false, false><<<grid, 320, tc_gemm_smem(false), st>>>(g);
    if (prof_on && g.prof) {
        std::vector<long long> h(n_blocks * 8);
        cudaStreamSynchronize(st);
        cudaMemcpy(h.data(), g.prof, n_blocks * 64, cudaMemcpyDeviceToHost);
        cudaFree(g.prof);
        double acc[5] = {0, 0, 0, 0, 0}, items = 0, cols = 0; size_t n = 0;
        for (size_t b = 0; b < n_blocks; ++b) {
            const long long* q = &h[b * 8];
            if (!q[0] || !q[5] || !q[6]) continue;
            acc[0] += (double)q[1]; acc[1] += (double)q[2]; acc[2] += (double)q[3]; acc[3] += (double)q[4]; acc[4] += (double)(q[5] - q[0]);
            items += (double)q[6]; cols += (double)q[7]; ++n;
        }
        if (n) fprintf(stderr, "tc_gemm glu=%d blocks %zu, items %.0f (avg cols %.0f): cycles per item: MMA thread waiting for operands %.0f, for tensor memory %.0f; "
                               "epilogue waiting for accumulators %.0f, reading + arithmetic + stores %.0f; whole block per item %.0f\n",
                       wu ? 1 : 0, n, items, cols / items, acc[0] / items, acc[1] / items, acc[2] / items, acc[3] / items, acc[4] / items);
    }
    c->launches += 4;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return itb_fail(c, "FP4 tensor path: launch", e);
    return true;
}
// The status word of the last pass: 0 fine; 3 / 4 / 5: a (bounded) wait of the producer / the MMA warp / an epilogue warp ran out.
int itb_tc_status(itb_ctx* c, cudaStream_t st) {
    int v = 0;
    if (!c->tc_status) return 0;
    cudaMemcpyAsync(&v, c->tc_status, 4, cudaMemcpyDeviceToHost, st);
    cudaStreamSynchronize(st);
    return v;
}

// FP4 activation quantiser on its own (tests against the CPU statement, src/ops/naive.rs:755-788): x[n] (n a multiple of 16) ->
// one UE4M3 scale code per 16 elements and one E2M1 code per element (a byte each, like the CPU record).
extern "C" int itb_fp4_quantize(itb_ctx* c, const float* x, size_t n, uint8_t* scales_out, uint8_t* codes_out) {
    if (n % 16) { itb_fail_msg(c, "fp4_quantize: length must be a multiple of 16"); return 1; }
    float* dx = nullptr; uint8_t *ds = nullptr, *dc = nullptr;
    if (cudaMalloc(&dx, n * 4) != cudaSuccess || cudaMalloc(&ds, n / 16) != cudaSuccess || cudaMalloc(&dc, n) != cudaSuccess) {
        cudaFree(dx); cudaFree(ds); itb_fail_msg(c, "fp4_quantize: out of device memory"); return 1;
    }
    cudaMemcpyAsync(dx, x, n * 4, cudaMemcpyHostToDevice, c->stream);
    k_fp4_quant_plain<<<(unsigned)((n / 16 + 127) / 128), 128, 0, c->stream>>>(dx, n / 16, ds, dc);
    ITB_LAUNCHED(c);
    cudaMemcpyAsync(scales_out, ds, n / 16, cudaMemcpyDeviceToHost, c->stream);
    cudaMemcpyAsync(codes_out, dc, n, cudaMemcpyDeviceToHost, c->stream);
    cudaError_t e = cudaStreamSynchronize(c->stream);
    cudaFree(dx); cudaFree(ds); cudaFree(dc);
    if (e != cudaSuccess) { itb_fail(c, "fp4_quantize", e); return 1; }
    return 0;
}

// =====================================================================================================
// Dense Q8_0 matmuls of many-row passes on the tensor cores, bit for bit
// =====================================================================================================
// The CPU path's Q8_0 dot (src/ops/naive.rs:676-712) is, per 32-element block, an integer dot product, converted to f32,
// times (weight scale * activation scale), added to the row's sum in block order. The integer dot of 128 weight rows against
// 128 activation rows is ONE tcgen05.mma kind::i8 (M 128, N 128, K 32, s32 accumulators in tensor memory, not accumulating);
// four accumulator buffers rotate through the 512 columns, so the tensor core runs blocks ahead while eight warps read a
// finished block back (tcgen05.ld) and apply the two scales and the addition in the CPU's own order and rounding. The result
// equals the CPU path to the bit; what bounds the kernel is those four f32 instructions per (output, block) on the CUDA
// cores -- the same count the mma.sync kernels pay, without their shared-memory operand traffic.
// Operand images ("K32 block": 128 rows x 32 int8 = 4096 B as [2 chunks of 16 B][16][8 rows][16 B], K-major, no swizzle;
// descriptor leading offset 2048, stride offset 128) are made once per weight matrix and once per pass for the activations.
namespace {

constexpr int Q8_KB = 4;           // K32 blocks per pipeline stage
constexpr int Q8_STAGES = 5;
constexpr int Q8_STAGE_BYTES = 2 * Q8_KB * 4096 + 2 * Q8_KB * 128 * 4;     // A | B | weight scales | activation scales

// kind::i8: s32 accumulators (2 at bit 4), signed 8-bit operands (1 at bits 7 and 10), both K-major, M x N
__host__ __device__ constexpr uint32_t tc_idesc_i8(int m, int n) { return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }

// int8 rows -> K32 block images, scales -> f32 per (row tile, block, row). One thread per (row, block); rows past n_rows are zeros.
// scales16 (f16, per weight row and block) or scales32 (f32, per activation row and block): whichever is not null.
__global__ void k_q8_tile(const int8_t* q, const uint16_t* scales16, const float* scales32, int n_rows, int n_in, uint8_t* img, float* sc_out) {
    const int kbs = n_in / 32;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x, total = (size_t)((n_rows + 127) / 128) * 128 * kbs;
    if (idx >= total) return;
    const int kb = (int)(idx % kbs); const size_t row = idx / kbs;
    const int rt = (int)(row / 128), r = (int)(row % 128);
    uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
    float sc = 0.0f;
    if (row < (size_t)n_rows) {
        const uint4* src = (const uint4*)(q + row * n_in + (size_t)kb * 32);
        lo = src[0]; hi = src[1];
        sc = scales16 ? f16_bits_to_f32(scales16[row * kbs + kb]) : scales32[row * kbs + kb];
    }
    uint8_t* blk = img + ((size_t)rt * kbs + kb) * 4096;
    *(uint4*)(blk + (r >> 3) * 128 + (r & 7) * 16) = lo;
    *(uint4*)(blk + 2048 + (r >> 3) * 128 + (r & 7) * 16) = hi;
    sc_out[((size_t)rt * kbs + kb) * 128 + r] = sc;
}

struct TcQ8 {
    const uint8_t* a_img; const float* a_sc;      // weights: [row tile][block][4096 B], [row tile][block][128]
    const uint8_t* b_img; const float* b_sc;      // activations of the pass, the same form over token tiles
    int kbs, n_rows, n_out;
    float* out; size_t stride; int mode;          // out[token][row]; mode 1: += (the residual add of an output projection)
    int* status;
    long long* prof;                              // optional: 8 cycle counts per block (ITB_TC_PROF=1)
};
// grid (n_out / 128, token tiles); block 320: warps 0-7 read accumulators back and scale (lane quarter = warp % 4, column half =
// warp / 4), warp 8 fetches operands, warp 9 issues the MMAs.
__global__ void __launch_bounds__(320, 1) k_tc_q8(TcQ8 p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ unsigned long long s_full[Q8_STAGES], s_empty[Q8_STAGES], s_dfull[4], s_dfree[4];
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int rt = blockIdx.x, tt = blockIdx.y, kbs = p.kbs, n_stage = kbs / Q8_KB;
    const uint32_t sbase = tc_smem(smem);
    if (tid == 0) {
        for (int s = 0; s < Q8_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&s_full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 9;" ::"r"(tc_smem(&s_empty[s])) : "memory");      // the MMAs' commit + 8 warps done with the scales
        }
        for (int i = 0; i < 4; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&s_dfull[i])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;" ::"r"(tc_smem(&s_dfree[i])) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (wid == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(tc_smem(&s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tm = s_tmem;
    constexpr uint32_t O_B = Q8_KB * 4096, O_SA = 2 * Q8_KB * 4096, O_SB = O_SA + Q8_KB * 128 * 4;
    bool ok = true;
    if (wid == 8 && lane == 0) {
        const size_t a0 = (size_t)rt * kbs, b0 = (size_t)tt * kbs;
        for (int st = 0; st < n_stage && ok; ++st) {
            const int s = st % Q8_STAGES;
            if (st >= Q8_STAGES) ok = tc_mbar_wait(tc_smem(&s_empty[s]), ((st / Q8_STAGES) - 1) & 1, 2000000000ull);
            if (!ok) break;
            const uint32_t full = tc_smem(&s_full[s]), dst = sbase + s * Q8_STAGE_BYTES;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"((uint32_t)Q8_STAGE_BYTES) : "memory");
            const size_t kb0 = (size_t)st * Q8_KB;
            tc_bulk(dst, p.a_img + (a0 + kb0) * 4096, Q8_KB * 4096, full);
            tc_bulk(dst + O_B, p.b_img + (b0 + kb0) * 4096, Q8_KB * 4096, full);
            tc_bulk(dst + O_SA, p.a_sc + (a0 + kb0) * 128, Q8_KB * 128 * 4, full);
            tc_bulk(dst + O_SB, p.b_sc + (b0 + kb0) * 128, Q8_KB * 128 * 4, full);
        }
        if (!ok) atomicCAS(p.status, 0, 3);
    } else if (wid == 9 && lane == 0) {
        const uint32_t idesc = tc_idesc_i8(128, 128);
        const uint64_t dA = tc_desc(sbase, 2048, 128), dB = tc_desc(sbase + O_B, 2048, 128);
        for (int b = 0; b < kbs && ok; ++b) {
            const int s = (b / Q8_KB) % Q8_STAGES, k = b % Q8_KB, db = b & 3;
            if (k == 0) {
                ok = tc_mbar_wait(tc_smem(&s_full[s]), ((b / Q8_KB) / Q8_STAGES) & 1, 2000000000ull);
                if (!ok) break;
            }
            if (b >= 4) {
                ok = tc_mbar_wait(tc_smem(&s_dfree[db]), ((b >> 2) - 1) & 1, 2000000000ull);
                if (!ok) break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t so = (uint32_t)s * (Q8_STAGE_BYTES >> 4) + 256u * k;
            asm volatile(
                "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }\n"
                ::"r"(tm + 128u * db), "l"(dA + so), "l"(dB + so), "r"(idesc), "r"(0u) : "memory");
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&s_dfull[db])) : "memory");
            if (k == Q8_KB - 1) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&s_empty[s])) : "memory");
        }
        if (!ok) atomicCAS(p.status, 0, 4);
    } else if (wid < 8) {
        const int quarter = wid & 3, half = wid >> 2, row = quarter * 32 + lane;
        float acc[64];
#pragma unroll
        for (int j = 0; j < 64; ++j) acc[j] = 0.0f;
        uint32_t d0[32], d1[32];
        // start reading 32 of this warp's 64 columns of block b's accumulators (asynchronous: tcgen05.wait::ld ends it); the first
        // half of a block also waits for the block's MMA (and, at a stage's first block, for the stage's scales)
        auto fetch = [&](int b, int h, uint32_t (&d)[32]) {
            const int s = (b / Q8_KB) % Q8_STAGES, k = b % Q8_KB, db = b & 3;
            if (h == 0) {
                if (k == 0) ok = ok && __all_sync(0xffffffffu, tc_mbar_wait(tc_smem(&s_full[s]), ((b / Q8_KB) / Q8_STAGES) & 1, 2000000000ull));
                ok = ok && __all_sync(0xffffffffu, tc_mbar_wait(tc_smem(&s_dfull[db]), (b >> 2) & 1, 2000000000ull));
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            if (!ok) return;
            const uint32_t ta = tm + 128u * db + 64u * half + 32u * h + ((uint32_t)(quarter * 32) << 16);
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]),
                           "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]), "=r"(d[16]), "=r"(d[17]), "=r"(d[18]), "=r"(d[19]), "=r"(d[20]), "=r"(d[21]), "=r"(d[22]),
                           "=r"(d[23]), "=r"(d[24]), "=r"(d[25]), "=r"(d[26]), "=r"(d[27]), "=r"(d[28]), "=r"(d[29]), "=r"(d[30]), "=r"(d[31]) : "r"(ta) : "memory");
        };
        // scale and add 32 columns of block b in the CPU's order: sum += (float)dot * (dw * dx). The conversion is exact either way
        // (|dot| <= 32 * 127 * 127 < 2^23); through the magic constant 1.5 * 2^23 it is an integer add and a float add instead of
        // a quarter-rate convert.
        auto scale_add = [&](int b, int h, const uint32_t (&d)[32]) {
            const int s = (b / Q8_KB) % Q8_STAGES, k = b % Q8_KB;
            const float* sa = (const float*)(smem + (size_t)s * Q8_STAGE_BYTES + O_SA) + k * 128;
            const float* sb = (const float*)(smem + (size_t)s * Q8_STAGE_BYTES + O_SB) + k * 128 + 64 * half + 32 * h;
            const float dw = sa[row];
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 dx = *(const float4*)(sb + j);
                const float dxs[4] = {dx.x, dx.y, dx.z, dx.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float f = __fadd_rn(__uint_as_float(0x4b400000u + d[j + i]), -12582912.0f);
                    acc[32 * h + j + i] = __fadd_rn(acc[32 * h + j + i], __fmul_rn(f, __fmul_rn(dw, dxs[i])));
                }
            }
        };
        long long* pf = p.prof ? p.prof + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 8 : nullptr;
        long long t_wait = 0, t_fetch = 0; const long long t_begin = clock64();
        fetch(0, 0, d0); fetch(0, 1, d1);
#pragma unroll 1
        for (int b = 0; b < kbs && ok; ++b) {
            const long long tw0 = clock64();
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");      // both halves of block b are in registers
            t_wait += clock64() - tw0;
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(&s_dfree[b & 3])) : "memory");
            scale_add(b, 0, d0);
            const long long tf0 = clock64();
            if (b + 1 < kbs) fetch(b + 1, 0, d0);                             // lands while the second half is being added
            t_fetch += clock64() - tf0;
            scale_add(b, 1, d1);
            if (b + 1 < kbs) fetch(b + 1, 1, d1);
            if (b % Q8_KB == Q8_KB - 1) {
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(&s_empty[(b / Q8_KB) % Q8_STAGES])) : "memory");
            }
        }
        if (pf && tid == 0) { pf[0] = clock64() - t_begin; pf[1] = t_wait; pf[2] = t_fetch; pf[3] = kbs; }
        if (ok && __shfl_sync(0xffffffffu, *(volatile int*)p.status, 0) == 0) {
            const size_t orow = (size_t)rt * 128 + row;
            // mode 1 reads what it adds to: all of a batch's reads first, then the stores (a read placed after a store that may
            // alias it waits for nothing, but the compiler keeps their order, and one read-add-store at a time is a memory round
            // trip per column)
#pragma unroll
            for (int j0 = 0; j0 < 64; j0 += 16) {
                float old[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = tt * 128 + 64 * half + j0 + j;
                    old[j] = (p.mode && tok < p.n_rows) ? p.out[(size_t)tok * p.stride + orow] : 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = tt * 128 + 64 * half + j0 + j;
                    if (tok < p.n_rows) p.out[(size_t)tok * p.stride + orow] = p.mode ? __fadd_rn(old[j], acc[j0 + j]) : acc[j0 + j];
                }
            }
        } else if (!ok) atomicCAS(p.status, 0, 5);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (wid == 9) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tm) : "memory");
}
constexpr size_t tc_q8_smem() { return (size_t)Q8_STAGES * Q8_STAGE_BYTES + 128; }

}  // namespace

bool itb_tc_q8_shape_ok(const DevQ8& w) { return w.n_in % (32 * Q8_KB) == 0 && w.n_out % 128 == 0 && w.q && w.s; }
// out[token][row] (+)= W x for n_rows quantised activation rows (xq int8 [n_rows][n_in], xs f32 [n_rows][n_in / 32]). False: not run.
bool itb_tc_q8_gemm(itb_ctx* c, cudaStream_t st, const DevQ8& w, const int8_t* xq, const float* xs, int n_rows, float* out, size_t stride, int mode, bool same_acts) {
    if (!itb_tc_q8_shape_ok(w) || n_rows <= 0) return false;
    const size_t kbs = w.n_in / 32, rts = w.n_out / 128, tts = ((size_t)n_rows + 127) / 128;
    auto it = c->tc_weights.find(w.q);
    if (it == c->tc_weights.end()) {
        itb_ctx::TcWeights t;
        if (cudaMalloc(&t.img, rts * kbs * 4096) != cudaSuccess) { cudaGetLastError(); return itb_fail_msg(c, "Q8_0 tensor path: out of device memory for the tiled weights"); }
        if (cudaMalloc(&t.sf, rts * kbs * 128 * 4) != cudaSuccess) { cudaFree(t.img); cudaGetLastError(); return itb_fail_msg(c, "Q8_0 tensor path: out of device memory for the tiled weights"); }
        t.bytes = rts * kbs * (4096 + 512);
        const size_t n = rts * 128 * kbs;
        k_q8_tile<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(w.q, w.s, nullptr, w.n_out, w.n_in, t.img, (float*)t.sf);
        c->launches++;
        it = c->tc_weights.emplace(w.q, t).first;
    }
    size_t cap1 = c->tc_status ? 1 : 0;
    bool ok = tc_grow(&c->tc_status, &cap1, 1, st) && tc_grow(&c->tc_q8_b, &c->tc_cap_q8b, tts * kbs * 4096, st) && tc_grow(&c->tc_q8_sx, &c->tc_cap_q8sx, tts * kbs * 128, st);
    if (!ok) return itb_fail_msg(c, "Q8_0 tensor path: out of device memory for the pass");
    // same_acts: the caller vouches that xq/xs hold what the previous call's did (consecutive matmuls over one quantised row set)
    if (!same_acts || c->tc_q8_src != xq || c->tc_q8_src_rows != n_rows || c->tc_q8_src_in != w.n_in) {
        const size_t n = tts * 128 * kbs;
        k_q8_tile<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(xq, nullptr, xs, n_rows, w.n_in, c->tc_q8_b, c->tc_q8_sx);
        c->launches++;
        c->tc_q8_src = xq; c->tc_q8_src_rows = n_rows; c->tc_q8_src_in = w.n_in;
    }
    cudaMemsetAsync(c->tc_status, 0, 4, st);
    TcQ8 g{};
    g.a_img = it->second.img; g.a_sc = (const float*)it->second.sf; g.b_img = c->tc_q8_b; g.b_sc = c->tc_q8_sx; g.kbs = (int)kbs; g.n_rows = n_rows; g.n_out = w.n_out;
    g.out = out; g.stride = stride; g.mode = mode; g.status = c->tc_status;
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(k_tc_q8, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_q8_smem()); attr = true; }
    static const bool prof_on = getenv("ITB_TC_PROF") != nullptr;
    const size_t n_blocks = rts * tts;
    if (prof_on) { cudaMalloc(&g.prof, n_blocks * 64); cudaMemsetAsync(g.prof, 0, n_blocks * 64, st); }
    k_tc_q8<<<dim3((unsigned)rts, (unsigned)tts), 320, tc_q8_smem(), st>>>(g);
    c->launches++;
    if (prof_on && g.prof) {
        std::vector<long long> h(n_blocks * 8);
        cudaStreamSynchronize(st);
        cudaMemcpy(h.data(), g.prof, n_blocks * 64, cudaMemcpyDeviceToHost);
        cudaFree(g.prof);
        double a[3] = {0, 0, 0}; size_t n = 0;
        for (size_t b = 0; b < n_blocks; ++b) if (h[b * 8]) { a[0] += (double)h[b * 8]; a[1] += (double)h[b * 8 + 1]; a[2] += (double)h[b * 8 + 2]; ++n; }
        if (n) fprintf(stderr, "tc_q8 %d x %d, %zu K32 blocks, %zu blocks: cycles per K32 block %.0f (waiting for the accumulator loads %.0f, for the next block's MMA %.0f)\n",
                       w.n_out, n_rows, kbs, n, a[0] / n / kbs, a[1] / n / kbs, a[2] / n / kbs);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return itb_fail(c, "Q8_0 tensor path: launch", e);
    return true;
}

// =====================================================================================================
// Dense Q8_0 matmuls of many-row passes as f16 tensor-core GEMMs (tolerance class, opts dense=f16tc)
// =====================================================================================================
// Both operands are dequantised once -- the weights when first used, the pass's Q8_0-quantised activation rows (the same
// quantisation the CPU path applies, src/ops/naive.rs:676-712) once per row set -- to f16 (value = int8 * block scale, rounded
// to nearest even: 2^-12 relative per element; with bf16 operands, 2^-9, a 4-layer model's logits were 0.3 off), laid out as
// K-major operand tiles, and multiplied by tcgen05.mma kind::f16 with f32 accumulators in tensor memory. What differs from the CPU path: that rounding, and the tensor core's summation order in
// place of the per-block order. A tile is 128 weight rows x 256 tokens; two accumulator buffers fill the 512 columns of tensor
// memory, so the MMAs of one tile run while eight warps store the previous one. Persistent blocks, one per SM, token tile
// fastest: the blocks running at one time share a few weight tiles and all of the pass's activation tiles in L2.
// Operand images ("K16 block": rows x 16 f16 = rows x 32 B as [2 chunks of 16 B][rows / 8][8 rows][16 B], no swizzle; descriptor
// leading offset rows * 16, stride offset 128).
namespace {

constexpr int HF_KB = 4;                 // K16 blocks per pipeline stage (64 elements)
constexpr int HF_STAGES = 4;
constexpr int HF_N = 256;                // tokens per tile
constexpr int HF_A_BLK = 128 * 32, HF_B_BLK = HF_N * 32;
constexpr int HF_STAGE_BYTES = HF_KB * (HF_A_BLK + HF_B_BLK);

// kind::f16: f32 accumulators (1 at bit 4), f16 operands (0 at bits 7 and 10), both K-major, M x N
__host__ __device__ constexpr uint32_t tc_idesc_f16(int m, int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }

__device__ __forceinline__ uint32_t f16x2_rn(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// Q8_0 rows -> f16 K16 block images of ROWS-row tiles. One thread per (row, K16 block); a warp takes 8 rows x 4 blocks, so it
// reads 64 contiguous bytes per row and writes 128 contiguous bytes per block and chunk. Rows past n_rows are zeros.
// scales16 (f16, per weight row and 32-element block) or scales32 (f32, per activation row and block): whichever is not null.
template <int ROWS>
__global__ void k_f16_tile(const int8_t* q, const uint16_t* scales16, const float* scales32, int n_rows, int n_in, uint8_t* img) {
    const int kbs = n_in / 16;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x, total = (size_t)((n_rows + ROWS - 1) / ROWS) * ROWS * kbs;
    if (idx >= total) return;
    const int r_lo = (int)(idx & 7), kb_lo = (int)((idx >> 3) & 3);
    const size_t rest = idx >> 5;
    const int kb = (int)(rest % (size_t)(kbs / 4)) * 4 + kb_lo;
    const size_t row = (rest / (size_t)(kbs / 4)) * 8 + r_lo;
    const int rt = (int)(row / ROWS), r = (int)(row % ROWS);
    uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
    if (row < (size_t)n_rows) {
        const uint4 v = *(const uint4*)(q + row * n_in + (size_t)kb * 16);
        const size_t si = row * (size_t)(n_in / 32) + (kb >> 1);
        const float sc = scales16 ? f16_bits_to_f32(scales16[si]) : scales32[si];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float f0 = (float)(int8_t)(w[i] & 0xff) * sc, f1 = (float)(int8_t)((w[i] >> 8) & 0xff) * sc;
            const float f2 = (float)(int8_t)((w[i] >> 16) & 0xff) * sc, f3 = (float)(int8_t)(w[i] >> 24) * sc;
            o[2 * i] = f16x2_rn(f0, f1); o[2 * i + 1] = f16x2_rn(f2, f3);
        }
        lo = make_uint4(o[0], o[1], o[2], o[3]); hi = make_uint4(o[4], o[5], o[6], o[7]);
    }
    uint8_t* blk = img + ((size_t)rt * kbs + kb) * (size_t)(ROWS * 32);
    *(uint4*)(blk + (r >> 3) * 128 + (r & 7) * 16) = lo;
    *(uint4*)(blk + ROWS * 16 + (r >> 3) * 128 + (r & 7) * 16) = hi;
}

struct TcHf {
    const uint8_t* a_img;                         // weights: [row tile][K16 block][4096 B]
    const uint8_t* b_img;                         // activations of the pass: [token tile][K16 block][8192 B]
    int kbs, n_rows, n_rt, n_tt;                  // K16 blocks, tokens, row tiles, token tiles
    float* out; size_t stride; int mode;          // out[token][row]; mode 1: += (the residual add of an output projection)
    int* status;
    long long* prof;                              // optional: 8 cycle counts per block (ITB_TC_PROF=1)
};
// grid: one block per SM (or per work item, if fewer); block 320: warps 0-7 store accumulators (lane quarter = warp % 4, column half
// = warp / 4), warp 8 fetches operands, warp 9 issues the MMAs.
__global__ void __launch_bounds__(320, 1) k_tc_f16(TcHf p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ unsigned long long s_full[HF_STAGES], s_empty[HF_STAGES], s_acc[2], s_free[2];
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int n_work = p.n_rt * p.n_tt, kbs = p.kbs, n_stage = kbs / HF_KB;
    if ((int)blockIdx.x >= n_work) return;
    const uint32_t sbase = tc_smem(smem);
    if (tid == 0) {
        for (int s = 0; s < HF_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&s_full[s])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&s_empty[s])) : "memory");
        }
        for (int i = 0; i < 2; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem(&s_acc[i])) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;" ::"r"(tc_smem(&s_free[i])) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (wid == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(tc_smem(&s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tm = s_tmem;
    const unsigned long long limit = 2000000000ull;
    long long* pf = p.prof ? p.prof + (size_t)blockIdx.x * 8 : nullptr;
    if (pf && tid == 0) pf[0] = clock64();
    bool ok = true;
    if (wid == 8 && lane == 0) {
        int it = 0;
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
            const size_t a0 = (size_t)(w / p.n_tt) * kbs, b0 = (size_t)(w % p.n_tt) * kbs;
            for (int st = 0; st < n_stage; ++st, ++it) {
                const int s = it % HF_STAGES;
                if (it >= HF_STAGES) ok = tc_mbar_wait(tc_smem(&s_empty[s]), ((it / HF_STAGES) - 1) & 1, limit);
                if (!ok) break;
                const uint32_t full = tc_smem(&s_full[s]), dst = sbase + s * HF_STAGE_BYTES;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full), "r"((uint32_t)HF_STAGE_BYTES) : "memory");
                const size_t kb0 = (size_t)st * HF_KB;
                tc_bulk(dst, p.a_img + (a0 + kb0) * HF_A_BLK, HF_KB * HF_A_BLK, full);
                tc_bulk(dst + HF_KB * HF_A_BLK, p.b_img + (b0 + kb0) * HF_B_BLK, HF_KB * HF_B_BLK, full);
            }
        }
        if (!ok) atomicCAS(p.status, 0, 3);
    } else if (wid == 9 && lane == 0) {
        const uint32_t idesc = tc_idesc_f16(128, HF_N);
        const uint64_t dA = tc_desc(sbase, 128 * 16, 128), dB = tc_desc(sbase + HF_KB * HF_A_BLK, HF_N * 16, 128);
        int it = 0, item = 0;
        long long t_load = 0, t_free = 0;
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++item) {
            const int buf = item & 1;
            if (item >= 2) {                                  // the warps that store have read this buffer's previous tile
                const long long c0 = pf ? clock64() : 0;
                ok = tc_mbar_wait(tc_smem(&s_free[buf]), ((item >> 1) - 1) & 1, limit);
                if (pf) t_free += clock64() - c0;
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            for (int st = 0; st < n_stage; ++st, ++it) {
                const int s = it % HF_STAGES;
                const long long c0 = pf ? clock64() : 0;
                ok = tc_mbar_wait(tc_smem(&s_full[s]), (it / HF_STAGES) & 1, limit);
                if (pf) t_load += clock64() - c0;
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t so = (uint32_t)s * (HF_STAGE_BYTES >> 4);
#pragma unroll
                for (int k = 0; k < HF_KB; ++k) {
                    asm volatile(
                        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }\n"
                        ::"r"(tm + (uint32_t)(HF_N * buf)), "l"(dA + so + (uint32_t)(k * (HF_A_BLK >> 4))), "l"(dB + so + (uint32_t)(k * (HF_B_BLK >> 4))), "r"(idesc),
                          "r"((st | k) ? 1u : 0u) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&s_empty[s])) : "memory");
            }
            if (!ok) break;
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem(&s_acc[buf])) : "memory");
        }
        if (!ok) atomicCAS(p.status, 0, 4);
        if (pf) { pf[1] = t_load; pf[2] = t_free; }
    } else if (wid < 8) {
        const int quarter = wid & 3, half = wid >> 2, row = quarter * 32 + lane;
        int item = 0;
        long long t_wait = 0, t_work = 0;
        for (int w = blockIdx.x; w < n_work; w += gridDim.x, ++item) {
            const int buf = item & 1, rt = w / p.n_tt, tt = w % p.n_tt;
            const long long k0 = pf ? clock64() : 0;
            ok = __all_sync(0xffffffffu, tc_mbar_wait(tc_smem(&s_acc[buf]), (item >> 1) & 1, limit));
            if (!ok || __shfl_sync(0xffffffffu, *(volatile int*)p.status, 0) != 0) break;
            const long long k1 = pf ? clock64() : 0;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* ocol = p.out + (size_t)rt * 128 + row;
#pragma unroll 1
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t d[32];
                const uint32_t ta = tm + (uint32_t)(HF_N * buf + 128 * half + 32 * ch) + ((uint32_t)(quarter * 32) << 16);
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                             : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]),
                               "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]), "=r"(d[16]), "=r"(d[17]), "=r"(d[18]), "=r"(d[19]), "=r"(d[20]), "=r"(d[21]), "=r"(d[22]),
                               "=r"(d[23]), "=r"(d[24]), "=r"(d[25]), "=r"(d[26]), "=r"(d[27]), "=r"(d[28]), "=r"(d[29]), "=r"(d[30]), "=r"(d[31]) : "r"(ta) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (ch == 3) {
                    // the whole buffer has been read: it goes back to the MMA warp
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem(&s_free[buf])) : "memory");
                }
                const int tok0 = tt * HF_N + 128 * half + 32 * ch;
                // mode 1 reads what it adds to: 16 reads first, then their stores (one read-add-store at a time is a memory round
                // trip per column: the compiler keeps a read behind the store before it)
#pragma unroll
                for (int j0 = 0; j0 < 32; j0 += 16) {
                    float old[16];
                    float* o0 = ocol + (size_t)(tok0 + j0) * p.stride;
#pragma unroll
                    for (int j = 0; j < 16; ++j) old[j] = (p.mode && tok0 + j0 + j < p.n_rows) ? o0[(size_t)j * p.stride] : 0.0f;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (tok0 + j0 + j < p.n_rows) o0[(size_t)j * p.stride] = old[j] + __uint_as_float(d[j0 + j]);
                }
            }
            if (pf) { t_wait += k1 - k0; t_work += clock64() - k1; }
        }
        if (!ok) atomicCAS(p.status, 0, 5);
        if (pf && tid == 0) { pf[3] = t_wait; pf[4] = t_work; pf[6] = item; }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (wid == 9) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tm) : "memory");
    if (pf && tid == 0) pf[5] = clock64();
}
constexpr size_t tc_f16_smem() { return (size_t)HF_STAGES * HF_STAGE_BYTES + 128; }

}  // namespace

bool itb_tc_f16_shape_ok(const DevQ8& w) { return w.n_in % (16 * HF_KB) == 0 && w.n_out % 128 == 0 && w.q && w.s; }
// out[token][row] (+)= W x for n_rows quantised activation rows (xq int8 [n_rows][n_in], xs f32 [n_rows][n_in / 32]). False: not run.
bool itb_tc_f16_gemm(itb_ctx* c, cudaStream_t st, const DevQ8& w, const int8_t* xq, const float* xs, int n_rows, float* out, size_t stride, int mode, bool same_acts) {
    if (!itb_tc_f16_shape_ok(w) || n_rows <= 0) return false;
    const size_t kbs = w.n_in / 16, rts = w.n_out / 128, tts = ((size_t)n_rows + HF_N - 1) / HF_N;
    auto it = c->tc_weights.find(w.s);                       // keyed by the scale array: the int8 images of dense=q8tc are keyed by w.q
    if (it == c->tc_weights.end()) {
        itb_ctx::TcWeights t;
        if (cudaMalloc(&t.img, rts * kbs * HF_A_BLK) != cudaSuccess) { cudaGetLastError(); return itb_fail_msg(c, "f16 tensor path: out of device memory for the tiled weights"); }
        t.sf = nullptr; t.bytes = rts * kbs * HF_A_BLK;
        const size_t n = rts * 128 * kbs;
        k_f16_tile<128><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(w.q, w.s, nullptr, w.n_out, w.n_in, t.img);
        c->launches++;
        it = c->tc_weights.emplace(w.s, t).first;
    }
    size_t cap1 = c->tc_status ? 1 : 0;
    bool ok = tc_grow(&c->tc_status, &cap1, 1, st) && tc_grow(&c->tc_hf_b, &c->tc_cap_hfb, tts * kbs * HF_B_BLK, st);
    if (!ok) return itb_fail_msg(c, "f16 tensor path: out of device memory for the pass");
    // same_acts: the caller vouches that xq/xs hold what the previous call's did (consecutive matmuls over one quantised row set)
    if (!same_acts || c->tc_hf_src != xq || c->tc_hf_src_rows != n_rows || c->tc_hf_src_in != w.n_in) {
        const size_t n = tts * HF_N * kbs;
        k_f16_tile<HF_N><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(xq, nullptr, xs, n_rows, w.n_in, c->tc_hf_b);
        c->launches++;
        c->tc_hf_src = xq; c->tc_hf_src_rows = n_rows; c->tc_hf_src_in = w.n_in;
    }
    cudaMemsetAsync(c->tc_status, 0, 4, st);
    TcHf g{};
    g.a_img = it->second.img; g.b_img = c->tc_hf_b; g.kbs = (int)kbs; g.n_rows = n_rows; g.n_rt = (int)rts; g.n_tt = (int)tts;
    g.out = out; g.stride = stride; g.mode = mode; g.status = c->tc_status;
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(k_tc_f16, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_f16_smem()); attr = true; }
    static const bool prof_on = getenv("ITB_TC_PROF") != nullptr;
    const size_t n_blocks = std::min<size_t>((size_t)c->sm_count, rts * tts);
    if (prof_on) { cudaMalloc(&g.prof, n_blocks * 64); cudaMemsetAsync(g.prof, 0, n_blocks * 64, st); }
    k_tc_f16<<<(unsigned)n_blocks, 320, tc_f16_smem(), st>>>(g);
    c->launches++;
    if (prof_on && g.prof) {
        std::vector<long long> h(n_blocks * 8);
        cudaStreamSynchronize(st);
        cudaMemcpy(h.data(), g.prof, n_blocks * 64, cudaMemcpyDeviceToHost);
        cudaFree(g.prof);
        double a[5] = {0, 0, 0, 0, 0}, items = 0;
        for (size_t b = 0; b < n_blocks; ++b) {
            const long long* q = &h[b * 8];
            if (!q[0] || !q[5] || !q[6]) continue;
            a[0] += (double)q[1]; a[1] += (double)q[2]; a[2] += (double)q[3]; a[3] += (double)q[4]; a[4] += (double)(q[5] - q[0]); items += (double)q[6];
        }
        if (items > 0) fprintf(stderr, "tc_f16 %d x %d x %d, items %.0f: cycles per item: MMA thread waiting for operands %.0f, for tensor memory %.0f; stores waiting for accumulators %.0f, "
                                       "reading + stores %.0f; whole block per item %.0f\n", w.n_out, n_rows, w.n_in, items, a[0] / items, a[1] / items, a[2] / items, a[3] / items, a[4] / items);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return itb_fail(c, "f16 tensor path: launch", e);
    return true;
}
