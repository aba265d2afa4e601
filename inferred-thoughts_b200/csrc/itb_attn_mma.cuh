// Causal attention of a many-token pass on the tensor cores (the job of kernels/attention_mma.cuh in the reference): for
// one KV head, the query heads that share it and a run of consecutive tokens form a 128-row tile; K and V tiles of 64
// positions stream through shared memory once per tile (so a position's keys are read once per 128 / group tokens, not once
// per token and head), scores and weighted values are m16n8k16 matrix products in the cache's own 16-bit type with f32
// accumulators, and the softmax is the running (max, sum) form. Tolerance class: q and the probabilities are rounded to the
// cache's type and the sums are reassociated; exact=1 passes keep the CPU-order kernels (itb_attn_exact.cuh).
//
// The result leaves as one "split" of the split-K form (unnormalised values, running max and sum per (row, head)), so the
// pass's usual combine kernel applies the division, the sigmoid gate and the Q8_0 quantisation.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "itb_tile.cuh"

namespace {

constexpr int AM_ROWS = 128;       // (token, head) rows per block
constexpr int AM_KV = 64;          // positions per K/V tile

struct AmParams {
    const float* q;                // [rows][n_head][hd], normed and rotated
    const uint16_t* kslab; const uint16_t* vslab; size_t slab_stride;   // [seq][n_ctx][kv_dim]
    const int* npos;               // positions visible to each row (its own included)
    int n_tok, kv_dim, n_head, n_head_kv, group;
    float scale;
    float* part_acc; float* part_ml;        // [(row, head)][hd], [(row, head)][2]
};

__device__ __forceinline__ uint32_t am_pack(float a, float b, bool bf16) {
    if (bf16) { const __nv_bfloat162 v = __floats2bfloat162_rn(a, b); return *(const uint32_t*)&v; }
    const __half2 v = __floats2half2_rn(a, b);
    return *(const uint32_t*)&v;
}
__device__ __forceinline__ void am_ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void am_ldsm4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void am_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Shared-memory tiles are rows of HD 16-bit values; the 16-byte chunks of a row are permuted by the row's low three bits so
// that the eight rows one ldmatrix phase touches fall on different banks.
template <int HD>
__device__ __forceinline__ uint32_t am_off(int row, int chunk) { return (uint32_t)(row * (HD * 2) + ((chunk ^ (row & 7)) << 4)); }

// grid (ceil(n_tok / (128 / group)), n_head_kv, n_seq); block 256 (8 warps x 16 rows).
template <int HD, bool BF16>
__global__ void __launch_bounds__(256, 1) k_attn_mma(AmParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int ROW_B = HD * 2, CH = HD / 8;                 // bytes and 16-byte chunks per row
    constexpr int Q_B = AM_ROWS * ROW_B, T_B = AM_KV * ROW_B;
    const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(smem), sK = sQ + Q_B, sV = sK + 2 * T_B;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int group = p.group, bm = AM_ROWS / group, t0 = blockIdx.x * bm, hk = blockIdx.y, seq = blockIdx.z;
    const int n_valid_tok = min(bm, p.n_tok - t0);
    const size_t row0 = (size_t)seq * p.n_tok + t0;
    const int kv_end = p.npos[row0 + n_valid_tok - 1];         // positions ascend inside a pass: the tile's last token sees the most
    const uint16_t* kbase = p.kslab + (size_t)seq * p.slab_stride + (size_t)hk * HD;
    const uint16_t* vbase = p.vslab + (size_t)seq * p.slab_stride + (size_t)hk * HD;

    auto load_kv = [&](int tile, int buf) {
        const int kv0 = tile * AM_KV;
        for (int i = tid; i < AM_KV * CH; i += 256) {
            const int r = i / CH, c = i % CH, pos = kv0 + r;
            const bool ok = pos < kv_end;
            const size_t g = (size_t)(ok ? pos : 0) * p.kv_dim + c * 8;
            cp_async16(smem + Q_B + buf * T_B + am_off<HD>(r, c), kbase + g, ok);
            cp_async16(smem + Q_B + 2 * T_B + buf * T_B + am_off<HD>(r, c), vbase + g, ok);
        }
        cp_async_commit();
    };
    load_kv(0, 0);
    // q rows: (token t0 + m / group, head hk * group + m % group), rounded to the cache's type
    for (int i = tid; i < AM_ROWS * (HD / 4); i += 256) {
        const int m = i / (HD / 4), c4 = i % (HD / 4), tq = m / group, g = m % group;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tq < n_valid_tok) v = *(const float4*)(p.q + ((row0 + tq) * p.n_head + hk * group + g) * HD + c4 * 4);
        const uint2 w = make_uint2(am_pack(v.x, v.y, BF16), am_pack(v.z, v.w, BF16));
        *(uint2*)(smem + am_off<HD>(m, c4 >> 1) + (c4 & 1) * 8) = w;
    }
    // this thread's two rows of the warp's 16
    const int m_lo = wid * 16 + (lane >> 2), m_hi = m_lo + 8;
    const int tq_lo = m_lo / group, tq_hi = m_hi / group;
    const int np_lo = tq_lo < n_valid_tok ? p.npos[row0 + tq_lo] : 0, np_hi = tq_hi < n_valid_tok ? p.npos[row0 + tq_hi] : 0;
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = 0.f; o[i][1] = 0.f; o[i][2] = 0.f; o[i][3] = 0.f; }
    float mx_lo = -INFINITY, mx_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    const int n_tiles = (kv_end + AM_KV - 1) / AM_KV;
    const int warp_np_max = __reduce_max_sync(0xffffffffu, max(np_lo, np_hi));
#pragma unroll 1
    for (int tile = 0; tile < n_tiles; ++tile) {
        const int buf = tile & 1, kv0 = tile * AM_KV;
        if (tile + 1 < n_tiles) load_kv(tile + 1, buf ^ 1); else cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (kv0 < warp_np_max) {              // a warp whose rows all end before this tile has nothing to add
            const uint32_t kt = sK + buf * T_B, vt = sV + buf * T_B;
            float s[AM_KV / 8][4];
#pragma unroll
            for (int i = 0; i < AM_KV / 8; ++i) { s[i][0] = 0.f; s[i][1] = 0.f; s[i][2] = 0.f; s[i][3] = 0.f; }
#pragma unroll 2
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t a[4];
                am_ldsm4(sQ + am_off<HD>(wid * 16 + (lane & 15), kk * 2 + (lane >> 4)), a);
#pragma unroll
                for (int np = 0; np < AM_KV / 16; ++np) {
                    uint32_t b[4];
                    const int mi = lane >> 3, pos = np * 16 + (mi >> 1) * 8 + (lane & 7);
                    am_ldsm4(kt + am_off<HD>(pos, kk * 2 + (mi & 1)), b);
                    am_mma<BF16>(s[2 * np], a, b[0], b[1]);
                    am_mma<BF16>(s[2 * np + 1], a, b[2], b[3]);
                }
            }
            // scale, causal mask, running max
            float t_lo = -INFINITY, t_hi = -INFINITY;
#pragma unroll
            for (int i = 0; i < AM_KV / 8; ++i) {
                const int c = kv0 + i * 8 + (lane & 3) * 2;
                s[i][0] = c < np_lo ? s[i][0] * p.scale : -INFINITY; s[i][1] = c + 1 < np_lo ? s[i][1] * p.scale : -INFINITY;
                s[i][2] = c < np_hi ? s[i][2] * p.scale : -INFINITY; s[i][3] = c + 1 < np_hi ? s[i][3] * p.scale : -INFINITY;
                t_lo = fmaxf(t_lo, fmaxf(s[i][0], s[i][1])); t_hi = fmaxf(t_hi, fmaxf(s[i][2], s[i][3]));
            }
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 1)); t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 2));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 1)); t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 2));
            const float n_lo = fmaxf(mx_lo, t_lo), n_hi = fmaxf(mx_hi, t_hi);
            const float f_lo = n_lo == -INFINITY ? 1.0f : __expf(mx_lo - n_lo), f_hi = n_hi == -INFINITY ? 1.0f : __expf(mx_hi - n_hi);
            const float b_lo = n_lo == -INFINITY ? 0.0f : n_lo, b_hi = n_hi == -INFINITY ? 0.0f : n_hi;
            mx_lo = n_lo; mx_hi = n_hi;
            float r_lo = 0.f, r_hi = 0.f;
            uint32_t pa[AM_KV / 16][4];
#pragma unroll
            for (int i = 0; i < AM_KV / 8; ++i) {
                const float e0 = __expf(s[i][0] - b_lo), e1 = __expf(s[i][1] - b_lo), e2 = __expf(s[i][2] - b_hi), e3 = __expf(s[i][3] - b_hi);
                r_lo += e0 + e1; r_hi += e2 + e3;
                pa[i >> 1][(i & 1) * 2] = am_pack(e0, e1, BF16);
                pa[i >> 1][(i & 1) * 2 + 1] = am_pack(e2, e3, BF16);
            }
            l_lo = l_lo * f_lo + r_lo; l_hi = l_hi * f_hi + r_hi;       // per-lane partial sums: the quad is added up at the end
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) { o[i][0] *= f_lo; o[i][1] *= f_lo; o[i][2] *= f_hi; o[i][3] *= f_hi; }
#pragma unroll
            for (int kk = 0; kk < AM_KV / 16; ++kk) {
#pragma unroll
                for (int dp = 0; dp < HD / 16; ++dp) {
                    uint32_t b[4];
                    const int mi = lane >> 3, pos = kk * 16 + (mi & 1) * 8 + (lane & 7);
                    am_ldsm4_t(vt + am_off<HD>(pos, dp * 2 + (mi >> 1)), b);
                    am_mma<BF16>(o[2 * dp], pa[kk], b[0], b[1]);
                    am_mma<BF16>(o[2 * dp + 1], pa[kk], b[2], b[3]);
                }
            }
        }
        __syncthreads();                      // every warp is done with this buffer before the next load overwrites it
    }
    cp_async_wait<0>();
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    auto store = [&](int m, int tq, float mx, float l, int half) {
        if (tq >= n_valid_tok) return;
        const size_t th = (row0 + tq) * p.n_head + hk * group + m % group;
        float* acc = p.part_acc + th * HD + (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) *(float2*)(acc + i * 8) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
        if ((lane & 3) == 0) { p.part_ml[th * 2] = mx; p.part_ml[th * 2 + 1] = l; }
    };
    store(m_lo, tq_lo, mx_lo, l_lo, 0);
    store(m_hi, tq_hi, mx_hi, l_hi, 1);
}
template <int HD>
constexpr size_t attn_mma_smem() { return (size_t)AM_ROWS * HD * 2 + 4 * (size_t)AM_KV * HD * 2; }

}  // namespace
