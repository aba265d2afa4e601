// Multi-token Q8_0 and NVFP4 matmuls on the int8 tensor-core path (mma.sync m16n8k32 / m16n8k16), exact:
// one MMA covers exactly one quantisation block (32 for Q8_0, 16 for an NVFP4 sub-block), its int32 result is
// scaled by (d_weight * d_activation) and added to an f32 accumulator in ascending block order -- the CPU
// path's chain (src/ops/naive.rs:691-734) to the bit, for every (token, row) at once. The reference reaches
// the same result the same way on its own hardware (kernels/mma_int8.cuh:264 there).
//
// Within a block the k order is free (an integer sum), so a thread takes 8 CONTIGUOUS bytes of a row for its
// two 4-byte fragment registers and the activation side uses the same mapping: all loads are 8 bytes wide.
#pragma once
#include "itb_gemv.cuh"

__device__ __forceinline__ void mma_s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
__device__ __forceinline__ void mma_s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0), "r"(0), "r"(0), "r"(0));
}

// Four E2M1 codes (low 16 bits of w) to four signed int8 of the doubled values (src/quant/mod.rs:265).
__device__ __forceinline__ uint32_t fp4x4_to_s8(uint32_t w) {
    const uint32_t P0 = 0x03020100u, P1 = 0x0c080604u, H = 0x80808080u;
    uint32_t pos = prmt_raw(P0, P1, w), neg = prmt_raw(P0, P1, w ^ 0x8888u);
    // per-byte pos - neg without a SIMD instruction: every magnitude is below 128, so (pos | 0x80) - neg never
    // borrows across bytes and flipping the top bit back leaves the two's-complement byte
    return ((pos | H) - neg) ^ H;
}

constexpr int MMA_TOK = 32;     // tokens per block tile (4 n-tiles of 8)
constexpr int MMA_ROWS = 128;   // rows per block tile (8 warps x 16)
__host__ __device__ __forceinline__ int mma_act_stride(int k) { return k + 32; }   // bytes; the pad keeps 8-byte LDS conflict-free

// Activation tile of up to 32 tokens into shared memory: int8 [32][k+32], scales [32][k/32].
__device__ __forceinline__ void mma_stage_act(const int8_t* xq, const float* xs, int k, int t0, int n_tok, int8_t* sq, float* ss) {
    const int nb = k / 32, stride = mma_act_stride(k);
    for (int i = threadIdx.x; i < MMA_TOK * (k / 16); i += blockDim.x) {
        int t = i / (k / 16), c = i % (k / 16);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t0 + t < n_tok) v = *(const uint4*)(xq + (size_t)(t0 + t) * k + c * 16);
        *(uint4*)(sq + (size_t)t * stride + c * 16) = v;
    }
    for (int i = threadIdx.x; i < MMA_TOK * nb; i += blockDim.x) {
        int t = i / nb;
        ss[i] = t0 + t < n_tok ? xs[(size_t)(t0 + t) * nb + i % nb] : 0.0f;
    }
    __syncthreads();
}

// One warp: 16 rows [r0, r0+16) of a Q8_0 matrix against NJ n-tiles (8 tokens each, first tile jb) of the staged
// 32-token tile. acc[j][0..3] follow the MMA C layout: rows g and g+8 (g = lane/4), tokens 8(jb+j)+2t and +1
// (t = lane%4). The loads of UNR k-blocks are issued before their MMAs so several are in flight per warp.
template <int NJ, int UNR>
__device__ __forceinline__ void mma_q8_rows16(const DevQ8& w, int r0, const int8_t* sq, const float* ss, int jb, float (&acc)[NJ][4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int k = w.n_in, nb = k / 32, stride = mma_act_stride(k);
    const int ra = min(r0 + g, w.n_out - 1), rb = min(r0 + g + 8, w.n_out - 1);
    const int8_t* pa = w.q + (size_t)ra * k + 8 * t;
    const int8_t* pb = w.q + (size_t)rb * k + 8 * t;
    const uint16_t* sa = w.s + (size_t)ra * nb;
    const uint16_t* sb = w.s + (size_t)rb * nb;
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;
    for (int b0 = 0; b0 < nb; b0 += UNR) {
        uint2 va[UNR], vb[UNR];
        uint16_t ha[UNR], hb[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int b = min(b0 + u, nb - 1);
            va[u] = __ldg((const uint2*)(pa + b * 32)); vb[u] = __ldg((const uint2*)(pb + b * 32));
            ha[u] = __ldg(sa + b); hb[u] = __ldg(sb + b);
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int b = b0 + u;
            if (b < nb) {
                const float dwa = f16_bits_to_f32(ha[u]), dwb = f16_bits_to_f32(hb[u]);
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const int tj = 8 * (jb + j);
                    const uint2 x = *(const uint2*)(sq + (size_t)(tj + g) * stride + b * 32 + 8 * t);
                    int c[4];
                    mma_s8_k32(c, va[u].x, vb[u].x, va[u].y, vb[u].y, x.x, x.y);
                    const float dx0 = ss[(tj + 2 * t) * nb + b], dx1 = ss[(tj + 2 * t + 1) * nb + b];
                    acc[j][0] += (float)c[0] * (dwa * dx0);
                    acc[j][1] += (float)c[1] * (dwa * dx1);
                    acc[j][2] += (float)c[2] * (dwb * dx0);
                    acc[j][3] += (float)c[3] * (dwb * dx1);
                }
            }
        }
    }
}

// As above for an NVFP4 matrix (nibbles [rows][k/2], UE4M3 scales [rows][k/16]): one k16 MMA per 16-element
// sub-block, term (dy*d)*(float)sum folded ascending (src/ops/naive.rs:714-734). dy is the Q8_0 scale of the
// 32-block the sub-block lies in.
template <int NJ, int UNR>
__device__ __forceinline__ void mma_fp4_rows16(const uint8_t* nib, const uint8_t* sc, int k, int n_rows, int r0, const int8_t* sq,
                                               const float* ss, int jb, float (&acc)[NJ][4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nsb = k / 16, nb = k / 32, stride = mma_act_stride(k);
    const int ra = min(r0 + g, n_rows - 1), rb = min(r0 + g + 8, n_rows - 1);
    const uint8_t* pa = nib + (size_t)ra * (k / 2) + 2 * t;   // 4 codes = 2 bytes per thread and sub-block
    const uint8_t* pb = nib + (size_t)rb * (k / 2) + 2 * t;
    const uint8_t* sa = sc + (size_t)ra * nsb;
    const uint8_t* sb = sc + (size_t)rb * nsb;
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;
    for (int s0 = 0; s0 < nsb; s0 += UNR) {
        uint16_t wa[UNR], wb[UNR];
        uint8_t ca[UNR], cb[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int s = min(s0 + u, nsb - 1);
            // elements 4t..4t+3 of the sub-block on both sides (any fixed bijection of k is fine)
            wa[u] = __ldg((const uint16_t*)(pa + s * 8)); wb[u] = __ldg((const uint16_t*)(pb + s * 8));
            ca[u] = __ldg(sa + s); cb[u] = __ldg(sb + s);
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int s = s0 + u;
            if (s < nsb) {
                const uint32_t a0 = fp4x4_to_s8(wa[u]), a1 = fp4x4_to_s8(wb[u]);
                const float da = ue4m3_half_dev(ca[u]), db = ue4m3_half_dev(cb[u]);
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const int tj = 8 * (jb + j);
                    const uint32_t x = *(const uint32_t*)(sq + (size_t)(tj + g) * stride + s * 16 + 4 * t);
                    int c[4];
                    mma_s8_k16(c, a0, a1, x);
                    const float dy0 = ss[(tj + 2 * t) * nb + (s >> 1)], dy1 = ss[(tj + 2 * t + 1) * nb + (s >> 1)];
                    acc[j][0] += dy0 * da * (float)c[0];
                    acc[j][1] += dy1 * da * (float)c[1];
                    acc[j][2] += dy0 * db * (float)c[2];
                    acc[j][3] += dy1 * db * (float)c[3];
                }
            }
        }
    }
}

// Visit the warp's results: f(token_in_tile, row, value).
template <int NJ, class F>
__device__ __forceinline__ void mma_foreach(const float (&acc)[NJ][4], int r0, int n_rows, int jb, F f) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int tj = 8 * (jb + j) + 2 * t;
        if (r0 + g < n_rows) { f(tj, r0 + g, acc[j][0]); f(tj + 1, r0 + g, acc[j][1]); }
        if (r0 + g + 8 < n_rows) { f(tj, r0 + g + 8, acc[j][2]); f(tj + 1, r0 + g + 8, acc[j][3]); }
    }
}
