// Pipelined multi-token matmuls: a block owns 64 weight rows x TOK tokens and walks k in chunks of KC elements
// through a ring of cp.async stages (weights, their scales, the Q8_0 activations and their scales all arrive by
// 16-byte asynchronous copies, several chunks in flight), so DRAM latency is paid once per block instead of once
// per k-block. The arithmetic is the exact chain of itb_mma.cuh: one int8 MMA per quantisation block, its int32
// sum scaled and added to an f32 accumulator in ascending block order (src/ops/naive.rs:691-734).
//
// 8 warps, split TH ways over the tile's tokens and 8/TH ways over its rows: TH=1 -> warp w owns rows 16*w.. and all
// 8*NJ tokens (128 rows: for the few rows an expert sees, every weight is decoded by exactly one warp); TH=2 -> 64 rows
// x 16*NJ tokens (wide token tiles); TH=4 -> 32 rows x 32*NJ tokens (batched decode of dense matrices: small blocks,
// so every SM gets several and their pipelines overlap). NJ = groups of 8 tokens per warp. Token rows
// are named by a per-tile index array so the same loop serves dense matmuls (consecutive rows) and grouped
// experts (rows gathered by an expert's pair list).
#pragma once
#include "itb_mma.cuh"

namespace {

constexpr int TILE_STAGES = 4;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;   // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

// KIND: MK_Q8 (int8 rows, f16 scale per 32) or MK_FP4 (E2M1 nibbles in element order, UE4M3 scale per 16).
template <int KIND, int NJ, int KC, int TH = 2>
struct TileCfg {
    static constexpr int ROWS = 128 / TH;
    static constexpr int TOK = 8 * NJ * TH;
    static constexpr int WB = KIND == MK_Q8 ? KC : KC / 2;            // weight bytes per row and chunk
    static constexpr int WSTR = WB + (KIND == MK_Q8 ? 32 : 16);       // padded row stride: fragment reads hit distinct banks
    static constexpr int SB = KIND == MK_Q8 ? KC / 32 * 2 : KC / 16;  // scale bytes per row and chunk
    static constexpr int XSTR = KC + (KIND == MK_Q8 ? 32 : 16);
    static constexpr int XSB = KC / 32 * 4;                           // activation scale bytes per token and chunk
    static constexpr int XSF = KC / 32 + 4;                           // padded scale row in floats (distinct banks for the 4 token pairs)
    static constexpr int OFF_WS = ROWS * WSTR;
    static constexpr int OFF_XQ = OFF_WS + ROWS * SB;
    static constexpr int OFF_XS = OFF_XQ + TOK * XSTR;
    static constexpr int STAGE = OFF_XS + TOK * XSF * 4;
    static_assert(WB % 16 == 0 && SB % 16 == 0 && XSB % 16 == 0 && STAGE % 16 == 0, "16-byte copies");
};
template <int KIND, int NJ, int KC, int TH = 2>
static inline size_t tile_smem(int k) {
    int n = k / KC; if (n > TILE_STAGES) n = TILE_STAGES; if (n < 1) n = 1;
    return (size_t)n * TileCfg<KIND, NJ, KC, TH>::STAGE + 64 * 4;
}

// One (ROWS-row, TOK-token) tile. wq/ws: the matrix's quants and scales (row-major, k elements per row); rows
// [r0, r0+ROWS) clamped to n_rows-1. tok_idx[TOK] (shared memory): activation row of each tile token or -1.
// Results in acc[NJ][4] in the MMA C layout for the warp's rows {g, g+8} and tokens 8*j + 2t, +1 of its token share.
template <int KIND, int NJ, int KC, int TH>
__device__ __forceinline__ void tile_gemm(const uint8_t* wq, const uint8_t* ws, int k, int n_rows, int r0, const int8_t* xq, const float* xs,
                                          const int* tok_idx, unsigned char* ring, int n_stage, float (&acc)[NJ][4]) {
    using C = TileCfg<KIND, NJ, KC, TH>;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, g = lane >> 2, t = lane & 3;
    const int n_chunk = k / KC, nb = k / 32;
    const size_t wrow = KIND == MK_Q8 ? (size_t)k : (size_t)k / 2, srow = KIND == MK_Q8 ? (size_t)nb * 2 : (size_t)k / 16;
    auto load = [&](int c) {
        unsigned char* st = ring + (size_t)(c % n_stage) * C::STAGE;
        constexpr int WP = C::WB / 16, SP = C::SB / 16, XP = KC / 16, XSP = C::XSB / 16;
        for (int i = tid; i < C::ROWS * WP; i += 256) {
            const int r = i / WP, p = i % WP, row = min(r0 + r, n_rows - 1);
            cp_async16(st + r * C::WSTR + p * 16, wq + (size_t)row * wrow + (size_t)c * C::WB + p * 16, true);
        }
        for (int i = tid; i < C::ROWS * SP; i += 256) {
            const int r = i / SP, p = i % SP, row = min(r0 + r, n_rows - 1);
            cp_async16(st + C::OFF_WS + r * C::SB + p * 16, ws + (size_t)row * srow + (size_t)c * C::SB + p * 16, true);
        }
        for (int i = tid; i < C::TOK * XP; i += 256) {
            const int tk = i / XP, p = i % XP, src = tok_idx[tk];
            cp_async16(st + C::OFF_XQ + tk * C::XSTR + p * 16, xq + (size_t)max(src, 0) * k + (size_t)c * KC + p * 16, src >= 0);
        }
        for (int i = tid; i < C::TOK * XSP; i += 256) {
            const int tk = i / XSP, p = i % XSP, src = tok_idx[tk];
            cp_async16(st + C::OFF_XS + tk * C::XSF * 4 + p * 16, (const unsigned char*)(xs + (size_t)max(src, 0) * nb) + (size_t)c * C::XSB + p * 16, src >= 0);
        }
    };
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;
    for (int c = 0; c < n_stage - 1; ++c) { if (c < n_chunk) load(c); cp_async_commit(); }
    constexpr int RG = 8 / TH;   // row groups of 16 among the 8 warps
    const int rw = (wid % RG) * 16, tb = (wid / RG) * NJ * 8;
    for (int c = 0; c < n_chunk; ++c) {
        if (n_stage == 1) { __syncthreads(); load(c); cp_async_commit(); }
        if (n_stage >= 4) cp_async_wait<2>(); else if (n_stage == 3) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();
        if (n_stage > 1) { if (c + n_stage - 1 < n_chunk) load(c + n_stage - 1); cp_async_commit(); }
        const unsigned char* st = ring + (size_t)(c % n_stage) * C::STAGE;
        const unsigned char* wa = st + (rw + g) * C::WSTR;
        const unsigned char* wb = wa + 8 * C::WSTR;
        const unsigned char* sa = st + C::OFF_WS + (rw + g) * C::SB;
        const unsigned char* sb = sa + 8 * C::SB;
        const unsigned char* xq_s = st + C::OFF_XQ;
        const float* xs_s = (const float*)(st + C::OFF_XS);
        if (KIND == MK_Q8) {
#pragma unroll 2
            for (int b = 0; b < KC / 32; ++b) {
                const uint2 va = *(const uint2*)(wa + b * 32 + 8 * t), vb = *(const uint2*)(wb + b * 32 + 8 * t);
                const float dwa = f16_bits_to_f32(*(const uint16_t*)(sa + 2 * b)), dwb = f16_bits_to_f32(*(const uint16_t*)(sb + 2 * b));
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const int tj = tb + 8 * j;
                    const uint2 x = *(const uint2*)(xq_s + (tj + g) * C::XSTR + b * 32 + 8 * t);
                    int cc[4];
                    mma_s8_k32(cc, va.x, vb.x, va.y, vb.y, x.x, x.y);
                    const float dx0 = xs_s[(tj + 2 * t) * C::XSF + b], dx1 = xs_s[(tj + 2 * t + 1) * C::XSF + b];
                    acc[j][0] += i2f_small(cc[0]) * (dwa * dx0);
                    acc[j][1] += i2f_small(cc[1]) * (dwa * dx1);
                    acc[j][2] += i2f_small(cc[2]) * (dwb * dx0);
                    acc[j][3] += i2f_small(cc[3]) * (dwb * dx1);
                }
            }
        } else {
#pragma unroll 2
            for (int s = 0; s < KC / 16; s += 2) {
                // the two sub-blocks of one 32-block; elements 4t..4t+3 of each on both sides (within a block the k order is free)
                const uint32_t a0 = fp4x4_to_s8(*(const uint16_t*)(wa + s * 8 + 2 * t)), a1 = fp4x4_to_s8(*(const uint16_t*)(wb + s * 8 + 2 * t));
                const uint32_t c0 = fp4x4_to_s8(*(const uint16_t*)(wa + s * 8 + 8 + 2 * t)), c1 = fp4x4_to_s8(*(const uint16_t*)(wb + s * 8 + 8 + 2 * t));
                float da0, da1, db0, db1;
                ue4m3x2_half(*(const uint16_t*)(sa + s), da0, da1);
                ue4m3x2_half(*(const uint16_t*)(sb + s), db0, db1);
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const int tj = tb + 8 * j;
                    const uint32_t x0 = *(const uint32_t*)(xq_s + (tj + g) * C::XSTR + s * 16 + 4 * t);
                    const uint32_t x1 = *(const uint32_t*)(xq_s + (tj + g) * C::XSTR + s * 16 + 16 + 4 * t);
                    int cc[4], dd[4];
                    mma_s8_k16(cc, a0, a1, x0);
                    mma_s8_k16(dd, c0, c1, x1);
                    const float dy0 = xs_s[(tj + 2 * t) * C::XSF + (s >> 1)], dy1 = xs_s[(tj + 2 * t + 1) * C::XSF + (s >> 1)];
                    acc[j][0] += dy0 * da0 * i2f_small(cc[0]);
                    acc[j][1] += dy1 * da0 * i2f_small(cc[1]);
                    acc[j][2] += dy0 * db0 * i2f_small(cc[2]);
                    acc[j][3] += dy1 * db0 * i2f_small(cc[3]);
                    acc[j][0] += dy0 * da1 * i2f_small(dd[0]);
                    acc[j][1] += dy1 * da1 * i2f_small(dd[1]);
                    acc[j][2] += dy0 * db1 * i2f_small(dd[2]);
                    acc[j][3] += dy1 * db1 * i2f_small(dd[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();   // the ring may be refilled by the caller's next tile
}

// Visit this warp's results: f(token_in_tile, row, value).
template <int NJ, int TH, class F>
__device__ __forceinline__ void tile_foreach(const float (&acc)[NJ][4], int r0, int n_rows, F f) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    constexpr int RG = 8 / TH;
    const int ra = r0 + (wid % RG) * 16 + g, rb = ra + 8, tb = (wid / RG) * NJ * 8;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int tj = tb + 8 * j + 2 * t;
        if (ra < n_rows) { f(tj, ra, acc[j][0]); f(tj + 1, ra, acc[j][1]); }
        if (rb < n_rows) { f(tj, rb, acc[j][2]); f(tj + 1, rb, acc[j][3]); }
    }
}

// Dense Q8_0 matmul: grid (ceil(rows/ROWS), ceil(n_tok/TOK)). mode 0: out = v; mode 1: out += v.
template <int NJ, int KC, int TH>
__global__ void __launch_bounds__(256) k_tile_q8(DevQ8 w, const int8_t* xq, const float* xs, int n_tok, float* out, size_t out_stride, int mode, int n_stage) {
    extern __shared__ __align__(16) unsigned char smem[];
    using C = TileCfg<MK_Q8, NJ, KC, TH>;
    int* tok_idx = (int*)smem;
    const int t0 = blockIdx.y * C::TOK, r0 = blockIdx.x * C::ROWS;
    if ((int)threadIdx.x < C::TOK) { const int ti = t0 + (int)threadIdx.x; tok_idx[threadIdx.x] = ti < n_tok ? ti : -1; }
    __syncthreads();
    float acc[NJ][4];
    tile_gemm<MK_Q8, NJ, KC, TH>((const uint8_t*)w.q, (const uint8_t*)w.s, w.n_in, w.n_out, r0, xq, xs, tok_idx, smem + 256, n_stage, acc);
    tile_foreach<NJ, TH>(acc, r0, w.n_out, [&](int t, int row, float v) {
        if (t0 + t < n_tok) { float* o = out + (size_t)(t0 + t) * out_stride + row; *o = mode ? *o + v : v; }
    });
}

// Up to three dense Q8_0 matrices over the same quantised rows in one launch (the input projections of a layer; the shared
// expert's gate and up): grid.x runs over the matrices' row tiles one after the other. A matrix of 512 rows alone is 16 blocks.
struct Q8Multi { DevQ8 w[3]; float* out[3]; size_t stride[3]; int tiles[3]; int n; };
template <int NJ, int KC, int TH>
__global__ void __launch_bounds__(256) k_tile_q8_multi(Q8Multi p, const int8_t* xq, const float* xs, int n_tok, int n_stage) {
    extern __shared__ __align__(16) unsigned char smem[];
    using C = TileCfg<MK_Q8, NJ, KC, TH>;
    int* tok_idx = (int*)smem;
    int m = 0, bx = blockIdx.x;
    while (m + 1 < p.n && bx >= p.tiles[m]) { bx -= p.tiles[m]; ++m; }
    const DevQ8 w = p.w[m];
    float* out = p.out[m];
    const size_t out_stride = p.stride[m];
    const int t0 = blockIdx.y * C::TOK, r0 = bx * C::ROWS;
    if ((int)threadIdx.x < C::TOK) { const int ti = t0 + (int)threadIdx.x; tok_idx[threadIdx.x] = ti < n_tok ? ti : -1; }
    __syncthreads();
    float acc[NJ][4];
    tile_gemm<MK_Q8, NJ, KC, TH>((const uint8_t*)w.q, (const uint8_t*)w.s, w.n_in, w.n_out, r0, xq, xs, tok_idx, smem + 256, n_stage, acc);
    tile_foreach<NJ, TH>(acc, r0, w.n_out, [&](int t, int row, float v) {
        if (t0 + t < n_tok) out[(size_t)(t0 + t) * out_stride + row] = v;
    });
}

// Gate and up of one expert for the pairs routed to it, SiLU-gated (src/ops/mod.rs:1105-1117):
// h[pair][row] = silu(gate.x * s_gate) * (up.x * s_up). grid (n_expert, ceil(ff/ROWS)); pair p reads activation row p / n_used.
template <int NJ, int KC, int TH>
__global__ void __launch_bounds__(256) k_tile_glu(DevFp4 gate, DevFp4 up, const int8_t* xq, const float* xs, int n_used, const int* off, const int* list,
                                                  float* h, int n_stage) {
    extern __shared__ __align__(16) unsigned char smem[];
    using C = TileCfg<MK_FP4, NJ, KC, TH>;
    int* tok_idx = (int*)smem;
    const int e = blockIdx.x, k = gate.n_in, ff = gate.n_out;
    const int p0 = off[e], p1 = off[e + 1];
    if (p0 >= p1) return;
    const int el = fp4_slot(gate, e);
    if (el < 0) return;
    const int r0 = blockIdx.y * C::ROWS;
    const size_t eo = (size_t)el * ff;
    const bool has_g = gate.scale2 != nullptr, has_u = up.scale2 != nullptr;
    const float sg2 = has_g ? gate.scale2[el] : 1.0f, su2 = has_u ? up.scale2[el] : 1.0f;
    for (int t0 = p0; t0 < p1; t0 += C::TOK) {
        __syncthreads();
        if ((int)threadIdx.x < C::TOK) { const int ti = t0 + (int)threadIdx.x; tok_idx[threadIdx.x] = ti < p1 ? list[ti] / n_used : -1; }
        __syncthreads();
        float g[NJ][4], u[NJ][4];
        tile_gemm<MK_FP4, NJ, KC, TH>(gate.nib + eo * (k / 2), gate.sc + eo * (k / 16), k, ff, r0, xq, xs, tok_idx, smem + 256, n_stage, g);
        tile_gemm<MK_FP4, NJ, KC, TH>(up.nib + eo * (k / 2), up.sc + eo * (k / 16), k, ff, r0, xq, xs, tok_idx, smem + 256, n_stage, u);
#pragma unroll
        for (int j = 0; j < NJ; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float gv = has_g ? g[j][i] * sg2 : g[j][i], uv = has_u ? u[j][i] * su2 : u[j][i]; g[j][i] = silu_f(gv) * uv; }
        tile_foreach<NJ, TH>(g, r0, ff, [&](int t, int row, float v) {
            if (t0 + t < p1) h[(size_t)list[t0 + t] * ff + row] = v;
        });
    }
}

// Down projection of one expert for its pairs (src/ops/mod.rs:1049-1088): o[pair][row], times the expert's second
// scale. grid (n_expert, ceil(n_out/ROWS)); pair p reads activation row p / div (1: a row per pair; n_used: a row per
// token; larger than the pair count: one row for all).
template <int NJ, int KC, int TH>
__global__ void __launch_bounds__(256) k_tile_down(DevFp4 down, const int8_t* hq, const float* hs, const int* off, const int* list, float* o, int n_stage,
                                                   int div = 1) {
    extern __shared__ __align__(16) unsigned char smem[];
    using C = TileCfg<MK_FP4, NJ, KC, TH>;
    int* tok_idx = (int*)smem;
    const int e = blockIdx.x, k = down.n_in, n_out = down.n_out;
    const int p0 = off[e], p1 = off[e + 1];
    if (p0 >= p1) return;
    const int el = fp4_slot(down, e);
    if (el < 0) return;
    const int r0 = blockIdx.y * C::ROWS;
    const size_t eo = (size_t)el * n_out;
    const bool has_s = down.scale2 != nullptr;
    const float s2 = has_s ? down.scale2[el] : 1.0f;
    for (int t0 = p0; t0 < p1; t0 += C::TOK) {
        __syncthreads();
        if ((int)threadIdx.x < C::TOK) { const int ti = t0 + (int)threadIdx.x; tok_idx[threadIdx.x] = ti < p1 ? list[ti] / div : -1; }
        __syncthreads();
        float acc[NJ][4];
        tile_gemm<MK_FP4, NJ, KC, TH>(down.nib + eo * (k / 2), down.sc + eo * (k / 16), k, n_out, r0, hq, hs, tok_idx, smem + 256, n_stage, acc);
        tile_foreach<NJ, TH>(acc, r0, n_out, [&](int t, int row, float v) {
            if (t0 + t < p1) o[(size_t)list[t0 + t] * n_out + row] = has_s ? v * s2 : v;
        });
    }
}

}  // namespace
