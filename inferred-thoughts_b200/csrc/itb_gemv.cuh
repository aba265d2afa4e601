// Row-streaming GEMV cores for decode: HBM-bound, 16-byte coalesced weight loads, integer dot per
// quantisation block, and an order-preserving f32 fold so every output equals the CPU path's
// `sumf += term_b` chain to the bit (src/ops/naive.rs:691-734).
//
// Shape of the code: small loop bodies and many warps. A decode GEMV touches every instruction once per
// row, so straight-line unrolled kernels spend their time fetching instructions; here a warp loops over
// its rows RP at a time with all loads of a trip issued before the first dot.
//
// Work split inside a warp: G lanes share a row (G = power of two dividing the row's unit count),
// 32/G rows run side by side, RP such groups per pass. Each lane owns fixed K-columns, computes the
// integer sums of its 32-element units, turns them into f32 terms in shared memory; then one lane per row
// folds that row's terms in ascending order.
#pragma once
#include "itb_internal.cuh"

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// ---- activation prologues ------------------------------------------------------------------------
// RMSNorm of one row into shared memory: f32 squares, f64 accumulation (tree), (x*scale)*w
// (src/ops/naive.rs:139-152, :633-640). `red` holds blockDim.x/32 doubles.
// With xq/xs given, the vector path also quantises the normalised row to Q8_0 in the same pass (8 consecutive lanes hold
// one 32-block; src/ops/naive.rs:653-675) and returns true; otherwise the caller quantises from xn.
__device__ __forceinline__ bool block_rms_norm(const float* __restrict__ x, const float* __restrict__ w, int n, float eps,
                                               float* xn, double* red, int8_t* xq = nullptr, float* xs = nullptr) {
    const int wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if ((n & 3) == 0 && n <= 16 * (int)blockDim.x && ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)xn)) & 15) == 0) {
        // the row and the norm weights as float4, every load in flight before the first use: one memory round trip
        float4 xv[4], wv[4];
        const int nv = n >> 2;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < nv) { xv[j] = ((const float4*)x)[i]; wv[j] = __ldg((const float4*)w + i); }
        }
        double acc = 0.0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if ((int)(threadIdx.x + j * blockDim.x) < nv)
                acc += (double)(xv[j].x * xv[j].x) + (double)(xv[j].y * xv[j].y) + (double)(xv[j].z * xv[j].z) + (double)(xv[j].w * xv[j].w);
        acc = warp_sum_d(acc);
        if ((threadIdx.x & 31) == 0) red[wid] = acc;
        __syncthreads();
        // the warps' partial sums in warp order, by one lane per warp (the f64 unit is slow: every thread adding all of them
        // was most of this prologue), handed to the others by shuffle
        double tot = 0.0;
        if ((threadIdx.x & 31) == 0) for (int i = 0; i < nw; ++i) tot += red[i];
        tot = __shfl_sync(0xffffffffu, tot, 0);
        const float mean = (float)(tot / (double)n);
        const float sc = 1.0f / sqrtf(mean + eps);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < nv) { o = make_float4(xv[j].x * sc * wv[j].x, xv[j].y * sc * wv[j].y, xv[j].z * sc * wv[j].z, xv[j].w * sc * wv[j].w); ((float4*)xn)[i] = o; }
            if (xq && (int)(j * blockDim.x) < nv) {      // whole warps take this branch together: nv and blockDim are multiples of 8 and 32
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
        __syncthreads();
        return xq != nullptr;
    }
    double acc = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { float v = x[i]; xn[i] = v; acc += (double)(v * v); }
    acc = warp_sum_d(acc);
    if ((threadIdx.x & 31) == 0) red[wid] = acc;
    __syncthreads();
    double tot = 0.0;
    if ((threadIdx.x & 31) == 0) for (int i = 0; i < nw; ++i) tot += red[i];
    tot = __shfl_sync(0xffffffffu, tot, 0);
    float mean = (float)(tot / (double)n);
    float sc = 1.0f / sqrtf(mean + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) xn[i] = xn[i] * sc * w[i];
    __syncthreads();
    return false;
}

// One Q8_0 block of 32 values held one per lane (src/ops/naive.rs:653-675): d = amax/127 through f16,
// q = roundf(v * (1/d)). Returns the lane's quant; *d_out (all lanes) the f16-rounded scale.
__device__ __forceinline__ int8_t warp_quant_q8(float v, float* d_out) {
    float amax = warp_max(fabsf(v));
    float d = amax / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    float r = roundf(v * id);
    *d_out = __half2float(__float2half_rn(d));
    return (int8_t)fminf(127.0f, fmaxf(-128.0f, r));
}
// Q8_0 activation quantiser over a row in shared or global memory: one warp per 32-block.
__device__ __forceinline__ void block_quant_q8(const float* xn, int n, int8_t* xq, float* xs) {
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b = wid; b < n / 32; b += nw) {
        float d;
        xq[b * 32 + lane] = warp_quant_q8(xn[b * 32 + lane], &d);
        if (lane == 0) xs[b] = d;
    }
    __syncthreads();
}

// log2 of the lanes sharing a row: the largest power of two (<= 32) dividing the row's unit count.
__host__ __device__ __forceinline__ int lanes_shift(int units) {
    int sh = 0;
    while (sh < 5 && units % (2 << sh) == 0) sh++;
    return sh;
}
// shared-memory floats one warp needs for its term matrix
__host__ __device__ __forceinline__ int terms_floats(int rp, int gsh, int n_terms) { return rp * (32 >> gsh) * (n_terms + 1); }

// E2M1 codes to doubled integer magnitudes {0,1,2,3,4,6,8,12} (src/quant/mod.rs:265) with one byte
// permute per four codes: the selector's bit 3 asks for the sign of the selected (positive) byte, i.e. 0,
// so `prmt(pool, w)` yields the magnitudes of the positive codes and zeros elsewhere, and the same on
// `w ^ 0x8888` yields the magnitudes of the negative codes.
// (The __byte_perm intrinsic masks bit 3 of each selector, so the PTX instruction is issued directly.)
__device__ __forceinline__ uint32_t prmt_raw(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ int fp4_dot8(uint32_t w, uint32_t a0, uint32_t a1) {
    const uint32_t P0 = 0x03020100u, P1 = 0x0c080604u;
    uint32_t n = w ^ 0x88888888u;
    int pos = __dp4a((int)prmt_raw(P0, P1, w), (int)a0, 0);
    pos = __dp4a((int)prmt_raw(P0, P1, w >> 16), (int)a1, pos);
    int neg = __dp4a((int)prmt_raw(P0, P1, n), (int)a0, 0);
    neg = __dp4a((int)prmt_raw(P0, P1, n >> 16), (int)a1, neg);
    return pos - neg;
}

// Matrix kinds the row cores understand. Plane A: Q8_0 int8 quants (n_in bytes per row) or NVFP4 nibbles
// (n_in/2); plane B: f16 scales per 32 (n_in/16 bytes per row) or UE4M3 codes per 16 (n_in/16).
enum { MK_Q8 = 0, MK_FP4 = 1 };
template <int KIND> __host__ __device__ __forceinline__ int plane_a_bytes(int n_in) { return KIND == MK_Q8 ? n_in : n_in / 2; }
__host__ __device__ __forceinline__ int plane_b_bytes(int n_in) { return n_in / 16; }
// f32 terms per row: one per Q8_0 block of 32, or one per NVFP4 sub-block of 16.
template <int KIND> __host__ __device__ __forceinline__ int row_terms(int n_in) { return KIND == MK_Q8 ? n_in / 32 : n_in / 16; }

// One lane's 32-element unit of one row: 32 bytes (Q8_0) or 16 bytes (NVFP4) of weights plus the 2 scale bytes.
struct UnitW { uint4 a, b; uint32_t s; };
template <int KIND>
__device__ __forceinline__ void unit_load(UnitW& w, const uint8_t* pa, const uint8_t* pb, int u) {
    if (KIND == MK_Q8) { w.a = ld_stream16(pa + u * 32); w.b = ld_stream16(pa + u * 32 + 16); }
    else w.a = ld_stream16(pa + u * 16);
    w.s = __ldg((const uint16_t*)(pb + u * 2));
}
// The unit's f32 term(s) into t (row's term array), against the activation unit xa|xb with scale dx.
template <int KIND>
__device__ __forceinline__ void unit_terms(const UnitW& w, const uint4& xa, const uint4& xb, float dx, float* t, int u) {
    if (KIND == MK_Q8) {
        int s = 0;
        s = __dp4a((int)w.a.x, (int)xa.x, s); s = __dp4a((int)w.a.y, (int)xa.y, s);
        s = __dp4a((int)w.a.z, (int)xa.z, s); s = __dp4a((int)w.a.w, (int)xa.w, s);
        s = __dp4a((int)w.b.x, (int)xb.x, s); s = __dp4a((int)w.b.y, (int)xb.y, s);
        s = __dp4a((int)w.b.z, (int)xb.z, s); s = __dp4a((int)w.b.w, (int)xb.w, s);
        t[u] = i2f_small(s) * (f16_bits_to_f32((uint16_t)w.s) * dx);           // src/ops/naive.rs:701
    } else {
        int s0 = fp4_dot8(w.a.x, xa.x, xa.y) + fp4_dot8(w.a.y, xa.z, xa.w);
        int s1 = fp4_dot8(w.a.z, xb.x, xb.y) + fp4_dot8(w.a.w, xb.z, xb.w);
        float d0, d1;
        ue4m3x2_half(w.s, d0, d1);
        t[2 * u] = dx * d0 * i2f_small(s0);                                    // src/ops/naive.rs:730
        t[2 * u + 1] = dx * d1 * i2f_small(s1);
    }
}
// Ascending fold of one row's terms.
__device__ __forceinline__ float fold_terms(const float* t, int nt) {
    float sum = 0.0f;
#pragma unroll 16
    for (int b = 0; b < nt; ++b) sum += t[b];   // a deep unroll keeps the loads ahead of the dependent adds
    return sum;
}

// Rows [r0, r1) of one matrix (planes pa/pb, row 0 first) against one quantised activation (xq, xs in shared
// memory). terms: warp-private shared scratch of terms_floats(RP, gsh, row_terms) floats. epi(row, value) is
// called by one lane per row. UB units per lane and trip are loaded before the first dot.
template <int KIND, int RP, int UB, class Epi>
__device__ __forceinline__ void rows_direct_ub(const uint8_t* __restrict__ pa, const uint8_t* __restrict__ pb, int n_in, int r0, int r1,
                                            const int8_t* xq, const float* xs, float* terms, int gsh, Epi epi) {
    const int G = 1 << gsh, lane = threadIdx.x & 31, sub = lane & (G - 1), slot = lane >> gsh;
    const int SLOTS = 32 >> gsh, ROWS = RP * SLOTS;
    const int nunits = n_in >> 5, nt = row_terms<KIND>(n_in), stride = nt + 1;
    const int arb = plane_a_bytes<KIND>(n_in), brb = plane_b_bytes(n_in);
#pragma unroll 1
    for (int r = r0; r < r1; r += ROWS) {
#pragma unroll 1
        for (int u0 = sub; u0 < nunits; u0 += UB * G) {
            UnitW w[UB][RP];
#pragma unroll
            for (int i = 0; i < RP; ++i) {
                int row = r + i * SLOTS + slot;
                if (row < r1) {
#pragma unroll
                    for (int h = 0; h < UB; ++h)
                        if (u0 + h * G < nunits) unit_load<KIND>(w[h][i], pa + (size_t)row * arb, pb + (size_t)row * brb, u0 + h * G);
                }
            }
#pragma unroll
            for (int h = 0; h < UB; ++h) {
                if (u0 + h * G < nunits) {
                    const int u = u0 + h * G;
                    const uint4 xa = *(const uint4*)(xq + u * 32), xb = *(const uint4*)(xq + u * 32 + 16);
                    const float dx = xs[u];
#pragma unroll
                    for (int i = 0; i < RP; ++i)
                        if (r + i * SLOTS + slot < r1) unit_terms<KIND>(w[h][i], xa, xb, dx, terms + (i * SLOTS + slot) * stride, u);
                }
            }
        }
        __syncwarp();
        if (lane < ROWS && r + lane < r1) epi(r + lane, fold_terms(terms + lane * stride, nt));
        __syncwarp();
    }
}

// A list of independent row-dots, each with its own weight row and its own activation: item k of [0, n) is
// described by src(k, pa, pb, xq, xs) (weight planes of THE ROW, activation in shared memory). One pass
// takes RP*(32/G) items with every load issued before the first dot; epi(k, value) by one lane per item.
template <int KIND, int RP, int UB = 1, class Src, class Epi>
__device__ __forceinline__ void rows_list(int n, int n_in, float* terms, int gsh, Src src, Epi epi) {
    const int G = 1 << gsh, lane = threadIdx.x & 31, sub = lane & (G - 1), slot = lane >> gsh;
    const int SLOTS = 32 >> gsh, ROWS = RP * SLOTS;
    const int nunits = n_in >> 5, nt = row_terms<KIND>(n_in), stride = nt + 1;
#pragma unroll 1
    for (int k0 = 0; k0 < n; k0 += ROWS) {
        const uint8_t *pa[RP], *pb[RP];
        const int8_t* xq[RP];
        const float* xs[RP];
#pragma unroll
        for (int i = 0; i < RP; ++i) {
            int k = k0 + i * SLOTS + slot;
            if (k < n) src(k, pa[i], pb[i], xq[i], xs[i]);
        }
#pragma unroll 1
        for (int u0 = sub; u0 < nunits; u0 += UB * G) {
            UnitW w[UB][RP];
#pragma unroll
            for (int h = 0; h < UB; ++h)
#pragma unroll
                for (int i = 0; i < RP; ++i)
                    if (k0 + i * SLOTS + slot < n && u0 + h * G < nunits) unit_load<KIND>(w[h][i], pa[i], pb[i], u0 + h * G);
#pragma unroll
            for (int h = 0; h < UB; ++h)
#pragma unroll
                for (int i = 0; i < RP; ++i)
                    if (k0 + i * SLOTS + slot < n && u0 + h * G < nunits) {
                        const int u = u0 + h * G;
                        const uint4 xa = *(const uint4*)(xq[i] + u * 32), xb = *(const uint4*)(xq[i] + u * 32 + 16);
                        unit_terms<KIND>(w[h][i], xa, xb, xs[i][u], terms + (i * SLOTS + slot) * stride, u);
                    }
        }
        __syncwarp();
        if (lane < ROWS && k0 + lane < n) epi(k0 + lane, fold_terms(terms + lane * stride, nt));
        __syncwarp();
    }
}

// As rows_direct_ub, but the terms of up to `br` rows are collected first and then folded by `br` lanes at
// once: the fold is a serial chain per row, so folding one or two rows at a time leaves most lanes idle and
// costs as many instructions as the dots themselves. terms: br * (row_terms + 1) floats, warp-private.
template <int KIND, int RP, int UB, class Epi>
__device__ __forceinline__ void rows_batched(const uint8_t* __restrict__ pa, const uint8_t* __restrict__ pb, int n_in, int r0, int r1,
                                             const int8_t* xq, const float* xs, float* terms, int br, int gsh, Epi epi) {
    const int G = 1 << gsh, lane = threadIdx.x & 31, sub = lane & (G - 1), slot = lane >> gsh;
    const int SLOTS = 32 >> gsh, ROWS = RP * SLOTS;
    const int nunits = n_in >> 5, nt = row_terms<KIND>(n_in), stride = nt + 1;
    const int arb = plane_a_bytes<KIND>(n_in), brb = plane_b_bytes(n_in);
    br = min(br, 32) / ROWS * ROWS;   // whole passes per batch (the caller sizes terms for at least one pass)
#pragma unroll 1
    for (int rb = r0; rb < r1; rb += br) {
        const int rend = min(r1, rb + br);
#pragma unroll 1
        for (int r = rb; r < rend; r += ROWS) {
#pragma unroll 1
            for (int u0 = sub; u0 < nunits; u0 += UB * G) {
                UnitW w[UB][RP];
#pragma unroll
                for (int i = 0; i < RP; ++i) {
                    const int row = r + i * SLOTS + slot;
                    if (row < rend) {
#pragma unroll
                        for (int h = 0; h < UB; ++h)
                            if (u0 + h * G < nunits) unit_load<KIND>(w[h][i], pa + (size_t)row * arb, pb + (size_t)row * brb, u0 + h * G);
                    }
                }
#pragma unroll
                for (int h = 0; h < UB; ++h) {
                    if (u0 + h * G < nunits) {
                        const int u = u0 + h * G;
                        const uint4 xa = *(const uint4*)(xq + u * 32), xb = *(const uint4*)(xq + u * 32 + 16);
                        const float dx = xs[u];
#pragma unroll
                        for (int i = 0; i < RP; ++i) {
                            const int row = r + i * SLOTS + slot;
                            if (row < rend) unit_terms<KIND>(w[h][i], xa, xb, dx, terms + (row - rb) * stride, u);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (rb + lane < rend) epi(rb + lane, fold_terms(terms + lane * stride, nt));
        __syncwarp();
    }
}

template <int KIND, int RP, class Epi>
__device__ __forceinline__ void rows_direct(const uint8_t* __restrict__ pa, const uint8_t* __restrict__ pb, int n_in, int r0, int r1,
                                            const int8_t* xq, const float* xs, float* terms, int gsh, Epi epi) {
    rows_direct_ub<KIND, RP, 2>(pa, pb, n_in, r0, r1, xq, xs, terms, gsh, epi);
}
template <int RP, class Epi>
__device__ __forceinline__ void q8_rows(const DevQ8& w, int r0, int r1, const int8_t* xq, const float* xs, float* terms, int gsh, Epi epi) {
    rows_direct<MK_Q8, RP>((const uint8_t*)w.q, (const uint8_t*)w.s, w.n_in, r0, r1, xq, xs, terms, gsh, epi);
}
template <int RP, class Epi>
__device__ __forceinline__ void fp4_rows(const uint8_t* nib, const uint8_t* sc, int n_in, int r0, int r1, const int8_t* xq,
                                         const float* xs, float* terms, int gsh, Epi epi) {
    rows_direct<MK_FP4, RP>(nib, sc, n_in, r0, r1, xq, xs, terms, gsh, epi);
}

// ---- F32 rows --------------------------------------------------------------------------------------
// EXACT: serial-k left fold per output like the CPU path (src/ops/naive.rs:845-849). A warp takes one row at a time: the lanes
// fetch the weights (coalesced) and put the products w[k] * x[k] of a tile of the row into the warp's shared scratch, then
// lane 0 adds the tile's terms in k order -- the adds are the only dependent chain (n_in of them, about 4 cycles each);
// chains of different warps overlap. `tile`: warp-private scratch of `tile_floats` floats (at least 128).
// Otherwise: lane-strided partial sums and a shuffle tree (order differs, value within rounding); `tile` unused.
template <bool EXACT, class Epi>
__device__ __forceinline__ void f32_rows(const float* __restrict__ w, int n_in, int r0, int r1, const float* x, float* tile, Epi epi, int tile_floats = 1024) {
    const int lane = threadIdx.x & 31;
    if (EXACT) {
        float* t16 = tile + ((4 - (int)(((uintptr_t)tile >> 2) & 3)) & 3);     // 16-byte aligned view of the scratch (still an offset from `tile`: shared-memory loads stay shared-memory loads)
        const int T = max(128, (tile_floats - 4) / 128 * 128);
#pragma unroll 1
        for (int r = r0; r < r1; ++r) {
            const float* p = w + (size_t)r * n_in;
            float sum = 0.0f;
#pragma unroll 1
            for (int t0 = 0; t0 < n_in; t0 += T) {
                const int tn = min(T, n_in - t0);
#pragma unroll 4
                for (int k = lane * 4; k < tn; k += 128) {
                    if (k + 4 <= tn) {
                        const float4 wv = __ldg((const float4*)(p + t0 + k)), xv = *(const float4*)(x + t0 + k);
                        *(float4*)(t16 + k) = make_float4(wv.x * xv.x, wv.y * xv.y, wv.z * xv.z, wv.w * xv.w);
                    } else {
                        for (int j = k; j < tn; ++j) t16[j] = __ldg(p + t0 + j) * x[t0 + j];
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    // the chain: 16 terms are in registers while the next 16 are on their way from shared memory
                    int k = 0;
                    if (tn >= 32) {
                        float4 a0 = *(const float4*)(t16), a1 = *(const float4*)(t16 + 4), a2 = *(const float4*)(t16 + 8), a3 = *(const float4*)(t16 + 12);
#pragma unroll 1
                        for (; k + 32 <= tn; k += 16) {
                            const float4 b0 = *(const float4*)(t16 + k + 16), b1 = *(const float4*)(t16 + k + 20), b2 = *(const float4*)(t16 + k + 24), b3 = *(const float4*)(t16 + k + 28);
                            sum += a0.x; sum += a0.y; sum += a0.z; sum += a0.w; sum += a1.x; sum += a1.y; sum += a1.z; sum += a1.w;
                            sum += a2.x; sum += a2.y; sum += a2.z; sum += a2.w; sum += a3.x; sum += a3.y; sum += a3.z; sum += a3.w;
                            a0 = b0; a1 = b1; a2 = b2; a3 = b3;
                        }
                        sum += a0.x; sum += a0.y; sum += a0.z; sum += a0.w; sum += a1.x; sum += a1.y; sum += a1.z; sum += a1.w;
                        sum += a2.x; sum += a2.y; sum += a2.z; sum += a2.w; sum += a3.x; sum += a3.y; sum += a3.z; sum += a3.w;
                        k += 16;
                    }
                    for (; k < tn; ++k) sum += t16[k];
                }
                __syncwarp();
            }
            if (lane == 0) epi(r, sum);
        }
    } else {
#pragma unroll 1
        for (int r = r0; r < r1; ++r) {
            const float* p = w + (size_t)r * n_in;
            float s = 0.0f;
#pragma unroll 1
            for (int k0 = lane * 4; k0 < n_in; k0 += 128 * 8) {
                float4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) if (k0 + 128 * j < n_in) v[j] = __ldg((const float4*)(p + k0 + 128 * j));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int k = k0 + 128 * j;
                    if (k < n_in) s += v[j].x * x[k] + v[j].y * x[k + 1] + v[j].z * x[k + 2] + v[j].w * x[k + 3];
                }
            }
            s = warp_sum(s);
            if (lane == 0) epi(r, s);
        }
    }
}

// Serial-k F32 rows, 32 rows per warp: lane = row, every lane folds ITS row in k order (product and sum rounded separately,
// src/ops/naive.rs:49-56), so 32 chains run side by side at one add latency per k for all of them. The unit's weights come
// from the k-major copy (DevF32::wt): a stage of 256 k is 32 KB in one piece, fetched by ONE bulk asynchronous copy that
// signals the stage's `full` mbarrier; in shared memory lane r reads word k * 32 + r, no conflicts. The copies are issued
// by ANOTHER warp (f32_unit_feed): the folding warp does nothing but wait for a stage, fold it and hand the slot back
// (`empty` mbarrier), so the chain of adds is the only thing on its critical path. Four stages keep enough bytes in flight
// for one warp to stream at the pace of the chain. Waits are bounded: one that runs out stores `F32S_FAIL` in *err and the
// fold goes on over whatever the slot holds (the host reads *err after the step). n_in a multiple of 256.
constexpr int F32S_K = 256, F32S_STAGES = 4, F32S_STAGE_FLOATS = 32 * F32S_K, F32S_FLOATS = F32S_STAGES * F32S_STAGE_FLOATS;
constexpr int F32S_FAIL = 0x7001;
__device__ __forceinline__ bool f32s_wait(unsigned long long* bar, uint32_t parity, int* err) {
    const uint32_t b = (uint32_t)__cvta_generic_to_shared(bar);
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(ok) : "r"(b), "r"(parity) : "memory");
        if (ok) return true;
        if (clock64() - t0 > 2000000000ll) { if (err) atomicExch(err, F32S_FAIL); return false; }
    }
}
// One lane of the feeding warp: stage t of the unit into slot t % stages; first = the stages issued before anything was folded
// (no slot to wait for), then one stage per slot the folding warp hands back.
__device__ __forceinline__ void f32_unit_issue(const float* wt_unit, int t, float* ring, unsigned long long* full) {
    const int slot = t % F32S_STAGES;
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(full + slot);
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(ring + slot * F32S_STAGE_FLOATS);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)(F32S_STAGE_FLOATS * 4)) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(wt_unit + (size_t)t * F32S_STAGE_FLOATS), "r"((uint32_t)(F32S_STAGE_FLOATS * 4)), "r"(bar) : "memory");
}
__device__ __forceinline__ void f32_unit_feed(const float* wt_unit, int n_in, float* ring, unsigned long long* full, unsigned long long* empty, int* err) {
    const int nst = n_in / F32S_K;
    for (int t = F32S_STAGES; t < nst; ++t) {
        if (!f32s_wait(empty + t % F32S_STAGES, (uint32_t)(t / F32S_STAGES - 1) & 1u, err)) return;
        f32_unit_issue(wt_unit, t, ring, full);
    }
}
template <class Epi>
__device__ __forceinline__ void f32_rows32_serial(int n_in, int r0, int nr, const float* x, const float* ring, unsigned long long* full,
                                                  unsigned long long* empty, int* err, Epi epi) {
    const int lane = threadIdx.x & 31, nst = n_in / F32S_K;
    float sum = 0.0f;
#pragma unroll 1
    for (int t = 0; t < nst; ++t) {
        const int slot = t % F32S_STAGES;
        f32s_wait(full + slot, (uint32_t)(t / F32S_STAGES) & 1u, err);
        const float* col = ring + slot * F32S_STAGE_FLOATS + lane;
        const float* xs = x + t * F32S_K;
        // the products of the next 16 k are formed while the current 16 are added: the adds are the only chain
        float pa[16], pb[16];
        auto prod = [&](float (&pr)[16], int k0) {
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                const float4 xv = *(const float4*)(xs + k0 + i);
                pr[i] = __fmul_rn(col[(k0 + i) * 32], xv.x); pr[i + 1] = __fmul_rn(col[(k0 + i + 1) * 32], xv.y);
                pr[i + 2] = __fmul_rn(col[(k0 + i + 2) * 32], xv.z); pr[i + 3] = __fmul_rn(col[(k0 + i + 3) * 32], xv.w);
            }
        };
        prod(pa, 0);
#pragma unroll 2
        for (int k0 = 0; k0 < F32S_K; k0 += 32) {
            prod(pb, k0 + 16);
#pragma unroll
            for (int i = 0; i < 16; ++i) sum = __fadd_rn(sum, pa[i]);
            if (k0 + 32 < F32S_K) prod(pa, k0 + 32);
#pragma unroll
            for (int i = 0; i < 16; ++i) sum = __fadd_rn(sum, pb[i]);
        }
        __syncwarp();                           // every lane has read the slot: hand it back
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"((uint32_t)__cvta_generic_to_shared(empty + slot)) : "memory");
    }
    if (lane < nr) epi(r0 + lane, sum);
}

// Contiguous share [lo, hi) of n items for part `i` of `parts`.
__device__ __forceinline__ void share(int n, int parts, int i, int& lo, int& hi) {
    lo = (int)(((long long)n * i) / parts);
    hi = (int)(((long long)n * (i + 1)) / parts);
}
