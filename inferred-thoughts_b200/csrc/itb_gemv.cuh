// Row-streaming GEMV cores for decode: HBM-bound, 16-byte coalesced weight loads, integer dot per
// quantisation block, and an order-preserving f32 fold so every output equals the CPU path's
// `sumf += term_b` chain to the bit (src/ops/naive.rs:691-734).
//
// Work split inside a warp: G lanes share a row (G = power of two dividing the row's block count),
// 32/G rows run side by side, RP such groups per pass. Each lane owns fixed K-columns, computes the
// integer sums of its blocks, turns them into f32 terms in shared memory; then one lane per row folds
// that row's terms in ascending block order.
#pragma once
#include "itb_internal.cuh"

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// ---- activation prologues ------------------------------------------------------------------------
// RMSNorm of one row into shared memory: f32 squares, f64 accumulation (tree), (x*scale)*w
// (src/ops/naive.rs:139-152, :633-640). `red` holds blockDim.x/32 doubles.
__device__ __forceinline__ void block_rms_norm(const float* __restrict__ x, const float* __restrict__ w, int n, float eps,
                                               float* xn, double* red) {
    double acc = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { float v = x[i]; xn[i] = v; acc += (double)(v * v); }
    acc = warp_sum_d(acc);
    int wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if ((threadIdx.x & 31) == 0) red[wid] = acc;
    __syncthreads();
    double tot = 0.0;
    for (int i = 0; i < nw; ++i) tot += red[i];
    float mean = (float)(tot / (double)n);
    float sc = 1.0f / sqrtf(mean + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) xn[i] = xn[i] * sc * w[i];
    __syncthreads();
}

// Q8_0 activation quantiser over a row in shared memory (src/ops/naive.rs:653-675): one warp per
// 32-block, d = amax/127 through f16, q = roundf(v * (1/d)).
__device__ __forceinline__ void block_quant_q8(const float* xn, int n, int8_t* xq, float* xs) {
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b = wid; b < n / 32; b += nw) {
        float v = xn[b * 32 + lane];
        float amax = warp_max(fabsf(v));
        float d = amax / 127.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        float r = roundf(v * id);
        xq[b * 32 + lane] = (int8_t)fminf(127.0f, fmaxf(-128.0f, r));
        if (lane == 0) xs[b] = __half2float(__float2half_rn(d));
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

// ---- Q8_0 rows -------------------------------------------------------------------------------------
// Rows [r0, r1) of `w` for this warp against one quantised activation (xq, xs in shared memory).
// terms: warp-private shared scratch of RP*(32/G)*(nb+1) floats. epi(row, value) is called by one lane.
template <int RP, class Epi>
__device__ __forceinline__ void q8_rows(const DevQ8& w, int r0, int r1, const int8_t* xq, const float* xs, float* terms, int gsh, Epi epi) {
    const int G = 1 << gsh, lane = threadIdx.x & 31, sub = lane & (G - 1), slot = lane >> gsh;
    const int SLOTS = 32 >> gsh, ROWS = RP * SLOTS;
    const int nb = w.n_in >> 5, stride = nb + 1;
    for (int r = r0; r < r1; r += ROWS) {
        for (int b = sub; b < nb; b += G) {
            uint4 wa[RP], wb[RP];
            uint16_t ws[RP];
#pragma unroll
            for (int i = 0; i < RP; ++i) {
                int row = r + i * SLOTS + slot;
                if (row < r1) {
                    const int8_t* p = w.q + (size_t)row * w.n_in + b * 32;
                    wa[i] = ld_stream16(p); wb[i] = ld_stream16(p + 16);
                    ws[i] = __ldg(w.s + (size_t)row * nb + b);
                }
            }
            const uint4 xa = *(const uint4*)(xq + b * 32), xb = *(const uint4*)(xq + b * 32 + 16);
            const float dx = xs[b];
#pragma unroll
            for (int i = 0; i < RP; ++i) {
                int row = r + i * SLOTS + slot;
                if (row < r1) {
                    int s = 0;
                    s = __dp4a((int)wa[i].x, (int)xa.x, s); s = __dp4a((int)wa[i].y, (int)xa.y, s);
                    s = __dp4a((int)wa[i].z, (int)xa.z, s); s = __dp4a((int)wa[i].w, (int)xa.w, s);
                    s = __dp4a((int)wb[i].x, (int)xb.x, s); s = __dp4a((int)wb[i].y, (int)xb.y, s);
                    s = __dp4a((int)wb[i].z, (int)xb.z, s); s = __dp4a((int)wb[i].w, (int)xb.w, s);
                    terms[(i * SLOTS + slot) * stride + b] = (float)s * (f16_bits_to_f32(ws[i]) * dx);
                }
            }
        }
        __syncwarp();
        if (lane < ROWS && r + lane < r1) {
            const float* t = terms + lane * stride;
            float sum = 0.0f;
            for (int b = 0; b < nb; ++b) sum += t[b];
            epi(r + lane, sum);
        }
        __syncwarp();
    }
}

// ---- NVFP4 rows ------------------------------------------------------------------------------------
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

// Rows [r0, r1) of one NVFP4 matrix (nib: [rows][n_in/2], sc: [rows][n_in/16]) against a Q8_0 activation
// (src/ops/naive.rs:714-734): term per 16-element sub-block = (dy*d)*(float)(lo+hi), folded ascending.
// A lane's unit is a 16-byte chunk = two sub-blocks.
template <int RP, class Epi>
__device__ __forceinline__ void fp4_rows(const uint8_t* __restrict__ nib, const uint8_t* __restrict__ sc, int n_in, int r0, int r1,
                                         const int8_t* xq, const float* xs, float* terms, int gsh, Epi epi) {
    const int G = 1 << gsh, lane = threadIdx.x & 31, sub = lane & (G - 1), slot = lane >> gsh;
    const int SLOTS = 32 >> gsh, ROWS = RP * SLOTS;
    const int nch = n_in >> 5, nsb = n_in >> 4, stride = nsb + 1;
    for (int r = r0; r < r1; r += ROWS) {
        for (int ch = sub; ch < nch; ch += G) {
            uint4 wv[RP];
            uint16_t sv[RP];
#pragma unroll
            for (int i = 0; i < RP; ++i) {
                int row = r + i * SLOTS + slot;
                if (row < r1) {
                    wv[i] = ld_stream16(nib + (size_t)row * (n_in >> 1) + ch * 16);
                    sv[i] = __ldg((const uint16_t*)(sc + (size_t)row * nsb) + ch);
                }
            }
            const uint4 xa = *(const uint4*)(xq + ch * 32), xb = *(const uint4*)(xq + ch * 32 + 16);
            const float dy = xs[ch];  // a 32-element Q8_0 block spans both sub-blocks of the chunk
#pragma unroll
            for (int i = 0; i < RP; ++i) {
                int row = r + i * SLOTS + slot;
                if (row < r1) {
                    int s0 = fp4_dot8(wv[i].x, xa.x, xa.y) + fp4_dot8(wv[i].y, xa.z, xa.w);
                    int s1 = fp4_dot8(wv[i].z, xb.x, xb.y) + fp4_dot8(wv[i].w, xb.z, xb.w);
                    float d0 = ue4m3_half_dev(sv[i] & 0xff), d1 = ue4m3_half_dev(sv[i] >> 8);
                    float* t = terms + (i * SLOTS + slot) * stride + ch * 2;
                    t[0] = dy * d0 * (float)s0;
                    t[1] = dy * d1 * (float)s1;
                }
            }
        }
        __syncwarp();
        if (lane < ROWS && r + lane < r1) {
            const float* t = terms + lane * stride;
            float sum = 0.0f;
            for (int b = 0; b < nsb; ++b) sum += t[b];
            epi(r + lane, sum);
        }
        __syncwarp();
    }
}

// ---- F32 rows --------------------------------------------------------------------------------------
// EXACT: serial-k left fold per output like the CPU path (src/ops/naive.rs:845-849); 32 rows per warp,
// tiles staged through shared memory so global reads stay coalesced. tile: warp-private 32*33 floats.
// Otherwise: lane-strided partial sums and a shuffle tree (order differs, value within rounding).
template <bool EXACT, class Epi>
__device__ __forceinline__ void f32_rows(const float* __restrict__ w, int n_in, int r0, int r1, const float* x, float* tile, Epi epi) {
    const int lane = threadIdx.x & 31;
    if (EXACT) {
        for (int r = r0; r < r1; r += 32) {
            float sum = 0.0f;
            for (int k0 = 0; k0 < n_in; k0 += 32) {
#pragma unroll 8
                for (int rr = 0; rr < 32; ++rr)
                    tile[rr * 33 + lane] = (r + rr < r1 && k0 + lane < n_in) ? __ldg(w + (size_t)(r + rr) * n_in + k0 + lane) : 0.0f;
                __syncwarp();
                int kn = min(32, n_in - k0);
                for (int k = 0; k < kn; ++k) sum += tile[lane * 33 + k] * x[k0 + k];
                __syncwarp();
            }
            if (r + lane < r1) epi(r + lane, sum);
        }
    } else {
        for (int r = r0; r < r1; ++r) {
            const float* p = w + (size_t)r * n_in;
            float s = 0.0f;
            for (int k = lane * 4; k < n_in; k += 128) {
                float4 v = __ldg((const float4*)(p + k));
                s += v.x * x[k] + v.y * x[k + 1] + v.z * x[k + 2] + v.w * x[k + 3];
            }
            s = warp_sum(s);
            if (lane == 0) epi(r, s);
        }
    }
}

// Contiguous share [lo, hi) of n items for part `i` of `parts`.
__device__ __forceinline__ void share(int n, int parts, int i, int& lo, int& hi) {
    lo = (int)(((long long)n * i) / parts);
    hi = (int)(((long long)n * (i + 1)) / parts);
}
