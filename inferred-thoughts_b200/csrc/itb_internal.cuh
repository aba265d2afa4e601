// Internal declarations shared by the library's translation units.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/itb.h"

// ------------------------------------------------------------------ device-side weight layouts
// Q8_0 matrix repacked from 34-byte blocks (src/quant/mod.rs:90-106) into two planes so rows can be
// read with 16-byte loads: quants [n_out][n_in] int8, scales [n_out][n_in/32] f16 bits.
struct DevQ8 {
    const int8_t* q = nullptr;
    const uint16_t* s = nullptr;
    int n_in = 0, n_out = 0;
};
// NVFP4 stack repacked from 36-byte blocks (src/quant/mod.rs:338-357): nibbles [E][n_out][n_in/2] with
// nibble k of byte-pair order = element order (low nibble first), scales [E][n_out][n_in/16] UE4M3 codes
// with bit 7 cleared and 0x7f mapped to 0 (both read as the reference reads them, src/quant/mod.rs:271-284).
struct DevFp4 {
    const uint8_t* nib = nullptr;
    const uint8_t* sc = nullptr;
    const float* scale2 = nullptr;  // per expert, or null
    int n_in = 0, n_out = 0, n_expert = 0;
    int expert_lo = 0;              // first expert stored (expert-parallel shard); ids are global
    const int* slot_map = nullptr;  // tiered experts: global id -> slot in the HBM pool (nib/sc/scale2 are the pool), -1 = not resident
};
#ifdef __CUDACC__
// Where expert `e` of a stack lives on this device: its index into nib/sc/scale2, or -1 (stored elsewhere / not resident).
__device__ __forceinline__ int fp4_slot(const DevFp4& w, int e) {
    if (w.slot_map) return w.slot_map[e];
    const int el = e - w.expert_lo;
    return (el < 0 || el >= w.n_expert) ? -1 : el;
}
#endif
struct DevF32 {
    const float* w = nullptr;
    int n_in = 0, n_out = 0;
    // optional second copy for the serial-k one-token path: units of 32 rows, k-major inside a unit ([unit][k][32 rows], rows
    // past n_out zero), so that 128 k of a unit are 16 KB in one piece and a lane per row reads them without bank conflicts
    const float* wt = nullptr;
};

// ------------------------------------------------------------------ context
struct Mirror {
    void* dev = nullptr;
    size_t bytes = 0;
    bool device_current = false;
};
struct WeightEntry {
    uint32_t ty = 0;
    size_t n_in = 0, n_out = 0, n_expert = 1;
    void* a = nullptr;  // Q8: quants; FP4: nibbles; F32/F16: values as f32
    void* b = nullptr;  // Q8: scales; FP4: block scales
    float* scale2 = nullptr;
    size_t bytes = 0;
};

struct itb_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::string error;       // sticky first error
    std::string error_out;   // storage handed back by take_error
    bool kv_bf16 = false;
    bool exact = true;
    bool in_pass = false;
    uint64_t launches = 0;
    int sm_count = 148;
    std::unordered_map<const void*, Mirror> mirrors;
    std::unordered_map<const void*, Mirror> states;   // recurrent slabs: device owns after first touch
    std::unordered_map<const void*, Mirror> kv;       // KV slabs, keyed by host slab address
    std::unordered_map<const void*, WeightEntry> weights;
    // current device route (src/ops/cuda/ops/mod.rs:299-302)
    int32_t* route_ids = nullptr;
    int* pair_off = nullptr; int* pair_list = nullptr; size_t pair_cap = 0, pair_experts = 0;   // pairs grouped by expert (many-row expert matmuls)
    float* route_w = nullptr;
    size_t route_cap = 0, route_n_tok = 0, route_n_used = 0;
    // scratch for activation quantisation
    int8_t* xq = nullptr; float* xs = nullptr; size_t xq_cap = 0;
    float* tmp_f32 = nullptr; size_t tmp_cap = 0;
    const void* last_state_key = nullptr;
    size_t mirror_bytes = 0, weight_bytes = 0;
    // FP4 tensor-core expert path (itb_tc.cu): expert stacks re-tiled once (keyed by the stack's nibble plane), per-pass scratch
    struct TcWeights { uint8_t* img = nullptr; uint8_t* sf = nullptr; size_t bytes = 0; };
    std::unordered_map<const void*, TcWeights> tc_weights;
    void* tc_tiles = nullptr; int* tc_n_tiles = nullptr; int* tc_slot_tile = nullptr; uint8_t* tc_b_img = nullptr; uint8_t* tc_b_sf = nullptr; int* tc_status = nullptr;
    uint8_t* tc_codes = nullptr; uint8_t* tc_scales = nullptr;      // the pass's activation rows as FP4 records
    size_t tc_cap_tiles = 0, tc_cap_slots = 0, tc_cap_b = 0, tc_cap_sf = 0, tc_cap_codes = 0, tc_cap_scales = 0;
    // Q8_0 tensor path: the pass's activation rows as K32 block images (kept for a following matmul over the same rows)
    uint8_t* tc_q8_b = nullptr; float* tc_q8_sx = nullptr; size_t tc_cap_q8b = 0, tc_cap_q8sx = 0;
    const void* tc_q8_src = nullptr; int tc_q8_src_rows = 0, tc_q8_src_in = 0;
    uint8_t* tc_hf_b = nullptr; size_t tc_cap_hfb = 0;                 // dense=f16tc: the pass's activation rows as f16 operand tiles
    const void* tc_hf_src = nullptr; int tc_hf_src_rows = 0, tc_hf_src_in = 0;
    bool f16tc = false;     // opts dense=f16tc: many-row passes run the dense Q8_0 matmuls as f16 tcgen05 GEMMs over dequantised operands (tolerance class)
    bool q8tc = false;       // opts dense=q8tc: many-row passes run the dense Q8_0 matmuls as tcgen05 int8 MMAs (bit-identical results)
    bool fp4tc = false;      // opts experts=fp4tc: many-row passes multiply FP4 activations on the tensor cores
    bool gdn_chunk = false;  // opts gdn=chunk: many-token passes run the delta rule chunk-parallel even under exact=1 (exact=0 always does)
    bool attn_mma = false;   // opts attn=mma: many-token passes run attention as 16-bit matrix products even under exact=1 (exact=0 always does)
};
// Routed experts over expert-grouped pairs on the FP4 tensor cores (itb_tc.cu). wu != null: out[pair] = silu(Wg x * s_g) * (Wu x * s_u);
// else out[pair] = W x * s. x: f32 rows on the device, the row of slot s is pair_list[s] / rows_div. False: not run (shape or memory).
bool itb_tc_experts(itb_ctx* c, cudaStream_t st, const DevFp4& wg, const DevFp4* wu, const float* x, int rows_div, const int* pair_off,
                    const int* pair_list, int n_pairs, float* out);
bool itb_tc_shape_ok(const DevFp4& w);
bool itb_tc_q8_shape_ok(const DevQ8& w);
bool itb_tc_f16_shape_ok(const DevQ8& w);
bool itb_tc_f16_gemm(itb_ctx* c, cudaStream_t st, const DevQ8& w, const int8_t* xq, const float* xs, int n_rows, float* out, size_t stride, int mode, bool same_acts);
bool itb_tc_q8_gemm(itb_ctx* c, cudaStream_t st, const DevQ8& w, const int8_t* xq, const float* xs, int n_rows, float* out, size_t stride, int mode, bool same_acts);
void itb_tc_free(itb_ctx* c);

bool itb_fail(itb_ctx* c, const char* what, cudaError_t e);
bool itb_fail_msg(itb_ctx* c, const std::string& msg);
#define ITB_CUDA(c, call)                                              \
    do {                                                               \
        cudaError_t e__ = (call);                                      \
        if (e__ != cudaSuccess) { itb_fail((c), #call, e__); return; } \
    } while (0)
#define ITB_CUDA_RET(c, call, ret)                                           \
    do {                                                                     \
        cudaError_t e__ = (call);                                            \
        if (e__ != cudaSuccess) { itb_fail((c), #call, e__); return (ret); } \
    } while (0)
#define ITB_LAUNCHED(c)                                                  \
    do {                                                                 \
        (c)->launches++;                                                 \
        cudaError_t e__ = cudaGetLastError();                            \
        if (e__ != cudaSuccess) itb_fail((c), "kernel launch", e__);     \
    } while (0)

// mirrors (itb_ctx.cu)
float* itb_mirror_in(itb_ctx* c, const float* host, size_t len);
float* itb_mirror_out(itb_ctx* c, const float* host, size_t len);
float* itb_mirror_inout(itb_ctx* c, float* host, size_t len);
float* itb_state_slab(itb_ctx* c, float* host, size_t len);
uint16_t* itb_kv_slab(itb_ctx* c, const uint16_t* host, size_t len);
const WeightEntry* itb_weight(itb_ctx* c, const uint8_t* data, size_t bytes, uint32_t ty, size_t n_in, size_t n_out,
                              size_t n_expert, const uint8_t* scale, size_t scale_bytes);
bool itb_ensure_route(itb_ctx* c, size_t n_pairs);
bool itb_ensure_xq(itb_ctx* c, size_t n_elems);

// repack (itb_ctx.cu): raw reference-layout bytes on the device -> kernel layouts
void itb_repack_q8(cudaStream_t st, const uint8_t* raw, int8_t* q, uint16_t* s, size_t n_blocks_total);
void itb_repack_fp4(cudaStream_t st, const uint8_t* raw, uint8_t* nib, uint8_t* sc, size_t n_blocks64_total);
void itb_f16_to_f32(cudaStream_t st, const uint16_t* raw, float* out, size_t n);

// ------------------------------------------------------------------ device helpers
#ifdef __CUDACC__
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Two UE4M3 scale codes (bit 7 clear, 0x7f already mapped to 0: plain positive e4m3) to their halved f32 values by
// the hardware e4m3 -> f16 conversion, which is exact for every code.
__device__ __forceinline__ void ue4m3x2_half(uint32_t two, float& lo, float& hi) {
    uint32_t h2;
    asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(h2) : "r"(two));
    const __half2 hh = *reinterpret_cast<const __half2*>(&h2);
    lo = __low2float(hh) * 0.5f; hi = __high2float(hh) * 0.5f;
}

// Exact int32 -> f32 for |v| < 2^22 without the conversion pipe: add v to the bit pattern of 1.5 * 2^23, whose ulp is
// 1, and subtract 1.5 * 2^23 again (block sums here stay below 32 * 127 * 127 < 2^19).
__device__ __forceinline__ float i2f_small(int v) { return __int_as_float(0x4B400000 + v) - 12582912.0f; }

// Phase timeline (observability): when a buffer is armed (itb_timeline_arm), thread 0 of block 0 of a launch that was
// given a slot stores %globaltimer at each TL(kernel, phase) site into buf[slot * 16 + phase] -- a plain store, nothing to
// wait for. Slots are the launch ordinals of one decode step; slot < 0 = not recorded.
static __device__ unsigned long long* g_tl_buf = nullptr;
static __device__ unsigned int g_tl_cap = 0;
__device__ __forceinline__ void tl_mark(int slot, unsigned kernel, unsigned phase) {
    if (slot >= 0 && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && g_tl_buf && (unsigned)slot < g_tl_cap) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_tl_buf[(size_t)slot * 16 + phase] = (t << 8) | kernel;
    }
}
// The same from whichever thread of block 0 calls it (one caller per mark).
__device__ __forceinline__ void tl_mark_any(int slot, unsigned kernel, unsigned phase) {
    if (slot >= 0 && blockIdx.x == 0 && g_tl_buf && (unsigned)slot < g_tl_cap) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_tl_buf[(size_t)slot * 16 + phase] = (t << 8) | kernel;
    }
}
#define TL(kernel, phase) tl_mark(p.tl_slot, (kernel), (phase))
enum { TLK_EMBED = 1, TLK_IN_PROJ, TLK_GDN_CORE, TLK_OUT_PROJ, TLK_ATTN_PREP, TLK_ATTN_PART, TLK_ATTN_COMB, TLK_MOE_GLU, TLK_MOE_DOWN, TLK_ARGMAX_P, TLK_ARGMAX_A };

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start while
// its predecessor still runs. pdl_trigger() lets the successor be scheduled; pdl_wait() returns once every
// predecessor grid has completed and its writes are visible. Before pdl_wait() a kernel may touch only memory no
// kernel of the same chain writes (weights, its own layer's state). Both are no-ops in an ordinary launch.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Byte ranges a later kernel of the step will stream (weights and state: they do not depend on what the kernels in between
// compute). Every block of the kernel that carries the hint asks for its share of them to be brought into L2 while the kernel
// runs, so the memory system keeps streaming through the step's dependent stages. (Every block, because a bulk prefetch is
// carried out by the issuing SM's copy engine at that SM's bandwidth: one block asking for 27 MB holds its kernel open for
// far longer than the kernel lasts.) A hint only: nothing waits for it.
struct L2Hint { const void* p[8]; unsigned n[8]; };
__device__ __forceinline__ void l2_hint(const L2Hint& h, unsigned part, unsigned n_parts, int lane) {
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
        if (!h.p[i]) continue;
        const uintptr_t a = ((uintptr_t)h.p[i] + 15) & ~(uintptr_t)15, z = ((uintptr_t)h.p[i] + h.n[i]) & ~(uintptr_t)15;
        if (z <= a) continue;
        // this block's share, in 16-byte units, split over the warp's lanes in pieces of 4 KB
        const unsigned long long units = (z - a) >> 4, per = (units + n_parts - 1) / n_parts;
        const unsigned long long u0 = min(units, per * part), u1 = min(units, u0 + per);
        for (unsigned long long u = u0 + (unsigned long long)lane * 256u; u < u1; u += 32u * 256u) {
            const unsigned sz = (unsigned)(min((unsigned long long)256u, u1 - u) << 4);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a + (u << 4)), "r"(sz) : "memory");
        }
    }
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// expf and logf as the C library computes them. The reference CPU path calls the platform's libm (Rust's f32::exp and
// f32::ln), whose single-precision routines are fast table-driven approximations evaluated in double: close to, but not
// always, the correctly rounded result (measured against glibc: (float)exp((double)x) differs from expf(x) for 0.06 % of
// inputs, (float)log((double)x) from logf(x) for 1.2 %). A last-bit difference in a GatedDeltaNet decay gate stays in the
// recurrent state for good, so both functions follow the library here instead of being "more exact" than it.
//
// exp_f: the published algorithm of the library routine (exp(x) = 2^(k/32) * 2^(r/32), k = round(x * 32/ln2) by the
// add-and-subtract-1.5*2^52 trick, 2^(i/32) from a 32-entry table, 2^(r/32) by a cubic polynomial, all in double, one
// final rounding to float), restated. The table is 2^(i/32) rounded to nearest double minus i << 47, generated from integer
// arithmetic; the three polynomial coefficients and 32/ln2 are the routine's published constants. Host and device share the
// code: tests compare the host build with the C library's expf on millions of inputs (mismatches: about 1 in 10^8).
#define ITB_EXP2_TAB                                                                                   \
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull, \
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull, \
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull, \
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull, \
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull, \
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull, \
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull, \
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull,
#ifdef __CUDACC__
// In global memory, read through the L1/read-only path: lanes ask for different entries, which the constant bank would serialise.
static __device__ const unsigned long long c_exp2_tab[32] = {ITB_EXP2_TAB};
#endif
__host__ __device__ inline float itb_expf_lib(float x, const unsigned long long* tab) {
    const double N = 32.0, inv_ln2_n = 0x1.71547652b82fep+0 * N, shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / N / N / N, c1 = 0x1.ebfce50fac4f3p-3 / N / N, c2 = 0x1.62e42ff0c52d6p-1 / N;
    if (!(x > -88.0f && x < 88.0f)) {
        if (x != x) return x + x;
        if (x > 0x1.62e42ep6f) return __builtin_huge_valf();     // above log(2^128)
        if (x < -0x1.9fe368p6f) return 0.0f;                     // below log(2^-150)
    }
    double z = inv_ln2_n * (double)x;
    double kd = z + shift;
    unsigned long long ki;
#ifdef __CUDA_ARCH__
    ki = (unsigned long long)__double_as_longlong(kd);
#else
    __builtin_memcpy(&ki, &kd, 8);
#endif
    kd -= shift;
    const double r = z - kd;
    const unsigned long long t = tab[ki & 31] + (ki << 47);
    double s;
#ifdef __CUDA_ARCH__
    s = __longlong_as_double((long long)t);
#else
    __builtin_memcpy(&s, &t, 8);
#endif
    z = c0 * r + c1;
    const double r2 = r * r;
    double y = c2 * r + 1.0;
    y = z * r2 + y;
    y = y * s;
    return (float)y;
}
// log_f: correctly rounded (through the f64 unit), then moved by the one ulp the host's logf differs by, read from a table
// the context builds on the host by calling logf on every float of [1, 2^29) -- the whole range softplus can ask for
// (ln(1 + e^a), a <= 20) -- two bits per float. Without a table (g_logf_fix null) the correctly rounded value stands.
static __device__ const uint32_t* g_logf_fix = nullptr;
static __device__ uint32_t g_logf_fix_n = 0;
#ifdef __CUDACC__
// Not inlined: one copy per kernel keeps the instruction footprint small.
static __device__ __noinline__ float exp_f(float x) { return itb_expf_lib(x, c_exp2_tab); }
static __device__ __noinline__ float log_f(float x) {
    float v = (float)log((double)x);
    const uint32_t idx = __float_as_uint(x) - 0x3f800000u;
    if (g_logf_fix && idx < g_logf_fix_n) {
        const uint32_t f = (g_logf_fix[idx >> 4] >> ((idx & 15u) * 2u)) & 3u;
        v = __uint_as_float(__float_as_uint(v) + (f == 1u ? 1u : 0u) - (f == 2u ? 1u : 0u));   // results here are positive: +1 bit = +1 ulp
    }
    return v;
}
#endif
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + exp_f(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + exp_f(-x)); }
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    uint32_t b = __float_as_uint(f);
    if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x40);
    b += 0x7fffu + ((b >> 16) & 1u);
    return (uint16_t)(b >> 16);
}
// UE4M3 scale code (bit 7 already cleared, 0x7f already mapped to 0), halved: (8+m)*2^(e-11) or m*2^-10.
__device__ __forceinline__ float ue4m3_half_dev(uint32_t x) {
    uint32_t e = (x >> 3) & 0xf, m = x & 7;
    float mant = (float)(e == 0 ? m : 8 + m);
    float p = __uint_as_float((e == 0 ? 117u : 116u + e) << 23);
    return x == 0 ? 0.0f : mant * p;
}
#endif
