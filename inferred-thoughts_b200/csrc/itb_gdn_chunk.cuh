// Chunked-parallel gated delta rule for many-token passes (the job of the batched kernel in kernels/gdn.cuh of the reference).
//
// Per value head the CPU path runs, token by token (src/ops/naive.rs:86-135):
//     S <- g_t S;   d_t = beta_t (v_t - S k_t);   S <- S + d_t k_t^T;   o_t = S q_t          (S: [value row j][key i])
// Over a chunk of C tokens with state S0 at its start, G_t = g_1 ... g_t and L_t = log G_t, the same recurrence reads
//     (I + A) D = diag(beta) V - diag(beta G) K S0^T,    A[t][s] = beta_t exp(L_t - L_s) (k_t . k_s) for s < t
//     O         = diag(G) Q S0^T + P D,                   P[t][s] = exp(L_t - L_s) (q_t . k_s)       for s <= t
//     S_C       = G_C S0 + D^T diag(exp(L_C - L_s)) K
// so with T = (I + A)^-1, W = T diag(beta G) K and U = T diag(beta) V:  D = U - W S0^T. Everything that does not involve the
// state (A, T, W, U, P, the scaled q and k) is computed for ALL chunks at once (k_gdn_chunk_prep, a block per chunk and head);
// what remains serial is three small matrix products per chunk (k_gdn_chunk_scan, a block per head and 32 value rows, since
// value rows never mix). Sums are reassociated against the token-by-token order: tolerance class, in f32 throughout (the
// decay ratios go through logs, so a chunk that forgets everything underflows to zero instead of dividing by it).
// exact=1 passes keep the serial-order scan (k_gdn_scan).
#pragma once
#include "itb_tile.cuh"

namespace {

constexpr int GC = 64;             // tokens per chunk
constexpr int GC_VS = 32;          // value rows per block of the scan
// Scratch of one (chunk, value head), floats: W | Qg | Kd | U (each GC x SK) | P (GC x GC) | G_C, pad
template <int SK> __host__ __device__ constexpr size_t gdn_chunk_floats() { return (size_t)4 * GC * SK + GC * GC + 4; }

__device__ __forceinline__ float4 ld4(const float* p) { return *(const float4*)p; }

// grid (chunks per sequence, n_v, n_seq); block 256.
template <int SK>
__global__ void __launch_bounds__(256) k_gdn_chunk_prep(const float* qh, const float* kh, const float* vh, const float* gb, int n_tok, int n_k, int n_v,
                                                        float* scratch) {
    constexpr int ST = SK + 4;     // shared rows 16-byte aligned and on different banks
    extern __shared__ __align__(16) unsigned char smem[];
    float* Ks = (float*)smem;                  // [GC][ST]
    float* Qs = Ks + GC * ST;
    float* Vs = Qs + GC * ST;
    float* As = Vs + GC * ST;                  // [GC][GC + 4]: A, strictly lower
    float* L = As + GC * (GC + 4);             // [GC] cumulative log decay
    float* Bt = L + GC;                        // [GC] beta
    const int ch = blockIdx.x, h = blockIdx.y, seq = blockIdx.z, khd = h % n_k, tid = threadIdx.x;
    const int t0 = ch * GC, nv = min(GC, n_tok - t0), n_ch = gridDim.x;
    const size_t row0 = (size_t)seq * n_tok + t0;
    float* out = scratch + (((size_t)seq * n_ch + ch) * n_v + h) * gdn_chunk_floats<SK>();
    float* Wg = out; float* Qg = Wg + GC * SK; float* Kd = Qg + GC * SK; float* Ug = Kd + GC * SK; float* Pg = Ug + GC * SK;
    for (int i = tid; i < GC * (SK / 4); i += 256) {
        const int t = i / (SK / 4), c = (i % (SK / 4)) * 4;
        const bool ok = t < nv;
        cp_async16(Ks + t * ST + c, kh + ((row0 + (ok ? t : 0)) * n_k + khd) * SK + c, ok);
        cp_async16(Qs + t * ST + c, qh + ((row0 + (ok ? t : 0)) * n_k + khd) * SK + c, ok);
        cp_async16(Vs + t * ST + c, vh + ((row0 + (ok ? t : 0)) * n_v + h) * SK + c, ok);
    }
    cp_async_commit();
    if (tid < 32) {                            // cumulative log decay: an inclusive scan over the chunk's 64 tokens, two per lane
        const int a = 2 * tid, b = a + 1;
        const float la = a < nv ? __logf(gb[((row0 + a) * n_v + h) * 2]) : 0.0f, lb = b < nv ? __logf(gb[((row0 + b) * n_v + h) * 2]) : 0.0f;
        float s = la + lb;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const float v = __shfl_up_sync(0xffffffffu, s, o); if (tid >= o) s += v; }
        L[a] = s - lb; L[b] = s;
        Bt[a] = a < nv ? gb[((row0 + a) * n_v + h) * 2 + 1] : 0.0f; Bt[b] = b < nv ? gb[((row0 + b) * n_v + h) * 2 + 1] : 0.0f;
    }
    cp_async_wait<0>();
    __syncthreads();
    // A and P: thread -> token t (lanes on consecutive rows: no bank conflicts) and 16 of the chunk's positions s (a row every
    // lane reads together); pairs past the diagonal are skipped
    {
        const int t = tid & 63, s0 = (tid >> 6) * 16;
        float kk[16], qk[16];
#pragma unroll
        for (int b = 0; b < 16; ++b) { kk[b] = 0.f; qk[b] = 0.f; }
        if (s0 <= t) {
            for (int i = 0; i < SK; i += 4) {
                const float4 kt = ld4(Ks + t * ST + i), qt = ld4(Qs + t * ST + i);
#pragma unroll
                for (int b = 0; b < 16; ++b) {
                    const float4 ks = ld4(Ks + (s0 + b) * ST + i);
                    kk[b] = __fmaf_rn(kt.x, ks.x, kk[b]); kk[b] = __fmaf_rn(kt.y, ks.y, kk[b]); kk[b] = __fmaf_rn(kt.z, ks.z, kk[b]); kk[b] = __fmaf_rn(kt.w, ks.w, kk[b]);
                    qk[b] = __fmaf_rn(qt.x, ks.x, qk[b]); qk[b] = __fmaf_rn(qt.y, ks.y, qk[b]); qk[b] = __fmaf_rn(qt.z, ks.z, qk[b]); qk[b] = __fmaf_rn(qt.w, ks.w, qk[b]);
                }
            }
        }
#pragma unroll
        for (int b = 0; b < 16; ++b) {
            const int sp = s0 + b;
            const float dec = sp <= t ? __expf(L[t] - L[sp]) : 0.0f;
            As[t * (GC + 4) + sp] = sp < t ? Bt[t] * dec * kk[b] : 0.0f;
            Pg[t * GC + sp] = dec * qk[b];
        }
    }
    __syncthreads();
    // (I + A) X = RHS by forward substitution, a column of [beta G K | beta V] per thread, the column's 64 entries in registers
    if (tid < 2 * SK) {
        const bool is_w = tid < SK;
        const int c = is_w ? tid : tid - SK;
        const float* src = is_w ? Ks : Vs;
        float x[GC];
#pragma unroll
        for (int t = 0; t < GC; ++t) {
            float acc = Bt[t] * (is_w ? __expf(L[t]) : 1.0f) * src[t * ST + c];
#pragma unroll
            for (int s4 = 0; s4 + 4 <= t; s4 += 4) {
                const float4 a = ld4(As + t * (GC + 4) + s4);
                acc = __fmaf_rn(-a.x, x[s4], acc); acc = __fmaf_rn(-a.y, x[s4 + 1], acc); acc = __fmaf_rn(-a.z, x[s4 + 2], acc); acc = __fmaf_rn(-a.w, x[s4 + 3], acc);
            }
#pragma unroll
            for (int s = t & ~3; s < t; ++s) acc = __fmaf_rn(-As[t * (GC + 4) + s], x[s], acc);
            x[t] = acc;
            (is_w ? Wg : Ug)[t * SK + c] = acc;
        }
    }
    // the decayed q and k the scan multiplies the state with
    const float lc = L[GC - 1];
    for (int i = tid; i < GC * SK; i += 256) {
        const int t = i / SK, c = i % SK;
        Qg[i] = __expf(L[t]) * Qs[t * ST + c];
        Kd[i] = __expf(lc - L[t]) * Ks[t * ST + c];
    }
    if (tid == 0) Pg[GC * GC] = __expf(lc);
}
template <int SK> constexpr size_t gdn_chunk_prep_smem() { return (size_t)(3 * GC * (SK + 4) + GC * (GC + 4) + 2 * GC) * 4; }

// grid (n_v, SK / 32, n_seq); block 256. The state slice [32 value rows][SK keys] lives in shared memory across the chunks.
template <int SK>
__global__ void __launch_bounds__(256) k_gdn_chunk_scan(const float* scratch, int n_tok, int n_v, float* state, size_t state_stride, float* out) {
    constexpr int ST = SK + 4, DS = GC_VS + 4, PS = GC + 4;
    extern __shared__ __align__(16) unsigned char smem[];
    float* S = (float*)smem;                   // [32][ST]
    float* D = S + GC_VS * ST;                 // [GC][DS]
    float* Ws = D + GC * DS;                   // [GC][ST]
    float* Qs = Ws + GC * ST;
    float* Ks = Qs + GC * ST;
    float* Us = Ks + GC * ST;                  // [GC][DS]
    float* Ps = Us + GC * DS;                  // [GC][PS]
    __shared__ float s_gc[2];
    const int h = blockIdx.x, vs0 = blockIdx.y * GC_VS, seq = blockIdx.z, tid = threadIdx.x;
    const int n_ch = (n_tok + GC - 1) / GC;
    float* sg = state + (size_t)seq * state_stride + ((size_t)h * SK + vs0) * SK;
    for (int i = tid; i < GC_VS * (SK / 4); i += 256) {
        const int j = i / (SK / 4), c = (i % (SK / 4)) * 4;
        *(float4*)(S + j * ST + c) = ld4(sg + (size_t)j * SK + c);
    }
    auto chunk = [&](int ch) { return scratch + (((size_t)seq * n_ch + ch) * n_v + h) * gdn_chunk_floats<SK>(); };
    auto load_rows = [&](float* dst, const float* src) {       // GC x SK
        for (int i = tid; i < GC * (SK / 4); i += 256) { const int t = i / (SK / 4), c = (i % (SK / 4)) * 4; cp_async16(dst + t * ST + c, src + (size_t)t * SK + c, true); }
    };
    auto load_w = [&](int ch) { if (ch < n_ch) load_rows(Ws, chunk(ch)); cp_async_commit(); };
    auto load_qp = [&](int ch) {           // Q, P and the U slice
        if (ch < n_ch) {
            const float* b = chunk(ch);
            load_rows(Qs, b + GC * SK);
            for (int i = tid; i < GC * (GC / 4); i += 256) { const int t = i / (GC / 4), c = (i % (GC / 4)) * 4; cp_async16(Ps + t * PS + c, b + 4 * GC * SK + t * GC + c, true); }
            for (int i = tid; i < GC * (GC_VS / 4); i += 256) { const int t = i / (GC_VS / 4), c = (i % (GC_VS / 4)) * 4; cp_async16(Us + t * DS + c, b + 3 * GC * SK + (size_t)t * SK + vs0 + c, true); }
        }
        cp_async_commit();
    };
    auto load_ku = [&](int ch) {
        if (ch < n_ch) {
            const float* b = chunk(ch);
            load_rows(Ks, b + 2 * GC * SK);
            if (tid == 0) s_gc[ch & 1] = b[4 * GC * SK + GC * GC];
        }
        cp_async_commit();
    };
    load_w(0); load_qp(0); load_ku(0);
    // thread -> 4 tokens x value rows {jq, jq + 16} for the products with the state; 4 value rows x 4 keys for the state update
    const int tq = (tid >> 4) * 4, jq = tid & 15;
    const int uj = (tid >> 5) * 4, ui = (tid & 31) * 4;
#pragma unroll 1
    for (int ch = 0; ch < n_ch; ++ch) {
        const int t0 = ch * GC, nv = min(GC, n_tok - t0);
        cp_async_wait<2>();                    // W of this chunk (the groups behind it: its Q/P and K/U)
        __syncthreads();                       // ... and the state as the previous chunk left it
        float acc[4][2];
        // D = U - W S^T
#pragma unroll
        for (int a = 0; a < 4; ++a) { acc[a][0] = 0.f; acc[a][1] = 0.f; }
        for (int i = 0; i < SK; i += 4) {
            const float4 s0 = ld4(S + jq * ST + i), s1 = ld4(S + (jq + 16) * ST + i);
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float4 w = ld4(Ws + (tq + a) * ST + i);
                acc[a][0] = __fmaf_rn(w.x, s0.x, acc[a][0]); acc[a][0] = __fmaf_rn(w.y, s0.y, acc[a][0]); acc[a][0] = __fmaf_rn(w.z, s0.z, acc[a][0]); acc[a][0] = __fmaf_rn(w.w, s0.w, acc[a][0]);
                acc[a][1] = __fmaf_rn(w.x, s1.x, acc[a][1]); acc[a][1] = __fmaf_rn(w.y, s1.y, acc[a][1]); acc[a][1] = __fmaf_rn(w.z, s1.z, acc[a][1]); acc[a][1] = __fmaf_rn(w.w, s1.w, acc[a][1]);
            }
        }
        __syncthreads();                       // every thread is done with W
        load_w(ch + 1);
        cp_async_wait<2>();                    // Q, P and U of this chunk (behind them: K, the next W)
        __syncthreads();
#pragma unroll
        for (int a = 0; a < 4; ++a) { D[(tq + a) * DS + jq] = Us[(tq + a) * DS + jq] - acc[a][0]; D[(tq + a) * DS + jq + 16] = Us[(tq + a) * DS + jq + 16] - acc[a][1]; }
        // O = Qg S^T + P D
#pragma unroll
        for (int a = 0; a < 4; ++a) { acc[a][0] = 0.f; acc[a][1] = 0.f; }
        for (int i = 0; i < SK; i += 4) {
            const float4 s0 = ld4(S + jq * ST + i), s1 = ld4(S + (jq + 16) * ST + i);
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float4 w = ld4(Qs + (tq + a) * ST + i);
                acc[a][0] = __fmaf_rn(w.x, s0.x, acc[a][0]); acc[a][0] = __fmaf_rn(w.y, s0.y, acc[a][0]); acc[a][0] = __fmaf_rn(w.z, s0.z, acc[a][0]); acc[a][0] = __fmaf_rn(w.w, s0.w, acc[a][0]);
                acc[a][1] = __fmaf_rn(w.x, s1.x, acc[a][1]); acc[a][1] = __fmaf_rn(w.y, s1.y, acc[a][1]); acc[a][1] = __fmaf_rn(w.z, s1.z, acc[a][1]); acc[a][1] = __fmaf_rn(w.w, s1.w, acc[a][1]);
            }
        }
        __syncthreads();                       // D is complete
        for (int s = 0; s < GC; s += 4) {
            float d0[4], d1[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) { d0[b] = D[(s + b) * DS + jq]; d1[b] = D[(s + b) * DS + jq + 16]; }
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float4 pr = ld4(Ps + (tq + a) * PS + s);
                acc[a][0] = __fmaf_rn(pr.x, d0[0], acc[a][0]); acc[a][0] = __fmaf_rn(pr.y, d0[1], acc[a][0]); acc[a][0] = __fmaf_rn(pr.z, d0[2], acc[a][0]); acc[a][0] = __fmaf_rn(pr.w, d0[3], acc[a][0]);
                acc[a][1] = __fmaf_rn(pr.x, d1[0], acc[a][1]); acc[a][1] = __fmaf_rn(pr.y, d1[1], acc[a][1]); acc[a][1] = __fmaf_rn(pr.z, d1[2], acc[a][1]); acc[a][1] = __fmaf_rn(pr.w, d1[3], acc[a][1]);
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
            if (tq + a < nv) {
                float* o = out + (((size_t)seq * n_tok + t0 + tq + a) * n_v + h) * SK + vs0;
                o[jq] = acc[a][0]; o[jq + 16] = acc[a][1];
            }
        // S = G_C S + D^T Kd
        float up[4][4];
        const float gc = s_gc[ch & 1];
#pragma unroll
        for (int a = 0; a < 4; ++a) { const float4 v = ld4(S + (uj + a) * ST + ui); up[a][0] = v.x * gc; up[a][1] = v.y * gc; up[a][2] = v.z * gc; up[a][3] = v.w * gc; }
        __syncthreads();                       // every thread has read the old state (products above) and is done with Q, P and U
        load_qp(ch + 1);
        cp_async_wait<2>();                    // K of this chunk (behind it: the next W, the next Q/P/U)
        __syncthreads();
        for (int s = 0; s < GC; ++s) {
            const float4 dv = ld4(D + s * DS + uj), kv = ld4(Ks + s * ST + ui);
            const float dd[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                up[a][0] = __fmaf_rn(dd[a], kv.x, up[a][0]); up[a][1] = __fmaf_rn(dd[a], kv.y, up[a][1]);
                up[a][2] = __fmaf_rn(dd[a], kv.z, up[a][2]); up[a][3] = __fmaf_rn(dd[a], kv.w, up[a][3]);
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) *(float4*)(S + (uj + a) * ST + ui) = make_float4(up[a][0], up[a][1], up[a][2], up[a][3]);
        __syncthreads();                       // K and D are free, the new state is in place
        load_ku(ch + 1);
    }
    cp_async_wait<0>();
    __syncthreads();
    for (int i = tid; i < GC_VS * (SK / 4); i += 256) {
        const int j = i / (SK / 4), c = (i % (SK / 4)) * 4;
        *(float4*)(sg + (size_t)j * SK + c) = ld4(S + j * ST + c);
    }
}
template <int SK> constexpr size_t gdn_chunk_scan_smem() { return (size_t)(GC_VS * (SK + 4) + 2 * GC * (GC_VS + 4) + 3 * GC * (SK + 4) + GC * (GC + 4)) * 4; }

}  // namespace
