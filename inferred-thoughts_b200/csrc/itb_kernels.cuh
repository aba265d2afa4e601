// Device kernels shared by the op-level seam (itb_ops.cu) and the fused engine (itb_engine.cu).
#pragma once
#include "itb_gemv.cuh"
#include "itb_mma.cuh"

namespace {  // each translation unit gets its own copy of these kernels

// ---- elementwise / small ops (one thread per element; src/ops/naive.rs:246-357, src/ops/mod.rs:600-1270) ----
__global__ void k_silu_mul(float* g, const float* u, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) g[i] = silu_f(g[i]) * u[i];
}
__global__ void k_sigmoid_mul(float* x, const float* g, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= sigmoid_f(g[i]);
}
__global__ void k_scale(float* x, size_t n, float s) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= s;
}
__global__ void k_add_assign(float* a, const float* b, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] += b[i];
}
__global__ void k_add_scaled(float* a, const float* b, size_t n, float s, const float* logit) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (logit) s = sigmoid_f(logit[0]);
    if (i < n) a[i] += b[i] * s;
}
__global__ void k_add_scaled_rows(float* acc, size_t n, const float* rows, const float* scales, size_t n_rows) {
    size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    float v = 0.0f;
    for (size_t e = 0; e < n_rows; ++e) v += scales[e] * rows[e * n + j];
    acc[j] = v;
}
__global__ void k_gather_chunks(const float* src, size_t chunk, size_t stride, size_t offset, float* out, size_t out_len) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < out_len) out[i] = src[(i / chunk) * stride + offset + i % chunk];
}
__global__ void k_scatter_chunks(const float* src, size_t src_len, size_t chunk, size_t stride, size_t offset, float* dst) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < src_len) dst[offset + (i / chunk) * stride + i % chunk] = src[i];
}
__global__ void k_kv_write(uint16_t* slab, size_t offset, const float* src, size_t n, int bf16) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) slab[offset + i] = bf16 ? f32_to_bf16_bits(src[i]) : f32_to_f16_bits(src[i]);
}

// RMSNorm over rows of nd (block per row); out may alias x. w has nd entries (src/ops/naive.rs:139-164).
__global__ void k_rms_norm(const float* x, const float* w, int nd, float eps, float* out) {
    extern __shared__ __align__(16) unsigned char smem[];
    double* red = (double*)smem;
    float* xn = (float*)(red + 32);
    const float* row = x + (size_t)blockIdx.x * nd;
    block_rms_norm(row, w, nd, eps, xn, red);
    for (int i = threadIdx.x; i < nd; i += blockDim.x) out[(size_t)blockIdx.x * nd + i] = xn[i];
}

// L2 norm per head: warp per head, f64 tree sum, 1/max(sqrtf((float)sum), eps) (src/ops/naive.rs:254-273).
__global__ void k_l2_norm_heads(float* x, size_t n_heads, int hd, float eps) {
    size_t h = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (h >= n_heads) return;
    int lane = threadIdx.x & 31;
    float* p = x + h * hd;
    double acc = 0.0;
    for (int i = lane; i < hd; i += 32) acc += (double)(p[i] * p[i]);
    acc = warp_sum_d(acc);
    float sc = 1.0f / fmaxf(sqrtf((float)acc), eps);
    for (int i = lane; i < hd; i += 32) p[i] *= sc;
}

// Row softmax, warp per row: max, exp, serial-order-free sum (tolerance class: expf) (src/ops/naive.rs:362-376).
__global__ void k_softmax_rows(float* x, size_t n_rows, int row) {
    size_t r = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    int lane = threadIdx.x & 31;
    float* p = x + r * row;
    float mx = -INFINITY;
    for (int i = lane; i < row; i += 32) mx = fmaxf(mx, p[i]);
    mx = warp_max(mx);
    // The CPU sums serially in index order; lane 0 does the same so the sum's rounding matches.
    for (int i = lane; i < row; i += 32) p[i] = exp_f(p[i] - mx);
    __syncwarp();
    float sum = 0.0f;
    if (lane == 0) for (int i = 0; i < row; ++i) sum += p[i];
    sum = __shfl_sync(0xffffffffu, sum, 0);
    for (int i = lane; i < row; i += 32) p[i] /= sum;
}

// Partial NEOX RoPE; the angle is computed in f64 like the CPU path (src/ops/naive.rs:180-218).
// One thread per (row, head, pair). pos_base + row index gives the position; pos_dev (optional)
// overrides with a per-row device position.
__global__ void k_rope(float* x, size_t n_rows, int n_heads, int hd, int n_rot, float theta, size_t pos_base, const int* pos_dev) {
    int half = n_rot / 2;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = n_rows * n_heads * half;
    if (i >= total) return;
    int pr = (int)(i % half);
    size_t hh = i / half;
    size_t t = hh / n_heads;
    double pos = pos_dev ? (double)pos_dev[t] : (double)(pos_base + t);
    double freq = pow((double)theta, -2.0 * (double)pr / (double)n_rot);
    double th = pos * freq;
    float sn = (float)sin(th), cs = (float)cos(th);
    float* head = x + hh * hd;
    float x0 = head[pr], x1 = head[pr + half];
    head[pr] = x0 * cs - x1 * sn;
    head[pr + half] = x0 * sn + x1 * cs;
}

// Depthwise causal conv + SiLU with the window kept oldest-first; tokens in order per channel
// (src/ops/naive.rs:275-315). state [nc][keep], w [nc][kernel].
__global__ void k_ssm_conv(float* state, const float* x, size_t n_tok, int nc, const float* w, int kernel, float* out) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nc) return;
    int keep = kernel - 1;
    float past[8], wt[8];
    for (int k = 0; k < keep; ++k) past[k] = state[(size_t)c * keep + k];
    for (int k = 0; k < kernel; ++k) wt[k] = w[(size_t)c * kernel + k];
    for (size_t t = 0; t < n_tok; ++t) {
        float xv = x[t * nc + c];
        float sum = 0.0f;
        for (int k = 0; k < keep; ++k) sum += past[k] * wt[k];
        sum += xv * wt[keep];
        out[t * nc + c] = silu_f(sum);
        for (int k = 0; k + 1 < keep; ++k) past[k] = past[k + 1];
        past[keep - 1] = xv;
    }
    for (int k = 0; k < keep; ++k) state[(size_t)c * keep + k] = past[k];
}

// Gated delta rule (src/ops/naive.rs:86-135): block = (value head, slice of ROWS value rows), one thread
// per row, the row's keys walked serially so every sum has the CPU's order. The slice of state lives in
// shared memory across the tokens of the call. q,k: [n_tok][n_k*sk]; v,out: [n_tok][n_v*sv].
template <int ROWS>
__global__ void k_delta_rule(const float* q, const float* k, const float* v, const float* alpha, const float* beta,
                             const float* ssm_a, const float* dt_bias, size_t n_tok, int sk, int sv, int n_k, int n_v,
                             float* state, float* out) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* S = (float*)smem;             // [ROWS][sk+1]
    float* kq = S + ROWS * (sk + 1);     // k[sk], q[sk] (pre-scaled)
    int h = blockIdx.x, j0 = blockIdx.y * ROWS, kh = h % n_k;
    int tid = threadIdx.x;               // blockDim.x == ROWS * 4 loaders; thread < ROWS computes
    float* sg = state + ((size_t)h * sv + j0) * sk;
    int rows = min(ROWS, sv - j0);
    for (int i = tid; i < rows * sk; i += blockDim.x) S[(i / sk) * (sk + 1) + i % sk] = sg[i];
    float q_scale = 1.0f / sqrtf((float)sk);
    for (size_t t = 0; t < n_tok; ++t) {
        __syncthreads();
        for (int i = tid; i < sk; i += blockDim.x) {
            kq[i] = k[(t * n_k + kh) * sk + i];
            kq[sk + i] = q[(t * n_k + kh) * sk + i] * q_scale;
        }
        __syncthreads();
        if (tid < rows) {
            float a = alpha[t * n_v + h] + dt_bias[h];
            float sp = a > 20.0f ? a : log_f(1.0f + exp_f(a));
            float g = exp_f(sp * ssm_a[h]);
            float b = sigmoid_f(beta[t * n_v + h]);
            float* row = S + tid * (sk + 1);
            float pred = 0.0f;
            for (int i = 0; i < sk; ++i) { float s = row[i] * g; row[i] = s; pred += s * kq[i]; }
            float d = b * (v[(t * n_v + h) * sv + j0 + tid] - pred);
            float o = 0.0f;
            for (int i = 0; i < sk; ++i) { float s = row[i] + kq[i] * d; row[i] = s; o += s * kq[sk + i]; }
            out[(t * n_v + h) * sv + j0 + tid] = o;
        }
    }
    __syncthreads();
    for (int i = tid; i < rows * sk; i += blockDim.x) sg[i] = S[(i / sk) * (sk + 1) + i % sk];
}

// Top-k routing per token (src/ops/mod.rs:1191-1216): n_used rounds of arg-max with strict '>' and ties to
// the lower id, weights p/max(sum, 6.103515625e-5) with the sum taken serially in pick order.
// Block (256 threads) per token, n_expert <= 1024.
__device__ __forceinline__ void block_topk(const float* p, int n_expert, int n_used, int32_t* ids, float* wts, float* sval, int* sidx) {
    int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
    __shared__ int picked[16];
    for (int r = 0; r < n_used; ++r) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = tid; e < n_expert; e += blockDim.x) {
            bool taken = false;
            for (int i = 0; i < r; ++i) taken |= picked[i] == e;
            float v = p[e];
            if (!taken && (bi == 0x7fffffff || v > bv)) { bv = v; bi = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if (lane == 0) { sval[wid] = bv; sidx[wid] = bi; }
        __syncthreads();
        if (tid == 0) {
            float v0 = sval[0]; int i0 = sidx[0];
            for (int w = 1; w < nw; ++w) {
                if (sidx[w] != 0x7fffffff && (i0 == 0x7fffffff || sval[w] > v0 || (sval[w] == v0 && sidx[w] < i0))) { v0 = sval[w]; i0 = sidx[w]; }
            }
            picked[r] = i0;
        }
        __syncthreads();
    }
    if (tid == 0) {
        float sum = 0.0f;
        for (int i = 0; i < n_used; ++i) sum += p[picked[i]];
        float denom = fmaxf(sum, 6.103515625e-5f);
        for (int i = 0; i < n_used; ++i) { ids[i] = picked[i]; wts[i] = p[picked[i]] / denom; }
    }
    __syncthreads();
}
// The same rule inside ONE warp, probabilities in registers (expert e = lane + 32*j), no block barrier:
// every round is a lane-local scan plus a five-step shuffle reduction. All lanes return the picks in
// ids/wts (arrays of 16). p may be shared or global memory; n_expert <= 32*EPL.
template <int EPL>
__device__ __forceinline__ void warp_topk(const float* p, int n_expert, int n_used, int32_t* ids, float* wts) {
    const int lane = threadIdx.x & 31;
    float v[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = lane + 32 * j < n_expert ? p[lane + 32 * j] : 0.0f;
    uint32_t taken = 0;
#pragma unroll
    for (int j = 0; j < EPL; ++j) if (lane + 32 * j >= n_expert) taken |= 1u << j;
    float sum = 0.0f;
    for (int r = 0; r < n_used; ++r) {
        float bv = -INFINITY; int bi = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < EPL; ++j)   // ascending ids within the lane: strict '>' keeps the lower one
            if (!((taken >> j) & 1u) && (bi == 0x7fffffff || v[j] > bv)) { bv = v[j]; bi = lane + 32 * j; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
        ids[r] = bi; wts[r] = bv;
        sum += bv;                      // summed in pick order (src/ops/mod.rs:1211)
    }
    float denom = fmaxf(sum, 6.103515625e-5f);
    for (int r = 0; r < n_used; ++r) wts[r] = wts[r] / denom;
}
__device__ __forceinline__ void warp_topk_any(const float* p, int n_expert, int n_used, int32_t* ids, float* wts) {
    if (n_expert <= 32) warp_topk<1>(p, n_expert, n_used, ids, wts);
    else if (n_expert <= 128) warp_topk<4>(p, n_expert, n_used, ids, wts);
    else if (n_expert <= 256) warp_topk<8>(p, n_expert, n_used, ids, wts);
    else if (n_expert <= 512) warp_topk<16>(p, n_expert, n_used, ids, wts);
    else warp_topk<32>(p, n_expert, n_used, ids, wts);
}

__global__ void k_route(const float* probs, int n_expert, int n_used, int32_t* ids, float* wts) {
    __shared__ float sval[32];
    __shared__ int sidx[32];
    size_t t = blockIdx.x;
    block_topk(probs + t * n_expert, n_expert, n_used, ids + t * n_used, wts + t * n_used, sval, sidx);
}

// Weighted expert sum + gated shared expert (src/ops/mod.rs:1134-1171): ascending picks, shared last.
__global__ void k_moe_finish(float* out, size_t at, int n, const float* rows, const float* wts, int n_used, size_t n_tok,
                             const float* shared, const float* logit, size_t logit_at) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tok * n) return;
    size_t t = i / n; int j = (int)(i % n);
    float g = sigmoid_f(logit[logit_at + t]);
    float v = 0.0f;
    for (int e = 0; e < n_used; ++e) v += wts[t * n_used + e] * rows[(t * n_used + e) * n + j];
    v += shared[t * n + j] * g;
    out[at + t * n + j] = v;
}

// Q8_0 activation quantiser, block per row of n_in (src/ops/naive.rs:653-675).
__global__ void k_quant_q8(const float* x, int n_in, int8_t* xq, float* xs) {
    size_t t = blockIdx.x;
    block_quant_q8(x + t * n_in, n_in, xq + t * n_in, xs + t * (n_in / 32));
}

// ---- op-level matmuls: grid (row blocks, tokens or pairs) ----
__global__ void k_matmul_q8(DevQ8 w, const int8_t* xq_g, const float* xs_g, float* out) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int RP = 4;
    int nb = w.n_in / 32, gsh = lanes_shift(nb);
    int8_t* xq = (int8_t*)smem;
    float* xs = (float*)(smem + w.n_in);
    float* terms = xs + nb + (threadIdx.x >> 5) * terms_floats(RP, gsh, nb);
    size_t t = blockIdx.y;
    for (int i = threadIdx.x; i < w.n_in / 16; i += blockDim.x) ((uint4*)xq)[i] = ((const uint4*)(xq_g + t * w.n_in))[i];
    for (int i = threadIdx.x; i < nb; i += blockDim.x) xs[i] = xs_g[t * nb + i];
    __syncthreads();
    int b0, b1, r0, r1;
    share(w.n_out, gridDim.x, blockIdx.x, b0, b1);
    share(b1 - b0, blockDim.x >> 5, threadIdx.x >> 5, r0, r1);
    float* o = out + t * w.n_out;
    q8_rows<RP>(w, b0 + r0, b0 + r1, xq, xs, terms, gsh, [&](int row, float v) { o[row] = v; });
}

// NVFP4 rows for (token,pick) pairs: pair i uses expert ids[i] (or expert 0 when ids is null), activation row
// x_row(i) and writes out row i, times the expert's second scale (src/ops/mod.rs:1049-1088).
__global__ void k_matmul_fp4(DevFp4 w, const int32_t* ids, int n_used, int rows_mode, const int8_t* xq_g, const float* xs_g, float* out) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int RP = 4;
    int nb = w.n_in / 32, nsb = w.n_in / 16, gsh = lanes_shift(nb);
    int8_t* xq = (int8_t*)smem;
    float* xs = (float*)(smem + w.n_in);
    float* terms = xs + nb + (threadIdx.x >> 5) * terms_floats(RP, gsh, nsb);
    size_t i = blockIdx.y;
    int e = ids ? ids[i] : 0;
    size_t xr = rows_mode == 0 ? i : rows_mode == 1 ? i / n_used : 0;  // rows==picks / rows==n_tok / single row
    for (int k = threadIdx.x; k < w.n_in / 16; k += blockDim.x) ((uint4*)xq)[k] = ((const uint4*)(xq_g + xr * w.n_in))[k];
    for (int k = threadIdx.x; k < nb; k += blockDim.x) xs[k] = xs_g[xr * nb + k];
    __syncthreads();
    int el = e - w.expert_lo;
    if (el < 0 || el >= w.n_expert) return;  // not stored on this device (expert-parallel shard)
    const uint8_t* nib = w.nib + (size_t)el * w.n_out * (w.n_in / 2);
    const uint8_t* sc = w.sc + (size_t)el * w.n_out * nsb;
    float s2 = w.scale2 ? w.scale2[el] : 1.0f;
    bool has_s2 = w.scale2 != nullptr;
    int b0, b1, r0, r1;
    share(w.n_out, gridDim.x, blockIdx.x, b0, b1);
    share(b1 - b0, blockDim.x >> 5, threadIdx.x >> 5, r0, r1);
    float* o = out + i * w.n_out;
    fp4_rows<RP>(nib, sc, w.n_in, b0 + r0, b0 + r1, xq, xs, terms, gsh, [&](int row, float v) { o[row] = has_s2 ? v * s2 : v; });
}

// Multi-token matmuls on the int8 MMA path: grid (row tiles, token tiles of 32). A warp owns 16 rows and NJ of
// the tile's 4 groups of 8 tokens: NJ=4, 8 warps and 128 rows per block when there are many token tiles (prefill);
// NJ=1, 16 warps and 64 rows per block for one token tile (batched decode), where the only other source of
// parallelism is the rows and 4x the warps keep 4x the weight bytes in flight.
// mode 0: out[t][row] = v; mode 1: out[t][row] += v (residual add).
template <int NJ>
__global__ void __launch_bounds__(NJ == 4 ? 256 : 512) k_gemm_q8(DevQ8 w, const int8_t* xq, const float* xs, int n_tok, float* out, size_t out_stride, int mode) {
    extern __shared__ __align__(16) unsigned char smem[];
    int8_t* sq = (int8_t*)smem;
    float* ss = (float*)(sq + (size_t)MMA_TOK * mma_act_stride(w.n_in));
    const int wid = threadIdx.x >> 5;
    const int t0 = blockIdx.y * MMA_TOK;
    const int r0 = NJ == 4 ? blockIdx.x * MMA_ROWS + wid * 16 : blockIdx.x * 64 + (wid >> 2) * 16, jb = NJ == 4 ? 0 : (wid & 3);
    mma_stage_act(xq, xs, w.n_in, t0, n_tok, sq, ss);
    if (r0 >= w.n_out || t0 + 8 * jb >= n_tok) return;
    float acc[NJ][4];
    mma_q8_rows16<NJ, NJ == 4 ? 4 : 8>(w, r0, sq, ss, jb, acc);
    mma_foreach<NJ>(acc, r0, w.n_out, jb, [&](int t, int row, float v) {
        if (t0 + t < n_tok) { float* o = out + (size_t)(t0 + t) * out_stride + row; *o = mode ? *o + v : v; }
    });
}
// Dense NVFP4 matrix (one expert), 128 rows x 32 tokens per block; `s2` multiplies the result when has_s2 (the
// tensor's second scale).
__global__ void __launch_bounds__(256) k_gemm_fp4(const uint8_t* nib, const uint8_t* sc, int k, int n_rows, const int8_t* xq, const float* xs,
                                                  int n_tok, float* out, size_t out_stride, float s2, int has_s2) {
    extern __shared__ __align__(16) unsigned char smem[];
    int8_t* sq = (int8_t*)smem;
    float* ss = (float*)(sq + (size_t)MMA_TOK * mma_act_stride(k));
    const int t0 = blockIdx.y * MMA_TOK, r0 = blockIdx.x * MMA_ROWS + (threadIdx.x >> 5) * 16;
    mma_stage_act(xq, xs, k, t0, n_tok, sq, ss);
    if (r0 >= n_rows) return;
    float acc[4][4];
    mma_fp4_rows16<4, 8>(nib, sc, k, n_rows, r0, sq, ss, 0, acc);
    mma_foreach<4>(acc, r0, n_rows, 0, [&](int t, int row, float v) {
        if (t0 + t < n_tok) out[(size_t)(t0 + t) * out_stride + row] = has_s2 ? v * s2 : v;
    });
}
static inline size_t gemm_smem(int k) { return (size_t)MMA_TOK * mma_act_stride(k) + (size_t)MMA_TOK * (k / 32) * 4; }

template <bool EXACT>
__global__ void k_matmul_f32(DevF32 w, const float* x, float* out) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* xs = (float*)smem;
    float* tile = xs + w.n_in + (threadIdx.x >> 5) * (32 * 33);
    size_t t = blockIdx.y;
    for (int i = threadIdx.x; i < w.n_in; i += blockDim.x) xs[i] = x[t * w.n_in + i];
    __syncthreads();
    int b0, b1, r0, r1;
    share(w.n_out, gridDim.x, blockIdx.x, b0, b1);
    int nw = blockDim.x >> 5, wid = threadIdx.x >> 5;
    share(b1 - b0, nw, wid, r0, r1);
    float* o = out + t * w.n_out;
    f32_rows<EXACT>(w.w, w.n_in, b0 + r0, b0 + r1, xs, tile, [&](int row, float v) { o[row] = v; }, 32 * 33);
}

// ---- attention, split over positions (flash-decoding form; tolerance class like the reference's
// device kernels, kernels/attention.cuh:61-195 there) ----
// grid (n_head_kv, n_q, n_split); block 256. Each warp walks positions p0+warp, +8, ...; a lane owns
// hd/32 contiguous dims; all `group` query heads of the kv head are scored against each K row read.
// Partials: m, l per (t, head, split) and acc[hd].
constexpr int ATTN_MIN_SPLIT = 64;   // a split never covers fewer positions than this (short contexts use few splits)
template <int HD, int MAXG>
__global__ void k_attn_partial(const float* q, const uint16_t* kslab, const uint16_t* vslab, int kv_dim, int n_pos_last, int n_q,
                               int n_head, int n_head_kv, float scale, int bf16, const int* n_pos_dev,
                               float* part_acc, float* part_ml, int rows_per_seq = 0, size_t slab_stride = 0) {
    constexpr int DPL = HD / 32;  // dims per lane
    int hk = blockIdx.x, t = blockIdx.y, sp = blockIdx.z, n_split = gridDim.z;
    pdl_trigger(); pdl_wait();
    if (rows_per_seq > 0) {       // rows of several sequences in one launch: row t reads the slabs of sequence t / rows_per_seq
        const size_t so = (size_t)(t / rows_per_seq) * slab_stride;
        kslab += so; vslab += so;
    }
    int group = n_head / n_head_kv;
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int n_pos = n_pos_dev ? n_pos_dev[t] : n_pos_last - n_q + 1 + t;
    int per = max(ATTN_MIN_SPLIT, (n_pos + n_split - 1) / n_split);
    int p0 = sp * per, p1 = min(n_pos, p0 + per);
    if (p0 >= p1) {   // no positions in this split: neutral partials
        for (int idx = threadIdx.x; idx < group * HD; idx += blockDim.x) {
            size_t o = (((size_t)t * n_head + hk * group + idx / HD) * n_split + sp);
            part_acc[o * HD + idx % HD] = 0.0f;
            if (idx % HD == 0) { part_ml[o * 2] = -INFINITY; part_ml[o * 2 + 1] = 0.0f; }
        }
        return;
    }
    float qr[MAXG][DPL];
#pragma unroll
    for (int g = 0; g < MAXG; ++g)
#pragma unroll
        for (int d = 0; d < DPL; ++d)
            qr[g][d] = g < group ? q[((size_t)t * n_head + hk * group + g) * HD + lane * DPL + d] : 0.0f;
    float m[MAXG], l[MAXG], acc[MAXG][DPL];
#pragma unroll
    for (int g = 0; g < MAXG; ++g) { m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[g][d] = 0.0f; }
    constexpr int PU = 4;   // positions per trip: their K and V rows are all requested before the first is used
    for (int pb = p0 + wid; pb < p1; pb += PU * nw) {
        uint16_t kb[PU][DPL], vb[PU][DPL];
#pragma unroll
        for (int u = 0; u < PU; ++u) {
            const int p = pb + u * nw;
            if (p < p1) {
                const uint16_t* kr = kslab + (size_t)p * kv_dim + hk * HD + lane * DPL;
                const uint16_t* vr = vslab + (size_t)p * kv_dim + hk * HD + lane * DPL;
                if (DPL == 8) { *(uint4*)kb[u] = *(const uint4*)kr; *(uint4*)vb[u] = *(const uint4*)vr; }
                else if (DPL == 4) { *(uint2*)kb[u] = *(const uint2*)kr; *(uint2*)vb[u] = *(const uint2*)vr; }
                else { *(uint32_t*)kb[u] = *(const uint32_t*)kr; *(uint32_t*)vb[u] = *(const uint32_t*)vr; }
            }
        }
#pragma unroll
        for (int u = 0; u < PU; ++u) {
            if (pb + u * nw >= p1) break;
            float kf[DPL], vf[DPL];
#pragma unroll
            for (int d = 0; d < DPL; ++d) {
                kf[d] = bf16 ? bf16_bits_to_f32(kb[u][d]) : f16_bits_to_f32(kb[u][d]);
                vf[d] = bf16 ? bf16_bits_to_f32(vb[u][d]) : f16_bits_to_f32(vb[u][d]);
            }
#pragma unroll
            for (int g = 0; g < MAXG; ++g) {
                if (g < group) {
                    float s = 0.0f;
#pragma unroll
                    for (int d = 0; d < DPL; ++d) s += qr[g][d] * kf[d];
                    s = warp_sum(s) * scale;
                    float mn = fmaxf(m[g], s);
                    float corr = __expf(m[g] - mn), pw = __expf(s - mn);
                    l[g] = l[g] * corr + pw;
#pragma unroll
                    for (int d = 0; d < DPL; ++d) acc[g][d] = acc[g][d] * corr + pw * vf[d];
                    m[g] = mn;
                }
            }
        }
    }
    // merge the block's warps through shared memory
    extern __shared__ __align__(16) unsigned char smem[];
    float* s_ml = (float*)smem;              // [nw][MAXG][2]
    float* s_acc = s_ml + nw * MAXG * 2;     // [nw][MAXG][HD]
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
        if (lane == 0) { s_ml[(wid * MAXG + g) * 2] = m[g]; s_ml[(wid * MAXG + g) * 2 + 1] = l[g]; }
#pragma unroll
        for (int d = 0; d < DPL; ++d) s_acc[(wid * MAXG + g) * HD + lane * DPL + d] = acc[g][d];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * HD; idx += blockDim.x) {
        int g = idx / HD, d = idx % HD;
        float M = -INFINITY;
        for (int w = 0; w < nw; ++w) M = fmaxf(M, s_ml[(w * MAXG + g) * 2]);
        float L = 0.0f, A = 0.0f;
        for (int w = 0; w < nw; ++w) {
            float mw = s_ml[(w * MAXG + g) * 2];
            float c = mw == -INFINITY ? 0.0f : __expf(mw - M);
            L += s_ml[(w * MAXG + g) * 2 + 1] * c;
            A += s_acc[(w * MAXG + g) * HD + d] * c;
        }
        size_t o = (((size_t)t * n_head + hk * group + g) * n_split + sp);
        part_acc[o * HD + d] = A;
        if (d == 0) { part_ml[o * 2] = M; part_ml[o * 2 + 1] = L; }
    }
}

// Combine the splits; optional output gate sigmoid(gate) fused (src/model/qwen35.rs:1216-1218).
// grid (n_q * n_head); block HD threads.
__global__ void k_attn_combine(const float* part_acc, const float* part_ml, int n_split, int hd, const float* gate, float* out) {
    size_t th = blockIdx.x;
    int d = threadIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < n_split; ++s) M = fmaxf(M, part_ml[(th * n_split + s) * 2]);
    float L = 0.0f, A = 0.0f;
    for (int s = 0; s < n_split; ++s) {
        float ms = part_ml[(th * n_split + s) * 2];
        float c = ms == -INFINITY ? 0.0f : __expf(ms - M);
        L += part_ml[(th * n_split + s) * 2 + 1] * c;
        A += part_acc[(th * n_split + s) * hd + d] * c;
    }
    float v = A / L;
    if (gate) v *= sigmoid_f(gate[th * hd + d]);
    out[th * hd + d] = v;
}

}  // namespace
