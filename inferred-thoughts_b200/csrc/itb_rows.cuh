// Kernels of the engine's multi-row path: several tokens at once, either one token of each of many sequences
// (batched decode) or many consecutive tokens of one sequence (prefill). Rows are token-major; row i belongs to
// sequence i / n_tok and is its token number i % n_tok of this pass. Matmuls run on the int8 MMA kernels
// (itb_mma.cuh, every weight row read once per 32 rows); the kernels here are the rest of a layer. All keep the
// CPU path's arithmetic order, so a prefill is bit-identical to feeding the tokens one at a time, which the
// reference asserts of its own backends (tests/qwen35.rs:94-139 there).
#pragma once
#include "itb_kernels.cuh"

namespace {

// RMSNorm + Q8_0 quantisation of each row (src/ops/naive.rs:139-152, :653-675): normalised f32 row, int8 quants,
// scales. grid = rows, block 256.
__global__ void __launch_bounds__(256) k_norm_quant(const float* x, const float* w, int n, float eps, float* xn_out, int8_t* xq, float* xs) {
    extern __shared__ __align__(16) unsigned char smem[];
    double* red = (double*)smem;
    float* xn = (float*)(red + 32);
    const size_t r = blockIdx.x;
    block_rms_norm(x + r * n, w, n, eps, xn, red);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b = wid; b < n / 32; b += nw) {
        float v = xn[b * 32 + lane], d;
        xq[r * n + b * 32 + lane] = warp_quant_q8(v, &d);
        if (lane == 0) xs[r * (n / 32) + b] = d;
        if (xn_out) xn_out[r * n + b * 32 + lane] = v;
    }
}

// Depthwise causal conv over the tokens of each sequence in order (src/ops/naive.rs:275-315); writes the
// PRE-activation sum in place and leaves the window advanced. grid (ceil(nc/128), n_seq).
__global__ void k_conv_rows(float* state, size_t state_stride, float* x, int n_tok, int nc, const float* w, int kernel) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (c >= nc) return;
    const int keep = kernel - 1;
    float* st = state + (size_t)s * state_stride + (size_t)c * keep;
    float past[8], wt[8];
    for (int k = 0; k < keep; ++k) past[k] = st[k];
    for (int k = 0; k < kernel; ++k) wt[k] = w[(size_t)c * kernel + k];
    for (int t = 0; t < n_tok; ++t) {
        float* px = x + ((size_t)s * n_tok + t) * nc + c;
        const float xv = *px;
        float sum = 0.0f;
        for (int k = 0; k < keep; ++k) sum += past[k] * wt[k];
        sum += xv * wt[keep];
        *px = sum;
        for (int k = 0; k + 1 < keep; ++k) past[k] = past[k + 1];
        past[keep - 1] = xv;
    }
    for (int k = 0; k < keep; ++k) st[k] = past[k];
}

// Everything of the GatedDeltaNet block that does not depend on the state, per row: SiLU of the conv sums,
// l2-norm of q and k (q also scaled by 1/sqrt(sk)), the decay g and the write strength beta
// (src/model/qwen35.rs:1280-1316, src/ops/naive.rs:101-107, :254-273). grid (rows, 2*n_k + n_v), block sk.
__global__ void k_gdn_pre(const float* conv, int cd, const float* alpha, const float* beta, const float* ssm_a, const float* dt_bias,
                          int sk, int n_k, int n_v, float eps, float* qh, float* kh, float* vh, float* gb) {
    __shared__ double red[8];
    const size_t r = blockIdx.x;
    const int u = blockIdx.y, d = threadIdx.x, key_dim = n_k * sk;
    const float* cv = conv + r * cd;
    if (u < 2 * n_k) {
        const bool is_q = u < n_k;
        const int h = is_q ? u : u - n_k;
        float v = silu_f(cv[(is_q ? 0 : key_dim) + h * sk + d]);
        double acc = warp_sum_d((double)(v * v));
        if ((d & 31) == 0) red[d >> 5] = acc;
        __syncthreads();
        double tot = 0.0;
        for (int w = 0; w < sk / 32; ++w) tot += red[w];
        float sc = 1.0f / fmaxf(sqrtf((float)tot), eps);
        v = v * sc;
        if (is_q) v = v * (1.0f / sqrtf((float)sk));
        (is_q ? qh : kh)[(r * n_k + h) * sk + d] = v;
    } else {
        const int h = u - 2 * n_k;
        vh[(r * n_v + h) * sk + d] = silu_f(cv[2 * key_dim + h * sk + d]);
        if (d == 0) {
            float a = alpha[r * n_v + h] + dt_bias[h];
            float sp = a > 20.0f ? a : log_f(1.0f + exp_f(a));
            gb[(r * n_v + h) * 2] = exp_f(sp * ssm_a[h]);
            gb[(r * n_v + h) * 2 + 1] = sigmoid_f(beta[r * n_v + h]);
        }
    }
}

// The recurrence itself (src/ops/naive.rs:109-132): block = (value head, slice of ROWS value rows, sequence), one
// thread per value row, keys walked serially, the slice of state held in shared memory across the pass's tokens.
template <int ROWS>
__global__ void k_gdn_scan(const float* qh, const float* kh, const float* vh, const float* gb, int n_tok, int sk, int n_k, int n_v,
                           float* state, size_t state_stride, float* out) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* S = (float*)smem;             // [ROWS][sk+1]
    float* kq = S + ROWS * (sk + 1);     // k[sk] | q[sk]
    const int h = blockIdx.x, j0 = blockIdx.y * ROWS, s = blockIdx.z, khd = h % n_k, tid = threadIdx.x;
    float* sg = state + (size_t)s * state_stride + ((size_t)h * sk + j0) * sk;
    for (int i = tid; i < ROWS * sk; i += blockDim.x) S[(i / sk) * (sk + 1) + i % sk] = sg[i];
    for (int t = 0; t < n_tok; ++t) {
        const size_t r = (size_t)s * n_tok + t;
        __syncthreads();
        for (int i = tid; i < sk; i += blockDim.x) {
            kq[i] = kh[(r * n_k + khd) * sk + i];
            kq[sk + i] = qh[(r * n_k + khd) * sk + i];
        }
        __syncthreads();
        if (tid < ROWS) {
            const float g = gb[(r * n_v + h) * 2], b = gb[(r * n_v + h) * 2 + 1];
            float* row = S + tid * (sk + 1);
            float pred = 0.0f;
#pragma unroll 4
            for (int i = 0; i < sk; ++i) { float v = row[i] * g; row[i] = v; pred += v * kq[i]; }
            const float d = b * (vh[(r * n_v + h) * sk + j0 + tid] - pred);
            float o = 0.0f;
#pragma unroll 4
            for (int i = 0; i < sk; ++i) { float v = row[i] + kq[i] * d; row[i] = v; o += v * kq[sk + i]; }
            out[(r * n_v + h) * sk + j0 + tid] = o;
        }
    }
    __syncthreads();
    for (int i = tid; i < ROWS * sk; i += blockDim.x) sg[i] = S[(i / sk) * (sk + 1) + i % sk];
}

// Gated RMSNorm of the recurrence's output, the SiLU(z) gate and the Q8_0 quantisation of the result
// (src/model/qwen35.rs:1319-1325). grid (rows, n_v), block sv.
__global__ void k_gdn_post(const float* o, const float* z, const float* norm_w, int sv, int n_v, float eps, int8_t* out_q, float* out_s) {
    __shared__ double red[8];
    const size_t r = blockIdx.x;
    const int h = blockIdx.y, d = threadIdx.x;
    const size_t idx = (r * n_v + h) * sv + d;
    const float v = o[idx];
    double acc = warp_sum_d((double)(v * v));
    if ((d & 31) == 0) red[d >> 5] = acc;
    __syncthreads();
    double tot = 0.0;
    for (int w = 0; w < sv / 32; ++w) tot += red[w];
    const float mean = (float)(tot / (double)sv);
    const float sc = 1.0f / sqrtf(mean + eps);
    const float core = v * sc * norm_w[d];
    const float val = silu_f(z[idx]) * core;
    float dq;
    const int8_t q = warp_quant_q8(val, &dq);
    out_q[idx] = q;
    if ((d & 31) == 0) out_s[idx / 32] = dq;
}

// Attention prologue per (row, head): as k_attn_prep, the row's sequence and position derived from the pass
// shape: sequence = row / n_tok, position = pos[sequence] + row % n_tok. grid (n_head + 2*n_head_kv, rows).
struct AttnPrepRows {
    const float* qg; const float* k; const float* v;
    const float* q_norm; const float* k_norm;
    float* q_out; float* g_out;
    uint16_t* kslab; uint16_t* vslab; size_t slab_stride;
    const int* pos; int* npos_out; int n_tok;
    int hd, n_head, n_head_kv, n_rot; float theta, eps; int bf16;
};
__global__ void k_attn_prep_rows(AttnPrepRows p) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* val = (float*)smem;
    __shared__ double red[8];
    const int job = blockIdx.x, d = threadIdx.x, hd = p.hd, kvd = p.n_head_kv * hd;
    const size_t r = blockIdx.y;
    const int s = (int)(r / p.n_tok), pos = p.pos[s] + (int)(r % p.n_tok);
    if (job == 0 && d == 0) p.npos_out[r] = pos + 1;
    const bool is_q = job < p.n_head, is_k = !is_q && job < p.n_head + p.n_head_kv;
    const int hk = is_q ? job : is_k ? job - p.n_head : job - p.n_head - p.n_head_kv;
    float v;
    if (is_q) {
        v = p.qg[r * 2 * hd * p.n_head + (size_t)hk * 2 * hd + d];
        p.g_out[(r * p.n_head + hk) * hd + d] = p.qg[r * 2 * hd * p.n_head + (size_t)hk * 2 * hd + hd + d];
    } else {
        v = (is_k ? p.k : p.v)[r * kvd + hk * hd + d];
    }
    if (is_q || is_k) {
        double acc = warp_sum_d((double)(v * v));
        if ((d & 31) == 0) red[d >> 5] = acc;
        __syncthreads();
        double tot = 0.0;
        for (int w = 0; w < hd / 32; ++w) tot += red[w];
        float mean = (float)(tot / (double)hd);
        float sc = 1.0f / sqrtf(mean + p.eps);
        v = v * sc * (is_q ? p.q_norm : p.k_norm)[d];
        val[d] = v;
        __syncthreads();
        const int half = p.n_rot / 2;
        if (d < half) {
            double freq = pow((double)p.theta, -2.0 * (double)d / (double)p.n_rot);
            double th = (double)pos * freq;
            float sn = (float)sin(th), cs = (float)cos(th);
            float x0 = val[d], x1 = val[d + half];
            val[d] = x0 * cs - x1 * sn;
            val[d + half] = x0 * sn + x1 * cs;
        }
        __syncthreads();
        v = val[d];
    }
    if (is_q) p.q_out[(r * p.n_head + hk) * hd + d] = v;
    else {
        uint16_t* slab = (is_k ? p.kslab : p.vslab) + (size_t)s * p.slab_stride + (size_t)pos * kvd + hk * hd + d;
        *slab = p.bf16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v);
    }
}

// Combine of the attention splits per (row, head) with the sigmoid gate and Q8_0 quantisation; positions per row.
__global__ void k_attn_combine_rows(const float* part_acc, const float* part_ml, int n_split, int hd, const float* gate,
                                    const int* n_pos_row, int n_head, int8_t* out_q, float* out_s) {
    const size_t th = blockIdx.x;
    const int d = threadIdx.x;
    const size_t r = th / n_head;
    const int n_pos = n_pos_row[r], per = max(ATTN_MIN_SPLIT, (n_pos + n_split - 1) / n_split), n_act = (n_pos + per - 1) / per;
    float M = -INFINITY;
    for (int s = 0; s < n_act; ++s) M = fmaxf(M, part_ml[(th * n_split + s) * 2]);
    float L = 0.0f, A = 0.0f;
    for (int s = 0; s < n_act; ++s) {
        float ms = part_ml[(th * n_split + s) * 2];
        float c = ms == -INFINITY ? 0.0f : __expf(ms - M);
        L += part_ml[(th * n_split + s) * 2 + 1] * c;
        A += part_acc[(th * n_split + s) * hd + d] * c;
    }
    float v = A / L;
    v *= sigmoid_f(gate[th * hd + d]);
    float dq;
    int8_t q = warp_quant_q8(v, &dq);
    out_q[th * hd + d] = q;
    if ((d & 31) == 0) out_s[(th * hd + d) / 32] = dq;
}

__global__ void k_advance_pos(int* pos, int n_seq, int by) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_seq) pos[i] += by;
}
// Rows of the last token of each sequence, gathered for the LM head: out[s] = x[s*n_tok + n_tok-1].
__global__ void k_gather_last(const float* x, int n, int n_tok, float* out) {
    const int s = blockIdx.x;
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[(size_t)s * n + i] = x[((size_t)s * n_tok + n_tok - 1) * n + i];
}

}  // namespace
