// Attention in the CPU path's own order (src/ops/naive.rs:420-466): per (query row, kv head) the scores are left-fold dot
// products over the head dimension, the softmax subtracts the maximum, sums its exponentials in position order and divides,
// and every output element is a left fold over the positions. None of that is reassociated here, so the result equals the
// CPU's bit for bit (the exponential is the C library's, itb_internal.cuh); the parallelism is across positions for the
// scores, across (head, dimension) for the outputs, with the inherently serial chains (head_dim adds per score, n_pos adds
// per softmax sum, n_pos multiply-adds per output) one thread each. Selected by exact=1; exact=0 keeps the split-K kernels,
// which reassociate the sums (tolerance class) and are faster at long contexts.
#pragma once
#include "itb_kernels.cuh"

namespace {

constexpr int AX_TP = 64;          // positions per block of the scores kernel
constexpr int AX_QSTRIDE_PAD = 4;  // q rows in shared memory are head_dim + 4 floats apart: the heads of a group hit different banks

__device__ __forceinline__ float kv_elem(uint32_t word, int hi, int bf16) {
    const uint16_t h = (uint16_t)(word >> (hi * 16));
    return bf16 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h);
}

// scores[row][head][s] = (sum_i q[i] * k_s[i], i ascending) * scale for s < n_pos(row).
// grid (ceil(n_pos_max / AX_TP), n_head_kv, rows); block AX_TP * group threads: thread = (position in tile, head of the group).
struct AxScores {
    const float* q; const uint16_t* kslab; size_t slab_stride; int rows_per_seq;   // q [rows][n_head][hd]; row r reads the slab of sequence r / rows_per_seq
    const int* n_pos_dev; int n_pos_last, n_q;                                      // per-row positions, or n_pos_last - n_q + 1 + row
    int kv_dim, hd, n_head, n_head_kv; float scale; int bf16;
    float* scores; int s_stride;                                                    // [rows][n_head][s_stride]
};
__global__ void k_attn_scores_exact(AxScores p) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* qs = (float*)smem;                                    // [group][hd + pad]
    const int hk = blockIdx.y, r = blockIdx.z, hd = p.hd, group = p.n_head / p.n_head_kv, qst = hd + AX_QSTRIDE_PAD;
    pdl_trigger(); pdl_wait();
    const int n_pos = p.n_pos_dev ? p.n_pos_dev[r] : p.n_pos_last - p.n_q + 1 + r;
    const int p0 = blockIdx.x * AX_TP;
    if (p0 >= n_pos) return;
    for (int i = threadIdx.x; i < group * hd; i += blockDim.x)
        qs[(i / hd) * qst + i % hd] = p.q[((size_t)r * p.n_head + hk * group) * hd + i];
    __syncthreads();
    const int g = threadIdx.x % group, s = p0 + threadIdx.x / group;
    if (s >= n_pos) return;
    const uint16_t* key = p.kslab + (size_t)(r / max(1, p.rows_per_seq)) * p.slab_stride + (size_t)s * p.kv_dim + hk * hd;
    const float* qg = qs + g * qst;
    float dot = 0.0f;
#pragma unroll 2
    for (int i = 0; i < hd; i += 8) {
        const uint4 kw = *(const uint4*)(key + i);
        const float4 q0 = *(const float4*)(qg + i), q1 = *(const float4*)(qg + i + 4);
        dot += q0.x * kv_elem(kw.x, 0, p.bf16); dot += q0.y * kv_elem(kw.x, 1, p.bf16);
        dot += q0.z * kv_elem(kw.y, 0, p.bf16); dot += q0.w * kv_elem(kw.y, 1, p.bf16);
        dot += q1.x * kv_elem(kw.z, 0, p.bf16); dot += q1.y * kv_elem(kw.z, 1, p.bf16);
        dot += q1.z * kv_elem(kw.w, 0, p.bf16); dot += q1.w * kv_elem(kw.w, 1, p.bf16);
    }
    p.scores[((size_t)r * p.n_head + hk * group + g) * p.s_stride + s] = dot * p.scale;
}

// Softmax of one (row, head)'s scores and the weighted sum of the values for 32 dimensions of that head.
// grid (hd / 32, n_head, rows); block 256: everyone on the softmax, then warp 0 walks the positions (a lane per dimension, one
// multiply-add chain each) over value tiles the other warps stage in shared memory one tile ahead.
// gate != null: times sigmoid(gate) (src/model/qwen35.rs:1216-1218); out_q != null: the result leaves quantised to Q8_0 (the
// output projection's own quantisation), else as f32 in out.
constexpr int AX_VT = 128;         // positions per staged value tile
struct AxOut {
    const float* scores; int s_stride;
    const uint16_t* vslab; size_t slab_stride; int rows_per_seq;
    const int* n_pos_dev; int n_pos_last, n_q;
    int kv_dim, hd, n_head, n_head_kv, bf16;
    const float* gate; float* out; int8_t* out_q; float* out_s;
    int weights_ready;             // the scores buffer already holds the softmax weights (k_attn_softmax_exact ran): skip the softmax here
};
__global__ void __launch_bounds__(256) k_attn_out_exact(AxOut p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float s_red[8];
    __shared__ float s_sum;
    const int j = blockIdx.x, h = blockIdx.y, r = blockIdx.z, hd = p.hd, group = p.n_head / p.n_head_kv, hk = h / group;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    pdl_trigger(); pdl_wait();
    const int n_pos = p.n_pos_dev ? p.n_pos_dev[r] : p.n_pos_last - p.n_q + 1 + r;
    float* w = (float*)smem;                                      // [n_pos] scores -> exponentials -> weights
    uint16_t* vt = (uint16_t*)(w + ((n_pos + 3) & ~3));           // [2][AX_VT][32]
    const float* sc = p.scores + ((size_t)r * p.n_head + h) * p.s_stride;
    const uint16_t* vbase = p.vslab + (size_t)(r / max(1, p.rows_per_seq)) * p.slab_stride + hk * hd + j * 32;
    auto stage = [&](int tile) {                                  // warps 1..7: tile `tile` of the values into its buffer
        const int s0 = tile * AX_VT, ns = min(AX_VT, n_pos - s0);
        uint16_t* dst = vt + (tile & 1) * AX_VT * 32;
        for (int i = tid - 32; i < ns * 4; i += 224) {            // 4 x 16 bytes per position
            const int s = i >> 2, q = i & 3;
            *(uint4*)(dst + s * 32 + q * 8) = *(const uint4*)(vbase + (size_t)(s0 + s) * p.kv_dim + q * 8);
        }
    };
    if (wid > 0 && n_pos > 0) stage(0);
    if (p.weights_ready) {
        for (int s = tid; s < n_pos; s += 256) w[s] = sc[s];
    } else {
        float mx = -INFINITY;
        for (int s = tid; s < n_pos; s += 256) { const float v = sc[s]; w[s] = v; mx = fmaxf(mx, v); }
        mx = warp_max(mx);
        if (lane == 0) s_red[wid] = mx;
        __syncthreads();
        mx = s_red[0];
        for (int k = 1; k < 8; ++k) mx = fmaxf(mx, s_red[k]);
        for (int s = tid; s < n_pos; s += 256) w[s] = exp_f(w[s] - mx);
        __syncthreads();
        if (tid == 0) {                                               // the sum in position order
            float sum = 0.0f;
            int s = 0;
            for (; s + 4 <= n_pos; s += 4) { const float4 e = *(const float4*)(w + s); sum += e.x; sum += e.y; sum += e.z; sum += e.w; }
            for (; s < n_pos; ++s) sum += w[s];
            s_sum = sum;
        }
        __syncthreads();
        {
            const float sum = s_sum;
            for (int s = tid; s < n_pos; s += 256) w[s] /= sum;
        }
    }
    __syncthreads();
    float o = 0.0f;
    const int n_tiles = (n_pos + AX_VT - 1) / AX_VT;
    for (int t = 0; t < n_tiles; ++t) {
        if (wid > 0) { if (t + 1 < n_tiles) stage(t + 1); }
        else {
            const int s0 = t * AX_VT, ns = min(AX_VT, n_pos - s0);
            const uint16_t* src = vt + (t & 1) * AX_VT * 32 + lane;
            const float* ws = w + s0;
#pragma unroll 8
            for (int s = 0; s < ns; ++s) {
                const uint16_t hb = src[s * 32];
                o += ws[s] * (p.bf16 ? bf16_bits_to_f32(hb) : f16_bits_to_f32(hb));
            }
        }
        __syncthreads();
    }
    if (wid == 0) {
        const size_t idx = ((size_t)r * p.n_head + h) * hd + j * 32 + lane;
        if (p.gate) o *= sigmoid_f(p.gate[idx]);
        if (p.out_q) {
            float dq;
            const int8_t q = warp_quant_q8(o, &dq);
            p.out_q[idx] = q;
            if (lane == 0) p.out_s[idx / 32] = dq;
        } else p.out[idx] = o;
    }
}
// The softmax of one (row, head)'s scores on its own, in place (many-row passes: the eight blocks that share a head's weights in
// k_attn_out_exact would each recompute them, and the library-exact exponential is the expensive part): maximum, exponentials,
// the sum in position order by one thread, the division. grid (n_head, rows), block 256; dynamic shared memory n_pos_max floats.
struct AxSoft { float* scores; int s_stride; const int* n_pos_dev; int n_pos_last, n_q, n_head; };
__global__ void __launch_bounds__(256) k_attn_softmax_exact(AxSoft p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float s_red[8];
    __shared__ float s_sum;
    float* w = (float*)smem;
    const int h = blockIdx.x, r = blockIdx.y, tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int n_pos = p.n_pos_dev ? p.n_pos_dev[r] : p.n_pos_last - p.n_q + 1 + r;
    float* sc = p.scores + ((size_t)r * p.n_head + h) * p.s_stride;
    float mx = -INFINITY;
    for (int s = tid; s < n_pos; s += 256) { const float v = sc[s]; w[s] = v; mx = fmaxf(mx, v); }
    mx = warp_max(mx);
    if (lane == 0) s_red[wid] = mx;
    __syncthreads();
    mx = s_red[0];
    for (int k = 1; k < 8; ++k) mx = fmaxf(mx, s_red[k]);
    for (int s = tid; s < n_pos; s += 256) w[s] = exp_f(w[s] - mx);
    __syncthreads();
    if (tid == 0) {
        float sum = 0.0f;
        int s = 0;
        for (; s + 4 <= n_pos; s += 4) { const float4 e = *(const float4*)(w + s); sum += e.x; sum += e.y; sum += e.z; sum += e.w; }
        for (; s < n_pos; ++s) sum += w[s];
        s_sum = sum;
    }
    __syncthreads();
    const float sum = s_sum;
    for (int s = tid; s < n_pos; s += 256) sc[s] = w[s] / sum;
}
inline size_t attn_out_exact_smem(int n_pos_max) { return (size_t)((n_pos_max + 3) & ~3) * 4 + 2 * AX_VT * 32 * 2; }
inline size_t attn_scores_exact_smem(int hd, int group) { return (size_t)group * (hd + AX_QSTRIDE_PAD) * 4; }

}  // namespace
