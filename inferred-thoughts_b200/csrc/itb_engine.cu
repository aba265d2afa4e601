// Model + engine level: the token loop as a short chain of fused kernels replayed as one CUDA graph.
//
// Restates, natively, what the reference drives through its op seam: Qwen35::forward
// (src/model/qwen35.rs:956-1127), the attention block (:1138-1223), the GatedDeltaNet block
// (:1232-1328), the routed FFN (:1587-1699) and Engine::{prefill,decode,generate}
// (src/engine/mod.rs:352-437). The arithmetic of every matmul, norm, conv, delta-rule and routing
// step keeps the CPU path's order; only exp() and the attention reduction are tolerance class.
#include <algorithm>
#include <memory>

#include "itb_kernels.cuh"
#include "synth_model.h"

void itb_attend_dev(itb_ctx* c, cudaStream_t st, const float* q, const uint16_t* k, const uint16_t* v, int kv_dim, int n_pos, int n_q,
                    int hd, int n_head, int n_head_kv, float scale, int bf16, const int* n_pos_dev, const float* gate,
                    float* part_acc, float* part_ml, int n_split, float* out);
void itb_synth_f32(cudaStream_t st, uint64_t key, size_t n, int dist, float sd, float* out);
void itb_synth_q8_raw(cudaStream_t st, uint64_t key, size_t n_blocks, int dist, float sd, uint8_t* raw);
void itb_synth_fp4_raw(cudaStream_t st, uint64_t key, size_t per_expert, size_t e_lo, size_t e_hi, int dist, float sd,
                       unsigned* amax_tmp, float* scale2, uint8_t* raw);

// =====================================================================================================
// Fused kernels
// =====================================================================================================
struct InProj {
    const float* x; int x_stride;                 // [B][n_embd] residual stream (or embedding rows)
    const float* norm_w; float eps; int n_embd;
    int nq; DevQ8 q[3]; float* qout[3]; int qstride[3];
    int nf; DevF32 f[2]; float* fout[2]; int fstride[2];
    const float* conv_w; float* conv_state; int conv_kernel; size_t conv_state_stride;  // conv epilogue on q[0]
    int8_t* xq_out; float* xs_out;                // optional copy of the quantised normed row, [B][n_embd]
    int exact;
};

// RMSNorm + Q8_0 quantise prologue, then up to three Q8_0 matrices and two F32 matrices against the same
// row. Warps 0..nw-2 stream the Q8_0 rows; the last warp of a block takes one unit of F32 rows.
// With conv_w set, rows of q[0] go through the depthwise causal conv + SiLU (src/ops/naive.rs:275-315) in
// the epilogue, the lane that owns a row also advancing that channel's window.
__global__ void __launch_bounds__(288) k_in_proj(InProj p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int RP = 4;
    const int n = p.n_embd, nb = n / 32, gsh = lanes_shift(nb);
    double* red = (double*)smem;
    float* xn = (float*)(red + 32);
    int8_t* xq = (int8_t*)(xn + n);
    float* xs = (float*)(xq + n);
    float* scratch = xs + nb;
    const int b = blockIdx.y, wid = threadIdx.x >> 5, nw = blockDim.x >> 5, nwq = nw - 1;
    block_rms_norm(p.x + (size_t)b * p.x_stride, p.norm_w, n, p.eps, xn, red);
    block_quant_q8(xn, n, xq, xs);
    if (p.xq_out && blockIdx.x == 0) {
        for (int i = threadIdx.x; i < n; i += blockDim.x) p.xq_out[(size_t)b * n + i] = xq[i];
        for (int i = threadIdx.x; i < nb; i += blockDim.x) p.xs_out[(size_t)b * nb + i] = xs[i];
    }
    if (wid < nwq) {
        float* terms = scratch + wid * terms_floats(RP, gsh, nb);
        int total = 0;
        for (int m = 0; m < p.nq; ++m) total += p.q[m].n_out;
        int b0, b1, r0, r1;
        share(total, gridDim.x, blockIdx.x, b0, b1);
        share(b1 - b0, nwq, wid, r0, r1);
        r0 += b0; r1 += b0;
        int base = 0;
        for (int m = 0; m < p.nq; ++m) {
            int lo = max(r0, base) - base, hi = min(r1, base + p.q[m].n_out) - base;
            if (lo < hi) {
                float* o = p.qout[m] + (size_t)b * p.qstride[m];
                if (m == 0 && p.conv_w) {
                    const int kernel = p.conv_kernel, keep = kernel - 1;
                    float* st = p.conv_state + (size_t)b * p.conv_state_stride;
                    q8_rows<RP>(p.q[m], lo, hi, xq, xs, terms, gsh, [&](int row, float v) {
                        float* past = st + (size_t)row * keep;
                        const float* w = p.conv_w + (size_t)row * kernel;
                        float sum = 0.0f;
                        for (int k = 0; k < keep; ++k) sum += past[k] * w[k];
                        sum += v * w[keep];
                        o[row] = silu_f(sum);
                        for (int k = 0; k + 1 < keep; ++k) past[k] = past[k + 1];
                        past[keep - 1] = v;
                    });
                } else {
                    q8_rows<RP>(p.q[m], lo, hi, xq, xs, terms, gsh, [&](int row, float v) { o[row] = v; });
                }
            }
            base += p.q[m].n_out;
        }
    } else {
        // F32 rows: units of 32 rows (serial-k mode) or 4 rows; unit u goes to block u.
        const int unit = p.exact ? 32 : 4;
        float* tile = scratch + nwq * terms_floats(RP, gsh, nb);
        int ubase = 0;
        for (int m = 0; m < p.nf; ++m) {
            int units = (p.f[m].n_out + unit - 1) / unit;
            for (int u = (int)blockIdx.x - ubase; u < units; u += gridDim.x) {
                if (u < 0) continue;
                int lo = u * unit, hi = min(p.f[m].n_out, lo + unit);
                float* o = p.fout[m] + (size_t)b * p.fstride[m];
                if (p.exact) f32_rows<true>(p.f[m].w, n, lo, hi, xn, tile, [&](int row, float v) { o[row] = v; });
                else f32_rows<false>(p.f[m].w, n, lo, hi, xn, tile, [&](int row, float v) { o[row] = v; });
            }
            ubase = (ubase + units) % gridDim.x;
        }
    }
}
static size_t in_proj_smem(int n, int nw) {
    int nb = n / 32, gsh = lanes_shift(nb);
    return 256 + (size_t)n * 4 + n + (size_t)nb * 4 + (size_t)(nw - 1) * terms_floats(4, gsh, nb) * 4 + 32 * 33 * 4;
}

// Output projection with the residual add fused: x[b] += W . quantise(a[b]) (src/model/qwen35.rs:1017, :1220, :1325).
struct OutProj { const float* a; int a_stride; int n_in; DevQ8 w; float* x; int x_stride; };
__global__ void __launch_bounds__(256) k_out_proj(OutProj p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int RP = 4;
    const int n = p.n_in, nb = n / 32, gsh = lanes_shift(nb);
    float* an = (float*)smem;
    int8_t* aq = (int8_t*)(an + n);
    float* as = (float*)(aq + n);
    const int b = blockIdx.y, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float* terms = as + nb + wid * terms_floats(RP, gsh, nb);
    for (int i = threadIdx.x; i < n; i += blockDim.x) an[i] = p.a[(size_t)b * p.a_stride + i];
    __syncthreads();
    block_quant_q8(an, n, aq, as);
    int b0, b1, r0, r1;
    share(p.w.n_out, gridDim.x, blockIdx.x, b0, b1);
    share(b1 - b0, nw, wid, r0, r1);
    float* x = p.x + (size_t)b * p.x_stride;
    q8_rows<RP>(p.w, b0 + r0, b0 + r1, aq, as, terms, gsh, [&](int row, float v) { x[row] += v; });
}
static size_t out_proj_smem(int n, int nw) {
    int nb = n / 32, gsh = lanes_shift(nb);
    return (size_t)n * 4 + n + (size_t)nb * 4 + (size_t)nw * terms_floats(4, gsh, nb) * 4;
}

// GatedDeltaNet core for one (value head, sequence): l2-norm of q and k, gated delta rule over the
// head's [sv][sk] state, gated RMSNorm and the SiLU(z) gate (src/model/qwen35.rs:1298-1322,
// src/ops/naive.rs:86-135, :254-273). One thread per value row, keys walked serially.
struct GdnCore {
    const float* conv; int conv_stride;           // [B][conv_dim] = q | k | v after conv + SiLU
    const float* z; const float* alpha; const float* beta;  // [B][value_dim], [B][n_v], [B][n_v]
    const float* ssm_a; const float* dt_bias; const float* ssm_norm;
    float* state; size_t state_stride;             // [B][n_v][sv][sk]
    float* out;                                    // [B][value_dim]: silu(z) * norm(core)
    int sk, sv, n_k, n_v; float eps;
};
__global__ void __launch_bounds__(256) k_gdn_core(GdnCore p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int sk = p.sk, sv = p.sv, h = blockIdx.x, b = blockIdx.y, kh = h % p.n_k, tid = threadIdx.x;
    const int lane = tid & 31, wid = tid >> 5;
    float* S = (float*)smem;                 // [sv][sk+1]
    float* kq = S + sv * (sk + 1);           // k[sk] | q[sk]
    float* o = kq + 2 * sk;                  // [sv]
    __shared__ double red2[8];
    const int key_dim = p.n_k * sk;
    const float* cv = p.conv + (size_t)b * p.conv_stride;
    float* sg = p.state + (size_t)b * p.state_stride + (size_t)h * sv * sk;
    for (int i = tid; i < sv * sk / 4; i += blockDim.x) {
        float4 v = ((const float4*)sg)[i];
        int r = (i * 4) / sk, c0 = (i * 4) % sk;
        float* d = S + r * (sk + 1) + c0;
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    }
    // warp 0 normalises k, warp 1 normalises q (f64 tree sum, narrowing before the root)
    if (wid < 2) {
        const float* src = cv + (wid == 0 ? key_dim : 0) + kh * sk;
        double acc = 0.0;
        for (int i = lane; i < sk; i += 32) { float v = src[i]; acc += (double)(v * v); }
        acc = warp_sum_d(acc);
        float sc = 1.0f / fmaxf(sqrtf((float)acc), p.eps);
        float qs = 1.0f / sqrtf((float)sk);
        for (int i = lane; i < sk; i += 32) {
            float v = src[i] * sc;
            kq[wid * sk + i] = wid == 0 ? v : v * qs;
        }
    }
    __syncthreads();
    if (tid < sv) {
        float a = p.alpha[(size_t)b * p.n_v + h] + p.dt_bias[h];
        float sp = a > 20.0f ? a : log_f(1.0f + exp_f(a));
        float g = exp_f(sp * p.ssm_a[h]);
        float bt = sigmoid_f(p.beta[(size_t)b * p.n_v + h]);
        float* row = S + tid * (sk + 1);
        float pred = 0.0f;
        for (int i = 0; i < sk; ++i) { float s = row[i] * g; row[i] = s; pred += s * kq[i]; }
        float d = bt * (cv[2 * key_dim + h * sv + tid] - pred);
        float acc = 0.0f;
        for (int i = 0; i < sk; ++i) { float s = row[i] + kq[i] * d; row[i] = s; acc += s * kq[sk + i]; }
        o[tid] = acc;
    }
    __syncthreads();
    // gated RMSNorm over the head's sv outputs, then * silu(z)
    {
        double acc = 0.0;
        for (int i = tid; i < sv; i += blockDim.x) acc += (double)(o[i] * o[i]);
        acc = warp_sum_d(acc);
        if (lane == 0) red2[wid] = acc;
        __syncthreads();
        double tot = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red2[w];
        float mean = (float)(tot / (double)sv);
        float sc = 1.0f / sqrtf(mean + p.eps);
        if (tid < sv) {
            float core = o[tid] * sc * p.ssm_norm[tid];
            size_t idx = (size_t)b * p.n_v * sv + (size_t)h * sv + tid;
            p.out[idx] = silu_f(p.z[idx]) * core;
        }
    }
    for (int i = tid; i < sv * sk / 4; i += blockDim.x) {
        int r = (i * 4) / sk, c0 = (i * 4) % sk;
        const float* s = S + r * (sk + 1) + c0;
        ((float4*)sg)[i] = make_float4(s[0], s[1], s[2], s[3]);
    }
}

// Attention prologue per head: de-interleave q|gate, QK RMSNorm, partial NEOX RoPE at the sequence's
// position, KV write (src/model/qwen35.rs:1175-1198). grid (n_head + 2*n_head_kv, B), block = head_dim.
struct AttnPrep {
    const float* qg; const float* k; const float* v;      // [B][2*hd*n_head], [B][kv_dim], [B][kv_dim]
    const float* q_norm; const float* k_norm;
    float* q_out; float* g_out;                            // [B][n_head*hd]
    uint16_t* kslab; uint16_t* vslab; size_t slab_stride;  // per sequence [n_ctx][kv_dim]
    const int* pos; int* npos_out;                         // position of this token; positions to attend over
    int hd, n_head, n_head_kv, n_rot; float theta, eps; int bf16;
};
__global__ void k_attn_prep(AttnPrep p) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* val = (float*)smem;  // [hd]
    __shared__ double red[8];
    const int job = blockIdx.x, b = blockIdx.y, d = threadIdx.x, hd = p.hd, kvd = p.n_head_kv * hd;
    const int pos = p.pos[b];
    if (job == 0 && d == 0) p.npos_out[b] = pos + 1;
    const bool is_q = job < p.n_head, is_k = !is_q && job < p.n_head + p.n_head_kv;
    const int hk = is_q ? job : is_k ? job - p.n_head : job - p.n_head - p.n_head_kv;
    float v;
    if (is_q) {
        v = p.qg[(size_t)b * 2 * hd * p.n_head + (size_t)hk * 2 * hd + d];
        p.g_out[((size_t)b * p.n_head + hk) * hd + d] = p.qg[(size_t)b * 2 * hd * p.n_head + (size_t)hk * 2 * hd + hd + d];
    } else {
        v = (is_k ? p.k : p.v)[(size_t)b * kvd + hk * hd + d];
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
    if (is_q) p.q_out[((size_t)b * p.n_head + hk) * hd + d] = v;
    else {
        uint16_t* slab = (is_k ? p.kslab : p.vslab) + (size_t)b * p.slab_stride + (size_t)pos * kvd + hk * hd + d;
        *slab = p.bf16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v);
    }
}

// Routed experts, gated half: softmax over all experts, top-k, then for every pick
// h = silu(gate_e . x * s_g) * (up_e . x * s_u) (src/model/qwen35.rs:1626-1656, src/ops/mod.rs:1105-1117).
// Every block redoes the (tiny) softmax + top-k so no grid-wide step separates routing from the experts.
struct MoeGlu {
    const float* router; int n_expert, n_used;      // [B][n_expert] logits
    const int8_t* xq; const float* xs; int n_embd;  // quantised normed row [B][n_embd]
    DevFp4 gate, up;
    float* h;                                       // [B][n_used][ff]
    int32_t* ids_out; float* w_out;                 // [B][n_used]
};
__global__ void __launch_bounds__(256) k_moe_glu(MoeGlu p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int RP = 4;
    __shared__ float sval[32];
    __shared__ int sidx[32];
    __shared__ int32_t ids[16];
    __shared__ float wts[16];
    const int n = p.n_embd, nb = n / 32, nsb = n / 16, gsh = lanes_shift(nb), ff = p.gate.n_out;
    const int b = blockIdx.y, tid = threadIdx.x, wid = tid >> 5, nw = blockDim.x >> 5, lane = tid & 31;
    float* probs = (float*)smem;                  // [n_expert]
    int8_t* xq = (int8_t*)(probs + p.n_expert);
    float* xs = (float*)(xq + n);
    float* terms = xs + nb + wid * terms_floats(RP, gsh, nsb);
    for (int i = tid; i < n / 16; i += blockDim.x) ((uint4*)xq)[i] = ((const uint4*)(p.xq + (size_t)b * n))[i];
    for (int i = tid; i < nb; i += blockDim.x) xs[i] = p.xs[(size_t)b * nb + i];
    // softmax (src/ops/naive.rs:362-376): max, exp, serial sum in index order, divide
    const float* lg = p.router + (size_t)b * p.n_expert;
    float mx = -INFINITY;
    for (int i = tid; i < p.n_expert; i += blockDim.x) mx = fmaxf(mx, lg[i]);
    mx = warp_max(mx);
    if (lane == 0) sval[wid] = mx;
    __syncthreads();
    mx = sval[0];
    for (int w = 1; w < nw; ++w) mx = fmaxf(mx, sval[w]);
    __syncthreads();
    for (int i = tid; i < p.n_expert; i += blockDim.x) probs[i] = exp_f(lg[i] - mx);
    __syncthreads();
    if (tid == 0) { float s = 0.0f; for (int i = 0; i < p.n_expert; ++i) s += probs[i]; sval[0] = s; }
    __syncthreads();
    float sum = sval[0];
    __syncthreads();
    for (int i = tid; i < p.n_expert; i += blockDim.x) probs[i] /= sum;
    __syncthreads();
    block_topk(probs, p.n_expert, p.n_used, ids, wts, sval, sidx);
    if (blockIdx.x == 0 && tid < p.n_used) {
        p.ids_out[(size_t)b * p.n_used + tid] = ids[tid];
        p.w_out[(size_t)b * p.n_used + tid] = wts[tid];
    }
    int b0, b1, r0, r1;
    share(p.n_used * ff, gridDim.x, blockIdx.x, b0, b1);
    share(b1 - b0, nw, wid, r0, r1);
    r0 += b0; r1 += b0;
    for (int i = 0; i < p.n_used; ++i) {
        int lo = max(r0, i * ff) - i * ff, hi = min(r1, (i + 1) * ff) - i * ff;
        if (lo >= hi) continue;
        int el = ids[i] - p.gate.expert_lo;
        if (el < 0 || el >= p.gate.n_expert) continue;
        float* h = p.h + ((size_t)b * p.n_used + i) * ff;
        const size_t eo = (size_t)el * ff;
        const bool has_g = p.gate.scale2 != nullptr, has_u = p.up.scale2 != nullptr;
        const float sg2 = has_g ? p.gate.scale2[el] : 1.0f, su2 = has_u ? p.up.scale2[el] : 1.0f;
        fp4_rows<RP>(p.gate.nib + eo * (n / 2), p.gate.sc + eo * nsb, n, lo, hi, xq, xs, terms, gsh,
                     [&](int row, float v) { h[row] = has_g ? v * sg2 : v; });
        fp4_rows<RP>(p.up.nib + eo * (n / 2), p.up.sc + eo * nsb, n, lo, hi, xq, xs, terms, gsh,
                     [&](int row, float v) { float u = has_u ? v * su2 : v; h[row] = silu_f(h[row]) * u; });
    }
}
static size_t moe_glu_smem(int n_expert, int n, int nw) {
    int nb = n / 32, gsh = lanes_shift(nb);
    return (size_t)n_expert * 4 + n + (size_t)nb * 4 + (size_t)nw * terms_floats(4, gsh, n / 16) * 4;
}

// Routed experts, second half, with the whole FFN tail fused: down projections of the picks, the shared
// expert's SiLU gate and down projection, the weighted sum in pick order, the sigmoid-gated shared term
// and the residual add (src/model/qwen35.rs:1659-1699, src/ops/mod.rs:1134-1171, src/model/qwen35.rs:1090).
struct MoeDown {
    const float* h; int n_used, ff;                // [B][n_used][ff]
    const int32_t* ids; const float* wts;          // [B][n_used]
    DevFp4 down;
    const float* sg; const float* su; int sff;     // shared expert gate/up outputs [B][sff]
    DevQ8 shared_down;
    const float* logit;                            // [B]
    float* x; int x_stride;                        // residual, [B][n_embd]
    int local_only;                                // expert-parallel: write partial sums to `partial` instead
    float* partial;
};
__global__ void __launch_bounds__(256) k_moe_down(MoeDown p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int RP = 4;
    const int ff = p.ff, sff = p.sff, nbf = ff / 32, nbs = sff / 32;
    const int gf = lanes_shift(nbf), gs = lanes_shift(nbs);
    const int b = blockIdx.y, tid = threadIdx.x, wid = tid >> 5, nw = blockDim.x >> 5;
    const int n_out = p.down.n_out;
    float* hf = (float*)smem;                                   // [max(ff,sff)] staging
    int8_t* hq = (int8_t*)(hf + max(ff, sff));                  // [n_used][ff]
    float* hs = (float*)(hq + p.n_used * ff);                   // [n_used][nbf]
    int8_t* sq = (int8_t*)(hs + p.n_used * nbf);                // [sff]
    float* ss = (float*)(sq + sff);                             // [nbs]
    int b0, b1, r0, r1;
    share(n_out, gridDim.x, blockIdx.x, b0, b1);
    float* acc = ss + nbs;                                      // [rows of this block]
    int tf = max(terms_floats(RP, gf, ff / 16), terms_floats(RP, gs, nbs));
    float* terms = acc + (b1 - b0 + 1) + wid * tf;
    for (int i = 0; i < p.n_used; ++i) {
        for (int k = tid; k < ff; k += blockDim.x) hf[k] = p.h[((size_t)b * p.n_used + i) * ff + k];
        __syncthreads();
        block_quant_q8(hf, ff, hq + i * ff, hs + i * nbf);
    }
    for (int k = tid; k < sff; k += blockDim.x) hf[k] = silu_f(p.sg[(size_t)b * sff + k]) * p.su[(size_t)b * sff + k];
    __syncthreads();
    block_quant_q8(hf, sff, sq, ss);
    share(b1 - b0, nw, wid, r0, r1);
    r0 += b0; r1 += b0;
    const int lane = tid & 31;
    for (int r = r0 + lane; r < r1; r += 32) acc[r - b0] = 0.0f;
    __syncwarp();
    const int nsb = ff / 16;
    for (int i = 0; i < p.n_used; ++i) {
        int el = p.ids[(size_t)b * p.n_used + i] - p.down.expert_lo;
        if (el < 0 || el >= p.down.n_expert) continue;
        const size_t eo = (size_t)el * n_out;
        const bool has_s = p.down.scale2 != nullptr;
        const float s2 = has_s ? p.down.scale2[el] : 1.0f, wt = p.wts[(size_t)b * p.n_used + i];
        fp4_rows<RP>(p.down.nib + eo * (ff / 2), p.down.sc + eo * nsb, ff, r0, r1, hq + i * ff, hs + i * nbf, terms, gf,
                     [&](int row, float v) { float o = has_s ? v * s2 : v; acc[row - b0] += wt * o; });
        __syncwarp();
    }
    if (p.local_only) {
        for (int r = r0 + lane; r < r1; r += 32) p.partial[(size_t)b * n_out + r] = acc[r - b0];
        return;
    }
    const float g = sigmoid_f(p.logit[b]);
    float* x = p.x + (size_t)b * p.x_stride;
    q8_rows<RP>(p.shared_down, r0, r1, sq, ss, terms, gs, [&](int row, float v) {
        float t = acc[row - b0];
        t += v * g;
        x[row] += t;
    });
}
static size_t moe_down_smem(int n_used, int ff, int sff, int rows_per_block, int nw) {
    int gf = lanes_shift(ff / 32), gs = lanes_shift(sff / 32);
    int tf = std::max(terms_floats(4, gf, ff / 16), terms_floats(4, gs, sff / 32));
    return (size_t)std::max(ff, sff) * 4 + (size_t)n_used * ff + (size_t)n_used * (ff / 32) * 4 + sff + (size_t)(sff / 32) * 4 +
           (size_t)(rows_per_block + 2) * 4 + (size_t)nw * tf * 4 + 64;
}

__global__ void k_embed(const float* table, int n_embd, const int32_t* tokens, float* x) {
    int b = blockIdx.x;
    const float* row = table + (size_t)tokens[b] * n_embd;
    for (int i = threadIdx.x; i < n_embd; i += blockDim.x) x[(size_t)b * n_embd + i] = row[i];
}

// Greedy argmax with strict '>' (lowest index wins, src/profile.rs:192-213), feeding the choice back as the
// next input token and advancing the position. One block per sequence.
__global__ void k_argmax_advance(const float* logits, int n_vocab, int32_t* tokens, int* pos, int32_t* next_out,
                                 int32_t* history, int* step_counter, int n_seq) {
    __shared__ float sv[32];
    __shared__ int si[32];
    int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const float* l = logits + (size_t)b * n_vocab;
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = tid; i < n_vocab; i += blockDim.x) { float v = l[i]; if (bi == 0x7fffffff || v > bv) { bv = v; bi = i; } }
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[wid] = bv; si[wid] = bi; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (si[w] != 0x7fffffff && (bi == 0x7fffffff || sv[w] > bv || (sv[w] == bv && si[w] < bi))) { bv = sv[w]; bi = si[w]; }
        tokens[b] = bi;
        next_out[b] = bi;
        pos[b] += 1;
        if (history) history[(size_t)step_counter[0] * n_seq + b] = bi;
    }
    if (b == 0 && tid == 0 && history) { __threadfence(); }
}
__global__ void k_bump(int* counter) { counter[0] += 1; }

// =====================================================================================================
// Model
// =====================================================================================================
struct DevTensor {
    uint32_t ty = 0;
    size_t n_in = 0, n_out = 0, n_expert = 1;
    void* a = nullptr; void* b = nullptr; float* scale2 = nullptr;
    size_t e_lo = 0, e_cnt = 0;  // experts stored
    size_t bytes = 0;
};
struct DevLayer {
    bool recurrent = false;
    const float *attn_norm = nullptr, *ffn_norm = nullptr;
    DevQ8 wq, wk, wv, wo; const float *q_norm = nullptr, *k_norm = nullptr;
    DevQ8 wqkv, wgate, ssm_out; DevF32 ssm_alpha, ssm_beta;
    const float *conv1d = nullptr, *ssm_a = nullptr, *dt_bias = nullptr, *ssm_norm = nullptr;
    DevF32 gate_inp, shared_gate_inp; DevFp4 gate, up, down; DevQ8 shared_gate, shared_up, shared_down;
};
struct itb_model {
    itb_ctx* c = nullptr;
    itb_model_dims d{};
    std::map<std::string, DevTensor> t;
    std::vector<DevLayer> layers;
    DevF32 tok_embd; const float* output_norm = nullptr; DevQ8 output;
    bool finalized = false;
    uint32_t expert_lo = 0, expert_hi = 0;
    size_t bytes = 0;
};

static synth::ModelDims to_synth(const itb_model_dims& d) {
    synth::ModelDims s;
    static_assert(sizeof(synth::ModelDims) == sizeof(itb_model_dims), "dims layouts must match");
    memcpy(&s, &d, sizeof s);
    return s;
}

extern "C" int itb_model_create(itb_ctx* c, const itb_model_dims* d, itb_model** out) {
    *out = nullptr;
    auto bad = [&](const char* m) { itb_fail_msg(c, std::string("model: ") + m); return 1; };
    // src/model/qwen35.rs:361-486: the relationships the forward pass assumes
    if (d->n_head_kv == 0 || d->n_head % d->n_head_kv) return bad("query heads do not divide into kv heads");
    if (d->ssm_dt_rank == 0 || d->ssm_d_inner % d->ssm_dt_rank) return bad("inner size does not divide into value heads");
    if (d->ssm_n_group == 0 || d->ssm_dt_rank % d->ssm_n_group) return bad("value heads do not divide into key heads");
    if (d->ssm_d_inner / d->ssm_dt_rank != d->ssm_d_state) return bad("the recurrence assumes a square state");
    if (d->full_attention_interval == 0) return bad("full_attention_interval must be non-zero");
    if (d->n_rot > d->head_dim || d->n_rot % 2) return bad("rope.dimension_count exceeds head_dim or is odd");
    if (d->n_expert_used == 0 || d->n_expert_used > d->n_expert || d->n_expert_used > 16) return bad("expert_used_count out of range");
    if (d->n_embd % 64 || d->expert_ff % 64 || d->shared_ff % 32 || d->ssm_d_inner % 32 || (d->head_dim * d->n_head) % 32) return bad("dimensions must be whole quantisation blocks");
    if (d->head_dim != 64 && d->head_dim != 128 && d->head_dim != 256) return bad("head_dim must be 64, 128 or 256");
    if (d->ssm_d_state > 128 || d->ssm_d_conv < 2 || d->ssm_d_conv > 8 || d->n_expert > 1024) return bad("dimension beyond what the kernels hold");
    itb_model* m = new itb_model();
    m->c = c; m->d = *d;
    *out = m;
    return 0;
}
extern "C" void itb_model_destroy(itb_model* m) {
    if (!m) return;
    cudaStreamSynchronize(m->c->stream);
    for (auto& kv : m->t) { cudaFree(kv.second.a); cudaFree(kv.second.b); cudaFree(kv.second.scale2); }
    delete m;
}

// raw reference-layout bytes already on the device -> kernel layout
static int adopt_raw(itb_model* m, const std::string& name, uint32_t ty, size_t n_in, size_t n_out, size_t n_expert,
                     size_t e_lo, size_t e_cnt, uint8_t* raw, float* scale2_dev) {
    itb_ctx* c = m->c;
    DevTensor t;
    t.ty = ty; t.n_in = n_in; t.n_out = n_out; t.n_expert = n_expert; t.e_lo = e_lo; t.e_cnt = e_cnt;
    size_t elems = n_in * n_out * e_cnt;
    if (ty == ITB_Q8_0) {
        ITB_CUDA_RET(c, cudaMalloc(&t.a, elems), 1); ITB_CUDA_RET(c, cudaMalloc(&t.b, elems / 32 * 2), 1);
        itb_repack_q8(c->stream, raw, (int8_t*)t.a, (uint16_t*)t.b, elems / 32);
        t.bytes = elems + elems / 16;
    } else if (ty == ITB_NVFP4) {
        ITB_CUDA_RET(c, cudaMalloc(&t.a, elems / 2), 1); ITB_CUDA_RET(c, cudaMalloc(&t.b, elems / 16), 1);
        itb_repack_fp4(c->stream, raw, (uint8_t*)t.a, (uint8_t*)t.b, elems / 64);
        t.scale2 = scale2_dev;
        t.bytes = elems / 2 + elems / 16;
    } else return 1;
    c->launches++;
    auto it = m->t.find(name);
    if (it != m->t.end()) { cudaFree(it->second.a); cudaFree(it->second.b); cudaFree(it->second.scale2); m->bytes -= it->second.bytes; }
    m->t[name] = t;
    m->bytes += t.bytes;
    m->finalized = false;
    return 0;
}

static const synth::TensorSpec* find_spec(const std::vector<synth::TensorSpec>& v, const std::string& n) {
    for (auto& s : v) if (s.name == n) return &s;
    return nullptr;
}

extern "C" int itb_model_set_tensor(itb_model* m, const char* name, uint32_t ty, const void* data, size_t bytes,
                                    const float* scale, size_t n_scale) {
    itb_ctx* c = m->c;
    auto specs = synth::model_tensors(to_synth(m->d));
    const synth::TensorSpec* s = find_spec(specs, name);
    if (!s) { itb_fail_msg(c, std::string("set_tensor: unknown tensor ") + name); return 1; }
    if (s->ty != ty) { itb_fail_msg(c, std::string("set_tensor: ") + name + " has a storage type this path has no kernel for"); return 1; }
    if (bytes != s->bytes()) { itb_fail_msg(c, std::string("set_tensor: wrong byte count for ") + name); return 1; }
    if (ty == ITB_F32) {
        DevTensor t; t.ty = ty; t.n_in = s->n_in; t.n_out = s->n_out; t.bytes = bytes;
        ITB_CUDA_RET(c, cudaMalloc(&t.a, bytes), 1);
        ITB_CUDA_RET(c, cudaMemcpyAsync(t.a, data, bytes, cudaMemcpyHostToDevice, c->stream), 1);
        ITB_CUDA_RET(c, cudaStreamSynchronize(c->stream), 1);
        auto it = m->t.find(name);
        if (it != m->t.end()) { cudaFree(it->second.a); m->bytes -= it->second.bytes; }
        m->t[name] = t; m->bytes += bytes; m->finalized = false;
        return 0;
    }
    uint8_t* raw = nullptr;
    ITB_CUDA_RET(c, cudaMalloc(&raw, bytes), 1);
    cudaMemcpyAsync(raw, data, bytes, cudaMemcpyHostToDevice, c->stream);
    float* s2 = nullptr;
    if (ty == ITB_NVFP4 && scale && n_scale >= s->n_expert) {
        cudaMalloc(&s2, s->n_expert * 4);
        cudaMemcpyAsync(s2, scale, s->n_expert * 4, cudaMemcpyHostToDevice, c->stream);
    }
    int rc = adopt_raw(m, name, ty, s->n_in, s->n_out, s->n_expert, 0, s->n_expert, raw, s2);
    cudaError_t e = cudaStreamSynchronize(c->stream);
    cudaFree(raw);
    if (e != cudaSuccess) { itb_fail(c, "set_tensor", e); return 1; }
    return rc;
}

extern "C" int itb_model_synth(itb_model* m, uint64_t seed, uint32_t e_lo, uint32_t e_hi) {
    itb_ctx* c = m->c;
    auto specs = synth::model_tensors(to_synth(m->d));
    if (e_hi == 0) { e_lo = 0; e_hi = m->d.n_expert; }
    if (e_hi > m->d.n_expert || e_lo >= e_hi) { itb_fail_msg(c, "model_synth: bad expert range"); return 1; }
    m->expert_lo = e_lo; m->expert_hi = e_hi;
    size_t max_raw = 0;
    for (auto& s : specs) {
        size_t cnt = s.n_expert > 1 ? (e_hi - e_lo) : 1;
        if (s.ty != synth::TY_F32) max_raw = std::max<size_t>(max_raw, s.bytes() / s.n_expert * cnt);
    }
    uint8_t* raw = nullptr; unsigned* amax = nullptr;
    ITB_CUDA_RET(c, cudaMalloc(&raw, max_raw + 64), 1);
    ITB_CUDA_RET(c, cudaMalloc(&amax, (size_t)m->d.n_expert * 4), 1);
    int rc = 0;
    for (auto& s : specs) {
        uint64_t key = synth::tensor_key(seed, s.name.c_str());
        if (s.ty == synth::TY_F32) {
            DevTensor t; t.ty = ITB_F32; t.n_in = s.n_in; t.n_out = s.n_out; t.bytes = s.bytes();
            if (cudaMalloc(&t.a, t.bytes) != cudaSuccess) { itb_fail_msg(c, "model_synth: out of device memory"); rc = 1; break; }
            itb_synth_f32(c->stream, key, s.elems(), s.dist, s.std_, (float*)t.a);
            c->launches++;
            auto it = m->t.find(s.name);
            if (it != m->t.end()) { cudaFree(it->second.a); m->bytes -= it->second.bytes; }
            m->t[s.name] = t; m->bytes += t.bytes;
        } else if (s.ty == synth::TY_Q8_0) {
            itb_synth_q8_raw(c->stream, key, s.elems() / 32, s.dist, s.std_, raw);
            c->launches++;
            if ((rc = adopt_raw(m, s.name, ITB_Q8_0, s.n_in, s.n_out, 1, 0, 1, raw, nullptr))) break;
        } else {
            float* s2 = nullptr;
            size_t cnt = e_hi - e_lo;
            if (cudaMalloc(&s2, cnt * 4) != cudaSuccess) { itb_fail_msg(c, "model_synth: out of device memory"); rc = 1; break; }
            itb_synth_fp4_raw(c->stream, key, s.n_in * s.n_out, e_lo, e_hi, s.dist, s.std_, amax, s2, raw);
            c->launches += 2;
            if ((rc = adopt_raw(m, s.name, ITB_NVFP4, s.n_in, s.n_out, s.n_expert, e_lo, cnt, raw, s2))) break;
        }
        // raw is reused by the next tensor: order the reuse behind this tensor's repack
        if (cudaStreamSynchronize(c->stream) != cudaSuccess) { itb_fail_msg(c, "model_synth: device error"); rc = 1; break; }
    }
    cudaFree(raw); cudaFree(amax);
    m->finalized = false;
    return rc;
}

extern "C" int itb_model_synth_read(itb_model* m, uint64_t seed, const char* name, void* out, size_t bytes, float* scale_out) {
    itb_ctx* c = m->c;
    auto specs = synth::model_tensors(to_synth(m->d));
    const synth::TensorSpec* s = find_spec(specs, name);
    if (!s || bytes != s->bytes()) { itb_fail_msg(c, std::string("synth_read: unknown tensor or wrong size: ") + name); return 1; }
    uint64_t key = synth::tensor_key(seed, s->name.c_str());
    uint8_t* raw = nullptr; unsigned* amax = nullptr; float* s2 = nullptr;
    ITB_CUDA_RET(c, cudaMalloc(&raw, bytes + 64), 1);
    if (s->ty == synth::TY_F32) itb_synth_f32(c->stream, key, s->elems(), s->dist, s->std_, (float*)raw);
    else if (s->ty == synth::TY_Q8_0) itb_synth_q8_raw(c->stream, key, s->elems() / 32, s->dist, s->std_, raw);
    else {
        cudaMalloc(&amax, s->n_expert * 4); cudaMalloc(&s2, s->n_expert * 4);
        itb_synth_fp4_raw(c->stream, key, s->n_in * s->n_out, 0, s->n_expert, s->dist, s->std_, amax, s2, raw);
        if (scale_out) cudaMemcpyAsync(scale_out, s2, s->n_expert * 4, cudaMemcpyDeviceToHost, c->stream);
    }
    c->launches++;
    cudaMemcpyAsync(out, raw, bytes, cudaMemcpyDeviceToHost, c->stream);
    cudaError_t e = cudaStreamSynchronize(c->stream);
    cudaFree(raw); cudaFree(amax); cudaFree(s2);
    if (e != cudaSuccess) { itb_fail(c, "synth_read", e); return 1; }
    return 0;
}

static bool finalize(itb_model* m) {
    if (m->finalized) return true;
    itb_ctx* c = m->c;
    const itb_model_dims& d = m->d;
    bool ok = true;
    auto get = [&](const std::string& n) -> const DevTensor* {
        auto it = m->t.find(n);
        if (it == m->t.end()) { itb_fail_msg(c, "model: missing tensor " + n); ok = false; return nullptr; }
        return &it->second;
    };
    auto q8 = [&](const std::string& n) { const DevTensor* t = get(n); return t ? DevQ8{(const int8_t*)t->a, (const uint16_t*)t->b, (int)t->n_in, (int)t->n_out} : DevQ8{}; };
    auto f32 = [&](const std::string& n) { const DevTensor* t = get(n); return t ? DevF32{(const float*)t->a, (int)t->n_in, (int)t->n_out} : DevF32{}; };
    auto vec = [&](const std::string& n) { const DevTensor* t = get(n); return t ? (const float*)t->a : nullptr; };
    auto fp4 = [&](const std::string& n) {
        const DevTensor* t = get(n);
        return t ? DevFp4{(const uint8_t*)t->a, (const uint8_t*)t->b, t->scale2, (int)t->n_in, (int)t->n_out, (int)t->e_cnt, (int)t->e_lo} : DevFp4{};
    };
    m->tok_embd = f32("token_embd.weight");
    m->output_norm = vec("output_norm.weight");
    m->output = q8("output.weight");
    m->layers.assign(d.n_layer, DevLayer{});
    for (uint32_t i = 0; i < d.n_layer && ok; ++i) {
        std::string P = "blk." + std::to_string(i) + ".";
        DevLayer& L = m->layers[i];
        L.recurrent = (i + 1) % d.full_attention_interval != 0;   // src/model/qwen35.rs:329-331
        L.attn_norm = vec(P + "attn_norm.weight");
        L.ffn_norm = vec(P + "post_attention_norm.weight");
        if (L.recurrent) {
            L.wqkv = q8(P + "attn_qkv.weight"); L.wgate = q8(P + "attn_gate.weight"); L.ssm_out = q8(P + "ssm_out.weight");
            L.ssm_alpha = f32(P + "ssm_alpha.weight"); L.ssm_beta = f32(P + "ssm_beta.weight");
            L.conv1d = vec(P + "ssm_conv1d.weight"); L.ssm_a = vec(P + "ssm_a"); L.dt_bias = vec(P + "ssm_dt.bias");
            L.ssm_norm = vec(P + "ssm_norm.weight");
        } else {
            L.wq = q8(P + "attn_q.weight"); L.wk = q8(P + "attn_k.weight"); L.wv = q8(P + "attn_v.weight");
            L.wo = q8(P + "attn_output.weight");
            L.q_norm = vec(P + "attn_q_norm.weight"); L.k_norm = vec(P + "attn_k_norm.weight");
        }
        L.gate_inp = f32(P + "ffn_gate_inp.weight"); L.shared_gate_inp = f32(P + "ffn_gate_inp_shexp.weight");
        L.gate = fp4(P + "ffn_gate_exps.weight"); L.up = fp4(P + "ffn_up_exps.weight"); L.down = fp4(P + "ffn_down_exps.weight");
        L.shared_gate = q8(P + "ffn_gate_shexp.weight"); L.shared_up = q8(P + "ffn_up_shexp.weight");
        L.shared_down = q8(P + "ffn_down_shexp.weight");
    }
    m->finalized = ok;
    return ok;
}

// Algorithmic bytes of one decode step: every weight row read once (Q8_0 34/32 B, NVFP4 36/64 B, F32 4 B per
// element; routed experts only the `distinct` ones hit per layer), recurrent state read + written, KV read
// at `n_pos`, one embedding row (src/model/qwen35.rs:880-938 counts the same way).
extern "C" uint64_t itb_model_decode_bytes(itb_model* m, uint32_t n_seq, uint32_t n_pos, uint32_t distinct) {
    const itb_model_dims& d = m->d;
    auto q8 = [](uint64_t a, uint64_t b) { return a * b / 32 * 34; };
    auto f4 = [](uint64_t a, uint64_t b) { return a * b / 64 * 36; };
    uint64_t H = d.n_embd, key_dim = (uint64_t)d.ssm_d_state * d.ssm_n_group, vd = d.ssm_d_inner, cd = 2 * key_dim + vd;
    uint64_t qd = (uint64_t)d.head_dim * d.n_head, kvd = (uint64_t)d.head_dim * d.n_head_kv;
    uint64_t ffn = 3 * (uint64_t)distinct * f4(H, d.expert_ff) + H * d.n_expert * 4 + 2 * q8(H, d.shared_ff) + q8(d.shared_ff, H) + H * 4;
    uint64_t gdn = q8(H, cd) + q8(H, vd) + q8(vd, H) + 2 * H * d.ssm_dt_rank * 4 + cd * d.ssm_d_conv * 4 +
                   (uint64_t)n_seq * 2 * ((uint64_t)d.ssm_dt_rank * d.ssm_d_state * d.ssm_d_state + (d.ssm_d_conv - 1) * cd) * 4;
    uint64_t att = q8(H, 2 * qd) + 2 * q8(H, kvd) + q8(qd, H) + (uint64_t)n_seq * 2 * kvd * 2 * n_pos;
    uint64_t total = q8(H, d.n_vocab) + (uint64_t)n_seq * H * 4;
    for (uint32_t i = 0; i < d.n_layer; ++i) total += ffn + (((i + 1) % d.full_attention_interval != 0) ? gdn : att);
    return total;
}

// =====================================================================================================
// Engine
// =====================================================================================================
struct itb_engine {
    itb_model* m = nullptr;
    itb_ctx* c = nullptr;
    uint32_t n_ctx = 0, B = 0, n_attn = 0, n_rec = 0;
    std::vector<int> slot_of;  // absolute layer -> attention slot or recurrent slot
    // state
    uint16_t *kslab = nullptr, *vslab = nullptr;   // [n_attn][B][n_ctx][kv_dim]
    float *conv_state = nullptr, *ssm_state = nullptr;  // [n_rec][B][...]
    int* pos = nullptr; int* npos = nullptr; int32_t* tokens = nullptr; int32_t* next = nullptr;
    // activations
    float *x = nullptr, *qkvc = nullptr, *z = nullptr, *alpha = nullptr, *beta = nullptr, *zc = nullptr;
    float *qg = nullptr, *kbuf = nullptr, *vbuf = nullptr, *qn = nullptr, *gate = nullptr, *att = nullptr;
    float *part_acc = nullptr, *part_ml = nullptr;
    float *router = nullptr, *shlogit = nullptr, *sg = nullptr, *su = nullptr, *h = nullptr, *logits = nullptr;
    int8_t* xq = nullptr; float* xs = nullptr;
    int32_t* route_ids = nullptr; float* route_w = nullptr;  // [n_layer][B][n_used]
    int32_t* history = nullptr; int* step_counter = nullptr; uint32_t history_cap = 0;
    int32_t* prompt = nullptr; size_t prompt_cap = 0;
    int n_split = 1;
    cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_ms = 0.0f;
    uint64_t launches_per_step = 0;
    std::vector<uint32_t> host_pos;
    std::vector<void*> allocs;
};

template <class T>
static bool dalloc(itb_engine* e, T** p, size_t count) {
    if (cudaMalloc((void**)p, std::max<size_t>(count, 1) * sizeof(T)) != cudaSuccess) return itb_fail_msg(e->c, "engine: out of device memory");
    cudaMemsetAsync(*p, 0, std::max<size_t>(count, 1) * sizeof(T), e->c->stream);
    e->allocs.push_back(*p);
    return true;
}

static void set_smem(const void* fn, size_t bytes) { cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes); }

// One decode step for all B sequences, enqueued on `st`.
static void enqueue_step(itb_engine* e, cudaStream_t st) {
    itb_model* m = e->m; itb_ctx* c = e->c;
    const itb_model_dims& d = m->d;
    const int B = e->B, H = d.n_embd, sms = c->sm_count;
    const int key_dim = d.ssm_d_state * d.ssm_n_group, vd = d.ssm_d_inner, cd = 2 * key_dim + vd;
    const int qd = d.head_dim * d.n_head, kvd = d.head_dim * d.n_head_kv;
    const int NW_IN = 9, NW = 8;
    uint64_t launches = 0;
    k_embed<<<B, 256, 0, st>>>(m->tok_embd.w, H, e->tokens, e->x); launches++;
    const size_t smem_in = in_proj_smem(H, NW_IN);
    set_smem((const void*)k_in_proj, smem_in);
    for (uint32_t il = 0; il < d.n_layer; ++il) {
        const DevLayer& L = m->layers[il];
        if (L.recurrent) {
            int rs = e->slot_of[il];
            InProj p{};
            p.x = e->x; p.x_stride = H; p.norm_w = L.attn_norm; p.eps = d.rms_eps; p.n_embd = H;
            p.nq = 2; p.q[0] = L.wqkv; p.qout[0] = e->qkvc; p.qstride[0] = cd; p.q[1] = L.wgate; p.qout[1] = e->z; p.qstride[1] = vd;
            p.nf = 2; p.f[0] = L.ssm_alpha; p.fout[0] = e->alpha; p.fstride[0] = d.ssm_dt_rank;
            p.f[1] = L.ssm_beta; p.fout[1] = e->beta; p.fstride[1] = d.ssm_dt_rank;
            p.conv_w = L.conv1d; p.conv_kernel = d.ssm_d_conv; p.conv_state_stride = (size_t)cd * (d.ssm_d_conv - 1);
            p.conv_state = e->conv_state + (size_t)rs * B * p.conv_state_stride;
            p.exact = c->exact;
            int gx = std::min(sms, std::max(1, (cd + vd) / 8));
            k_in_proj<<<dim3(gx, B), NW_IN * 32, smem_in, st>>>(p); launches++;
            GdnCore g{};
            g.conv = e->qkvc; g.conv_stride = cd; g.z = e->z; g.alpha = e->alpha; g.beta = e->beta;
            g.ssm_a = L.ssm_a; g.dt_bias = L.dt_bias; g.ssm_norm = L.ssm_norm;
            g.state_stride = (size_t)d.ssm_dt_rank * d.ssm_d_state * d.ssm_d_state;
            g.state = e->ssm_state + (size_t)rs * B * g.state_stride;
            g.out = e->zc; g.sk = d.ssm_d_state; g.sv = d.ssm_d_state; g.n_k = d.ssm_n_group; g.n_v = d.ssm_dt_rank; g.eps = d.rms_eps;
            size_t smem_g = (size_t)(g.sv * (g.sk + 1) + 2 * g.sk + g.sv) * 4;
            set_smem((const void*)k_gdn_core, smem_g);
            k_gdn_core<<<dim3(d.ssm_dt_rank, B), 256, smem_g, st>>>(g); launches++;
            OutProj o{e->zc, vd, vd, L.ssm_out, e->x, H};
            size_t smem_o = out_proj_smem(vd, NW);
            set_smem((const void*)k_out_proj, smem_o);
            k_out_proj<<<dim3(std::min(sms, std::max(1, H / 8)), B), NW * 32, smem_o, st>>>(o); launches++;
        } else {
            int as = e->slot_of[il];
            InProj p{};
            p.x = e->x; p.x_stride = H; p.norm_w = L.attn_norm; p.eps = d.rms_eps; p.n_embd = H;
            p.nq = 3; p.q[0] = L.wq; p.qout[0] = e->qg; p.qstride[0] = 2 * qd; p.q[1] = L.wk; p.qout[1] = e->kbuf; p.qstride[1] = kvd;
            p.q[2] = L.wv; p.qout[2] = e->vbuf; p.qstride[2] = kvd;
            p.exact = c->exact;
            int gx = std::min(sms, std::max(1, (2 * qd + 2 * kvd) / 8));
            k_in_proj<<<dim3(gx, B), NW_IN * 32, smem_in, st>>>(p); launches++;
            AttnPrep a{};
            a.qg = e->qg; a.k = e->kbuf; a.v = e->vbuf; a.q_norm = L.q_norm; a.k_norm = L.k_norm; a.q_out = e->qn; a.g_out = e->gate;
            a.slab_stride = (size_t)e->n_ctx * kvd;
            a.kslab = e->kslab + (size_t)as * B * a.slab_stride; a.vslab = e->vslab + (size_t)as * B * a.slab_stride;
            a.pos = e->pos; a.npos_out = e->npos; a.hd = d.head_dim; a.n_head = d.n_head; a.n_head_kv = d.n_head_kv; a.n_rot = d.n_rot;
            a.theta = d.rope_theta; a.eps = d.rms_eps; a.bf16 = c->kv_bf16;
            k_attn_prep<<<dim3(d.n_head + 2 * d.n_head_kv, B), d.head_dim, d.head_dim * 4, st>>>(a); launches++;
            // one launch per sequence: each has its own slab and position
            for (int b = 0; b < B; ++b) {
                size_t po = (size_t)b * d.n_head * e->n_split;
                itb_attend_dev(c, st, e->qn + (size_t)b * qd, a.kslab + (size_t)b * a.slab_stride, a.vslab + (size_t)b * a.slab_stride, kvd, 0, 1,
                               d.head_dim, d.n_head, d.n_head_kv, 1.0f / sqrtf((float)d.head_dim), c->kv_bf16, e->npos + b,
                               e->gate + (size_t)b * qd, e->part_acc + po * d.head_dim, e->part_ml + po * 2, e->n_split,
                               e->att + (size_t)b * qd);
                launches += 2; c->launches -= 2;
            }
            OutProj o{e->att, qd, qd, L.wo, e->x, H};
            size_t smem_o = out_proj_smem(qd, NW);
            set_smem((const void*)k_out_proj, smem_o);
            k_out_proj<<<dim3(std::min(sms, std::max(1, H / 8)), B), NW * 32, smem_o, st>>>(o); launches++;
        }
        // routed FFN
        InProj f{};
        f.x = e->x; f.x_stride = H; f.norm_w = L.ffn_norm; f.eps = d.rms_eps; f.n_embd = H;
        f.nq = 2; f.q[0] = L.shared_gate; f.qout[0] = e->sg; f.qstride[0] = d.shared_ff; f.q[1] = L.shared_up; f.qout[1] = e->su; f.qstride[1] = d.shared_ff;
        f.nf = 2; f.f[0] = L.gate_inp; f.fout[0] = e->router; f.fstride[0] = d.n_expert;
        f.f[1] = L.shared_gate_inp; f.fout[1] = e->shlogit; f.fstride[1] = 1;
        f.xq_out = e->xq; f.xs_out = e->xs; f.exact = c->exact;
        int units = c->exact ? (d.n_expert + 31) / 32 + 1 : (d.n_expert + 3) / 4 + 1;
        int gxf = std::min(sms, std::max(units, (int)(2 * d.shared_ff) / 8));
        k_in_proj<<<dim3(gxf, B), NW_IN * 32, smem_in, st>>>(f); launches++;
        MoeGlu g{};
        g.router = e->router; g.n_expert = d.n_expert; g.n_used = d.n_expert_used; g.xq = e->xq; g.xs = e->xs; g.n_embd = H;
        g.gate = L.gate; g.up = L.up; g.h = e->h;
        g.ids_out = e->route_ids + (size_t)il * B * d.n_expert_used; g.w_out = e->route_w + (size_t)il * B * d.n_expert_used;
        size_t smem_g = moe_glu_smem(d.n_expert, H, NW);
        set_smem((const void*)k_moe_glu, smem_g);
        k_moe_glu<<<dim3(std::min(sms, std::max(1, (int)(d.n_expert_used * d.expert_ff) / 8)), B), NW * 32, smem_g, st>>>(g); launches++;
        MoeDown w{};
        w.h = e->h; w.n_used = d.n_expert_used; w.ff = d.expert_ff; w.ids = g.ids_out; w.wts = g.w_out; w.down = L.down;
        w.sg = e->sg; w.su = e->su; w.sff = d.shared_ff; w.shared_down = L.shared_down; w.logit = e->shlogit; w.x = e->x; w.x_stride = H;
        int gxd = std::min(sms, std::max(1, H / 8));
        size_t smem_d = moe_down_smem(d.n_expert_used, d.expert_ff, d.shared_ff, (H + gxd - 1) / gxd + 1, NW);
        set_smem((const void*)k_moe_down, smem_d);
        k_moe_down<<<dim3(gxd, B), NW * 32, smem_d, st>>>(w); launches++;
    }
    InProj hp{};
    hp.x = e->x; hp.x_stride = H; hp.norm_w = m->output_norm; hp.eps = d.rms_eps; hp.n_embd = H;
    hp.nq = 1; hp.q[0] = m->output; hp.qout[0] = e->logits; hp.qstride[0] = d.n_vocab; hp.exact = c->exact;
    k_in_proj<<<dim3(std::min(sms * 2, std::max(1, (int)d.n_vocab / 8)), B), NW_IN * 32, smem_in, st>>>(hp); launches++;
    k_argmax_advance<<<B, 1024, 0, st>>>(e->logits, d.n_vocab, e->tokens, e->pos, e->next, e->history, e->step_counter, B); launches++;
    k_bump<<<1, 1, 0, st>>>(e->step_counter); launches++;
    e->launches_per_step = launches;
}

extern "C" int itb_engine_create(itb_model* m, uint32_t n_ctx, uint32_t n_seq, itb_engine** out) {
    *out = nullptr;
    itb_ctx* c = m->c;
    if (!finalize(m)) return 1;
    if (n_seq == 0 || n_ctx == 0) { itb_fail_msg(c, "engine: n_seq and n_ctx must be positive"); return 1; }
    if (m->expert_hi && (m->expert_lo != 0 || m->expert_hi != m->d.n_expert)) {
        itb_fail_msg(c, "engine: this model holds an expert shard; use the expert-parallel engine"); return 1;
    }
    const itb_model_dims& d = m->d;
    auto e = std::make_unique<itb_engine>();
    e->m = m; e->c = c; e->n_ctx = n_ctx; e->B = n_seq;
    e->slot_of.resize(d.n_layer);
    for (uint32_t i = 0; i < d.n_layer; ++i) e->slot_of[i] = m->layers[i].recurrent ? (int)e->n_rec++ : (int)e->n_attn++;
    const size_t B = n_seq, H = d.n_embd, key_dim = (size_t)d.ssm_d_state * d.ssm_n_group, vd = d.ssm_d_inner, cd = 2 * key_dim + vd;
    const size_t qd = (size_t)d.head_dim * d.n_head, kvd = (size_t)d.head_dim * d.n_head_kv;
    e->n_split = (int)std::max<size_t>(1, std::min<size_t>({(size_t)64, ((size_t)n_ctx + 127) / 128, (size_t)(2 * c->sm_count) / d.n_head_kv + 1}));
    itb_engine* E = e.get();
    bool ok = dalloc(E, &e->kslab, (size_t)e->n_attn * B * n_ctx * kvd) && dalloc(E, &e->vslab, (size_t)e->n_attn * B * n_ctx * kvd) &&
              dalloc(E, &e->conv_state, (size_t)e->n_rec * B * cd * (d.ssm_d_conv - 1)) &&
              dalloc(E, &e->ssm_state, (size_t)e->n_rec * B * d.ssm_dt_rank * d.ssm_d_state * d.ssm_d_state) &&
              dalloc(E, &e->pos, B) && dalloc(E, &e->npos, B) && dalloc(E, &e->tokens, B) && dalloc(E, &e->next, B) && dalloc(E, &e->x, B * H) &&
              dalloc(E, &e->qkvc, B * cd) && dalloc(E, &e->z, B * vd) && dalloc(E, &e->alpha, B * d.ssm_dt_rank) &&
              dalloc(E, &e->beta, B * d.ssm_dt_rank) && dalloc(E, &e->zc, B * vd) && dalloc(E, &e->qg, B * 2 * qd) &&
              dalloc(E, &e->kbuf, B * kvd) && dalloc(E, &e->vbuf, B * kvd) && dalloc(E, &e->qn, B * qd) && dalloc(E, &e->gate, B * qd) &&
              dalloc(E, &e->att, B * qd) && dalloc(E, &e->part_acc, B * d.n_head * e->n_split * d.head_dim) &&
              dalloc(E, &e->part_ml, B * d.n_head * e->n_split * 2) && dalloc(E, &e->router, B * d.n_expert) &&
              dalloc(E, &e->shlogit, B) && dalloc(E, &e->sg, B * d.shared_ff) && dalloc(E, &e->su, B * d.shared_ff) &&
              dalloc(E, &e->h, B * d.n_expert_used * d.expert_ff) && dalloc(E, &e->logits, B * d.n_vocab) &&
              dalloc(E, &e->xq, B * H) && dalloc(E, &e->xs, B * H / 32) &&
              dalloc(E, &e->route_ids, (size_t)d.n_layer * B * d.n_expert_used) && dalloc(E, &e->route_w, (size_t)d.n_layer * B * d.n_expert_used) &&
              dalloc(E, &e->step_counter, 1);
    if (!ok) { for (void* p : e->allocs) cudaFree(p); return 1; }
    e->host_pos.assign(B, 0);
    cudaEventCreate(&e->ev0); cudaEventCreate(&e->ev1);
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) { itb_fail_msg(c, "engine: device error during set-up"); return 1; }
    *out = e.release();
    return 0;
}

static void drop_graph(itb_engine* e) {
    if (e->exec) cudaGraphExecDestroy(e->exec);
    if (e->graph) cudaGraphDestroy(e->graph);
    e->exec = nullptr; e->graph = nullptr;
}

extern "C" void itb_engine_destroy(itb_engine* e) {
    if (!e) return;
    cudaStreamSynchronize(e->c->stream);
    drop_graph(e);
    for (void* p : e->allocs) cudaFree(p);
    cudaFree(e->history); cudaFree(e->prompt);
    cudaEventDestroy(e->ev0); cudaEventDestroy(e->ev1);
    delete e;
}

// src/engine/mod.rs:296-308: back to an empty sequence; recurrent state and positions zeroed.
extern "C" void itb_engine_reset(itb_engine* e) {
    const itb_model_dims& d = e->m->d;
    size_t cd = 2 * (size_t)d.ssm_d_state * d.ssm_n_group + d.ssm_d_inner;
    cudaStream_t st = e->c->stream;
    cudaMemsetAsync(e->conv_state, 0, (size_t)e->n_rec * e->B * cd * (d.ssm_d_conv - 1) * 4, st);
    cudaMemsetAsync(e->ssm_state, 0, (size_t)e->n_rec * e->B * d.ssm_dt_rank * d.ssm_d_state * d.ssm_d_state * 4, st);
    cudaMemsetAsync(e->pos, 0, e->B * 4, st);
    cudaStreamSynchronize(st);
    std::fill(e->host_pos.begin(), e->host_pos.end(), 0u);
}
extern "C" uint32_t itb_engine_pos(itb_engine* e, uint32_t seq) { return seq < e->B ? e->host_pos[seq] : 0; }
extern "C" float itb_engine_last_ms(itb_engine* e) { return e->last_ms; }
extern "C" uint64_t itb_engine_launches_per_step(itb_engine* e) { return e->launches_per_step; }

static bool ensure_graph(itb_engine* e) {
    if (e->exec) return true;
    itb_ctx* c = e->c;
    cudaStream_t st = c->stream;
    // one eager step's worth of attribute set-up happens inside enqueue_step; capture it once
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return itb_fail_msg(c, "engine: cannot begin capture");
    enqueue_step(e, st);
    cudaError_t err = cudaStreamEndCapture(st, &e->graph);
    if (err != cudaSuccess) return itb_fail(c, "engine: capture", err);
    err = cudaGraphInstantiate(&e->exec, e->graph, 0);
    if (err != cudaSuccess) return itb_fail(c, "engine: graph instantiate", err);
    return true;
}

static bool run_steps(itb_engine* e, uint32_t steps, bool timed) {
    itb_ctx* c = e->c;
    if (!ensure_graph(e)) return false;
    for (uint32_t b = 0; b < e->B; ++b)
        if (e->host_pos[b] + steps > e->n_ctx) return itb_fail_msg(c, "context overflow: the step would write past n_ctx");  // src/model/qwen35.rs:984-990
    if (timed) cudaEventRecord(e->ev0, c->stream);
    for (uint32_t s = 0; s < steps; ++s) {
        cudaError_t err = cudaGraphLaunch(e->exec, c->stream);
        if (err != cudaSuccess) return itb_fail(c, "engine: graph launch", err);
    }
    c->launches += (uint64_t)steps * e->launches_per_step;
    if (timed) cudaEventRecord(e->ev1, c->stream);
    for (uint32_t b = 0; b < e->B; ++b) e->host_pos[b] += steps;
    return true;
}

extern "C" int itb_engine_decode(itb_engine* e, const uint32_t* tokens, float* logits_out, uint32_t* next_out) {
    itb_ctx* c = e->c;
    cudaStream_t st = c->stream;
    ITB_CUDA_RET(c, cudaMemcpyAsync(e->tokens, tokens, e->B * 4, cudaMemcpyHostToDevice, st), 1);
    if (!run_steps(e, 1, true)) return 1;
    if (next_out) cudaMemcpyAsync(next_out, e->next, e->B * 4, cudaMemcpyDeviceToHost, st);
    if (logits_out) cudaMemcpyAsync(logits_out, e->logits, (size_t)e->B * e->m->d.n_vocab * 4, cudaMemcpyDeviceToHost, st);
    ITB_CUDA_RET(c, cudaStreamSynchronize(st), 1);
    cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1);
    return 0;
}

extern "C" int itb_engine_decode_loop(itb_engine* e, const uint32_t* first, uint32_t steps, uint32_t* tokens_out) {
    itb_ctx* c = e->c;
    cudaStream_t st = c->stream;
    if (steps == 0) return 0;
    if (e->history_cap < steps) {
        cudaStreamSynchronize(st);
        drop_graph(e);  // the graph holds the history pointer
        cudaFree(e->history);
        ITB_CUDA_RET(c, cudaMalloc(&e->history, (size_t)steps * e->B * 4), 1);
        e->history_cap = steps;
    }
    ITB_CUDA_RET(c, cudaMemcpyAsync(e->tokens, first, e->B * 4, cudaMemcpyHostToDevice, st), 1);
    cudaMemsetAsync(e->step_counter, 0, 4, st);
    if (!run_steps(e, steps, true)) return 1;
    if (tokens_out) cudaMemcpyAsync(tokens_out, e->history, (size_t)steps * e->B * 4, cudaMemcpyDeviceToHost, st);
    ITB_CUDA_RET(c, cudaStreamSynchronize(st), 1);
    cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1);
    return 0;
}

// Prefill, token by token through the decode graph: the state left behind and the last logits are those of
// a batched pass (the reference asserts the two are identical, tests/qwen35.rs:94-139 there).
extern "C" int itb_engine_prefill(itb_engine* e, const uint32_t* tokens, size_t n, float* logits_out) {
    itb_ctx* c = e->c;
    cudaStream_t st = c->stream;
    if (n == 0) { itb_fail_msg(c, "prefill: no tokens supplied"); return 1; }
    for (uint32_t b = 0; b < e->B; ++b)
        if (e->host_pos[b] + n > e->n_ctx) { itb_fail_msg(c, "context overflow: the prompt would write past n_ctx"); return 1; }
    if (e->prompt_cap < n * e->B) {
        cudaStreamSynchronize(st);
        cudaFree(e->prompt);
        ITB_CUDA_RET(c, cudaMalloc(&e->prompt, n * e->B * 4), 1);
        e->prompt_cap = n * e->B;
    }
    std::vector<int32_t> tr(n * e->B);  // [t][b]
    for (size_t b = 0; b < e->B; ++b)
        for (size_t t = 0; t < n; ++t) {
            if (tokens[b * n + t] >= e->m->d.n_vocab) { itb_fail_msg(c, "token id out of range"); return 1; }
            tr[t * e->B + b] = (int32_t)tokens[b * n + t];
        }
    ITB_CUDA_RET(c, cudaMemcpyAsync(e->prompt, tr.data(), tr.size() * 4, cudaMemcpyHostToDevice, st), 1);
    cudaEventRecord(e->ev0, st);
    for (size_t t = 0; t < n; ++t) {
        cudaMemcpyAsync(e->tokens, e->prompt + t * e->B, e->B * 4, cudaMemcpyDeviceToDevice, st);
        if (!run_steps(e, 1, false)) return 1;
    }
    cudaEventRecord(e->ev1, st);
    if (logits_out) cudaMemcpyAsync(logits_out, e->logits, (size_t)e->B * e->m->d.n_vocab * 4, cudaMemcpyDeviceToHost, st);
    ITB_CUDA_RET(c, cudaStreamSynchronize(st), 1);
    cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1);
    return 0;
}

// src/engine/mod.rs:399-437 for sequence 0 of a single-sequence engine.
extern "C" long itb_engine_generate(itb_engine* e, const uint32_t* prompt, size_t n_prompt, size_t max_new, uint32_t* out) {
    itb_ctx* c = e->c;
    if (e->B != 1) { itb_fail_msg(c, "generate: single-sequence engines only"); return -1; }
    if (itb_engine_prefill(e, prompt, n_prompt, nullptr)) return -1;
    uint32_t next = 0;
    ITB_CUDA_RET(c, cudaMemcpy(&next, e->next, 4, cudaMemcpyDeviceToHost), -1);
    size_t produced = 0;
    for (size_t i = 0; i < max_new; ++i) {
        out[produced++] = next;
        if (produced == max_new) break;
        if (e->host_pos[0] + 1 >= e->n_ctx) break;  // StopReason::ContextFull
        uint32_t tok = next;
        if (itb_engine_decode(e, &tok, nullptr, &next)) return -1;
    }
    return (long)produced;
}

extern "C" int itb_engine_read_routes(itb_engine* e, int32_t* ids, size_t cap) {
    size_t n = (size_t)e->m->d.n_layer * e->B * e->m->d.n_expert_used;
    if (cap < n) { itb_fail_msg(e->c, "read_routes: buffer too small"); return 1; }
    ITB_CUDA_RET(e->c, cudaMemcpy(ids, e->route_ids, n * 4, cudaMemcpyDeviceToHost), 1);
    return 0;
}
extern "C" int itb_engine_read_ssm_state(itb_engine* e, uint32_t seq, uint32_t il, float* out, size_t len) {
    const itb_model_dims& d = e->m->d;
    if (il >= d.n_layer || !e->m->layers[il].recurrent || seq >= e->B) { itb_fail_msg(e->c, "read_ssm_state: not a recurrent layer"); return 1; }
    size_t per = (size_t)d.ssm_dt_rank * d.ssm_d_state * d.ssm_d_state;
    if (len != per) { itb_fail_msg(e->c, "read_ssm_state: wrong length"); return 1; }
    ITB_CUDA_RET(e->c, cudaStreamSynchronize(e->c->stream), 1);
    ITB_CUDA_RET(e->c, cudaMemcpy(out, e->ssm_state + ((size_t)e->slot_of[il] * e->B + seq) * per, per * 4, cudaMemcpyDeviceToHost), 1);
    return 0;
}
