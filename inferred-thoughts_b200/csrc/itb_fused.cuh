// Fused decode kernels of the engine: one kernel per dependent stage of a layer, written lean -- small loop
// bodies, 16 warps per block, prologues done once, and every activation quantised to Q8_0 by the kernel
// that produces it (the consumer's matmul would quantise it the same way, src/ops/naive.rs:49-56).
#pragma once
#include "itb_kernels.cuh"

namespace {

constexpr int RPG = 2;          // row groups per pass in the streaming GEMVs
constexpr int NWG = 16;         // warps per block in the GEMV kernels
constexpr int CONV_CAP = 8;     // rows per warp whose conv window and taps are fetched ahead (8 floats each)

// ------------------------------------------------------------------------------------------------------
// Input projections: RMSNorm + Q8_0 quantise prologue, then up to three Q8_0 matrices and two F32 matrices
// against the same row (src/model/qwen35.rs:1010, :1167-1179, :1262-1273, :1626). With conv_w set, rows of
// q[0] go through the depthwise causal conv (src/ops/naive.rs:275-315) in the epilogue -- the lane that owns
// a row also advances that channel's window -- and the PRE-activation sum is stored: the consumer applies SiLU.
struct InProj {
    const float* x; int x_stride;                 // [B][n_embd] residual stream
    const float* norm_w; float eps; int n_embd;
    int nq; DevQ8 q[3]; float* qout[3]; int qstride[3];
    int nf; DevF32 f[2]; float* fout[2]; int fstride[2];
    const float* conv_w; float* conv_state; int conv_kernel; size_t conv_state_stride;
    int8_t* xq_out; float* xs_out;                // optional copy of the quantised normed row, [B][n_embd]
    int exact; int br;                             // br: rows whose terms a warp collects before folding them together
    int f32_ring; int* err;                        // serial-k F32 rows through the block's ring (in_proj_smem counts it): the number of 32-row units, 0 = off; status word of its bounded waits
    int tl_slot;                                   // phase-timeline slot of this launch (-1: none)
    L2Hint hint;                                   // what the kernels after this one will stream
};

__global__ void __launch_bounds__(NWG * 32) k_in_proj(InProj p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int n = p.n_embd, nb = n / 32, gsh = lanes_shift(nb);
    const int b = blockIdx.y, wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    TL(TLK_IN_PROJ, 0);
    pdl_trigger();
    double* red = (double*)smem;
    float* xn = (float*)(red + 32);
    int8_t* xq = (int8_t*)(xn + n);
    float* xs = (float*)(xq + n);
    float* tile = xs + nb;                                        // 32*33 floats, serial-k F32 mode only
    const int tfl = p.br * (nb + 1);
    float* terms = tile + (p.exact ? 32 * 33 : 0) + wid * (tfl + CONV_CAP * 8);
    float* cpre = terms + tfl;
    // the block's ring for serial-k F32 rows: after every warp's scratch, 16-byte aligned, its mbarriers behind it
    // (offset arithmetic on the shared array itself: a pointer that went through an integer would be read with generic loads)
    const size_t ring_off = ((size_t)((const unsigned char*)(tile + (p.exact ? 32 * 33 : 0) + nw * (tfl + CONV_CAP * 8)) - smem) + 127) & ~(size_t)127;
    float* ring = (float*)(smem + ring_off);
    unsigned long long* ring_full = (unsigned long long*)(ring + F32S_FLOATS);
    unsigned long long* ring_empty = ring_full + F32S_STAGES;
    // serial-k F32 units: unit u belongs to block gridDim.x - 1 - u; there the last warp folds and the one before it feeds the
    // ring, and neither takes Q8_0 rows (the fold is the longest thing in the kernel)
    const int my_unit = p.f32_ring ? (int)gridDim.x - 1 - (int)blockIdx.x : -1;
    const bool unit_block = my_unit >= 0 && my_unit < p.f32_ring;
    const float* unit_w = nullptr; float* unit_out = nullptr; int unit_r0 = 0, unit_nr = 0;
    if (unit_block) {
        int u = my_unit;
        for (int m = 0; m < p.nf; ++m) {
            const int units = (p.f[m].n_out + 31) / 32;
            if (u < units) {
                unit_w = p.f[m].wt + (size_t)u * 32 * n; unit_out = p.fout[m] + (size_t)b * p.fstride[m];
                unit_r0 = u * 32; unit_nr = min(32, p.f[m].n_out - u * 32);
                break;
            }
            u -= units;
        }
        if (threadIdx.x == 0) {
            for (int i = 0; i < F32S_STAGES; ++i) {
                asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(ring_full + i)) : "memory");
                asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(ring_empty + i)) : "memory");
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    // Q8_0 rows go to the blocks without a unit when those are most of the grid: the folding warp then has its scheduler to
    // itself from the start (its fold is the longest thing in the kernel, and four warps to a scheduler slow its chain)
    const bool spare_units = p.f32_ring > 0 && 2 * p.f32_ring <= (int)gridDim.x;
    const int gq = spare_units ? (int)gridDim.x - p.f32_ring : (int)gridDim.x;
    const int nwq = unit_block ? nw - 2 : nw;                     // warps that take Q8_0 rows
    // this warp's share of the concatenated Q8_0 rows
    int total = 0;
    for (int m = 0; m < p.nq; ++m) total += p.q[m].n_out;
    int b0 = 0, b1 = 0, r0, r1;
    if ((int)blockIdx.x < gq) share(total, gq, blockIdx.x, b0, b1);
    share(b1 - b0, nwq, min(wid, nwq - 1), r0, r1);
    r0 += b0; r1 += b0;
    if (wid >= nwq) r1 = r0;
    const int keep = p.conv_kernel - 1;
    int conv_lo = 0;
    if (p.conv_w && r0 < min(r1, p.q[0].n_out)) {
        // conv window and taps of the rows this warp will finish, fetched before anything depends on them
        const int nr = min(min(r1, p.q[0].n_out) - r0, CONV_CAP);
        const float* cs = p.conv_state + (size_t)b * p.conv_state_stride + (size_t)r0 * keep;
        const float* cw = p.conv_w + (size_t)r0 * p.conv_kernel;
        for (int i = lane; i < nr * keep; i += 32) cpre[(i / keep) * 8 + i % keep] = cs[i];
        for (int i = lane; i < nr * p.conv_kernel; i += 32) cpre[(i / p.conv_kernel) * 8 + keep + i % p.conv_kernel] = cw[i];
        conv_lo = r0;
    }
    if (unit_block) {
        __syncthreads();                                          // the ring's barriers exist
        if (wid == nw - 2 && lane == 0)
            for (int t = 0; t < F32S_STAGES && t < n / F32S_K; ++t) f32_unit_issue(unit_w, t, ring, ring_full);
    }
    pdl_wait();
    TL(TLK_IN_PROJ, 1);
    const bool quantised = block_rms_norm(p.x + (size_t)b * p.x_stride, p.norm_w, n, p.eps, xn, red, xq, xs);
    TL(TLK_IN_PROJ, 2);
    if (!quantised) block_quant_q8(xn, n, xq, xs);
    TL(TLK_IN_PROJ, 3);
    if (p.xq_out && blockIdx.x == 0) {
        for (int i = threadIdx.x; i < n / 16; i += blockDim.x) ((uint4*)(p.xq_out + (size_t)b * n))[i] = ((const uint4*)xq)[i];
        for (int i = threadIdx.x; i < nb; i += blockDim.x) p.xs_out[(size_t)b * nb + i] = xs[i];
    }
    // F32 rows. Serial-k: this block's unit, if it has one (the weights' first stages were requested before the norm; see below).
    // Otherwise a row per warp handed out from the far end of the grid's warps: serial fold over staged products, or shuffle tree.
    if (p.f32_ring) {
        if (unit_block && wid == nw - 1)
            f32_rows32_serial(n, unit_r0, unit_nr, xn, ring, ring_full, ring_empty, p.err, [&](int row, float v) { unit_out[row] = v; });
        else if (unit_block && wid == nw - 2 && lane == 0)
            f32_unit_feed(unit_w, n, ring, ring_full, ring_empty, p.err);
    } else {
        const int ngw = gridDim.x * nw, gw = ngw - 1 - (wid * (int)gridDim.x + (int)blockIdx.x);
        int ubase = 0;
#pragma unroll 1
        for (int m = 0; m < p.nf; ++m) {
            float* o = p.fout[m] + (size_t)b * p.fstride[m];
            for (int r = gw - ubase; r < p.f[m].n_out; r += ngw) {
                if (r < 0) continue;
                if (p.exact) f32_rows<true>(p.f[m].w, n, r, r + 1, xn, terms, [&](int row, float v) { o[row] = v; }, tfl);
                else f32_rows<false>(p.f[m].w, n, r, r + 1, xn, terms, [&](int row, float v) { o[row] = v; });
            }
            ubase = (ubase + p.f[m].n_out) % ngw;
        }
    }
    int base = 0;
#pragma unroll 1
    for (int m = 0; m < p.nq; ++m) {
        const int lo = max(r0, base) - base, hi = min(r1, base + p.q[m].n_out) - base;
        if (lo < hi) {
            float* o = p.qout[m] + (size_t)b * p.qstride[m];
            if (m == 0 && p.conv_w) {
                float* cs = p.conv_state + (size_t)b * p.conv_state_stride;
                const float* cw = p.conv_w;
                const int kernel = p.conv_kernel;
                rows_batched<MK_Q8, 2, 2>((const uint8_t*)p.q[m].q, (const uint8_t*)p.q[m].s, n, lo, hi, xq, xs, terms, p.br, gsh, [&](int row, float v) {
                    float* past = cs + (size_t)row * keep;
                    const bool pre = row - conv_lo < CONV_CAP;
                    const float* pin = pre ? cpre + (row - conv_lo) * 8 : past;
                    const float* w = pre ? cpre + (row - conv_lo) * 8 + keep : cw + (size_t)row * kernel;
                    float sum = 0.0f;
                    for (int k = 0; k < keep; ++k) sum += pin[k] * w[k];
                    sum += v * w[keep];
                    o[row] = sum;
                    for (int k = 0; k + 1 < keep; ++k) past[k] = pin[k + 1];
                    past[keep - 1] = v;
                });
            } else {
                rows_batched<MK_Q8, 2, 2>((const uint8_t*)p.q[m].q, (const uint8_t*)p.q[m].s, n, lo, hi, xq, xs, terms, p.br, gsh,
                                          [&](int row, float v) { o[row] = v; });
            }
        }
        base += p.q[m].n_out;
    }
    // this warp's own rows are in: the memory system is free for what the next kernels will stream
    if (wid == 0) l2_hint(p.hint, blockIdx.y * gridDim.x + blockIdx.x, gridDim.x * gridDim.y, lane);
    TL(TLK_IN_PROJ, 4);
    TL(TLK_IN_PROJ, 5);
}
// br a multiple of the pass size 2 * (32 >> gsh)
size_t in_proj_smem(int n, int exact, int br, int f32_ring = 0) {
    int nb = n / 32;
    return 256 + (size_t)n * 5 + (size_t)nb * 4 + (exact ? 32 * 33 * 4 : 0) + (size_t)NWG * (br * (nb + 1) + CONV_CAP * 8) * 4 + 64 +
           (f32_ring ? (size_t)F32S_FLOATS * 4 + 2 * F32S_STAGES * 8 + 128 : 0);
}

// ------------------------------------------------------------------------------------------------------
// Output projection with the residual add fused: x[b] += W . a[b], the activation arriving already quantised
// (src/model/qwen35.rs:1017, :1220, :1325).
struct OutProj { const int8_t* aq; const float* as; int n_in; DevQ8 w; float* x; int x_stride; int br; int tl_slot; L2Hint hint; };
__global__ void __launch_bounds__(NWG * 32) k_out_proj(OutProj p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int n = p.n_in, nb = n / 32, gsh = lanes_shift(nb);
    const int b = blockIdx.y, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int8_t* aq = (int8_t*)smem;
    float* as = (float*)(aq + n);
    float* terms = as + nb + wid * (p.br * (nb + 1));
    int b0, b1, r0, r1;
    share(p.w.n_out, gridDim.x, blockIdx.x, b0, b1);
    share(b1 - b0, nw, wid, r0, r1);
    TL(TLK_OUT_PROJ, 0);
    pdl_trigger();
    pdl_wait();
    TL(TLK_OUT_PROJ, 1);
    for (int i = threadIdx.x; i < n / 16; i += blockDim.x) ((uint4*)aq)[i] = ((const uint4*)(p.aq + (size_t)b * n))[i];
    for (int i = threadIdx.x; i < nb; i += blockDim.x) as[i] = p.as[(size_t)b * nb + i];
    __syncthreads();
    TL(TLK_OUT_PROJ, 2);
    float* x = p.x + (size_t)b * p.x_stride;
    rows_batched<MK_Q8, 1, 4>((const uint8_t*)p.w.q, (const uint8_t*)p.w.s, n, b0 + r0, b0 + r1, aq, as, terms, p.br, gsh,
                              [&](int row, float v) { x[row] += v; });
    if (wid == 0) l2_hint(p.hint, blockIdx.y * gridDim.x + blockIdx.x, gridDim.x * gridDim.y, threadIdx.x & 31);
    TL(TLK_OUT_PROJ, 3);
}
size_t out_proj_smem(int n, int br) {
    int nb = n / 32;
    return (size_t)n + (size_t)nb * 4 + (size_t)NWG * br * (nb + 1) * 4 + 64;
}

// ------------------------------------------------------------------------------------------------------
// GatedDeltaNet core for one (value head, sequence): SiLU of the conv sums, l2-norm of q and k, gated delta
// rule over the head's [sv][sk] state, gated RMSNorm, the SiLU(z) gate, and the Q8_0 quantisation the output
// projection would apply (src/model/qwen35.rs:1280-1325, src/ops/naive.rs:86-135, :254-273). One thread per
// value row, keys walked serially so every sum has the CPU's order.
struct GdnCore {
    const float* conv; int conv_stride;           // [B][conv_dim] = q | k | v conv sums (pre-SiLU)
    const float* z; const float* alpha; const float* beta;
    const float* ssm_a; const float* dt_bias; const float* ssm_norm;
    float* state; size_t state_stride;
    int8_t* out_q; float* out_s;                  // [B][value_dim] int8, [B][value_dim/32] scales
    int sk, sv, n_k, n_v; float eps;
    int tl_slot;
};
template <int SK>
__global__ void __launch_bounds__(256) k_gdn_core(GdnCore p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int sk = SK, sv = SK, LD = SK * SK / 4 / 256;   // float4 loads per thread
    const int h = blockIdx.x, b = blockIdx.y, kh = h % p.n_k, tid = threadIdx.x;
    const int lane = tid & 31, wid = tid >> 5;
    float* S = (float*)smem;                 // [sv][sk+1]
    float* kq = S + sv * (sk + 1);           // k[sk] | q[sk]
    float* o = kq + 2 * sk;                  // [sv]
    __shared__ double red2[8];
    __shared__ float s_gb[2];
    const int key_dim = p.n_k * sk;
    const float* cv = p.conv + (size_t)b * p.conv_stride;
    float* sg = p.state + (size_t)b * p.state_stride + (size_t)h * sv * sk;
    TL(TLK_GDN_CORE, 0);
    pdl_trigger();
    // the state belongs to this layer alone: its loads are in flight while the predecessor kernel finishes
    float4 ld[LD];
#pragma unroll
    for (int i = 0; i < LD; ++i) ld[i] = __ldcs((const float4*)sg + tid + i * 256);
    const float r_dt = p.dt_bias[h], r_a = p.ssm_a[h], r_nw = p.ssm_norm[tid < sv ? tid : 0];
    pdl_wait();
    TL(TLK_GDN_CORE, 1);
    // every other global operand is requested now too, so the kernel has one memory round trip
    const float r_alpha = p.alpha[(size_t)b * p.n_v + h], r_beta = p.beta[(size_t)b * p.n_v + h];
    const size_t oidx = (size_t)b * p.n_v * sv + (size_t)h * sv + (tid < sv ? tid : 0);
    const float r_z = p.z[oidx];
    // SiLU of this head's conv sums: threads [0, 2*sk) take k then q, threads [0, sv) their v element later
    if (tid < 2 * sk) kq[tid] = silu_f(cv[(tid < sk ? key_dim : 0) + kh * sk + (tid < sk ? tid : tid - sk)]);
    float vj = 0.0f;
    if (tid < sv) vj = silu_f(cv[2 * key_dim + h * sv + tid]);
#pragma unroll
    for (int i = 0; i < LD; ++i) {
        int e = (tid + i * 256) * 4, r = e / sk, c0 = e % sk;
        float* d = S + r * (sk + 1) + c0;
        d[0] = ld[i].x; d[1] = ld[i].y; d[2] = ld[i].z; d[3] = ld[i].w;
    }
    __syncthreads();
    TL(TLK_GDN_CORE, 2);
    // warp 0 normalises k, warp 1 normalises q (f64 tree sum, narrowing before the root)
    if (wid < 2) {
        float* src = kq + wid * sk;
        double acc = 0.0;
        for (int i = lane; i < sk; i += 32) { float v = src[i]; acc += (double)(v * v); }
        acc = warp_sum_d(acc);
        float sc = 1.0f / fmaxf(sqrtf((float)acc), p.eps);
        float qs = 1.0f / sqrtf((float)sk);
        for (int i = lane; i < sk; i += 32) {
            float v = src[i] * sc;
            src[i] = wid == 0 ? v : v * qs;
        }
    } else if (wid == 2) {
        // the head's decay and write strength, once (three library-exact exponentials and a logarithm: on the f64 unit they were
        // half of the update phase when each of its four warps computed them for itself)
        float a = r_alpha + r_dt;
        float sp = a > 20.0f ? a : log_f(1.0f + exp_f(a));
        float g = exp_f(sp * r_a);
        float bt = sigmoid_f(r_beta);
        if (lane == 0) { s_gb[0] = g; s_gb[1] = bt; }
    }
    __syncthreads();
    TL(TLK_GDN_CORE, 3);
    if (tid < sv) {
        const float g = s_gb[0], bt = s_gb[1];
        // the thread's state row lives in registers for both passes (src/ops/naive.rs:109-132 order: decay, predict, update, read out)
        float* row = S + tid * (sk + 1);
        float R[SK];
#pragma unroll
        for (int i = 0; i < SK; ++i) R[i] = row[i];
        float pred = 0.0f;
#pragma unroll
        for (int i = 0; i < SK; i += 4) {
            const float4 k4 = *(const float4*)(kq + i);
            R[i] = R[i] * g; pred += R[i] * k4.x;
            R[i + 1] = R[i + 1] * g; pred += R[i + 1] * k4.y;
            R[i + 2] = R[i + 2] * g; pred += R[i + 2] * k4.z;
            R[i + 3] = R[i + 3] * g; pred += R[i + 3] * k4.w;
        }
        float d = bt * (vj - pred);
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < SK; i += 4) {
            const float4 k4 = *(const float4*)(kq + i), q4 = *(const float4*)(kq + SK + i);
            R[i] = R[i] + k4.x * d; acc += R[i] * q4.x;
            R[i + 1] = R[i + 1] + k4.y * d; acc += R[i + 1] * q4.y;
            R[i + 2] = R[i + 2] + k4.z * d; acc += R[i + 2] * q4.z;
            R[i + 3] = R[i + 3] + k4.w * d; acc += R[i + 3] * q4.w;
        }
#pragma unroll
        for (int i = 0; i < SK; ++i) row[i] = R[i];
        o[tid] = acc;
    }
    __syncthreads();
    TL(TLK_GDN_CORE, 4);
    {
        double acc = 0.0;
        for (int i = tid; i < sv; i += blockDim.x) acc += (double)(o[i] * o[i]);
        acc = warp_sum_d(acc);
        if (lane == 0) red2[wid] = acc;
        __syncthreads();
        double tot = 0.0;
        if (lane == 0) for (int w = 0; w < 8; ++w) tot += red2[w];      // one lane per warp adds (slow f64 unit), the rest get it by shuffle
        tot = __shfl_sync(0xffffffffu, tot, 0);
        float mean = (float)(tot / (double)sv);
        float sc = 1.0f / sqrtf(mean + p.eps);
        if (tid < sv) {   // whole warps: sv is a multiple of 32
            float core = o[tid] * sc * r_nw;
            size_t idx = oidx;
            float val = silu_f(r_z) * core;
            float dq;
            int8_t q = warp_quant_q8(val, &dq);
            p.out_q[idx] = q;
            if (lane == 0) p.out_s[idx / 32] = dq;
        }
    }
#pragma unroll
    for (int i = 0; i < LD; ++i) {
        int e = (tid + i * 256) * 4, r = e / sk, c0 = e % sk;
        const float* s = S + r * (sk + 1) + c0;
        __stcs((float4*)sg + tid + i * 256, make_float4(s[0], s[1], s[2], s[3]));
    }
    TL(TLK_GDN_CORE, 5);
}

// ------------------------------------------------------------------------------------------------------
// Attention prologue per head: de-interleave q|gate, QK RMSNorm, partial NEOX RoPE at the sequence's
// position, KV write (src/model/qwen35.rs:1175-1198). grid (n_head + 2*n_head_kv, B), block = head_dim.
struct AttnPrep {
    const float* qg; const float* k; const float* v;
    const float* q_norm; const float* k_norm;
    float* q_out; float* g_out;
    uint16_t* kslab; uint16_t* vslab; size_t slab_stride;
    const int* pos; int* npos_out;
    int hd, n_head, n_head_kv, n_rot; float theta, eps; int bf16;
    int tl_slot;
};
__global__ void k_attn_prep(AttnPrep p) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* val = (float*)smem;
    __shared__ double red[8];
    const int job = blockIdx.x, b = blockIdx.y, d = threadIdx.x, hd = p.hd, kvd = p.n_head_kv * hd;
    TL(TLK_ATTN_PREP, 0);
    pdl_trigger(); pdl_wait();
    TL(TLK_ATTN_PREP, 1);
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
        if ((d & 31) == 0) for (int w = 0; w < hd / 32; ++w) tot += red[w];      // one lane per warp adds (slow f64 unit), the rest get it by shuffle
        tot = __shfl_sync(0xffffffffu, tot, 0);
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

// Combine of the attention splits for the engine: as k_attn_combine, over the splits that hold positions only,
// with the sigmoid output gate (src/model/qwen35.rs:1216-1218) and the Q8_0 quantisation the output projection
// would apply. grid (B * n_head), block hd.
__global__ void k_attn_combine_q(const float* part_acc, const float* part_ml, int n_split, int hd, const float* gate,
                                 const int* n_pos_dev, int n_head, int8_t* out_q, float* out_s) {
    const size_t th = blockIdx.x;
    const int d = threadIdx.x, b = (int)(th / n_head);
    pdl_trigger(); pdl_wait();
    const int n_pos = n_pos_dev[b], per = max(ATTN_MIN_SPLIT, (n_pos + n_split - 1) / n_split), n_act = (n_pos + per - 1) / per;
    // splits in trips of 8 with every load of a trip in flight; the combine itself keeps ascending split order
    const float gt = gate[th * hd + d];
    float M = -INFINITY;
    for (int s0 = 0; s0 < n_act; s0 += 8) {
        float mv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) mv[j] = s0 + j < n_act ? part_ml[(th * n_split + s0 + j) * 2] : -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) M = fmaxf(M, mv[j]);
    }
    float L = 0.0f, A = 0.0f;
    for (int s0 = 0; s0 < n_act; s0 += 8) {
        float mv[8], lv[8], av[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const bool in = s0 + j < n_act;
            mv[j] = in ? part_ml[(th * n_split + s0 + j) * 2] : -INFINITY;
            lv[j] = in ? part_ml[(th * n_split + s0 + j) * 2 + 1] : 0.0f;
            av[j] = in ? part_acc[(th * n_split + s0 + j) * hd + d] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (s0 + j < n_act) {
                const float c = mv[j] == -INFINITY ? 0.0f : __expf(mv[j] - M);
                L += lv[j] * c;
                A += av[j] * c;
            }
        }
    }
    float v = A / L;
    v *= sigmoid_f(gt);
    float dq;
    int8_t q = warp_quant_q8(v, &dq);
    out_q[th * hd + d] = q;
    if ((d & 31) == 0) out_s[(th * hd + d) / 32] = dq;
}

// ------------------------------------------------------------------------------------------------------
// Routed experts, gated half. One block per 32 output rows of one pick (so the block can quantise its own
// Q8_0 block of the result), plus one block per 32 rows of the shared expert's activation.
// Warp 0 redoes the routing (softmax over all experts, top-k; src/model/qwen35.rs:1626-1638,
// src/ops/mod.rs:1191-1216) while the others fetch the activation; then
// h = silu(gate_e . x * s_g) * (up_e . x * s_u) (src/ops/mod.rs:1105-1117) -> Q8_0.
constexpr int MOE_CAND = 512;   // 32 groups x 16 picks at most (n_expert <= 1024, n_used <= 16)
struct MoeGlu {
    const float* router; int n_expert, n_used;
    const int8_t* xq; const float* xs; int n_embd;
    DevFp4 gate, up;
    const float* sg; const float* su; int sff;     // shared expert's gate/up outputs [B][sff]
    int8_t* hq; float* hs;                          // [B][n_used*ff] int8, [B][n_used*ff/32]
    int8_t* sq; float* ss;                          // [B][sff] int8, [B][sff/32]: silu(sg)*su quantised
    int32_t* ids_out; float* w_out;
    int shared_row;                                 // -1: every row has a shared expert activation; r: only row r, held at index 0 (expert-parallel step)
    // expert-parallel step over peer memory: row b's quantised activation and router logits were stored into this GPU's memory
    // by rank b; its flag wait_flags[b] reaches *wait_seq when they are all there (bounded wait; *err set if it runs out)
    const unsigned* wait_flags; const unsigned* wait_seq; int* err;
    const uint8_t* down_nib; const uint8_t* down_sc; size_t down_bytes;   // the down stack (nibble bytes per expert), for the L2 hint; null: none
    int tl_slot;
};
constexpr int EP_WAIT_FAIL = 0x7002;
// Bounded wait of one thread for a flag another GPU stores (system scope); the caller synchronises its block afterwards.
__device__ __forceinline__ void ep_wait_flag(const unsigned* flag, unsigned seq, int* err) {
    if (err && *(volatile int*)err) return;      // a wait of this step already ran out: the step is lost, do not wait again
    const long long t0 = clock64();
    for (;;) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v == seq) return;
        if (clock64() - t0 > 10000000000ll) { if (err) atomicExch(err, EP_WAIT_FAIL); return; }     // about five seconds: ranks may enter a step that far apart
    }
}
__global__ void __launch_bounds__(NWG * 32) k_moe_glu(MoeGlu p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int32_t s_ids[16];
    __shared__ float s_wts[16];
    __shared__ float s_gu[64];
    __shared__ float s_sum;
    __shared__ float s_cand_p[MOE_CAND];        // the first n_used of every 32-group: probability and id
    __shared__ int s_cand_i[MOE_CAND];
    const int n = p.n_embd, nb = n / 32, nsb = n / 16, gsh = lanes_shift(nb), ff = p.gate.n_out, upp = ff / 32;
    const int b = blockIdx.y, tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    const int unit = blockIdx.x, n_units = p.n_used * upp;
    TL(TLK_MOE_GLU, 0);
    pdl_trigger(); pdl_wait();
    TL(TLK_MOE_GLU, 1);
    if (unit >= n_units) {
        // shared expert: silu(gate) * up for 32 elements, quantised (src/model/qwen35.rs:1669-1678)
        if (wid == 0 && (p.shared_row < 0 || p.shared_row == b)) {
            const size_t sb = p.shared_row < 0 ? (size_t)b : 0;
            const int k = (unit - n_units) * 32 + lane;
            float v = silu_f(p.sg[sb * p.sff + k]) * p.su[sb * p.sff + k];
            float dq;
            int8_t q = warp_quant_q8(v, &dq);
            p.sq[sb * p.sff + k] = q;
            if (lane == 0) p.ss[sb * (p.sff / 32) + (unit - n_units)] = dq;
        }
        return;
    }
    if (p.wait_flags) {
        if (tid == 0) ep_wait_flag(p.wait_flags + b, *p.wait_seq, p.err);
        __syncthreads();
    }
    float* probs = (float*)smem;                  // [n_expert rounded up to 32]
    int8_t* xq = (int8_t*)(probs + ((p.n_expert + 31) & ~31));
    float* xs = (float*)(xq + n);
    float* terms = xs + nb + wid * terms_floats(4, gsh, nsb);
    {
        // softmax numerators (src/ops/naive.rs:362-376) by the whole block: every warp finds the max itself
        const float* lg = p.router + (size_t)b * p.n_expert;
        float mx = -INFINITY;
        if (p.n_expert <= 512) {
            float lv[16];   // every load of the warp's pass over the logits in flight at once
#pragma unroll
            for (int j = 0; j < 16; ++j) lv[j] = lane + 32 * j < p.n_expert ? lg[lane + 32 * j] : -INFINITY;
#pragma unroll
            for (int j = 0; j < 16; ++j) mx = fmaxf(mx, lv[j]);
        } else {
            for (int i = lane; i < p.n_expert; i += 32) mx = fmaxf(mx, lg[i]);
        }
        mx = warp_max(mx);
        const int ne32 = (p.n_expert + 31) & ~31;
        for (int i = tid; i < ne32; i += blockDim.x) probs[i] = i < p.n_expert ? exp_f(lg[i] - mx) : 0.0f;
        for (int i = tid; i < n / 16; i += blockDim.x) ((uint4*)xq)[i] = ((const uint4*)(p.xq + (size_t)b * n))[i];
        for (int i = tid; i < nb; i += blockDim.x) xs[i] = p.xs[(size_t)b * nb + i];
    }
    __syncthreads();
    TL(TLK_MOE_GLU, 2);
    // softmax denominator: serial sum in index order (src/ops/naive.rs:362-376), one thread
    if (tid == 0) {
        float sum = 0.0f;
#pragma unroll 1
        for (int i0 = 0; i0 < p.n_expert; i0 += 32) {
            float4 q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = *(const float4*)(probs + i0 + 4 * j);
            const int lim = p.n_expert - i0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (4 * j < lim) sum += q[j].x;
                if (4 * j + 1 < lim) sum += q[j].y;
                if (4 * j + 2 < lim) sum += q[j].z;
                if (4 * j + 3 < lim) sum += q[j].w;
            }
        }
        s_sum = sum;
    }
    __syncthreads();
    {
        const float sum = s_sum;
        for (int i = tid; i < p.n_expert; i += blockDim.x) probs[i] /= sum;
    }
    __syncthreads();
    // top-k without serial rounds, in two stages of counting. An expert's place in an order is the number of experts
    // that beat it: greater probability, or equal and lower id (src/ops/mod.rs:1191-1216 picks by strict '>' scanning
    // ascending ids). Stage 1: every 32-group ranks itself by shuffles and keeps its first n_used; stage 2: those
    // candidates (the overall picks are among them) are ranked against each other.
    {
        const int ng = (p.n_expert + 31) >> 5, nu = p.n_used;
        for (int g = wid; g < ng; g += (int)(blockDim.x >> 5)) {
            const int t = g * 32 + lane;
            const float v = t < p.n_expert ? probs[t] : -1.0f;
            int rank = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float q = __shfl_sync(0xffffffffu, v, j);
                rank += (int)(q > v) | ((int)(q == v) & (int)(j < lane));   // bitwise: no branches
            }
            if (rank < nu) { s_cand_p[g * nu + rank] = v; s_cand_i[g * nu + rank] = t < p.n_expert ? t : -1; }
        }
        __syncthreads();
        const int cnt = ng * nu;
        for (int c = tid; c < cnt; c += blockDim.x) {
            const float v = s_cand_p[c];
            const int id = s_cand_i[c];
            if (id < 0) continue;
            int rank = 0;
#pragma unroll 8
            for (int j = 0; j < cnt; ++j) {   // unrolled so the shared-memory reads run ahead of the compares
                const float q = s_cand_p[j];
                const int qi = s_cand_i[j];
                rank += (int)(qi >= 0) & ((int)(q > v) | ((int)(q == v) & (int)(qi < id)));
            }
            if (rank < nu) { s_ids[rank] = id; s_wts[rank] = v; }
        }
    }
    __syncthreads();
    if (tid == 0) {
        float sum = 0.0f;
        for (int r = 0; r < p.n_used; ++r) sum += s_wts[r];                 // summed in pick order (src/ops/mod.rs:1211)
        const float denom = fmaxf(sum, 6.103515625e-5f);
        for (int r = 0; r < p.n_used; ++r) {
            const float w = s_wts[r] / denom;
            s_wts[r] = w;
            if (unit == 0) { p.ids_out[(size_t)b * p.n_used + r] = s_ids[r]; p.w_out[(size_t)b * p.n_used + r] = w; }
        }
    }
    __syncthreads();
    TL(TLK_MOE_GLU, 3);
    const int pick = unit / upp, row0 = (unit % upp) * 32;
    const int el = s_ids[pick] - p.gate.expert_lo;
    if (el < 0 || el >= p.gate.n_expert) return;   // this pick's expert lives on another device
    // 64 row-dots (32 gate rows, 32 up rows) spread over the block's warps
    const size_t eo = (size_t)el * ff;
    const bool has_g = p.gate.scale2 != nullptr, has_u = p.up.scale2 != nullptr;
    const float sg2 = has_g ? p.gate.scale2[el] : 1.0f, su2 = has_u ? p.up.scale2[el] : 1.0f;   // in flight under the row dots
    int k0, k1;
    share(64, blockDim.x >> 5, wid, k0, k1);
    const uint8_t* gn = p.gate.nib + eo * (n / 2); const uint8_t* gs = p.gate.sc + eo * nsb;
    const uint8_t* un = p.up.nib + eo * (n / 2); const uint8_t* us = p.up.sc + eo * nsb;
    rows_list<MK_FP4, 4, 2>(k1 - k0, n, terms, gsh,
        [&](int k, const uint8_t*& pa, const uint8_t*& pb, const int8_t*& q, const float*& s) {
            const int kk = k0 + k, row = row0 + (kk & 31);
            pa = (kk < 32 ? gn : un) + (size_t)row * (n / 2);
            pb = (kk < 32 ? gs : us) + (size_t)row * nsb;
            q = xq; s = xs;
        },
        [&](int k, float v) { s_gu[k0 + k] = v; });
    if (p.down_nib && b < 4 && wid == (int)(blockDim.x >> 5) - 1) {
        // this pick's down-projection weights, which the next kernel streams: into L2 while this one runs (the pick's blocks share them out)
        L2Hint h{};
        h.p[0] = p.down_nib + (size_t)el * p.down_bytes; h.n[0] = (unsigned)p.down_bytes;
        h.p[1] = p.down_sc + (size_t)el * (p.down_bytes / 8); h.n[1] = (unsigned)(p.down_bytes / 8);
        l2_hint(h, unit % upp, upp, lane);
    }
    __syncthreads();
    TL(TLK_MOE_GLU, 4);
    if (wid == 0) {
        float g = s_gu[lane], u = s_gu[32 + lane];
        if (has_g) g = g * sg2;
        if (has_u) u = u * su2;
        float v = silu_f(g) * u;
        float dq;
        int8_t q = warp_quant_q8(v, &dq);
        p.hq[((size_t)b * p.n_used + pick) * ff + row0 + lane] = q;
        if (lane == 0) p.hs[((size_t)b * p.n_used + pick) * upp + unit % upp] = dq;
    }
    TL(TLK_MOE_GLU, 5);
}
size_t moe_glu_smem(int n_expert, int n) {
    int nb = n / 32, gsh = lanes_shift(nb);
    return (size_t)((n_expert + 31) & ~31) * 4 + n + (size_t)nb * 4 + (size_t)NWG * terms_floats(4, gsh, n / 16) * 4 + 64;
}

// ------------------------------------------------------------------------------------------------------
// Routed experts, second half, with the whole FFN tail fused: down projections of the picks and of the
// shared expert, the weighted sum in pick order, the sigmoid-gated shared term and the residual add
// (src/model/qwen35.rs:1659-1699, src/ops/mod.rs:1134-1171, src/model/qwen35.rs:1090). A warp takes one
// output row at a time and runs all its streams (picks + shared) in one pass, so their loads share one round trip.
struct MoeDown {
    const int8_t* hq; const float* hs; int n_used, ff;
    const int32_t* ids; const float* wts;
    DevFp4 down;
    const int8_t* sq; const float* ss; int sff;
    DevQ8 shared_down;
    const float* logit;
    float* x; int x_stride;
    int local_only; float* partial;
    // expert-parallel step: rows are the gathered rows of all ranks; every local pick's output row goes to
    // o_pairs[(b * n_used + k)][n_out] (others are left as they are: zero), and only row own_row (activation at index 0)
    // gets its shared-expert row into shd; no combine and no residual here.
    float* o_pairs; int own_row; float* shd;
    float* o_rows[8];                               // non-null: row b's picks go to o_rows[b][k][n_out] (rank b's memory) instead of o_pairs
    int tl_slot;
};
template <int RP, bool PAIRS = false>
__global__ void __launch_bounds__(NWG * 32) k_moe_down(MoeDown p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_el[16];
    __shared__ float s_wt[16];
    __shared__ float s_g;
    __shared__ int s_loc[16], s_nloc;        // picks whose expert is stored here, in pick order (expert-parallel pairs mode)
    const int ff = p.ff, sff = p.sff, nbf = ff / 32, nbs = sff / 32, nsb = ff / 16;
    const int gf = lanes_shift(nbf), gs = lanes_shift(nbs);
    const int b = blockIdx.y, tid = threadIdx.x, wid = tid >> 5, nw = blockDim.x >> 5, lane = tid & 31;
    const int n_out = p.down.n_out;
    int8_t* hq = (int8_t*)smem;                           // [n_used][ff]
    float* hs = (float*)(hq + p.n_used * ff);             // [n_used][nbf]
    int8_t* sq = (int8_t*)(hs + p.n_used * nbf);          // [sff]
    float* ss = (float*)(sq + sff);                       // [nbs]
    const int tf = max(terms_floats(RP, gf, nsb), terms_floats(1, gs, nbs));
    float* terms = ss + nbs + wid * (tf + 32);
    float* outv = terms + tf;                             // this warp's per-stream results
    int b0, b1, r0, r1;
    share(n_out, gridDim.x, blockIdx.x, b0, b1);
    share(b1 - b0, nw, wid, r0, r1);
    TL(TLK_MOE_DOWN, 0);
    pdl_trigger();
    pdl_wait();
    TL(TLK_MOE_DOWN, 1);
    for (int i = tid; i < p.n_used * ff / 16; i += blockDim.x) ((uint4*)hq)[i] = ((const uint4*)(p.hq + (size_t)b * p.n_used * ff))[i];
    for (int i = tid; i < p.n_used * nbf; i += blockDim.x) hs[i] = p.hs[(size_t)b * p.n_used * nbf + i];
    constexpr bool pairs = PAIRS;            // compile-time: the one-GPU kernel carries none of the expert-parallel branches
    const size_t shb = pairs ? 0 : (size_t)b;        // where this row's shared-expert activation and gate logit sit
    if (!pairs || b == p.own_row) {
        for (int i = tid; i < sff / 16; i += blockDim.x) ((uint4*)sq)[i] = ((const uint4*)(p.sq + shb * sff))[i];
        for (int i = tid; i < nbs; i += blockDim.x) ss[i] = p.ss[shb * nbs + i];
    }
    if (tid < p.n_used) {
        int el = p.ids[(size_t)b * p.n_used + tid] - p.down.expert_lo;
        s_el[tid] = (el < 0 || el >= p.down.n_expert) ? -1 : el;
        s_wt[tid] = p.wts[(size_t)b * p.n_used + tid];
    }
    if (tid == 32 && !pairs) s_g = sigmoid_f(p.logit[b]);
    __syncthreads();
    if (pairs && tid == 0) { int n = 0; for (int k = 0; k < p.n_used; ++k) if (s_el[k] >= 0) s_loc[n++] = k; s_nloc = n; }
    if (pairs) __syncthreads();
    TL(TLK_MOE_DOWN, 2);
    const bool has_s = p.down.scale2 != nullptr;
    float* x = p.x + (size_t)b * p.x_stride;
    // lane k keeps pick k's second scale; the load is issued here and first used after the row dots, so it costs no round trip
    const float s2k = (has_s && lane < p.n_used && s_el[lane] >= 0) ? p.down.scale2[s_el[lane]] : 1.0f;
#pragma unroll 1
    for (int row = b0 + r0; row < b0 + r1; ++row) {
        // routed picks: item k = pick k of this row (pairs mode: the k-th LOCAL pick, so no row of an absent expert is read)
        rows_list<MK_FP4, RP>(pairs ? s_nloc : p.n_used, ff, terms, gf,
            [&](int k, const uint8_t*& pa, const uint8_t*& pb, const int8_t*& q, const float*& s) {
                const int pk = pairs ? s_loc[k] : k;
                const int el = max(s_el[pk], 0);
                pa = p.down.nib + ((size_t)el * n_out + row) * (ff / 2);
                pb = p.down.sc + ((size_t)el * n_out + row) * nsb;
                q = hq + pk * ff; s = hs + pk * nbf;
            },
            [&](int k, float v) { outv[pairs ? s_loc[k] : k] = v; });
        float sh = 0.0f;
        if (pairs) {
            if (b == p.own_row) {
                rows_list<MK_Q8, 1>(1, sff, terms, gs,
                    [&](int, const uint8_t*& pa, const uint8_t*& pb, const int8_t*& q, const float*& s) {
                        pa = (const uint8_t*)p.shared_down.q + (size_t)row * sff;
                        pb = (const uint8_t*)p.shared_down.s + (size_t)row * (sff / 16);
                        q = sq; s = ss;
                    },
                    [&](int, float v) { p.shd[row] = v; });
            }
            __syncwarp();
            if (lane < p.n_used && s_el[lane] >= 0) {
                float* orow = p.o_rows[0] ? p.o_rows[b] + (size_t)lane * n_out : p.o_pairs + ((size_t)b * p.n_used + lane) * n_out;
                orow[row] = has_s ? outv[lane] * s2k : outv[lane];
            }
            __syncwarp();
            continue;
        }
        if (!p.local_only) {
            rows_list<MK_Q8, 1>(1, sff, terms, gs,
                [&](int, const uint8_t*& pa, const uint8_t*& pb, const int8_t*& q, const float*& s) {
                    pa = (const uint8_t*)p.shared_down.q + (size_t)row * sff;
                    pb = (const uint8_t*)p.shared_down.s + (size_t)row * (sff / 16);
                    q = sq; s = ss;
                },
                [&](int, float v) { outv[31] = v; });
        }
        __syncwarp();
        if (has_s && lane < p.n_used) outv[lane] = outv[lane] * s2k;
        __syncwarp();
        if (lane == 0) {
            float acc = 0.0f;                                   // experts in pick order from zero, shared last
            for (int k = 0; k < p.n_used; ++k) {
                if (s_el[k] < 0) continue;
                acc += s_wt[k] * outv[k];
            }
            if (p.local_only) p.partial[(size_t)b * n_out + row] = acc;
            else { sh = outv[31]; acc += sh * s_g; x[row] += acc; }
        }
        __syncwarp();
    }
    TL(TLK_MOE_DOWN, 3);
}
size_t moe_down_smem(int n_used, int ff, int sff, int rp) {
    int gf = lanes_shift(ff / 32), gs = lanes_shift(sff / 32);
    int tf = std::max(terms_floats(rp, gf, ff / 16), terms_floats(1, gs, sff / 32));
    return (size_t)n_used * ff + (size_t)n_used * (ff / 32) * 4 + sff + (size_t)(sff / 32) * 4 + (size_t)NWG * (tf + 32) * 4 + 64;
}

// ------------------------------------------------------------------------------------------------------
__global__ void k_embed(const float* table, int n_embd, const int32_t* tokens, float* x) {
    int b = blockIdx.x;
    pdl_trigger(); pdl_wait();
    const float* row = table + (size_t)tokens[b] * n_embd;
    if ((n_embd & 3) == 0) {
        const int nv = n_embd >> 2;
        float4* dst = (float4*)(x + (size_t)b * n_embd);
        for (int i0 = threadIdx.x; i0 < nv; i0 += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) if (i0 + j * (int)blockDim.x < nv) v[j] = __ldg((const float4*)row + i0 + j * blockDim.x);
#pragma unroll
            for (int j = 0; j < 4; ++j) if (i0 + j * (int)blockDim.x < nv) dst[i0 + j * blockDim.x] = v[j];
        }
        return;
    }
    for (int i = threadIdx.x; i < n_embd; i += blockDim.x) x[(size_t)b * n_embd + i] = row[i];
}

// Greedy argmax with strict '>' (lowest index wins, src/profile.rs:192-213) in two stages: partial
// (value, index) pairs per sequence, then one warp per sequence that also feeds the choice back as the next
// input token, advances the position and appends to the history.
constexpr int ARGMAX_PARTS = 64;
__device__ __forceinline__ void argmax_merge(float& bv, int& bi, float ov, int oi) {
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
}
__global__ void __launch_bounds__(256) k_argmax_partial(const float* logits, int n_vocab, float* pv, int* pi) {
    __shared__ float sv[8];
    __shared__ int si[8];
    int part = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    int lo, hi;
    share(n_vocab, gridDim.x, part, lo, hi);
    pdl_trigger(); pdl_wait();
    const float* l = logits + (size_t)b * n_vocab;
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i0 = lo + tid; i0 < hi; i0 += 8 * blockDim.x) {
        float v[8];   // eight strided loads in flight per trip; the scan below keeps ascending index order per thread
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = i0 + j * (int)blockDim.x < hi ? l[i0 + j * blockDim.x] : -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = i0 + j * blockDim.x;
            if (i < hi && (bi == 0x7fffffff || v[j] > bv)) { bv = v[j]; bi = i; }
        }
    }
    for (int o = 16; o > 0; o >>= 1) argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) { sv[wid] = bv; si[wid] = bi; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 8; ++w) argmax_merge(bv, bi, sv[w], si[w]);
        pv[(size_t)b * gridDim.x + part] = bv; pi[(size_t)b * gridDim.x + part] = bi;
    }
}
__global__ void k_argmax_advance(const float* pv, const int* pi, int n_part, int32_t* tokens, int* pos, int32_t* next_out,
                                 int32_t* history, int history_cap, int* step_counter, int n_seq) {
    int b = blockIdx.x, lane = threadIdx.x;
    pdl_trigger(); pdl_wait();
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = lane; i < n_part; i += 32) argmax_merge(bv, bi, pv[(size_t)b * n_part + i], pi[(size_t)b * n_part + i]);
    for (int o = 16; o > 0; o >>= 1) argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) {
        tokens[b] = bi;
        next_out[b] = bi;
        pos[b] += 1;
        int s = step_counter[b];
        if (history && s < history_cap) history[(size_t)s * n_seq + b] = bi;
        step_counter[b] = s + 1;
    }
}

}  // namespace
