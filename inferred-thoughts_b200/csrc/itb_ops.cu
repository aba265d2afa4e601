// The op-level seam: one extern "C" entry per method of the reference's backend trait
// (src/ops/mod.rs:489-1426), operating on host-address-keyed device mirrors.
#include "itb_kernels.cuh"
#include "itb_attn_exact.cuh"
#include "itb_gdn_chunk.cuh"
#include "itb_attn_mma.cuh"
#include "itb_rows.cuh"

static inline unsigned blocks_for(size_t n, int per = 256) { return (unsigned)((n + per - 1) / per); }

#define EW_LAUNCH(c, kernel, n, ...)                                      \
    do {                                                                  \
        if ((n) > 0) {                                                    \
            kernel<<<blocks_for(n), 256, 0, (c)->stream>>>(__VA_ARGS__);  \
            ITB_LAUNCHED(c);                                              \
        }                                                                 \
    } while (0)

extern "C" void itb_silu_mul(itb_ctx* c, float* gate, const float* up, size_t n) {
    float* g = itb_mirror_inout(c, gate, n); const float* u = itb_mirror_in(c, up, n);
    if (!g || !u) return;
    EW_LAUNCH(c, k_silu_mul, n, g, u, n);
}
extern "C" void itb_sigmoid_mul(itb_ctx* c, float* x, const float* gate, size_t n) {
    float* xd = itb_mirror_inout(c, x, n); const float* g = itb_mirror_in(c, gate, n);
    if (!xd || !g) return;
    EW_LAUNCH(c, k_sigmoid_mul, n, xd, g, n);
}
extern "C" void itb_scale(itb_ctx* c, float* buf, size_t n, float s) {
    float* b = itb_mirror_inout(c, buf, n);
    if (!b) return;
    EW_LAUNCH(c, k_scale, n, b, n, s);
}
extern "C" void itb_add_assign(itb_ctx* c, float* a, const float* b, size_t n) {
    float* ad = itb_mirror_inout(c, a, n); const float* bd = itb_mirror_in(c, b, n);
    if (!ad || !bd) return;
    EW_LAUNCH(c, k_add_assign, n, ad, bd, n);
}
extern "C" void itb_add_scaled(itb_ctx* c, float* a, const float* b, size_t n, float s) {
    float* ad = itb_mirror_inout(c, a, n); const float* bd = itb_mirror_in(c, b, n);
    if (!ad || !bd) return;
    EW_LAUNCH(c, k_add_scaled, n, ad, bd, n, s, (const float*)nullptr);
}
extern "C" void itb_add_scaled_sigmoid(itb_ctx* c, float* acc, const float* b, size_t n, const float* logit) {
    float* ad = itb_mirror_inout(c, acc, n); const float* bd = itb_mirror_in(c, b, n); const float* lg = itb_mirror_in(c, logit, 1);
    if (!ad || !bd || !lg) return;
    EW_LAUNCH(c, k_add_scaled, n, ad, bd, n, 0.0f, lg);
}
extern "C" void itb_add_scaled_rows(itb_ctx* c, float* acc, size_t n, const float* rows, const float* scales, size_t n_rows) {
    const float* r = itb_mirror_in(c, rows, n * n_rows); const float* s = itb_mirror_in(c, scales, n_rows);
    float* a = itb_mirror_out(c, acc, n);
    if (!a || !r || !s) return;
    EW_LAUNCH(c, k_add_scaled_rows, n, a, n, r, s, n_rows);
}
extern "C" void itb_gather_chunks(itb_ctx* c, const float* src, size_t src_len, size_t chunk, size_t stride, size_t offset,
                                  float* out, size_t out_len) {
    if (chunk == 0 || out_len % chunk) { itb_fail_msg(c, "gather_chunks: out is not whole chunks"); return; }
    size_t n_chunks = out_len / chunk;
    if (n_chunks && (n_chunks - 1) * stride + offset + chunk > src_len) { itb_fail_msg(c, "gather_chunks: reads past src"); return; }
    const float* s = itb_mirror_in(c, src, src_len); float* o = itb_mirror_out(c, out, out_len);
    if (!s || !o) return;
    EW_LAUNCH(c, k_gather_chunks, out_len, s, chunk, stride, offset, o, out_len);
}
extern "C" void itb_scatter_chunks(itb_ctx* c, const float* src, size_t src_len, size_t chunk, size_t stride, size_t offset,
                                   float* dst, size_t dst_len) {
    if (chunk == 0 || src_len % chunk) { itb_fail_msg(c, "scatter_chunks: src is not whole chunks"); return; }
    size_t n_chunks = src_len / chunk;
    if (n_chunks && (n_chunks - 1) * stride + offset + chunk > dst_len) { itb_fail_msg(c, "scatter_chunks: writes past dst"); return; }
    const float* s = itb_mirror_in(c, src, src_len); float* d = itb_mirror_inout(c, dst, dst_len);
    if (!s || !d) return;
    EW_LAUNCH(c, k_scatter_chunks, src_len, s, src_len, chunk, stride, offset, d);
}

extern "C" void itb_rms_norm(itb_ctx* c, const float* x, size_t x_len, const float* w, size_t nd, float eps, float* out) {
    if (nd == 0 || x_len % nd) { itb_fail_msg(c, "rms_norm: x is not whole rows"); return; }
    const float* xd = itb_mirror_in(c, x, x_len); const float* wd = itb_mirror_in(c, w, nd);
    float* od = itb_mirror_out(c, out, x_len);
    if (!xd || !wd || !od) return;
    k_rms_norm<<<(unsigned)(x_len / nd), 256, 32 * 8 + nd * 4, c->stream>>>(xd, wd, (int)nd, eps, od);
    ITB_LAUNCHED(c);
}
extern "C" void itb_rms_norm_heads(itb_ctx* c, float* x, size_t len, const float* w, size_t head_dim, float eps) {
    if (head_dim == 0 || len % head_dim) { itb_fail_msg(c, "rms_norm_heads: x is not whole heads"); return; }
    float* xd = itb_mirror_inout(c, x, len); const float* wd = itb_mirror_in(c, w, head_dim);
    if (!xd || !wd) return;
    k_rms_norm<<<(unsigned)(len / head_dim), 64, 32 * 8 + head_dim * 4, c->stream>>>(xd, wd, (int)head_dim, eps, xd);
    ITB_LAUNCHED(c);
}
extern "C" void itb_l2_norm_heads(itb_ctx* c, float* x, size_t len, size_t head_dim, float eps) {
    if (head_dim == 0 || len % head_dim) { itb_fail_msg(c, "l2_norm_heads: x is not whole heads"); return; }
    float* xd = itb_mirror_inout(c, x, len);
    if (!xd) return;
    size_t nh = len / head_dim;
    k_l2_norm_heads<<<blocks_for(nh, 8), 256, 0, c->stream>>>(xd, nh, (int)head_dim, eps);
    ITB_LAUNCHED(c);
}
extern "C" void itb_softmax(itb_ctx* c, float* x, size_t len, size_t row) {
    if (row == 0) return;
    if (len % row) { itb_fail_msg(c, "softmax: x is not whole rows"); return; }
    float* xd = itb_mirror_inout(c, x, len);
    if (!xd) return;
    k_softmax_rows<<<blocks_for(len / row, 8), 256, 0, c->stream>>>(xd, len / row, (int)row);
    ITB_LAUNCHED(c);
}
extern "C" void itb_rope_neox(itb_ctx* c, float* x, size_t len, size_t pos, size_t head_dim, size_t n_rot, size_t n_heads, float theta) {
    size_t per_row = head_dim * n_heads;
    if (per_row == 0 || len % per_row || n_rot % 2 || n_rot > head_dim) { itb_fail_msg(c, "rope_neox: bad shape"); return; }
    float* xd = itb_mirror_inout(c, x, len);
    if (!xd) return;
    size_t n_rows = len / per_row, total = n_rows * n_heads * (n_rot / 2);
    EW_LAUNCH(c, k_rope, total, xd, n_rows, (int)n_heads, (int)head_dim, (int)n_rot, theta, pos, (const int*)nullptr);
}
extern "C" void itb_kv_write(itb_ctx* c, uint16_t* slab, size_t slab_len, size_t offset, const float* src, size_t n) {
    if (offset + n > slab_len) { itb_fail_msg(c, "kv_write: past the slab"); return; }
    uint16_t* sd = itb_kv_slab(c, slab, slab_len); const float* s = itb_mirror_in(c, src, n);
    if (!sd || !s) return;
    EW_LAUNCH(c, k_kv_write, n, sd, offset, s, n, (int)c->kv_bf16);
}
extern "C" void itb_ssm_conv(itb_ctx* c, float* state, size_t state_len, const float* x, size_t x_len, const float* w,
                             size_t w_len, size_t kernel, float* out) {
    if (kernel < 2 || kernel > 9 || w_len % kernel) { itb_fail_msg(c, "ssm_conv: bad kernel width"); return; }
    size_t nc = w_len / kernel;
    if (state_len != nc * (kernel - 1) || x_len % nc) { itb_fail_msg(c, "ssm_conv: bad shape"); return; }
    float* sd = itb_state_slab(c, state, state_len);
    const float* xd = itb_mirror_in(c, x, x_len); const float* wd = itb_mirror_in(c, w, w_len);
    float* od = itb_mirror_out(c, out, x_len);
    if (!sd || !xd || !wd || !od) return;
    k_ssm_conv<<<blocks_for(nc, 128), 128, 0, c->stream>>>(sd, xd, x_len / nc, (int)nc, wd, (int)kernel, od);
    ITB_LAUNCHED(c);
}
// What the chunk kernels take per token besides k and v: q scaled by 1/sqrt(sk), the decay g and the write strength beta
// (src/ops/naive.rs:101-107). One thread per q element; the first n_tok * n_v threads also do a (token, head)'s g and beta.
__global__ void k_gdn_op_pre(const float* q, const float* alpha, const float* beta, const float* ssm_a, const float* dt_bias, size_t n_tok, int kper, int n_v,
                             float q_scale, float* qs, float* gb) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_tok * kper) qs[i] = q[i] * q_scale;
    if (i < n_tok * n_v) {
        const int h = (int)(i % n_v);
        const float a = alpha[i] + dt_bias[h];
        const float sp = a > 20.0f ? a : log_f(1.0f + exp_f(a));
        gb[i * 2] = exp_f(sp * ssm_a[h]);
        gb[i * 2 + 1] = sigmoid_f(beta[i]);
    }
}
extern "C" void itb_delta_rule(itb_ctx* c, const itb_delta* d, float* state, size_t state_len, float* out, size_t out_len) {
    size_t kper = d->n_k_heads * d->head_k_dim, vper = d->n_v_heads * d->head_v_dim, nt = d->n_tokens;
    if (state_len != d->n_v_heads * d->head_k_dim * d->head_v_dim || out_len != nt * vper || d->n_k_heads == 0) {
        itb_fail_msg(c, "delta_rule: bad shape"); return;
    }
    float* sd = itb_state_slab(c, state, state_len);
    const float* q = itb_mirror_in(c, d->q, nt * kper); const float* k = itb_mirror_in(c, d->k, nt * kper);
    const float* v = itb_mirror_in(c, d->v, nt * vper);
    const float* al = itb_mirror_in(c, d->alpha, nt * d->n_v_heads); const float* be = itb_mirror_in(c, d->beta, nt * d->n_v_heads);
    const float* sa = itb_mirror_in(c, d->ssm_a, d->n_v_heads); const float* dt = itb_mirror_in(c, d->dt_bias, d->n_v_heads);
    float* od = itb_mirror_out(c, out, out_len);
    if (!sd || !q || !k || !v || !al || !be || !sa || !dt || !od) return;
    constexpr int ROWS = 32;
    int sk = (int)d->head_k_dim, sv = (int)d->head_v_dim;
    if (c->gdn_chunk && nt >= 32 && sk == 128 && sv == 128) {
        // gdn=chunk: the chunk-parallel form (tolerance class). Scaled q, decay and write strength per token first, then the two kernels.
        const int n_k = (int)d->n_k_heads, n_v = (int)d->n_v_heads, n_ch = (int)((nt + GC - 1) / GC);
        const size_t need = nt * kper + nt * n_v * 2 + (size_t)n_ch * n_v * gdn_chunk_floats<128>();
        if (c->tmp_cap < need) {
            cudaStreamSynchronize(c->stream);
            cudaFree(c->tmp_f32); c->tmp_f32 = nullptr; c->tmp_cap = 0;
            if (cudaMalloc(&c->tmp_f32, need * 4) != cudaSuccess) { cudaGetLastError(); itb_fail_msg(c, "delta_rule: out of device memory for the chunk scratch"); return; }
            c->tmp_cap = need;
        }
        float* qs = c->tmp_f32; float* gbd = qs + nt * kper; float* scr = gbd + nt * n_v * 2;
        k_gdn_op_pre<<<(unsigned)((nt * kper + 255) / 256), 256, 0, c->stream>>>(q, al, be, sa, dt, nt, n_k * sk, n_v, 1.0f / sqrtf((float)sk), qs, gbd);
        static bool attr = false;
        if (!attr) {
            cudaFuncSetAttribute(k_gdn_chunk_prep<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gdn_chunk_prep_smem<128>());
            cudaFuncSetAttribute(k_gdn_chunk_scan<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gdn_chunk_scan_smem<128>());
            attr = true;
        }
        k_gdn_chunk_prep<128><<<dim3(n_ch, n_v, 1), 256, gdn_chunk_prep_smem<128>(), c->stream>>>(qs, k, v, gbd, (int)nt, n_k, n_v, scr);
        k_gdn_chunk_scan<128><<<dim3(n_v, sk / GC_VS, 1), 256, gdn_chunk_scan_smem<128>(), c->stream>>>(scr, (int)nt, n_v, sd, (size_t)n_v * sk * sk, od);
        ITB_LAUNCHED(c);
        return;
    }
    dim3 grid((unsigned)d->n_v_heads, (unsigned)((sv + ROWS - 1) / ROWS));
    size_t smem = (size_t)(ROWS * (sk + 1) + 2 * sk) * 4;
    k_delta_rule<ROWS><<<grid, 128, smem, c->stream>>>(q, k, v, al, be, sa, dt, nt, sk, sv, (int)d->n_k_heads, (int)d->n_v_heads, sd, od);
    ITB_LAUNCHED(c);
}

// ------------------------------------------------------------------ matmuls
static bool quantize_rows(itb_ctx* c, const float* xd, size_t n_rows, size_t n_in) {
    if (!itb_ensure_xq(c, n_rows * n_in)) return false;
    k_quant_q8<<<(unsigned)n_rows, 256, 0, c->stream>>>(xd, (int)n_in, c->xq, c->xs);
    ITB_LAUNCHED(c);
    return true;
}

static void launch_q8(itb_ctx* c, const WeightEntry* w, size_t n_tok, float* od) {
    DevQ8 dw{(const int8_t*)w->a, (const uint16_t*)w->b, (int)w->n_in, (int)w->n_out};
    if (c->f16tc && n_tok >= 64 && itb_tc_f16_shape_ok(dw) && itb_tc_f16_gemm(c, c->stream, dw, c->xq, c->xs, (int)n_tok, od, w->n_out, 0, false)) {
        ITB_LAUNCHED(c);      // opts dense=f16tc: many rows as one f16 tensor-core GEMM (tolerance class)
        return;
    }
    if (n_tok >= 2 && w->n_in % 32 == 0 && gemm_smem((int)w->n_in) <= 200 * 1024) {
        // several tokens: every weight row is read once per 32 tokens, on the int8 tensor-core path
        size_t sm = gemm_smem((int)w->n_in);
        cudaFuncSetAttribute(k_gemm_q8<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        dim3 g((unsigned)((w->n_out + MMA_ROWS - 1) / MMA_ROWS), (unsigned)((n_tok + MMA_TOK - 1) / MMA_TOK));
        k_gemm_q8<4><<<g, 256, sm, c->stream>>>(dw, c->xq, c->xs, (int)n_tok, od, w->n_out, 0);
        ITB_LAUNCHED(c);
        return;
    }
    int nb = (int)w->n_in / 32, gsh = lanes_shift(nb), nw = 8;
    int gx = (int)std::min<size_t>((w->n_out + 31) / 32, (size_t)c->sm_count * 2);
    if (gx < 1) gx = 1;
    size_t smem = w->n_in + nb * 4 + (size_t)nw * terms_floats(4, gsh, nb) * 4;
    dim3 grid(gx, (unsigned)n_tok);
    cudaFuncSetAttribute(k_matmul_q8, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k_matmul_q8<<<grid, nw * 32, smem, c->stream>>>(dw, c->xq, c->xs, od);
    ITB_LAUNCHED(c);
}

// The pairs of a pass sorted by expert: pair_off[e .. e+1) bounds expert e's slots of pair_list.
static bool group_pairs(itb_ctx* c, const int32_t* ids, size_t n_pairs, size_t E) {
    if (c->pair_cap < n_pairs || c->pair_experts < E) {
        cudaStreamSynchronize(c->stream);
        cudaFree(c->pair_off); cudaFree(c->pair_list); c->pair_off = nullptr; c->pair_list = nullptr; c->pair_cap = 0; c->pair_experts = 0;
        if (cudaMalloc(&c->pair_off, (E + 1) * 4) != cudaSuccess || cudaMalloc(&c->pair_list, n_pairs * 4) != cudaSuccess) return itb_fail_msg(c, "experts: out of device memory");
        c->pair_cap = n_pairs; c->pair_experts = E;
    }
    k_group_pairs_fast<<<1, 1024, E * 4, c->stream>>>(ids, (int)n_pairs, (int)E, c->pair_off, c->pair_list);
    ITB_LAUNCHED(c);
    return true;
}
// experts=fp4tc: FP4 activations times FP4 weights on the tensor cores (the reference's default device arithmetic,
// src/ops/cuda/mod.rs:239-248 there; CPU statement with fp4 activations: src/ops/naive.rs:755-837). True when the pass ran there.
static bool experts_tc(itb_ctx* c, const itb_experts* g, const itb_experts* u, const itb_route_t* r, const float* xd, size_t x_len, float* od) {
    if (!c->fp4tc || g->ggml_type != ITB_NVFP4 || (u && u->ggml_type != ITB_NVFP4) || g->n_expert > 1024) return false;
    const WeightEntry* wg = itb_weight(c, g->data, g->bytes, g->ggml_type, g->n_in, g->n_out, g->n_expert, g->scale, g->scale_bytes);
    const WeightEntry* wu = u ? itb_weight(c, u->data, u->bytes, u->ggml_type, u->n_in, u->n_out, u->n_expert, u->scale, u->scale_bytes) : nullptr;
    if (!wg || (u && !wu)) return false;
    DevFp4 dg{(const uint8_t*)wg->a, (const uint8_t*)wg->b, wg->scale2, (int)wg->n_in, (int)wg->n_out, (int)wg->n_expert, 0};
    DevFp4 du = dg;
    if (wu) du = DevFp4{(const uint8_t*)wu->a, (const uint8_t*)wu->b, wu->scale2, (int)wu->n_in, (int)wu->n_out, (int)wu->n_expert, 0};
    if (!itb_tc_shape_ok(dg) || (wu && !itb_tc_shape_ok(du))) return false;
    const size_t n_pairs = r->n_tok * r->n_used, rows = x_len / g->n_in;
    const int div = rows == n_pairs ? 1 : rows > 1 ? (int)r->n_used : 0x7fffffff;
    if (!group_pairs(c, c->route_ids, n_pairs, g->n_expert)) return true;      // failed loudly: nothing else runs
    itb_tc_experts(c, c->stream, dg, wu ? &du : nullptr, xd, div, c->pair_off, c->pair_list, (int)n_pairs, od);
    return true;
}
// ids==nullptr: dense NVFP4 matrix, one "pair" per token reading its own row.
static void launch_fp4(itb_ctx* c, const WeightEntry* w, const int32_t* ids, size_t n_pairs, int n_used, int rows_mode, float* od) {
    if (!ids && n_pairs >= 2 && gemm_smem((int)w->n_in) <= 200 * 1024) {
        size_t sm = gemm_smem((int)w->n_in);
        cudaFuncSetAttribute(k_gemm_fp4, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        dim3 g((unsigned)((w->n_out + MMA_ROWS - 1) / MMA_ROWS), (unsigned)((n_pairs + MMA_TOK - 1) / MMA_TOK));
        k_gemm_fp4<<<g, 256, sm, c->stream>>>((const uint8_t*)w->a, (const uint8_t*)w->b, (int)w->n_in, (int)w->n_out, c->xq, c->xs,
                                             (int)n_pairs, od, w->n_out, 1.0f, 0);
        ITB_LAUNCHED(c);
        return;
    }
    DevFp4 dw{(const uint8_t*)w->a, (const uint8_t*)w->b, w->scale2, (int)w->n_in, (int)w->n_out, (int)w->n_expert, 0};
    if (ids && n_pairs >= 16 && w->n_in % 256 == 0 && w->n_expert <= 1024) {
        // many pairs: group them by expert and run each expert's rows through the int8-MMA tiles, so an expert's weights
        // are read once (the reference groups the same way, kernels/moe.cuh:62-133 there)
        const size_t E = w->n_expert;
        if (!group_pairs(c, ids, n_pairs, E)) return;
        const int per_e = (int)((n_pairs + E - 1) / E), nj = per_e <= 8 ? 1 : per_e <= 16 ? 2 : per_e <= 32 ? 4 : 0;
        const int ns = std::min((int)w->n_in / 256, TILE_STAGES);
        const int div = rows_mode == 0 ? 1 : rows_mode == 1 ? n_used : 0x7fffffff;
#define EXP_TILE(NJ, TH)                                                                                                          \
    do {                                                                                                                         \
        cudaFuncSetAttribute(k_tile_down<NJ, 256, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);                 \
        k_tile_down<NJ, 256, TH><<<dim3((unsigned)E, (unsigned)((w->n_out + 128 / TH - 1) / (128 / TH))), 256,                    \
                                   tile_smem<MK_FP4, NJ, 256, TH>((int)w->n_in), c->stream>>>(dw, c->xq, c->xs, c->pair_off, c->pair_list, od, ns, div); \
    } while (0)
        if (nj == 1) EXP_TILE(1, 1); else if (nj == 2) EXP_TILE(2, 1); else if (nj == 4) EXP_TILE(4, 1); else EXP_TILE(4, 2);
#undef EXP_TILE
        ITB_LAUNCHED(c);
        return;
    }
    int nb = (int)w->n_in / 32, nsb = (int)w->n_in / 16, gsh = lanes_shift(nb), nw = 8;
    int gx = (int)std::min<size_t>((w->n_out + 31) / 32, (size_t)c->sm_count * 2);
    if (gx < 1) gx = 1;
    size_t smem = w->n_in + nb * 4 + (size_t)nw * terms_floats(4, gsh, nsb) * 4;
    dim3 grid(gx, (unsigned)n_pairs);
    cudaFuncSetAttribute(k_matmul_fp4, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k_matmul_fp4<<<grid, nw * 32, smem, c->stream>>>(dw, ids, n_used, rows_mode, c->xq, c->xs, od);
    ITB_LAUNCHED(c);
}

static void launch_f32(itb_ctx* c, const WeightEntry* w, const float* xd, size_t n_tok, float* od) {
    DevF32 dw{(const float*)w->a, (int)w->n_in, (int)w->n_out};
    int nw = 4;
    int gx = (int)std::min<size_t>((w->n_out + 31) / 32, (size_t)c->sm_count * 2);
    if (gx < 1) gx = 1;
    size_t smem = w->n_in * 4 + (size_t)nw * 32 * 33 * 4;
    dim3 grid(gx, (unsigned)n_tok);
    if (c->exact) {
        cudaFuncSetAttribute(k_matmul_f32<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k_matmul_f32<true><<<grid, nw * 32, smem, c->stream>>>(dw, xd, od);
    } else {
        cudaFuncSetAttribute(k_matmul_f32<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k_matmul_f32<false><<<grid, nw * 32, smem, c->stream>>>(dw, xd, od);
    }
    ITB_LAUNCHED(c);
}

static void matmul_dev(itb_ctx* c, const itb_weights* w, const float* xd, size_t n_tok, float* od) {
    const WeightEntry* we = itb_weight(c, w->data, w->bytes, w->ggml_type, w->n_in, w->n_out, 1, nullptr, 0);
    if (!we) return;
    if (we->ty == ITB_Q8_0) { if (quantize_rows(c, xd, n_tok, w->n_in)) launch_q8(c, we, n_tok, od); }
    else if (we->ty == ITB_NVFP4) { if (quantize_rows(c, xd, n_tok, w->n_in)) launch_fp4(c, we, nullptr, n_tok, 1, 0, od); }
    else launch_f32(c, we, xd, n_tok, od);
}

extern "C" void itb_matmul(itb_ctx* c, const itb_weights* w, const float* x, size_t x_len, float* out, size_t out_len) {
    if (w->n_in == 0 || x_len % w->n_in || out_len != x_len / w->n_in * w->n_out) { itb_fail_msg(c, "matmul: bad shape"); return; }
    const float* xd = itb_mirror_in(c, x, x_len); float* od = itb_mirror_out(c, out, out_len);
    if (!xd || !od) return;
    matmul_dev(c, w, xd, x_len / w->n_in, od);
}
extern "C" void itb_matmul_pair(itb_ctx* c, const itb_weights* a, const itb_weights* b, const float* x, size_t x_len,
                                float* out_a, size_t out_a_len, float* out_b, size_t out_b_len) {
    if (a->n_in != b->n_in || a->n_in == 0 || x_len % a->n_in) { itb_fail_msg(c, "matmul_pair: bad shape"); return; }
    size_t nt = x_len / a->n_in;
    if (out_a_len != nt * a->n_out || out_b_len != nt * b->n_out) { itb_fail_msg(c, "matmul_pair: bad output length"); return; }
    const float* xd = itb_mirror_in(c, x, x_len);
    float* oa = itb_mirror_out(c, out_a, out_a_len); float* ob = itb_mirror_out(c, out_b, out_b_len);
    if (!xd || !oa || !ob) return;
    matmul_dev(c, a, xd, nt, oa);
    matmul_dev(c, b, xd, nt, ob);
}

// ------------------------------------------------------------------ routing and experts
extern "C" void itb_route(itb_ctx* c, float* probs, size_t len, size_t n_expert, size_t n_used, itb_route_t* out) {
    if (n_expert == 0 || len % n_expert || n_used == 0 || n_used > 16 || n_used > n_expert || n_expert > 4096) {
        itb_fail_msg(c, "route: bad shape"); return;
    }
    size_t nt = len / n_expert;
    const float* p = itb_mirror_in(c, probs, len);
    if (!p || !itb_ensure_route(c, nt * n_used)) return;
    k_route<<<(unsigned)nt, 256, 0, c->stream>>>(p, (int)n_expert, (int)n_used, c->route_ids, c->route_w);
    ITB_LAUNCHED(c);
    c->route_n_tok = nt; c->route_n_used = n_used;
    out->on_device = 1; out->n_used = n_used; out->n_tok = nt; out->ids = nullptr; out->weights = nullptr;
}
extern "C" void itb_read_route(itb_ctx* c, int32_t* ids, float* weights, size_t n) {
    if (n > c->route_n_tok * c->route_n_used) { itb_fail_msg(c, "read_route: more than the current route holds"); return; }
    ITB_CUDA(c, cudaMemcpyAsync(ids, c->route_ids, n * 4, cudaMemcpyDeviceToHost, c->stream));
    ITB_CUDA(c, cudaMemcpyAsync(weights, c->route_w, n * 4, cudaMemcpyDeviceToHost, c->stream));
    ITB_CUDA(c, cudaStreamSynchronize(c->stream));
}
// A host-chosen route is honoured by staging it into the device route (src/ops/cuda/ops/moe.rs:878-921).
// The kernels index shared memory and the expert stack with these ids, so a host-built route is checked here, before any
// copy or launch: n_used within [1, min(16, n_expert)], every id within [0, n_expert).
static bool stage_route(itb_ctx* c, const itb_route_t* r, size_t n_expert) {
    if (r->n_used == 0 || r->n_used > 16 || r->n_used > n_expert) return itb_fail_msg(c, "route: n_used out of range");
    if (r->on_device) return c->route_n_tok == r->n_tok && c->route_n_used == r->n_used ? true : itb_fail_msg(c, "route: device route does not match");
    size_t n = r->n_tok * r->n_used;
    if (!r->ids) return itb_fail_msg(c, "route: host route without ids");
    for (size_t i = 0; i < n; ++i)
        if (r->ids[i] >= n_expert) return itb_fail_msg(c, "route: expert id out of range");
    if (!itb_ensure_route(c, n)) return false;
    std::vector<int32_t> ids(n);
    for (size_t i = 0; i < n; ++i) ids[i] = (int32_t)r->ids[i];
    cudaMemcpyAsync(c->route_ids, ids.data(), n * 4, cudaMemcpyHostToDevice, c->stream);
    if (r->weights) cudaMemcpyAsync(c->route_w, r->weights, n * 4, cudaMemcpyHostToDevice, c->stream);
    cudaStreamSynchronize(c->stream);
    c->route_n_tok = r->n_tok; c->route_n_used = r->n_used;
    return true;
}
static void experts_dev(itb_ctx* c, const itb_experts* w, const itb_route_t* r, const float* xd, size_t x_len, float* od) {
    if (w->ggml_type != ITB_NVFP4) { itb_fail_msg(c, "routed experts: only NVFP4 has a kernel here"); return; }  // src/ops/mod.rs:29-55
    const WeightEntry* we = itb_weight(c, w->data, w->bytes, w->ggml_type, w->n_in, w->n_out, w->n_expert, w->scale, w->scale_bytes);
    if (!we) return;
    size_t n_pairs = r->n_tok * r->n_used, rows = x_len / w->n_in;
    int mode = rows == n_pairs ? 0 : rows > 1 ? 1 : 2;
    if (!quantize_rows(c, xd, rows, w->n_in)) return;
    launch_fp4(c, we, c->route_ids, n_pairs, (int)r->n_used, mode, od);
}
extern "C" void itb_matmul_experts(itb_ctx* c, const itb_experts* w, const itb_route_t* r, const float* x, size_t x_len,
                                   float* out, size_t out_len) {
    if (w->n_in == 0 || x_len % w->n_in || out_len != r->n_tok * r->n_used * w->n_out) { itb_fail_msg(c, "matmul_experts: bad shape"); return; }
    if (!stage_route(c, r, w->n_expert)) return;
    const float* xd = itb_mirror_in(c, x, x_len); float* od = itb_mirror_out(c, out, out_len);
    if (!xd || !od) return;
    if (experts_tc(c, w, nullptr, r, xd, x_len, od)) return;
    experts_dev(c, w, r, xd, x_len, od);
}
extern "C" void itb_moe_glu(itb_ctx* c, const itb_experts* gate, const itb_experts* up, const itb_route_t* r, const float* x,
                            size_t x_len, float* out, size_t out_len, float* scratch) {
    if (gate->n_in != up->n_in || gate->n_out != up->n_out || out_len != r->n_tok * r->n_used * gate->n_out) {
        itb_fail_msg(c, "moe_glu: bad shape"); return;
    }
    if (gate->n_expert != up->n_expert) { itb_fail_msg(c, "moe_glu: gate and up stacks differ in expert count"); return; }
    if (!stage_route(c, r, gate->n_expert)) return;
    const float* xd = itb_mirror_in(c, x, x_len);
    float* od = itb_mirror_out(c, out, out_len); float* sd = itb_mirror_out(c, scratch, out_len);
    if (!xd || !od || !sd) return;
    if (experts_tc(c, gate, up, r, xd, x_len, od)) return;
    experts_dev(c, gate, r, xd, x_len, od);
    experts_dev(c, up, r, xd, x_len, sd);
    EW_LAUNCH(c, k_silu_mul, out_len, od, sd, out_len);
}
extern "C" void itb_moe_finish(itb_ctx* c, float* out, size_t out_len, size_t at, size_t n, const float* rows, size_t rows_len,
                               const itb_route_t* r, const float* shared, const float* logit, size_t logit_at) {
    size_t nt = r->n_tok;
    if (rows_len != nt * r->n_used * n || at + nt * n > out_len) { itb_fail_msg(c, "moe_finish: bad shape"); return; }
    if (!stage_route(c, r, r->on_device ? 16 : 4096)) return;   // the combine reads the weights only; ids just have to be sane
    float* od = itb_mirror_inout(c, out, out_len);
    const float* rd = itb_mirror_in(c, rows, rows_len); const float* sh = itb_mirror_in(c, shared, nt * n);
    const float* lg = itb_mirror_in(c, logit, logit_at + nt);
    if (!od || !rd || !sh || !lg) return;
    EW_LAUNCH(c, k_moe_finish, nt * n, od, at, (int)n, rd, c->route_w, (int)r->n_used, nt, sh, lg, logit_at);
}

// ------------------------------------------------------------------ attention
void itb_attend_dev(itb_ctx* c, cudaStream_t st, const float* q, const uint16_t* k, const uint16_t* v, int kv_dim, int n_pos, int n_q,
                    int hd, int n_head, int n_head_kv, float scale, int bf16, const int* n_pos_dev, const float* gate,
                    float* part_acc, float* part_ml, int n_split, float* out) {
    int group = n_head / n_head_kv, nw = 8;
    dim3 grid(n_head_kv, n_q, n_split);
    size_t smem = (size_t)nw * 8 * 2 * 4 + (size_t)nw * 8 * hd * 4;
#define ATT_CASE(H)                                                                                                   \
    case H:                                                                                                           \
        cudaFuncSetAttribute(k_attn_partial<H, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
        k_attn_partial<H, 8><<<grid, nw * 32, smem, st>>>(q, k, v, kv_dim, n_pos, n_q, n_head, n_head_kv, scale, bf16, \
                                                          n_pos_dev, part_acc, part_ml);                              \
        break;
    if (group > 8) { itb_fail_msg(c, "attend: more than 8 query heads per kv head"); return; }
    switch (hd) { ATT_CASE(64) ATT_CASE(128) ATT_CASE(256) default: itb_fail_msg(c, "attend: head_dim must be 64, 128 or 256"); return; }
#undef ATT_CASE
    ITB_LAUNCHED(c);
    k_attn_combine<<<(unsigned)(n_q * n_head), hd, 0, st>>>(part_acc, part_ml, n_split, hd, gate, out);
    ITB_LAUNCHED(c);
}

// Row i of an n_q-row call sees first + i positions; the many-token kernel's one split divided out.
__global__ void k_attn_mma_npos(int* npos, int n_q, int first) { const int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n_q) npos[i] = first + i; }
__global__ void k_attn_mma_finish(const float* acc, const float* ml, int hd, float* out) {
    const size_t th = blockIdx.x;
    out[th * hd + threadIdx.x] = acc[th * hd + threadIdx.x] / ml[th * 2 + 1];
}
extern "C" void itb_attend(itb_ctx* c, const itb_attn* a, float* out, size_t out_len) {
    size_t per = a->n_head * a->head_dim;
    if (per == 0 || a->q_len % per || a->n_head_kv == 0 || a->n_head % a->n_head_kv) { itb_fail_msg(c, "attend: bad shape"); return; }
    size_t n_q = a->q_len / per;
    if (out_len != a->q_len || a->n_pos < n_q || a->n_pos * a->kv_dim > a->slab_len) { itb_fail_msg(c, "attend: bad lengths"); return; }
    const float* qd = itb_mirror_in(c, a->q, a->q_len);
    uint16_t* kd = itb_kv_slab(c, a->k, a->slab_len); uint16_t* vd = itb_kv_slab(c, a->v, a->slab_len);
    float* od = itb_mirror_out(c, out, out_len);
    if (!qd || !kd || !vd || !od) return;
    if (c->attn_mma && n_q >= 16 && AM_ROWS % (a->n_head / a->n_head_kv) == 0 && a->kv_dim % 8 == 0 &&
        (a->head_dim == 64 || a->head_dim == 128 || a->head_dim == 256)) {
        // attn=mma: the many-token kernel (tolerance class): per-row visible positions, one "split", then the division
        const int group = (int)(a->n_head / a->n_head_kv), hd = (int)a->head_dim;
        const size_t rows = n_q * a->n_head, need_f = rows * hd + rows * 2 + n_q;
        if (c->tmp_cap < need_f) {
            cudaStreamSynchronize(c->stream);
            cudaFree(c->tmp_f32); c->tmp_f32 = nullptr; c->tmp_cap = 0;
            if (cudaMalloc(&c->tmp_f32, need_f * 4) != cudaSuccess) { cudaGetLastError(); itb_fail_msg(c, "cudaMalloc(attention partials)"); return; }
            c->tmp_cap = need_f;
        }
        float* pa = c->tmp_f32; float* pm = pa + rows * hd; int* npos = (int*)(pm + rows * 2);
        k_attn_mma_npos<<<(unsigned)((n_q + 255) / 256), 256, 0, c->stream>>>(npos, (int)n_q, (int)(a->n_pos - n_q + 1));
        AmParams ap{};
        ap.q = qd; ap.kslab = kd; ap.vslab = vd; ap.slab_stride = 0; ap.npos = npos; ap.n_tok = (int)n_q; ap.kv_dim = (int)a->kv_dim;
        ap.n_head = (int)a->n_head; ap.n_head_kv = (int)a->n_head_kv; ap.group = group; ap.scale = a->scale; ap.part_acc = pa; ap.part_ml = pm;
        const dim3 ga((unsigned)((n_q + AM_ROWS / group - 1) / (AM_ROWS / group)), (unsigned)a->n_head_kv, 1);
#define AM_CASE(HD)                                                                                                                        \
    case HD:                                                                                                                                \
        cudaFuncSetAttribute(k_attn_mma<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_mma_smem<HD>());                  \
        cudaFuncSetAttribute(k_attn_mma<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_mma_smem<HD>());                 \
        if (c->kv_bf16) k_attn_mma<HD, true><<<ga, 256, attn_mma_smem<HD>(), c->stream>>>(ap);                                              \
        else k_attn_mma<HD, false><<<ga, 256, attn_mma_smem<HD>(), c->stream>>>(ap);                                                        \
        break;
        switch (hd) { AM_CASE(64) AM_CASE(128) AM_CASE(256) }
#undef AM_CASE
        k_attn_mma_finish<<<(unsigned)rows, hd, 0, c->stream>>>(pa, pm, hd, od);
        ITB_LAUNCHED(c);
        return;
    }
    if (c->exact && a->kv_dim % 8 == 0 && a->n_head / a->n_head_kv <= 8 && (a->head_dim == 64 || a->head_dim == 128 || a->head_dim == 256) &&
        attn_out_exact_smem((int)a->n_pos) <= 200 * 1024) {
        // the CPU path's own order (src/ops/naive.rs:420-466): scores, then softmax and weighted values per 32 dimensions of a head
        const size_t need_s = n_q * a->n_head * a->n_pos;
        if (c->tmp_cap < need_s) {
            cudaFree(c->tmp_f32);
            if (cudaMalloc(&c->tmp_f32, need_s * 4) != cudaSuccess) { c->tmp_f32 = nullptr; c->tmp_cap = 0; itb_fail_msg(c, "cudaMalloc(attention scores)"); return; }
            c->tmp_cap = need_s;
        }
        const int group = (int)(a->n_head / a->n_head_kv);
        AxScores sp{};
        sp.q = qd; sp.kslab = kd; sp.slab_stride = 0; sp.rows_per_seq = (int)n_q; sp.n_pos_dev = nullptr; sp.n_pos_last = (int)a->n_pos; sp.n_q = (int)n_q;
        sp.kv_dim = (int)a->kv_dim; sp.hd = (int)a->head_dim; sp.n_head = (int)a->n_head; sp.n_head_kv = (int)a->n_head_kv; sp.scale = a->scale; sp.bf16 = c->kv_bf16;
        sp.scores = c->tmp_f32; sp.s_stride = (int)a->n_pos;
        k_attn_scores_exact<<<dim3((unsigned)((a->n_pos + AX_TP - 1) / AX_TP), (unsigned)a->n_head_kv, (unsigned)n_q), AX_TP * group,
                              attn_scores_exact_smem((int)a->head_dim, group), c->stream>>>(sp);
        ITB_LAUNCHED(c);
        AxOut op{};
        op.scores = c->tmp_f32; op.s_stride = (int)a->n_pos; op.vslab = vd; op.slab_stride = 0; op.rows_per_seq = (int)n_q; op.n_pos_dev = nullptr;
        op.n_pos_last = (int)a->n_pos; op.n_q = (int)n_q; op.kv_dim = (int)a->kv_dim; op.hd = (int)a->head_dim; op.n_head = (int)a->n_head;
        op.n_head_kv = (int)a->n_head_kv; op.bf16 = c->kv_bf16; op.gate = nullptr; op.out = od; op.out_q = nullptr; op.out_s = nullptr;
        static bool attr = false;
        if (!attr) { cudaFuncSetAttribute(k_attn_out_exact, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); attr = true; }
        k_attn_out_exact<<<dim3((unsigned)(a->head_dim / 32), (unsigned)a->n_head, (unsigned)n_q), 256, attn_out_exact_smem((int)a->n_pos), c->stream>>>(op);
        ITB_LAUNCHED(c);
        return;
    }
    int n_split = (int)std::max<size_t>(1, std::min<size_t>((a->n_pos + 63) / 64, (size_t)(2 * c->sm_count) / (a->n_head_kv * n_q) + 1));
    size_t need = n_q * a->n_head * n_split * (a->head_dim + 2);
    if (c->tmp_cap < need) {
        cudaFree(c->tmp_f32);
        if (cudaMalloc(&c->tmp_f32, need * 4) != cudaSuccess) { itb_fail_msg(c, "cudaMalloc(attention partials)"); return; }
        c->tmp_cap = need;
    }
    float* pa = c->tmp_f32; float* pm = pa + n_q * a->n_head * n_split * a->head_dim;
    itb_attend_dev(c, c->stream, qd, kd, vd, (int)a->kv_dim, (int)a->n_pos, (int)n_q, (int)a->head_dim, (int)a->n_head,
                   (int)a->n_head_kv, a->scale, (int)c->kv_bf16, nullptr, nullptr, pa, pm, n_split, od);
}

// ------------------------------------------------------------------ the kernels' exp and log on their own
void itb_ops_use_logf_fix(const uint32_t* dev_tab, uint32_t n) {
    cudaMemcpyToSymbol(g_logf_fix, &dev_tab, sizeof dev_tab);
    cudaMemcpyToSymbol(g_logf_fix_n, &n, sizeof n);
}
__global__ void k_eval_unary(int kind, const float* in, size_t n, float* out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = kind == 0 ? exp_f(in[i]) : log_f(in[i]);
}
// kind 0: exp as every kernel here computes it; 1: log. Host arrays in and out (tests compare with the C library).
extern "C" int itb_eval_unary(itb_ctx* c, int kind, const float* in, size_t n, float* out) {
    float *di = nullptr, *dd = nullptr;
    if (cudaMalloc(&di, n * 4) != cudaSuccess || cudaMalloc(&dd, n * 4) != cudaSuccess) { cudaFree(di); itb_fail_msg(c, "eval_unary: out of device memory"); return 1; }
    cudaMemcpyAsync(di, in, n * 4, cudaMemcpyHostToDevice, c->stream);
    if (n) k_eval_unary<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(kind, di, n, dd);
    ITB_LAUNCHED(c);
    cudaMemcpyAsync(out, dd, n * 4, cudaMemcpyDeviceToHost, c->stream);
    cudaError_t e = cudaStreamSynchronize(c->stream);
    cudaFree(di); cudaFree(dd);
    if (e != cudaSuccess) { itb_fail(c, "eval_unary", e); return 1; }
    return 0;
}
