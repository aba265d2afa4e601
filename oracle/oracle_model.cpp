// CPU oracle, model level. TEST INFRASTRUCTURE ONLY (see oracle.h).
// Restates Qwen35::forward (src/model/qwen35.rs:956-1127), attention (:1138-1223),
// gated_delta (:1232-1328) and moe_batch (:1587-1699) over the op-level oracle.
#include "oracle.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace orc {

static const size_t MOE_CHUNK = 512;  // src/model/qwen35.rs:650

namespace {
struct Scratch {
    std::vector<float> x, normed, mixed, ffn_out, qg, q, g, k, v, attn, qkv, z, alpha, beta, conv, q_part, k_part,
        v_part, core, router, e_gate, e_up, e_out, e_in, g_all, u_all, o_all, shexp_logit, last, final_norm;
};
}  // namespace

// src/model/qwen35.rs:1138-1223
static void attention(const Config& c, const LayerWeights& L, size_t slot, size_t start_pos, size_t n, KvCache& kv,
                      Scratch& s) {
    size_t hd = c.head_dim, kd = c.kv_dim();
    matmul(L.wq, s.normed.data(), n * c.n_embd, s.qg.data());
    gather_chunks(s.qg.data(), hd, 2 * hd, 0, s.q.data(), n * hd * c.n_head);
    gather_chunks(s.qg.data(), hd, 2 * hd, hd, s.g.data(), n * hd * c.n_head);
    matmul(L.wk, s.normed.data(), n * c.n_embd, s.k.data());
    matmul(L.wv, s.normed.data(), n * c.n_embd, s.v.data());
    rms_norm_heads(s.q.data(), n * hd * c.n_head, L.q_norm, hd, c.rms_eps);
    rms_norm_heads(s.k.data(), n * kd, L.k_norm, hd, c.rms_eps);
    rope_neox(s.q.data(), n * hd * c.n_head, start_pos, hd, c.n_rot, c.n_head, c.rope_theta);
    rope_neox(s.k.data(), n * kd, start_pos, hd, c.n_rot, c.n_head_kv, c.rope_theta);
    kv_write(kv.k_layer(slot), start_pos * kd, s.k.data(), n * kd, kv.bf16);
    kv_write(kv.v_layer(slot), start_pos * kd, s.v.data(), n * kd, kv.bf16);
    Attn a{s.q.data(), n * hd * c.n_head, kv.k_layer(slot), kv.v_layer(slot), kd, start_pos + n, hd,
           c.n_head,   c.n_head_kv,       1.0f / sqrtf((float)hd), kv.bf16};
    attend(a, s.attn.data());
    sigmoid_mul(s.attn.data(), s.g.data(), n * hd * c.n_head);
    matmul(L.wo, s.attn.data(), n * hd * c.n_head, s.mixed.data());
}

// src/model/qwen35.rs:1232-1328
static void gated_delta(const Config& c, const LayerWeights& L, size_t il, size_t n, RecurrentState& rs, Scratch& s) {
    size_t kdim = c.key_dim(), vdim = c.value_dim(), cdim = c.conv_dim();
    matmul(L.wqkv, s.normed.data(), n * c.n_embd, s.qkv.data());
    matmul(L.wgate, s.normed.data(), n * c.n_embd, s.z.data());
    matmul(L.ssm_alpha, s.normed.data(), n * c.n_embd, s.alpha.data());
    matmul(L.ssm_beta, s.normed.data(), n * c.n_embd, s.beta.data());
    ssm_conv(rs.conv_of(il), s.qkv.data(), n * cdim, L.conv1d, cdim * c.ssm_d_conv, c.ssm_d_conv, s.conv.data());
    gather_chunks(s.conv.data(), kdim, cdim, 0, s.q_part.data(), n * kdim);
    gather_chunks(s.conv.data(), kdim, cdim, kdim, s.k_part.data(), n * kdim);
    gather_chunks(s.conv.data(), vdim, cdim, 2 * kdim, s.v_part.data(), n * vdim);
    l2_norm_heads(s.q_part.data(), n * kdim, c.head_k_dim(), c.rms_eps);
    l2_norm_heads(s.k_part.data(), n * kdim, c.head_k_dim(), c.rms_eps);
    Delta d{s.q_part.data(), s.k_part.data(), s.v_part.data(), s.alpha.data(), s.beta.data(), L.ssm_a, L.dt_bias,
            n, c.head_k_dim(), c.head_v_dim(), c.n_k_heads(), c.n_v_heads()};
    delta_rule(d, rs.ssm_of(il), s.core.data());
    rms_norm_heads(s.core.data(), n * vdim, L.ssm_norm, c.head_v_dim(), c.rms_eps);
    silu_mul(s.z.data(), s.core.data(), n * vdim);
    matmul(L.ssm_out, s.z.data(), n * vdim, s.mixed.data());
}

// src/model/qwen35.rs:1587-1699
static void moe_batch(const Config& c, const LayerWeights& L, size_t at, size_t n, Scratch& s, int fp4act,
                      std::vector<int32_t>* log) {
    size_t nd = c.n_embd;
    float* x = s.e_in.data();
    gather_chunks(s.normed.data(), n * nd, n * nd, at, x, n * nd);
    matmul(L.gate_inp, x, n * nd, s.router.data());
    matmul(L.shared_gate_inp, x, n * nd, s.shexp_logit.data());
    softmax(s.router.data(), n * c.n_expert, c.n_expert);
    Route r;
    route(s.router.data(), n * c.n_expert, c.n_expert, c.n_expert_used, r);
    if (log) for (size_t id : r.ids) log->push_back((int32_t)id);
    size_t pairs = n * c.n_expert_used, ff = pairs * c.expert_ff;
    moe_glu(L.gate, L.up, r, x, n * nd, s.g_all.data(), s.u_all.data(), fp4act);
    matmul_experts(L.down, r, s.g_all.data(), ff, s.o_all.data(), fp4act);
    size_t sff = n * c.shared_ff;
    matmul(L.shared_gate, x, n * nd, s.e_gate.data());
    matmul(L.shared_up, x, n * nd, s.e_up.data());
    // src/model/qwen35.rs:1668-1682: an NVFP4 file's second scale per matmul, applied to its output before anything reads it
    if (L.has_shared_s[1]) scale(s.e_up.data(), sff, L.shared_s[1]);
    if (L.has_shared_s[0]) scale(s.e_gate.data(), sff, L.shared_s[0]);
    silu_mul(s.e_gate.data(), s.e_up.data(), sff);
    matmul(L.shared_down, s.e_gate.data(), sff, s.e_out.data());
    if (L.has_shared_s[2]) scale(s.e_out.data(), n * nd, L.shared_s[2]);
    moe_finish(s.ffn_out.data(), at, nd, s.o_all.data(), r, s.e_out.data(), s.shexp_logit.data(), 0);
}

int Model::forward(const uint32_t* tokens, size_t n, size_t start_pos, KvCache& kv, RecurrentState& rs, float* logits,
                   RouteLog* log) {
    const Config& c = w.cfg;
    if (n == 0) return 2;
    if (start_pos + n > kv.n_ctx) return 1;  // src/model/qwen35.rs:984-990, before any write
    for (size_t t = 0; t < n; ++t) if (tokens[t] >= c.n_vocab) return 3;
    size_t nd = c.n_embd;
    Scratch s;
    auto z = [&](std::vector<float>& b, size_t k) { b.assign(n * k, 0.0f); };
    z(s.x, nd); z(s.normed, nd); z(s.mixed, nd); z(s.ffn_out, nd); z(s.qg, c.q_gate_dim());
    z(s.q, c.head_dim * c.n_head); z(s.g, c.head_dim * c.n_head); z(s.k, c.kv_dim()); z(s.v, c.kv_dim());
    z(s.attn, c.head_dim * c.n_head); z(s.qkv, c.conv_dim()); z(s.z, c.value_dim()); z(s.alpha, c.n_v_heads());
    z(s.beta, c.n_v_heads()); z(s.conv, c.conv_dim()); z(s.q_part, c.key_dim()); z(s.k_part, c.key_dim());
    z(s.v_part, c.value_dim()); z(s.core, c.value_dim());
    size_t nt = std::min(n, MOE_CHUNK);
    s.router.assign(nt * c.n_expert, 0.f);
    s.e_gate.assign(nt * std::max(c.expert_ff, c.shared_ff), 0.f);
    s.e_up.assign(nt * std::max(c.expert_ff, c.shared_ff), 0.f);
    s.e_out.assign(nt * nd, 0.f); s.e_in.assign(nt * nd, 0.f);
    s.g_all.assign(nt * c.n_expert_used * c.expert_ff, 0.f);
    s.u_all.assign(nt * c.n_expert_used * c.expert_ff, 0.f);
    s.o_all.assign(nt * c.n_expert_used * nd, 0.f);
    s.shexp_logit.assign(nt, 0.f);
    s.last.assign(nd, 0.f); s.final_norm.assign(nd, 0.f);

    // embed: the table is F32 here, so dequantisation is a copy (src/model/qwen35.rs:865-873).
    for (size_t t = 0; t < n; ++t) std::memcpy(&s.x[t * nd], w.tok_embd.row(tokens[t]), nd * 4);

    size_t slot = 0;
    for (size_t il = 0; il < c.n_layer; ++il) {
        const LayerWeights& L = w.layers[il];
        rms_norm(s.x.data(), n * nd, L.attn_norm, nd, c.rms_eps, s.normed.data());
        if (c.is_recurrent(il)) gated_delta(c, L, il, n, rs, s);
        else { attention(c, L, slot, start_pos, n, kv, s); slot++; }
        add_assign(s.x.data(), s.mixed.data(), n * nd);
        rms_norm(s.x.data(), n * nd, L.ffn_norm, nd, c.rms_eps, s.normed.data());
        std::vector<int32_t> ids;
        for (size_t t = 0; t < n;) {
            size_t take = std::min(MOE_CHUNK, n - t);
            moe_batch(c, L, t * nd, take, s, fp4act, log ? &ids : nullptr);
            t += take;
        }
        if (log) log->ids.insert(log->ids.end(), ids.begin(), ids.end());
        add_assign(s.x.data(), s.ffn_out.data(), n * nd);
    }
    kv.len = start_pos + n;  // src/model/qwen35.rs:1106
    gather_chunks(s.x.data(), nd, nd, (n - 1) * nd, s.last.data(), nd);
    rms_norm(s.last.data(), nd, w.output_norm, nd, c.rms_eps, s.final_norm.data());
    matmul(w.output, s.final_norm.data(), nd, logits);
    if (w.has_output_s) scale(logits, c.n_vocab, w.output_s);   // src/model/qwen35.rs:1117-1120
    return 0;
}

}  // namespace orc
