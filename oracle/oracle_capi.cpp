// C entry points of the CPU oracle, for ctypes. TEST INFRASTRUCTURE ONLY (see oracle.h).
#include <cmath>
#include <cstring>
#include <atomic>
#include <algorithm>
#include <map>
#include <memory>
#include <string>
#include <thread>

#include "../inferred-thoughts_b200/csrc/synth_model.h"
#include "oracle.h"

using namespace orc;

namespace {
struct OrcModel {
    synth::ModelDims dims;
    std::vector<synth::TensorSpec> specs;
    std::map<std::string, std::vector<uint8_t>> data;   // reference-layout bytes by tensor name
    std::map<std::string, std::vector<float>> scales;   // NVFP4 second scales by tensor name
    Model model;
    bool linked = false;
    KvCache kv;
    RecurrentState rs;
    RouteLog log;
    bool want_log = false;
};

Weights W(OrcModel& m, const std::string& name, uint32_t ty, size_t n_in, size_t n_out) {
    return Weights{m.data.at(name).data(), ty, n_in, n_out};
}
Experts E(OrcModel& m, const std::string& name, size_t n_in, size_t n_out, size_t n_expert) {
    auto it = m.scales.find(name);
    return Experts{m.data.at(name).data(), T_NVFP4, n_in, n_out, n_expert,
                   it == m.scales.end() ? nullptr : it->second.data()};
}
const float* V(OrcModel& m, const std::string& name) { return (const float*)m.data.at(name).data(); }
// A dense matrix that a file may carry as Q8_0 or as NVFP4 (shared experts, LM head): told apart by its byte count.
Weights WQ(OrcModel& m, const std::string& name, size_t n_in, size_t n_out) {
    const auto& d = m.data.at(name);
    const uint32_t ty = d.size() == n_in * n_out / 64 * 36 ? T_NVFP4 : T_Q8_0;
    return Weights{d.data(), ty, n_in, n_out};
}
// `<weight>.scale`, one f32 (src/model/mod.rs:351-361): true and *v set when the model carries it.
bool scalar(OrcModel& m, const std::string& name, float* v) {
    auto it = m.data.find(name);
    if (it == m.data.end() || it->second.size() != 4) return false;
    std::memcpy(v, it->second.data(), 4);
    return true;
}

void link(OrcModel& m) {
    const auto& d = m.dims;
    Config c{};
    c.n_layer = d.n_layer; c.n_embd = d.n_embd; c.n_head = d.n_head; c.n_head_kv = d.n_head_kv;
    c.head_dim = d.head_dim; c.n_vocab = d.n_vocab; c.rope_theta = d.rope_theta; c.rms_eps = d.rms_eps;
    c.n_rot = d.n_rot; c.ssm_d_conv = d.ssm_d_conv; c.ssm_d_inner = d.ssm_d_inner; c.ssm_d_state = d.ssm_d_state;
    c.ssm_dt_rank = d.ssm_dt_rank; c.ssm_n_group = d.ssm_n_group; c.full_attention_interval = d.full_attention_interval;
    c.n_expert = d.n_expert; c.n_expert_used = d.n_expert_used; c.expert_ff = d.expert_ff; c.shared_ff = d.shared_ff;
    ModelWeights& w = m.model.w;
    w.cfg = c;
    w.tok_embd = W(m, "token_embd.weight", T_F32, c.n_embd, c.n_vocab);
    w.output_norm = V(m, "output_norm.weight");
    w.output = WQ(m, "output.weight", c.n_embd, c.n_vocab);
    w.has_output_s = scalar(m, "output.scale", &w.output_s);
    w.layers.assign(c.n_layer, LayerWeights{});
    for (size_t i = 0; i < c.n_layer; ++i) {
        std::string P = "blk." + std::to_string(i) + ".";
        LayerWeights& L = w.layers[i];
        L.attn_norm = V(m, P + "attn_norm.weight");
        L.ffn_norm = V(m, P + "post_attention_norm.weight");
        if (c.is_recurrent(i)) {
            L.wqkv = W(m, P + "attn_qkv.weight", T_Q8_0, c.n_embd, c.conv_dim());
            L.wgate = W(m, P + "attn_gate.weight", T_Q8_0, c.n_embd, c.value_dim());
            L.conv1d = V(m, P + "ssm_conv1d.weight");
            L.ssm_beta = W(m, P + "ssm_beta.weight", T_F32, c.n_embd, c.n_v_heads());
            L.ssm_alpha = W(m, P + "ssm_alpha.weight", T_F32, c.n_embd, c.n_v_heads());
            L.ssm_a = V(m, P + "ssm_a");
            L.dt_bias = V(m, P + "ssm_dt.bias");
            L.ssm_norm = V(m, P + "ssm_norm.weight");
            L.ssm_out = W(m, P + "ssm_out.weight", T_Q8_0, c.value_dim(), c.n_embd);
        } else {
            L.wq = W(m, P + "attn_q.weight", T_Q8_0, c.n_embd, c.q_gate_dim());
            L.wk = W(m, P + "attn_k.weight", T_Q8_0, c.n_embd, c.kv_dim());
            L.wv = W(m, P + "attn_v.weight", T_Q8_0, c.n_embd, c.kv_dim());
            L.wo = W(m, P + "attn_output.weight", T_Q8_0, c.head_dim * c.n_head, c.n_embd);
            L.q_norm = V(m, P + "attn_q_norm.weight");
            L.k_norm = V(m, P + "attn_k_norm.weight");
        }
        L.gate_inp = W(m, P + "ffn_gate_inp.weight", T_F32, c.n_embd, c.n_expert);
        L.gate = E(m, P + "ffn_gate_exps.weight", c.n_embd, c.expert_ff, c.n_expert);
        L.up = E(m, P + "ffn_up_exps.weight", c.n_embd, c.expert_ff, c.n_expert);
        L.down = E(m, P + "ffn_down_exps.weight", c.expert_ff, c.n_embd, c.n_expert);
        L.shared_gate = WQ(m, P + "ffn_gate_shexp.weight", c.n_embd, c.shared_ff);
        L.shared_up = WQ(m, P + "ffn_up_shexp.weight", c.n_embd, c.shared_ff);
        L.shared_down = WQ(m, P + "ffn_down_shexp.weight", c.shared_ff, c.n_embd);
        L.has_shared_s[0] = scalar(m, P + "ffn_gate_shexp.scale", &L.shared_s[0]);
        L.has_shared_s[1] = scalar(m, P + "ffn_up_shexp.scale", &L.shared_s[1]);
        L.has_shared_s[2] = scalar(m, P + "ffn_down_shexp.scale", &L.shared_s[2]);
        L.shared_gate_inp = W(m, P + "ffn_gate_inp_shexp.weight", T_F32, c.n_embd, 1);
    }
    m.linked = true;
}
}  // namespace

extern "C" {

// ---- formats ----
float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_ue4m3_to_f32(uint8_t x) { return ue4m3_to_f32(x); }
uint8_t orc_fp32_to_ue4m3_rn(float x) { return fp32_to_ue4m3_rn(x); }
uint8_t orc_e2m1_code(float x, float e) { return e2m1_code(x, e); }
void orc_dequantize(uint32_t ty, const uint8_t* data, float* out, size_t n) {
    if (ty == T_Q8_0) dequantize_q8_0(data, out, n);
    else if (ty == T_NVFP4) dequantize_nvfp4(data, out, n);
    else if (ty == T_F16) for (size_t i = 0; i < n; ++i) out[i] = f16_to_f32((uint16_t)(data[2 * i] | data[2 * i + 1] << 8));
    else std::memcpy(out, data, n * 4);
}
void orc_q8_0_blocks(const float* x, size_t n, uint8_t* out) {
    QuantizedRow q; q.from_f32(x, n);
    auto b = q.to_blocks(); std::memcpy(out, b.data(), b.size());
}
void orc_fp4_activation(const float* x, size_t n, uint8_t* scales, uint8_t* codes) {
    Fp4Row r; r.from_f32(x, n);
    std::memcpy(scales, r.scales.data(), r.scales.size()); std::memcpy(codes, r.codes.data(), r.codes.size());
}
float orc_vec_dot_nvfp4_q8_0(const uint8_t* w, const float* x, size_t n) {
    QuantizedRow q; q.from_f32(x, n); return dot_nvfp4_q8_0(w, n, q);
}
float orc_vec_dot_nvfp4_fp4(const uint8_t* w, const float* x, size_t n) {
    Fp4Row q; q.from_f32(x, n); return dot_nvfp4_fp4(w, n, q);
}
float orc_vec_dot_q8_0(const uint8_t* w, const float* x, size_t n) {
    QuantizedRow q; q.from_f32(x, n); return dot_q8_0_q8_0(w, n, q);
}

// ---- ops ----
void orc_set_threads(int n) { set_threads(n); }
int orc_hw_threads() { return (int)std::thread::hardware_concurrency(); }
void orc_rms_norm(const float* x, size_t x_len, const float* w, size_t nd, float eps, float* out) { rms_norm(x, x_len, w, nd, eps, out); }
void orc_rms_norm_heads(float* x, size_t len, const float* w, size_t hd, float eps) { rms_norm_heads(x, len, w, hd, eps); }
void orc_matmul(uint32_t ty, const uint8_t* data, size_t n_in, size_t n_out, const float* x, size_t x_len, float* out, int fp4act) {
    Weights w{data, ty, n_in, n_out};
    if (fp4act) matmul_fp4act(w, x, x_len, out); else matmul(w, x, x_len, out);
}
void orc_rope_neox(float* x, size_t len, size_t pos, size_t hd, size_t n_rot, size_t n_heads, float theta) { rope_neox(x, len, pos, hd, n_rot, n_heads, theta); }
void orc_softmax(float* x, size_t len, size_t row) { softmax(x, len, row); }
void orc_attend(const float* q, size_t q_len, const uint16_t* k, const uint16_t* v, size_t kv_dim, size_t n_pos,
                size_t head_dim, size_t n_head, size_t n_head_kv, float scale, int kv_bf16, float* out) {
    Attn a{q, q_len, k, v, kv_dim, n_pos, head_dim, n_head, n_head_kv, scale, kv_bf16};
    attend(a, out);
}
void orc_silu_mul(float* g, const float* u, size_t n) { silu_mul(g, u, n); }
void orc_sigmoid_mul(float* x, const float* g, size_t n) { sigmoid_mul(x, g, n); }
void orc_scale(float* b, size_t n, float s) { scale(b, n, s); }
void orc_add_assign(float* a, const float* b, size_t n) { add_assign(a, b, n); }
void orc_add_scaled(float* a, const float* b, size_t n, float s) { add_scaled(a, b, n, s); }
void orc_add_scaled_rows(float* acc, size_t n, const float* rows, const float* scales, size_t n_rows) { add_scaled_rows(acc, n, rows, scales, n_rows); }
void orc_add_scaled_sigmoid(float* acc, const float* b, size_t n, const float* logit) { add_scaled_sigmoid(acc, b, n, logit); }
void orc_l2_norm_heads(float* x, size_t len, size_t hd, float eps) { l2_norm_heads(x, len, hd, eps); }
void orc_ssm_conv(float* state, const float* x, size_t x_len, const float* w, size_t w_len, size_t kernel, float* out) { ssm_conv(state, x, x_len, w, w_len, kernel, out); }
void orc_gather_chunks(const float* src, size_t chunk, size_t stride, size_t offset, float* out, size_t out_len) { gather_chunks(src, chunk, stride, offset, out, out_len); }
void orc_scatter_chunks(const float* src, size_t src_len, size_t chunk, size_t stride, size_t offset, float* dst) { scatter_chunks(src, src_len, chunk, stride, offset, dst); }
void orc_delta_rule(const float* q, const float* k, const float* v, const float* alpha, const float* beta,
                    const float* ssm_a, const float* dt_bias, size_t n_tokens, size_t hk, size_t hv, size_t nk,
                    size_t nv, float* state, float* out) {
    Delta d{q, k, v, alpha, beta, ssm_a, dt_bias, n_tokens, hk, hv, nk, nv};
    delta_rule(d, state, out);
}
void orc_kv_write(uint16_t* slab, size_t offset, const float* src, size_t n, int bf16) { kv_write(slab, offset, src, n, bf16); }
void orc_route(const float* probs, size_t len, size_t n_expert, size_t n_used, int32_t* ids, float* weights) {
    Route r; route(probs, len, n_expert, n_used, r);
    for (size_t i = 0; i < r.ids.size(); ++i) { ids[i] = (int32_t)r.ids[i]; weights[i] = r.weights[i]; }
}
static Route mk_route(const int32_t* ids, const float* weights, size_t n_pairs, size_t n_used) {
    Route r; r.n_used = n_used;
    r.ids.assign(ids, ids + n_pairs);
    if (weights) r.weights.assign(weights, weights + n_pairs);
    return r;
}
void orc_matmul_experts(const uint8_t* data, size_t n_in, size_t n_out, size_t n_expert, const float* scale,
                        const int32_t* ids, size_t n_pairs, size_t n_used, const float* x, size_t x_len, float* out, int fp4act) {
    Experts w{data, T_NVFP4, n_in, n_out, n_expert, scale};
    matmul_experts(w, mk_route(ids, nullptr, n_pairs, n_used), x, x_len, out, fp4act);
}
void orc_moe_glu(const uint8_t* gate, const float* gscale, const uint8_t* up, const float* uscale, size_t n_in, size_t n_out,
                 size_t n_expert, const int32_t* ids, size_t n_pairs, size_t n_used, const float* x, size_t x_len,
                 float* out, int fp4act) {
    Experts g{gate, T_NVFP4, n_in, n_out, n_expert, gscale}, u{up, T_NVFP4, n_in, n_out, n_expert, uscale};
    std::vector<float> scratch(n_pairs * n_out);
    moe_glu(g, u, mk_route(ids, nullptr, n_pairs, n_used), x, x_len, out, scratch.data(), fp4act);
}
void orc_moe_finish(float* out, size_t at, size_t n, const float* rows, const int32_t* ids, const float* weights,
                    size_t n_pairs, size_t n_used, const float* shared, const float* logit, size_t logit_at) {
    moe_finish(out, at, n, rows, mk_route(ids, weights, n_pairs, n_used), shared, logit, logit_at);
}
// The C library's expf (kind 0) / logf (kind 1) over an array: what Rust's f32::exp / f32::ln call on this platform
// (src/ops/naive.rs:101-106, :246-252, :362-376 use them).
void orc_libm(int kind, const float* in, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) out[i] = kind == 0 ? expf(in[i]) : logf(in[i]);
}
uint32_t orc_argmax(const float* logits, size_t n, uint32_t* second) { return argmax_top2(logits, n, second); }

// ---- synthetic tensors and model ----
uint64_t orc_tensor_key(uint64_t seed, const char* name) { return synth::tensor_key(seed, name); }
float orc_synth_value(uint64_t key, uint64_t i, int dist, float sd) { return synth::value(key, i, dist, sd); }

void* orc_model_create(const synth::ModelDims* dims) {
    auto* m = new OrcModel();
    m->dims = *dims;
    m->specs = synth::model_tensors(*dims);
    return m;
}
void orc_model_destroy(void* h) { delete (OrcModel*)h; }
size_t orc_model_n_tensors(void* h) { return ((OrcModel*)h)->specs.size(); }
// name/type/shape of tensor i; returns its byte size.
size_t orc_model_tensor_info(void* h, size_t i, char* name, size_t cap, uint32_t* ty, uint64_t* n_in, uint64_t* n_out,
                             uint64_t* n_expert, int* has_scale) {
    auto& t = ((OrcModel*)h)->specs[i];
    snprintf(name, cap, "%s", t.name.c_str());
    *ty = t.ty; *n_in = t.n_in; *n_out = t.n_out; *n_expert = t.n_expert; *has_scale = t.has_scale;
    return t.bytes();
}
// Generate every tensor on the CPU (threaded over tensors).
void orc_model_synth(void* h, uint64_t seed, int n_threads) {
    auto* m = (OrcModel*)h;
    for (auto& t : m->specs) {
        m->data[t.name].resize(t.bytes());
        if (t.has_scale) m->scales[t.name].resize(t.n_expert);
    }
    std::vector<std::thread> th;
    std::atomic<size_t> next_v(0); std::atomic<size_t>* next = &next_v;
    auto work = [&]() {
        for (;;) {
            size_t i = next->fetch_add(1);
            if (i >= m->specs.size()) break;
            auto& t = m->specs[i];
            synth::generate_tensor_cpu(t, seed, m->data[t.name].data(), t.has_scale ? m->scales[t.name].data() : nullptr);
        }
    };
    for (int i = 1; i < n_threads; ++i) th.emplace_back(work);
    work();
    for (auto& t : th) t.join();
    link(*m);
}
// Supply a tensor's bytes (and NVFP4 second scales) from outside, e.g. copied back from a device.
int orc_model_set_tensor(void* h, const char* name, const uint8_t* bytes, size_t n, const float* scale, size_t n_scale) {
    auto* m = (OrcModel*)h;
    m->data[name].assign(bytes, bytes + n);
    if (scale) m->scales[name].assign(scale, scale + n_scale);
    m->linked = false;
    return 0;
}
const uint8_t* orc_model_tensor_data(void* h, const char* name) { return ((OrcModel*)h)->data.at(name).data(); }
const float* orc_model_tensor_scale(void* h, const char* name) {
    auto* m = (OrcModel*)h; auto it = m->scales.find(name);
    return it == m->scales.end() ? nullptr : it->second.data();
}
void orc_model_begin(void* h, size_t n_ctx, int kv_bf16, int fp4act) {
    auto* m = (OrcModel*)h;
    if (!m->linked) link(*m);
    const Config& c = m->model.w.cfg;
    size_t n_attn = 0;
    for (size_t i = 0; i < c.n_layer; ++i) if (!c.is_recurrent(i)) n_attn++;
    m->kv.init(n_attn, n_ctx, c.kv_dim(), kv_bf16);
    m->rs.init(c.n_layer, c.conv_state_len(), c.ssm_state_len());
    m->model.fp4act = fp4act;
    m->log.ids.clear();
}
void orc_model_log_routes(void* h, int on) { ((OrcModel*)h)->want_log = on != 0; }
size_t orc_model_pos(void* h) { return ((OrcModel*)h)->kv.len; }
// One forward pass appended at the current position (src/engine/mod.rs:310-324).
int orc_model_forward(void* h, const uint32_t* tokens, size_t n, float* logits) {
    auto* m = (OrcModel*)h;
    return m->model.forward(tokens, n, m->kv.len, m->kv, m->rs, logits, m->want_log ? &m->log : nullptr);
}
size_t orc_model_route_log(void* h, int32_t* out, size_t cap) {
    auto* m = (OrcModel*)h;
    size_t n = m->log.ids.size();
    if (out) std::memcpy(out, m->log.ids.data(), std::min(n, cap) * 4);
    return n;
}
void orc_model_clear_route_log(void* h) { ((OrcModel*)h)->log.ids.clear(); }
// Recurrent state and KV slabs, for state-left-behind checks.
float* orc_model_ssm_state(void* h, size_t il) { return ((OrcModel*)h)->rs.ssm_of(il); }
float* orc_model_conv_state(void* h, size_t il) { return ((OrcModel*)h)->rs.conv_of(il); }
uint16_t* orc_model_k_slab(void* h, size_t slot) { return ((OrcModel*)h)->kv.k_layer(slot); }
uint16_t* orc_model_v_slab(void* h, size_t slot) { return ((OrcModel*)h)->kv.v_layer(slot); }

// Greedy generation (src/engine/mod.rs:399-437): chunked prefill (max_batch), then one token at a time.
// Returns the number of tokens produced; `margins` (optional) receives top1-top2 logit gaps.
size_t orc_model_generate(void* h, const uint32_t* prompt, size_t n_prompt, size_t max_new, size_t max_batch,
                          uint32_t* out, float* margins) {
    auto* m = (OrcModel*)h;
    size_t nv = m->model.w.cfg.n_vocab;
    std::vector<float> logits(nv);
    for (size_t t = 0; t < n_prompt; t += max_batch) {
        size_t take = std::min(max_batch, n_prompt - t);
        if (orc_model_forward(h, prompt + t, take, logits.data())) return 0;
    }
    size_t produced = 0;
    for (size_t i = 0; i < max_new; ++i) {
        uint32_t second, next = argmax_top2(logits.data(), nv, &second);
        if (margins) margins[produced] = logits[next] - logits[second];
        out[produced++] = next;
        if (produced == max_new) break;
        if (m->kv.len + 1 >= m->kv.n_ctx) break;
        if (orc_model_forward(h, &next, 1, logits.data())) break;
    }
    return produced;
}

}  // extern "C"
