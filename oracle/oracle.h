// CPU oracle for the hybrid-MoE token loop: a C++ restatement of the reference's scalar
// backend (src/ops/naive.rs), the seam defaults (src/ops/mod.rs) and the qwen35moe forward
// pass (src/model/qwen35.rs).
//
// THIS IS TEST INFRASTRUCTURE, NOT THE PRODUCT. Only the test-suite, the smoke check and the
// CPU-baseline leg of the benchmark may call it. It is deliberately scalar and order-preserving:
// every f32 accumulation walks the same order as the reference so results can be compared to
// the bit. Build with -O2 -ffp-contract=off (the reference never contracts to FMA; the one
// explicit fused multiply-add is written as fmaf).
//
// Parity status: op level PINNED by the reference's own fixtures (NVFP4xQ8_0 dots, Q8_0
// activation bytes, Q8_0/F16/F32 dequantisation) and restated known-answer tests; whole-model
// level UNPINNED (the reference's model tests need checkpoint files that are not available),
// held instead by the reference's self-consistency invariants (batched == token-by-token,
// split prefill == single prefill).
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

namespace orc {

// ---- formats (src/quant/half.rs:29-114, src/quant/mod.rs:265-357) ----
float f16_to_f32(uint16_t h);
uint16_t f32_to_f16(float f);
uint16_t f32_to_bf16(float f);  // RN-even; the reference has only the decoder (half.rs:61-63)
float bf16_to_f32(uint16_t h);
extern const int8_t KVALUES_MXFP4[16];
float ue4m3_to_f32(uint8_t x);
uint8_t fp32_to_ue4m3_rn(float x);
void dequantize_q8_0(const uint8_t* data, float* out, size_t n);
void dequantize_nvfp4(const uint8_t* data, float* out, size_t n);

enum GgmlType : uint32_t { T_F32 = 0, T_F16 = 1, T_Q8_0 = 8, T_NVFP4 = 40 };
size_t row_bytes(uint32_t ty, size_t n_in);

// ---- activation quantisers and dots (src/ops/naive.rs:647-861) ----
struct QuantizedRow {
    std::vector<float> scales;
    std::vector<int8_t> quants;
    void from_f32(const float* x, size_t n);
    std::vector<uint8_t> to_blocks() const;
};
float dot_q8_0_q8_0(const uint8_t* row, size_t n_in, const QuantizedRow& x);
float dot_nvfp4_q8_0(const uint8_t* row, size_t n_in, const QuantizedRow& x);
struct Fp4Row {
    std::vector<uint8_t> scales, codes;
    void from_f32(const float* x, size_t n);
};
uint8_t e2m1_code(float x, float e);
float dot_nvfp4_fp4(const uint8_t* row, size_t n_in, const Fp4Row& x);
float dot_row(uint32_t ty, const uint8_t* row, const float* x, size_t n_in);

// ---- seam types (src/ops/mod.rs:62-455) ----
struct Weights {
    const uint8_t* data = nullptr;
    uint32_t ty = T_F32;
    size_t n_in = 0, n_out = 0;
    const uint8_t* row(size_t j) const { return data + j * row_bytes(ty, n_in); }
};
struct Experts {
    const uint8_t* data = nullptr;
    uint32_t ty = T_NVFP4;
    size_t n_in = 0, n_out = 0, n_expert = 0;
    const float* scale = nullptr;  // n_expert entries or null (= 1.0)
    size_t stride() const { return row_bytes(ty, n_in) * n_out; }
    Weights expert(size_t e) const { return Weights{data + e * stride(), ty, n_in, n_out}; }
};
struct Route {
    std::vector<size_t> ids;
    std::vector<float> weights;
    size_t n_used = 0;
    size_t n_tok() const { return ids.size() / (n_used ? n_used : 1); }
};
struct Attn {
    const float* q; size_t q_len;
    const uint16_t* k; const uint16_t* v;
    size_t kv_dim, n_pos, head_dim, n_head, n_head_kv;
    float scale;
    int kv_bf16 = 0;  // 0: f16 bits (the reference); 1: bf16 bits (extension)
    size_t group() const { return n_head / n_head_kv; }
    size_t n_q() const { return q_len / (n_head * head_dim); }
    size_t n_pos_of(size_t t) const { return n_pos - n_q() + 1 + t; }
};
struct Delta {
    const float *q, *k, *v, *alpha, *beta, *ssm_a, *dt_bias;
    size_t n_tokens, head_k_dim, head_v_dim, n_k_heads, n_v_heads;
};

// ---- ops (src/ops/naive.rs:138-466, src/ops/mod.rs:600-1425) ----
// n_threads > 1 splits independent output rows across threads; each row is computed by the same
// scalar code in the same order, so results do not depend on the thread count (the design of
// the reference's threaded CPU backends, src/ops/spin.rs:1-25).
void set_threads(int n);
int get_threads();

void rms_norm(const float* x, size_t x_len, const float* w, size_t nd, float eps, float* out);
void rms_norm_heads(float* x, size_t len, const float* w, size_t head_dim, float eps);
void matmul(const Weights& w, const float* x, size_t x_len, float* out);
void matmul_fp4act(const Weights& w, const float* x, size_t x_len, float* out);  // NVFP4 x FP4 (naive.rs:819)
void rope_neox(float* x, size_t len, size_t pos, size_t head_dim, size_t n_rot, size_t n_heads, float theta);
void softmax(float* x, size_t len, size_t row);
void attend(const Attn& a, float* out);
void silu_mul(float* gate, const float* up, size_t n);
void sigmoid_mul(float* x, const float* g, size_t n);
void scale(float* buf, size_t n, float s);
void add_assign(float* a, const float* b, size_t n);
void add_scaled(float* a, const float* b, size_t n, float s);
void add_scaled_rows(float* acc, size_t n, const float* rows, const float* scales, size_t n_rows);
void add_scaled_sigmoid(float* acc, const float* b, size_t n, const float* logit);
void l2_norm_heads(float* x, size_t len, size_t head_dim, float eps);
void ssm_conv(float* state, const float* x, size_t x_len, const float* w, size_t w_len, size_t kernel, float* out);
void gather_chunks(const float* src, size_t chunk, size_t stride, size_t offset, float* out, size_t out_len);
void scatter_chunks(const float* src, size_t src_len, size_t chunk, size_t stride, size_t offset, float* dst);
void delta_rule(const Delta& d, float* state, float* out);
void kv_write(uint16_t* slab, size_t offset, const float* src, size_t n, int bf16);
void route(const float* probs, size_t len, size_t n_expert, size_t n_used, Route& out);
void matmul_experts(const Experts& w, const Route& r, const float* x, size_t x_len, float* out, int fp4act);
void moe_glu(const Experts& gate, const Experts& up, const Route& r, const float* x, size_t x_len,
             float* out, float* scratch, int fp4act);
void moe_finish(float* out, size_t at, size_t n, const float* rows, const Route& r,
                const float* shared, const float* logit, size_t logit_at);

// ---- model (src/model/qwen35.rs) ----
struct Config {
    size_t n_layer, n_embd, n_head, n_head_kv, head_dim, n_vocab;
    float rope_theta, rms_eps;
    size_t n_rot;
    size_t ssm_d_conv, ssm_d_inner, ssm_d_state, ssm_dt_rank, ssm_n_group;
    size_t full_attention_interval;
    size_t n_expert, n_expert_used, expert_ff, shared_ff;
    size_t q_gate_dim() const { return head_dim * 2 * n_head; }
    size_t kv_dim() const { return n_head_kv * head_dim; }
    size_t head_k_dim() const { return ssm_d_state; }
    size_t head_v_dim() const { return ssm_d_inner / ssm_dt_rank; }
    size_t n_k_heads() const { return ssm_n_group; }
    size_t n_v_heads() const { return ssm_dt_rank; }
    size_t key_dim() const { return head_k_dim() * n_k_heads(); }
    size_t value_dim() const { return head_v_dim() * n_v_heads(); }
    size_t conv_dim() const { return key_dim() * 2 + value_dim(); }
    size_t ssm_state_len() const { return head_k_dim() * head_v_dim() * n_v_heads(); }
    size_t conv_state_len() const { return (ssm_d_conv - 1) * conv_dim(); }
    bool is_recurrent(size_t il) const { return (il + 1) % full_attention_interval != 0; }
};

struct LayerWeights {
    const float* attn_norm; const float* ffn_norm;
    // attention mixer
    Weights wq, wk, wv, wo; const float* q_norm; const float* k_norm;
    // delta mixer
    Weights wqkv, wgate, ssm_beta, ssm_alpha, ssm_out;
    const float *conv1d, *ssm_a, *dt_bias, *ssm_norm;
    // routed FFN
    Weights gate_inp, shared_gate, shared_up, shared_down, shared_gate_inp;
    Experts gate, up, down;
    // An NVFP4 file's second scale per shared-expert matmul (gate, up, down), applied to its output (src/model/qwen35.rs:1668-1682)
    float shared_s[3] = {1.0f, 1.0f, 1.0f}; bool has_shared_s[3] = {false, false, false};
};

struct ModelWeights {
    Config cfg;
    Weights tok_embd;  // F32 [n_vocab][n_embd]
    const float* output_norm;
    Weights output;
    float output_s = 1.0f; bool has_output_s = false;   // `output.scale`, the LM head's second scale, NVFP4 only (src/model/qwen35.rs:736-737, :1118)
    std::vector<LayerWeights> layers;
};

// KV cache (src/cache/mod.rs:33-253) and recurrent state (src/cache/recurrent.rs:31-141).
struct KvCache {
    size_t n_layer = 0, n_ctx = 0, kv_dim = 0, len = 0;
    int bf16 = 0;
    std::vector<uint16_t> k, v;  // [layer][pos][kv_dim]
    void init(size_t layers, size_t ctx, size_t dim, int use_bf16) {
        n_layer = layers; n_ctx = ctx; kv_dim = dim; len = 0; bf16 = use_bf16;
        k.assign(layers * ctx * dim, 0); v.assign(layers * ctx * dim, 0);
    }
    uint16_t* k_layer(size_t s) { return k.data() + s * n_ctx * kv_dim; }
    uint16_t* v_layer(size_t s) { return v.data() + s * n_ctx * kv_dim; }
};
struct RecurrentState {
    size_t n_layer = 0, conv_len = 0, ssm_len = 0;
    std::vector<float> conv, ssm;
    void init(size_t layers, size_t cl, size_t sl) {
        n_layer = layers; conv_len = cl; ssm_len = sl;
        conv.assign(layers * cl, 0.f); ssm.assign(layers * sl, 0.f);
    }
    float* conv_of(size_t il) { return conv.data() + il * conv_len; }
    float* ssm_of(size_t il) { return ssm.data() + il * ssm_len; }
};

// Per-pass record of the integer routing decisions, for bit-exact comparison.
struct RouteLog { std::vector<int32_t> ids; };  // [layer][token][n_used]

struct Model {
    ModelWeights w;
    int fp4act = 0;  // 0: routed experts multiply Q8_0 activations (the CPU reference path);
                     // 1: FP4 activations (naive.rs:819 dot_nvfp4_fp4, the tensor-core oracle)
    // forward (src/model/qwen35.rs:956-1127). Returns 0, or 1 on context overflow (cache untouched).
    int forward(const uint32_t* tokens, size_t n, size_t start_pos, KvCache& kv, RecurrentState& rs,
                float* logits, RouteLog* log = nullptr);
};

// greedy argmax, strict '>' so ties keep the lower index (src/profile.rs:192-213).
uint32_t argmax_top2(const float* logits, size_t n, uint32_t* second);

}  // namespace orc
