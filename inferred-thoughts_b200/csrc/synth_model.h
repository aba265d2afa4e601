// Tensor inventory of a synthetic qwen35moe-structured model: names (GGUF spelling, as loaded by
// src/model/qwen35.rs:755-858), storage types, shapes and value distributions. Host-only.
// Shared by the device generator and by the CPU generator used in tests, so both sides name the
// same tensors in the same order and feed them the same keys.
#pragma once
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <vector>

#include "synth.h"

namespace synth {

struct ModelDims {
    uint32_t n_layer, n_embd, n_head, n_head_kv, head_dim, n_vocab;
    float rope_theta, rms_eps;
    uint32_t n_rot, ssm_d_conv, ssm_d_inner, ssm_d_state, ssm_dt_rank, ssm_n_group, full_attention_interval;
    uint32_t n_expert, n_expert_used, expert_ff, shared_ff;
};

enum : uint32_t { TY_F32 = 0, TY_F16 = 1, TY_Q8_0 = 8, TY_NVFP4 = 40 };

struct TensorSpec {
    std::string name;
    uint32_t ty;
    uint64_t n_in, n_out, n_expert;  // n_expert = 1 for plain matrices; vectors are n_out = 1
    int dist;
    float std_;
    bool has_scale;  // NVFP4: a per-expert f32 second scale tensor "<name minus .weight>.scale" accompanies it
    uint64_t elems() const { return n_in * n_out * n_expert; }
    uint64_t bytes() const {
        uint64_t e = elems();
        return ty == TY_F32 ? e * 4 : ty == TY_F16 ? e * 2 : ty == TY_Q8_0 ? e / 32 * 34 : e / 64 * 36;
    }
};

inline bool is_recurrent(const ModelDims& d, uint32_t il) { return (il + 1) % d.full_attention_interval != 0; }

// Every tensor of the model, in generation order (globals, then by layer).
inline std::vector<TensorSpec> model_tensors(const ModelDims& d) {
    std::vector<TensorSpec> v;
    const float S = 0.02f;
    auto mat = [&](const std::string& n, uint32_t ty, uint64_t n_in, uint64_t n_out) {
        v.push_back({n, ty, n_in, n_out, 1, DIST_NORMAL, S, false});
    };
    auto vec = [&](const std::string& n, uint64_t len, int dist, float sd) {
        v.push_back({n, TY_F32, len, 1, 1, dist, sd, false});
    };
    uint64_t head_v = d.ssm_d_inner / d.ssm_dt_rank, key_dim = (uint64_t)d.ssm_d_state * d.ssm_n_group;
    uint64_t conv_dim = 2 * key_dim + d.ssm_d_inner;
    mat("token_embd.weight", TY_F32, d.n_embd, d.n_vocab);
    vec("output_norm.weight", d.n_embd, DIST_ONE_PLUS, S);
    mat("output.weight", TY_Q8_0, d.n_embd, d.n_vocab);
    for (uint32_t i = 0; i < d.n_layer; ++i) {
        char p[64]; snprintf(p, sizeof p, "blk.%u.", i);
        std::string P(p);
        vec(P + "attn_norm.weight", d.n_embd, DIST_ONE_PLUS, S);
        vec(P + "post_attention_norm.weight", d.n_embd, DIST_ONE_PLUS, S);
        if (is_recurrent(d, i)) {
            mat(P + "attn_qkv.weight", TY_Q8_0, d.n_embd, conv_dim);
            mat(P + "attn_gate.weight", TY_Q8_0, d.n_embd, d.ssm_d_inner);
            v.push_back({P + "ssm_conv1d.weight", TY_F32, d.ssm_d_conv, conv_dim, 1, DIST_NORMAL, S, false});
            mat(P + "ssm_beta.weight", TY_F32, d.n_embd, d.ssm_dt_rank);
            mat(P + "ssm_alpha.weight", TY_F32, d.n_embd, d.ssm_dt_rank);
            vec(P + "ssm_a", d.ssm_dt_rank, DIST_NEG_ABS, 1.0f);
            vec(P + "ssm_dt.bias", d.ssm_dt_rank, DIST_NORMAL, S);
            vec(P + "ssm_norm.weight", head_v, DIST_ONE_PLUS, S);
            mat(P + "ssm_out.weight", TY_Q8_0, d.ssm_d_inner, d.n_embd);
        } else {
            mat(P + "attn_q.weight", TY_Q8_0, d.n_embd, (uint64_t)d.head_dim * 2 * d.n_head);
            mat(P + "attn_k.weight", TY_Q8_0, d.n_embd, (uint64_t)d.head_dim * d.n_head_kv);
            mat(P + "attn_v.weight", TY_Q8_0, d.n_embd, (uint64_t)d.head_dim * d.n_head_kv);
            mat(P + "attn_output.weight", TY_Q8_0, (uint64_t)d.head_dim * d.n_head, d.n_embd);
            vec(P + "attn_q_norm.weight", d.head_dim, DIST_ONE_PLUS, S);
            vec(P + "attn_k_norm.weight", d.head_dim, DIST_ONE_PLUS, S);
        }
        mat(P + "ffn_gate_inp.weight", TY_F32, d.n_embd, d.n_expert);
        v.push_back({P + "ffn_gate_exps.weight", TY_NVFP4, d.n_embd, d.expert_ff, d.n_expert, DIST_NORMAL, S, true});
        v.push_back({P + "ffn_up_exps.weight", TY_NVFP4, d.n_embd, d.expert_ff, d.n_expert, DIST_NORMAL, S, true});
        v.push_back({P + "ffn_down_exps.weight", TY_NVFP4, d.expert_ff, d.n_embd, d.n_expert, DIST_NORMAL, S, true});
        mat(P + "ffn_gate_shexp.weight", TY_Q8_0, d.n_embd, d.shared_ff);
        mat(P + "ffn_up_shexp.weight", TY_Q8_0, d.n_embd, d.shared_ff);
        mat(P + "ffn_down_shexp.weight", TY_Q8_0, d.shared_ff, d.n_embd);
        mat(P + "ffn_gate_inp_shexp.weight", TY_F32, d.n_embd, 1);
    }
    return v;
}

// CPU generation of one tensor into reference-layout bytes. `scale_out` receives n_expert f32 for
// NVFP4 tensors (may be null otherwise).
inline void generate_tensor_cpu(const TensorSpec& t, uint64_t seed, uint8_t* out, float* scale_out) {
    uint64_t key = tensor_key(seed, t.name.c_str());
    uint64_t per_expert = t.n_in * t.n_out;
    if (t.ty == TY_F32) {
        float* o = (float*)out;
        for (uint64_t i = 0; i < t.elems(); ++i) o[i] = value(key, i, t.dist, t.std_);
    } else if (t.ty == TY_Q8_0) {
        float blk[32];
        for (uint64_t b = 0; b < t.elems() / 32; ++b) {
            for (int j = 0; j < 32; ++j) blk[j] = value(key, b * 32 + j, t.dist, t.std_);
            quantize_q8_0_block(blk, out + b * 34);
        }
    } else if (t.ty == TY_NVFP4) {
        std::vector<float> vals(per_expert);
        for (uint64_t e = 0; e < t.n_expert; ++e) {
            float amax = 0.0f;
            for (uint64_t i = 0; i < per_expert; ++i) {
                vals[i] = value(key, e * per_expert + i, t.dist, t.std_);
                amax = fmaxf(amax, fabsf(vals[i]));
            }
            float s2 = nvfp4_second_scale(amax);
            if (scale_out) scale_out[e] = s2;
            for (uint64_t b = 0; b < per_expert / 64; ++b)
                quantize_nvfp4_block(&vals[b * 64], s2, out + (e * per_expert / 64 + b) * 36);
        }
    }
}

}  // namespace synth
