// Model + engine level: the token loop as a short chain of fused kernels replayed as one CUDA graph.
//
// Restates, natively, what the reference drives through its op seam: Qwen35::forward
// (src/model/qwen35.rs:956-1127), the attention block (:1138-1223), the GatedDeltaNet block
// (:1232-1328), the routed FFN (:1587-1699) and Engine::{prefill,decode,generate}
// (src/engine/mod.rs:352-437). The arithmetic of every matmul, norm, conv, delta-rule and routing
// step keeps the CPU path's order; only exp() and the attention reduction are tolerance class.
#include <algorithm>
#include <chrono>
#include <array>
#include <memory>

#include "itb_kernels.cuh"
#include "synth_model.h"
#include "itb_tier.h"

void itb_attend_dev(itb_ctx* c, cudaStream_t st, const float* q, const uint16_t* k, const uint16_t* v, int kv_dim, int n_pos, int n_q,
                    int hd, int n_head, int n_head_kv, float scale, int bf16, const int* n_pos_dev, const float* gate,
                    float* part_acc, float* part_ml, int n_split, float* out);
void itb_synth_f32(cudaStream_t st, uint64_t key, size_t n, int dist, float sd, float* out);
void itb_synth_q8_raw(cudaStream_t st, uint64_t key, size_t n_blocks, int dist, float sd, uint8_t* raw);
void itb_synth_fp4_raw(cudaStream_t st, uint64_t key, size_t per_expert, size_t e_lo, size_t e_hi, int dist, float sd,
                       unsigned* amax_tmp, float* scale2, uint8_t* raw);

#include "itb_fused.cuh"
#include "itb_mega.cuh"
#include "itb_rows.cuh"
#include "itb_attn_exact.cuh"
#include "itb_attn_mma.cuh"
#include "itb_gdn_chunk.cuh"

void itb_engine_use_logf_fix(const uint32_t* dev_tab, uint32_t n) {
    cudaMemcpyToSymbol(g_logf_fix, &dev_tab, sizeof dev_tab);
    cudaMemcpyToSymbol(g_logf_fix_n, &n, sizeof n);
}

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
    // a file may carry the shared expert as NVFP4 with one second scale per matmul (src/model/mod.rs:351-361,
    // src/model/qwen35.rs:1668-1682): then the Q8_0 views above are empty and these hold it (gate, up, down)
    DevFp4 shared4[3]; float shared_s[3] = {1.0f, 1.0f, 1.0f}; bool has_shared_s[3] = {false, false, false};
};
struct itb_model {
    itb_ctx* c = nullptr;
    itb_model_dims d{};
    std::map<std::string, DevTensor> t;
    std::vector<DevLayer> layers;
    DevF32 tok_embd; const float* output_norm = nullptr; DevQ8 output;
    DevFp4 output4; float output_s = 1.0f; bool has_output_s = false;   // the LM head as NVFP4 with `output.scale` (src/model/qwen35.rs:736-737, :1118)
    bool dense_fp4 = false;                  // some shared expert or the LM head is NVFP4: steps run the multi-row kernels
    std::map<std::string, float> scalars;    // `<weight>.scale` of the dense NVFP4 matrices
    bool finalized = false;
    uint32_t expert_lo = 0, expert_hi = 0;
    size_t bytes = 0;
    // routed experts moved to pinned host memory (itb_model_offload_experts): per layer, per stack (gate, up, down)
    struct HostStack { uint8_t* nib = nullptr; uint8_t* sc = nullptr; std::vector<float> s2; size_t nib_per = 0, sc_per = 0; bool has_s2 = false; };
    std::vector<std::array<HostStack, 3>> host_experts;
    bool offloaded = false;
    std::vector<void*> extra;      // device copies this model made beside its tensors (k-major F32 copies)
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
    if ((d->ssm_d_state != 64 && d->ssm_d_state != 128) || d->ssm_d_conv < 2 || d->ssm_d_conv > 8 || d->n_expert > 1024) return bad("dimension beyond what the kernels hold");
    itb_model* m = new itb_model();
    m->c = c; m->d = *d;
    *out = m;
    return 0;
}
extern "C" void itb_model_dims_of(itb_model* m, itb_model_dims* out) { *out = m->d; }
extern "C" void itb_model_destroy(itb_model* m) {
    if (!m) return;
    cudaStreamSynchronize(m->c->stream);
    for (auto& kv : m->t) { cudaFree(kv.second.a); cudaFree(kv.second.b); cudaFree(kv.second.scale2); }
    for (auto& l : m->host_experts) for (auto& h : l) { cudaFreeHost(h.nib); cudaFreeHost(h.sc); }
    for (void* p : m->extra) cudaFree(p);
    delete m;
}

// raw reference-layout bytes already on the device -> kernel layout
static int adopt_raw(itb_model* m, const std::string& name, uint32_t ty, size_t n_in, size_t n_out, size_t n_expert,
                     size_t e_lo, size_t e_cnt, uint8_t* raw, float* scale2_dev) {
    itb_ctx* c = m->c;
    DevTensor t;
    t.ty = ty; t.n_in = n_in; t.n_out = n_out; t.n_expert = n_expert; t.e_lo = e_lo; t.e_cnt = e_cnt;
    size_t elems = n_in * n_out * e_cnt;
    // both planes or neither: a failed second allocation gives the first one back, and nothing is launched
    auto two = [&](size_t a_bytes, size_t b_bytes) {
        if (cudaMalloc(&t.a, a_bytes) != cudaSuccess) { t.a = nullptr; return itb_fail_msg(c, "model: out of device memory for " + name); }
        if (cudaMalloc(&t.b, b_bytes) != cudaSuccess) { cudaFree(t.a); t.a = t.b = nullptr; return itb_fail_msg(c, "model: out of device memory for " + name); }
        return true;
    };
    if (ty == ITB_Q8_0) {
        if (!two(elems, elems / 32 * 2)) return 1;
        itb_repack_q8(c->stream, raw, (int8_t*)t.a, (uint16_t*)t.b, elems / 32);
        t.bytes = elems + elems / 16;
    } else if (ty == ITB_NVFP4) {
        if (!two(elems / 2, elems / 16)) return 1;
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
    const std::string nm(name);
    auto dense_fp4_ok = [](const std::string& n) {
        return n == "output.weight" || n.find("ffn_gate_shexp.weight") != std::string::npos || n.find("ffn_up_shexp.weight") != std::string::npos ||
               n.find("ffn_down_shexp.weight") != std::string::npos;
    };
    if (nm.size() > 6 && nm.compare(nm.size() - 6, 6, ".scale") == 0) {
        // `<weight>.scale`: the one-element second scale of a dense NVFP4 matrix (the experts' per-expert scales travel with set_tensor's `scale`)
        const std::string wname = nm.substr(0, nm.size() - 6) + ".weight";
        if (!dense_fp4_ok(wname) || !find_spec(specs, wname.c_str())) { itb_fail_msg(c, std::string("set_tensor: no weight takes the scalar ") + name); return 1; }
        if (ty != ITB_F32 || bytes != 4) { itb_fail_msg(c, std::string("set_tensor: ") + name + " must be one f32"); return 1; }
        float v; memcpy(&v, data, 4);
        m->scalars[nm] = v; m->finalized = false;
        return 0;
    }
    const synth::TensorSpec* s = find_spec(specs, name);
    if (!s) { itb_fail_msg(c, std::string("set_tensor: unknown tensor ") + name); return 1; }
    const bool as_fp4 = ty == ITB_NVFP4 && s->ty == synth::TY_Q8_0 && dense_fp4_ok(nm) && s->n_in % 64 == 0;
    if (s->ty != ty && !as_fp4) { itb_fail_msg(c, std::string("set_tensor: ") + name + " has a storage type this path has no kernel for"); return 1; }
    if (bytes != (as_fp4 ? s->n_in * s->n_out / 64 * 36 : s->bytes())) { itb_fail_msg(c, std::string("set_tensor: wrong byte count for ") + name); return 1; }
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
    if (as_fp4) {
        // a dense NVFP4 matrix: its one-element `.scale` (handed over with the weight, as the GGUF loader does, or set by name)
        // is kept on the host and applied to the matmul's result
        if (scale && n_scale >= 1) m->scalars[nm.substr(0, nm.size() - 7) + ".scale"] = scale[0];
        scale = nullptr; n_scale = 0;
    }
    uint8_t* raw = nullptr;
    ITB_CUDA_RET(c, cudaMalloc(&raw, bytes), 1);
    if (cudaMemcpyAsync(raw, data, bytes, cudaMemcpyHostToDevice, c->stream) != cudaSuccess) { cudaFree(raw); itb_fail_msg(c, std::string("set_tensor: upload failed for ") + name); return 1; }
    float* s2 = nullptr;
    if (ty == ITB_NVFP4 && scale && n_scale >= s->n_expert) {
        if (cudaMalloc(&s2, s->n_expert * 4) != cudaSuccess) { cudaStreamSynchronize(c->stream); cudaFree(raw); itb_fail_msg(c, std::string("set_tensor: out of device memory for ") + name); return 1; }
        cudaMemcpyAsync(s2, scale, s->n_expert * 4, cudaMemcpyHostToDevice, c->stream);
    }
    int rc = adopt_raw(m, name, ty, s->n_in, s->n_out, s->n_expert, 0, s->n_expert, raw, s2);
    if (rc) cudaFree(s2);
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

// w[n_out][n_in] -> units of 32 rows, k-major inside a unit: wt[(u * n_in + k) * 32 + r] = w[u * 32 + r][k] (zero past n_out).
__global__ void k_f32_kmajor(const float* w, int n_in, int n_out, float* wt) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, total = (size_t)((n_out + 31) / 32) * n_in * 32;
    if (i >= total) return;
    const int r = (int)(i % 32); const size_t uk = i / 32; const int k = (int)(uk % n_in), u = (int)(uk / n_in), row = u * 32 + r;
    wt[i] = row < n_out ? w[(size_t)row * n_in + k] : 0.0f;
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
    // the small F32 matrices of the one-token step (router, shared-expert gate, alpha, beta) also k-major, for the serial-k fold
    auto f32k = [&](const std::string& n) {
        DevF32 w = f32(n);
        if (!w.w || !c->exact) return w;
        const size_t total = (size_t)((w.n_out + 31) / 32) * w.n_in * 32;
        float* wt = nullptr;
        if (cudaMalloc(&wt, total * 4) != cudaSuccess) { cudaGetLastError(); return w; }      // without the copy the row-per-warp path serves
        k_f32_kmajor<<<(unsigned)((total + 255) / 256), 256, 0, c->stream>>>(w.w, w.n_in, w.n_out, wt);
        m->extra.push_back(wt); m->bytes += total * 4;
        w.wt = wt;
        return w;
    };
    auto vec = [&](const std::string& n) { const DevTensor* t = get(n); return t ? (const float*)t->a : nullptr; };
    auto fp4 = [&](const std::string& n) {
        const DevTensor* t = get(n);
        return t ? DevFp4{(const uint8_t*)t->a, (const uint8_t*)t->b, t->scale2, (int)t->n_in, (int)t->n_out, (int)t->e_cnt, (int)t->e_lo} : DevFp4{};
    };
    // a dense matrix that may be stored as Q8_0 or as NVFP4: one of the two views is filled
    auto dense = [&](const std::string& n, DevQ8* q, DevFp4* f4, float* sc, bool* has_sc) {
        const DevTensor* t = get(n);
        *q = DevQ8{}; *f4 = DevFp4{}; *has_sc = false;
        if (!t) return;
        if (t->ty == ITB_NVFP4) {
            *f4 = DevFp4{(const uint8_t*)t->a, (const uint8_t*)t->b, nullptr, (int)t->n_in, (int)t->n_out, 1, 0};
            m->dense_fp4 = true;
            auto it = m->scalars.find(n.substr(0, n.size() - 7) + ".scale");
            if (it != m->scalars.end()) { *sc = it->second; *has_sc = true; }
        } else *q = DevQ8{(const int8_t*)t->a, (const uint16_t*)t->b, (int)t->n_in, (int)t->n_out};
    };
    m->dense_fp4 = false;
    m->tok_embd = f32("token_embd.weight");
    m->output_norm = vec("output_norm.weight");
    dense("output.weight", &m->output, &m->output4, &m->output_s, &m->has_output_s);
    m->layers.assign(d.n_layer, DevLayer{});
    for (uint32_t i = 0; i < d.n_layer && ok; ++i) {
        std::string P = "blk." + std::to_string(i) + ".";
        DevLayer& L = m->layers[i];
        L.recurrent = (i + 1) % d.full_attention_interval != 0;   // src/model/qwen35.rs:329-331
        L.attn_norm = vec(P + "attn_norm.weight");
        L.ffn_norm = vec(P + "post_attention_norm.weight");
        if (L.recurrent) {
            L.wqkv = q8(P + "attn_qkv.weight"); L.wgate = q8(P + "attn_gate.weight"); L.ssm_out = q8(P + "ssm_out.weight");
            L.ssm_alpha = f32k(P + "ssm_alpha.weight"); L.ssm_beta = f32k(P + "ssm_beta.weight");
            L.conv1d = vec(P + "ssm_conv1d.weight"); L.ssm_a = vec(P + "ssm_a"); L.dt_bias = vec(P + "ssm_dt.bias");
            L.ssm_norm = vec(P + "ssm_norm.weight");
        } else {
            L.wq = q8(P + "attn_q.weight"); L.wk = q8(P + "attn_k.weight"); L.wv = q8(P + "attn_v.weight");
            L.wo = q8(P + "attn_output.weight");
            L.q_norm = vec(P + "attn_q_norm.weight"); L.k_norm = vec(P + "attn_k_norm.weight");
        }
        L.gate_inp = f32k(P + "ffn_gate_inp.weight"); L.shared_gate_inp = f32k(P + "ffn_gate_inp_shexp.weight");
        L.gate = fp4(P + "ffn_gate_exps.weight"); L.up = fp4(P + "ffn_up_exps.weight"); L.down = fp4(P + "ffn_down_exps.weight");
        dense(P + "ffn_gate_shexp.weight", &L.shared_gate, &L.shared4[0], &L.shared_s[0], &L.has_shared_s[0]);
        dense(P + "ffn_up_shexp.weight", &L.shared_up, &L.shared4[1], &L.shared_s[1], &L.has_shared_s[1]);
        dense(P + "ffn_down_shexp.weight", &L.shared_down, &L.shared4[2], &L.shared_s[2], &L.has_shared_s[2]);
    }
    m->finalized = ok;
    return ok;
}

// Move the routed-expert stacks to pinned host memory and free their device copies: what an expert-tiered engine
// (itb_engine_create_tiered) starts from. Everything else stays on the device.
extern "C" int itb_model_offload_experts(itb_model* m) {
    itb_ctx* c = m->c;
    if (m->offloaded) return 0;
    if (!finalize(m)) return 1;
    if (m->expert_hi && (m->expert_lo != 0 || m->expert_hi != m->d.n_expert)) { itb_fail_msg(c, "offload: the model holds an expert shard"); return 1; }
    const itb_model_dims& d = m->d;
    cudaStreamSynchronize(c->stream);
    m->host_experts.assign(d.n_layer, {});
    const char* names[3] = {"ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"};
    for (uint32_t il = 0; il < d.n_layer; ++il)
        for (int k = 0; k < 3; ++k) {
            DevTensor& t = m->t["blk." + std::to_string(il) + "." + names[k]];
            itb_model::HostStack& h = m->host_experts[il][k];
            h.nib_per = t.n_out * t.n_in / 2; h.sc_per = t.n_out * t.n_in / 16;
            const size_t nb = h.nib_per * t.n_expert, sb = h.sc_per * t.n_expert;
            if (cudaMallocHost(&h.nib, nb) != cudaSuccess || cudaMallocHost(&h.sc, sb) != cudaSuccess) { itb_fail_msg(c, "offload: out of pinned host memory"); return 1; }
            ITB_CUDA_RET(c, cudaMemcpy(h.nib, t.a, nb, cudaMemcpyDeviceToHost), 1);
            ITB_CUDA_RET(c, cudaMemcpy(h.sc, t.b, sb, cudaMemcpyDeviceToHost), 1);
            h.has_s2 = t.scale2 != nullptr;
            h.s2.assign(t.n_expert, 1.0f);
            if (h.has_s2) ITB_CUDA_RET(c, cudaMemcpy(h.s2.data(), t.scale2, t.n_expert * 4, cudaMemcpyDeviceToHost), 1);
            cudaFree(t.a); cudaFree(t.b); cudaFree(t.scale2);
            m->bytes -= nb + sb;
            t.a = nullptr; t.b = nullptr; t.scale2 = nullptr;
        }
    m->offloaded = true;
    m->finalized = false;
    return finalize(m) ? 0 : 1;
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

// ---------------------------------------------------------------------------------------------------------
// Expert parallelism (src/ops/mod.rs:1024-1048 describes the reference's placement seam). Routed experts are
// sharded by contiguous ranges across ranks, everything else is replicated and every rank decodes its own
// sequences. Per MoE layer the ranks all-gather the quantised rows and their routing, each rank runs its own
// experts over the pairs that name them (the grouped kernels skip experts stored elsewhere), and a sum
// reduce-scatter brings every pair's output row back to the rank that owns the token. Each output row has
// exactly one non-zero contribution, so the reduction is exact and the pick-order combine that follows gives
// the single-GPU bits. NCCL is bound at run time from the library already in the process (no link-time
// dependency: a single-GPU user never loads it).
#include <dlfcn.h>
struct NcclApi {
    typedef struct { char internal[128]; } UniqueId;
    int (*GetUniqueId)(UniqueId*) = nullptr;
    int (*CommInitRank)(void**, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*CommAbort)(void*) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*ReduceScatter)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*Send)(const void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
    static constexpr int Int8 = 0, Int32 = 2, Float32 = 7, Sum = 0;   // ncclDataType_t / ncclRedOp_t values of the public ABI
};
static NcclApi& nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api;
    tried = true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);   // the copy the process already holds
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return api;
#define NCCL_SYM(f) *(void**)&api.f = dlsym(h, "nccl" #f)
    NCCL_SYM(GetUniqueId); NCCL_SYM(CommInitRank); NCCL_SYM(CommDestroy); NCCL_SYM(AllGather); NCCL_SYM(ReduceScatter);
    NCCL_SYM(GroupStart); NCCL_SYM(GroupEnd); NCCL_SYM(GetErrorString); NCCL_SYM(CommAbort); NCCL_SYM(Send); NCCL_SYM(Recv);
#undef NCCL_SYM
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.ReduceScatter && api.GroupStart && api.GroupEnd;
    return api;
}
struct EpState {
    void* comm = nullptr;
    int rank = 0, world = 1;
    int8_t* gxq = nullptr; float* gxs = nullptr; int32_t* gids = nullptr;   // gathered rows of all ranks, rank-major
    float* o_mine = nullptr;                                                // this rank's pairs after the reduce-scatter
    float* gw = nullptr;                                                    // routing weights of the gathered rows [world][n_used] (fused one-token step)
    float* grouter = nullptr;                                               // gathered router logits [world][n_expert] (fused one-token step)
    int* agree_dev = nullptr; int* agree_host = nullptr;                    // one "this rank is ready" flag per rank (ep_agree)
    bool broken = false;                                                    // the communicator was aborted after a failure mid-pass
    // packed all-to-all dispatch/combine of eager many-row passes: this rank's pairs sorted by owner rank (send side), the
    // pairs it received (every one names a local expert), the per-rank counts of all ranks
    int8_t* sxq = nullptr; float* sxs = nullptr; int32_t* sids = nullptr;   // [R*K] rows in owner order
    int8_t* rxq = nullptr; float* rxs = nullptr; int32_t* rids = nullptr;   // received pairs (capacity a2a_cap)
    float* o_back = nullptr;                                                // this rank's pairs' outputs, in owner order
    int32_t* owner = nullptr; int* own_off = nullptr; int* own_list = nullptr;
    int* cnt_dev = nullptr; int* cnt_host = nullptr;                        // [W][W]: cnt[s][d] = pairs rank s sends to rank d
    size_t a2a_cap = 0;
    // the one-token step over peer memory (NVLink loads and stores instead of two small NCCL collectives per layer): one
    // region per rank, the same layout on every rank -- per layer the rows all ranks push here (quantised activation, its
    // scales, router logits), the output rows of this rank's picks that the serving ranks store here, and one flag per
    // (layer, peer) for each direction; peers' regions are opened through CUDA IPC
    bool p2p = false;
    bool p2p_rows = false;                   // the same for the steps of an engine with several sequences (rows form, see ep_p2p_setup)
    unsigned char* region = nullptr; size_t region_bytes = 0;
    unsigned char* peer[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};   // peer[rank] = region
    unsigned char** peer_dev = nullptr;      // the same table on the device
    unsigned* seq = nullptr;                 // device: the step number the flags carry
    size_t g_slot = 0, g_layer = 0, o_layer = 0, off_g = 0, off_o = 0, off_gf = 0, off_of = 0;
};

// ---- packed all-to-all dispatch/combine (expert parallel, eager many-row passes) ----
// The send/receive plan of one rank from the count matrix cnt[s][d] (pairs rank s sends to rank d): offsets into its send
// buffer (owner order) and into its receive buffer (source-rank order), and the total it receives. Plain host arithmetic,
// exported for the CPU tests.
extern "C" int itb_ep_a2a_plan(const int* cnt, int world, int rank, int* send_off, int* recv_off, int* n_recv) {
    if (world < 1 || rank < 0 || rank >= world) return 1;
    int so = 0, ro = 0;
    for (int r = 0; r < world; ++r) {
        if (cnt[rank * world + r] < 0 || cnt[r * world + rank] < 0) return 1;
        send_off[r] = so; so += cnt[rank * world + r];
        recv_off[r] = ro; ro += cnt[r * world + rank];
    }
    send_off[world] = so; recv_off[world] = ro;
    *n_recv = ro;
    return 0;
}
__global__ void k_ep_owner(const int32_t* ids, int n, int per_rank, int32_t* owner) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) owner[i] = ids[i] / per_rank;
}
// Slot s of the owner-sorted order holds pair list[s] of row list[s] / n_used: its quantised row, scales and expert id.
__global__ void k_ep_pack(const int8_t* xq, const float* xs, const int32_t* ids, const int* list, int n_pairs, int n_used, int H,
                          int8_t* sxq, float* sxs, int32_t* sids) {
    const int cpr = H / 16, spr = H / 32;                 // 16-byte chunks and scales per row
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_pairs * cpr) return;
    const int slot = (int)(i / cpr), ch = (int)(i % cpr), pair = list[slot], row = pair / n_used;
    ((uint4*)(sxq + (size_t)slot * H))[ch] = ((const uint4*)(xq + (size_t)row * H))[ch];
    if (ch < spr) sxs[(size_t)slot * spr + ch] = xs[(size_t)row * spr + ch];
    if (ch == 0) sids[slot] = ids[pair];
}
__global__ void k_ep_unsort(const float* o_back, const int* list, int n_pairs, int H, float* o_mine) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_pairs * (H / 4)) return;
    const int slot = (int)(i / (H / 4)), c4 = (int)(i % (H / 4));
    ((float4*)(o_mine + (size_t)list[slot] * H))[c4] = ((const float4*)(o_back + (size_t)slot * H))[c4];
}

// ---- the expert-parallel one-token step over peer memory ----
__global__ void k_ep_tick(unsigned* seq) { if (threadIdx.x == 0 && blockIdx.x == 0) seq[0] += 1; }
// This rank's row of layer il -- quantised activation, scales, router logits -- stored into every rank's region (its own
// included), then that rank's flag for (layer, this rank) set to the step number with system-scope release. A block per
// destination rank. The predecessor produced the row: wait for it (programmatic dependent launch) before reading.
__global__ void __launch_bounds__(256) k_ep_push(const int8_t* xq, const float* xs, const float* router, int H, int E, unsigned char* const* peer,
                                                 size_t off_xq, size_t off_xs, size_t off_router, size_t off_flag, const unsigned* seq) {
    pdl_trigger(); pdl_wait();
    unsigned char* base = peer[blockIdx.x];
    const int nq = H / 16, ns = H / 32 / 4, nr = E / 4;           // 16-byte pieces of the three parts
    for (int i = threadIdx.x; i < nq + ns + nr; i += blockDim.x) {
        if (i < nq) ((uint4*)(base + off_xq))[i] = ((const uint4*)xq)[i];
        else if (i < nq + ns) ((uint4*)(base + off_xs))[i - nq] = ((const uint4*)xs)[i - nq];
        else ((uint4*)(base + off_router))[i - nq - ns] = ((const uint4*)router)[i - nq - ns];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* flag = (unsigned*)(base + off_flag);
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq[0]) : "memory");
    }
}
// After the down projection stored this rank's served picks into their owners' regions: tell every rank so. The stores
// came from the predecessor kernel; its completion (waited for here) made them visible.
__global__ void k_ep_signal(unsigned char* const* peer, size_t off_flag, const unsigned* seq) {
    pdl_trigger(); pdl_wait();
    __threadfence_system();
    unsigned* flag = (unsigned*)(peer[blockIdx.x] + off_flag);
    if (threadIdx.x == 0) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq[0]) : "memory");
}
// k_moe_finish_rows for the one local row, once every rank has signalled (bounded wait): weighted sum of the picks' rows in
// pick order, the sigmoid-gated shared expert, the residual (src/ops/mod.rs:1134-1190). The rows were written by other GPUs:
// read past L1.
__global__ void __launch_bounds__(256) k_ep_finish(float* x, int n, const float* o, const float* wts, int n_used, const float* shared, const float* logit,
                                                   const unsigned* flags, int world, const unsigned* seq, int* err) {
    pdl_trigger(); pdl_wait();
    if (threadIdx.x < world) ep_wait_flag(flags + threadIdx.x, seq[0], err);
    __syncthreads();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = sigmoid_f(logit[0]);
    float v = 0.0f;
    for (int k = 0; k < n_used; ++k) v += wts[k] * __ldcg(o + (size_t)k * n + i);
    v += shared[i] * g;
    x[i] += v;
}

// ---- the same for steps of several sequences per rank (the multi-row kernels) ----
// This rank's rows of layer il -- quantised activations, scales, routing ids -- stored into every rank's region, then that
// rank's flag for (layer, this rank). A block per destination rank.
__global__ void __launch_bounds__(256) k_ep_push_rows(const int8_t* xq, const float* xs, const int32_t* ids, int n_xq16, int n_xs16, int n_ids,
                                                      unsigned char* const* peer, size_t off_xq, size_t off_xs, size_t off_ids, size_t off_flag, const unsigned* seq) {
    unsigned char* base = peer[blockIdx.x];
    for (int i = threadIdx.x; i < n_xq16; i += blockDim.x) ((uint4*)(base + off_xq))[i] = ((const uint4*)xq)[i];
    for (int i = threadIdx.x; i < n_xs16; i += blockDim.x) ((uint4*)(base + off_xs))[i] = ((const uint4*)xs)[i];
    for (int i = threadIdx.x; i < n_ids; i += blockDim.x) ((int32_t*)(base + off_ids))[i] = ids[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* flag = (unsigned*)(base + off_flag);
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq[0]) : "memory");
    }
}
// Every rank's flag of one layer and direction has reached this step's number (bounded waits; *err set if one runs out).
// One warp; the kernels after it read what the peers stored.
__global__ void k_ep_wait(const unsigned* flags, int world, const unsigned* seq, int* err) {
    if ((int)threadIdx.x < world) ep_wait_flag(flags + threadIdx.x, seq[0], err);
}
// The output rows of the pairs this rank served (the pairs of all ranks' rows that name one of its experts), each stored
// into its OWNER's region at the pair's place; rows of pairs served elsewhere are never read. A block per pair.
__global__ void __launch_bounds__(256) k_ep_scatter_rows(const float* o_all, const int32_t* gids, int pairs_per_rank, int e_per, int rank, int H,
                                                         unsigned char* const* peer, size_t off_o) {
    const int pr = blockIdx.x;
    if (gids[pr] / e_per != rank) return;
    const int src = pr / pairs_per_rank, j = pr % pairs_per_rank;
    float4* dst = (float4*)(peer[src] + off_o) + (size_t)j * (H / 4);
    const float4* from = (const float4*)(o_all + (size_t)pr * H);
    for (int i = threadIdx.x; i < H / 4; i += blockDim.x) dst[i] = from[i];
}

// Expert tiering: the routed experts live in pinned host memory (itb_model_offload_experts); `capacity` (layer, expert)
// slots of gate+up+down live in HBM pools, chosen by GCLOCK. Per MoE layer of a pass the routing ids come to the host,
// missing experts are copied into victims' slots on the engine's stream, the id -> slot table is refreshed, and the
// grouped expert kernels read through the table.
struct TierState {
    GClock* g = nullptr;
    size_t capacity = 0;
    uint8_t* pool_nib[3] = {nullptr, nullptr, nullptr};
    uint8_t* pool_sc[3] = {nullptr, nullptr, nullptr};
    float* pool_s2[3] = {nullptr, nullptr, nullptr};
    int* slot_map = nullptr;                 // device [n_layer][n_expert]
    int* slot_map_host = nullptr;            // pinned mirror
    int32_t* ids_host = nullptr;             // pinned [R * K]
    float* s2_stage = nullptr;               // pinned [capacity * 3]: second scales in flight to the pools
    size_t s2_at = 0;
    uint64_t bytes_moved = 0;
    std::vector<char> dirty;                 // slot_map rows to refresh
    // the prefetch hint (src/ops/mod.rs:915-924), applied inside the engine: while layer il's experts run, the experts layer
    // il + 1's router would pick on THIS layer's router input are copied in on a second stream
    int prefetch_k = 0;                      // guesses per row (0: off)
    cudaStream_t stream2 = nullptr; cudaEvent_t ev_fetch = nullptr; bool fetch_pending = false;
    int32_t* guess_dev = nullptr; int32_t* guess_host = nullptr; float* guess_w = nullptr; float* guess_logits = nullptr;
    float* s2_guess = nullptr; size_t s2_guess_cap = 0;     // pinned staging of the guesses' second scales (their copies outlive the call)
    std::vector<char> guessed;               // per slot: filled by a guess and not used yet
    uint64_t fetched = 0, prefetch_reads = 0, prefetch_used = 0, picks_wait_us = 0, lookups = 0, host_reads = 0;
};

struct itb_engine {
    itb_model* m = nullptr;
    EpState* ep = nullptr;   // set in expert-parallel engines
    TierState* tier = nullptr;   // set in expert-tiered engines
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
    float* scores = nullptr; size_t scores_cap = 0;    // exact attention: [rows][n_head][n_ctx] scores (grown on demand)
    float *router = nullptr, *shlogit = nullptr, *sg = nullptr, *su = nullptr, *h = nullptr, *logits = nullptr;
    int8_t* xq = nullptr; float* xs = nullptr;
    int32_t* route_ids = nullptr; float* route_w = nullptr;  // [n_layer][B][n_used]
    int32_t* history = nullptr; int* step_counter = nullptr; uint32_t history_cap = 0;
    int* err = nullptr; float* arg_v = nullptr; int* arg_i = nullptr;
    int8_t *aq = nullptr, *hq = nullptr, *sq = nullptr; float *as = nullptr, *hs = nullptr, *ss = nullptr;  // producer-quantised activations
    float* gdn_scratch = nullptr; size_t gdn_scratch_cap = 0;     // chunk-parallel delta rule: W, Qg, Kd, U, P of every (chunk, value head) of a pass
    float *h_all = nullptr, *o_all = nullptr, *shd = nullptr, *qkvc2 = nullptr; int *pair_off = nullptr, *pair_list = nullptr;  // grouped experts (multi-row path)
    int32_t* prompt = nullptr; size_t prompt_cap = 0;
    int n_split = 1, n_split_rows = 4;
    uint32_t R = 0;                                   // rows the multi-row pass can hold (>= B)
    uint32_t last_n_tok = 1;                          // tokens per sequence in the most recent pass
    float *xn = nullptr, *qh = nullptr, *kh = nullptr, *vh = nullptr, *gb = nullptr, *core = nullptr, *xlast = nullptr;
    cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr;
    // the one-kernel decode step (itb_mega.cuh): stage table, launch shape, parameters; mega < 0: not yet decided
    int mega = -1; MStage* mega_stages = nullptr; MegaParams mp{}; size_t mega_smem = 0; int mega_grid = 0;
    unsigned* mega_sync = nullptr; float* mega_core = nullptr; float* mega_part = nullptr; float* mega_argv = nullptr; int* mega_argi = nullptr;
    std::string mega_why;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_ms = 0.0f;
    uint64_t launches_per_step = 0;
    std::vector<uint32_t> host_pos;
    std::vector<void*> allocs;
};

// Per-launch CUDA-event timing of one eagerly launched step, grouped by kernel class.
enum KClass { KC_EMBED, KC_GDN_IN, KC_GDN_CORE, KC_OUT_PROJ, KC_ATTN_IN, KC_ATTN_PREP, KC_ATTN, KC_FFN_IN, KC_MOE_GLU, KC_MOE_DOWN,
              KC_LM_HEAD, KC_ARGMAX, KC_COUNT };
static const char* const KC_NAMES[KC_COUNT] = {"k_embed", "k_in_proj[gdn]", "k_gdn_core", "k_out_proj", "k_in_proj[attn]", "k_attn_prep",
                                               "k_attn_partial+combine", "k_in_proj[ffn]", "k_moe_glu", "k_moe_down",
                                               "k_in_proj[lm_head]", "k_argmax_advance"};
struct StepProf {
    std::vector<cudaEvent_t> ev;
    std::vector<int> cls;
    std::vector<uint64_t> bytes;
    void mark(int c, uint64_t b, cudaStream_t st) {
        cudaEvent_t e; cudaEventCreate(&e); cudaEventRecord(e, st);
        ev.push_back(e); cls.push_back(c); bytes.push_back(b);
    }
};
// Keeps the stream busy for a bounded time so a whole step can be queued behind it and then run back to back.
__global__ void k_hold(long long cycles) {
    long long t0 = clock64();
    while (clock64() - t0 < cycles) {}
}

template <class T>
static bool dalloc(itb_engine* e, T** p, size_t count) {
    if (cudaMalloc((void**)p, std::max<size_t>(count, 1) * sizeof(T)) != cudaSuccess) return itb_fail_msg(e->c, "engine: out of device memory");
    cudaMemsetAsync(*p, 0, std::max<size_t>(count, 1) * sizeof(T), e->c->stream);
    e->allocs.push_back(*p);
    return true;
}

static void set_smem(const void* fn, size_t bytes) {
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) fprintf(stderr, "[itb] cudaFuncSetAttribute(%zu bytes) failed: %s\n", bytes, cudaGetErrorString(e));
}

// Launch with (pdl) or without the programmatic-serialization attribute: with it the kernel may be scheduled
// while its predecessor in the stream still runs and orders itself by griddepcontrol.wait (pdl_wait()).
template <class... KA, class... A>
static void launch_k(bool pdl, void (*k)(KA...), dim3 g, dim3 b, size_t sm, cudaStream_t st, A&&... a) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = g; cfg.blockDim = b; cfg.dynamicSmemBytes = sm; cfg.stream = st;
    cudaLaunchAttribute at{};
    at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &at; cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t err = cudaLaunchKernelEx(&cfg, k, KA(std::forward<A>(a))...);
    if (err != cudaSuccess) fprintf(stderr, "[itb] kernel launch failed: %s\n", cudaGetErrorString(err));
}

constexpr size_t SMEM_BUDGET = 200 * 1024;   // dynamic shared memory the row-streaming kernels are allowed (set_smem below)

// Attention in the CPU path's order (itb_attn_exact.cuh) for `rows` query rows: scores, then softmax + weighted values + gate +
// Q8_0 quantisation into e->aq / e->as. Needs a row stride of whole 16-byte spans; the scores buffer holds n_ctx per (row, head).
static bool exact_attention_ok(const itb_engine* e) { return e->c->exact && (e->m->d.head_dim * e->m->d.n_head_kv) % 8 == 0 && e->m->d.n_head / e->m->d.n_head_kv <= 8; }
static void drop_graph(itb_engine* e);
static bool ensure_scores(itb_engine* e, size_t rows) {
    const size_t need = rows * e->m->d.n_head * e->n_ctx;
    if (e->scores_cap >= need) return true;
    cudaStreamSynchronize(e->c->stream);
    drop_graph(e);        // a captured step holds the old pointer
    cudaFree(e->scores); e->scores = nullptr; e->scores_cap = 0;
    if (cudaMalloc(&e->scores, need * 4) != cudaSuccess) { cudaGetLastError(); return itb_fail_msg(e->c, "engine: out of device memory for the attention scores"); }
    e->scores_cap = need;
    return true;
}
static void enqueue_exact_attention(itb_engine* e, cudaStream_t st, bool pdl, const uint16_t* kslab, const uint16_t* vslab, size_t slab_stride,
                                    int rows, int rows_per_seq, int n_pos_max) {
    const itb_model_dims& d = e->m->d;
    const int hd = d.head_dim, group = d.n_head / d.n_head_kv, kvd = hd * d.n_head_kv;
    static bool attr = false;
    if (!attr) { set_smem((const void*)k_attn_out_exact, 200 * 1024); attr = true; }
    AxScores a{};
    a.q = e->qn; a.kslab = kslab; a.slab_stride = slab_stride; a.rows_per_seq = rows_per_seq; a.n_pos_dev = e->npos; a.kv_dim = kvd; a.hd = hd;
    a.n_head = d.n_head; a.n_head_kv = d.n_head_kv; a.scale = 1.0f / sqrtf((float)hd); a.bf16 = e->c->kv_bf16; a.scores = e->scores; a.s_stride = (int)e->n_ctx;
    launch_k(pdl, k_attn_scores_exact, dim3((n_pos_max + AX_TP - 1) / AX_TP, d.n_head_kv, rows), dim3(AX_TP * group), attn_scores_exact_smem(hd, group), st, a);
    AxOut o{};
    if (rows >= 8) {
        // many rows: the softmax once per (row, head), in place, instead of once per block of the weighted-value kernel
        AxSoft sm{e->scores, (int)e->n_ctx, e->npos, 0, 0, (int)d.n_head};
        static bool attr2 = false;
        if (!attr2) { set_smem((const void*)k_attn_softmax_exact, 200 * 1024); attr2 = true; }
        launch_k(pdl, k_attn_softmax_exact, dim3(d.n_head, rows), dim3(256), (size_t)((n_pos_max + 3) & ~3) * 4, st, sm);
        o.weights_ready = 1;
    }
    o.scores = e->scores; o.s_stride = (int)e->n_ctx; o.vslab = vslab; o.slab_stride = slab_stride; o.rows_per_seq = rows_per_seq; o.n_pos_dev = e->npos;
    o.kv_dim = kvd; o.hd = hd; o.n_head = d.n_head; o.n_head_kv = d.n_head_kv; o.bf16 = e->c->kv_bf16; o.gate = e->gate; o.out_q = e->aq; o.out_s = e->as;
    launch_k(pdl, k_attn_out_exact, dim3(hd / 32, d.n_head, rows), dim3(256), attn_out_exact_smem(n_pos_max), st, o);
}

// One decode step for all B sequences, enqueued on `st`.
static void enqueue_step(itb_engine* e, cudaStream_t st, StepProf* prof = nullptr) {
    itb_model* m = e->m; itb_ctx* c = e->c;
    const itb_model_dims& d = m->d;
    const int B = e->B, H = d.n_embd, sms = c->sm_count;
    const int key_dim = d.ssm_d_state * d.ssm_n_group, vd = d.ssm_d_inner, cd = 2 * key_dim + vd;
    const int qd = d.head_dim * d.n_head, kvd = d.head_dim * d.n_head_kv;
    const int TPB = NWG * 32;
    uint64_t launches = 0;
    int tl = 0;   // phase-timeline slots: launch ordinals of the structured kernels of this step
    // overlap each kernel's launch and weight prefetch with its predecessor's tail (off while profiling per kernel)
    static const bool pdl_env = !(getenv("ITB_PDL") && atoi(getenv("ITB_PDL")) == 0);
    const bool pdl = pdl_env && !prof;
    auto q8b = [](uint64_t a, uint64_t b) { return a * b / 32 * 34; };
    auto f4b = [](uint64_t a, uint64_t b) { return a * b / 64 * 36; };
#define MARK(cls, by) do { launches++; if (prof) prof->mark((cls), (uint64_t)(by), st); } while (0)
    // grid for a row-streaming kernel: about two rows per warp and pass, one block of 16 warps per SM
    auto grid_rows = [&](int rows) { return std::max(1, std::min(sms, (rows + 2 * NWG - 1) / (2 * NWG))); };
    // rows a warp folds together: what it owns, rounded up to whole passes, at most 32
    const int pass_in = 2 * (32 >> lanes_shift(H / 32));
    auto launch_in = [&](InProj& p, int rows, int gx) {
        int per_warp = (rows + gx * NWG - 1) / (gx * NWG) + 1;
        p.br = std::min(std::max(32 / pass_in, 1) * pass_in, (per_warp + pass_in - 1) / pass_in * pass_in);
        // the warps' term matrices must fit the block's shared memory (wide rows: fewer rows folded together)
        const int cap = (int)(((SMEM_BUDGET - 256 - (size_t)H * 5 - (size_t)(H / 32) * 4 - (c->exact ? 32 * 33 * 4 : 0) - 64) / (NWG * 4) - CONV_CAP * 8) / (H / 32 + 1));
        p.br = std::max(pass_in, std::min(p.br, cap / pass_in * pass_in));
        p.f32_ring = 0; p.err = e->err;
        if (c->exact && p.nf) {
            // serial-k F32 rows: 32 to a warp (a lane per row) through the block's ring, when every unit gets a block of its own
            // and the ring fits; otherwise a row per warp, staged in the warp's term scratch (make it hold the whole row)
            int units = 0;
            for (int m = 0; m < p.nf; ++m) units += (p.f[m].n_out + 31) / 32;
            bool kmajor = true;
            for (int m = 0; m < p.nf; ++m) kmajor = kmajor && p.f[m].wt;
            if (kmajor && units <= gx && NWG >= 4 && H % F32S_K == 0 && H / F32S_K >= F32S_STAGES && in_proj_smem(H, 1, p.br, 1) <= SMEM_BUDGET) p.f32_ring = units;
            else {
                const int want = (H + H / 32) / (H / 32 + 1) + 1;
                p.br = std::max(p.br, std::min((want + pass_in - 1) / pass_in * pass_in, cap / pass_in * pass_in));
            }
        }
        p.tl_slot = tl++;
        launch_k(pdl, k_in_proj, dim3(gx, B), TPB, in_proj_smem(H, c->exact, p.br, p.f32_ring), st, p);
    };
    auto launch_out = [&](OutProj& o, int n_in) {
        int gx = std::max(1, std::min(sms, H / NWG)), pass = 32 >> lanes_shift(n_in / 32);
        int per_warp = (H + gx * NWG - 1) / (gx * NWG) + 1;
        o.br = std::min(std::max(32 / pass, 1) * pass, (per_warp + pass - 1) / pass * pass);
        const int cap = (int)((SMEM_BUDGET - (size_t)n_in - (size_t)(n_in / 32) * 4 - 64) / (NWG * 4) / (n_in / 32 + 1));
        o.br = std::max(pass, std::min(o.br, cap / pass * pass));
        o.tl_slot = tl++;
        launch_k(pdl, k_out_proj, dim3(gx, B), TPB, out_proj_smem(n_in, o.br), st, o);
    };
    // L2 hints: each kernel names what the kernels after it will stream. Off unless ITB_L2_HINT=1: measured on the 35B shape the
    // step does not get faster with them (2.99 ms against 2.94 ms without, hints issued as each block finishes its own rows; 3.17 ms
    // with the hints issued at the start of each kernel, where they queue ahead of the kernel's own loads) -- the kernels wait on
    // their dependent stages, not on the latency of the weight stream.
    static const bool hints_on = getenv("ITB_L2_HINT") && atoi(getenv("ITB_L2_HINT")) == 1;
    const bool hints = hints_on && !prof;
    auto hint_add = [&](L2Hint& h, const void* ptr, size_t bytes) {
        if (!hints || !ptr || !bytes) return;
        for (int i = 0; i < 8; ++i)
            if (!h.p[i]) { h.p[i] = ptr; h.n[i] = (unsigned)std::min<size_t>(bytes, 64u << 20); return; }
    };
    auto hint_q8 = [&](L2Hint& h, const DevQ8& w) {
        hint_add(h, w.q, (size_t)w.n_in * w.n_out); hint_add(h, w.s, (size_t)(w.n_in / 32) * w.n_out * 2);
    };
    auto hint_f32 = [&](L2Hint& h, const DevF32& w) {
        if (c->exact && w.wt) hint_add(h, w.wt, (size_t)((w.n_out + 31) / 32) * 32 * w.n_in * 4);
        else hint_add(h, w.w, (size_t)w.n_in * w.n_out * 4);
    };
    // the input projections of layer `il` (what its first kernel streams)
    auto hint_layer_in = [&](L2Hint& h, uint32_t il) {
        if (il >= d.n_layer) return;
        const DevLayer& L = m->layers[il];
        if (L.recurrent) { hint_q8(h, L.wqkv); hint_q8(h, L.wgate); hint_f32(h, L.ssm_alpha); hint_f32(h, L.ssm_beta); }
        else { hint_q8(h, L.wq); hint_q8(h, L.wk); hint_q8(h, L.wv); }
    };
    static bool attrs_set = false;
    if (!attrs_set) {
        set_smem((const void*)k_in_proj, 200 * 1024); set_smem((const void*)k_out_proj, 200 * 1024);
        set_smem((const void*)k_moe_glu, 100 * 1024);
        set_smem((const void*)k_moe_down<1>, 100 * 1024); set_smem((const void*)k_moe_down<2>, 100 * 1024);
        set_smem((const void*)k_moe_down<4>, 100 * 1024); set_smem((const void*)k_moe_down<8>, 100 * 1024);
        set_smem((const void*)k_moe_down<1, true>, 100 * 1024); set_smem((const void*)k_moe_down<2, true>, 100 * 1024);
        set_smem((const void*)k_moe_down<4, true>, 100 * 1024); set_smem((const void*)k_moe_down<8, true>, 100 * 1024);
        set_smem((const void*)k_gdn_core<128>, 100 * 1024); set_smem((const void*)k_gdn_core<64>, 100 * 1024);
        attrs_set = true;
    }
    if (prof) prof->mark(-1, 0, st);
    const bool p2p = e->ep && e->ep->p2p;
    if (p2p) { k_ep_tick<<<1, 32, 0, st>>>(e->ep->seq); launches++; }    // the step number the peers' flags will carry
    launch_k(pdl, k_embed, B, 256, 0, st, m->tok_embd.w, H, e->tokens, e->x); MARK(KC_EMBED, (uint64_t)B * H * 8);
    for (uint32_t il = 0; il < d.n_layer; ++il) {
        const DevLayer& L = m->layers[il];
        if (L.recurrent) {
            int rs = e->slot_of[il];
            size_t state_stride = (size_t)d.ssm_dt_rank * d.ssm_d_state * d.ssm_d_state;
            InProj p{};
            p.x = e->x; p.x_stride = H; p.norm_w = L.attn_norm; p.eps = d.rms_eps; p.n_embd = H;
            p.nq = 2; p.q[0] = L.wqkv; p.qout[0] = e->qkvc; p.qstride[0] = cd; p.q[1] = L.wgate; p.qout[1] = e->z; p.qstride[1] = vd;
            p.nf = 2; p.f[0] = L.ssm_alpha; p.fout[0] = e->alpha; p.fstride[0] = d.ssm_dt_rank;
            p.f[1] = L.ssm_beta; p.fout[1] = e->beta; p.fstride[1] = d.ssm_dt_rank;
            p.conv_w = L.conv1d; p.conv_kernel = d.ssm_d_conv; p.conv_state_stride = (size_t)cd * (d.ssm_d_conv - 1);
            p.conv_state = e->conv_state + (size_t)rs * B * p.conv_state_stride;
            p.exact = c->exact;
            hint_q8(p.hint, L.ssm_out);
            hint_add(p.hint, e->ssm_state + (size_t)rs * B * state_stride, std::min<size_t>((size_t)B, 4) * state_stride * 4);
            launch_in(p, cd + vd, grid_rows(cd + vd));
            MARK(KC_GDN_IN, q8b(H, cd) + q8b(H, vd) + 2ull * H * d.ssm_dt_rank * 4 + (uint64_t)cd * d.ssm_d_conv * 4 +
                                (uint64_t)B * (2ull * cd * (d.ssm_d_conv - 1) * 4 + (H + cd + vd) * 4));
            GdnCore g{};
            g.conv = e->qkvc; g.conv_stride = cd; g.z = e->z; g.alpha = e->alpha; g.beta = e->beta;
            g.ssm_a = L.ssm_a; g.dt_bias = L.dt_bias; g.ssm_norm = L.ssm_norm;
            g.state_stride = state_stride; g.state = e->ssm_state + (size_t)rs * B * state_stride;
            g.out_q = e->aq; g.out_s = e->as; g.sk = d.ssm_d_state; g.sv = d.ssm_d_state; g.n_k = d.ssm_n_group; g.n_v = d.ssm_dt_rank; g.eps = d.rms_eps;
            g.tl_slot = tl++;
            size_t smem_g = (size_t)(g.sv * (g.sk + 1) + 2 * g.sk + g.sv) * 4;
            if (d.ssm_d_state == 128) launch_k(pdl, k_gdn_core<128>, dim3(d.ssm_dt_rank, B), 256, smem_g, st, g);
            else launch_k(pdl, k_gdn_core<64>, dim3(d.ssm_dt_rank, B), 256, smem_g, st, g);
            MARK(KC_GDN_CORE, (uint64_t)B * (2ull * g.state_stride * 4 + (cd + 2ull * vd) * 4));
            OutProj o{e->aq, e->as, vd, L.ssm_out, e->x, H};
            hint_q8(o.hint, L.shared_gate); hint_q8(o.hint, L.shared_up); hint_f32(o.hint, L.gate_inp); hint_f32(o.hint, L.shared_gate_inp);
            launch_out(o, vd);
            MARK(KC_OUT_PROJ, q8b(vd, H) + (uint64_t)B * (vd + 2ull * H) * 4);
        } else {
            int as = e->slot_of[il];
            InProj p{};
            p.x = e->x; p.x_stride = H; p.norm_w = L.attn_norm; p.eps = d.rms_eps; p.n_embd = H;
            p.nq = 3; p.q[0] = L.wq; p.qout[0] = e->qg; p.qstride[0] = 2 * qd; p.q[1] = L.wk; p.qout[1] = e->kbuf; p.qstride[1] = kvd;
            p.q[2] = L.wv; p.qout[2] = e->vbuf; p.qstride[2] = kvd;
            p.exact = c->exact;
            hint_q8(p.hint, L.wo);
            launch_in(p, 2 * qd + 2 * kvd, grid_rows(2 * qd + 2 * kvd));
            MARK(KC_ATTN_IN, q8b(H, 2 * qd) + 2 * q8b(H, kvd) + (uint64_t)B * (H + 2ull * qd + 2ull * kvd) * 4);
            AttnPrep a{};
            a.qg = e->qg; a.k = e->kbuf; a.v = e->vbuf; a.q_norm = L.q_norm; a.k_norm = L.k_norm; a.q_out = e->qn; a.g_out = e->gate;
            a.slab_stride = (size_t)e->n_ctx * kvd;
            a.kslab = e->kslab + (size_t)as * B * a.slab_stride; a.vslab = e->vslab + (size_t)as * B * a.slab_stride;
            a.pos = e->pos; a.npos_out = e->npos; a.hd = d.head_dim; a.n_head = d.n_head; a.n_head_kv = d.n_head_kv; a.n_rot = d.n_rot;
            a.theta = d.rope_theta; a.eps = d.rms_eps; a.bf16 = c->kv_bf16;
            a.tl_slot = tl++;
            launch_k(pdl, k_attn_prep, dim3(d.n_head + 2 * d.n_head_kv, B), d.head_dim, d.head_dim * 4, st, a);
            MARK(KC_ATTN_PREP, (uint64_t)B * (4ull * qd + 3ull * kvd) * 4);
            if (exact_attention_ok(e) && e->scores) {
                // exact mode: the CPU path's own order. The step is replayed from a graph, so the grids cover the whole context and
                // blocks past the sequence's length leave at once.
                enqueue_exact_attention(e, st, pdl, a.kslab, a.vslab, a.slab_stride, B, 1, (int)e->n_ctx);
                MARK(KC_ATTN, 2ull * kvd * 2 * (e->host_pos[0] + 1) + 3ull * qd * 4); MARK(KC_ATTN, 0);
            } else {
            // split-K partials, one launch per sequence (own slab, own position), then one combine for all
            const float scale = 1.0f / sqrtf((float)d.head_dim);
            const int nwa = 8;
            const size_t smem_a = (size_t)nwa * 8 * 2 * 4 + (size_t)nwa * 8 * d.head_dim * 4;
            for (int b = 0; b < B; ++b) {
                size_t po = (size_t)b * d.n_head * e->n_split;
                dim3 grid(d.n_head_kv, 1, e->n_split);
#define ATT_CASE(HD)                                                                                                             \
    case HD:                                                                                                                      \
        set_smem((const void*)k_attn_partial<HD, 8>, smem_a);                                                                     \
        launch_k(pdl, k_attn_partial<HD, 8>, grid, nwa * 32, smem_a, st, e->qn + (size_t)b * qd, a.kslab + (size_t)b * a.slab_stride,        \
            a.vslab + (size_t)b * a.slab_stride, kvd, 0, 1, d.n_head, d.n_head_kv, scale, c->kv_bf16, e->npos + b,                 \
            e->part_acc + po * d.head_dim, e->part_ml + po * 2, 0, (size_t)0);                                                    \
        break;
                switch (d.head_dim) { ATT_CASE(64) ATT_CASE(128) ATT_CASE(256) }
#undef ATT_CASE
                MARK(KC_ATTN, 2ull * kvd * 2 * (e->host_pos[b] + 1) + 3ull * qd * 4);
            }
            launch_k(pdl, k_attn_combine_q, B * d.n_head, d.head_dim, 0, st, e->part_acc, e->part_ml, e->n_split, d.head_dim, e->gate, e->npos,
                                                                  d.n_head, e->aq, e->as);
            MARK(KC_ATTN, 0);
            }
            OutProj o{e->aq, e->as, qd, L.wo, e->x, H};
            hint_q8(o.hint, L.shared_gate); hint_q8(o.hint, L.shared_up); hint_f32(o.hint, L.gate_inp); hint_f32(o.hint, L.shared_gate_inp);
            launch_out(o, qd);
            MARK(KC_OUT_PROJ, q8b(qd, H) + (uint64_t)B * (qd + 2ull * H) * 4);
        }
        // routed FFN
        InProj f{};
        f.x = e->x; f.x_stride = H; f.norm_w = L.ffn_norm; f.eps = d.rms_eps; f.n_embd = H;
        f.nq = 2; f.q[0] = L.shared_gate; f.qout[0] = e->sg; f.qstride[0] = d.shared_ff; f.q[1] = L.shared_up; f.qout[1] = e->su; f.qstride[1] = d.shared_ff;
        f.nf = 2; f.f[0] = L.gate_inp; f.fout[0] = e->router; f.fstride[0] = d.n_expert;
        f.f[1] = L.shared_gate_inp; f.fout[1] = e->shlogit; f.fstride[1] = 1;
        f.xq_out = e->xq; f.xs_out = e->xs; f.exact = c->exact;
        hint_q8(f.hint, L.shared_down);
        if (il + 1 < d.n_layer) hint_layer_in(f.hint, il + 1); else hint_add(f.hint, m->output.q, std::min((size_t)48 << 20, (size_t)m->output.n_in * m->output.n_out));
        int gxf = c->exact ? sms : std::max(grid_rows(2 * d.shared_ff), std::min(2 * sms, (int)(d.n_expert + 1 + NWG - 1) / NWG));   // serial-k F32 rows: one per SM
        launch_in(f, 2 * d.shared_ff, gxf);
        MARK(KC_FFN_IN, (uint64_t)H * d.n_expert * 4 + 2 * q8b(H, d.shared_ff) + (uint64_t)H * 4 + (uint64_t)B * (2ull * H + d.n_expert + 2ull * d.shared_ff) * 4);
        const int W = e->ep ? e->ep->world : 1, RW = B * W;   // rows the expert kernels see: ours, or every rank's (expert parallel)
        MoeGlu g{};
        g.router = e->router; g.n_expert = d.n_expert; g.n_used = d.n_expert_used; g.xq = e->xq; g.xs = e->xs; g.n_embd = H;
        g.gate = L.gate; g.up = L.up; g.sg = e->sg; g.su = e->su; g.sff = d.shared_ff;
        g.hq = e->hq; g.hs = e->hs; g.sq = e->sq; g.ss = e->ss;
        g.ids_out = e->route_ids + (size_t)il * e->R * d.n_expert_used; g.w_out = e->route_w + (size_t)il * e->R * d.n_expert_used;
        g.shared_row = -1;
        if (hints && !L.down.slot_map) { g.down_nib = L.down.nib; g.down_sc = L.down.sc; g.down_bytes = (size_t)L.down.n_out * (L.down.n_in / 2); }
        if (p2p) {
            // every rank's quantised row and router logits (B is 1 here), pushed by each rank into every rank's region over NVLink;
            // k_moe_glu's blocks for row r wait for rank r's flag. No NCCL call, no zero-filled buffer.
            EpState* q = e->ep;
            const size_t base = q->off_g + (size_t)il * q->g_layer, o_xq = base, o_xs = base + (size_t)W * H, o_r = o_xs + (size_t)W * (H / 32) * 4;
            launch_k(pdl, k_ep_push, dim3(W), dim3(256), 0, st, (const int8_t*)e->xq, (const float*)e->xs, (const float*)e->router, (int)H, (int)d.n_expert,
                     (unsigned char* const*)q->peer_dev, o_xq + (size_t)q->rank * H, o_xs + (size_t)q->rank * (H / 32) * 4, o_r + (size_t)q->rank * d.n_expert * 4,
                     q->off_gf + ((size_t)il * 8 + q->rank) * 4, (const unsigned*)q->seq);
            launches++;
            g.router = (const float*)(q->region + o_r); g.xq = (const int8_t*)(q->region + o_xq); g.xs = (const float*)(q->region + o_xs);
            g.shared_row = q->rank; g.ids_out = q->gids; g.w_out = q->gw;
            g.wait_flags = (const unsigned*)(q->region + q->off_gf + (size_t)il * 8 * 4); g.wait_seq = q->seq; g.err = e->err;
        }
        if (e->ep && !p2p) {
            // every rank's quantised row and router logits (B is 1 here): the kernels below then serve the picks that name a local expert
            NcclApi& nc = nccl_api();
            nc.GroupStart();
            nc.AllGather(e->xq, e->ep->gxq, (size_t)H, NcclApi::Int8, e->ep->comm, st);
            nc.AllGather(e->xs, e->ep->gxs, (size_t)(H / 32), NcclApi::Float32, e->ep->comm, st);
            nc.AllGather(e->router, e->ep->grouter, (size_t)d.n_expert, NcclApi::Float32, e->ep->comm, st);
            nc.GroupEnd();
            launches++;
            cudaMemsetAsync(e->o_all, 0, (size_t)W * d.n_expert_used * H * sizeof(float), st);
            g.router = e->ep->grouter; g.xq = e->ep->gxq; g.xs = e->ep->gxs; g.shared_row = e->ep->rank;
            g.ids_out = e->ep->gids; g.w_out = e->ep->gw;
        }
        g.tl_slot = tl++;
        launch_k(pdl, k_moe_glu, dim3(d.n_expert_used * (d.expert_ff / 32) + d.shared_ff / 32, RW), TPB, moe_glu_smem(d.n_expert, H), st, g);
        MARK(KC_MOE_GLU, (uint64_t)B * (2ull * d.n_expert_used * f4b(H, d.expert_ff) + (uint64_t)d.n_expert_used * d.expert_ff * 4));
        MoeDown w{};
        w.hq = e->hq; w.hs = e->hs; w.n_used = d.n_expert_used; w.ff = d.expert_ff; w.ids = g.ids_out; w.wts = g.w_out; w.down = L.down;
        w.sq = e->sq; w.ss = e->ss; w.sff = d.shared_ff; w.shared_down = L.shared_down; w.logit = e->shlogit; w.x = e->x; w.x_stride = H;
        if (e->ep) { w.o_pairs = e->o_all; w.own_row = e->ep->rank; w.shd = e->shd; }
        if (p2p) for (int r = 0; r < W; ++r) w.o_rows[r] = (float*)(e->ep->peer[r] + e->ep->off_o + (size_t)il * e->ep->o_layer);
        {
            int slots = 32 >> lanes_shift(d.expert_ff / 32), need = ((int)d.n_expert_used + slots - 1) / slots;
            int rp = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
            dim3 grid(std::max(1, std::min(sms, (H + NWG - 1) / NWG)), RW);
            w.tl_slot = tl++;
            size_t smem_d = moe_down_smem(d.n_expert_used, d.expert_ff, d.shared_ff, rp);
            if (e->ep) {
                if (rp == 1) launch_k(pdl, k_moe_down<1, true>, grid, TPB, smem_d, st, w);
                else if (rp == 2) launch_k(pdl, k_moe_down<2, true>, grid, TPB, smem_d, st, w);
                else if (rp == 4) launch_k(pdl, k_moe_down<4, true>, grid, TPB, smem_d, st, w);
                else launch_k(pdl, k_moe_down<8, true>, grid, TPB, smem_d, st, w);
            } else if (rp == 1) launch_k(pdl, k_moe_down<1>, grid, TPB, smem_d, st, w);
            else if (rp == 2) launch_k(pdl, k_moe_down<2>, grid, TPB, smem_d, st, w);
            else if (rp == 4) launch_k(pdl, k_moe_down<4>, grid, TPB, smem_d, st, w);
            else launch_k(pdl, k_moe_down<8>, grid, TPB, smem_d, st, w);
        }
        if (p2p) {
            // the served picks' rows were stored straight into their owners' regions: tell every rank, then combine this rank's
            // own row once every rank has told it (pick order, gated shared expert, residual: as k_moe_down does on one GPU)
            EpState* q = e->ep;
            launch_k(pdl, k_ep_signal, dim3(W), dim3(32), 0, st, (unsigned char* const*)q->peer_dev, q->off_of + ((size_t)il * 8 + q->rank) * 4, (const unsigned*)q->seq);
            launch_k(pdl, k_ep_finish, dim3((H + 255) / 256), dim3(256), 0, st, e->x, (int)H, (const float*)(q->region + q->off_o + (size_t)il * q->o_layer),
                     (const float*)(q->gw + (size_t)q->rank * d.n_expert_used), (int)d.n_expert_used, (const float*)e->shd, (const float*)e->shlogit,
                     (const unsigned*)(q->region + q->off_of + (size_t)il * 8 * 4), W, (const unsigned*)q->seq, e->err);
            launches += 2;
            cudaMemcpyAsync(e->route_ids + (size_t)il * e->R * d.n_expert_used, q->gids + (size_t)q->rank * d.n_expert_used, d.n_expert_used * 4, cudaMemcpyDeviceToDevice, st);
            cudaMemcpyAsync(e->route_w + (size_t)il * e->R * d.n_expert_used, q->gw + (size_t)q->rank * d.n_expert_used, d.n_expert_used * 4, cudaMemcpyDeviceToDevice, st);
        } else if (e->ep) {
            // each pick's output row comes home (exactly one rank wrote it: an exact sum), then the pick-order combine, the
            // gated shared expert and the residual add, as k_moe_down does them on one GPU
            const size_t KH = (size_t)d.n_expert_used * H;
            nccl_api().ReduceScatter(e->o_all, e->ep->o_mine, KH, NcclApi::Float32, NcclApi::Sum, e->ep->comm, st);
            k_moe_finish_rows<<<(unsigned)((H + 255) / 256), 256, 0, st>>>(e->x, H, e->ep->o_mine, e->ep->gw + (size_t)e->ep->rank * d.n_expert_used,
                                                                          d.n_expert_used, e->shd, e->shlogit, (size_t)H);
            launches += 2;
            // the routing this rank's token got, where read_routes looks for it
            cudaMemcpyAsync(e->route_ids + (size_t)il * e->R * d.n_expert_used, e->ep->gids + (size_t)e->ep->rank * d.n_expert_used,
                            d.n_expert_used * 4, cudaMemcpyDeviceToDevice, st);
            cudaMemcpyAsync(e->route_w + (size_t)il * e->R * d.n_expert_used, e->ep->gw + (size_t)e->ep->rank * d.n_expert_used,
                            d.n_expert_used * 4, cudaMemcpyDeviceToDevice, st);
        }
        MARK(KC_MOE_DOWN, (uint64_t)B * d.n_expert_used * f4b(d.expert_ff, H) + q8b(d.shared_ff, H) + (uint64_t)B * ((uint64_t)d.n_expert_used * d.expert_ff + 2ull * H) * 4);
    }
    InProj hp{};
    hp.x = e->x; hp.x_stride = H; hp.norm_w = m->output_norm; hp.eps = d.rms_eps; hp.n_embd = H;
    hp.nq = 1; hp.q[0] = m->output; hp.qout[0] = e->logits; hp.qstride[0] = d.n_vocab; hp.exact = c->exact;
    launch_in(hp, d.n_vocab, grid_rows(d.n_vocab));
    MARK(KC_LM_HEAD, q8b(H, d.n_vocab) + (uint64_t)B * (H + d.n_vocab) * 4);
    launch_k(pdl, k_argmax_partial, dim3(ARGMAX_PARTS, B), 256, 0, st, e->logits, d.n_vocab, e->arg_v, e->arg_i); launches++;
    launch_k(pdl, k_argmax_advance, B, 32, 0, st, e->arg_v, e->arg_i, ARGMAX_PARTS, e->tokens, e->pos, e->next, e->history, (int)e->history_cap, e->step_counter, B);
    MARK(KC_ARGMAX, (uint64_t)B * d.n_vocab * 4);
#undef MARK
    e->launches_per_step = launches;
}

// Make the experts a layer's routing names resident (see TierState). Blocks on the stream once to read the ids.
static void tier_copy_in(itb_engine* e, cudaStream_t st, uint32_t il, int32_t ex, int slot, float* stage, size_t* stage_at) {
    TierState* t = e->tier;
    for (int k = 0; k < 3; ++k) {
        const itb_model::HostStack& h = e->m->host_experts[il][k];
        cudaMemcpyAsync(t->pool_nib[k] + (size_t)slot * h.nib_per, h.nib + (size_t)ex * h.nib_per, h.nib_per, cudaMemcpyHostToDevice, st);
        cudaMemcpyAsync(t->pool_sc[k] + (size_t)slot * h.sc_per, h.sc + (size_t)ex * h.sc_per, h.sc_per, cudaMemcpyHostToDevice, st);
        stage[*stage_at] = h.s2[(size_t)ex];
        cudaMemcpyAsync(t->pool_s2[k] + slot, stage + *stage_at, 4, cudaMemcpyHostToDevice, st);
        ++*stage_at;
        t->bytes_moved += h.nib_per + h.sc_per + 4;
    }
    t->fetched++;
}
// n_guess: guesses for layer il + 1 in t->guess_dev (0: none). Their copies go to the second stream and overlap this layer's
// expert kernels; the next call makes the engine's stream wait for them before anything reads the pools.
static bool tier_ensure(itb_engine* e, cudaStream_t st, uint32_t il, const int32_t* ids_dev, size_t n_pairs, size_t n_guess) {
    TierState* t = e->tier; itb_model* m = e->m; itb_ctx* c = e->c;
    const size_t E = m->d.n_expert;
    const auto w0 = std::chrono::steady_clock::now();
    bool got = cudaMemcpyAsync(t->ids_host, ids_dev, n_pairs * 4, cudaMemcpyDeviceToHost, st) == cudaSuccess;
    if (n_guess) got = got && cudaMemcpyAsync(t->guess_host, t->guess_dev, n_guess * 4, cudaMemcpyDeviceToHost, st) == cudaSuccess;
    if (!got || cudaStreamSynchronize(st) != cudaSuccess) return itb_fail_msg(c, "tiered experts: cannot read the routing ids");
    t->picks_wait_us += (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - w0).count();
    if (t->fetch_pending) {      // the guesses made for this layer: landed before it reads (device), and their staging is free again (host)
        cudaStreamWaitEvent(st, t->ev_fetch, 0); cudaEventSynchronize(t->ev_fetch); t->fetch_pending = false;
    }
    t->g->next_pass();
    t->s2_at = 0;
    for (size_t i = 0; i < n_pairs; ++i) {
        const int32_t ex = t->ids_host[i];
        if (ex < 0 || (size_t)ex >= E) return itb_fail_msg(c, "tiered experts: routing id out of range");
        const int64_t key = (int64_t)il * (int64_t)E + ex;
        bool hit = false; int64_t evicted = -1;
        const int slot = t->g->touch(key, &hit, &evicted);
        if (slot < 0) return itb_fail_msg(c, "tiered experts: a pass needs more distinct experts than the HBM pool holds");
        t->lookups++;
        if (hit) {
            if (t->guessed[(size_t)slot]) { t->guessed[(size_t)slot] = 0; t->prefetch_used++; }
            continue;
        }
        t->host_reads++;
        t->guessed[(size_t)slot] = 0;
        if (evicted >= 0) { t->slot_map_host[evicted] = -1; t->dirty[(size_t)evicted / E] = 1; }
        tier_copy_in(e, st, il, ex, slot, t->s2_stage, &t->s2_at);
        t->slot_map_host[key] = slot; t->dirty[il] = 1;
    }
    if (n_guess && il + 1 < m->d.n_layer) {
        bool any = false;
        size_t g_at = 0;
        for (size_t i = 0; i < n_guess; ++i) {
            const int32_t ex = t->guess_host[i];
            if (ex < 0 || (size_t)ex >= E || g_at + 3 > t->s2_guess_cap) continue;
            const int64_t key = (int64_t)(il + 1) * (int64_t)E + ex;
            int64_t evicted = -1;
            const int slot = t->g->prefetch(key, &evicted);
            if (slot < 0) continue;
            if (evicted >= 0) { t->slot_map_host[evicted] = -1; t->dirty[(size_t)evicted / E] = 1; }
            tier_copy_in(e, t->stream2, il + 1, ex, slot, t->s2_guess, &g_at);
            t->guessed[(size_t)slot] = 1; t->prefetch_reads++;
            t->slot_map_host[key] = slot; t->dirty[il + 1] = 1;
            any = true;
        }
        if (any) { cudaEventRecord(t->ev_fetch, t->stream2); t->fetch_pending = true; }
    }
    for (size_t r = 0; r < t->dirty.size(); ++r)
        if (t->dirty[r]) { cudaMemcpyAsync(t->slot_map + r * E, t->slot_map_host + r * E, E * 4, cudaMemcpyHostToDevice, st); t->dirty[r] = 0; }
    return true;
}
static DevFp4 tier_stack(const itb_engine* e, uint32_t il, int k, const DevFp4& shape) {
    const TierState* t = e->tier;
    DevFp4 w = shape;
    w.nib = t->pool_nib[k]; w.sc = t->pool_sc[k];
    w.scale2 = e->m->host_experts[il][k].has_s2 ? t->pool_s2[k] : nullptr;
    w.n_expert = (int)t->capacity; w.expert_lo = 0;
    w.slot_map = t->slot_map + (size_t)il * e->m->d.n_expert;
    return w;
}

// ---------------------------------------------------------------------------------------------------------
// The multi-row pass: n_seq sequences x n_tok consecutive tokens each (rows = n_seq * n_tok <= e->R), token ids in
// `tok_rows` (device, row-major). Batched decode is (B, 1); a prefill chunk of one sequence is (1, T).
// Ends with the LM head on each sequence's last row, the greedy argmax and the position advance.
// Buffers of the packed all-to-all of an expert-parallel engine, made by the prefill entry point BEFORE the ranks exchange
// their ready flags (so a rank that cannot allocate makes every rank refuse, and all ranks take the same path afterwards).
// A rank can receive every pair of every rank: capacity world * R * n_used pairs. False only when memory ran out.
static bool ep_a2a_prepare(itb_engine* e) {
    EpState* q = e->ep;
    NcclApi& nc = nccl_api();
    if (!q || !nc.Send || !nc.Recv || getenv("ITB_EP_A2A_OFF")) return true;      // the all-gather / reduce-scatter form serves
    const itb_model_dims& d = e->m->d;
    if (d.n_expert % q->world || d.n_embd % 32) return true;
    const size_t H = d.n_embd, K = d.n_expert_used, W = q->world, mine = (size_t)e->R * K, cap = W * mine;
    if (q->a2a_cap >= cap) return true;
    cudaStreamSynchronize(e->c->stream);
    bool ok = cudaMalloc(&q->sxq, mine * H) == cudaSuccess && cudaMalloc(&q->sxs, mine * (H / 32) * 4) == cudaSuccess && cudaMalloc(&q->sids, mine * 4) == cudaSuccess &&
              cudaMalloc(&q->rxq, cap * H) == cudaSuccess && cudaMalloc(&q->rxs, cap * (H / 32) * 4) == cudaSuccess && cudaMalloc(&q->rids, cap * 4) == cudaSuccess &&
              cudaMalloc(&q->o_back, mine * H * 4) == cudaSuccess && cudaMalloc(&q->owner, mine * 4) == cudaSuccess && cudaMalloc(&q->own_off, (W + 1) * 4) == cudaSuccess &&
              cudaMalloc(&q->own_list, mine * 4) == cudaSuccess && cudaMalloc(&q->cnt_dev, W * (W + 1) * 4) == cudaSuccess &&
              cudaMallocHost(&q->cnt_host, W * (W + 1) * 4) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        cudaFree(q->sxq); cudaFree(q->sxs); cudaFree(q->sids); cudaFree(q->rxq); cudaFree(q->rxs); cudaFree(q->rids); cudaFree(q->o_back); cudaFree(q->owner);
        cudaFree(q->own_off); cudaFree(q->own_list); cudaFree(q->cnt_dev); if (q->cnt_host) cudaFreeHost(q->cnt_host);
        q->sxq = q->rxq = nullptr; q->sxs = q->rxs = q->o_back = nullptr; q->sids = q->rids = q->owner = nullptr; q->own_off = q->own_list = q->cnt_dev = q->cnt_host = nullptr;
        return itb_fail_msg(e->c, "expert-parallel engine: out of device memory for the all-to-all buffers");
    }
    q->a2a_cap = cap;
    return true;
}

// The region and the peers' mappings for the one-token step over peer memory. Every rank runs this at engine creation, in
// step: allocate, exchange the IPC handles through the communicator, open the peers', then agree (one more all-gather) that
// EVERY rank succeeded -- otherwise all of them keep the NCCL form. ITB_EP_P2P=0 keeps the NCCL form too.
static void ep_p2p_setup(itb_engine* e) {
    EpState* q = e->ep;
    itb_ctx* c = e->c;
    NcclApi& nc = nccl_api();
    const itb_model_dims& d = e->m->d;
    const int W = q->world;
    if (e->B > 64 || W > 8 || d.n_embd % 128 || d.n_expert % 4 || d.n_expert % W || (getenv("ITB_EP_P2P") && atoi(getenv("ITB_EP_P2P")) == 0)) return;
    const size_t H = d.n_embd, E = d.n_expert, K = d.n_expert_used, NL = d.n_layer, RB = e->B;
    // one sequence: the fused one-token kernels (they gather the router logits and route every rank's row themselves);
    // several: the multi-row kernels (each rank routes its own rows and the ids travel)
    const bool rows = RB != 1;
    q->g_slot = 0;
    q->g_layer = rows ? (((size_t)W * RB * (H + H / 32 * 4 + K * 4) + 127) & ~(size_t)127)      // per layer: [W][RB][H] int8 | [W][RB][H/32] f32 | [W][RB][K] i32
                      : (((size_t)W * (H + H / 32 * 4 + E * 4) + 127) & ~(size_t)127);          // per layer: [W][H] int8 | [W][H/32] f32 | [W][E] f32
    q->o_layer = RB * K * H * 4;
    q->off_g = 0; q->off_o = q->off_g + NL * q->g_layer; q->off_gf = q->off_o + NL * q->o_layer; q->off_of = q->off_gf + NL * 8 * 4;
    q->region_bytes = q->off_of + NL * 8 * 4;
    bool ok = cudaMalloc(&q->region, q->region_bytes) == cudaSuccess && cudaMalloc(&q->seq, 4) == cudaSuccess && cudaMalloc(&q->peer_dev, 8 * sizeof(void*)) == cudaSuccess;
    cudaIpcMemHandle_t mine{}, *all_h = nullptr; unsigned char* hbuf = nullptr; int* flags_dev = nullptr;
    std::vector<cudaIpcMemHandle_t> handles(W);
    std::vector<int> flags(W, 0);
    if (ok) {
        cudaMemsetAsync(q->region, 0, q->region_bytes, c->stream); cudaMemsetAsync(q->seq, 0, 4, c->stream);
        ok = cudaIpcGetMemHandle(&mine, q->region) == cudaSuccess;
    }
    ok = cudaMalloc(&hbuf, (size_t)(W + 1) * sizeof mine) == cudaSuccess && cudaMalloc(&flags_dev, (size_t)(W + 1) * 4) == cudaSuccess && ok;
    // the handle exchange is a collective: every rank enters it whatever happened before (a failed rank sends zeros)
    if (hbuf && flags_dev) {
        cudaMemcpyAsync(hbuf + (size_t)W * sizeof mine, &mine, sizeof mine, cudaMemcpyHostToDevice, c->stream);
        nc.AllGather(hbuf + (size_t)W * sizeof mine, hbuf, sizeof mine, NcclApi::Int8, q->comm, c->stream);
        cudaMemcpyAsync(handles.data(), hbuf, (size_t)W * sizeof mine, cudaMemcpyDeviceToHost, c->stream);
        if (cudaStreamSynchronize(c->stream) != cudaSuccess) ok = false;
        (void)all_h;
        for (int r = 0; r < W && ok; ++r) {
            if (r == q->rank) { q->peer[r] = q->region; continue; }
            void* ptr = nullptr;
            if (cudaIpcOpenMemHandle(&ptr, handles[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); ok = false; break; }
            q->peer[r] = (unsigned char*)ptr;
        }
        int okf = ok ? 1 : 0;
        cudaMemcpyAsync(flags_dev + W, &okf, 4, cudaMemcpyHostToDevice, c->stream);
        nc.AllGather(flags_dev + W, flags_dev, 1, NcclApi::Int32, q->comm, c->stream);
        cudaMemcpyAsync(flags.data(), flags_dev, (size_t)W * 4, cudaMemcpyDeviceToHost, c->stream);
        if (cudaStreamSynchronize(c->stream) != cudaSuccess) ok = false;
        for (int r = 0; r < W; ++r) ok = ok && flags[r] == 1;
    } else ok = false;       // (a rank that could not even allocate the exchange buffers cannot take part: with identical ranks this is all or none)
    cudaFree(hbuf); cudaFree(flags_dev);
    if (ok) {
        cudaMemcpy(q->peer_dev, q->peer, 8 * sizeof(void*), cudaMemcpyHostToDevice);
        if (rows) q->p2p_rows = true; else q->p2p = true;
    } else {
        for (int r = 0; r < W; ++r) if (r != q->rank && q->peer[r]) { cudaIpcCloseMemHandle(q->peer[r]); q->peer[r] = nullptr; }
        cudaFree(q->region); cudaFree(q->seq); cudaFree(q->peer_dev); q->region = nullptr; q->seq = nullptr; q->peer_dev = nullptr;
    }
}

static uint64_t enqueue_rows(itb_engine* e, cudaStream_t st, int n_seq, int n_tok, const int32_t* tok_rows) {
    itb_model* m = e->m; itb_ctx* c = e->c;
    const itb_model_dims& d = m->d;
    const int R = n_seq * n_tok, H = d.n_embd, sms = c->sm_count;
    const int sk = d.ssm_d_state, n_k = d.ssm_n_group, n_v = d.ssm_dt_rank;
    const int key_dim = sk * n_k, vd = d.ssm_d_inner, cd = 2 * key_dim + vd;
    const int qd = d.head_dim * d.n_head, kvd = d.head_dim * d.n_head_kv;
    const int TPB = NWG * 32;
    uint64_t launches = 0;
    static bool attrs_set = false;
    if (!attrs_set) {
        set_smem((const void*)k_gemm_q8<4>, 200 * 1024); set_smem((const void*)k_gemm_q8<1>, 200 * 1024);
        set_smem((const void*)k_glu_grouped, 200 * 1024); set_smem((const void*)k_down_grouped, 200 * 1024);
        set_smem((const void*)k_matmul_f32_rows<20>, 64 * 1024); set_smem((const void*)k_matmul_f32_rows<24>, 64 * 1024);
        set_smem((const void*)k_matmul_f32_rows<28>, 64 * 1024); set_smem((const void*)k_matmul_f32_rows<32>, 64 * 1024);
        set_smem((const void*)k_tile_q8<1, 256, 4>, 226 * 1024); set_smem((const void*)k_tile_q8<4, 256, 2>, 226 * 1024);
        set_smem((const void*)k_tile_q8_multi<1, 256, 4>, 226 * 1024);
        set_smem((const void*)k_sgemm_serial_small<false>, sgemm_small_smem()); set_smem((const void*)k_sgemm_serial_small<true>, sgemm_small_smem());
        set_smem((const void*)k_gdn_chunk_prep<128>, gdn_chunk_prep_smem<128>()); set_smem((const void*)k_gdn_chunk_scan<128>, gdn_chunk_scan_smem<128>());
        set_smem((const void*)k_tile_glu<1, 256, 1>, 226 * 1024); set_smem((const void*)k_tile_down<1, 256, 1>, 226 * 1024);
        set_smem((const void*)k_tile_glu<2, 256, 1>, 226 * 1024); set_smem((const void*)k_tile_down<2, 256, 1>, 226 * 1024);
        set_smem((const void*)k_tile_glu<4, 256, 1>, 226 * 1024); set_smem((const void*)k_tile_down<4, 256, 1>, 226 * 1024);
        set_smem((const void*)k_tile_glu<4, 256, 2>, 226 * 1024); set_smem((const void*)k_tile_down<4, 256, 2>, 226 * 1024);
        set_smem((const void*)k_matmul_f32<true>, 100 * 1024); set_smem((const void*)k_matmul_f32<false>, 100 * 1024);
        attrs_set = true;
    }
    // Pipelined tile kernels when k is a multiple of the chunk (every matrix of the 35B and 177B shapes); the
    // direct-load MMA kernels otherwise.
    cudaStreamCaptureStatus cap_rows = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(st, &cap_rows);
    const bool q8tc = c->q8tc && n_tok > 1 && cap_rows == cudaStreamCaptureStatusNone;
    const bool f16tc = c->f16tc && n_tok > 1 && cap_rows == cudaStreamCaptureStatusNone;
    // same: this matmul reads the quantised rows the previous one read (their tensor-core images are still current)
    auto gemm_n = [&](const DevQ8& w, const int8_t* xq, const float* xs, float* out, size_t stride, int mode, int R, bool same = false) {
        const int k = w.n_in;
        if (f16tc && R >= 64 && itb_tc_f16_shape_ok(w)) {
            // many rows, dense=f16tc (tolerance class): both operands dequantised to f16, one tcgen05 GEMM with f32 accumulators
            if (itb_tc_f16_gemm(c, st, w, xq, xs, R, out, stride, mode, same)) { launches++; return; }
        }
        if (q8tc && R >= 64 && itb_tc_q8_shape_ok(w)) {
            // many rows, dense=q8tc: integer dots of 128 x 128 (row, token) pairs per tcgen05 MMA, scaled and summed in the CPU's order
            if (itb_tc_q8_gemm(c, st, w, xq, xs, R, out, stride, mode, same)) { launches++; return; }
        }
        const bool skinny = R <= 32;
        if (skinny && k % 256 == 0) {
            const int ns = std::min(k / 256, TILE_STAGES);
            k_tile_q8<1, 256, 4><<<dim3((w.n_out + 31) / 32, (R + 31) / 32), 256, tile_smem<MK_Q8, 1, 256, 4>(k), st>>>(w, xq, xs, R, out, stride, mode, ns);
        } else if (!skinny && k % 256 == 0) {
            const int ns = std::min(k / 256, TILE_STAGES);
            k_tile_q8<4, 256, 2><<<dim3((w.n_out + 63) / 64, (R + 63) / 64), 256, tile_smem<MK_Q8, 4, 256, 2>(k), st>>>(w, xq, xs, R, out, stride, mode, ns);
        } else if (skinny) k_gemm_q8<1><<<dim3((w.n_out + 63) / 64, 1), 512, gemm_smem(w.n_in), st>>>(w, xq, xs, R, out, stride, mode);
        else k_gemm_q8<4><<<dim3((w.n_out + MMA_ROWS - 1) / MMA_ROWS, (R + MMA_TOK - 1) / MMA_TOK), 256, gemm_smem(w.n_in), st>>>(w, xq, xs, R, out, stride, mode);
        launches++;
    };
    auto gemm = [&](const DevQ8& w, const int8_t* xq, const float* xs, float* out, size_t stride, int mode, bool same = false) { gemm_n(w, xq, xs, out, stride, mode, R, same); };
    // two or three dense matrices over the same quantised rows (mode 0): with few rows (batched decode) one launch for all of
    // them; otherwise one after the other, the later ones told that the rows' tensor-core images are current
    auto gemm_multi = [&](int n, const DevQ8* const* w, float* const* out, const size_t* stride, const int8_t* xq, const float* xs) {
        bool one = R <= 32 && n <= 3;
        for (int i = 0; i < n; ++i) one = one && w[i]->q && w[i]->n_in == w[0]->n_in && w[i]->n_in % 256 == 0;
        if (one) {
            Q8Multi p{};
            p.n = n;
            int tiles = 0;
            for (int i = 0; i < n; ++i) { p.w[i] = *w[i]; p.out[i] = out[i]; p.stride[i] = stride[i]; p.tiles[i] = (w[i]->n_out + 31) / 32; tiles += p.tiles[i]; }
            const int k = w[0]->n_in, ns = std::min(k / 256, TILE_STAGES);
            k_tile_q8_multi<1, 256, 4><<<dim3(tiles, (R + 31) / 32), 256, tile_smem<MK_Q8, 1, 256, 4>(k), st>>>(p, xq, xs, R, ns);
            launches++;
            return;
        }
        for (int i = 0; i < n; ++i) gemm(*w[i], xq, xs, out[i], stride[i], 0, i > 0);
    };
    // A dense matrix stored as NVFP4 (shared experts, LM head of an NVFP4 file): int8 activations x E2M1 weights in the CPU
    // order (src/ops/naive.rs:714-734), then the tensor's second scale on the result (src/model/qwen35.rs:1668-1682).
    auto gemm_fp4d = [&](const DevFp4& w, const int8_t* xq, const float* xs, float* out, int rows, bool has_s, float sc) {
        if (rows >= 2 && gemm_smem(w.n_in) <= 200 * 1024) {
            set_smem((const void*)k_gemm_fp4, gemm_smem(w.n_in));
            k_gemm_fp4<<<dim3((w.n_out + MMA_ROWS - 1) / MMA_ROWS, (rows + MMA_TOK - 1) / MMA_TOK), 256, gemm_smem(w.n_in), st>>>(
                w.nib, w.sc, w.n_in, w.n_out, xq, xs, rows, out, (size_t)w.n_out, sc, has_s ? 1 : 0);
            launches++;
            return;
        }
        const int nb = w.n_in / 32, nsb = w.n_in / 16, gsh = lanes_shift(nb), nw = 8;
        const int gx = std::max(1, std::min((w.n_out + 31) / 32, 2 * sms));
        const size_t smem = (size_t)w.n_in + (size_t)nb * 4 + (size_t)nw * terms_floats(4, gsh, nsb) * 4;
        set_smem((const void*)k_matmul_fp4, smem);
        k_matmul_fp4<<<dim3(gx, rows), nw * 32, smem, st>>>(w, nullptr, 1, 0, xq, xs, out);
        launches++;
        if (has_s) { const size_t n = (size_t)rows * w.n_out; k_scale<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(out, n, sc); launches++; }
    };
    auto f32mm = [&](const DevF32& w, const float* x, float* out) {
        if (!c->exact && f16tc && w.n_in % SGS_K == 0 && R >= 64) {
            // tolerance-class passes: the serial-order tiles with fused multiply-adds (a chain per (row, output), k in order)
            const int big = ((w.n_out + SG_T - 1) / SG_T) * ((R + SG_T - 1) / SG_T);
            if (big >= sms / 2) k_sgemm_serial<true><<<dim3((w.n_out + SG_T - 1) / SG_T, (R + SG_T - 1) / SG_T), 256, 0, st>>>(w, x, R, out);
            else k_sgemm_serial_small<true><<<dim3((w.n_out + 15) / 16, (R + 15) / 16), 256, sgemm_small_smem(), st>>>(w, x, R, out);
            launches++;
            return;
        }
        if (!c->exact && w.n_in % 512 == 0 && w.n_in <= 4096) {
            const dim3 g((w.n_out + 7) / 8, (R + F32_TOK - 1) / F32_TOK);
            const size_t sm = (size_t)F32_TOK * w.n_in * 4;
            switch (w.n_in / 128) {
#define F32_CASE(NV) case NV: k_matmul_f32_rows<NV><<<g, 256, sm, st>>>(w, x, R, out); break;
                F32_CASE(4) F32_CASE(8) F32_CASE(12) F32_CASE(16) F32_CASE(20) F32_CASE(24) F32_CASE(28) F32_CASE(32)
#undef F32_CASE
            }
            launches++;
            return;
        }
        if (c->exact && w.n_in % SGS_K == 0) {
            // a chain per (row, output), a thread per 4 x 4 of them, k in order (also for a few rows: the tile's k loop is as long as a row's chain either way)
            const int big = ((w.n_out + SG_T - 1) / SG_T) * ((R + SG_T - 1) / SG_T);
            if (big >= sms / 2) k_sgemm_serial<false><<<dim3((w.n_out + SG_T - 1) / SG_T, (R + SG_T - 1) / SG_T), 256, 0, st>>>(w, x, R, out);
            else k_sgemm_serial_small<false><<<dim3((w.n_out + 15) / 16, (R + 15) / 16), 256, sgemm_small_smem(), st>>>(w, x, R, out);
            launches++;
            return;
        }
        const int nw = 4;
        dim3 g(std::max(1, std::min(2 * sms, (w.n_out + 31) / 32)), R);
        size_t sm = (size_t)w.n_in * 4 + (size_t)nw * 32 * 33 * 4;
        if (c->exact) k_matmul_f32<true><<<g, nw * 32, sm, st>>>(w, x, out);
        else k_matmul_f32<false><<<g, nw * 32, sm, st>>>(w, x, out);
        launches++;
    };
    // two F32 matrices over the same rows: one launch where both take the small serial-order tiles, else one after the other
    auto f32mm2 = [&](const DevF32& wa, float* oa, const DevF32& wb, float* ob, const float* x) {
        const bool fused = !c->exact && f16tc && R >= 64;
        const int big_a = ((wa.n_out + SG_T - 1) / SG_T) * ((R + SG_T - 1) / SG_T), big_b = ((wb.n_out + SG_T - 1) / SG_T) * ((R + SG_T - 1) / SG_T);
        if ((c->exact || fused) && wa.n_in == wb.n_in && wa.n_in % SGS_K == 0 && big_a < sms / 2 && big_b < sms / 2) {
            const dim3 g((std::max(wa.n_out, wb.n_out) + 15) / 16, (R + 15) / 16, 2);
            if (fused) k_sgemm_serial_small<true><<<g, 256, sgemm_small_smem(), st>>>(wa, x, R, oa, wb, ob);
            else k_sgemm_serial_small<false><<<g, 256, sgemm_small_smem(), st>>>(wa, x, R, oa, wb, ob);
            launches++;
            return;
        }
        f32mm(wa, x, oa); f32mm(wb, x, ob);
    };
    const size_t smem_nq = 256 + (size_t)H * 4;
    if (e->ep && e->ep->p2p_rows && n_tok == 1 && R == (int)e->B) { k_ep_tick<<<1, 32, 0, st>>>(e->ep->seq); launches++; }    // the step number the peers' flags will carry
    k_embed<<<R, 256, 0, st>>>(m->tok_embd.w, H, tok_rows, e->x); launches++;
    for (uint32_t il = 0; il < d.n_layer; ++il) {
        const DevLayer& L = m->layers[il];
        k_norm_quant<<<R, 256, smem_nq, st>>>(e->x, L.attn_norm, H, d.rms_eps, e->xn, e->xq, e->xs); launches++;
        if (L.recurrent) {
            const int rs = e->slot_of[il];
            const size_t state_stride = (size_t)n_v * sk * sk, conv_stride = (size_t)cd * (d.ssm_d_conv - 1);
            {
                const DevQ8* ws[2] = {&L.wqkv, &L.wgate}; float* os[2] = {e->qkvc, e->z}; const size_t ss[2] = {(size_t)cd, (size_t)vd};
                gemm_multi(2, ws, os, ss, e->xq, e->xs);
            }
            f32mm2(L.ssm_alpha, e->alpha, L.ssm_beta, e->beta, e->xn);
            float* cst = e->conv_state + (size_t)rs * e->B * conv_stride;
            if (d.ssm_d_conv == 4 && n_tok >= CONV_T) k_conv_rows4<<<dim3((cd + 127) / 128, n_seq * ((n_tok + CONV_T - 1) / CONV_T)), 128, 0, st>>>(cst, conv_stride, e->qkvc, e->qkvc2, n_tok, cd, L.conv1d);
            else k_conv_rows<<<dim3((cd + 127) / 128, R), 128, 0, st>>>(cst, conv_stride, e->qkvc, e->qkvc2, n_tok, cd, L.conv1d, d.ssm_d_conv);
            launches++;
            k_conv_state<<<dim3((cd + 127) / 128, n_seq), 128, 0, st>>>(cst, conv_stride, e->qkvc, n_tok, cd, d.ssm_d_conv); launches++;
            k_gdn_pre<<<dim3(R, 2 * n_k + n_v), sk, 0, st>>>(e->qkvc2, cd, e->alpha, e->beta, L.ssm_a, L.dt_bias, sk, n_k, n_v, d.rms_eps,
                                                            e->qh, e->kh, e->vh, e->gb); launches++;
            const size_t chunk_need = (size_t)n_seq * ((n_tok + GC - 1) / GC) * n_v * gdn_chunk_floats<128>();
            if ((c->gdn_chunk || !c->exact) && n_tok >= 32 && sk == 128 && e->gdn_scratch_cap >= chunk_need) {
                // many tokens: everything that does not touch the state for all chunks at once, then three small products per chunk
                float* sst = e->ssm_state + (size_t)rs * e->B * state_stride;
                k_gdn_chunk_prep<128><<<dim3((n_tok + GC - 1) / GC, n_v, n_seq), 256, gdn_chunk_prep_smem<128>(), st>>>(e->qh, e->kh, e->vh, e->gb, n_tok, n_k, n_v, e->gdn_scratch);
                k_gdn_chunk_scan<128><<<dim3(n_v, sk / GC_VS, n_seq), 256, gdn_chunk_scan_smem<128>(), st>>>(e->gdn_scratch, n_tok, n_v, sst, state_stride, e->core);
                launches++;
            } else {
                const dim3 gs(n_v, sk / 32, n_seq);
                float* sst = e->ssm_state + (size_t)rs * e->B * state_stride;
                if (sk == 128) k_gdn_scan<128><<<gs, 128, 0, st>>>(e->qh, e->kh, e->vh, e->gb, n_tok, n_k, n_v, sst, state_stride, e->core);
                else k_gdn_scan<64><<<gs, 128, 0, st>>>(e->qh, e->kh, e->vh, e->gb, n_tok, n_k, n_v, sst, state_stride, e->core);   // 64 or 128 only (checked at model creation)
            }
            launches++;
            k_gdn_post<<<dim3(R, n_v), sk, 0, st>>>(e->core, e->z, L.ssm_norm, sk, n_v, d.rms_eps, e->aq, e->as); launches++;
            gemm(L.ssm_out, e->aq, e->as, e->x, H, 1);
        } else {
            const int as = e->slot_of[il];
            {
                const DevQ8* ws[3] = {&L.wq, &L.wk, &L.wv}; float* os[3] = {e->qg, e->kbuf, e->vbuf}; const size_t ss[3] = {(size_t)2 * qd, (size_t)kvd, (size_t)kvd};
                gemm_multi(3, ws, os, ss, e->xq, e->xs);
            }
            AttnPrepRows a{};
            a.qg = e->qg; a.k = e->kbuf; a.v = e->vbuf; a.q_norm = L.q_norm; a.k_norm = L.k_norm; a.q_out = e->qn; a.g_out = e->gate;
            a.slab_stride = (size_t)e->n_ctx * kvd;
            a.kslab = e->kslab + (size_t)as * e->B * a.slab_stride; a.vslab = e->vslab + (size_t)as * e->B * a.slab_stride;
            a.pos = e->pos; a.npos_out = e->npos; a.n_tok = n_tok; a.hd = d.head_dim; a.n_head = d.n_head; a.n_head_kv = d.n_head_kv;
            a.n_rot = d.n_rot; a.theta = d.rope_theta; a.eps = d.rms_eps; a.bf16 = c->kv_bf16;
            k_attn_prep_rows<<<dim3(d.n_head + 2 * d.n_head_kv, R), d.head_dim, d.head_dim * 4, st>>>(a); launches++;
            const float scale = 1.0f / sqrtf((float)d.head_dim);
            const int nwa = 8, ns = n_tok > 1 ? e->n_split_rows : e->n_split;
            const size_t smem_a = (size_t)nwa * 8 * 2 * 4 + (size_t)nwa * 8 * d.head_dim * 4;
            const int group = d.n_head / d.n_head_kv;
            if ((c->attn_mma || !c->exact) && n_tok >= 16 && AM_ROWS % group == 0 && (d.head_dim == 64 || d.head_dim == 128 || d.head_dim == 256) && kvd % 8 == 0) {
                // many tokens: causal attention as matrix products over (token, head) tiles, one "split" handed to the combine
                AmParams ap{};
                ap.q = e->qn; ap.kslab = a.kslab; ap.vslab = a.vslab; ap.slab_stride = a.slab_stride; ap.npos = e->npos; ap.n_tok = n_tok; ap.kv_dim = kvd;
                ap.n_head = d.n_head; ap.n_head_kv = d.n_head_kv; ap.group = group; ap.scale = scale; ap.part_acc = e->part_acc; ap.part_ml = e->part_ml;
                const dim3 ga((n_tok + AM_ROWS / group - 1) / (AM_ROWS / group), d.n_head_kv, n_seq);
#define AM_CASE(HD)                                                                                                      \
    case HD:                                                                                                              \
        set_smem((const void*)k_attn_mma<HD, true>, attn_mma_smem<HD>()); set_smem((const void*)k_attn_mma<HD, false>, attn_mma_smem<HD>()); \
        if (c->kv_bf16) k_attn_mma<HD, true><<<ga, 256, attn_mma_smem<HD>(), st>>>(ap);                                    \
        else k_attn_mma<HD, false><<<ga, 256, attn_mma_smem<HD>(), st>>>(ap);                                              \
        break;
                switch (d.head_dim) { AM_CASE(64) AM_CASE(128) AM_CASE(256) }
#undef AM_CASE
                launches++;
                k_attn_combine_rows<<<R * d.n_head, d.head_dim, 0, st>>>(e->part_acc, e->part_ml, 1, d.head_dim, e->gate, e->npos, d.n_head, e->aq, e->as); launches++;
            } else if (exact_attention_ok(e) && e->scores_cap >= (size_t)R * d.n_head * e->n_ctx) {
                uint32_t top = 0;
                for (int sq = 0; sq < n_seq; ++sq) top = std::max(top, e->host_pos[sq] + (uint32_t)n_tok);
                if (n_tok == 1) top = e->n_ctx;        // a decode pass is replayed from a graph: its launches must hold any length
                enqueue_exact_attention(e, st, false, a.kslab, a.vslab, a.slab_stride, R, n_tok, (int)std::min<uint32_t>(top, e->n_ctx));
                launches += 2;
            } else {
            {
                dim3 grid(d.n_head_kv, R, ns);
#define ATT_CASE(HD)                                                                                                          \
    case HD:                                                                                                                   \
        set_smem((const void*)k_attn_partial<HD, 8>, smem_a);                                                                  \
        k_attn_partial<HD, 8><<<grid, nwa * 32, smem_a, st>>>(e->qn, a.kslab, a.vslab, kvd, 0, n_tok, d.n_head, d.n_head_kv,    \
            scale, c->kv_bf16, e->npos, e->part_acc, e->part_ml, n_tok, a.slab_stride);                                        \
        break;
                switch (d.head_dim) { ATT_CASE(64) ATT_CASE(128) ATT_CASE(256) }
#undef ATT_CASE
                launches++;
            }
            k_attn_combine_rows<<<R * d.n_head, d.head_dim, 0, st>>>(e->part_acc, e->part_ml, ns, d.head_dim, e->gate, e->npos, d.n_head,
                                                                    e->aq, e->as); launches++;
            }
            gemm(L.wo, e->aq, e->as, e->x, H, 1);
        }
        // routed FFN
        k_norm_quant<<<R, 256, smem_nq, st>>>(e->x, L.ffn_norm, H, d.rms_eps, e->xn, e->xq, e->xs); launches++;
        if (!L.shared4[0].nib && !L.shared4[1].nib) {
            const DevQ8* ws[2] = {&L.shared_gate, &L.shared_up}; float* os[2] = {e->sg, e->su}; const size_t ss[2] = {(size_t)d.shared_ff, (size_t)d.shared_ff};
            gemm_multi(2, ws, os, ss, e->xq, e->xs);
        } else {
            if (L.shared4[0].nib) gemm_fp4d(L.shared4[0], e->xq, e->xs, e->sg, R, L.has_shared_s[0], L.shared_s[0]);
            else gemm(L.shared_gate, e->xq, e->xs, e->sg, d.shared_ff, 0);
            if (L.shared4[1].nib) gemm_fp4d(L.shared4[1], e->xq, e->xs, e->su, R, L.has_shared_s[1], L.shared_s[1]);
            else gemm(L.shared_up, e->xq, e->xs, e->su, d.shared_ff, 0, !L.shared4[0].nib);
        }
        f32mm2(L.gate_inp, e->router, L.shared_gate_inp, e->shlogit, e->xn);
        {
            const int K = d.n_expert_used, E = d.n_expert, ff = d.expert_ff;
            int32_t* ids = e->route_ids + (size_t)il * e->R * K;
            float* wts = e->route_w + (size_t)il * e->R * K;
            k_route_rows<<<(R + 3) / 4, 128, (size_t)4 * ((E + 31) & ~31) * 4, st>>>(e->router, R, E, K, ids, wts); launches++;
            // expert parallel: the pairs of every rank's rows, rank-major; otherwise just ours
            const int W = e->ep ? e->ep->world : 1;
            int P = W * R * K, Kt = K;                  // pairs the expert kernels see; pairs per activation row among them
            const int8_t* xq_src = e->xq; const float* xs_src = e->xs; const int32_t* ids_src = ids;
            const bool a2a = e->ep && n_tok > 1 && cap_rows == cudaStreamCaptureStatusNone && e->ep->a2a_cap >= (size_t)e->ep->world * e->R * K;
            const bool p2r = e->ep && e->ep->p2p_rows && n_tok == 1 && R == (int)e->B;
            std::vector<int> a2a_soff, a2a_roff;
            if (a2a) {
                // eager many-row pass: packed all-to-all. Every (row, pick) pair goes to the rank that holds its expert -- its
                // quantised row, scales and id, nothing else -- and its output row comes back; no rank touches a pair it does
                // not serve. Counts are exchanged first (one small all-gather, read on the host: the sends are sized by them).
                EpState* q = e->ep;
                NcclApi& nc = nccl_api();
                const int PK = R * K;
                k_ep_owner<<<(PK + 255) / 256, 256, 0, st>>>(ids, PK, E / W, q->owner);
                k_group_pairs_fast<<<1, 1024, (size_t)W * 4, st>>>(q->owner, PK, W, q->own_off, q->own_list);
                k_ep_pack<<<(unsigned)(((size_t)PK * (H / 16) + 255) / 256), 256, 0, st>>>(e->xq, e->xs, ids, q->own_list, PK, K, H, q->sxq, q->sxs, q->sids);
                nc.AllGather(q->own_off, q->cnt_dev, (size_t)W + 1, NcclApi::Int32, q->comm, st);
                cudaMemcpyAsync(q->cnt_host, q->cnt_dev, (size_t)W * (W + 1) * 4, cudaMemcpyDeviceToHost, st);
                if (cudaStreamSynchronize(st) != cudaSuccess) { itb_fail_msg(c, "expert-parallel pass: the pair counts could not be read"); return launches; }
                std::vector<int> cnt((size_t)W * W);
                for (int sr = 0; sr < W; ++sr)
                    for (int dr = 0; dr < W; ++dr) cnt[(size_t)sr * W + dr] = q->cnt_host[sr * (W + 1) + dr + 1] - q->cnt_host[sr * (W + 1) + dr];
                a2a_soff.assign(W + 1, 0); a2a_roff.assign(W + 1, 0);
                int n_recv = 0;
                if (itb_ep_a2a_plan(cnt.data(), W, q->rank, a2a_soff.data(), a2a_roff.data(), &n_recv) || (size_t)n_recv > q->a2a_cap || a2a_soff[W] != PK) {
                    itb_fail_msg(c, "expert-parallel pass: inconsistent pair counts"); return launches;
                }
                nc.GroupStart();
                for (int r = 0; r < W; ++r) {
                    const size_t so = a2a_soff[r], sn = a2a_soff[r + 1] - a2a_soff[r], ro = a2a_roff[r], rn = a2a_roff[r + 1] - a2a_roff[r];
                    if (sn) {
                        nc.Send(q->sxq + so * H, sn * H, NcclApi::Int8, r, q->comm, st);
                        nc.Send(q->sxs + so * (H / 32), sn * (H / 32), NcclApi::Float32, r, q->comm, st);
                        nc.Send(q->sids + so, sn, NcclApi::Int32, r, q->comm, st);
                    }
                    if (rn) {
                        nc.Recv(q->rxq + ro * H, rn * H, NcclApi::Int8, r, q->comm, st);
                        nc.Recv(q->rxs + ro * (H / 32), rn * (H / 32), NcclApi::Float32, r, q->comm, st);
                        nc.Recv(q->rids + ro, rn, NcclApi::Int32, r, q->comm, st);
                    }
                }
                nc.GroupEnd();
                launches += 5;
                xq_src = q->rxq; xs_src = q->rxs; ids_src = q->rids; P = n_recv; Kt = 1;
            } else if (p2r) {
                // a step of several sequences over peer memory: this rank's rows and routing ids stored into every rank's region,
                // then wait (bounded) until every rank's have arrived here. No collective call, nothing zero-filled.
                EpState* q = e->ep;
                const size_t base = q->off_g + (size_t)il * q->g_layer, o_xq = base, o_xs = o_xq + (size_t)W * R * H, o_id = o_xs + (size_t)W * R * (H / 32) * 4;
                k_ep_push_rows<<<W, 256, 0, st>>>(e->xq, e->xs, ids, R * H / 16, R * (H / 32) / 4, R * K, (unsigned char* const*)q->peer_dev,
                                                  o_xq + (size_t)q->rank * R * H, o_xs + (size_t)q->rank * R * (H / 32) * 4, o_id + (size_t)q->rank * R * K * 4,
                                                  q->off_gf + ((size_t)il * 8 + q->rank) * 4, (const unsigned*)q->seq);
                k_ep_wait<<<1, 32, 0, st>>>((const unsigned*)(q->region + q->off_gf + (size_t)il * 8 * 4), W, (const unsigned*)q->seq, e->err);
                launches += 2;
                xq_src = (const int8_t*)(q->region + o_xq); xs_src = (const float*)(q->region + o_xs); ids_src = (const int32_t*)(q->region + o_id);
            } else if (e->ep) {
                NcclApi& nc = nccl_api();
                nc.GroupStart();
                nc.AllGather(e->xq, e->ep->gxq, (size_t)R * H, NcclApi::Int8, e->ep->comm, st);
                nc.AllGather(e->xs, e->ep->gxs, (size_t)R * (H / 32), NcclApi::Float32, e->ep->comm, st);
                nc.AllGather(ids, e->ep->gids, (size_t)R * K, NcclApi::Int32, e->ep->comm, st);
                nc.GroupEnd();
                launches++;
                xq_src = e->ep->gxq; xs_src = e->ep->gxs; ids_src = e->ep->gids;
                cudaMemsetAsync(e->o_all, 0, (size_t)P * H * sizeof(float), st);   // rows of pairs served elsewhere stay zero
            }
            DevFp4 Lg = L.gate, Lu = L.up, Ld = L.down;
            if (e->tier) {
                size_t n_guess = 0;
                if (e->tier->prefetch_k > 0 && il + 1 < d.n_layer) {
                    // the hint: layer il + 1's router on THIS layer's router input, top prefetch_k per row (src/ops/mod.rs:915-924)
                    const int pk = std::min<int>(e->tier->prefetch_k, std::min<int>(16, E));
                    f32mm(m->layers[il + 1].gate_inp, e->xn, e->tier->guess_logits);
                    k_route_rows<<<(R + 3) / 4, 128, (size_t)4 * ((E + 31) & ~31) * 4, st>>>(e->tier->guess_logits, R, E, pk, e->tier->guess_dev, e->tier->guess_w); launches++;
                    n_guess = (size_t)R * pk;
                }
                if (!tier_ensure(e, st, il, ids, (size_t)R * K, n_guess)) return launches;
                Lg = tier_stack(e, il, 0, L.gate); Lu = tier_stack(e, il, 1, L.up); Ld = tier_stack(e, il, 2, L.down);
            }
            if (P > 0) {
            if (E <= 1024) k_group_pairs_fast<<<1, 1024, (size_t)E * 4, st>>>(ids_src, P, E, e->pair_off, e->pair_list);
            else k_group_pairs<<<1, 256, (size_t)E * 4, st>>>(ids_src, P, E, e->pair_off, e->pair_list);
            launches++;
            const cudaStreamCaptureStatus cap_st = cap_rows;
            if (c->fp4tc && n_tok > 1 && !e->ep && !e->tier && cap_st == cudaStreamCaptureStatusNone && itb_tc_shape_ok(Lg) && itb_tc_shape_ok(Lu) && itb_tc_shape_ok(Ld)) {
                // many rows, experts=fp4tc: FP4 activations times FP4 weights on the tensor cores (the reference's default device
                // arithmetic, src/ops/cuda/mod.rs:239-248 there); gate/up + SiLU in one GEMM's epilogue, then down
                if (!itb_tc_experts(c, st, Lg, &Lu, e->xn, K, e->pair_off, e->pair_list, P, e->h_all) ||
                    !itb_tc_experts(c, st, Ld, nullptr, e->h_all, 1, e->pair_off, e->pair_list, P, e->o_all)) return launches;
                launches += 6;
            } else {
                // rows per expert decide the tile shape (a tile's empty token columns cost as much as full ones)
                const bool tile_w = H % 256 == 0 && ff % 256 == 0;
                // up to 32 rows per expert: 128 weight rows x 8*NJ tokens per block (every weight decoded by one warp); more: 64 x 64
                // (an expert-parallel rank serves all the pairs it sees with its own E / W experts)
                const int e_here = e->ep ? std::max(1, E / W) : E;
                const int per_e = (P + e_here - 1) / e_here, nj = per_e <= 8 ? 1 : per_e <= 16 ? 2 : per_e <= 32 ? 4 : 0;
                const int ns_g = std::min(H / 256, TILE_STAGES), ns_d = std::min(ff / 256, TILE_STAGES);
#define GLU_TILE(NJ, TH) k_tile_glu<NJ, 256, TH><<<dim3(E, (ff + 128 / TH - 1) / (128 / TH)), 256, tile_smem<MK_FP4, NJ, 256, TH>(H), st>>>(Lg, Lu, xq_src, xs_src, Kt, e->pair_off, e->pair_list, e->h_all, ns_g)
#define DOWN_TILE(NJ, TH) k_tile_down<NJ, 256, TH><<<dim3(E, (H + 128 / TH - 1) / (128 / TH)), 256, tile_smem<MK_FP4, NJ, 256, TH>(ff), st>>>(Ld, e->hq, e->hs, e->pair_off, e->pair_list, e->o_all, ns_d)
                if (tile_w) { if (nj == 1) GLU_TILE(1, 1); else if (nj == 2) GLU_TILE(2, 1); else if (nj == 4) GLU_TILE(4, 1); else GLU_TILE(4, 2); }
                else k_glu_grouped<<<dim3(E, (ff + MMA_ROWS - 1) / MMA_ROWS), 256, gemm_smem(H), st>>>(Lg, Lu, xq_src, xs_src, Kt, e->pair_off, e->pair_list, e->h_all);
                launches++;
                k_quant_rows<<<P, 128, 0, st>>>(e->h_all, ff, e->hq, e->hs); launches++;
                if (tile_w) { if (nj == 1) DOWN_TILE(1, 1); else if (nj == 2) DOWN_TILE(2, 1); else if (nj == 4) DOWN_TILE(4, 1); else DOWN_TILE(4, 2); }
#undef GLU_TILE
#undef DOWN_TILE
                else k_down_grouped<<<dim3(E, (H + MMA_ROWS - 1) / MMA_ROWS), 256, gemm_smem(ff), st>>>(Ld, e->hq, e->hs, e->pair_off, e->pair_list, e->o_all);
                launches++;
            }
            }
            const float* o_src = e->o_all;
            if (a2a) {
                // combine: every served pair's output row back to the rank that owns the row, then into pair order
                EpState* q = e->ep;
                NcclApi& nc = nccl_api();
                nc.GroupStart();
                for (int r = 0; r < W; ++r) {
                    const size_t so = a2a_soff[r], sn = a2a_soff[r + 1] - a2a_soff[r], ro = a2a_roff[r], rn = a2a_roff[r + 1] - a2a_roff[r];
                    if (rn) nc.Send(e->o_all + ro * H, rn * H, NcclApi::Float32, r, q->comm, st);
                    if (sn) nc.Recv(q->o_back + so * H, sn * H, NcclApi::Float32, r, q->comm, st);
                }
                nc.GroupEnd();
                k_ep_unsort<<<(unsigned)(((size_t)R * K * (H / 4) + 255) / 256), 256, 0, st>>>(q->o_back, q->own_list, R * K, H, q->o_mine);
                launches += 2;
                o_src = q->o_mine;
            } else if (p2r) {
                // every served pair's output row straight into its owner's region, every rank told, and this rank's rows complete
                // once every rank has told it (bounded wait)
                EpState* q = e->ep;
                k_ep_scatter_rows<<<P, 256, 0, st>>>(e->o_all, ids_src, R * K, E / W, q->rank, H, (unsigned char* const*)q->peer_dev, q->off_o + (size_t)il * q->o_layer);
                k_ep_signal<<<W, 32, 0, st>>>((unsigned char* const*)q->peer_dev, q->off_of + ((size_t)il * 8 + q->rank) * 4, (const unsigned*)q->seq);
                k_ep_wait<<<1, 32, 0, st>>>((const unsigned*)(q->region + q->off_of + (size_t)il * 8 * 4), W, (const unsigned*)q->seq, e->err);
                launches += 3;
                o_src = (const float*)(q->region + q->off_o + (size_t)il * q->o_layer);
            } else if (e->ep) {
                nccl_api().ReduceScatter(e->o_all, e->ep->o_mine, (size_t)R * K * H, NcclApi::Float32, NcclApi::Sum, e->ep->comm, st);
                launches++;
                o_src = e->ep->o_mine;
            }
            k_shared_act_rows<<<R, 128, 0, st>>>(e->sg, e->su, d.shared_ff, e->sq, e->ss); launches++;
            if (L.shared4[2].nib) gemm_fp4d(L.shared4[2], e->sq, e->ss, e->shd, R, L.has_shared_s[2], L.shared_s[2]);
            else gemm(L.shared_down, e->sq, e->ss, e->shd, H, 0);
            const size_t total = (size_t)R * H;
            k_moe_finish_rows<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(e->x, H, o_src, wts, K, e->shd, e->shlogit, total); launches++;
        }
    }
    // LM head on each sequence's last row
    const float* xl = e->x;
    if (n_tok > 1) { k_gather_last<<<n_seq, 256, 0, st>>>(e->x, H, n_tok, e->xlast); launches++; xl = e->xlast; }
    if (n_seq > 1) {
        // several sequences: one pass over the output matrix for all of them
        k_norm_quant<<<n_seq, 256, smem_nq, st>>>(xl, m->output_norm, H, d.rms_eps, nullptr, e->xq, e->xs); launches++;
        if (m->output4.nib) gemm_fp4d(m->output4, e->xq, e->xs, e->logits, n_seq, m->has_output_s, m->output_s);
        else gemm_n(m->output, e->xq, e->xs, e->logits, d.n_vocab, 0, n_seq);
    } else if (m->output4.nib) {
        k_norm_quant<<<1, 256, smem_nq, st>>>(xl, m->output_norm, H, d.rms_eps, nullptr, e->xq, e->xs); launches++;
        gemm_fp4d(m->output4, e->xq, e->xs, e->logits, 1, m->has_output_s, m->output_s);
    } else {
        InProj hp{};
        hp.x = xl; hp.x_stride = H; hp.norm_w = m->output_norm; hp.eps = d.rms_eps; hp.n_embd = H;
        hp.nq = 1; hp.q[0] = m->output; hp.qout[0] = e->logits; hp.qstride[0] = d.n_vocab; hp.exact = c->exact; hp.tl_slot = -1;
        {
            const int pass_in = 2 * (32 >> lanes_shift(H / 32));
            int gx = std::max(1, std::min(sms, ((int)d.n_vocab + 2 * NWG - 1) / (2 * NWG)));
            int per_warp = ((int)d.n_vocab + gx * NWG - 1) / (gx * NWG) + 1;
            hp.br = std::min(std::max(32 / pass_in, 1) * pass_in, (per_warp + pass_in - 1) / pass_in * pass_in);
            const int cap = (int)(((SMEM_BUDGET - 256 - (size_t)H * 5 - (size_t)(H / 32) * 4 - (c->exact ? 32 * 33 * 4 : 0) - 64) / (NWG * 4) - CONV_CAP * 8) / (H / 32 + 1));
            hp.br = std::max(pass_in, std::min(hp.br, cap / pass_in * pass_in));
            set_smem((const void*)k_in_proj, 200 * 1024);
            k_in_proj<<<dim3(gx, n_seq), TPB, in_proj_smem(H, c->exact, hp.br), st>>>(hp); launches++;
        }
    }
    k_argmax_partial<<<dim3(ARGMAX_PARTS, n_seq), 256, 0, st>>>(e->logits, d.n_vocab, e->arg_v, e->arg_i); launches++;
    if (n_tok > 1) { k_advance_pos<<<(n_seq + 127) / 128, 128, 0, st>>>(e->pos, n_seq, n_tok - 1); launches++; }
    k_argmax_advance<<<n_seq, 32, 0, st>>>(e->arg_v, e->arg_i, ARGMAX_PARTS, e->tokens, e->pos, e->next, e->history, (int)e->history_cap, e->step_counter, n_seq);
    launches++;
    return launches;
}

static int engine_create(itb_model* m, uint32_t n_ctx, uint32_t n_seq, int world, itb_engine** out, uint32_t rows_cap = 0) {
    *out = nullptr;
    itb_ctx* c = m->c;
    if (!finalize(m)) return 1;
    if (n_seq == 0 || n_ctx == 0) { itb_fail_msg(c, "engine: n_seq and n_ctx must be positive"); return 1; }
    if (world == 1 && m->expert_hi && (m->expert_lo != 0 || m->expert_hi != m->d.n_expert)) {
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
    e->R = std::max<uint32_t>(n_seq, getenv("ITB_ROWS") ? (uint32_t)atoi(getenv("ITB_ROWS")) : 512u);
    if (rows_cap) e->R = std::max<uint32_t>(n_seq, std::min<uint32_t>(e->R, rows_cap));   // tiered: a pass may not need more experts than the pool holds
    if (m->offloaded && !rows_cap) { itb_fail_msg(c, "engine: this model's experts are in host memory; use the tiered engine"); return 1; }
    const size_t R = e->R, K = d.n_expert_used, W = (size_t)world;   // W: ranks whose pairs the expert buffers hold
    const size_t n_parts = std::max<size_t>(B * d.n_head * e->n_split, R * d.n_head * e->n_split_rows);
    bool ok = dalloc(E, &e->kslab, (size_t)e->n_attn * B * n_ctx * kvd) && dalloc(E, &e->vslab, (size_t)e->n_attn * B * n_ctx * kvd) &&
              dalloc(E, &e->conv_state, (size_t)e->n_rec * B * cd * (d.ssm_d_conv - 1)) &&
              dalloc(E, &e->ssm_state, (size_t)e->n_rec * B * d.ssm_dt_rank * d.ssm_d_state * d.ssm_d_state) &&
              dalloc(E, &e->pos, B) && dalloc(E, &e->npos, R) && dalloc(E, &e->tokens, B) && dalloc(E, &e->next, B) && dalloc(E, &e->x, R * H) &&
              dalloc(E, &e->qkvc, R * cd) && dalloc(E, &e->z, R * vd) && dalloc(E, &e->alpha, R * d.ssm_dt_rank) &&
              dalloc(E, &e->beta, R * d.ssm_dt_rank) && dalloc(E, &e->qg, R * 2 * qd) &&
              dalloc(E, &e->kbuf, R * kvd) && dalloc(E, &e->vbuf, R * kvd) && dalloc(E, &e->qn, R * qd) && dalloc(E, &e->gate, R * qd) &&
              dalloc(E, &e->part_acc, n_parts * d.head_dim) && dalloc(E, &e->part_ml, n_parts * 2) && dalloc(E, &e->router, R * d.n_expert) &&
              dalloc(E, &e->shlogit, R) && dalloc(E, &e->sg, R * d.shared_ff) && dalloc(E, &e->su, R * d.shared_ff) &&
              dalloc(E, &e->logits, B * d.n_vocab) && dalloc(E, &e->xq, R * H) && dalloc(E, &e->xs, R * H / 32) &&
              dalloc(E, &e->route_ids, (size_t)d.n_layer * R * K) && dalloc(E, &e->route_w, (size_t)d.n_layer * R * K) &&
              dalloc(E, &e->step_counter, B) && dalloc(E, &e->err, 1) && dalloc(E, &e->arg_v, B * ARGMAX_PARTS) && dalloc(E, &e->arg_i, B * ARGMAX_PARTS) &&
              dalloc(E, &e->aq, R * std::max(vd, qd)) && dalloc(E, &e->as, R * std::max(vd, qd) / 32) &&
              dalloc(E, &e->hq, W * R * K * d.expert_ff) && dalloc(E, &e->hs, W * R * K * d.expert_ff / 32) &&
              dalloc(E, &e->sq, R * d.shared_ff) && dalloc(E, &e->ss, R * d.shared_ff / 32) &&
              dalloc(E, &e->xn, R * H) && dalloc(E, &e->qh, R * key_dim) && dalloc(E, &e->kh, R * key_dim) && dalloc(E, &e->vh, R * vd) &&
              dalloc(E, &e->gb, R * d.ssm_dt_rank * 2) && dalloc(E, &e->core, R * vd) && dalloc(E, &e->xlast, B * H) &&
              dalloc(E, &e->h_all, W * R * K * d.expert_ff) && dalloc(E, &e->o_all, W * R * K * H) && dalloc(E, &e->shd, R * H) &&
              dalloc(E, &e->qkvc2, R * cd) && dalloc(E, &e->pair_off, (size_t)d.n_expert + 1) && dalloc(E, &e->pair_list, W * R * K);
    if (!ok) { for (void* p : e->allocs) cudaFree(p); return 1; }
    e->host_pos.assign(B, 0);
    cudaEventCreate(&e->ev0); cudaEventCreate(&e->ev1);
    cudaMemsetAsync(e->h_all, 0, W * R * K * d.expert_ff * sizeof(float), c->stream);   // pairs served elsewhere are quantised too: keep them finite
    if (world > 1) {
        e->ep = new EpState();
        e->ep->world = world;
        if (!(dalloc(E, &e->ep->gxq, W * R * H) && dalloc(E, &e->ep->gxs, W * R * H / 32) && dalloc(E, &e->ep->gids, W * R * K) &&
              dalloc(E, &e->ep->o_mine, R * K * H) && dalloc(E, &e->ep->grouter, W * d.n_expert) && dalloc(E, &e->ep->gw, W * R * K) &&
              dalloc(E, &e->ep->agree_dev, W + 1) && cudaMallocHost(&e->ep->agree_host, (W + 1) * 4) == cudaSuccess)) { for (void* p : e->allocs) cudaFree(p); delete e->ep; return 1; }
    }
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) { itb_fail_msg(c, "engine: device error during set-up"); return 1; }
    if (exact_attention_ok(E) && !ensure_scores(E, B)) { for (void* p : e->allocs) cudaFree(p); return 1; }
    *out = e.release();
    return 0;
}

extern "C" int itb_engine_create(itb_model* m, uint32_t n_ctx, uint32_t n_seq, itb_engine** out) { return engine_create(m, n_ctx, n_seq, 1, out); }

extern "C" int itb_engine_create_tiered(itb_model* m, uint32_t n_ctx, uint32_t n_seq, uint32_t capacity, itb_engine** out) {
    *out = nullptr;
    itb_ctx* c = m->c;
    const itb_model_dims& d = m->d;
    if (!m->offloaded) { itb_fail_msg(c, "tiered engine: call itb_model_offload_experts first"); return 1; }
    const size_t n_keys = (size_t)d.n_layer * d.n_expert;
    if (capacity < n_seq * d.n_expert_used) { itb_fail_msg(c, "tiered engine: the pool must hold at least n_seq * n_expert_used experts"); return 1; }
    capacity = (uint32_t)std::min<size_t>(capacity, n_keys);
    if (engine_create(m, n_ctx, n_seq, 1, out, std::max<uint32_t>(1, capacity / d.n_expert_used))) return 1;
    itb_engine* e = *out;
    TierState* t = new TierState();
    e->tier = t;
    t->capacity = capacity;
    t->g = new GClock(capacity, n_keys);
    t->dirty.assign(d.n_layer, 1);
    bool ok = true;
    for (int k = 0; k < 3; ++k) {
        const itb_model::HostStack& h = m->host_experts[0][k];
        ok = ok && dalloc(e, &t->pool_nib[k], (size_t)capacity * h.nib_per) && dalloc(e, &t->pool_sc[k], (size_t)capacity * h.sc_per) &&
             dalloc(e, &t->pool_s2[k], (size_t)capacity);
    }
    ok = ok && dalloc(e, &t->slot_map, n_keys);
    ok = ok && cudaMallocHost(&t->slot_map_host, n_keys * 4) == cudaSuccess && cudaMallocHost(&t->ids_host, (size_t)e->R * d.n_expert_used * 4) == cudaSuccess &&
         cudaMallocHost(&t->s2_stage, (size_t)capacity * 3 * 4) == cudaSuccess;
    t->guessed.assign(capacity, 0);
    t->s2_guess_cap = (size_t)e->R * 16 * 3;
    t->prefetch_k = getenv("ITB_TIER_PREFETCH") ? std::max(0, atoi(getenv("ITB_TIER_PREFETCH"))) : 0;
    if (t->prefetch_k > 0) {
        ok = ok && dalloc(e, &t->guess_dev, (size_t)e->R * 16) && dalloc(e, &t->guess_w, (size_t)e->R * 16) && dalloc(e, &t->guess_logits, (size_t)e->R * d.n_expert) &&
             cudaMallocHost(&t->guess_host, (size_t)e->R * 16 * 4) == cudaSuccess && cudaMallocHost(&t->s2_guess, (size_t)e->R * 16 * 3 * 4) == cudaSuccess &&
             cudaStreamCreateWithFlags(&t->stream2, cudaStreamNonBlocking) == cudaSuccess && cudaEventCreateWithFlags(&t->ev_fetch, cudaEventDisableTiming) == cudaSuccess;
    }
    if (!ok) { itb_fail_msg(c, "tiered engine: out of memory"); itb_engine_destroy(e); *out = nullptr; return 1; }
    for (size_t i = 0; i < n_keys; ++i) t->slot_map_host[i] = -1;
    return 0;
}
// The reference's TierCounters (src/ops/mod.rs:360-401), as far as they exist here: what this engine's expert tier did since it
// was created, and the device's memory at the snapshot. Fields of the reference that describe its file tier (read_us,
// upload_us, writes_us, picks_copy_us, oversubscribed) have no counterpart: the lower tier here is pinned host memory.
extern "C" int itb_tier_counters(itb_engine* e, itb_tier_counters_t* o) {
    memset(o, 0, sizeof *o);
    size_t fr = 0, tot = 0;
    if (cudaMemGetInfo(&fr, &tot) == cudaSuccess) { o->vram_free = fr; o->vram_total = tot; }
    itb_ctx* c = e->c;
    o->mirrors = c->mirrors.size(); o->mirror_bytes = c->mirror_bytes; o->weight_bytes = e->m->bytes;
    {
        const itb_model_dims& d = e->m->d;
        size_t n_attn = 0;
        for (const DevLayer& L : e->m->layers) n_attn += L.recurrent ? 0 : 1;
        o->kv_bytes = n_attn * (size_t)e->B * e->n_ctx * d.head_dim * d.n_head_kv * 2 * 2;
    }
    if (e->tier) {
        const TierState* t = e->tier;
        size_t slot_bytes = 0;
        for (int k = 0; k < 3; ++k) slot_bytes += e->m->host_experts[0][k].nib_per + e->m->host_experts[0][k].sc_per + 4;
        o->fetched = t->fetched; o->fetch_bytes = t->bytes_moved; o->picks_wait_us = t->picks_wait_us; o->prefetch_reads = t->prefetch_reads;
        o->prefetch_used = t->prefetch_used; o->lookups = t->lookups; o->host_reads = t->host_reads; o->slot_bytes = slot_bytes; o->slots = t->capacity;
        o->pool_bytes = slot_bytes * t->capacity;
    }
    o->resident_bytes = o->weight_bytes + o->kv_bytes + o->mirror_bytes + o->pool_bytes;
    return 0;
}
// hits, misses, evictions, bytes copied host -> HBM since the engine was created
extern "C" void itb_engine_tier_stats(itb_engine* e, uint64_t* out4) {
    out4[0] = out4[1] = out4[2] = out4[3] = 0;
    if (!e->tier) return;
    out4[0] = e->tier->g->hits; out4[1] = e->tier->g->misses; out4[2] = e->tier->g->evictions; out4[3] = e->tier->bytes_moved;
}
// The residency policy on its own (host only, usable without a device): see itb_tier.h.
extern "C" void* itb_gclock_create(uint32_t capacity, uint32_t n_keys) { return capacity && n_keys ? new GClock(capacity, n_keys) : nullptr; }
extern "C" void itb_gclock_destroy(void* g) { delete (GClock*)g; }
extern "C" void itb_gclock_next_pass(void* g) { ((GClock*)g)->next_pass(); }
extern "C" int itb_gclock_touch(void* g, int64_t key, int* hit, int64_t* evicted) {
    GClock* q = (GClock*)g;
    if (key < 0 || (size_t)key >= q->slot_of.size()) return -2;
    bool h = false;
    const int s = q->touch(key, &h, evicted);
    *hit = h ? 1 : 0;
    return s;
}

extern "C" int itb_ep_unique_id(uint8_t* out128) {
    NcclApi& nc = nccl_api();
    if (!nc.ok) return 1;
    NcclApi::UniqueId id;
    if (nc.GetUniqueId(&id) != 0) return 1;
    memcpy(out128, id.internal, 128);
    return 0;
}

extern "C" int itb_engine_create_ep(itb_model* m, uint32_t n_ctx, uint32_t n_seq, const uint8_t* unique_id128, int rank, int world, itb_engine** out) {
    *out = nullptr;
    itb_ctx* c = m->c;
    NcclApi& nc = nccl_api();
    if (!nc.ok) { itb_fail_msg(c, "expert-parallel engine: libnccl.so.2 is not loadable in this process"); return 1; }
    const uint32_t E = m->d.n_expert;
    if (world < 2 || rank < 0 || rank >= world || E % (uint32_t)world) { itb_fail_msg(c, "expert-parallel engine: world must be >= 2 and divide n_expert"); return 1; }
    const uint32_t per = E / (uint32_t)world;
    if (m->expert_lo != per * (uint32_t)rank || m->expert_hi != per * (uint32_t)(rank + 1)) {
        itb_fail_msg(c, "expert-parallel engine: the model must hold exactly this rank's expert range"); return 1;
    }
    if (engine_create(m, n_ctx, n_seq, world, out)) return 1;
    itb_engine* e = *out;
    e->ep->rank = rank;
    NcclApi::UniqueId id;
    memcpy(id.internal, unique_id128, 128);
    int rc = nc.CommInitRank(&e->ep->comm, world, id, rank);
    if (rc != 0) {
        itb_fail_msg(c, (std::string("expert-parallel engine: ncclCommInitRank failed: ") + (nc.GetErrorString ? nc.GetErrorString(rc) : "?")).c_str());
        itb_engine_destroy(e); *out = nullptr; return 1;
    }
    ep_p2p_setup(e);
    return 0;
}

extern "C" int itb_engine_ep_transport(itb_engine* e) { return !e->ep ? 0 : (e->ep->p2p || e->ep->p2p_rows) ? 2 : 1; }

static void drop_graph(itb_engine* e) {
    if (e->exec) cudaGraphExecDestroy(e->exec);
    if (e->graph) cudaGraphDestroy(e->graph);
    e->exec = nullptr; e->graph = nullptr;
}

extern "C" void itb_engine_destroy(itb_engine* e) {
    if (!e) return;
    cudaStreamSynchronize(e->c->stream);
    drop_graph(e);
    if (e->ep) {
        EpState* q = e->ep;
        if (q->comm && !q->broken) nccl_api().CommDestroy(q->comm);
        cudaFreeHost(q->agree_host);
        for (int r = 0; r < q->world && r < 8; ++r) if (r != q->rank && q->peer[r]) cudaIpcCloseMemHandle(q->peer[r]);
        cudaFree(q->region); cudaFree(q->seq); cudaFree(q->peer_dev);
        cudaFree(q->sxq); cudaFree(q->sxs); cudaFree(q->sids); cudaFree(q->rxq); cudaFree(q->rxs); cudaFree(q->rids); cudaFree(q->o_back); cudaFree(q->owner);
        cudaFree(q->own_off); cudaFree(q->own_list); cudaFree(q->cnt_dev); if (q->cnt_host) cudaFreeHost(q->cnt_host);
        delete q; e->ep = nullptr;
    }
    if (e->tier) {
        TierState* t = e->tier;
        if (t->stream2) { cudaStreamSynchronize(t->stream2); cudaStreamDestroy(t->stream2); }
        if (t->ev_fetch) cudaEventDestroy(t->ev_fetch);
        cudaFreeHost(t->slot_map_host); cudaFreeHost(t->ids_host); cudaFreeHost(t->s2_stage); cudaFreeHost(t->guess_host); cudaFreeHost(t->s2_guess);
        delete t->g; delete t; e->tier = nullptr;
    }
    for (void* p : e->allocs) cudaFree(p);
    cudaFree(e->history); cudaFree(e->prompt); cudaFree(e->scores); cudaFree(e->gdn_scratch);
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
// Engine::checkpoint / restore (src/engine/mod.rs:255-294): the positions plus the recurrent state (conv windows and
// delta-rule state of every sequence). The KV cache needs no copy: positions past the checkpoint are no longer part of
// the sequence and the next tokens overwrite them. Layout: u32 magic, u32 n_seq, u32 pos[n_seq], conv f32[], ssm f32[].
static size_t ckpt_conv_floats(const itb_engine* e) {
    const itb_model_dims& d = e->m->d;
    const size_t cd = 2 * (size_t)d.ssm_d_state * d.ssm_n_group + d.ssm_d_inner;
    return (size_t)e->n_rec * e->B * cd * (d.ssm_d_conv - 1);
}
static size_t ckpt_ssm_floats(const itb_engine* e) {
    const itb_model_dims& d = e->m->d;
    return (size_t)e->n_rec * e->B * d.ssm_dt_rank * d.ssm_d_state * d.ssm_d_state;
}
extern "C" size_t itb_engine_checkpoint_bytes(itb_engine* e) { return 8 + (size_t)e->B * 4 + (ckpt_conv_floats(e) + ckpt_ssm_floats(e)) * 4; }
extern "C" int itb_engine_checkpoint(itb_engine* e, void* out, size_t cap) {
    itb_ctx* c = e->c;
    if (cap < itb_engine_checkpoint_bytes(e)) { itb_fail_msg(c, "checkpoint: buffer too small"); return 1; }
    uint32_t* h = (uint32_t*)out;
    h[0] = 0x4b435449u; h[1] = e->B;
    for (uint32_t b = 0; b < e->B; ++b) h[2 + b] = e->host_pos[b];
    float* f = (float*)(h + 2 + e->B);
    ITB_CUDA_RET(c, cudaMemcpyAsync(f, e->conv_state, ckpt_conv_floats(e) * 4, cudaMemcpyDeviceToHost, c->stream), 1);
    ITB_CUDA_RET(c, cudaMemcpyAsync(f + ckpt_conv_floats(e), e->ssm_state, ckpt_ssm_floats(e) * 4, cudaMemcpyDeviceToHost, c->stream), 1);
    ITB_CUDA_RET(c, cudaStreamSynchronize(c->stream), 1);
    return 0;
}
extern "C" int itb_engine_restore(itb_engine* e, const void* data, size_t bytes) {
    itb_ctx* c = e->c;
    const uint32_t* h = (const uint32_t*)data;
    if (bytes != itb_engine_checkpoint_bytes(e) || h[0] != 0x4b435449u || h[1] != e->B) { itb_fail_msg(c, "restore: not a checkpoint of an engine of this shape"); return 1; }
    for (uint32_t b = 0; b < e->B; ++b)
        if (h[2 + b] > e->n_ctx) { itb_fail_msg(c, "restore: the checkpoint stands past this engine's context"); return 1; }   // src/engine/mod.rs:276-281
    const float* f = (const float*)(h + 2 + e->B);
    ITB_CUDA_RET(c, cudaMemcpyAsync(e->pos, h + 2, (size_t)e->B * 4, cudaMemcpyHostToDevice, c->stream), 1);
    ITB_CUDA_RET(c, cudaMemcpyAsync(e->conv_state, f, ckpt_conv_floats(e) * 4, cudaMemcpyHostToDevice, c->stream), 1);
    ITB_CUDA_RET(c, cudaMemcpyAsync(e->ssm_state, f + ckpt_conv_floats(e), ckpt_ssm_floats(e) * 4, cudaMemcpyHostToDevice, c->stream), 1);
    ITB_CUDA_RET(c, cudaStreamSynchronize(c->stream), 1);
    for (uint32_t b = 0; b < e->B; ++b) e->host_pos[b] = h[2 + b];
    return 0;
}
extern "C" uint32_t itb_engine_pos(itb_engine* e, uint32_t seq) { return seq < e->B ? e->host_pos[seq] : 0; }
extern "C" float itb_engine_last_ms(itb_engine* e) { return e->last_ms; }
extern "C" uint64_t itb_engine_launches_per_step(itb_engine* e) { return e->launches_per_step; }

// ---------------------------------------------------------------------------------------------------------
// The one-kernel decode step. Decides once per engine whether the shape fits (single sequence, plain engine, every row a
// whole number of 16-byte scale spans, shared memory for at least two ring slots each); builds the stage table -- the same
// dependent stages enqueue_step launches as kernels -- and the shared-memory layout. ITB_MEGA=0 keeps the per-kernel step.
static bool mega_prepare(itb_engine* e) {
    if (e->mega >= 0) return e->mega == 1;
    e->mega = 0;
    itb_model* m = e->m; itb_ctx* c = e->c;
    const itb_model_dims& d = m->d;
    auto no = [&](const char* why) { e->mega_why = why; return false; };
    if (!(getenv("ITB_MEGA") && atoi(getenv("ITB_MEGA")) == 1)) return no("not asked for (ITB_MEGA=1 selects the one-kernel step)");
    if (e->B != 1 || e->ep || e->tier || e->m->dense_fp4) return no("single-sequence plain engines only");
    const int H = d.n_embd, sk = d.ssm_d_state, n_k = d.ssm_n_group, n_v = d.ssm_dt_rank;
    const int key_dim = sk * n_k, vd = d.ssm_d_inner, cd = 2 * key_dim + vd;
    const int qd = d.head_dim * d.n_head, kvd = d.head_dim * d.n_head_kv, ff = d.expert_ff, sff = d.shared_ff, K = d.n_expert_used;
    if (H % 256 || vd % 256 || qd % 256 || ff % 256 || sff % 256 || H > 8192) return no("a row is not a whole number of 256-element spans");
    if (d.n_head / d.n_head_kv > 8 || (int)d.head_dim > MG_CT || d.ssm_d_conv > 8) return no("attention group or conv width beyond the kernel");
    if (((d.n_expert + 31) / 32) * K > MOE_CAND) return no("too many routing candidates");
    int dev = 0, coop = 0, sms = c->sm_count;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (!coop) return no("no cooperative launch on this device");
    const int G = sms;
    auto per_block = [&](int n) { return (n + G - 1) / G + 1; };
    const int gdn_rows = per_block(n_v * sk), down_rows = per_block(H);
    if (gdn_rows > MG_CT || (gdn_rows + sk - 1) / sk + 1 > MG_MAX_LOCAL_HEADS) return no("too many delta-rule rows per block");
    // shared-memory layout
    const int nmax = std::max(H, std::max(vd, qd));
    auto up = [](size_t v) { return (v + 127) & ~(size_t)127; };
    const size_t act = up(std::max<size_t>((size_t)nmax + (size_t)nmax / 8 + (size_t)H * 4,
                                           (size_t)K * ff + (size_t)K * ff / 8 + sff + sff / 8 + (size_t)down_rows * (K + 1) * 4));
    const int max_nt = std::max({H / 16, vd / 32, qd / 32, ff / 16, sff / 32});
    const int group = d.n_head / d.n_head_kv, parts = MG_NW / group;
    size_t terms_need = std::max<size_t>({(size_t)gdn_rows * (sk + 1) + (size_t)MG_MAX_LOCAL_HEADS * (2 * sk + 2),
                                          (size_t)((d.n_expert + 31) & ~31u) + 2 * MOE_CAND,
                                          (size_t)group * parts * (2 + d.head_dim), (size_t)d.head_dim});
    int tw = std::max(560, 2 * (max_nt + 1));   // a warp holds at least two rows' terms
    while ((size_t)MG_NW * tw < terms_need) tw += 16;
    const size_t terms = up((size_t)MG_NW * tw * 4);
    size_t row_max = std::max<size_t>({(size_t)H * 4, (size_t)H + H / 16, (size_t)vd + vd / 16, (size_t)qd + qd / 16, (size_t)sff + sff / 16, (size_t)sk * 4});
    const size_t slot_b = up(std::max<size_t>(32 * ((size_t)H / 2 + H / 16), (size_t)down_rows * (ff / 2 + ff / 16)));
    cudaFuncAttributes fa{};
    if (cudaFuncGetAttributes(&fa, (const void*)k_mega) != cudaSuccess) return no("cannot query the kernel");
    int max_optin = 0;
    cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const long budget = (long)max_optin - (long)fa.sharedSizeBytes - 1024;
    const int ns_b = 2;
    size_t slot_a = up(std::max<size_t>(row_max, 16 * ((size_t)H + H / 16)));
    long left = budget - (long)(act + terms + ns_b * slot_b);
    int ns_a = (int)(left / (long)slot_a);
    while (ns_a < 2 && slot_a / 2 >= up(row_max)) { slot_a = up(slot_a / 2); ns_a = (int)(left / (long)slot_a); }
    if (left <= 0 || ns_a < 2) return no("not enough shared memory for the rings");
    ns_a = std::min(ns_a, MG_MAX_SLOTS);
    const size_t smem = act + terms + ns_a * slot_a + ns_b * slot_b;
    if (cudaFuncSetAttribute((const void*)k_mega, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { cudaGetLastError(); return no("cannot raise the shared-memory limit"); }
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_mega, MG_THREADS, smem) != cudaSuccess || occ < 1) { cudaGetLastError(); return no("the kernel does not fit an SM"); }
    // buffers the step needs beyond the engine's
    const int n_split = std::max(1, G / (int)d.n_head_kv);
    if (!dalloc(e, &e->mega_sync, 4) || !dalloc(e, &e->mega_core, (size_t)vd) || !dalloc(e, &e->mega_part, (size_t)d.n_head * n_split * (d.head_dim + 2)) ||
        !dalloc(e, &e->mega_argv, (size_t)G) || !dalloc(e, &e->mega_argi, (size_t)G)) return no("out of device memory");
    // the stage table
    std::vector<MStage> st;
    auto blank = [](int type) { MStage t; memset(&t, 0, sizeof t); t.type = type; return t; };
    st.push_back(blank(MS_EMBED));
    for (uint32_t il = 0; il < d.n_layer; ++il) {
        const DevLayer& L = m->layers[il];
        if (L.recurrent) {
            const int rs = e->slot_of[il];
            MStage a = blank(MS_ROWS);
            a.norm_w = L.attn_norm; a.nq = 2; a.q[0] = L.wqkv; a.qout[0] = e->qkvc; a.q[1] = L.wgate; a.qout[1] = e->z;
            a.nf = 2; a.f[0] = L.ssm_alpha; a.fout[0] = e->alpha; a.f[1] = L.ssm_beta; a.fout[1] = e->beta;
            a.conv_w = L.conv1d; a.conv_state = e->conv_state + (size_t)rs * cd * (d.ssm_d_conv - 1);
            st.push_back(a);
            MStage g = blank(MS_GDN);
            g.ssm_a = L.ssm_a; g.dt_bias = L.dt_bias; g.state = e->ssm_state + (size_t)rs * n_v * sk * sk;
            st.push_back(g);
            MStage o = blank(MS_OUT);
            o.ssm_norm = L.ssm_norm; o.w = L.ssm_out;
            st.push_back(o);
        } else {
            const int as = e->slot_of[il];
            MStage a = blank(MS_ROWS);
            a.norm_w = L.attn_norm; a.nq = 3; a.q[0] = L.wq; a.qout[0] = e->qg; a.q[1] = L.wk; a.qout[1] = e->kbuf; a.q[2] = L.wv; a.qout[2] = e->vbuf;
            st.push_back(a);
            MStage pr = blank(MS_ATTN_PREP);
            pr.q_norm = L.q_norm; pr.k_norm = L.k_norm;
            pr.kslab = e->kslab + (size_t)as * e->n_ctx * kvd; pr.vslab = e->vslab + (size_t)as * e->n_ctx * kvd;
            st.push_back(pr);
            MStage pa = blank(MS_ATTN_PART); pa.kslab = pr.kslab; pa.vslab = pr.vslab;
            st.push_back(pa);
            st.push_back(blank(MS_ATTN_COMB));
            MStage o = blank(MS_OUT);
            o.flags = MSF_OUT_ATTN; o.w = L.wo;
            st.push_back(o);
        }
        MStage f = blank(MS_ROWS);
        f.norm_w = L.ffn_norm; f.nq = 2; f.q[0] = L.shared_gate; f.qout[0] = e->sg; f.q[1] = L.shared_up; f.qout[1] = e->su;
        f.nf = 2; f.f[0] = L.gate_inp; f.fout[0] = e->router; f.f[1] = L.shared_gate_inp; f.fout[1] = e->shlogit;
        st.push_back(f);
        MStage gl = blank(MS_GLU);
        gl.norm_w = L.ffn_norm; gl.gate = L.gate; gl.up = L.up;
        gl.ids_out = e->route_ids + (size_t)il * e->R * K; gl.w_out = e->route_w + (size_t)il * e->R * K;
        st.push_back(gl);
        MStage dn = blank(MS_DOWN);
        dn.down = L.down; dn.shared_down = L.shared_down; dn.ids_out = gl.ids_out; dn.w_out = gl.w_out;
        st.push_back(dn);
    }
    MStage hd = blank(MS_ROWS);
    hd.flags = MSF_ARGMAX; hd.norm_w = m->output_norm; hd.nq = 1; hd.q[0] = m->output; hd.qout[0] = e->logits;
    st.push_back(hd);
    st.push_back(blank(MS_ADVANCE));
    if (!dalloc(e, &e->mega_stages, st.size())) return no("out of device memory");
    if (cudaMemcpyAsync(e->mega_stages, st.data(), st.size() * sizeof(MStage), cudaMemcpyHostToDevice, c->stream) != cudaSuccess ||
        cudaStreamSynchronize(c->stream) != cudaSuccess) return no("cannot upload the stage table");
    MegaParams& p = e->mp;
    memset(&p, 0, sizeof p);
    p.stages = e->mega_stages; p.n_stages = (int)st.size();
    p.H = H; p.n_vocab = d.n_vocab; p.cd = cd; p.vd = vd; p.key_dim = key_dim; p.sk = sk; p.n_k = n_k; p.n_v = n_v; p.conv_kernel = d.ssm_d_conv;
    p.qd = qd; p.kvd = kvd; p.hd = d.head_dim; p.n_head = d.n_head; p.n_head_kv = d.n_head_kv; p.n_rot = d.n_rot; p.n_expert = d.n_expert;
    p.n_used = K; p.ff = ff; p.sff = sff; p.n_ctx = e->n_ctx; p.eps = d.rms_eps; p.theta = d.rope_theta; p.exact = c->exact; p.kv_bf16 = c->kv_bf16;
    p.tok_embd = m->tok_embd.w;
    p.x = e->x; p.qkvc = e->qkvc; p.z = e->z; p.alpha = e->alpha; p.beta = e->beta; p.core = e->mega_core; p.qg = e->qg; p.kbuf = e->kbuf; p.vbuf = e->vbuf;
    p.qn = e->qn; p.gate = e->gate; p.part_acc = e->mega_part; p.part_ml = e->mega_part + (size_t)d.n_head * n_split * d.head_dim;
    p.router = e->router; p.shlogit = e->shlogit; p.sg = e->sg; p.su = e->su; p.logits = e->logits;
    p.aq = e->aq; p.as = e->as; p.hq = e->hq; p.hs = e->hs; p.sq = e->sq; p.ss = e->ss;
    p.tokens = e->tokens; p.pos = e->pos; p.next = e->next; p.step_counter = e->step_counter;
    p.arg_v = e->mega_argv; p.arg_i = e->mega_argi;
    p.bar = e->mega_sync; p.done = e->mega_sync + 1; p.err = e->err;
    p.n_split = n_split;
    p.wait_ns = getenv("ITB_MEGA_WAIT_MS") ? (unsigned long long)std::max(1, atoi(getenv("ITB_MEGA_WAIT_MS"))) * 1000000ull : MG_WAIT_NS;
    p.test_stall = getenv("ITB_MEGA_TEST_STALL") ? atoi(getenv("ITB_MEGA_TEST_STALL")) : 0;
    p.off_act = 0; p.off_terms = (int)act; p.off_ring_a = (int)(act + terms); p.off_ring_b = (int)(act + terms + ns_a * slot_a);
    p.ns_a = ns_a; p.ns_b = ns_b; p.slot_a = (int)slot_a; p.slot_b = (int)slot_b; p.tw_floats = tw;
    e->mega_smem = smem; e->mega_grid = G;
    e->mega = 1;
    return true;
}
// One decode step as one cooperative launch (every block resident: the grid barriers need it).
static bool enqueue_mega(itb_engine* e, cudaStream_t st) {
    MegaParams& p = e->mp;
    p.history = e->history; p.history_cap = (int)e->history_cap;
    void* args[] = {&p};
    cudaError_t err = cudaLaunchCooperativeKernel((const void*)k_mega, dim3(e->mega_grid), dim3(MG_THREADS), args, e->mega_smem, st);
    if (err != cudaSuccess) return itb_fail(e->c, "engine: cooperative launch of the decode step", err);
    e->launches_per_step = 1;
    return true;
}

// 1: single-token decode steps of this engine run as the one persistent kernel; 0: as the chain of fused kernels, with the
// reason in `why`. Decides now if no step has run yet.
extern "C" int itb_engine_decode_path(itb_engine* e, char* why, size_t cap) {
    const bool mega = mega_prepare(e);
    if (why && cap) snprintf(why, cap, "%s", mega ? "one persistent kernel per step" : e->mega_why.c_str());
    return mega ? 1 : 0;
}

static bool ensure_graph(itb_engine* e) {
    if (e->exec) return true;
    itb_ctx* c = e->c;
    cudaStream_t st = c->stream;
    // one eager step's worth of attribute set-up happens inside enqueue_step; capture it once
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return itb_fail_msg(c, "engine: cannot begin capture");
    if (e->B == 1 && !e->tier && !e->m->dense_fp4) enqueue_step(e, st);   // expert-parallel engines too: the step gathers and scatters around its expert kernels
    else e->launches_per_step = enqueue_rows(e, st, (int)e->B, 1, e->tokens);
    cudaError_t err = cudaStreamEndCapture(st, &e->graph);
    if (err != cudaSuccess) return itb_fail(c, "engine: capture", err);
    err = cudaGraphInstantiate(&e->exec, e->graph, 0);
    if (err != cudaSuccess) return itb_fail(c, "engine: graph instantiate", err);
    return true;
}

// The one-kernel step's waits are bounded: a wait that ran out stores (stage << 8) | reason in the status word and every
// block returns. Turn it into the sticky error and put the grid barrier's counters back.
static bool check_flag(itb_engine* e) {
    if (e->mega != 1 && !e->c->exact && !(e->ep && (e->ep->p2p || e->ep->p2p_rows))) return true;
    int f = 0;
    if (cudaMemcpy(&f, e->err, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return itb_fail_msg(e->c, "engine: cannot read the device status word");
    if (f == EP_WAIT_FAIL) {
        cudaMemset(e->err, 0, 4);
        return itb_fail_msg(e->c, "expert-parallel engine: a peer's rows never arrived in this rank's memory (bounded wait ran out)");
    }
    if (f == F32S_FAIL) {
        cudaMemset(e->err, 0, 4);
        return itb_fail_msg(e->c, "engine: an F32 weight row never arrived in its shared-memory ring (bounded wait ran out)");
    }
    if (f) {
        cudaMemset(e->err, 0, 4); cudaMemset(e->mega_sync, 0, 16);
        static const char* const why[] = {"?", "weights never arrived in the ring", "a ring slot was never released", "a grid barrier was never completed",
                                          "the routing picks were never published", "copies in flight did not land", "shape"};
        const int r = f & 255;
        return itb_fail_msg(e->c, std::string("engine: the decode step gave up at stage ") + std::to_string(f >> 8) + ": " + why[r >= 1 && r <= 6 ? r : 0] + " (bounded wait ran out)");
    }
    return true;
}

// Expert-parallel engines: a rank that returned early would leave its peers waiting inside the layer's collectives with
// nothing to end them. So every entry point first validates and allocates locally, then all ranks exchange one flag
// (a one-int all-gather that every rank always enters) and go on only if every rank is ready; otherwise every rank
// returns an error and none enqueues anything. A failure after work was enqueued aborts the communicator.
static bool ep_agree(itb_engine* e, bool ok) {
    if (!e->ep) return ok;
    itb_ctx* c = e->c;
    EpState* p = e->ep;
    if (p->broken) return itb_fail_msg(c, "expert-parallel engine: the communicator was aborted after an earlier failure");
    const int W = p->world;
    p->agree_host[W] = ok ? 1 : 0;
    bool sent = cudaMemcpyAsync(p->agree_dev + W, p->agree_host + W, 4, cudaMemcpyHostToDevice, c->stream) == cudaSuccess &&
                nccl_api().AllGather(p->agree_dev + W, p->agree_dev, 1, NcclApi::Int32, p->comm, c->stream) == 0 &&
                cudaMemcpyAsync(p->agree_host, p->agree_dev, (size_t)W * 4, cudaMemcpyDeviceToHost, c->stream) == cudaSuccess &&
                cudaStreamSynchronize(c->stream) == cudaSuccess;
    if (!sent) return itb_fail_msg(c, "expert-parallel engine: the ranks could not exchange their ready flags");
    for (int r = 0; r < W; ++r)
        if (!p->agree_host[r]) {
            if (ok) itb_fail_msg(c, "expert-parallel engine: rank " + std::to_string(r) + " refused this call (see its error); nothing was run");
            return false;
        }
    return true;
}
static void ep_abort(itb_engine* e) {
    if (!e->ep || e->ep->broken || !e->ep->comm) return;
    if (nccl_api().CommAbort) nccl_api().CommAbort(e->ep->comm);
    e->ep->broken = true;
}

// src/model/qwen35.rs:866 (TokenOutOfRange): refused on the host, before any copy or launch.
static bool tokens_in_range(itb_engine* e, const uint32_t* tokens, size_t n) {
    for (size_t i = 0; i < n; ++i)
        if (tokens[i] >= e->m->d.n_vocab) return itb_fail_msg(e->c, "token id out of range");
    return true;
}

static bool steps_use_graph(const itb_engine* e) {
    // expert-parallel steps hold NCCL calls; they are captured like the rest unless ITB_EP_GRAPH=0 asks for eager launches
    static const bool ep_graph = !(getenv("ITB_EP_GRAPH") && atoi(getenv("ITB_EP_GRAPH")) == 0);
    return (!e->ep || ep_graph) && !e->tier && e->mega != 1;   // a tiered step talks to the host between layers; the one-kernel step is one launch already
}
// Everything about `steps` decode steps that can fail before a launch: room in the context, the captured graph.
static bool steps_ready(itb_engine* e, uint32_t steps) {
    for (uint32_t b = 0; b < e->B; ++b)
        if (e->host_pos[b] + steps > e->n_ctx) return itb_fail_msg(e->c, "context overflow: the step would write past n_ctx");  // src/model/qwen35.rs:984-990
    if (mega_prepare(e)) return true;
    return !steps_use_graph(e) || ensure_graph(e);
}
// The steps themselves; steps_ready (and, for expert-parallel engines, ep_agree) came first.
static bool run_steps(itb_engine* e, uint32_t steps, bool timed) {
    itb_ctx* c = e->c;
    const bool use_graph = steps_use_graph(e);
    if (timed) cudaEventRecord(e->ev0, c->stream);
    for (uint32_t s = 0; s < steps; ++s) {
        if (e->mega == 1) {
            if (!enqueue_mega(e, c->stream)) return false;
        } else if (use_graph) {
            cudaError_t err = cudaGraphLaunch(e->exec, c->stream);
            if (err != cudaSuccess) { ep_abort(e); return itb_fail(c, "engine: graph launch", err); }
        } else {
            if (e->B == 1 && !e->tier && !e->m->dense_fp4) enqueue_step(e, c->stream);
            else e->launches_per_step = enqueue_rows(e, c->stream, (int)e->B, 1, e->tokens);
            if (!c->error.empty()) { ep_abort(e); return false; }
        }
    }
    c->launches += (uint64_t)steps * e->launches_per_step;
    if (timed) cudaEventRecord(e->ev1, c->stream);
    for (uint32_t b = 0; b < e->B; ++b) e->host_pos[b] += steps;
    e->last_n_tok = 1;
    return true;
}

extern "C" int itb_engine_decode(itb_engine* e, const uint32_t* tokens, float* logits_out, uint32_t* next_out) {
    itb_ctx* c = e->c;
    cudaStream_t st = c->stream;
    if (!ep_agree(e, tokens_in_range(e, tokens, e->B) && steps_ready(e, 1))) return 1;
    ITB_CUDA_RET(c, cudaMemcpyAsync(e->tokens, tokens, e->B * 4, cudaMemcpyHostToDevice, st), 1);
    if (!run_steps(e, 1, true)) return 1;
    if (next_out) cudaMemcpyAsync(next_out, e->next, e->B * 4, cudaMemcpyDeviceToHost, st);
    if (logits_out) cudaMemcpyAsync(logits_out, e->logits, (size_t)e->B * e->m->d.n_vocab * 4, cudaMemcpyDeviceToHost, st);
    ITB_CUDA_RET(c, cudaStreamSynchronize(st), 1);
    cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1);
    return check_flag(e) ? 0 : 1;
}

extern "C" int itb_engine_decode_loop(itb_engine* e, const uint32_t* first, uint32_t steps, uint32_t* tokens_out) {
    itb_ctx* c = e->c;
    cudaStream_t st = c->stream;
    if (steps == 0) return 0;
    bool ok = tokens_in_range(e, first, e->B);
    if (ok && e->history_cap < steps) {
        cudaStreamSynchronize(st);
        drop_graph(e);  // the graph holds the history pointer
        cudaFree(e->history); e->history = nullptr; e->history_cap = 0;
        if (cudaMalloc(&e->history, (size_t)steps * e->B * 4) != cudaSuccess) { e->history = nullptr; ok = itb_fail_msg(c, "decode_loop: out of device memory for the token history"); }
        else e->history_cap = steps;
    }
    if (!ep_agree(e, ok && steps_ready(e, steps))) return 1;
    ITB_CUDA_RET(c, cudaMemcpyAsync(e->tokens, first, e->B * 4, cudaMemcpyHostToDevice, st), 1);
    cudaMemsetAsync(e->step_counter, 0, e->B * 4, st);
    if (!run_steps(e, steps, true)) return 1;
    if (tokens_out) cudaMemcpyAsync(tokens_out, e->history, (size_t)steps * e->B * 4, cudaMemcpyDeviceToHost, st);
    ITB_CUDA_RET(c, cudaStreamSynchronize(st), 1);
    cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1);
    return check_flag(e) ? 0 : 1;
}

// Prefill in multi-row passes: every sequence advances `chunk` tokens per pass (rows = n_seq * chunk <= R), each
// weight row read once per 32 rows. The arithmetic order per token is the decode path's, so the state left
// behind and the logits equal a token-by-token run (the reference asserts the same of its own backends,
// tests/qwen35.rs:94-139 there). ITB_PREFILL_STEPWISE=1 runs the old token-by-token loop (A/B and tests).
extern "C" int itb_engine_prefill(itb_engine* e, const uint32_t* tokens, size_t n, float* logits_out) {
    itb_ctx* c = e->c;
    cudaStream_t st = c->stream;
    if (n == 0) { itb_fail_msg(c, "prefill: no tokens supplied"); return 1; }
    bool ok = true;
    for (uint32_t b = 0; b < e->B && ok; ++b)
        if (e->host_pos[b] + n > e->n_ctx) ok = itb_fail_msg(c, "context overflow: the prompt would write past n_ctx");
    ok = ok && tokens_in_range(e, tokens, n * e->B);
    if (ok && e->prompt_cap < n * e->B) {
        cudaStreamSynchronize(st);
        cudaFree(e->prompt); e->prompt = nullptr; e->prompt_cap = 0;
        if (cudaMalloc(&e->prompt, n * e->B * 4) != cudaSuccess) { e->prompt = nullptr; ok = itb_fail_msg(c, "prefill: out of device memory for the prompt"); }
        else e->prompt_cap = n * e->B;
    }
    // exact mode: room for the scores of a whole pass (up to 2 GB; beyond that the pass keeps the split-K attention)
    if (ok && exact_attention_ok(e) && getenv("ITB_PREFILL_STEPWISE") == nullptr) {
        const size_t rows = e->B * std::min(std::max<size_t>(1, e->R / e->B), n);
        if (rows * e->m->d.n_head * e->n_ctx * 4 <= ((size_t)2 << 30)) ok = ensure_scores(e, rows);
    }
    // chunk-parallel delta rule: room for what its first kernel hands its second, for the largest pass of this call
    if (ok && (c->gdn_chunk || !c->exact) && e->m->d.ssm_d_state == 128 && getenv("ITB_PREFILL_STEPWISE") == nullptr) {
        const size_t nt = std::min(std::max<size_t>(1, e->R / e->B), n);
        const size_t need = (size_t)e->B * ((nt + GC - 1) / GC) * e->m->d.ssm_dt_rank * gdn_chunk_floats<128>();
        if (nt >= 32 && e->gdn_scratch_cap < need) {
            cudaStreamSynchronize(st);
            cudaFree(e->gdn_scratch); e->gdn_scratch = nullptr; e->gdn_scratch_cap = 0;
            if (cudaMalloc(&e->gdn_scratch, need * 4) == cudaSuccess) e->gdn_scratch_cap = need;
            else cudaGetLastError();             // without it the passes keep the serial-order scan
        }
    }
    ok = ok && steps_ready(e, 0);   // a one-token pass replays the step graph: have it captured before anything is enqueued
    if (ok && e->ep && getenv("ITB_PREFILL_STEPWISE") == nullptr) ok = ep_a2a_prepare(e);
    if (!ep_agree(e, ok)) return 1;
    const bool stepwise = getenv("ITB_PREFILL_STEPWISE") != nullptr;
    const size_t chunk = stepwise ? 1 : std::max<size_t>(1, e->R / e->B);

    // token ids laid out pass by pass, row-major inside a pass: [pass][seq][t]
    std::vector<int32_t> tr(n * e->B);
    size_t off = 0;
    for (size_t t0 = 0; t0 < n; t0 += chunk) {
        const size_t nt = std::min(chunk, n - t0);
        for (size_t b = 0; b < e->B; ++b)
            for (size_t t = 0; t < nt; ++t) tr[off++] = (int32_t)tokens[b * n + t0 + t];
    }
    ITB_CUDA_RET(c, cudaMemcpyAsync(e->prompt, tr.data(), tr.size() * 4, cudaMemcpyHostToDevice, st), 1);
    cudaEventRecord(e->ev0, st);
    off = 0;
    for (size_t t0 = 0; t0 < n; t0 += chunk) {
        const size_t nt = std::min(chunk, n - t0);
        if (stepwise || (e->B == 1 && nt == 1)) {
            cudaMemcpyAsync(e->tokens, e->prompt + off, e->B * 4, cudaMemcpyDeviceToDevice, st);
            if (!run_steps(e, 1, false)) return 1;
        } else {
            c->launches += enqueue_rows(e, st, (int)e->B, (int)nt, e->prompt + off);
            if (!c->error.empty()) { ep_abort(e); return 1; }
            e->last_n_tok = (uint32_t)nt;
            for (uint32_t b = 0; b < e->B; ++b) e->host_pos[b] += (uint32_t)nt;
        }
        off += nt * e->B;
    }
    cudaEventRecord(e->ev1, st);
    if (logits_out) cudaMemcpyAsync(logits_out, e->logits, (size_t)e->B * e->m->d.n_vocab * 4, cudaMemcpyDeviceToHost, st);
    ITB_CUDA_RET(c, cudaStreamSynchronize(st), 1);
    cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1);
    return check_flag(e) && c->error.empty() ? 0 : 1;
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
    const size_t K = e->m->d.n_expert_used, per = (size_t)e->B * K, n = (size_t)e->m->d.n_layer * per;
    if (cap < n) { itb_fail_msg(e->c, "read_routes: buffer too small"); return 1; }
    ITB_CUDA_RET(e->c, cudaStreamSynchronize(e->c->stream), 1);
    const size_t nt = e->last_n_tok;   // the last pass held nt tokens per sequence: report each sequence's last one
    for (uint32_t il = 0; il < e->m->d.n_layer; ++il)
        for (uint32_t b = 0; b < e->B; ++b)
            ITB_CUDA_RET(e->c, cudaMemcpy(ids + il * per + b * K, e->route_ids + ((size_t)il * e->R + b * nt + nt - 1) * K, K * 4, cudaMemcpyDeviceToHost), 1);
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

// One eagerly launched step (no graph) with an event after every launch. The stream is first held busy for
// about a millisecond so the whole step is queued before it starts and the kernels run back to back, as they
// do under the graph. Fills per-class launch counts, summed milliseconds and summed algorithmic bytes.
extern "C" int itb_engine_profile_step(itb_engine* e, const uint32_t* tokens, itb_kernel_stat* out, size_t cap, size_t* n_out) {
    itb_ctx* c = e->c;
    cudaStream_t st = c->stream;
    if (e->B != 1 || e->ep || e->tier || e->m->dense_fp4) { itb_fail_msg(c, "profile_step: plain single-sequence engines only"); return 1; }
    if (!tokens_in_range(e, tokens, e->B) || !steps_ready(e, 1)) return 1;  // function attributes are set during capture
    ITB_CUDA_RET(c, cudaMemcpyAsync(e->tokens, tokens, e->B * 4, cudaMemcpyHostToDevice, st), 1);
    StepProf prof;
    k_hold<<<1, 1, 0, st>>>(3000000LL);
    enqueue_step(e, st, &prof);
    cudaError_t err = cudaStreamSynchronize(st);
    if (err != cudaSuccess) { itb_fail(c, "profile_step", err); return 1; }
    c->launches += e->launches_per_step;
    for (uint32_t b = 0; b < e->B; ++b) e->host_pos[b] += 1;
    std::vector<itb_kernel_stat> acc(KC_COUNT);
    for (int k = 0; k < KC_COUNT; ++k) { memset(&acc[k], 0, sizeof acc[k]); snprintf(acc[k].name, sizeof acc[k].name, "%s", KC_NAMES[k]); }
    for (size_t i = 1; i < prof.ev.size(); ++i) {
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, prof.ev[i - 1], prof.ev[i]);
        int k = prof.cls[i];
        acc[k].launches++; acc[k].ms += ms; acc[k].bytes += prof.bytes[i];
    }
    for (auto ev : prof.ev) cudaEventDestroy(ev);
    size_t n = std::min<size_t>(cap, KC_COUNT);
    for (size_t k = 0; k < n; ++k) out[k] = acc[k];
    if (n_out) *n_out = n;
    return 0;
}

// Phase timeline of the decode step's kernels (see tl_mark): arm `slots` launch slots of 16 phase stamps each (0 disarms),
// run steps, read back slots * 16 words: (nanoseconds << 8) | kernel id, 0 where nothing was recorded.
extern "C" int itb_timeline_arm(itb_engine* e, uint32_t slots) {
    static unsigned long long* buf = nullptr;
    static uint32_t cap = 0;
    cudaStreamSynchronize(e->c->stream);
    if (slots > cap) { cudaFree(buf); buf = nullptr; if (cudaMalloc(&buf, (size_t)slots * 128) != cudaSuccess) return 1; cap = slots; }
    if (slots) cudaMemset(buf, 0, (size_t)slots * 128);
    unsigned long long* b = slots ? buf : nullptr;
    const unsigned c = slots;
    if (cudaMemcpyToSymbol(g_tl_cap, &c, 4) != cudaSuccess || cudaMemcpyToSymbol(g_tl_buf, &b, 8) != cudaSuccess) return 1;
    return 0;
}
extern "C" long itb_timeline_read(itb_engine* e, uint64_t* out_words, uint32_t slots) {
    cudaStreamSynchronize(e->c->stream);
    unsigned cap = 0; unsigned long long* b = nullptr;
    if (cudaMemcpyFromSymbol(&cap, g_tl_cap, 4) != cudaSuccess || cudaMemcpyFromSymbol(&b, g_tl_buf, 8) != cudaSuccess || !b) return -1;
    const unsigned n = std::min(cap, slots);
    if (n && cudaMemcpy(out_words, b, (size_t)n * 128, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return (long)n;
}
