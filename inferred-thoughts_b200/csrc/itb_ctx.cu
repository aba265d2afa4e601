// Context, sticky error, host-address-keyed mirrors, weight upload + repack, pass protocol.
// Mirrors the reference's device-backend host layer (src/ops/cuda/ops/residency.rs:23-100,
// src/ops/cuda/ops/mod.rs:91-110, :559-633) with a plain CUDA-runtime implementation.
#include <math.h>
#include <string.h>

#include <thread>

#include "itb_internal.cuh"

void itb_ops_use_logf_fix(const uint32_t* dev_tab, uint32_t n);      // itb_ops.cu: points that unit's log_f at the table
void itb_engine_use_logf_fix(const uint32_t* dev_tab, uint32_t n);   // itb_engine.cu

static std::string g_create_error;

bool itb_fail_msg(itb_ctx* c, const std::string& msg) {
    if (c && c->error.empty()) c->error = msg;
    return false;
}
bool itb_fail(itb_ctx* c, const char* what, cudaError_t e) {
    return itb_fail_msg(c, std::string(what) + ": " + cudaGetErrorString(e));
}

extern "C" const char* itb_last_create_error(void) { return g_create_error.empty() ? nullptr : g_create_error.c_str(); }

// ------------------------------------------------------------------ the host C library's logf, as a correction table
// For every float x of [1, 2^29): how logf(x) differs from the correctly rounded (float)log((double)x) -- 0 same, 1 one
// ulp above, 2 one ulp below -- two bits each (61 MB). Built once per process with all host threads, uploaded once per
// device and kept for the life of the process; the kernels' log_f applies it (itb_internal.cuh).
static const uint32_t LOGF_FIX_N = 29u << 23;
static std::vector<uint32_t> g_logf_fix_host;
static uint32_t* g_logf_fix_dev[64];
static uint64_t g_logf_fix_odd = 0;      // floats whose two results are more than one ulp apart (left uncorrected)
static void build_logf_fix() {
    if (!g_logf_fix_host.empty()) return;
    g_logf_fix_host.assign(LOGF_FIX_N / 16, 0u);
    const unsigned nt = std::max(1u, std::thread::hardware_concurrency());
    std::vector<std::thread> th;
    std::vector<uint64_t> odd(nt, 0);
    const uint32_t words = LOGF_FIX_N / 16;
    for (unsigned t = 0; t < nt; ++t)
        th.emplace_back([=, &odd] {
            const uint32_t w0 = (uint32_t)((uint64_t)words * t / nt), w1 = (uint32_t)((uint64_t)words * (t + 1) / nt);
            for (uint32_t w = w0; w < w1; ++w) {
                uint32_t word = 0;
                for (uint32_t j = 0; j < 16; ++j) {
                    const uint32_t bits = 0x3f800000u + w * 16 + j;
                    float x; memcpy(&x, &bits, 4);
                    const float lib = logf(x), cr = (float)log((double)x);
                    uint32_t a, b; memcpy(&a, &lib, 4); memcpy(&b, &cr, 4);
                    const int32_t d = (int32_t)(a - b);
                    if (d == 1) word |= 1u << (2 * j);
                    else if (d == -1) word |= 2u << (2 * j);
                    else if (d != 0) odd[t]++;
                }
                g_logf_fix_host[w] = word;
            }
        });
    for (auto& t : th) t.join();
    for (uint64_t o : odd) g_logf_fix_odd += o;
}
static const uint32_t* logf_fix_on_device(int dev) {
    if (dev < 0 || dev >= 64) return nullptr;
    if (g_logf_fix_dev[dev]) return g_logf_fix_dev[dev];
    build_logf_fix();
    uint32_t* d = nullptr;
    if (cudaMalloc(&d, (size_t)LOGF_FIX_N / 4) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (cudaMemcpy(d, g_logf_fix_host.data(), (size_t)LOGF_FIX_N / 4, cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(d); cudaGetLastError(); return nullptr; }
    g_logf_fix_dev[dev] = d;
    return d;
}
// The restated expf on the host (tests compare it with the C library's).
extern "C" float itb_expf_host(float x) {
    static const unsigned long long tab[32] = {ITB_EXP2_TAB};
    return itb_expf_lib(x, tab);
}

extern "C" int itb_create(int device_ordinal, const char* opts, itb_ctx** out) {
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        g_create_error = std::string("no usable CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "count is 0");
        return 1;
    }
    if (device_ordinal < 0 || device_ordinal >= n) { g_create_error = "device ordinal out of range"; return 2; }
    if ((e = cudaSetDevice(device_ordinal)) != cudaSuccess) { g_create_error = cudaGetErrorString(e); return 3; }
    cudaDeviceProp p;
    cudaGetDeviceProperties(&p, device_ordinal);
    if (p.major != 10) {
        g_create_error = "this library is built for sm_100a only; found sm_" + std::to_string(p.major * 10 + p.minor);
        return 4;
    }
    itb_ctx* c = new itb_ctx();
    c->device = device_ordinal;
    c->sm_count = p.multiProcessorCount;
    if ((e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking)) != cudaSuccess) {
        g_create_error = cudaGetErrorString(e); delete c; return 5;
    }
    std::string o = opts ? opts : "";
    if (o.find("kv=bf16") != std::string::npos) c->kv_bf16 = true;
    if (o.find("exact=0") != std::string::npos) c->exact = false;
    if (o.find("experts=fp4tc") != std::string::npos) c->fp4tc = true;
    if (o.find("attn=mma") != std::string::npos) c->attn_mma = true;
    if (o.find("dense=q8tc") != std::string::npos) c->q8tc = true;
    if (o.find("dense=f16tc") != std::string::npos) c->f16tc = true;
    if (o.find("gdn=chunk") != std::string::npos) c->gdn_chunk = true;
    // libm=cr keeps log correctly rounded instead of following the host C library's logf (see itb_internal.cuh)
    const uint32_t* fix = o.find("libm=cr") != std::string::npos ? nullptr : logf_fix_on_device(device_ordinal);
    itb_ops_use_logf_fix(fix, fix ? LOGF_FIX_N : 0);
    itb_engine_use_logf_fix(fix, fix ? LOGF_FIX_N : 0);
    *out = c;
    return 0;
}

static void free_map(std::unordered_map<const void*, Mirror>& m) {
    for (auto& kv : m) cudaFree(kv.second.dev);
    m.clear();
}

extern "C" void itb_destroy(itb_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    free_map(c->mirrors); free_map(c->states); free_map(c->kv);
    for (auto& w : c->weights) { cudaFree(w.second.a); cudaFree(w.second.b); cudaFree(w.second.scale2); }
    cudaFree(c->pair_off); cudaFree(c->pair_list);
    itb_tc_free(c);
    cudaFree(c->route_ids); cudaFree(c->route_w); cudaFree(c->xq); cudaFree(c->xs); cudaFree(c->tmp_f32);
    cudaStreamDestroy(c->stream);
    delete c;
}

extern "C" const char* itb_take_error(itb_ctx* c) {
    if (!c) return "null context";
    if (c->error.empty()) {
        // surface asynchronous failures too
        cudaError_t e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) itb_fail(c, "stream", e);
        if (c->error.empty()) return nullptr;
    }
    c->error_out.swap(c->error);
    c->error.clear();
    return c->error_out.c_str();
}

extern "C" uint64_t itb_launch_count(itb_ctx* c) { return c->launches; }

// ------------------------------------------------------------------ mirrors
static Mirror* slot_for(itb_ctx* c, std::unordered_map<const void*, Mirror>& map, const void* key, size_t bytes) {
    auto it = map.find(key);
    if (it == map.end() || it->second.bytes < bytes) {
        Mirror m;
        cudaError_t e = cudaMalloc(&m.dev, bytes ? bytes : 4);
        if (e != cudaSuccess) { itb_fail(c, "cudaMalloc(mirror)", e); return nullptr; }
        m.bytes = bytes;
        if (it != map.end()) {
            // Grown under the same address: keep what the device already holds.
            m.device_current = it->second.device_current;
            if (m.device_current) {
                cudaMemcpyAsync(m.dev, it->second.dev, it->second.bytes, cudaMemcpyDeviceToDevice, c->stream);
                cudaStreamSynchronize(c->stream);
            }
            cudaFree(it->second.dev); c->mirror_bytes -= it->second.bytes; map.erase(it);
        }
        c->mirror_bytes += bytes;
        it = map.emplace(key, m).first;
    }
    return &it->second;
}

float* itb_mirror_in(itb_ctx* c, const float* host, size_t len) {
    Mirror* m = slot_for(c, c->mirrors, host, len * 4);
    if (!m) return nullptr;
    if (!m->device_current) {
        cudaError_t e = cudaMemcpyAsync(m->dev, host, len * 4, cudaMemcpyHostToDevice, c->stream);
        if (e != cudaSuccess) { itb_fail(c, "h2d", e); return nullptr; }
        // The host buffer is pageable and may change right after this call returns.
        cudaStreamSynchronize(c->stream);
        m->device_current = true;
    }
    return (float*)m->dev;
}
float* itb_mirror_out(itb_ctx* c, const float* host, size_t len) {
    Mirror* m = slot_for(c, c->mirrors, host, len * 4);
    if (!m) return nullptr;
    m->device_current = true;
    return (float*)m->dev;
}
float* itb_mirror_inout(itb_ctx* c, float* host, size_t len) { return itb_mirror_in(c, host, len); }

// Recurrent state: uploaded on first touch, then owned by the device until forget_state
// (src/ops/mod.rs:1394-1419).
float* itb_state_slab(itb_ctx* c, float* host, size_t len) {
    auto it = c->states.find(host);
    if (it == c->states.end() || it->second.bytes < len * 4) {
        Mirror* m = slot_for(c, c->states, host, len * 4);
        if (!m) return nullptr;
        cudaMemcpyAsync(m->dev, host, len * 4, cudaMemcpyHostToDevice, c->stream);
        cudaStreamSynchronize(c->stream);
        m->device_current = true;
        it = c->states.find(host);
    }
    c->last_state_key = host;
    return (float*)it->second.dev;
}
uint16_t* itb_kv_slab(itb_ctx* c, const uint16_t* host, size_t len) {
    auto it = c->kv.find(host);
    if (it == c->kv.end() || it->second.bytes < len * 2) {
        Mirror* m = slot_for(c, c->kv, host, len * 2);
        if (!m) return nullptr;
        cudaMemcpyAsync(m->dev, host, len * 2, cudaMemcpyHostToDevice, c->stream);
        cudaStreamSynchronize(c->stream);
        m->device_current = true;
        it = c->kv.find(host);
    }
    return (uint16_t*)it->second.dev;
}

extern "C" void itb_begin_pass(itb_ctx* c, size_t) {
    // Activation buffers may have been rewritten by the host between passes: every mirror is stale,
    // the allocations are kept (src/ops/cuda/ops/mod.rs:620-632).
    for (auto& m : c->mirrors) m.second.device_current = false;
    c->in_pass = true;
}
extern "C" void itb_end_pass(itb_ctx* c) { c->in_pass = false; }
extern "C" void itb_host_wrote(itb_ctx* c, const float* buf, size_t) {
    auto it = c->mirrors.find(buf);
    if (it != c->mirrors.end()) it->second.device_current = false;
}
extern "C" void itb_host_needs(itb_ctx* c, float* buf, size_t len) {
    auto it = c->mirrors.find(buf);
    if (it == c->mirrors.end() || !it->second.device_current) return;
    size_t bytes = len * 4 < it->second.bytes ? len * 4 : it->second.bytes;
    ITB_CUDA(c, cudaMemcpyAsync(buf, it->second.dev, bytes, cudaMemcpyDeviceToHost, c->stream));
    ITB_CUDA(c, cudaStreamSynchronize(c->stream));
}
extern "C" void itb_forget_state(itb_ctx* c) {
    cudaStreamSynchronize(c->stream);
    free_map(c->states);
}
extern "C" void itb_read_state(itb_ctx* c, float* host, size_t len) {
    auto it = c->states.find(host);
    if (it == c->states.end()) return;
    size_t bytes = len * 4 < it->second.bytes ? len * 4 : it->second.bytes;
    ITB_CUDA(c, cudaMemcpyAsync(host, it->second.dev, bytes, cudaMemcpyDeviceToHost, c->stream));
    ITB_CUDA(c, cudaStreamSynchronize(c->stream));
}
extern "C" void itb_read_kv(itb_ctx* c, uint16_t* slab, size_t len) {
    auto it = c->kv.find(slab);
    if (it == c->kv.end()) return;
    size_t bytes = len * 2 < it->second.bytes ? len * 2 : it->second.bytes;
    ITB_CUDA(c, cudaMemcpyAsync(slab, it->second.dev, bytes, cudaMemcpyDeviceToHost, c->stream));
    ITB_CUDA(c, cudaStreamSynchronize(c->stream));
}
extern "C" void itb_reserve_activations(itb_ctx*, size_t) {}
extern "C" void itb_prefetch_hint(itb_ctx*, const itb_weights*, const float*, size_t, size_t) {}

extern "C" int itb_config_report(itb_ctx* c, char* buf, size_t cap) {
    return snprintf(buf, cap, "backend=b200 sm=100a sms=%d kv=%s f32_dots=%s mirrors=%zu mirror_bytes=%zu weight_bytes=%zu",
                    c->sm_count, c->kv_bf16 ? "bf16" : "f16", c->exact ? "serial" : "tree", c->mirrors.size(),
                    c->mirror_bytes, c->weight_bytes);
}
extern "C" void itb_device_report(itb_ctx* c) {
    size_t fr = 0, tot = 0;
    cudaMemGetInfo(&fr, &tot);
    fprintf(stderr, "[itb] device %d: %d SMs, %.1f / %.1f GiB free\n", c->device, c->sm_count, fr / 1073741824.0,
            tot / 1073741824.0);
}

bool itb_ensure_route(itb_ctx* c, size_t n_pairs) {
    if (c->route_cap >= n_pairs) return true;
    cudaFree(c->route_ids); cudaFree(c->route_w);
    if (cudaMalloc(&c->route_ids, n_pairs * 4) != cudaSuccess || cudaMalloc(&c->route_w, n_pairs * 4) != cudaSuccess)
        return itb_fail_msg(c, "cudaMalloc(route)");
    c->route_cap = n_pairs;
    return true;
}
bool itb_ensure_xq(itb_ctx* c, size_t n) {
    if (c->xq_cap >= n) return true;
    cudaFree(c->xq); cudaFree(c->xs);
    if (cudaMalloc(&c->xq, n) != cudaSuccess || cudaMalloc(&c->xs, (n / 16 + 1) * 4) != cudaSuccess)
        return itb_fail_msg(c, "cudaMalloc(xq)");
    c->xq_cap = n;
    return true;
}

// ------------------------------------------------------------------ repack kernels
// One thread per Q8_0 block: 2 scale bytes + 32 quants -> planes.
__global__ void k_repack_q8(const uint8_t* __restrict__ raw, int8_t* __restrict__ q, uint16_t* __restrict__ s, size_t nb) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nb) return;
    const uint8_t* p = raw + b * 34;
    s[b] = (uint16_t)(p[0] | (p[1] << 8));
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = p[2 + 4 * i] | (p[3 + 4 * i] << 8) | (p[4 + 4 * i] << 16) | ((uint32_t)p[5 + 4 * i] << 24);
    uint4* dst = (uint4*)(q + b * 32);
    dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
    dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
}
// One thread per NVFP4 block of 64: 4 scale codes + 32 bytes whose byte 8s+j holds element 16s+j (low)
// and 16s+j+8 (high) -> scale plane and element-ordered nibbles (byte i of a sub-block = elements 2i, 2i+1).
__global__ void k_repack_fp4(const uint8_t* __restrict__ raw, uint8_t* __restrict__ nib, uint8_t* __restrict__ sc, size_t nb) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nb) return;
    const uint8_t* p = raw + b * 36;
    uint8_t out[32];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        uint8_t c = p[s];
        sc[b * 4 + s] = c == 0x7f ? 0 : c;
        uint8_t e[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) { e[j] = p[4 + 8 * s + j] & 0xf; e[j + 8] = p[4 + 8 * s + j] >> 4; }
#pragma unroll
        for (int i = 0; i < 8; ++i) out[8 * s + i] = e[2 * i] | (e[2 * i + 1] << 4);
    }
    uint4* dst = (uint4*)(nib + b * 32);
    const uint4* src = (const uint4*)out;
    dst[0] = src[0];
    dst[1] = src[1];
}
__global__ void k_f16_to_f32(const uint16_t* __restrict__ raw, float* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f16_bits_to_f32(raw[i]);
}
void itb_repack_q8(cudaStream_t st, const uint8_t* raw, int8_t* q, uint16_t* s, size_t nb) {
    if (nb) k_repack_q8<<<(unsigned)((nb + 255) / 256), 256, 0, st>>>(raw, q, s, nb);
}
void itb_repack_fp4(cudaStream_t st, const uint8_t* raw, uint8_t* nib, uint8_t* sc, size_t nb) {
    if (nb) k_repack_fp4<<<(unsigned)((nb + 255) / 256), 256, 0, st>>>(raw, nib, sc, nb);
}
void itb_f16_to_f32(cudaStream_t st, const uint16_t* raw, float* out, size_t n) {
    if (n) k_f16_to_f32<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(raw, out, n);
}

// Upload on first sight, keyed by the host pointer (src/ops/cuda/mod.rs:59-68).
const WeightEntry* itb_weight(itb_ctx* c, const uint8_t* data, size_t bytes, uint32_t ty, size_t n_in, size_t n_out,
                              size_t n_expert, const uint8_t* scale, size_t scale_bytes) {
    auto it = c->weights.find(data);
    if (it != c->weights.end()) {
        const WeightEntry& h = it->second;
        if (h.ty == ty && h.n_in == n_in && h.n_out == n_out && h.n_expert == n_expert) return &it->second;
        // The address now names a different tensor (the caller freed and reallocated): drop the old upload.
        cudaStreamSynchronize(c->stream);
        cudaFree(h.a); cudaFree(h.b); cudaFree(h.scale2);
        c->weight_bytes -= h.bytes;
        c->weights.erase(it);
    }
    WeightEntry w;
    w.ty = ty; w.n_in = n_in; w.n_out = n_out; w.n_expert = n_expert;
    size_t elems = n_in * n_out * n_expert;
    size_t want = ty == ITB_F32 ? elems * 4 : ty == ITB_F16 ? elems * 2 : ty == ITB_Q8_0 ? elems / 32 * 34 : ty == ITB_NVFP4 ? elems / 64 * 36 : 0;
    if (want == 0 || bytes < want) { itb_fail_msg(c, "weight: unsupported type or short buffer"); return nullptr; }
    if ((ty == ITB_Q8_0 && n_in % 32) || (ty == ITB_NVFP4 && n_in % 64)) { itb_fail_msg(c, "weight: row is not a whole number of blocks"); return nullptr; }
    uint8_t* raw = nullptr;
    cudaError_t e = cudaMalloc(&raw, want);
    if (e != cudaSuccess) { itb_fail(c, "cudaMalloc(weight staging)", e); return nullptr; }
    cudaMemcpyAsync(raw, data, want, cudaMemcpyHostToDevice, c->stream);
    // Every plane is allocated before any kernel runs; on a failure everything allocated so far is given back and the
    // caller gets "out of device memory" instead of a kernel writing through a null pointer.
    const bool want_s2 = scale && scale_bytes >= n_expert * 4;
    const size_t a_bytes = ty == ITB_F32 ? 0 : ty == ITB_F16 ? elems * 4 : ty == ITB_Q8_0 ? elems : elems / 2;
    const size_t b_bytes = ty == ITB_Q8_0 ? elems / 32 * 2 : ty == ITB_NVFP4 ? elems / 16 : 0;
    bool oom = false;
    if (a_bytes && cudaMalloc(&w.a, a_bytes) != cudaSuccess) { w.a = nullptr; oom = true; }
    if (!oom && b_bytes && cudaMalloc(&w.b, b_bytes) != cudaSuccess) { w.b = nullptr; oom = true; }
    if (!oom && want_s2 && cudaMalloc(&w.scale2, n_expert * 4) != cudaSuccess) { w.scale2 = nullptr; oom = true; }
    if (oom) {
        cudaStreamSynchronize(c->stream);
        cudaFree(raw); cudaFree(w.a); cudaFree(w.b); cudaFree(w.scale2);
        cudaGetLastError();
        itb_fail_msg(c, "weight: out of device memory");
        return nullptr;
    }
    if (ty == ITB_F32) { w.a = raw; raw = nullptr; w.bytes = want; }
    else if (ty == ITB_F16) {
        itb_f16_to_f32(c->stream, (const uint16_t*)raw, (float*)w.a, elems);
        w.bytes = elems * 4;
    } else if (ty == ITB_Q8_0) {
        itb_repack_q8(c->stream, raw, (int8_t*)w.a, (uint16_t*)w.b, elems / 32);
        w.bytes = elems + elems / 16;
    } else {
        itb_repack_fp4(c->stream, raw, (uint8_t*)w.a, (uint8_t*)w.b, elems / 64);
        w.bytes = elems / 2 + elems / 16;
    }
    if (want_s2) cudaMemcpyAsync(w.scale2, scale, n_expert * 4, cudaMemcpyHostToDevice, c->stream);
    e = cudaStreamSynchronize(c->stream);
    if (raw) cudaFree(raw);
    if (e != cudaSuccess) { cudaFree(w.a); cudaFree(w.b); cudaFree(w.scale2); itb_fail(c, "weight upload", e); return nullptr; }
    c->weight_bytes += w.bytes;
    return &c->weights.emplace(data, w).first->second;
}
