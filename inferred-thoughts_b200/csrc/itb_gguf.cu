// GGUF loader: maps a model file, reads the `qwen35moe` hyper-parameters from its metadata and hands every tensor
// to itb_model_set_tensor straight from the mapping (the reference does the same through src/gguf/mod.rs:143-296 and
// src/model/qwen35.rs:333-486, :755-858). Layout (GGUF v3, little-endian): "GGUF", version u32, tensor count u64,
// key/value count u64; key/values (string key, u32 type, value); tensor infos (string name, u32 n_dims, u64 dims,
// u32 ggml type, u64 offset); tensor data from the next multiple of `general.alignment` (default 32).
// Every read is bounds-checked; a corrupt file fails with the offset, never with a fault.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/itb.h"

namespace {

struct Cursor {
    const uint8_t* p; size_t n, pos = 0; bool ok = true;
    bool take(void* out, size_t k) {
        if (!ok || k > n - pos) { ok = false; return false; }
        memcpy(out, p + pos, k); pos += k; return true;
    }
    template <class T> T get() { T v{}; take(&v, sizeof v); return v; }
    std::string str() {
        const uint64_t len = get<uint64_t>();
        if (!ok || len > n - pos) { ok = false; return {}; }
        std::string s((const char*)p + pos, (size_t)len); pos += (size_t)len; return s;
    }
};
struct Value { uint32_t ty = 0; uint64_t u = 0; double f = 0; std::string s; };
struct TensorInfo { std::vector<uint64_t> dims; uint32_t ty = 0; uint64_t off = 0; };

size_t scalar_size(uint32_t ty) {   // GGUF metadata value types 0..12 (8 = string, 9 = array)
    switch (ty) { case 0: case 1: case 7: return 1; case 2: case 3: return 2; case 4: case 5: case 6: return 4; case 10: case 11: case 12: return 8; default: return 0; }
}
bool read_value(Cursor& c, uint32_t ty, Value& v) {
    v.ty = ty;
    switch (ty) {
        case 0: v.u = c.get<uint8_t>(); break;   case 1: v.u = (uint64_t)(int64_t)c.get<int8_t>(); break;
        case 2: v.u = c.get<uint16_t>(); break;  case 3: v.u = (uint64_t)(int64_t)c.get<int16_t>(); break;
        case 4: v.u = c.get<uint32_t>(); break;  case 5: v.u = (uint64_t)(int64_t)c.get<int32_t>(); break;
        case 6: v.f = c.get<float>(); break;     case 7: v.u = c.get<uint8_t>(); break;
        case 8: v.s = c.str(); break;
        case 10: v.u = c.get<uint64_t>(); break; case 11: v.u = (uint64_t)c.get<int64_t>(); break;
        case 12: v.f = c.get<double>(); break;
        case 9: {   // arrays are skipped (none is needed for the shapes), element by element for strings
            const uint32_t et = c.get<uint32_t>(); const uint64_t cnt = c.get<uint64_t>();
            if (et == 8) { for (uint64_t i = 0; i < cnt && c.ok; ++i) c.str(); }
            else { const size_t es = scalar_size(et); if (!es || cnt > (c.n - c.pos) / es) c.ok = false; else c.pos += (size_t)(cnt * es); }
            break;
        }
        default: c.ok = false;
    }
    return c.ok;
}

}  // namespace

extern "C" int itb_model_load_gguf(itb_ctx* ctx, const char* path, itb_model** out, char* err, size_t err_cap) {
    *out = nullptr;
    auto fail = [&](const std::string& m) { if (err && err_cap) { strncpy(err, m.c_str(), err_cap - 1); err[err_cap - 1] = 0; } return 1; };
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(std::string("cannot open ") + path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) { close(fd); return fail("not a GGUF file (too short)"); }
    const size_t len = (size_t)st.st_size;
    void* map = mmap(nullptr, len, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return fail("mmap failed");
    struct Unmap { void* p; size_t n; ~Unmap() { munmap(p, n); } } unmap{map, len};
    Cursor c{(const uint8_t*)map, len};
    char magic[4]; c.take(magic, 4);
    if (!c.ok || memcmp(magic, "GGUF", 4) != 0) return fail("bad magic: not a GGUF file");
    const uint32_t version = c.get<uint32_t>();
    if (version != 3) return fail("unsupported GGUF version " + std::to_string(version));
    const uint64_t n_tensor = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (!c.ok || n_tensor > (1u << 20) || n_kv > (1u << 20)) return fail("implausible header counts");
    std::map<std::string, Value> md;
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = c.str();
        const uint32_t ty = c.get<uint32_t>();
        Value v;
        if (!read_value(c, ty, v)) return fail("truncated or malformed metadata at byte " + std::to_string(c.pos));
        md[key] = v;
    }
    std::map<std::string, TensorInfo> ti;
    for (uint64_t i = 0; i < n_tensor; ++i) {
        std::string name = c.str();
        TensorInfo t;
        const uint32_t nd = c.get<uint32_t>();
        if (!c.ok || nd > 4) return fail("malformed tensor info at byte " + std::to_string(c.pos));
        for (uint32_t k = 0; k < nd; ++k) t.dims.push_back(c.get<uint64_t>());
        t.ty = c.get<uint32_t>(); t.off = c.get<uint64_t>();
        if (!c.ok) return fail("truncated tensor info at byte " + std::to_string(c.pos));
        ti[name] = t;
    }
    uint64_t align = 32;
    if (md.count("general.alignment")) align = md["general.alignment"].u;
    if (align == 0 || (align & (align - 1))) return fail("general.alignment is not a power of two");
    const uint64_t data0 = (c.pos + align - 1) / align * align;
    auto arch_it = md.find("general.architecture");
    if (arch_it == md.end() || (arch_it->second.s != "qwen35moe")) return fail("architecture is not qwen35moe");
    const std::string a = arch_it->second.s + ".";
    std::string missing;
    auto u32 = [&](const char* k) -> uint32_t { auto it = md.find(a + k); if (it == md.end()) { if (missing.empty()) missing = a + k; return 0; } return (uint32_t)it->second.u; };
    auto f32 = [&](const char* k) -> float { auto it = md.find(a + k); if (it == md.end()) { if (missing.empty()) missing = a + k; return 0; } return (float)it->second.f; };
    itb_model_dims d{};
    d.n_layer = u32("block_count"); d.n_embd = u32("embedding_length"); d.n_head = u32("attention.head_count");
    d.n_head_kv = u32("attention.head_count_kv"); d.head_dim = u32("attention.key_length");
    d.rope_theta = f32("rope.freq_base"); d.rms_eps = f32("attention.layer_norm_rms_epsilon"); d.n_rot = u32("rope.dimension_count");
    d.ssm_d_conv = u32("ssm.conv_kernel"); d.ssm_d_inner = u32("ssm.inner_size"); d.ssm_d_state = u32("ssm.state_size");
    d.ssm_dt_rank = u32("ssm.time_step_rank"); d.ssm_n_group = u32("ssm.group_count"); d.full_attention_interval = u32("full_attention_interval");
    d.n_expert = u32("expert_count"); d.n_expert_used = u32("expert_used_count"); d.expert_ff = u32("expert_feed_forward_length");
    d.shared_ff = u32("expert_shared_feed_forward_length");
    if (!missing.empty()) return fail("missing metadata key " + missing);
    auto emb = ti.find("token_embd.weight");
    if (emb == ti.end() || emb->second.dims.size() != 2) return fail("token_embd.weight missing or not 2-D");
    d.n_vocab = (uint32_t)emb->second.dims[1];
    itb_model* m = nullptr;
    if (itb_model_create(ctx, &d, &m)) { const char* e = itb_take_error(ctx); return fail(e ? e : "model create failed"); }
    for (auto& kv : ti) {
        const std::string& name = kv.first;
        const TensorInfo& t = kv.second;
        if (name.size() > 6 && name.compare(name.size() - 6, 6, ".scale") == 0) continue;   // consumed with its weight
        // bytes of the tensor: up to the next tensor's offset is not recorded, so take it from type and shape
        uint64_t elems = 1; for (uint64_t x : t.dims) elems *= x;
        uint64_t bytes = 0;
        switch (t.ty) { case 0: bytes = elems * 4; break; case 1: bytes = elems * 2; break; case 8: bytes = elems / 32 * 34; break; case 40: bytes = elems / 64 * 36; break;
                        default: itb_model_destroy(m); return fail("tensor " + name + " has GGML type " + std::to_string(t.ty) + ", which this path has no kernel for"); }
        if (t.off % align || data0 + t.off > len || bytes > len - (data0 + t.off)) { itb_model_destroy(m); return fail("tensor " + name + " lies outside the file"); }
        const float* scale = nullptr; size_t n_scale = 0;
        if (name.size() > 7 && name.compare(name.size() - 7, 7, ".weight") == 0) {
            auto sc = ti.find(name.substr(0, name.size() - 7) + ".scale");
            if (sc != ti.end()) {
                uint64_t se = 1; for (uint64_t x : sc->second.dims) se *= x;
                if (sc->second.ty != 0 || data0 + sc->second.off > len || se * 4 > len - (data0 + sc->second.off)) { itb_model_destroy(m); return fail("scale of " + name + " is not F32 inside the file"); }
                scale = (const float*)((const uint8_t*)map + data0 + sc->second.off); n_scale = (size_t)se;
            }
        }
        if (itb_model_set_tensor(m, name.c_str(), t.ty, (const uint8_t*)map + data0 + t.off, (size_t)bytes, scale, n_scale)) {
            const char* e = itb_take_error(ctx);
            std::string msg = e ? e : "set_tensor failed";
            itb_model_destroy(m);
            return fail(msg);
        }
    }
    *out = m;
    return 0;
}
