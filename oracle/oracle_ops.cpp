// CPU oracle, op level. TEST INFRASTRUCTURE ONLY (see oracle.h). Each function cites the
// reference lines it restates; accumulation orders are the reference's.
#include "oracle.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <thread>

namespace orc {

// ------------------------------------------------------------------ threading
static int g_threads = 1;
void set_threads(int n) { g_threads = n < 1 ? 1 : n; }
int get_threads() { return g_threads; }

// Rows are independent; a thread changes which rows it computes, never how (src/ops/spin.rs:1-25).
static void parallel_rows(size_t n, size_t work_per_row, const std::function<void(size_t, size_t)>& fn) {
    int nt = g_threads;
    if (nt <= 1 || n < 2 || n * work_per_row < (size_t)1 << 16) { fn(0, n); return; }
    if ((size_t)nt > n) nt = (int)n;
    std::vector<std::thread> th;
    size_t per = (n + nt - 1) / nt;
    for (int t = 1; t < nt; ++t) {
        size_t a = std::min(n, t * per), b = std::min(n, a + per);
        if (a < b) th.emplace_back([=, &fn] { fn(a, b); });
    }
    fn(0, std::min(n, per));
    for (auto& t : th) t.join();
}

// ------------------------------------------------------------------ formats
// src/quant/half.rs:29-59 (value semantics; the bit tricks there are an optimisation).
float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { e++; man <<= 1; } while ((man & 0x400) == 0);
            bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3ff) << 13;
        }
    } else if (exp == 0x1f) bits = sign | 0x7f800000u | man << 13;
    else bits = sign | (exp + 127 - 15) << 23 | man << 13;
    float f; std::memcpy(&f, &bits, 4); return f;
}

// src/quant/half.rs:71-114, round to nearest even.
uint16_t f32_to_f16(float f) {
    uint32_t bits; std::memcpy(&bits, &f, 4);
    uint16_t sign = (bits >> 16) & 0x8000;
    int exp = (bits >> 23) & 0xff;
    uint32_t mant = bits & 0x007fffff;
    if (exp == 0xff) return sign | 0x7c00 | (mant ? 0x0200 : 0);
    int e = exp - 127 + 15;
    if (e >= 0x1f) return sign | 0x7c00;
    if (e <= 0) {
        if (e < -10) return sign;
        uint32_t m = mant | 0x00800000;
        uint32_t shift = 14 - e;
        uint32_t half = m >> shift, rem = m & ((1u << shift) - 1), halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half & 1))) half++;
        return sign | (uint16_t)half;
    }
    uint32_t h = ((uint32_t)e << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fff;
    if (rem > 0x1000 || (rem == 0x1000 && (h & 1))) h++;
    return sign | (uint16_t)h;
}

uint16_t f32_to_bf16(float f) {
    uint32_t bits; std::memcpy(&bits, &f, 4);
    if ((bits & 0x7fffffff) > 0x7f800000) return (bits >> 16) | 0x40;  // NaN stays NaN
    uint32_t lsb = (bits >> 16) & 1;
    bits += 0x7fff + lsb;
    return bits >> 16;
}
float bf16_to_f32(uint16_t h) { uint32_t b = (uint32_t)h << 16; float f; std::memcpy(&f, &b, 4); return f; }

// src/quant/mod.rs:265 (doubled E2M1 values, sign in bit 3).
const int8_t KVALUES_MXFP4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

// src/quant/mod.rs:271-284: unsigned E4M3, bias 7, halved; 0 and 0x7f read as 0; bit 7 ignored.
float ue4m3_to_f32(uint8_t x) {
    if (x == 0 || x == 0x7f) return 0.0f;
    int exp = (x >> 3) & 0xf;
    float man = (float)(x & 7);
    float raw = exp == 0 ? man * std::ldexp(1.0f, -9) : (1.0f + man / 8.0f) * std::ldexp(1.0f, exp - 7);
    return raw * 0.5f;
}

// src/quant/mod.rs:321-336: RN-even to the positive E4M3 codes, saturating at 448 (code 0x7e).
uint8_t fp32_to_ue4m3_rn(float x) {
    if (!(x > 0.0f)) return 0;
    if (x >= 448.0f) return 0x7e;
    double v = (double)x;
    auto value = [](int c) { return 2.0 * (double)ue4m3_to_f32((uint8_t)c); };
    int lo = 0;
    for (int c = 1; c <= 0x7e; ++c) { if (value(c) <= v) lo = c; else break; }
    int hi = lo + 1;
    double below = v - value(lo), above = value(hi) - v;
    return (below < above || (below == above && (lo & 1) == 0)) ? (uint8_t)lo : (uint8_t)hi;
}

size_t row_bytes(uint32_t ty, size_t n_in) {
    switch (ty) {
        case T_F32: return n_in * 4;
        case T_F16: return n_in * 2;
        case T_Q8_0: return n_in / 32 * 34;   // src/gguf/types.rs:164
        case T_NVFP4: return n_in / 64 * 36;  // src/gguf/types.rs:206
    }
    return 0;
}

// src/quant/mod.rs:96-106
void dequantize_q8_0(const uint8_t* data, float* out, size_t n) {
    for (size_t b = 0; b < n / 32; ++b) {
        const uint8_t* blk = data + b * 34;
        float d = f16_to_f32((uint16_t)(blk[0] | blk[1] << 8));
        for (int j = 0; j < 32; ++j) out[b * 32 + j] = (float)(int8_t)blk[2 + j] * d;
    }
}

// src/quant/mod.rs:338-357
void dequantize_nvfp4(const uint8_t* data, float* out, size_t n) {
    for (size_t b = 0; b < n / 64; ++b) {
        const uint8_t* blk = data + b * 36;
        float* y = out + b * 64;
        for (int s = 0; s < 4; ++s) {
            float d = ue4m3_to_f32(blk[s]);
            const uint8_t* qs = blk + 4 + s * 8;
            for (int j = 0; j < 8; ++j) {
                y[s * 16 + j] = (float)KVALUES_MXFP4[qs[j] & 0xf] * d;
                y[s * 16 + j + 8] = (float)KVALUES_MXFP4[qs[j] >> 4] * d;
            }
        }
    }
}

// ------------------------------------------------------------------ quantisers and dots
// src/ops/naive.rs:653-675
void QuantizedRow::from_f32(const float* x, size_t n) {
    size_t nb = n / 32;
    scales.resize(nb); quants.resize(nb * 32);
    for (size_t b = 0; b < nb; ++b) {
        const float* blk = x + b * 32;
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(blk[j]));
        float d = amax / 127.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        scales[b] = f16_to_f32(f32_to_f16(d));
        for (int j = 0; j < 32; ++j) {
            float r = roundf(blk[j] * id);
            quants[b * 32 + j] = (int8_t)std::max(-128.0f, std::min(127.0f, r));
        }
    }
}

// src/ops/naive.rs:679-686
std::vector<uint8_t> QuantizedRow::to_blocks() const {
    std::vector<uint8_t> out;
    for (size_t b = 0; b < scales.size(); ++b) {
        uint16_t h = f32_to_f16(scales[b]);
        out.push_back(h & 0xff); out.push_back(h >> 8);
        for (int j = 0; j < 32; ++j) out.push_back((uint8_t)quants[b * 32 + j]);
    }
    return out;
}

// src/ops/naive.rs:691-704
float dot_q8_0_q8_0(const uint8_t* row, size_t n_in, const QuantizedRow& x) {
    float sumf = 0.0f;
    for (size_t i = 0; i < n_in / 32; ++i) {
        const uint8_t* blk = row + i * 34;
        float dw = f16_to_f32((uint16_t)(blk[0] | blk[1] << 8));
        const int8_t* qs = x.quants.data() + i * 32;
        int32_t sumi = 0;
        for (int j = 0; j < 32; ++j) sumi += (int32_t)(int8_t)blk[2 + j] * (int32_t)qs[j];
        sumf += (float)sumi * (dw * x.scales[i]);
    }
    return sumf;
}

// src/ops/naive.rs:714-734
float dot_nvfp4_q8_0(const uint8_t* row, size_t n_in, const QuantizedRow& x) {
    float sumf = 0.0f;
    for (size_t ib = 0; ib < n_in / 64; ++ib) {
        const uint8_t* blk = row + ib * 36;
        for (int s = 0; s < 4; ++s) {
            float d = ue4m3_to_f32(blk[s]);
            size_t q8 = 2 * ib + s / 2;
            int off = (s % 2) * 16;
            float dy = x.scales[q8];
            const int8_t* qa = x.quants.data() + q8 * 32;
            int32_t lo = 0, hi = 0;
            for (int j = 0; j < 8; ++j) {
                uint8_t qv = blk[4 + s * 8 + j];
                lo += (int32_t)qa[off + j] * (int32_t)KVALUES_MXFP4[qv & 0xf];
                hi += (int32_t)qa[off + j + 8] * (int32_t)KVALUES_MXFP4[qv >> 4];
            }
            sumf += dy * d * (float)(lo + hi);
        }
    }
    return sumf;
}

// src/ops/naive.rs:794-806
uint8_t e2m1_code(float x, float e) {
    static const float POS[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float ax = fabsf(x) * e;
    int best_i = 0;
    float best_err = fabsf(ax - POS[0]);
    for (int i = 1; i < 8; ++i) {
        float err = fabsf(ax - POS[i]);
        if (err < best_err) { best_i = i; best_err = err; }
    }
    return (uint8_t)(best_i | (x < 0.0f ? 8 : 0));
}

// src/ops/naive.rs:755-788
void Fp4Row::from_f32(const float* x, size_t n) {
    scales.clear(); codes.clear();
    static const int OFFS[5] = {0, -1, 1, -2, 2};
    for (size_t b = 0; b < n / 16; ++b) {
        const float* blk = x + b * 16;
        float amax = 0.0f;
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(blk[j]));
        int seed = fp32_to_ue4m3_rn(amax / 6.0f);
        float best_err = 3.40282347e+38f, best_scale = 0.0f;
        uint8_t best_code = 0;
        for (int o = 0; o < 5; ++o) {
            int code = seed + OFFS[o];
            if (code < 0 || code > 0x7e) continue;
            float sc = ue4m3_to_f32((uint8_t)code);
            float inv = sc > 0.0f ? 0.5f / sc : 0.0f;
            float err = 0.0f;
            for (int j = 0; j < 16; ++j) {
                uint8_t q = e2m1_code(blk[j], inv);
                float d = fabsf(blk[j]) - fabsf((float)KVALUES_MXFP4[q & 7]) * sc;
                err = fmaf(d, d, err);
            }
            if (err < best_err) { best_err = err; best_code = (uint8_t)code; best_scale = sc; }
        }
        float inv = best_scale > 0.0f ? 0.5f / best_scale : 0.0f;
        scales.push_back(best_code);
        for (int j = 0; j < 16; ++j) codes.push_back(e2m1_code(blk[j], inv));
    }
}

// src/ops/naive.rs:819-837
float dot_nvfp4_fp4(const uint8_t* row, size_t n_in, const Fp4Row& x) {
    float sumf = 0.0f;
    for (size_t ib = 0; ib < n_in / 64; ++ib) {
        const uint8_t* blk = row + ib * 36;
        for (int s = 0; s < 4; ++s) {
            size_t sub = 4 * ib + s;
            float d = ue4m3_to_f32(blk[s]) * ue4m3_to_f32(x.scales[sub]);
            const uint8_t* xc = x.codes.data() + sub * 16;
            int32_t sumi = 0;
            for (int k = 0; k < 8; ++k) {
                uint8_t qv = blk[4 + s * 8 + k];
                sumi += (int32_t)KVALUES_MXFP4[qv & 0xf] * (int32_t)KVALUES_MXFP4[xc[k]];
                sumi += (int32_t)KVALUES_MXFP4[qv >> 4] * (int32_t)KVALUES_MXFP4[xc[k + 8]];
            }
            sumf += d * (float)sumi;
        }
    }
    return sumf;
}

// src/ops/naive.rs:843-861 (sequential left fold)
float dot_row(uint32_t ty, const uint8_t* row, const float* x, size_t n_in) {
    float s = 0.0f;
    if (ty == T_F32) {
        for (size_t i = 0; i < n_in; ++i) { float w; std::memcpy(&w, row + 4 * i, 4); s += w * x[i]; }
    } else if (ty == T_F16) {
        for (size_t i = 0; i < n_in; ++i) s += f16_to_f32((uint16_t)(row[2 * i] | row[2 * i + 1] << 8)) * x[i];
    }
    return s;
}

// ------------------------------------------------------------------ ops
// src/ops/naive.rs:633-640
static float rms_scale(const float* x, size_t n, float eps) {
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) sum += (double)(x[i] * x[i]);
    float mean = (float)(sum / (double)n);
    return 1.0f / sqrtf(mean + eps);
}

// src/ops/naive.rs:139-152
void rms_norm(const float* x, size_t x_len, const float* w, size_t nd, float eps, float* out) {
    for (size_t r = 0; r < x_len / nd; ++r) {
        const float* row = x + r * nd; float* o = out + r * nd;
        float sc = rms_scale(row, nd, eps);
        for (size_t i = 0; i < nd; ++i) o[i] = row[i] * sc * w[i];
    }
}

// src/ops/naive.rs:154-164
void rms_norm_heads(float* x, size_t len, const float* w, size_t head_dim, float eps) {
    for (size_t h = 0; h < len / head_dim; ++h) {
        float* head = x + h * head_dim;
        float sc = rms_scale(head, head_dim, eps);
        for (size_t i = 0; i < head_dim; ++i) head[i] = head[i] * sc * w[i];
    }
}

// src/ops/naive.rs:38-83, 166-178
static void matmul_impl(const Weights& w, const float* x, size_t x_len, float* out, int fp4act) {
    size_t n_tok = x_len / w.n_in;
    for (size_t t = 0; t < n_tok; ++t) {
        const float* xt = x + t * w.n_in; float* ot = out + t * w.n_out;
        if (w.ty == T_Q8_0 || (w.ty == T_NVFP4 && !fp4act)) {
            QuantizedRow qx; qx.from_f32(xt, w.n_in);
            parallel_rows(w.n_out, w.n_in, [&](size_t a, size_t b) {
                for (size_t j = a; j < b; ++j)
                    ot[j] = w.ty == T_Q8_0 ? dot_q8_0_q8_0(w.row(j), w.n_in, qx) : dot_nvfp4_q8_0(w.row(j), w.n_in, qx);
            });
        } else if (w.ty == T_NVFP4) {
            Fp4Row qx; qx.from_f32(xt, w.n_in);
            parallel_rows(w.n_out, w.n_in, [&](size_t a, size_t b) {
                for (size_t j = a; j < b; ++j) ot[j] = dot_nvfp4_fp4(w.row(j), w.n_in, qx);
            });
        } else {
            parallel_rows(w.n_out, w.n_in, [&](size_t a, size_t b) {
                for (size_t j = a; j < b; ++j) ot[j] = dot_row(w.ty, w.row(j), xt, w.n_in);
            });
        }
    }
}
void matmul(const Weights& w, const float* x, size_t x_len, float* out) { matmul_impl(w, x, x_len, out, 0); }
void matmul_fp4act(const Weights& w, const float* x, size_t x_len, float* out) { matmul_impl(w, x, x_len, out, 1); }

// src/ops/naive.rs:180-218
void rope_neox(float* x, size_t len, size_t pos, size_t head_dim, size_t n_rot, size_t n_heads, float theta_base) {
    size_t per_row = head_dim * n_heads, half = n_rot / 2;
    for (size_t t = 0; t < len / per_row; ++t) {
        size_t p = pos + t;
        for (size_t h = 0; h < n_heads; ++h) {
            float* head = x + t * per_row + h * head_dim;
            for (size_t i = 0; i < half; ++i) {
                double freq = pow((double)theta_base, -2.0 * (double)i / (double)n_rot);
                double th = (double)p * freq;
                float sn = (float)sin(th), cs = (float)cos(th);
                float x0 = head[i], x1 = head[i + half];
                head[i] = x0 * cs - x1 * sn;
                head[i + half] = x0 * sn + x1 * cs;
            }
        }
    }
}

// src/ops/naive.rs:362-376
static void softmax_in_place(float* x, size_t n) {
    if (n == 0) return;
    float mx = -INFINITY;
    for (size_t i = 0; i < n; ++i) mx = fmaxf(mx, x[i]);
    float sum = 0.0f;
    for (size_t i = 0; i < n; ++i) { x[i] = expf(x[i] - mx); sum += x[i]; }
    for (size_t i = 0; i < n; ++i) x[i] /= sum;
}
void softmax(float* x, size_t len, size_t row) {
    if (row == 0) return;
    for (size_t r = 0; r < len; r += row) softmax_in_place(x + r, std::min(row, len - r));
}

// src/ops/naive.rs:420-466 for one (query row, kv head).
static void attend_kv_head(const Attn& a, size_t t, size_t h_kv, float* out, std::vector<float>& scores,
                           std::vector<float>& conv) {
    size_t hd = a.head_dim, group = a.group(), n_pos = a.n_pos_of(t);
    size_t off = h_kv * hd, q_row = t * a.n_head * hd;
    scores.resize(group * n_pos); conv.resize(hd);
    auto cvt = [&](uint16_t b) { return a.kv_bf16 ? bf16_to_f32(b) : f16_to_f32(b); };
    for (size_t s = 0; s < n_pos; ++s) {
        const uint16_t* key = a.k + s * a.kv_dim + off;
        for (size_t i = 0; i < hd; ++i) conv[i] = cvt(key[i]);
        for (size_t g = 0; g < group; ++g) {
            const float* q = a.q + q_row + (h_kv * group + g) * hd;
            float dot = 0.0f;
            for (size_t i = 0; i < hd; ++i) dot += q[i] * conv[i];
            scores[g * n_pos + s] = dot * a.scale;
        }
    }
    for (size_t g = 0; g < group; ++g) softmax_in_place(scores.data() + g * n_pos, n_pos);
    for (size_t i = 0; i < group * hd; ++i) out[i] = 0.0f;
    for (size_t s = 0; s < n_pos; ++s) {
        const uint16_t* val = a.v + s * a.kv_dim + off;
        for (size_t i = 0; i < hd; ++i) conv[i] = cvt(val[i]);
        for (size_t g = 0; g < group; ++g) {
            float w = scores[g * n_pos + s];
            float* o = out + g * hd;
            for (size_t i = 0; i < hd; ++i) o[i] += w * conv[i];
        }
    }
}

// src/ops/naive.rs:229-244
void attend(const Attn& a, float* out) {
    size_t per_kv = a.group() * a.head_dim, n_q = a.n_q();
    size_t units = n_q * a.n_head_kv;
    parallel_rows(units, a.n_pos * per_kv * 2, [&](size_t lo, size_t hi) {
        std::vector<float> scores, conv;
        for (size_t u = lo; u < hi; ++u) {
            size_t t = u / a.n_head_kv, h_kv = u % a.n_head_kv;
            attend_kv_head(a, t, h_kv, out + t * a.n_head * a.head_dim + h_kv * per_kv, scores, conv);
        }
    });
}

// src/ops/naive.rs:246-252
void silu_mul(float* gate, const float* up, size_t n) {
    for (size_t i = 0; i < n; ++i) { float g = gate[i]; gate[i] = g / (1.0f + expf(-g)) * up[i]; }
}
// src/ops/naive.rs:332-337
void sigmoid_mul(float* x, const float* g, size_t n) {
    for (size_t i = 0; i < n; ++i) x[i] *= 1.0f / (1.0f + expf(-g[i]));
}
// src/ops/mod.rs:600-604
void scale(float* buf, size_t n, float s) { for (size_t i = 0; i < n; ++i) buf[i] *= s; }
// src/ops/naive.rs:352-357
void add_assign(float* a, const float* b, size_t n) { for (size_t i = 0; i < n; ++i) a[i] += b[i]; }
// src/ops/mod.rs:1265-1270
void add_scaled(float* a, const float* b, size_t n, float s) { for (size_t i = 0; i < n; ++i) a[i] += b[i] * s; }
// src/ops/mod.rs:1228-1238
void add_scaled_rows(float* acc, size_t n, const float* rows, const float* scales, size_t n_rows) {
    for (size_t j = 0; j < n; ++j) {
        float v = 0.0f;
        for (size_t e = 0; e < n_rows; ++e) v += scales[e] * rows[e * n + j];
        acc[j] = v;
    }
}
// src/ops/mod.rs:1250-1253
void add_scaled_sigmoid(float* acc, const float* b, size_t n, const float* logit) {
    float s = 1.0f / (1.0f + expf(-logit[0]));
    add_scaled(acc, b, n, s);
}

// src/ops/naive.rs:254-273
void l2_norm_heads(float* x, size_t len, size_t head_dim, float eps) {
    for (size_t h = 0; h < len / head_dim; ++h) {
        float* head = x + h * head_dim;
        double sum = 0.0;
        for (size_t i = 0; i < head_dim; ++i) sum += (double)(head[i] * head[i]);
        float sc = 1.0f / fmaxf(sqrtf((float)sum), eps);
        for (size_t i = 0; i < head_dim; ++i) head[i] *= sc;
    }
}

// src/ops/naive.rs:275-315
void ssm_conv(float* state, const float* x, size_t x_len, const float* w, size_t w_len, size_t kernel, float* out) {
    size_t keep = kernel - 1, nc = w_len / kernel;
    for (size_t t = 0; t < x_len / nc; ++t) {
        const float* xt = x + t * nc; float* ot = out + t * nc;
        for (size_t c = 0; c < nc; ++c) {
            float* past = state + c * keep;
            float sum = 0.0f;
            for (size_t k = 0; k < keep; ++k) sum += past[k] * w[c * kernel + k];
            sum += xt[c] * w[c * kernel + keep];
            ot[c] = sum / (1.0f + expf(-sum));
            for (size_t k = 0; k + 1 < keep; ++k) past[k] = past[k + 1];
            past[keep - 1] = xt[c];
        }
    }
}

// src/ops/naive.rs:317-330
void gather_chunks(const float* src, size_t chunk, size_t stride, size_t offset, float* out, size_t out_len) {
    for (size_t c = 0; c < out_len / chunk; ++c) std::memcpy(out + c * chunk, src + c * stride + offset, chunk * 4);
}
// src/ops/mod.rs:730-742
void scatter_chunks(const float* src, size_t src_len, size_t chunk, size_t stride, size_t offset, float* dst) {
    for (size_t i = 0; i < src_len / chunk; ++i) std::memcpy(dst + offset + i * stride, src + i * chunk, chunk * 4);
}

// src/ops/naive.rs:86-135 (one token), 339-350 (tokens in order)
void delta_rule(const Delta& d, float* state, float* out) {
    size_t sk = d.head_k_dim, sv = d.head_v_dim;
    float q_scale = 1.0f / sqrtf((float)sk);
    size_t kper = d.n_k_heads * sk, vper = d.n_v_heads * sv;
    for (size_t t = 0; t < d.n_tokens; ++t) {
        parallel_rows(d.n_v_heads, sk * sv * 4, [&](size_t lo, size_t hi) {
            for (size_t h = lo; h < hi; ++h) {
                size_t kh = h % d.n_k_heads;  // modulo, not division (src/ops/mod.rs:411-413)
                const float* q = d.q + t * kper + kh * sk;
                const float* k = d.k + t * kper + kh * sk;
                const float* v = d.v + t * vper + h * sv;
                float* s = state + h * sk * sv;
                float a = d.alpha[t * d.n_v_heads + h] + d.dt_bias[h];
                float softplus = a > 20.0f ? a : logf(1.0f + expf(a));
                float g = expf(softplus * d.ssm_a[h]);
                float beta = 1.0f / (1.0f + expf(-d.beta[t * d.n_v_heads + h]));
                for (size_t i = 0; i < sk * sv; ++i) s[i] *= g;
                for (size_t j = 0; j < sv; ++j) {
                    float* row = s + j * sk;
                    float pred = 0.0f;
                    for (size_t i = 0; i < sk; ++i) pred += row[i] * k[i];
                    float delta = beta * (v[j] - pred);
                    for (size_t i = 0; i < sk; ++i) row[i] += k[i] * delta;
                    float o = 0.0f;
                    for (size_t i = 0; i < sk; ++i) o += row[i] * (q[i] * q_scale);
                    out[t * vper + h * sv + j] = o;
                }
            }
        });
    }
}

// src/ops/mod.rs:1421-1425 (f16); bf16 is this build's extension behind a switch.
void kv_write(uint16_t* slab, size_t offset, const float* src, size_t n, int bf16) {
    for (size_t i = 0; i < n; ++i) slab[offset + i] = bf16 ? f32_to_bf16(src[i]) : f32_to_f16(src[i]);
}

// src/ops/mod.rs:1191-1216
void route(const float* probs, size_t len, size_t n_expert, size_t n_used, Route& out) {
    size_t n_tok = len / (n_expert ? n_expert : 1);
    out.ids.clear(); out.weights.clear(); out.n_used = n_used;
    for (size_t t = 0; t < n_tok; ++t) {
        const float* p = probs + t * n_expert;
        size_t base = out.ids.size();
        for (size_t r = 0; r < n_used; ++r) {
            size_t best = SIZE_MAX;
            for (size_t e = 0; e < n_expert; ++e) {
                bool taken = false;
                for (size_t i = base; i < out.ids.size(); ++i) if (out.ids[i] == e) { taken = true; break; }
                if (taken) continue;
                if (best == SIZE_MAX || p[e] > p[best]) best = e;
            }
            out.ids.push_back(best);
        }
        float sum = 0.0f;
        for (size_t i = base; i < out.ids.size(); ++i) sum += p[out.ids[i]];
        float denom = fmaxf(sum, 6.103515625e-5f);
        for (size_t i = base; i < base + n_used; ++i) out.weights.push_back(p[out.ids[i]] / denom);
    }
}

// src/ops/mod.rs:1049-1088
void matmul_experts(const Experts& w, const Route& r, const float* x, size_t x_len, float* out, int fp4act) {
    size_t n_used = r.n_used ? r.n_used : 1, rows = x_len / w.n_in, np = r.ids.size();
    for (size_t i = 0; i < np; ++i) {
        size_t e = r.ids[i];
        size_t xr = rows == np ? i : (rows > 1 ? i / n_used : 0);
        float* row = out + i * w.n_out;
        matmul_impl(w.expert(e), x + xr * w.n_in, w.n_in, row, fp4act);
        if (w.scale) scale(row, w.n_out, w.scale[e]);
    }
}

// src/ops/mod.rs:1105-1117
void moe_glu(const Experts& gate, const Experts& up, const Route& r, const float* x, size_t x_len,
             float* out, float* scratch, int fp4act) {
    matmul_experts(gate, r, x, x_len, out, fp4act);
    matmul_experts(up, r, x, x_len, scratch, fp4act);
    silu_mul(out, scratch, r.ids.size() * gate.n_out);
}

// src/ops/mod.rs:1134-1171
void moe_finish(float* out, size_t at, size_t n, const float* rows, const Route& r,
                const float* shared, const float* logit, size_t logit_at) {
    size_t n_used = r.n_used ? r.n_used : 1, n_tok = r.weights.size() / n_used;
    for (size_t t = 0; t < n_tok; ++t) {
        float g = 1.0f / (1.0f + expf(-logit[logit_at + t]));
        const float* w = r.weights.data() + t * n_used;
        for (size_t j = 0; j < n; ++j) {
            float v = 0.0f;
            for (size_t e = 0; e < n_used; ++e) v += w[e] * rows[(t * n_used + e) * n + j];
            v += shared[t * n + j] * g;
            out[at + t * n + j] = v;
        }
    }
}

// src/profile.rs:192-213
uint32_t argmax_top2(const float* logits, size_t n, uint32_t* second) {
    size_t i1 = 0, i2 = SIZE_MAX;
    for (size_t i = 1; i < n; ++i) {
        float v = logits[i];
        if (v > logits[i1]) { i2 = i1; i1 = i; }
        else if (i2 == SIZE_MAX || v > logits[i2]) i2 = i;
    }
    if (second) *second = (uint32_t)i2;
    return (uint32_t)i1;
}

}  // namespace orc
