// Deterministic synthetic weights for the hybrid-MoE token loop, usable from host and device.
//
// The reference ships decoders only (src/quant/mod.rs); benchmark and parity inputs therefore
// come from this generator: a counter-based PRNG, a Gaussian built from IEEE add/mul/div/sqrt
// only (no libm, so the CPU and the GPU produce the same bits when neither contracts a*b+c),
// and the Q8_0 / NVFP4 weight quantisers. Element i of a tensor depends only on (key, i), so
// any shard can be generated independently and in any order.
//
// Compile device code with --fmad=false and host code with -ffp-contract=off.
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define SY_HD __host__ __device__ __forceinline__
#else
#define SY_HD inline
#endif

namespace synth {

SY_HD uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// FNV-1a over a tensor name; host only in practice.
inline uint64_t name_hash(const char* s) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (; *s; ++s) { h ^= (uint8_t)*s; h *= 0x100000001b3ull; }
    return h;
}
inline uint64_t tensor_key(uint64_t seed, const char* name) { return splitmix64(splitmix64(seed) ^ name_hash(name)); }

SY_HD uint64_t draw(uint64_t key, uint64_t i) { return splitmix64(key ^ (i * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull)); }

SY_HD double bits_to_double(uint64_t b) { double d; memcpy(&d, &b, 8); return d; }
SY_HD uint64_t double_to_bits(double d) { uint64_t b; memcpy(&b, &d, 8); return b; }
SY_HD float bits_to_float(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
SY_HD uint32_t float_to_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

// ln(x) for x >= 1 an integer-valued double below 2^33: exponent split plus the atanh series.
SY_HD double det_log(double x) {
    uint64_t b = double_to_bits(x);
    int e = (int)((b >> 52) & 0x7ff) - 1023;
    double m = bits_to_double((b & 0x000fffffffffffffull) | 0x3ff0000000000000ull);  // [1,2)
    if (m > 1.4142135623730951) { m = m * 0.5; e += 1; }
    double s = (m - 1.0) / (m + 1.0);
    double s2 = s * s;
    double p = 2.0 / 17.0;
    p = p * s2 + 2.0 / 15.0;
    p = p * s2 + 2.0 / 13.0;
    p = p * s2 + 2.0 / 11.0;
    p = p * s2 + 2.0 / 9.0;
    p = p * s2 + 2.0 / 7.0;
    p = p * s2 + 2.0 / 5.0;
    p = p * s2 + 2.0 / 3.0;
    p = p * s2 + 2.0;
    return (double)e * 0.6931471805599453 + p * s;
}

SY_HD double det_sin_small(double x) {  // |x| <= pi/4
    double x2 = x * x;
    double p = -1.0 / 1307674368000.0;   // -1/15!
    p = p * x2 + 1.0 / 6227020800.0;     //  1/13!
    p = p * x2 - 1.0 / 39916800.0;       // -1/11!
    p = p * x2 + 1.0 / 362880.0;         //  1/9!
    p = p * x2 - 1.0 / 5040.0;           // -1/7!
    p = p * x2 + 1.0 / 120.0;            //  1/5!
    p = p * x2 - 1.0 / 6.0;              // -1/3!
    return x + x * (x2 * p);
}
SY_HD double det_cos_small(double x) {  // |x| <= pi/4
    double x2 = x * x;
    double p = 1.0 / 20922789888000.0;   //  1/16!
    p = p * x2 - 1.0 / 87178291200.0;    // -1/14!
    p = p * x2 + 1.0 / 479001600.0;      //  1/12!
    p = p * x2 - 1.0 / 3628800.0;        // -1/10!
    p = p * x2 + 1.0 / 40320.0;          //  1/8!
    p = p * x2 - 1.0 / 720.0;            // -1/6!
    p = p * x2 + 1.0 / 24.0;             //  1/4!
    p = p * x2 - 0.5;
    return 1.0 + x2 * p;
}

// cos(2*pi*j/2^32) by integer quadrant reduction.
SY_HD double det_cos_turn(uint32_t j) {
    uint32_t q = j >> 30, r = j & 0x3fffffffu;
    const double HALF_PI = 1.5707963267948966;
    bool swap = r > 0x20000000u;
    double t = swap ? (double)(0x40000000u - r) : (double)r;
    double a = HALF_PI * (t * (1.0 / 1073741824.0));
    double c = swap ? det_sin_small(a) : det_cos_small(a);   // cos of the in-quadrant angle
    double s = swap ? det_cos_small(a) : det_sin_small(a);   // sin of the in-quadrant angle
    return q == 0 ? c : q == 1 ? -s : q == 2 ? -c : s;
}

// Standard normal deviate number i of stream `key` (Box-Muller, cosine branch).
SY_HD double gauss(uint64_t key, uint64_t i) {
    uint64_t r = draw(key, i);
    uint32_t hi = (uint32_t)(r >> 32), lo = (uint32_t)r;
    double k = (double)hi + 1.0;                        // u1 = k / 2^32 in (0, 1]
    double l = det_log(k) - 32.0 * 0.6931471805599453;  // ln u1 <= 0
    double rad = sqrt(-2.0 * l);
    return rad * det_cos_turn(lo);
}

// How a tensor's f32 values derive from the normal deviate z.
enum Dist : int {
    DIST_NORMAL = 0,     // std * z
    DIST_ONE_PLUS = 1,   // 1 + std * z            (norm weights)
    DIST_NEG_ABS = 2,    // -|std * z|             (ssm_a must be negative)
};
SY_HD float value(uint64_t key, uint64_t i, int dist, float std_) {
    float v = (float)(gauss(key, i) * (double)std_);
    if (dist == DIST_ONE_PLUS) return 1.0f + v;
    if (dist == DIST_NEG_ABS) return -fabsf(v);
    return v;
}

// ---- formats ----
SY_HD uint16_t f32_to_f16_rn(float f) {  // IEEE round-to-nearest-even (src/quant/half.rs:71-114 semantics)
    uint32_t bits = float_to_bits(f);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000);
    int exp = (int)((bits >> 23) & 0xff);
    uint32_t mant = bits & 0x007fffffu;
    if (exp == 0xff) return (uint16_t)(sign | 0x7c00 | (mant ? 0x0200 : 0));
    int e = exp - 127 + 15;
    if (e >= 0x1f) return (uint16_t)(sign | 0x7c00);
    if (e <= 0) {
        if (e < -10) return sign;
        uint32_t m = mant | 0x00800000u, shift = (uint32_t)(14 - e);
        uint32_t half = m >> shift, rem = m & ((1u << shift) - 1), halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half & 1))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t h = ((uint32_t)e << 10) | (mant >> 13), rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h++;
    return (uint16_t)(sign | h);
}

// Unsigned E4M3 scale, halved, 0 and 0x7f reading as 0 (src/quant/mod.rs:271-284).
SY_HD float ue4m3_half(uint8_t x) {
    if (x == 0 || x == 0x7f) return 0.0f;
    int exp = (x >> 3) & 0xf;
    int man = x & 7;
    // (8 + man) * 2^(exp - 7 - 3 - 1) for normals, man * 2^(-9 - 1) for subnormals: exact in f32.
    uint32_t pow2 = (uint32_t)(127 + (exp == 0 ? -10 : exp - 11)) << 23;
    return (float)(exp == 0 ? man : 8 + man) * bits_to_float(pow2);
}

// RN-even encoder onto codes 0..0x7e of the full-scale value 2*ue4m3_half(c), saturating at 448
// (src/quant/mod.rs:321-336).
SY_HD uint8_t ue4m3_encode_rn(float x) {
    if (!(x > 0.0f)) return 0;
    if (x >= 448.0f) return 0x7e;
    int lo = 0;
    for (int c = 1; c <= 0x7e; ++c) {
        if (2.0f * ue4m3_half((uint8_t)c) <= x) lo = c; else break;
    }
    float below = x - 2.0f * ue4m3_half((uint8_t)lo);        // exact: both are short binary values
    float above = 2.0f * ue4m3_half((uint8_t)(lo + 1)) - x;
    return (uint8_t)((below < above || (below == above && (lo & 1) == 0)) ? lo : lo + 1);
}

// Nearest E2M1 magnitude to |x|*e, first index on ties, sign in bit 3 (src/ops/naive.rs:794-806).
SY_HD uint8_t e2m1_nearest(float x, float e) {
    const float POS[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float ax = fabsf(x) * e;
    int best = 0;
    float best_err = fabsf(ax - POS[0]);
    for (int i = 1; i < 8; ++i) {
        float err = fabsf(ax - POS[i]);
        if (err < best_err) { best = i; best_err = err; }
    }
    return (uint8_t)(best | (x < 0.0f ? 8 : 0));
}

// ---- weight quantisers (this build's definition; the reference has none) ----
// Q8_0 block of 32: d = amax/127 stored as f16, q = roundf(v * (1/d)). 34 bytes out.
SY_HD void quantize_q8_0_block(const float* v, uint8_t* out) {
    float amax = 0.0f;
    for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
    float d = amax / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    uint16_t h = f32_to_f16_rn(d);
    out[0] = (uint8_t)(h & 0xff); out[1] = (uint8_t)(h >> 8);
    for (int j = 0; j < 32; ++j) {
        float r = roundf(v[j] * id);
        r = fminf(127.0f, fmaxf(-128.0f, r));
        out[2 + j] = (uint8_t)(int8_t)r;
    }
}

// NVFP4 block of 64 against the tensor's (or expert's) second scale s2 = amax/(6*448):
// per 16 values code c = rn((block_amax / s2) / 6), elements e2m1(v / s2, 0.5 / ue4m3_half(c)).
// Layout: 4 scale bytes, then byte 4+8s+j = code(j) | code(j+8) << 4 (src/quant/mod.rs:338-357).
SY_HD void quantize_nvfp4_block(const float* v, float s2, uint8_t* out) {
    for (int s = 0; s < 4; ++s) {
        const float* b = v + 16 * s;
        float amax = 0.0f;
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(b[j]));
        uint8_t c = s2 > 0.0f ? ue4m3_encode_rn((amax / s2) / 6.0f) : 0;
        float sc = ue4m3_half(c);
        float inv = sc > 0.0f ? 0.5f / sc : 0.0f;
        out[s] = c;
        for (int j = 0; j < 8; ++j) {
            uint8_t lo = s2 > 0.0f ? e2m1_nearest(b[j] / s2, inv) : 0;
            uint8_t hi = s2 > 0.0f ? e2m1_nearest(b[j + 8] / s2, inv) : 0;
            out[4 + 8 * s + j] = (uint8_t)(lo | (hi << 4));
        }
    }
}
SY_HD float nvfp4_second_scale(float amax) { return amax / (6.0f * 448.0f); }

}  // namespace synth
