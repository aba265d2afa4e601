// Kernels of the engine's multi-row path: several tokens at once, either one token of each of many sequences
// (batched decode) or many consecutive tokens of one sequence (prefill). Rows are token-major; row i belongs to
// sequence i / n_tok and is its token number i % n_tok of this pass. Matmuls run on the int8 MMA kernels
// (itb_mma.cuh, every weight row read once per 32 rows); the kernels here are the rest of a layer. All keep the
// CPU path's arithmetic order, so a prefill is bit-identical to feeding the tokens one at a time, which the
// reference asserts of its own backends (tests/qwen35.rs:94-139 there).
#pragma once
#include "itb_kernels.cuh"
#include "itb_tile.cuh"

namespace {

// F32 matrix against many rows (router logits, alpha/beta, shared-expert gate), tree mode. A block takes 8 weight rows
// (one per warp, held in registers) and F32_TOK token rows (staged in shared memory with every load in flight at once):
// two memory round trips per block, blocks for every (row group, token group). Per lane the products are summed in the
// order of f32_rows<false> (the one-token path), then the same shuffle tree, so a row gets the bits it gets alone.
// grid (ceil(n_out/8), ceil(n_rows/F32_TOK)), block 256, dynamic smem F32_TOK * n_in floats; n_in = 128 * NV.
constexpr int F32_TOK = 4;
template <int NV>
__global__ void __launch_bounds__(256) k_matmul_f32_rows(DevF32 w, const float* x, int n_rows, float* out) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* xs = (float*)smem;
    constexpr int n = 128 * NV;
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + wid, t0 = blockIdx.y * F32_TOK, nt = min(n_rows - t0, F32_TOK);
    float4 wv[NV];
    const float* wr = w.w + (size_t)min(row, w.n_out - 1) * n;
#pragma unroll
    for (int j = 0; j < NV; ++j) wv[j] = __ldg((const float4*)(wr + lane * 4 + 128 * j));
    constexpr int PER = F32_TOK * n / 4 / 256;   // float4 per thread of the token tile
    float4 xv[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = threadIdx.x + 256 * i, t = e / (n / 4);
        xv[i] = t < nt ? __ldg((const float4*)(x + (size_t)t0 * n) + e) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) ((float4*)xs)[threadIdx.x + 256 * i] = xv[i];
    __syncthreads();
    if (row >= w.n_out) return;
    for (int t = 0; t < nt; ++t) {
        const float* xr = xs + (size_t)t * n + lane * 4;
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const float4 v = *(const float4*)(xr + 128 * j);
            s += wv[j].x * v.x + wv[j].y * v.y + wv[j].z * v.z + wv[j].w * v.w;
        }
        s = warp_sum(s);
        if (lane == 0) out[(size_t)(t0 + t) * w.n_out + row] = s;
    }
}

// F32 matrix against many rows in the CPU path's own order (src/ops/naive.rs:49-56: a left fold over k of w[o][k] * x[r][k],
// product and sum rounded separately). With many rows there is a chain per (row, output), so no chain needs to be spread over
// lanes: a thread owns a 4 x 4 block of outputs and walks k in order -- a plain tiled SGEMM whose k loop is never reassociated
// or fused. grid (ceil(n_out / 64), ceil(n_rows / 64)), block 256; k tiles of 32 through shared memory, next tile in flight.
// FUSED (tolerance class, with opts dense=bf16tc): the same walk with one fused multiply-add per step -- half the instructions, and
// sums that differ from the CPU's by the product's rounding only.
constexpr int SG_T = 64, SG_K = 32;
template <bool FUSED = false>
__global__ void __launch_bounds__(256) k_sgemm_serial(DevF32 w, const float* __restrict__ x, int n_rows, float* out) {
    __shared__ float ws[2][SG_K][SG_T + 4], xs[2][SG_K][SG_T + 4];      // [k][output] and [k][row]: a thread reads 4 consecutive of each
    const int o0 = blockIdx.x * SG_T, r0 = blockIdx.y * SG_T, n = w.n_in;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;             // outputs 4*tx.., rows 4*ty..
    // loader: thread -> (line 0..63 of the tile, 8 consecutive k)
    const int ll = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 8;
    const float* wsrc = w.w + (size_t)min(o0 + ll, w.n_out - 1) * n + lk;
    const float* xsrc = x + (size_t)min(r0 + ll, n_rows - 1) * n + lk;
    float4 wa, wb, xa, xb;
    auto fetch = [&](int k0) {
        wa = __ldg((const float4*)(wsrc + k0)); wb = __ldg((const float4*)(wsrc + k0 + 4));
        xa = __ldg((const float4*)(xsrc + k0)); xb = __ldg((const float4*)(xsrc + k0 + 4));
    };
    auto stash = [&](int buf) {
        ws[buf][lk][ll] = wa.x; ws[buf][lk + 1][ll] = wa.y; ws[buf][lk + 2][ll] = wa.z; ws[buf][lk + 3][ll] = wa.w;
        ws[buf][lk + 4][ll] = wb.x; ws[buf][lk + 5][ll] = wb.y; ws[buf][lk + 6][ll] = wb.z; ws[buf][lk + 7][ll] = wb.w;
        xs[buf][lk][ll] = xa.x; xs[buf][lk + 1][ll] = xa.y; xs[buf][lk + 2][ll] = xa.z; xs[buf][lk + 3][ll] = xa.w;
        xs[buf][lk + 4][ll] = xb.x; xs[buf][lk + 5][ll] = xb.y; xs[buf][lk + 6][ll] = xb.z; xs[buf][lk + 7][ll] = xb.w;
    };
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    fetch(0); stash(0);
    __syncthreads();
    const int nk = n / SG_K;
    for (int t = 0; t < nk; ++t) {
        const int buf = t & 1;
        if (t + 1 < nk) fetch((t + 1) * SG_K);
#pragma unroll
        for (int kk = 0; kk < SG_K; ++kk) {
            const float4 wv = *(const float4*)&ws[buf][kk][4 * tx], xv = *(const float4*)&xs[buf][kk][4 * ty];
            const float wq[4] = {wv.x, wv.y, wv.z, wv.w}, xq[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = FUSED ? fmaf(wq[j], xq[i], acc[i][j]) : __fadd_rn(acc[i][j], __fmul_rn(wq[j], xq[i]));
        }
        if (t + 1 < nk) stash(buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + 4 * ty + i;
        if (r >= n_rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + 4 * tx + j;
            if (o < w.n_out) out[(size_t)r * w.n_out + o] = acc[i][j];
        }
    }
}

// The same for few rows or few outputs, where 64 x 64 tiles would leave most SMs idle: a thread per (row, output), 16 x 16 of
// them per block; every thread's k loop is the row's whole chain either way, so the small tile costs nothing but reuse. With
// so few blocks the global loads are what must not be waited for: tiles of 128 k arrive through a four-stage cp.async ring
// (three tiles in flight while one is folded). grid (ceil(n_out / 16), ceil(n_rows / 16)), block 256, dynamic shared memory
// sgemm_small_smem(); n_in a multiple of 128.
constexpr int SGS_K = 128, SGS_ST = SGS_K + 4, SGS_STAGES = 4;
constexpr size_t sgemm_small_smem() { return (size_t)SGS_STAGES * 2 * 16 * SGS_ST * 4; }
// Two matrices over the same rows in one launch (blockIdx.z picks; w1.w null: one matrix): the router and the shared expert's
// gate, or alpha and beta -- each alone is a handful of blocks walking a 2,048-long chain, and one after the other they cost twice.
template <bool FUSED = false>
__global__ void __launch_bounds__(256) k_sgemm_serial_small(DevF32 w0, const float* __restrict__ x, int n_rows, float* out0, DevF32 w1 = DevF32{}, float* out1 = nullptr) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* ring = (float*)smem;                    // [stage][w | x][16 lines][SGS_ST]
    const DevF32 w = blockIdx.z ? w1 : w0;
    float* out = blockIdx.z ? out1 : out0;
    if ((int)blockIdx.x * 16 >= w.n_out) return;
    const int o0 = blockIdx.x * 16, r0 = blockIdx.y * 16, n = w.n_in, nk = n / SGS_K;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;            // output o0 + tx, row r0 + ty
    auto fetch = [&](int t) {
        if (t < nk) {
            float* st = ring + (size_t)(t % SGS_STAGES) * 2 * 16 * SGS_ST;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = threadIdx.x + 256 * i, m = c >> 9, line = (c & 511) >> 5, k4 = (c & 31) * 4;      // 2 matrices x 16 lines x 32 chunks
                const float* src = m ? x + (size_t)min(r0 + line, n_rows - 1) * n : w.w + (size_t)min(o0 + line, w.n_out - 1) * n;
                cp_async16(st + (m * 16 + line) * SGS_ST + k4, src + (size_t)t * SGS_K + k4, true);
            }
        }
        cp_async_commit();
    };
    for (int t = 0; t < SGS_STAGES - 1; ++t) fetch(t);
    float acc = 0.0f;
    for (int t = 0; t < nk; ++t) {
        cp_async_wait<SGS_STAGES - 2>();
        __syncthreads();                           // tile t has landed for everyone; everyone is done with tile t - 1
        fetch(t + SGS_STAGES - 1);                 // into the slot tile t - 1 used
        const float* st = ring + (size_t)(t % SGS_STAGES) * 2 * 16 * SGS_ST;
        const float* wr = st + tx * SGS_ST; const float* xr = st + (16 + ty) * SGS_ST;
#pragma unroll 8
        for (int kk = 0; kk < SGS_K; kk += 4) {
            const float4 a = *(const float4*)(wr + kk), c = *(const float4*)(xr + kk);
            if (FUSED) { acc = fmaf(a.x, c.x, acc); acc = fmaf(a.y, c.y, acc); acc = fmaf(a.z, c.z, acc); acc = fmaf(a.w, c.w, acc); }
            else {
                acc = __fadd_rn(acc, __fmul_rn(a.x, c.x)); acc = __fadd_rn(acc, __fmul_rn(a.y, c.y));
                acc = __fadd_rn(acc, __fmul_rn(a.z, c.z)); acc = __fadd_rn(acc, __fmul_rn(a.w, c.w));
            }
        }
    }
    cp_async_wait<0>();
    if (r0 + ty < n_rows && o0 + tx < w.n_out) out[(size_t)(r0 + ty) * w.n_out + o0 + tx] = acc;
}

// RMSNorm + Q8_0 quantisation of each row (src/ops/naive.rs:139-152, :653-675): normalised f32 row, int8 quants,
// scales. grid = rows, block 256.
__global__ void __launch_bounds__(256) k_norm_quant(const float* x, const float* w, int n, float eps, float* xn_out, int8_t* xq, float* xs) {
    extern __shared__ __align__(16) unsigned char smem[];
    double* red = (double*)smem;
    float* xn = (float*)(red + 32);
    const size_t r = blockIdx.x;
    if (block_rms_norm(x + r * n, w, n, eps, xn, red, xq + r * n, xs + r * (n / 32))) {   // quantised in the same pass
        if (xn_out) for (int i = threadIdx.x; i < n / 4; i += blockDim.x) ((float4*)(xn_out + r * n))[i] = ((const float4*)xn)[i];
        return;
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b = wid; b < n / 32; b += nw) {
        float v = xn[b * 32 + lane], d;
        xq[r * n + b * 32 + lane] = warp_quant_q8(v, &d);
        if (lane == 0) xs[r * (n / 32) + b] = d;
        if (xn_out) xn_out[r * n + b * 32 + lane] = v;
    }
}

// Depthwise causal conv (src/ops/naive.rs:275-315), every (row, channel) on its own thread: the window of row t is
// the sequence's earlier rows of this pass, or the saved state where it reaches before the pass. Writes the
// PRE-activation sum to `out` (the input rows stay intact for the neighbours). grid (ceil(nc/128), rows).
__global__ void k_conv_rows(const float* state, size_t state_stride, const float* x, float* out, int n_tok, int nc, const float* w, int kernel) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nc) return;
    const size_t r = blockIdx.y;
    const int s = (int)(r / n_tok), t = (int)(r % n_tok), keep = kernel - 1;
    const float* st = state + (size_t)s * state_stride + (size_t)c * keep;
    float sum = 0.0f;
    for (int k = 0; k < keep; ++k) {
        const int idx = t - keep + k;
        const float past = idx >= 0 ? x[((size_t)s * n_tok + idx) * nc + c] : st[keep + idx];
        sum += past * w[(size_t)c * kernel + k];
    }
    sum += x[r * nc + c] * w[(size_t)c * kernel + keep];
    out[r * nc + c] = sum;
}
// The same for a kernel of 4 taps, CONV_T consecutive tokens of one sequence per thread: the three earlier inputs slide along
// in registers and the channel's taps are read once, so an output costs one load and one store instead of eight loads. The sums
// are the same expressions in the same order. grid (ceil(nc/128), n_seq * ceil(n_tok / CONV_T)).
constexpr int CONV_T = 8;
__global__ void __launch_bounds__(128) k_conv_rows4(const float* state, size_t state_stride, const float* __restrict__ x, float* __restrict__ out, int n_tok, int nc, const float* __restrict__ w) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nc) return;
    const int chunks = (n_tok + CONV_T - 1) / CONV_T, s = blockIdx.y / chunks, t0 = (blockIdx.y % chunks) * CONV_T;
    const float4 wv = *(const float4*)(w + (size_t)c * 4);
    const float* st = state + (size_t)s * state_stride + (size_t)c * 3;
    const float* xs = x + (size_t)s * n_tok * nc + c;
    float p0 = t0 >= 3 ? xs[(size_t)(t0 - 3) * nc] : st[t0], p1 = t0 >= 2 ? xs[(size_t)(t0 - 2) * nc] : st[t0 + 1], p2 = t0 >= 1 ? xs[(size_t)(t0 - 1) * nc] : st[t0 + 2];
    float cur[CONV_T];
#pragma unroll
    for (int i = 0; i < CONV_T; ++i) cur[i] = t0 + i < n_tok ? xs[(size_t)(t0 + i) * nc] : 0.0f;
#pragma unroll
    for (int i = 0; i < CONV_T; ++i) {
        if (t0 + i >= n_tok) break;
        float sum = 0.0f;
        sum += p0 * wv.x;
        sum += p1 * wv.y;
        sum += p2 * wv.z;
        sum += cur[i] * wv.w;
        out[((size_t)s * n_tok + t0 + i) * nc + c] = sum;
        p0 = p1; p1 = p2; p2 = cur[i];
    }
}
// The window each sequence leaves behind: its last kernel-1 inputs, oldest first. grid (ceil(nc/128), n_seq).
__global__ void k_conv_state(float* state, size_t state_stride, const float* x, int n_tok, int nc, int kernel) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (c >= nc) return;
    const int keep = kernel - 1;
    float* st = state + (size_t)s * state_stride + (size_t)c * keep;
    float nv[8];
    for (int k = 0; k < keep; ++k) {
        const int idx = n_tok - keep + k;
        nv[k] = idx >= 0 ? x[((size_t)s * n_tok + idx) * nc + c] : st[keep + idx];
    }
    for (int k = 0; k < keep; ++k) st[k] = nv[k];
}

// Everything of the GatedDeltaNet block that does not depend on the state, per row: SiLU of the conv sums,
// l2-norm of q and k (q also scaled by 1/sqrt(sk)), the decay g and the write strength beta
// (src/model/qwen35.rs:1280-1316, src/ops/naive.rs:101-107, :254-273). grid (rows, 2*n_k + n_v), block sk.
__global__ void k_gdn_pre(const float* conv, int cd, const float* alpha, const float* beta, const float* ssm_a, const float* dt_bias,
                          int sk, int n_k, int n_v, float eps, float* qh, float* kh, float* vh, float* gb) {
    __shared__ double red[8];
    const size_t r = blockIdx.x;
    const int u = blockIdx.y, d = threadIdx.x, key_dim = n_k * sk;
    const float* cv = conv + r * cd;
    if (u < 2 * n_k) {
        const bool is_q = u < n_k;
        const int h = is_q ? u : u - n_k;
        float v = silu_f(cv[(is_q ? 0 : key_dim) + h * sk + d]);
        double acc = warp_sum_d((double)(v * v));
        if ((d & 31) == 0) red[d >> 5] = acc;
        __syncthreads();
        double tot = 0.0;
        for (int w = 0; w < sk / 32; ++w) tot += red[w];
        float sc = 1.0f / fmaxf(sqrtf((float)tot), eps);
        v = v * sc;
        if (is_q) v = v * (1.0f / sqrtf((float)sk));
        (is_q ? qh : kh)[(r * n_k + h) * sk + d] = v;
    } else {
        const int h = u - 2 * n_k;
        vh[(r * n_v + h) * sk + d] = silu_f(cv[2 * key_dim + h * sk + d]);
        if (d == 0) {
            float a = alpha[r * n_v + h] + dt_bias[h];
            float sp = a > 20.0f ? a : log_f(1.0f + exp_f(a));
            gb[(r * n_v + h) * 2] = exp_f(sp * ssm_a[h]);
            gb[(r * n_v + h) * 2 + 1] = sigmoid_f(beta[r * n_v + h]);
        }
    }
}

// The recurrence itself (src/ops/naive.rs:109-132). A block is (value head, 32 value rows, sequence); a warp takes 8 of
// the rows, FOUR lanes per row, each lane holding a quarter of the row's state in registers across the pass's tokens.
// The CPU's serial sums over the 128 keys are kept to the bit: lane 0 of a row adds its quarter's products in order
// and hands the running sum to lane 1, and so on, so the chain is the CPU's chain; what the split buys is four times
// the warps (the chain's latency is hidden by other rows) and a quarter of the per-lane multiplies. The next token's
// k, q, v, g, beta are fetched while the current one is computed.
template <int SK>
__global__ void __launch_bounds__(128) k_gdn_scan(const float* qh, const float* kh, const float* vh, const float* gb, int n_tok, int n_k, int n_v,
                                                  float* state, size_t state_stride, float* out) {
    constexpr int CW = SK / 4;             // state columns per lane
    constexpr int DEPTH = 4;               // tokens whose operands are in flight (cp.async ring, one group per token)
    constexpr int SLOT = 2 * SK + 8 + 4;   // floats per token and warp: k | q | v of the warp's 8 rows | g, beta, pad
    __shared__ __align__(16) float ring_all[4][DEPTH][SLOT];
    const int h = blockIdx.x, s = blockIdx.z, khd = h % n_k, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int r = lane >> 2, part = lane & 3, j0 = blockIdx.y * 32 + wid * 8, j = j0 + r;      // j: value row of the head
    float* sg = state + (size_t)s * state_stride + ((size_t)h * SK + j) * SK + part * CW;
    float S[CW];
#pragma unroll
    for (int i = 0; i < CW; i += 4) { const float4 v = *(const float4*)(sg + i); S[i] = v.x; S[i + 1] = v.y; S[i + 2] = v.z; S[i + 3] = v.w; }
    auto fetch = [&](int t) {
        if (t < n_tok) {
            const size_t row = (size_t)s * n_tok + t;
            float* slot = ring_all[wid][t % DEPTH];
            if (lane * 4 < SK) {
                cp_async16(slot + lane * 4, kh + (row * n_k + khd) * SK + lane * 4, true);
                cp_async16(slot + SK + lane * 4, qh + (row * n_k + khd) * SK + lane * 4, true);
            }
            if (lane < 2) cp_async16(slot + 2 * SK + lane * 4, vh + (row * n_v + h) * SK + j0 + lane * 4, true);
            if (lane == 2) {
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(slot + 2 * SK + 8);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(gb + (row * n_v + h) * 2));
            }
        }
        cp_async_commit();
    };
    for (int t = 0; t < DEPTH - 1; ++t) fetch(t);
    float po[CW];
#pragma unroll
    for (int i = 0; i < CW; ++i) po[i] = 0.0f;
#pragma unroll 1
    for (int t = 0; t < n_tok; ++t) {
        cp_async_wait<DEPTH - 2>();
        __syncwarp();
        fetch(t + DEPTH - 1);            // refills the slot token t-1 used: every lane is past it (the __syncwarp above)
        const float* slot = ring_all[wid][t % DEPTH];
        const float v = slot[2 * SK + r], g = slot[2 * SK + 8], b = slot[2 * SK + 9];
        float kk[CW], pr[CW];
#pragma unroll
        for (int i = 0; i < CW; i += 4) {
            const float4 k4 = *(const float4*)(slot + part * CW + i);
            kk[i] = k4.x; kk[i + 1] = k4.y; kk[i + 2] = k4.z; kk[i + 3] = k4.w;
        }
#pragma unroll
        for (int i = 0; i < CW; ++i) { S[i] = S[i] * g; pr[i] = S[i] * kk[i]; }
        // Two serial sums side by side: this token's prediction (needed before the state can move on) and the
        // PREVIOUS token's read-out, whose products po were formed last trip. They do not depend on each other,
        // so their adds interleave and the second chain's latency disappears behind the first.
        float run = 0.0f, runo = 0.0f;
#pragma unroll
        for (int ph = 0; ph < 4; ++ph) {
            float a = run, c = runo;
#pragma unroll
            for (int i = 0; i < CW; ++i) { a += pr[i]; c += po[i]; }
            run = __shfl_sync(0xffffffffu, a, (lane & ~3) | ph);
            runo = __shfl_sync(0xffffffffu, c, (lane & ~3) | ph);
        }
        if (part == 0 && t > 0) out[(((size_t)s * n_tok + t - 1) * n_v + h) * SK + j] = runo;
        const float d = b * (v - run);
#pragma unroll
        for (int i = 0; i < CW; i += 4) {
            const float4 q4 = *(const float4*)(slot + SK + part * CW + i);
            S[i] = S[i] + kk[i] * d; po[i] = S[i] * q4.x;
            S[i + 1] = S[i + 1] + kk[i + 1] * d; po[i + 1] = S[i + 1] * q4.y;
            S[i + 2] = S[i + 2] + kk[i + 2] * d; po[i + 2] = S[i + 2] * q4.z;
            S[i + 3] = S[i + 3] + kk[i + 3] * d; po[i + 3] = S[i + 3] * q4.w;
        }
    }
    {
        float runo = 0.0f;                  // read-out of the last token
#pragma unroll
        for (int ph = 0; ph < 4; ++ph) {
            float c = runo;
#pragma unroll
            for (int i = 0; i < CW; ++i) c += po[i];
            runo = __shfl_sync(0xffffffffu, c, (lane & ~3) | ph);
        }
        if (part == 0 && n_tok > 0) out[(((size_t)s * n_tok + n_tok - 1) * n_v + h) * SK + j] = runo;
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < CW; i += 4) *(float4*)(sg + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
}

// Gated RMSNorm of the recurrence's output, the SiLU(z) gate and the Q8_0 quantisation of the result
// (src/model/qwen35.rs:1319-1325). grid (rows, n_v), block sv.
__global__ void k_gdn_post(const float* o, const float* z, const float* norm_w, int sv, int n_v, float eps, int8_t* out_q, float* out_s) {
    __shared__ double red[8];
    const size_t r = blockIdx.x;
    const int h = blockIdx.y, d = threadIdx.x;
    const size_t idx = (r * n_v + h) * sv + d;
    const float v = o[idx];
    double acc = warp_sum_d((double)(v * v));
    if ((d & 31) == 0) red[d >> 5] = acc;
    __syncthreads();
    double tot = 0.0;
    for (int w = 0; w < sv / 32; ++w) tot += red[w];
    const float mean = (float)(tot / (double)sv);
    const float sc = 1.0f / sqrtf(mean + eps);
    const float core = v * sc * norm_w[d];
    const float val = silu_f(z[idx]) * core;
    float dq;
    const int8_t q = warp_quant_q8(val, &dq);
    out_q[idx] = q;
    if ((d & 31) == 0) out_s[idx / 32] = dq;
}

// Attention prologue per (row, head): as k_attn_prep, the row's sequence and position derived from the pass
// shape: sequence = row / n_tok, position = pos[sequence] + row % n_tok. grid (n_head + 2*n_head_kv, rows).
struct AttnPrepRows {
    const float* qg; const float* k; const float* v;
    const float* q_norm; const float* k_norm;
    float* q_out; float* g_out;
    uint16_t* kslab; uint16_t* vslab; size_t slab_stride;
    const int* pos; int* npos_out; int n_tok;
    int hd, n_head, n_head_kv, n_rot; float theta, eps; int bf16;
};
__global__ void k_attn_prep_rows(AttnPrepRows p) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* val = (float*)smem;
    __shared__ double red[8];
    const int job = blockIdx.x, d = threadIdx.x, hd = p.hd, kvd = p.n_head_kv * hd;
    const size_t r = blockIdx.y;
    const int s = (int)(r / p.n_tok), pos = p.pos[s] + (int)(r % p.n_tok);
    if (job == 0 && d == 0) p.npos_out[r] = pos + 1;
    const bool is_q = job < p.n_head, is_k = !is_q && job < p.n_head + p.n_head_kv;
    const int hk = is_q ? job : is_k ? job - p.n_head : job - p.n_head - p.n_head_kv;
    float v;
    if (is_q) {
        v = p.qg[r * 2 * hd * p.n_head + (size_t)hk * 2 * hd + d];
        p.g_out[(r * p.n_head + hk) * hd + d] = p.qg[r * 2 * hd * p.n_head + (size_t)hk * 2 * hd + hd + d];
    } else {
        v = (is_k ? p.k : p.v)[r * kvd + hk * hd + d];
    }
    if (is_q || is_k) {
        double acc = warp_sum_d((double)(v * v));
        if ((d & 31) == 0) red[d >> 5] = acc;
        __syncthreads();
        double tot = 0.0;
        for (int w = 0; w < hd / 32; ++w) tot += red[w];
        float mean = (float)(tot / (double)hd);
        float sc = 1.0f / sqrtf(mean + p.eps);
        v = v * sc * (is_q ? p.q_norm : p.k_norm)[d];
        val[d] = v;
        __syncthreads();
        const int half = p.n_rot / 2;
        if (d < half) {
            double freq = pow((double)p.theta, -2.0 * (double)d / (double)p.n_rot);
            double th = (double)pos * freq;
            float sn = (float)sin(th), cs = (float)cos(th);
            float x0 = val[d], x1 = val[d + half];
            val[d] = x0 * cs - x1 * sn;
            val[d + half] = x0 * sn + x1 * cs;
        }
        __syncthreads();
        v = val[d];
    }
    if (is_q) p.q_out[(r * p.n_head + hk) * hd + d] = v;
    else {
        uint16_t* slab = (is_k ? p.kslab : p.vslab) + (size_t)s * p.slab_stride + (size_t)pos * kvd + hk * hd + d;
        *slab = p.bf16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v);
    }
}

// Combine of the attention splits per (row, head) with the sigmoid gate and Q8_0 quantisation; positions per row.
__global__ void k_attn_combine_rows(const float* part_acc, const float* part_ml, int n_split, int hd, const float* gate,
                                    const int* n_pos_row, int n_head, int8_t* out_q, float* out_s) {
    const size_t th = blockIdx.x;
    const int d = threadIdx.x;
    const size_t r = th / n_head;
    const int n_pos = n_pos_row[r], per = max(ATTN_MIN_SPLIT, (n_pos + n_split - 1) / n_split), n_act = (n_pos + per - 1) / per;
    float M = -INFINITY;
    for (int s = 0; s < n_act; ++s) M = fmaxf(M, part_ml[(th * n_split + s) * 2]);
    float L = 0.0f, A = 0.0f;
    for (int s = 0; s < n_act; ++s) {
        float ms = part_ml[(th * n_split + s) * 2];
        float c = ms == -INFINITY ? 0.0f : __expf(ms - M);
        L += part_ml[(th * n_split + s) * 2 + 1] * c;
        A += part_acc[(th * n_split + s) * hd + d] * c;
    }
    float v = A / L;
    v *= sigmoid_f(gate[th * hd + d]);
    float dq;
    int8_t q = warp_quant_q8(v, &dq);
    out_q[th * hd + d] = q;
    if ((d & 31) == 0) out_s[(th * hd + d) / 32] = dq;
}

__global__ void k_advance_pos(int* pos, int n_seq, int by) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_seq) pos[i] += by;
}
// Rows of the last token of each sequence, gathered for the LM head: out[s] = x[s*n_tok + n_tok-1].
__global__ void k_gather_last(const float* x, int n, int n_tok, float* out) {
    const int s = blockIdx.x;
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[(size_t)s * n + i] = x[((size_t)s * n_tok + n_tok - 1) * n + i];
}

}  // namespace

// =====================================================================================================
// Routed experts for many rows: route once per row, group the (row, pick) pairs by expert, and run each
// expert's rows through the int8-MMA NVFP4 kernels so an expert's weights are read once per pass
// (the reference groups the same way, kernels/moe.cuh:62-133 there; the order inside an expert is ascending
// pair index, so results do not depend on scheduling).
// =====================================================================================================
namespace {

// Softmax over all experts + top-k per row (src/model/qwen35.rs:1626-1638, src/ops/mod.rs:1191-1216). One warp per row.
__global__ void k_route_rows(const float* router, int n_rows, int n_expert, int n_used, int32_t* ids_out, float* w_out) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int ne32 = (n_expert + 31) & ~31;
    float* probs = (float*)smem + wid * ne32;
    const int r = blockIdx.x * nw + wid;
    if (r >= n_rows) return;
    const float* lg = router + (size_t)r * n_expert;
    float mx = -INFINITY;
    for (int i = lane; i < n_expert; i += 32) mx = fmaxf(mx, lg[i]);
    mx = warp_max(mx);
    for (int i = lane; i < ne32; i += 32) probs[i] = i < n_expert ? exp_f(lg[i] - mx) : 0.0f;
    __syncwarp();
    float sum = 0.0f;
    if (lane == 0) for (int i = 0; i < n_expert; ++i) sum += probs[i];
    sum = __shfl_sync(0xffffffffu, sum, 0);
    for (int i = lane; i < n_expert; i += 32) probs[i] /= sum;
    __syncwarp();
    int32_t ids[16];
    float wts[16];
    warp_topk_any(probs, n_expert, n_used, ids, wts);
    if (lane == 0)
        for (int k = 0; k < n_used; ++k) { ids_out[(size_t)r * n_used + k] = ids[k]; w_out[(size_t)r * n_used + k] = wts[k]; }
}

// Counting sort of the pairs by expert, ascending pair index inside an expert. One block, thread e owns expert e.
// off: [n_expert + 1], list: [n_pairs] pair indices.
__global__ void k_group_pairs(const int32_t* ids, int n_pairs, int n_expert, int* off, int* list) {
    extern __shared__ int cnt[];
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) {
        int c = 0;
        for (int i = 0; i < n_pairs; ++i) c += ids[i] == e;
        cnt[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < n_expert; ++e) { off[e] = acc; acc += cnt[e]; }
        off[n_expert] = acc;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) {
        int at = off[e];
        for (int i = 0; i < n_pairs; ++i) if (ids[i] == e) list[at++] = i;
    }
}

// Activation rows of up to 32 listed pairs into the MMA tile: pair p reads row p / div of (xq, xs).
__device__ __forceinline__ void stage_pairs(const int8_t* xq, const float* xs, int k, const int* list, int n, int div, int8_t* sq, float* ss) {
    const int nb = k / 32, stride = mma_act_stride(k);
    for (int i = threadIdx.x; i < MMA_TOK * (k / 16); i += blockDim.x) {
        int t = i / (k / 16), c = i % (k / 16);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < n) v = *(const uint4*)(xq + (size_t)(list[t] / div) * k + c * 16);
        *(uint4*)(sq + (size_t)t * stride + c * 16) = v;
    }
    for (int i = threadIdx.x; i < MMA_TOK * nb; i += blockDim.x) {
        int t = i / nb;
        ss[i] = t < n ? xs[(size_t)(list[t] / div) * nb + i % nb] : 0.0f;
    }
    __syncthreads();
}

// Gate and up of one expert for its pairs, SiLU-gated: h[pair][row] (src/ops/mod.rs:1105-1117). grid (n_expert, ff/128).
__global__ void __launch_bounds__(256) k_glu_grouped(DevFp4 gate, DevFp4 up, const int8_t* xq, const float* xs, int n_used,
                                                     const int* off, const int* list, float* h) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int e = blockIdx.x, k = gate.n_in, ff = gate.n_out, nsb = k / 16;
    const int p0 = off[e], p1 = off[e + 1];
    if (p0 >= p1) return;
    const int el = fp4_slot(gate, e);
    if (el < 0) return;
    int8_t* sq = (int8_t*)smem;
    float* ss = (float*)(sq + (size_t)MMA_TOK * mma_act_stride(k));
    const int r0 = blockIdx.y * MMA_ROWS + (threadIdx.x >> 5) * 16;
    const size_t eo = (size_t)el * ff;
    const bool has_g = gate.scale2 != nullptr, has_u = up.scale2 != nullptr;
    const float sg2 = has_g ? gate.scale2[el] : 1.0f, su2 = has_u ? up.scale2[el] : 1.0f;
    for (int t0 = p0; t0 < p1; t0 += MMA_TOK) {
        const int n = min(MMA_TOK, p1 - t0);
        __syncthreads();
        stage_pairs(xq, xs, k, list + t0, n, n_used, sq, ss);
        if (r0 < ff) {
            float g[4][4], u[4][4];
            mma_fp4_rows16<4, 8>(gate.nib + eo * (k / 2), gate.sc + eo * nsb, k, ff, r0, sq, ss, 0, g);
            mma_fp4_rows16<4, 8>(up.nib + eo * (k / 2), up.sc + eo * nsb, k, ff, r0, sq, ss, 0, u);
            const int lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int t = 8 * j + 2 * tq + (i & 1), row = r0 + gq + (i >> 1) * 8;
                    if (t < n && row < ff) {
                        float gv = has_g ? g[j][i] * sg2 : g[j][i], uv = has_u ? u[j][i] * su2 : u[j][i];
                        h[(size_t)list[t0 + t] * ff + row] = silu_f(gv) * uv;
                    }
                }
        }
    }
}

// Down projection of one expert for its pairs: o[pair][row], times the expert's second scale
// (src/ops/mod.rs:1049-1088). grid (n_expert, n_out/128). Activation rows are per pair (div = 1).
__global__ void __launch_bounds__(256) k_down_grouped(DevFp4 down, const int8_t* hq, const float* hs, const int* off, const int* list, float* o) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int e = blockIdx.x, k = down.n_in, n_out = down.n_out, nsb = k / 16;
    const int p0 = off[e], p1 = off[e + 1];
    if (p0 >= p1) return;
    const int el = fp4_slot(down, e);
    if (el < 0) return;
    int8_t* sq = (int8_t*)smem;
    float* ss = (float*)(sq + (size_t)MMA_TOK * mma_act_stride(k));
    const int r0 = blockIdx.y * MMA_ROWS + (threadIdx.x >> 5) * 16;
    const size_t eo = (size_t)el * n_out;
    const bool has_s = down.scale2 != nullptr;
    const float s2 = has_s ? down.scale2[el] : 1.0f;
    for (int t0 = p0; t0 < p1; t0 += MMA_TOK) {
        const int n = min(MMA_TOK, p1 - t0);
        __syncthreads();
        stage_pairs(hq, hs, k, list + t0, n, 1, sq, ss);
        if (r0 < n_out) {
            float acc[4][4];
            mma_fp4_rows16<4, 8>(down.nib + eo * (k / 2), down.sc + eo * nsb, k, n_out, r0, sq, ss, 0, acc);
            mma_foreach<4>(acc, r0, n_out, 0, [&](int t, int row, float v) {
                if (t < n) o[(size_t)list[t0 + t] * n_out + row] = has_s ? v * s2 : v;
            });
        }
    }
}

// Q8_0 quantisation of rows of f32 (block per row).
__global__ void k_quant_rows(const float* x, int n, int8_t* xq, float* xs) {
    const size_t r = blockIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b = wid; b < n / 32; b += nw) {
        float d;
        xq[r * n + b * 32 + lane] = warp_quant_q8(x[r * n + b * 32 + lane], &d);
        if (lane == 0) xs[r * (n / 32) + b] = d;
    }
}
// silu(gate) * up of the shared expert per row, quantised (src/model/qwen35.rs:1669-1678). block per row.
__global__ void k_shared_act_rows(const float* sg, const float* su, int n, int8_t* q, float* s) {
    const size_t r = blockIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int b = wid; b < n / 32; b += nw) {
        const size_t i = r * n + b * 32 + lane;
        float d;
        q[i] = warp_quant_q8(silu_f(sg[i]) * su[i], &d);
        if (lane == 0) s[r * (n / 32) + b] = d;
    }
}
// Weighted expert sum in pick order, gated shared expert, residual add (src/ops/mod.rs:1134-1171, src/model/qwen35.rs:1090).
__global__ void k_moe_finish_rows(float* x, int n, const float* o, const float* wts, int n_used, const float* shared, const float* logit, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t r = i / n; const int j = (int)(i % n);
    const float g = sigmoid_f(logit[r]);
    float v = 0.0f;
    for (int k = 0; k < n_used; ++k) v += wts[r * n_used + k] * o[(r * n_used + k) * n + j];
    v += shared[r * n + j] * g;
    x[i] += v;
}

}  // namespace

namespace {

// Pairs grouped by expert without a serial scan: counts by shared-memory atomics, an exclusive scan, then each
// pair takes the next free place of its expert. The order inside an expert depends on scheduling; results do
// not, since every pair is computed on its own. One block.
__global__ void __launch_bounds__(1024) k_group_pairs_fast(const int32_t* ids, int n_pairs, int n_expert, int* off, int* list) {
    extern __shared__ int cnt[];    // [n_expert] counts, then cursors
    __shared__ int s_off[1025];
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&cnt[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x < 32) {
        // warp scan over experts in chunks of 32
        int carry = 0;
        for (int e0 = 0; e0 < n_expert; e0 += 32) {
            const int e = e0 + threadIdx.x;
            const int c = e < n_expert ? cnt[e] : 0;
            int inc = c;
            for (int o = 1; o < 32; o <<= 1) { int v = __shfl_up_sync(0xffffffffu, inc, o); if ((int)threadIdx.x >= o) inc += v; }
            if (e < n_expert) { off[e] = carry + inc - c; s_off[e] = carry + inc - c; }
            carry += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (threadIdx.x == 0) off[n_expert] = carry;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) { const int e = ids[i]; list[s_off[e] + atomicAdd(&cnt[e], 1)] = i; }
}

}  // namespace
