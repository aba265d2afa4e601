// Device side of the deterministic synthetic-weight generator (synth.h): fills tensors in the file's
// block layouts directly in HBM, bit-identical to the CPU generator.
#include "itb_internal.cuh"
#include "synth.h"

__global__ void k_synth_f32(uint64_t key, uint64_t first, size_t n, int dist, float sd, float* out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = synth::value(key, first + i, dist, sd);
}
// One thread per Q8_0 block.
__global__ void k_synth_q8(uint64_t key, size_t n_blocks, int dist, float sd, uint8_t* raw) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    float v[32];
    for (int j = 0; j < 32; ++j) v[j] = synth::value(key, b * 32 + j, dist, sd);
    uint8_t o[34];
    synth::quantize_q8_0_block(v, o);
    for (int j = 0; j < 34; ++j) raw[b * 34 + j] = o[j];
}
// Per-expert max |v| (bits of a non-negative float order like unsigned integers).
__global__ void k_synth_amax(uint64_t key, uint64_t first_elem, size_t per_expert, int dist, float sd, unsigned* amax_bits) {
    size_t e = blockIdx.y;
    float m = 0.0f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < per_expert; i += (size_t)gridDim.x * blockDim.x)
        m = fmaxf(m, fabsf(synth::value(key, first_elem + e * per_expert + i, dist, sd)));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits + e, __float_as_uint(m));
}
// One thread per NVFP4 block of 64.
__global__ void k_synth_fp4(uint64_t key, uint64_t first_elem, size_t per_expert, size_t n_blocks, int dist, float sd,
                            const unsigned* amax_bits, float* scale2, uint8_t* raw) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    size_t e = (b * 64) / per_expert;
    float s2 = synth::nvfp4_second_scale(__uint_as_float(amax_bits[e]));
    if ((b * 64) % per_expert == 0) scale2[e] = s2;
    float v[64];
    for (int j = 0; j < 64; ++j) v[j] = synth::value(key, first_elem + b * 64 + j, dist, sd);
    uint8_t o[36];
    synth::quantize_nvfp4_block(v, s2, o);
    for (int j = 0; j < 36; ++j) raw[b * 36 + j] = o[j];
}

void itb_synth_f32(cudaStream_t st, uint64_t key, size_t n, int dist, float sd, float* out) {
    if (n) k_synth_f32<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(key, 0, n, dist, sd, out);
}
void itb_synth_q8_raw(cudaStream_t st, uint64_t key, size_t n_blocks, int dist, float sd, uint8_t* raw) {
    if (n_blocks) k_synth_q8<<<(unsigned)((n_blocks + 127) / 128), 128, 0, st>>>(key, n_blocks, dist, sd, raw);
}
// Experts [e_lo, e_hi) of a stack whose experts hold per_expert elements each; raw/scale2 index from e_lo.
void itb_synth_fp4_raw(cudaStream_t st, uint64_t key, size_t per_expert, size_t e_lo, size_t e_hi, int dist, float sd,
                       unsigned* amax_tmp, float* scale2, uint8_t* raw) {
    size_t ne = e_hi - e_lo;
    if (!ne) return;
    cudaMemsetAsync(amax_tmp, 0, ne * 4, st);
    dim3 g((unsigned)std::min<size_t>(64, (per_expert + 255) / 256), (unsigned)ne);
    k_synth_amax<<<g, 256, 0, st>>>(key, e_lo * per_expert, per_expert, dist, sd, amax_tmp);
    size_t nb = ne * per_expert / 64;
    k_synth_fp4<<<(unsigned)((nb + 63) / 64), 64, 0, st>>>(key, e_lo * per_expert, per_expert, nb, dist, sd, amax_tmp, scale2, raw);
}

extern "C" int itb_synth_values(itb_ctx* c, uint64_t key, uint64_t first, size_t n, int dist, float sd, float* out) {
    float* d = nullptr;
    ITB_CUDA_RET(c, cudaMalloc(&d, n * 4 + 4), 1);
    k_synth_f32<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(key, first, n, dist, sd, d);
    ITB_LAUNCHED(c);
    cudaError_t e = cudaMemcpyAsync(out, d, n * 4, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    cudaFree(d);
    if (e != cudaSuccess) { itb_fail(c, "synth_values", e); return 1; }
    return 0;
}
