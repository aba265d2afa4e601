// Decode attention for callers that must not allocate device memory.
//
// Who needs this: a serving loop that cannot tolerate the device-wide synchronisation cudaMalloc/cudaFree
// imply, or a host that handed this backend a fixed memory budget at start-up and forbids it to grow. Such a
// caller owns its q / KV / output buffers already; the only thing the ordinary entry point (itb_attend) would
// still allocate is the scratch that holds the split-K partial results. Here that scratch is a fixed array
// inside the library image, so the call allocates nothing -- no cudaMalloc, no cudaFree, no library routine
// that allocates.
//
// Limits (checked, with a message): one query row, n_head <= 64, head_dim in {64,128,256}, at most 8 query
// heads per KV head. The scratch is ITB_NOALLOC_SCRATCH_BYTES (about 2.1 MB) per GPU that loads the library,
// held until the process exits.
//
// Sharing: every call on a device uses the same array. Nothing in it has to start at zero -- each call first
// overwrites every partial it later reads (splits without positions get neutral values) -- but two calls that
// overlap on the GPU (different streams, or different threads) would overwrite each other's partials: run
// them one after the other.
//
// Threads: like the rest of the library, one host thread at a time (the first-call set-up below is not locked).
//
// First call on a device: looks up the array's device address (cudaGetSymbolAddress) and raises two kernels'
// dynamic shared-memory limit. Make that first call with the device current and before starting any stream
// capture; later calls only launch kernels.
#include "itb_kernels.cuh"

#define ITB_NOALLOC_MAX_HEADS 64
#define ITB_NOALLOC_MAX_HD 256
#define ITB_NOALLOC_MAX_SPLIT 32
#define ITB_NOALLOC_SCRATCH_FLOATS (ITB_NOALLOC_MAX_HEADS * ITB_NOALLOC_MAX_SPLIT * (ITB_NOALLOC_MAX_HD + 2))
#define ITB_NOALLOC_SCRATCH_BYTES (ITB_NOALLOC_SCRATCH_FLOATS * 4)

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_attn_scratch[ITB_NOALLOC_SCRATCH_FLOATS];

static float* g_scratch_dev[64];   // per device ordinal: the array's device address, looked up once
static bool g_ready[64];

static int fail(char* err, size_t cap, const char* msg) {
    if (err && cap) snprintf(err, cap, "%s", msg);
    return 1;
}

extern "C" int itb_attend_decode_noalloc(void* stream, const float* q_dev, const uint16_t* k_dev, const uint16_t* v_dev,
                                         size_t kv_dim, size_t n_pos, size_t head_dim, size_t n_head, size_t n_head_kv, float scale,
                                         int kv_bf16, float* out_dev, char* err, size_t err_cap) {
    if (!q_dev || !k_dev || !v_dev || !out_dev) return fail(err, err_cap, "attend_decode_noalloc: null device pointer");
    if (n_head == 0 || n_head_kv == 0 || n_head % n_head_kv) return fail(err, err_cap, "attend_decode_noalloc: query heads do not divide into kv heads");
    if (n_head > ITB_NOALLOC_MAX_HEADS) return fail(err, err_cap, "attend_decode_noalloc: more than 64 query heads exceeds the built-in scratch");
    if (n_head / n_head_kv > 8) return fail(err, err_cap, "attend_decode_noalloc: more than 8 query heads per kv head");
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return fail(err, err_cap, "attend_decode_noalloc: head_dim must be 64, 128 or 256");
    if (n_pos == 0 || n_pos > 0x7fffffffu || kv_dim < n_head_kv * head_dim) return fail(err, err_cap, "attend_decode_noalloc: bad n_pos or kv_dim");
    // The kernel reads head_dim/32 consecutive K (and V) elements per lane with one vector load, so every row of every
    // head must start on that boundary: kv_dim a multiple of head_dim/32 elements, the slabs aligned to 2*(head_dim/32) bytes.
    const size_t dpl = head_dim / 32;
    if (kv_dim > 0x7fffffffu || kv_dim % dpl) return fail(err, err_cap, "attend_decode_noalloc: kv_dim must be a multiple of head_dim/32 and fit an int");
    if (((uintptr_t)k_dev | (uintptr_t)v_dev) % (2 * dpl)) return fail(err, err_cap, "attend_decode_noalloc: k_dev and v_dev must be aligned to 2*(head_dim/32) bytes");
    if (((uintptr_t)q_dev | (uintptr_t)out_dev) % 4) return fail(err, err_cap, "attend_decode_noalloc: q_dev and out_dev must be 4-byte aligned");
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(err, err_cap, "attend_decode_noalloc: no current CUDA device");
    const size_t smem = (size_t)8 * 8 * 2 * 4 + (size_t)8 * 8 * head_dim * 4;
    if (!g_ready[dev]) {
        // once per device, with that device current: the symbol's address on THIS device
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_attn_scratch);
        if (e != cudaSuccess || !p) return fail(err, err_cap, cudaGetErrorString(e));
        e = cudaFuncSetAttribute(k_attn_partial<256, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 8 * 2 * 4 + 8 * 8 * 256 * 4);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(k_attn_partial<128, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 8 * 2 * 4 + 8 * 8 * 128 * 4);
        if (e != cudaSuccess) return fail(err, err_cap, cudaGetErrorString(e));
        g_scratch_dev[dev] = p;
        g_ready[dev] = true;
    }
    int n_split = (int)((n_pos + 255) / 256);
    if (n_split > ITB_NOALLOC_MAX_SPLIT) n_split = ITB_NOALLOC_MAX_SPLIT;
    float* part_acc = g_scratch_dev[dev];
    float* part_ml = part_acc + (size_t)n_head * n_split * head_dim;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((unsigned)n_head_kv, 1, (unsigned)n_split);
    switch (head_dim) {
        case 64: k_attn_partial<64, 8><<<grid, 256, smem, st>>>(q_dev, k_dev, v_dev, (int)kv_dim, (int)n_pos, 1, (int)n_head, (int)n_head_kv, scale, kv_bf16, nullptr, part_acc, part_ml); break;
        case 128: k_attn_partial<128, 8><<<grid, 256, smem, st>>>(q_dev, k_dev, v_dev, (int)kv_dim, (int)n_pos, 1, (int)n_head, (int)n_head_kv, scale, kv_bf16, nullptr, part_acc, part_ml); break;
        default: k_attn_partial<256, 8><<<grid, 256, smem, st>>>(q_dev, k_dev, v_dev, (int)kv_dim, (int)n_pos, 1, (int)n_head, (int)n_head_kv, scale, kv_bf16, nullptr, part_acc, part_ml); break;
    }
    k_attn_combine<<<(unsigned)n_head, (unsigned)head_dim, 0, st>>>(part_acc, part_ml, n_split, (int)head_dim, nullptr, out_dev);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(err, err_cap, cudaGetErrorString(e));
    return 0;
}
