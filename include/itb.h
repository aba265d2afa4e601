/* itb.h -- C ABI of the B200 backend for the Inferred-Thoughts hybrid-MoE token loop.
 *
 * The boundary this library drops in behind is the reference's backend trait `Ops`
 * (src/ops/mod.rs:489-1426), selected by `--backend` (src/main.rs:167-168, :535-625). Each
 * `itb_*` op below replaces one trait method; the citation beside it is the method it stands for.
 *
 * Conventions carried over from the reference's own device backend:
 *  - Activation buffers are HOST addresses used as handles: the library keeps a device mirror per
 *    host address (src/ops/cuda/ops/residency.rs:23-57). Never pass a sub-slice of a buffer the
 *    library has seen under another address (src/ops/mod.rs:531-536).
 *  - Ops return nothing; the first failure is kept and fetched with itb_take_error()
 *    (src/ops/cuda/ops/mod.rs:91-110).
 *  - Weights are borrowed host bytes in the file's block layout, uploaded and repacked on first
 *    sight, keyed by pointer (src/ops/cuda/mod.rs:59-68). Keep them alive and unmoved.
 *  - Single-threaded per context (src/ops/cuda/mod.rs:756).
 *
 * There is no CPU fallback: every entry point fails loudly when no CUDA device is usable.
 */
#ifndef ITB_H
#define ITB_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct itb_ctx itb_ctx;

/* ggml type codes understood (src/gguf/types.rs): 0 F32, 1 F16, 8 Q8_0 (34 B / 32), 40 NVFP4 (36 B / 64). */
enum { ITB_F32 = 0, ITB_F16 = 1, ITB_Q8_0 = 8, ITB_NVFP4 = 40 };

/* src/ops/mod.rs:62-92 `Weights` */
typedef struct { const uint8_t* data; size_t bytes; uint32_t ggml_type; size_t n_in, n_out; int pooled; } itb_weights;
/* src/ops/mod.rs:107-152 `Experts`; scale = n_expert little-endian f32 or NULL (= 1.0) */
typedef struct { const uint8_t* data; size_t bytes; uint32_t ggml_type; size_t n_in, n_out, n_expert;
                 const uint8_t* scale; size_t scale_bytes; } itb_experts;
/* src/ops/mod.rs:176-218 `Route`. on_device=1: ids/weights stay in the library (the ctx's current
 * route); on_device=0: host arrays of n_tok*n_used entries that the ops must honour. */
typedef struct { int on_device; size_t n_used, n_tok; const size_t* ids; const float* weights; } itb_route_t;
/* src/ops/mod.rs:228-276 `Attn`; k/v are the layer's slabs (host addresses, keys of device slabs). */
typedef struct { const float* q; size_t q_len; const uint16_t* k; const uint16_t* v; size_t slab_len;
                 size_t kv_dim, n_pos, head_dim, n_head, n_head_kv; float scale; } itb_attn;
/* src/ops/mod.rs:337-358 `Delta`; n_tokens is derived by the reference from v's length. */
typedef struct { const float *q, *k, *v, *alpha, *beta, *ssm_a, *dt_bias; size_t n_tokens,
                 head_k_dim, head_v_dim, n_k_heads, n_v_heads; } itb_delta;

/* ---- context ---- */
/* opts: "key=value,..." ; keys: kv=f16|bf16 (default f16, the reference's KV dtype, src/cache/mod.rs:8-15),
 * exact=0|1 (1, default: every sum in the CPU path's order -- F32 dots fold serially, attention walks positions in order --
 *   so results equal the CPU path bit for bit; 0: tree-summed F32 dots, split-K attention, and the many-token kernels below),
 * many-token passes (each also selectable on its own under exact=1; all tolerance class except dense=q8tc):
 *   dense=q8tc     dense Q8_0 matmuls as tcgen05 int8 MMAs per 32-element block, scales applied in CPU order (bit-identical),
 *   dense=f16tc    dense Q8_0 matmuls as f16 tcgen05 GEMMs: weights and the Q8_0-quantised activation rows dequantised to f16
 *                  (int8 * block scale, rounded to nearest), f32 accumulators; 2 more bytes of device memory per dense weight;
 *                  wins over dense=q8tc where both are given; with exact=0 the small F32 matrices run as fused-multiply-add tiles,
 *   experts=fp4tc  routed experts as FP4 x FP4 block-scaled tcgen05 GEMMs (the reference's default device arithmetic,
 *                  src/ops/cuda/mod.rs:239-248; exact=1 keeps the library-exact SiLU in their epilogue),
 *   attn=mma       causal attention as 16-bit matrix products over (token, head) tiles,
 *   gdn=chunk      the delta rule chunk-parallel (64-token chunks),
 * libm=cr (log stays correctly rounded; by default the kernels' log follows the host C library's logf bit for bit through a
 * correction table built at the first itb_create of the process, 61 MB per device, because that is what the CPU path calls). */
int         itb_create(int device_ordinal, const char* opts, itb_ctx** out);   /* 0 ok */
void        itb_destroy(itb_ctx*);
const char* itb_take_error(itb_ctx*);   /* NULL if none; clears (src/ops/cuda/ops/mod.rs:91-110) */
const char* itb_last_create_error(void);

/* ---- pass / residency protocol (src/ops/mod.rs:1360-1419) ---- */
void itb_begin_pass(itb_ctx*, size_t n_tokens);                /* :1372 */
void itb_end_pass(itb_ctx*);                                    /* :1376 */
void itb_host_wrote(itb_ctx*, const float* buf, size_t len);    /* :1360 */
void itb_host_needs(itb_ctx*, float* buf, size_t len);          /* :1363 */
void itb_forget_state(itb_ctx*);                                /* :1401 */
void itb_read_state(itb_ctx*, float* host, size_t len);         /* :1419 */
void itb_reserve_activations(itb_ctx*, size_t bytes);           /* :1305 */
/* KV slabs live on the device once written; this brings one home (tests, checkpoints). */
void itb_read_kv(itb_ctx*, uint16_t* slab, size_t slab_len);

/* ---- ops, one per trait method ---- */
void itb_rms_norm(itb_ctx*, const float* x, size_t x_len, const float* w, size_t w_len, float eps, float* out);   /* :497 */
void itb_rms_norm_heads(itb_ctx*, float* x, size_t len, const float* w, size_t head_dim, float eps);              /* :502 */
void itb_matmul(itb_ctx*, const itb_weights*, const float* x, size_t x_len, float* out, size_t out_len);          /* :520 */
void itb_matmul_pair(itb_ctx*, const itb_weights* a, const itb_weights* b, const float* x, size_t x_len,
                     float* out_a, size_t out_a_len, float* out_b, size_t out_b_len);                             /* :1012 */
void itb_rope_neox(itb_ctx*, float* x, size_t len, size_t pos, size_t head_dim, size_t n_rot, size_t n_heads, float theta); /* :545 */
void itb_softmax(itb_ctx*, float* x, size_t len, size_t row);                                                     /* :567 */
void itb_attend(itb_ctx*, const itb_attn*, float* out, size_t out_len);                                           /* :589 */
void itb_kv_write(itb_ctx*, uint16_t* slab, size_t slab_len, size_t offset, const float* src, size_t n);          /* :1421 */
void itb_silu_mul(itb_ctx*, float* gate, const float* up, size_t n);                                              /* :592 */
void itb_sigmoid_mul(itb_ctx*, float* x, const float* g, size_t n);                                               /* :746 */
void itb_scale(itb_ctx*, float* buf, size_t n, float s);                                                          /* :600 */
void itb_add_assign(itb_ctx*, float* a, const float* b, size_t n);                                                /* :788 */
void itb_add_scaled(itb_ctx*, float* a, const float* b, size_t n, float s);                                       /* :1265 */
void itb_add_scaled_rows(itb_ctx*, float* acc, size_t n, const float* rows, const float* scales, size_t n_rows);  /* :1228 */
void itb_add_scaled_sigmoid(itb_ctx*, float* acc, const float* b, size_t n, const float* logit);                  /* :1250 */
void itb_gather_chunks(itb_ctx*, const float* src, size_t src_len, size_t chunk, size_t stride, size_t offset,
                       float* out, size_t out_len);                                                               /* :664 */
void itb_scatter_chunks(itb_ctx*, const float* src, size_t src_len, size_t chunk, size_t stride, size_t offset,
                        float* dst, size_t dst_len);                                                              /* :730 */
void itb_l2_norm_heads(itb_ctx*, float* x, size_t len, size_t head_dim, float eps);                               /* :613 */
void itb_ssm_conv(itb_ctx*, float* state, size_t state_len, const float* x, size_t x_len, const float* w,
                  size_t w_len, size_t kernel, float* out);                                                       /* :647 */
void itb_delta_rule(itb_ctx*, const itb_delta*, float* state, size_t state_len, float* out, size_t out_len);      /* :785 */
/* Chooses on the device and returns on_device=1 in *out (src/ops/cuda/ops/mod.rs:299-302). */
void itb_route(itb_ctx*, float* probs, size_t len, size_t n_expert, size_t n_used, itb_route_t* out);               /* :1191 */
void itb_matmul_experts(itb_ctx*, const itb_experts*, const itb_route_t*, const float* x, size_t x_len,
                        float* out, size_t out_len);                                                              /* :1049 */
void itb_moe_glu(itb_ctx*, const itb_experts* gate, const itb_experts* up, const itb_route_t*, const float* x,
                 size_t x_len, float* out, size_t out_len, float* scratch);                                       /* :1105 */
void itb_moe_finish(itb_ctx*, float* out, size_t out_len, size_t at, size_t n, const float* rows, size_t rows_len,
                    const itb_route_t*, const float* shared, const float* logit, size_t logit_at);                  /* :1134 */
/* "A hint, not work" (src/ops/mod.rs:915-924): at this seam every expert stack a context has seen is wholly resident in HBM, so
 * there is nothing to fetch ahead and the call returns at once, as the trait's default does. The tiered engine applies the hint
 * itself (itb_tier_counters below). */
void itb_prefetch_hint(itb_ctx*, const itb_weights* next_router, const float* x, size_t x_len, size_t k);         /* :924 */
/* Brings the current device route home: n_tok*n_used ids and weights (tests; breaks graph capture). */
void itb_read_route(itb_ctx*, int32_t* ids, float* weights, size_t n);

/* ---- observability (src/ops/mod.rs:1300-1358) ---- */
int  itb_config_report(itb_ctx*, char* buf, size_t cap);
void itb_device_report(itb_ctx*);
/* kernels launched by this context since creation */
uint64_t itb_launch_count(itb_ctx*);

/* ==== model / engine level =====================================================================
 * The reference drives the ops above from Qwen35::forward (src/model/qwen35.rs:956-1127) under
 * Engine::{prefill,decode,generate} (src/engine/mod.rs:352-437). The same two layers are provided
 * natively so a token step is a handful of fused kernels replayed as one CUDA graph:
 * the reference hides launch cost the same way (src/ops/cuda/mod.rs:600-647).
 */
typedef struct {
    uint32_t n_layer, n_embd, n_head, n_head_kv, head_dim, n_vocab;
    float rope_theta, rms_eps;
    uint32_t n_rot, ssm_d_conv, ssm_d_inner, ssm_d_state, ssm_dt_rank, ssm_n_group, full_attention_interval;
    uint32_t n_expert, n_expert_used, expert_ff, shared_ff;
} itb_model_dims;   /* src/model/qwen35.rs:193-249 `Config` + `Moe` */

typedef struct itb_model itb_model;
typedef struct itb_engine itb_engine;

int  itb_model_create(itb_ctx*, const itb_model_dims*, itb_model** out);
void itb_model_destroy(itb_model*);
/* Tensor by GGUF name (src/model/qwen35.rs:755-858) from host bytes in the file's block layout.
 * `scale`: n_expert f32 for NVFP4 expert stacks (the `.scale` tensor), else NULL. */
int  itb_model_set_tensor(itb_model*, const char* name, uint32_t ggml_type, const void* data, size_t bytes,
                          const float* scale, size_t n_scale);
/* Load a GGUF v3 file of architecture qwen35moe (src/gguf/mod.rs:143-296, src/model/qwen35.rs:333-486, :755-858): the
 * hyper-parameters come from its metadata, every tensor (F32, F16, Q8_0, NVFP4, `<name>.scale` beside expert stacks) goes
 * to the device through itb_model_set_tensor straight from the mapping. On failure returns non-zero with a message in err. */
int  itb_model_load_gguf(itb_ctx*, const char* path, itb_model** out, char* err, size_t err_cap);
void itb_model_dims_of(itb_model*, itb_model_dims* out);   /* the hyper-parameters a model was created or loaded with */
/* Fill every tensor from the deterministic generator, on the device (seeded synthetic weights).
 * expert_lo/expert_hi restrict routed-expert storage to [lo,hi) (expert-parallel shard); 0,0 = all. */
int  itb_model_synth(itb_model*, uint64_t seed, uint32_t expert_lo, uint32_t expert_hi);
/* Regenerate one synthetic tensor in the file's block layout and copy it to the host. */
int  itb_model_synth_read(itb_model*, uint64_t seed, const char* name, void* out, size_t bytes, float* scale_out);
/* Algorithmic bytes one decode step reads/writes at the given fill (weights once, state r+w, KV read). */
uint64_t itb_model_decode_bytes(itb_model*, uint32_t n_seq, uint32_t n_pos, uint32_t distinct_experts_per_layer);

/* n_seq independent sequences (the reference engine holds one, src/engine/mod.rs:44-59). */
int  itb_engine_create(itb_model*, uint32_t n_ctx, uint32_t n_seq, itb_engine** out);
/* Expert tiering, HBM <-> pinned host memory (the reference's GCLOCK expert tiers: src/cache, src/ops/cuda/experts.rs:2179-2234,
 * ops/placement.rs:33-84). itb_model_offload_experts moves the routed-expert stacks of a loaded model to pinned host memory;
 * itb_engine_create_tiered then keeps `capacity` (layer, expert) entries (gate + up + down) in HBM pools. Per MoE layer of a
 * pass the routing ids are read on the host, missing experts are copied in over the slots GCLOCK gives up (entries the pass
 * itself uses are leased), and the grouped expert kernels read through an id -> slot table. Results are bit-identical to an
 * untiered engine. capacity >= n_seq * n_expert_used; a prefill pass is cut to capacity / n_expert_used rows.
 * itb_engine_tier_stats: hits, misses, evictions, bytes copied. itb_gclock_*: the policy alone (host only). */
int  itb_model_offload_experts(itb_model*);
int  itb_engine_create_tiered(itb_model*, uint32_t n_ctx, uint32_t n_seq, uint32_t capacity, itb_engine** out);
void itb_engine_tier_stats(itb_engine*, uint64_t* out4);
/* The reference's TierCounters (src/ops/mod.rs:360-401) for one engine, as far as they exist here: fetched / fetch_bytes: experts
 * copied from the host tier into an HBM slot; picks_wait_us: host time waiting for a layer's routing ids; prefetch_reads /
 * prefetch_used: experts brought in by the prefetch hint and how many of those a later pick hit (the hint of src/ops/mod.rs:915-924
 * is applied inside the tiered engine when ITB_TIER_PREFETCH=<guesses per row> is set at its creation: layer il + 1's router on
 * layer il's router input, copies on a second stream while layer il's experts run; it changes no value the model computes);
 * lookups / host_reads: expert picks and how many missed the pool; slots, slot_bytes, pool_bytes; vram_free / vram_total from the
 * driver; mirrors / mirror_bytes: activation copies of the op seam; weight_bytes, kv_bytes, resident_bytes. The reference's
 * file-tier fields (read_us, upload_us, writes_us, picks_copy_us, oversubscribed) have no counterpart: the lower tier is pinned
 * host memory. */
typedef struct { uint64_t fetched, fetch_bytes, picks_wait_us, prefetch_reads, prefetch_used, lookups, host_reads, slot_bytes, slots, pool_bytes,
                 vram_free, vram_total, mirrors, mirror_bytes, weight_bytes, kv_bytes, resident_bytes; } itb_tier_counters_t;
int  itb_tier_counters(itb_engine*, itb_tier_counters_t* out);
void* itb_gclock_create(uint32_t capacity, uint32_t n_keys);
void itb_gclock_destroy(void*);
void itb_gclock_next_pass(void*);
int  itb_gclock_touch(void*, int64_t key, int* hit, int64_t* evicted);   /* slot, or -1: every slot leased by this pass */
/* Phase timeline (observability; the reference's counterpart is its per-op profiler, src/profile.rs): arm `slots`
 * launch slots (0 disarms), run single-sequence decode steps, read back slots * 16 words. Thread 0 of block 0 of the
 * step's n-th structured launch stores (nanoseconds << 8) | kernel id at word n * 16 + phase for each of its phase
 * marks; words never written stay 0. Costs one predicate per mark when disarmed. */
int  itb_timeline_arm(itb_engine*, uint32_t slots);
long itb_timeline_read(itb_engine*, uint64_t* out_words, uint32_t slots);
/* Expert parallelism over `world` processes, one GPU each (the reference's placement seam: src/ops/mod.rs:1024-1048;
 * its grouped kernels: kernels/moe.cuh:62-133). The model must hold exactly experts [rank*E/world, (rank+1)*E/world)
 * (itb_model_synth with that range, or set_tensor of that slice); everything else is replicated and each rank runs its
 * own n_seq sequences. Per MoE layer: all-gather of the quantised rows and routing, local experts over the pairs that
 * name them, sum reduce-scatter of the per-pair output rows (one non-zero contribution each, so the result is exact and
 * equals the single-GPU bits). Every rank must make the same engine calls with the same shapes.
 * itb_ep_unique_id: 128 bytes naming a new NCCL communicator (rank 0 makes them; hand the same bytes to every rank). */
int  itb_ep_unique_id(uint8_t* out128);
int  itb_engine_create_ep(itb_model*, uint32_t n_ctx, uint32_t n_seq, const uint8_t* unique_id128, int rank, int world, itb_engine** out);
void itb_engine_destroy(itb_engine*);
void itb_engine_reset(itb_engine*);                                               /* src/engine/mod.rs:296-308 */
uint32_t itb_engine_pos(itb_engine*, uint32_t seq);
/* Engine::checkpoint / restore (src/engine/mod.rs:255-294): positions + recurrent state of every sequence into a host buffer of
 * itb_engine_checkpoint_bytes; restore returns the engine to it (the KV cache is simply truncated to the saved positions). */
size_t itb_engine_checkpoint_bytes(itb_engine*);
int  itb_engine_checkpoint(itb_engine*, void* out, size_t cap);
int  itb_engine_restore(itb_engine*, const void* data, size_t bytes);
/* Engine::prefill (src/engine/mod.rs:352-356) for every sequence in lockstep: tokens [n_seq][n] host ids in,
 * logits of each sequence's last token out, [n_seq][n_vocab] (may be NULL). */
int  itb_engine_prefill(itb_engine*, const uint32_t* tokens, size_t n, float* logits_out);
/* Engine::decode for every sequence at once: tokens[n_seq] in; logits_out [n_seq][n_vocab] (may be NULL),
 * next_out[n_seq] greedy argmax (strict '>', lowest index wins, src/profile.rs:192-213) (may be NULL). */
int  itb_engine_decode(itb_engine*, const uint32_t* tokens, float* logits_out, uint32_t* next_out);
/* Device-resident greedy loop: `steps` decode steps feeding each argmax back in, no host traffic inside. */
int  itb_engine_decode_loop(itb_engine*, const uint32_t* first_tokens, uint32_t steps, uint32_t* tokens_out);
/* Engine::generate (src/engine/mod.rs:399-437) for sequence 0: prefill, then greedy tokens; each step
 * copies the token id to the device and the chosen id back. Returns tokens produced, <0 on error. */
long itb_engine_generate(itb_engine*, const uint32_t* prompt, size_t n_prompt, size_t max_new, uint32_t* out);
/* Last step's routing decisions [moe layer][seq][n_used] (integer parity checks). */
int  itb_engine_read_routes(itb_engine*, int32_t* ids, size_t cap);
/* Recurrent state / KV of one sequence, layer il (absolute layer index) */
int  itb_engine_read_ssm_state(itb_engine*, uint32_t seq, uint32_t il, float* out, size_t len);
/* Device time of the last decode step or loop in milliseconds (CUDA events on the engine's stream). */
float itb_engine_last_ms(itb_engine*);
/* How single-token decode steps of this engine run: 1 = one persistent cooperative kernel per step (a block per SM walks the
 * step's stages with grid barriers between them while producer warps stream every stage's weights through shared-memory
 * rings with bulk asynchronous copies, ahead of the dependency chain); 0 = the chain of fused kernels replayed as a CUDA
 * graph (the reference hides launch cost the same way, src/ops/cuda/mod.rs:600-647), with the reason in `why`. The one-kernel
 * step needs a single-sequence plain engine and every matrix row a multiple of 256 elements, and is selected by ITB_MEGA=1.
 * Its waits are bounded (ITB_MEGA_WAIT_MS, default 2000): one that runs out makes the call fail with a message. */
int  itb_engine_decode_path(itb_engine*, char* why, size_t cap);
uint64_t itb_engine_launches_per_step(itb_engine*);

/* Per-kernel-class totals of one eagerly launched decode step, timed with a CUDA event after every launch:
 * launches, summed milliseconds, summed algorithmic bytes (weights once, state read+write, KV read). */
typedef struct { char name[32]; uint32_t launches; float ms; uint64_t bytes; } itb_kernel_stat;
int  itb_engine_profile_step(itb_engine*, const uint32_t* tokens, itb_kernel_stat* out, size_t cap, size_t* n_out);

/* Decode attention that allocates nothing. No counterpart in the reference: added for callers that must not
 * allocate device memory while serving (cudaMalloc/cudaFree synchronise the whole device) or that run under a
 * memory budget fixed at start-up. All pointers are DEVICE pointers the caller already owns: q [n_head*head_dim]
 * f32, k/v KV slabs (f16 bits, or bf16 bits if kv_bf16) position-major with stride kv_dim, out
 * [n_head*head_dim] f32; `stream` is a cudaStream_t (NULL = default stream). One query row attends over
 * positions [0, n_pos). The split-K partials live in a fixed ~2.1 MB array inside the library (held by every
 * GPU that loads it until the process exits); limits: n_head <= 64, head_dim in {64,128,256}, at most 8 query
 * heads per KV head -- anything beyond is refused with a message in `err`. Alignment (also checked): kv_dim a
 * multiple of head_dim/32 elements, k/v aligned to 2*(head_dim/32) bytes, q/out to 4 bytes. One host thread at a time,
 * like every other entry point. The first call on a device looks the
 * array's address up: make it with that device current and before any stream capture. Calls share the array, so
 * calls that overlap on the GPU race; issue them one after the other. Returns 0, or 1 with `err` filled. */
int  itb_attend_decode_noalloc(void* stream, const float* q_dev, const uint16_t* k_dev, const uint16_t* v_dev,
                               size_t kv_dim, size_t n_pos, size_t head_dim, size_t n_head, size_t n_head_kv, float scale,
                               int kv_bf16, float* out_dev, char* err, size_t err_cap);

/* The measured ceiling of the block-scaled FP4 tensor-core instruction this backend's expert GEMMs are built on
 * (tcgen05.mma kind::mxf4nvf4, M 128 x N `n` (128 or 256) x K 64 per instruction, f32 accumulators in tensor memory): one block
 * per SM issues `iters` accumulating MMAs on unchanging shared-memory operands, nothing else in the loop, and the accumulators
 * are verified afterwards -- the reference measures its own instructions' ceilings the same way (tests/cuda_ops.rs:5899-5925).
 * tflops_out: dense TFLOP/s, best of `reps` launches by CUDA events; status_out: 0 verified, 1 a (bounded) wait ran out,
 * 2 accumulators wrong; mma_cycles_out: SM cycles per MMA on the slowest block. Returns non-zero on a call error. */
int  itb_fp4_ceiling(itb_ctx*, int n, int iters, int reps, double* tflops_out, int* status_out, double* mma_cycles_out);
/* How an expert-parallel engine's one-token step moves rows between ranks: 2 = through peer memory (each rank stores its
 * quantised row and router logits into every rank's CUDA-IPC-mapped region and the served picks' output rows into their
 * owner's, with one flag per (layer, peer) and bounded waits; set up at creation when every rank could map every peer, and
 * ITB_EP_P2P is not 0), 1 = NCCL all-gather + reduce-scatter per layer, 0 = the engine is not expert parallel. */
int  itb_engine_ep_transport(itb_engine*);
/* Expert parallelism, many-row passes: the send/receive plan of the packed all-to-all that carries every (row, pick) pair to
 * the rank holding its expert and its output row back (the reference places experts by contiguous range, src/ops/mod.rs:1024-1048;
 * it has no multi-GPU path of its own). cnt[s * world + d] = pairs rank s sends to rank d (every rank has the whole matrix
 * after one small all-gather). Fills send_off[world + 1] (offsets into this rank's pairs sorted by owner rank) and
 * recv_off[world + 1] (offsets into its receive buffer, source-rank order) and *n_recv. Host arithmetic only; 0 ok. */
int  itb_ep_a2a_plan(const int* cnt, int world, int rank, int* send_off, int* recv_off, int* n_recv);
/* The FP4 activation quantiser of the tensor-core expert path on its own (opts "experts=fp4tc" selects that path for
 * itb_matmul_experts / itb_moe_glu and for the engine's many-row passes): x[n], n a multiple of 16 -> one UE4M3 scale code per
 * 16 elements and one E2M1 code (0..15) per element, the CPU statement's record (Fp4Row::from_f32, src/ops/naive.rs:755-788),
 * bit for bit. Host arrays. Returns 0, or 1 with the context's error set. */
int  itb_fp4_quantize(itb_ctx*, const float* x, size_t n, uint8_t* scales_out, uint8_t* codes_out);
/* exp and log as the kernels compute them, on their own (tests compare with the C library the reference CPU path calls:
 * Rust's f32::exp / f32::ln, src/ops/naive.rs:101-106, :246-252, :362-376). itb_expf_host: the same expf on the host, no
 * device needed. itb_eval_unary: kind 0 exp, 1 log, on the device over host arrays. */
float itb_expf_host(float x);
int  itb_eval_unary(itb_ctx*, int kind, const float* in, size_t n, float* out);
/* Device generator check: element i of stream `key` (tests compare with the CPU generator). */
int  itb_synth_values(itb_ctx*, uint64_t key, uint64_t first, size_t n, int dist, float std_, float* out);

#ifdef __cplusplus
}
#endif
#endif
