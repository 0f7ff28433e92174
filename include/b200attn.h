/*
 * b200attn — C ABI of the B200 (sm_100a) attention hot path for the Qwen3.5-0.8B hybrid stack:
 * the gated full-attention layer, the Gated DeltaNet linear-attention layer, their caches and the
 * graph-captured decode step.
 *
 * This is the drop-in boundary below the reference's C++ operator classes in src/backend/cuda
 * (qwen::cuda::CudaFullAttention, CudaKVCache, CudaLinearAttention[V2], CudaLinearAttnState and the
 * free launchers).  Every entry point names the reference interface it replaces (file:line relative
 * to the reference root).
 *
 * Conventions
 *   - plain C: opaque handles, POD structs, raw pointers, explicit cudaStream_t (passed as void*);
 *   - `d_` = device pointer, `h_` = host pointer;
 *   - activations cross the boundary as fp32 row-major [rows, hidden] exactly as the reference's
 *     layer code passes them (src/backend/cuda/kernels/cuda_engine.cu:116-120,134-139);
 *   - weights arrive as host fp32 row-major [out, in] (src/backend/cuda/WEIGHT_FORMAT.md:15-57);
 *   - every function returns 0 on success or a negative b200attn_status; nothing throws, prints,
 *     exits or traps.  b200attn_last_error() returns a thread-local message for the last failure;
 *   - there is no CPU fallback: without a usable CUDA device every compute entry returns
 *     B200ATTN_ERR_CUDA.
 */
#ifndef B200ATTN_H_
#define B200ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200ATTN_ABI_VERSION 1

typedef enum {
    B200ATTN_OK = 0,
    B200ATTN_ERR_INVALID = -1,     /* bad argument (null pointer, size/shape mismatch)          */
    B200ATTN_ERR_CUDA = -2,        /* CUDA runtime / cuBLAS failure                              */
    B200ATTN_ERR_NOMEM = -3,       /* device allocation failed, page pool or slot table exhausted */
    B200ATTN_ERR_NOT_READY = -4,   /* weights not set / graph not captured                       */
    B200ATTN_ERR_UNSUPPORTED = -5, /* shape outside the compiled kernels (head_dim != 256 ...)    */
    B200ATTN_ERR_DEVICE = -6       /* a kernel reported a device-side error word (bounded wait ran out) */
} b200attn_status;

/* Precision of the projection GEMMs around the attention cores. */
typedef enum {
    B200ATTN_PROJ_FP32 = 0, /* fp32 weights and activations (parity runs against the fp32 CPU reference) */
    B200ATTN_PROJ_FP16 = 1  /* fp16 weights and activations, fp32 accumulation (throughput runs)         */
} b200attn_proj_precision;

/* Storage type of the paged KV cache. */
typedef enum {
    B200ATTN_KV_INT8 = 0, /* INT8 codes + one fp32 scale per (token, kv head)                 */
    B200ATTN_KV_FP16 = 1  /* IEEE half                                                        */
} b200attn_kv_dtype;

typedef void* b200attn_stream;              /* cudaStream_t */
typedef struct b200attn_fa_s* b200attn_fa;             /* gated full-attention operator (weights + scratch) */
typedef struct b200attn_kv_pool_s* b200attn_kv_pool;   /* paged KV cache for all full-attention layers      */
typedef struct b200attn_la_s* b200attn_la;             /* Gated DeltaNet operator                           */
typedef struct b200attn_la_state_s* b200attn_la_state; /* recurrent + conv state for all DeltaNet layers    */
typedef struct b200attn_stack_s* b200attn_stack;       /* 24-layer hybrid stack with the captured decode step */

/* Text of the calling thread's last failure.  Replaces the reference's error channels: printf-and-continue
 * (src/backend/cuda/kernels/full_attention_cuda.cu:11-17) and std::runtime_error
 * (src/backend/cuda/include/cuda_error_handling.cuh:19-27). */
const char* b200attn_last_error(void);
/* B200ATTN_ABI_VERSION of the loaded library.  No reference counterpart. */
int b200attn_abi_version(void);

/* ------------------------------------------------------------------------------------------------
 * Paged KV cache.
 * Replaces qwen::cuda::CudaKVCache (src/backend/cuda/include/full_attention_cuda.hpp:11-33, impl
 * src/backend/cuda/kernels/full_attention_cuda.cu:252-356), CudaKVCacheINT8
 * (include/kv_int8_cuda.hpp:11-31) and the host bookkeeping of PagedKVCache
 * (include/paged_kv.hpp:18-58, kernels/paged_kv.cpp:17-201).
 *
 * Layout in HBM (page_tokens = 64):
 *   K codes  [layer][page][kv_head][page_tokens][head_dim]      int8 | half
 *   V codes  [layer][page][kv_head][head_dim][page_tokens]      int8 | half   (token-minor)
 *   scales   [layer][page][kv_head][page_tokens]  fp32, K and V separately    (INT8 only)
 *   block table [max_seqs][max_pages_per_seq] int32, lengths [layer][max_seqs] int32 (device-resident)
 * A sequence is addressed by the slot b200attn_kv_seq_alloc returns.  Lengths are kept per layer
 * like CudaKVCache::layer_lengths; every attention call on a layer appends to that layer.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int num_layers;        /* full-attention layers sharing the pool (6 in the hybrid stack)  */
    int num_kv_heads;      /* 2   */
    int head_dim;          /* 256 */
    int page_tokens;       /* must be 64 */
    int num_pages;         /* pages in the pool (each page spans all layers)                  */
    int max_seqs;          /* slots                                                           */
    int max_pages_per_seq; /* block-table width                                               */
    int kv_dtype;          /* b200attn_kv_dtype                                               */
} b200attn_kv_config;

/* CudaKVCache::reset (full_attention_cuda.cu:252-272) / PagedKVCache::initialize (paged_kv.cpp:17-47). */
int b200attn_kv_pool_create(const b200attn_kv_config* cfg, b200attn_kv_pool* out);
/* PagedKVCache::~PagedKVCache (paged_kv.cpp:13-15); CudaKVCache itself has no destructor
 * (full_attention_cuda.hpp:11-33) and leaks unless the caller frees its members. */
int b200attn_kv_pool_destroy(b200attn_kv_pool pool);
/* PagedKVCache::allocate_sequence (paged_kv.cpp:90-112): new slot with pages for reserve_tokens. */
int b200attn_kv_seq_alloc(b200attn_kv_pool pool, int reserve_tokens, int* slot_out);
/* PagedKVCache::append_tokens page growth (paged_kv.cpp:114-136) / CudaKVCache::ensure_capacity
 * (full_attention_cuda.cu:274-335): make sure the slot owns pages for total_tokens. */
int b200attn_kv_seq_reserve(b200attn_kv_pool pool, int slot, int total_tokens);
/* PagedKVCache::release_sequence (paged_kv.cpp:138-148). */
int b200attn_kv_seq_free(b200attn_kv_pool pool, int slot);
/* PagedKVCache::shrink_sequence (paged_kv.cpp:150-168): truncate a sequence to new_len tokens in every layer (layers
 * that hold fewer keep theirs) and return the pages wholly behind new_len to the pool, reserved-ahead pages included
 * (one page is always kept).  Synchronises with the device (lengths live there). */
int b200attn_kv_seq_shrink(b200attn_kv_pool pool, int slot, int new_len);
/* CudaKVCache::clear (full_attention_cuda.cu:337-356): all lengths to zero, pages kept. */
int b200attn_kv_clear(b200attn_kv_pool pool, b200attn_stream stream);
/* CudaKVCache::length (full_attention_cuda.hpp:26-28); host mirror of the device length. */
int b200attn_kv_seq_len(b200attn_kv_pool pool, int layer, int slot, int* len_out);
/* PagedKVCache::get_allocated_pages / get_used_pages (paged_kv.cpp:181-192). */
int b200attn_kv_pages(b200attn_kv_pool pool, int* total_out, int* used_out);
/* Reads (and clears) the pool's device-side status word: 0 = clean, 1 = slot out of range seen by a
 * kernel, 2 = append beyond the reserved pages (the write was skipped), 3/4 = a bounded wait inside
 * the decode / prefill attention kernel ran out, 8 = the prefill kernel found its shared-memory window
 * misaligned and did nothing.  Synchronises the device.  No reference counterpart:
 * the reference's kernels report nothing (full_attention_cuda.cu:11-17 prints and continues). */
int b200attn_kv_device_status(b200attn_kv_pool pool, int* code_out);
/* Quantise-on-append of already normalised/rotated K and raw V rows, the arithmetic of
 * fused_kv_cache_int8_kernel (full_attention_cuda.cu:128-147) and kv_append_int8
 * (kv_int8_cuda.cu:193-207): d_k, d_v fp32 [sum(h_counts), kv_heads*head_dim]; sequence i receives
 * h_counts[i] tokens at its current length on `layer`, and that length advances. */
int b200attn_kv_append(b200attn_kv_pool pool, int layer, const int* h_slots, const int* h_counts,
                       int n_seqs, const float* d_k, const float* d_v, b200attn_stream stream);
/* kv_get_int8 (kv_int8_cuda.cu:209-222) without dequantisation: gather one sequence's cache on one
 * layer into contiguous token-major arrays [len][kv_heads][head_dim] (int8 or half as stored) and,
 * for INT8, scales [len][kv_heads].  Scale pointers may be NULL for FP16 pools. */
int b200attn_kv_export(b200attn_kv_pool pool, int layer, int slot, void* d_k_codes, void* d_v_codes,
                       float* d_k_scale, float* d_v_scale, int max_tokens, b200attn_stream stream);

/* ------------------------------------------------------------------------------------------------
 * Gated full attention.
 * Replaces qwen::cuda::CudaFullAttention (include/full_attention_cuda.hpp:35-90).
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int hidden_size;    /* 1024 */
    int num_heads;      /* 8    */
    int num_kv_heads;   /* 2    */
    int head_dim;       /* 256 (q and kv) */
    int rotary_dim;     /* 64   */
    float rope_theta;   /* 1e7  */
    int proj_precision; /* b200attn_proj_precision */
    int max_batch;      /* decode rows the scratch is sized for */
    int max_prefill_rows; /* rows per prefill call the scratch is sized for */
} b200attn_fa_config;

typedef struct {
    const float* q_proj; /* [num_heads*head_dim*2, hidden]; per head: head_dim q rows then head_dim gate rows */
    const float* k_proj; /* [num_kv_heads*head_dim, hidden] */
    const float* v_proj; /* [num_kv_heads*head_dim, hidden] */
    const float* q_norm; /* [head_dim], enters as (1 + w) */
    const float* k_norm; /* [head_dim] */
    const float* o_proj; /* [hidden, num_heads*head_dim] */
} b200attn_fa_weights;

/* CudaFullAttention::CudaFullAttention (full_attention_cuda.cu:174-201). */
int b200attn_fa_create(const b200attn_fa_config* cfg, b200attn_fa* out);
/* CudaFullAttention::~CudaFullAttention (full_attention_cuda.cu:203-228). */
int b200attn_fa_destroy(b200attn_fa fa);
/* CudaFullAttention::set_weights (full_attention_cuda.cu:230-250); host pointers. */
int b200attn_fa_set_weights(b200attn_fa fa, const b200attn_fa_weights* h_w);
/* CudaFullAttention::forward_batch_prefill (full_attention_cuda.cu:644-715), causal and per
 * sequence: d_x / d_y fp32 [sum(h_counts), hidden]; sequence i contributes h_counts[i] rows, which
 * are appended to slot h_slots[i] at its current length on `layer`; each row attends to every
 * cached token of its sequence up to and including itself.  RoPE position = cache index. */
int b200attn_fa_prefill(b200attn_fa fa, b200attn_kv_pool pool, int layer, const int* h_slots,
                        const int* h_counts, int n_seqs, const float* d_x, float* d_y,
                        b200attn_stream stream);
/* CudaFullAttention::forward (full_attention_cuda.cu:369-449) for n_seqs independent sequences:
 * one new token per sequence, d_x / d_y fp32 [n_seqs, hidden], d_slots device int32 [n_seqs]; a slot of -1 marks an
 * inactive row (nothing is read or written for it, here and in b200attn_la_decode).
 * No host synchronisation and no allocation: safe inside stream capture. */
int b200attn_fa_decode(b200attn_fa fa, b200attn_kv_pool pool, int layer, const int* d_slots,
                       int n_seqs, const float* d_x, float* d_y, b200attn_stream stream);
/* Attention cores alone, for kernel-level checks and timing.
 * flash_attention_decode / flash_attention_decode_int8 (include/flash_attention.cuh:25-27,
 * include/flash_attention_int8.cuh:41-69): d_q fp32 [n_seqs, heads, head_dim] (already normalised
 * and rotated), reads each slot's cache on `layer` (length as stored), writes d_out fp32
 * [n_seqs, heads, head_dim] = softmax(q K^T / sqrt(head_dim)) V, no gate. */
int b200attn_fa_decode_core(b200attn_fa fa, b200attn_kv_pool pool, int layer, const int* d_slots,
                            int n_seqs, const float* d_q, float* d_out, b200attn_stream stream);
/* The same decode attention core for callers that cannot allocate device memory: hosts that must stay off
 * cudaMalloc / cudaFree once warm (both synchronise the device) or that run under a fixed device-memory
 * budget.  It takes no operator handle; its scratch (fp16 q, split partials) is a fixed array built into
 * the library (about 4.3 MB per GPU, held until exit), so it creates and frees nothing.  Limits: at most 32
 * sequences per call and pools with at most 512 pages per sequence (B200ATTN_ERR_INVALID beyond).  All calls
 * share that array: calls that overlap on the GPU race, serialise them.  The first call on each device looks
 * up the array's address; make it outside stream capture.  This entry point has no counterpart in the
 * reference. */
int b200attn_fa_decode_core_static(b200attn_kv_pool pool, int layer, const int* d_slots, int n_seqs,
                                   const float* d_q, float* d_out, b200attn_stream stream);
/* launch_flash_attn_v2_prefill* (include/fused_kernels.cuh:37-82) with a causal mask: d_q fp32
 * [rows, heads, head_dim], d_k / d_v fp32 [rows, kv_heads, head_dim]; rows are h_counts[i]
 * consecutive tokens of n_seqs sequences, each starting at position 0; d_out fp32
 * [rows, heads, head_dim].  use_tensor_cores = 0 runs the plain SIMT cross-check kernel. */
int b200attn_fa_prefill_core(b200attn_fa fa, const int* h_counts, int n_seqs, const float* d_q,
                             const float* d_k, const float* d_v, float* d_out, int use_tensor_cores,
                             b200attn_stream stream);

/* ------------------------------------------------------------------------------------------------
 * Gated DeltaNet linear attention.
 * Replaces qwen::cuda::CudaLinearAttention (include/linear_attention_cuda.hpp:24-90),
 * CudaLinearAttentionV2 (include/linear_attention_v2.cuh:10-70) and CudaLinearAttnState
 * (include/linear_attention_cuda.hpp:11-22).
 *
 * State layout in HBM:
 *   recurrent [layer][slot][heads][key_dim][value_dim] fp32
 *   conv      [layer][slot][conv_kernel-1][conv_dim]   fp32, row 0 = oldest input
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int hidden_size;    /* 1024 */
    int num_heads;      /* 16   */
    int key_dim;        /* 128  */
    int value_dim;      /* 128  */
    int conv_kernel;    /* 4    */
    int proj_precision; /* b200attn_proj_precision */
    int max_batch;
    int max_prefill_rows;
} b200attn_la_config;

typedef struct {
    const float* in_proj_qkv; /* [heads*(2*key_dim+value_dim), hidden] rows: all q, all k, all v */
    const float* in_proj_a;   /* [heads, hidden] */
    const float* in_proj_b;   /* [heads, hidden] */
    const float* in_proj_z;   /* [heads*value_dim, hidden] */
    const float* conv1d;      /* [conv_dim, conv_kernel]; tap conv_kernel-1 multiplies the current token */
    const float* a_log;       /* [heads] */
    const float* dt_bias;     /* [heads] */
    const float* norm;        /* [value_dim], plain weight (no 1 +) */
    const float* out_proj;    /* [hidden, heads*value_dim] */
} b200attn_la_weights;

typedef struct {
    int num_layers; /* DeltaNet layers sharing the state pool (18 in the hybrid stack) */
    int max_seqs;
    int num_heads, key_dim, value_dim, conv_kernel;
} b200attn_la_state_config;

/* CudaLinearAttention::CudaLinearAttention (linear_attention_cuda.cu:292-326). */
int b200attn_la_create(const b200attn_la_config* cfg, b200attn_la* out);
/* CudaLinearAttention::~CudaLinearAttention (linear_attention_cuda.cu:328-379). */
int b200attn_la_destroy(b200attn_la la);
/* CudaLinearAttention::set_weights (linear_attention_cuda.cu:412-466); host pointers. */
int b200attn_la_set_weights(b200attn_la la, const b200attn_la_weights* h_w);
/* Reads (and clears) the operator's device-side status word: 0 = clean, 6 = a bounded wait inside the
 * chunked prefill kernel ran out (the affected sequences' outputs and states are then undefined).
 * Synchronises the device.  No reference counterpart. */
int b200attn_la_device_status(b200attn_la la, int* code_out);
/* CudaLinearAttnState::reset (linear_attention_cuda.cu:266-282): allocate and zero. */
int b200attn_la_state_create(const b200attn_la_state_config* cfg, b200attn_la_state* out);
/* CudaLinearAttnState has no destructor (linear_attention_cuda.hpp:11-22); the reference's tests free
 * d_recurrent_state / d_conv_state by hand (tests/integration/v2_kernel_accuracy_validate.cu:181-190). */
int b200attn_la_state_destroy(b200attn_la_state st);
/* CudaLinearAttnState::clear (linear_attention_cuda.cu:284-290) for one slot (slot < 0: all). */
int b200attn_la_state_clear(b200attn_la_state st, int slot, b200attn_stream stream);
/* Copy one (layer, slot) state in or out in the reference's own layouts: d_recurrent fp32
 * [heads][key_dim*value_dim], d_conv fp32 [conv_dim][conv_kernel-1] with index 0 = newest
 * (src/backend/cpu/core/attention/language_linear_attn.hpp:7-35).  Either pointer may be NULL. */
int b200attn_la_state_import(b200attn_la_state st, int layer, int slot, const float* d_recurrent,
                             const float* d_conv, b200attn_stream stream);
/* The reverse copy, same layouts (language_linear_attn.hpp:7-35). */
int b200attn_la_state_export(b200attn_la_state st, int layer, int slot, float* d_recurrent,
                             float* d_conv, b200attn_stream stream);
/* CudaLinearAttention::forward_batch / CudaLinearAttentionV2::forward_batch
 * (linear_attention_cuda.cu:529-684, linear_attention_v2.cu:790-883) as a true causal sequence
 * pass: d_x / d_y fp32 [sum(h_counts), hidden], sequence i continues from the state in slot
 * h_slots[i] and leaves its final state there. */
int b200attn_la_prefill(b200attn_la la, b200attn_la_state st, int layer, const int* h_slots,
                        const int* h_counts, int n_seqs, const float* d_x, float* d_y,
                        b200attn_stream stream);
/* CudaLinearAttention::forward (linear_attention_cuda.cu:468-527) for n_seqs independent
 * sequences: one token each, d_slots device int32.  Safe inside stream capture. */
int b200attn_la_decode(b200attn_la la, b200attn_la_state st, int layer, const int* d_slots,
                       int n_seqs, const float* d_x, float* d_y, b200attn_stream stream);
/* The fused recurrent step alone (gated_delta_kernel + conv1d_update + l2norm + norm_gate of
 * linear_attention_cuda.cu:47-172 in one launch): d_mixed fp32 [n_seqs, 8224] is the fused input
 * projection of the step (columns: 6144 q|k|v pre-conv, 2048 z, 16 a, 16 b); d_out fp32 [n_seqs, 2048]
 * receives the gated, normalised head outputs (the input of out_proj).  Updates state and conv cache. */
int b200attn_la_decode_core(b200attn_la la, b200attn_la_state st, int layer, const int* d_slots,
                            int n_seqs, const float* d_mixed, float* d_out, b200attn_stream stream);
/* Recurrence core alone (gated_delta_batch_fused_v2_kernel, linear_attention_v2.cu:492-595):
 * d_q, d_k fp32 [rows, heads, key_dim] (already L2-normalised, q scaled), d_v fp32
 * [rows, heads, value_dim], d_g (log decay) and d_beta fp32 [rows, heads]; d_out fp32
 * [rows, heads, value_dim] = S_t^T q_t; states continue from / are left in the given slots.
 * use_tensor_cores = 0 runs the token-serial fp32 cross-check kernel. */
int b200attn_la_prefill_core(b200attn_la la, b200attn_la_state st, int layer, const int* h_slots,
                             const int* h_counts, int n_seqs, const float* d_q, const float* d_k,
                             const float* d_v, const float* d_g, const float* d_beta, float* d_out,
                             int use_tensor_cores, b200attn_stream stream);

/* ------------------------------------------------------------------------------------------------
 * Hybrid stack and the graph-captured decode step.
 * Replaces the attention-facing part of qwen::cuda::CudaEngine
 * (src/backend/cuda/include/cuda_engine.hpp:85-164): set_layer_weights, forward_batch_prefill
 * (cuda_engine.cu:354-389), forward_batch_decode (:327-352), reset_cache (:514-519) and the graph
 * capture of forward_batch_prefill_graph (:391-479), here applied to the decode step.
 * Layer i is full attention when i % 4 == 3, DeltaNet otherwise.  RMSNorm, the SwiGLU FFN, the
 * embedding gather and the tied LM head + greedy argmax are library GEMMs and small kernels.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int num_layers;        /* 24 */
    int hidden_size;       /* 1024 */
    int intermediate_size; /* 3584 */
    int vocab_size;        /* 248320 */
    int max_seqs;          /* sequences resident on this GPU */
    int max_seq_len;       /* prompt + generated tokens per sequence */
    int prefill_chunk_seqs; /* sequences per prefill pass (bounds activation scratch) */
    int kv_dtype;          /* b200attn_kv_dtype */
    int int8_weights;      /* 1: every matrix is quantised per output channel to INT8 codes (scale = absmax/127,
                              roundf; src/backend/cuda/kernels/mlp_cuda.cu:22-39) and the GEMMs use code*scale,
                              stored as fp16: the values are the INT8 ones, the bytes streamed are fp16 */
    float rms_eps;         /* 1e-6 */
} b200attn_stack_config;

typedef struct {
    const float* input_norm; /* [hidden], (1 + w) convention (src/backend/cuda/kernels/rmsnorm_cuda.cu:90-98) */
    const float* post_norm;  /* [hidden] */
    const float* ffn_gate;   /* [inter, hidden] */
    const float* ffn_up;     /* [inter, hidden] */
    const float* ffn_down;   /* [hidden, inter] */
    const b200attn_fa_weights* fa; /* non-NULL for full-attention layers */
    const b200attn_la_weights* la; /* non-NULL for DeltaNet layers */
} b200attn_layer_weights;

/* CudaEngine::CudaEngine (cuda_engine.cu:158-181, buffers :196-225): layers, caches and activation buffers. */
int b200attn_stack_create(const b200attn_stack_config* cfg, b200attn_stack* out);
/* CudaEngine::~CudaEngine (cuda_engine.cu:183-194). */
int b200attn_stack_destroy(b200attn_stack st);
/* CudaEngine::set_layer_weights (cuda_engine.cu:244-298). */
int b200attn_stack_set_layer_weights(b200attn_stack st, int layer, const b200attn_layer_weights* h_w);
/* Token embedding (tied with the LM head) [vocab, hidden] and final norm [hidden]; host pointers.
 * CudaTokenEmbedding::set_weight / CudaLMHead::set_weight as the benchmark driver calls them
 * (src/backend/cuda/performance_test.cu:196-202; CudaEngine::set_final_norm_weight / set_lm_head_weight, cuda_engine.cu:300-306). */
int b200attn_stack_set_embedding(b200attn_stack st, const float* h_embed, const float* h_final_norm);
/* Same, but the embedding is generated on the device as N(0, std) from `seed` (the 1 GB host copy
 * is not needed for throughput runs with random-init weights).  No reference counterpart. */
int b200attn_stack_init_embedding_random(b200attn_stack st, uint64_t seed, float std_dev,
                                         const float* h_final_norm);
/* Reads (and clears) the device-side status words of the stack (its KV pool, its DeltaNet operators and its own
 * GEMM kernels): 0 = clean, otherwise the first non-zero code found (codes as in b200attn_kv_device_status /
 * b200attn_la_device_status; 7 = a bounded wait inside a decode-step GEMM ran out).  Synchronises the device.
 * No reference counterpart. */
int b200attn_stack_device_status(b200attn_stack st, int* code_out);
/* CudaEngine::reset_cache (cuda_engine.cu:514-519). */
int b200attn_stack_reset(b200attn_stack st, b200attn_stream stream);
/* CudaEngine::forward_batch_prefill (cuda_engine.cu:354-389) for n_seqs sequences of prompt_len
 * tokens each (slots 0..n_seqs-1): d_tokens int32 [n_seqs, prompt_len]; writes the greedy next
 * token of every sequence to d_next int32 [n_seqs].  d_hidden_out (optional) receives the final
 * normalised hidden state of each sequence's last token, fp32 [n_seqs, hidden].  Asynchronous on `stream` (no
 * allocation, no host synchronisation); device-side failures show in b200attn_stack_device_status. */
int b200attn_stack_prefill(b200attn_stack st, int n_seqs, int prompt_len, const int* d_tokens,
                           int* d_next, float* d_hidden_out, b200attn_stream stream);
/* One decode step for n_seqs sequences, eager: CudaEngine::forward_batch_decode
 * (cuda_engine.cu:327-352).  d_tokens_in/out int32 [n_seqs]. */
int b200attn_stack_decode(b200attn_stack st, int n_seqs, const int* d_tokens_in, int* d_tokens_out,
                          b200attn_stream stream);
/* Capture that step once into a CUDA graph (cudaStreamBeginCapture / cudaGraphInstantiate as in
 * cuda_engine.cu:429-470); lengths, block tables and the token buffer are device-resident so one
 * graph replays for every step.  The step reads and writes an internal token buffer: seed it with
 * b200attn_stack_set_tokens, read it with b200attn_stack_get_tokens. */
int b200attn_decode_graph_capture(b200attn_stack st, int n_seqs, b200attn_stream stream);
/* cudaGraphLaunch (cuda_engine.cu:472-476): run `steps` captured steps back to back. */
int b200attn_decode_graph_launch(b200attn_stack st, int steps, b200attn_stream stream);
/* Seed / read the token buffer of the captured step (d_tokens int32 [n_seqs]).  The reference copies
 * token ids host -> device every step instead (performance_test.cu:297-312). */
int b200attn_stack_set_tokens(b200attn_stack st, const int* d_tokens, int n_seqs, b200attn_stream stream);
/* See b200attn_stack_set_tokens (performance_test.cu:313-319 reads the sampled ids back each step). */
int b200attn_stack_get_tokens(b200attn_stack st, int* d_tokens, int n_seqs, b200attn_stream stream);
/* ------------------------------------------------------------------------------------------------
 * Continuous batching on the stack's pools: admission into free rows and retirement between decode steps.  The
 * reference has only the page bookkeeping for it (PagedKVCache::allocate_sequence / append_tokens / release_sequence /
 * shrink_sequence, src/backend/cuda/kernels/paged_kv.cpp:90-168) and no caller.
 * Row r of a decode step is bound to a slot (KV pages + DeltaNet state); the device-resident row -> slot list keeps the
 * active rows dense at the front and marks the others -1, which every decode kernel skips, so ONE captured step over
 * max_seqs rows serves any number of active sequences.  All calls are host-synchronous bookkeeping except the prompt
 * pass of an admission; make them between steps.
 * ---------------------------------------------------------------------------------------------- */
/* Enter the mode: caches cleared, every row inactive, every slot's pages back in the pool (PagedKVCache::clear,
 * paged_kv.cpp:49-64).  b200attn_stack_reset leaves it. */
int b200attn_stack_begin_batching(b200attn_stack st, b200attn_stream stream);
/* Admit one sequence (PagedKVCache::allocate_sequence, paged_kv.cpp:90-112, plus the prompt pass the reference leaves
 * to its caller): takes a free slot, reserves pages for reserve_tokens (prompt + tokens to generate;
 * B200ATTN_ERR_NOMEM without side effects when rows or pages run out), clears its state, runs the prompt
 * (d_prompt int32 [prompt_len]) and leaves the first generated token in the row's entry of the token buffer. */
int b200attn_stack_admit(b200attn_stack st, const int* d_prompt, int prompt_len, int reserve_tokens, int* row_out,
                         b200attn_stream stream);
/* Retire the sequence in `row` (PagedKVCache::release_sequence, paged_kv.cpp:138-148): its pages go back to the pool
 * and the last active row moves into its place. */
int b200attn_stack_retire(b200attn_stack st, int row, b200attn_stream stream);
/* Active rows and (optionally, h_row_slots int[max_seqs]) the slot of every row.  No reference counterpart. */
int b200attn_stack_rows(b200attn_stack st, int* n_active_out, int* h_row_slots);
/* One decode step over rows [0, n_rows) of the internal token buffer (CudaEngine::forward_batch_decode,
 * cuda_engine.cu:327-352): the captured graph when it was captured for n_rows, eager launches otherwise. */
int b200attn_stack_step(b200attn_stack st, int n_rows, b200attn_stream stream);

/* Number of kernels this library launched on behalf of the calling thread since the last call
 * with reset != 0 (graph replays count the nodes of the captured step).  No reference counterpart. */
long long b200attn_launch_count(int reset);

/* ------------------------------------------------------------------------------------------------
 * Per-kernel device timing (the reference's LatencyStats over cudaEvent pairs,
 * src/backend/cuda/performance_test.cu:60-97, applied per kernel class).  While enabled, the prefill kernels and the
 * append are bracketed by an event pair on their own stream, and every launch of the two decode kernels gets a
 * device-side stamp slot (first CTA past its dependency wait .. last CTA done, on the GPU's global timer).  Stamps
 * also work for launches captured by b200attn_decode_graph_capture while profiling is on: every replay fills its
 * slots again, b200attn_profile_read sums and re-arms them.  Names: "fa_prefill", "fa_decode", "la_prefill",
 * "la_decode", "kv_append", and for the projections of the fused decode step "gemm_in" (input projections),
 * "gemm_ffn" (gate / up + SwiGLU), "gemm_res" (output projections with the residual add), "lm_head".  b200attn_profile_read synchronises the device and returns the summed device time and
 * launch count; b200attn_profile_reset forgets all pairs and slots (re-capture a graph that carried stamps).
 * ---------------------------------------------------------------------------------------------- */
int b200attn_profile_enable(int on);
int b200attn_profile_reset(void);
int b200attn_profile_read(const char* name, double* total_ms_out, long long* launches_out);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H_ */
