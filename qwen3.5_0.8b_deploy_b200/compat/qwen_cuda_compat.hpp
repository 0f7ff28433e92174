// Source-compatible stand-ins for the reference's attention operator classes, implemented on the b200attn C ABI.
//
// The class and member names, constructor defaults and method signatures are those of
//   src/backend/cuda/include/full_attention_cuda.hpp:11-58   (CudaKVCache, CudaFullAttention)
//   src/backend/cuda/include/linear_attention_cuda.hpp:11-51 (CudaLinearAttnState, CudaLinearAttention)
//   src/backend/cuda/include/linear_attention_v2.cuh:10-33   (CudaLinearAttentionV2)
//   src/backend/cuda/include/flash_attention.cuh:25-27, flash_attention_int8.cuh:41-69, fused_kernels.cuh:37-82,
//   kv_int8_cuda.hpp:11-43, paged_kv.hpp:18-58, cuda_engine.hpp:166-169   (free launchers and cache types, below)
// so the reference's layer code (src/backend/cuda/kernels/cuda_engine.cu:109-156) and its stand-alone checks
// (src/backend/cuda/verify_linear_attn_batch.cu, tests/integration/v2_kernel_accuracy_validate.cu) compile against
// this header instead.  Differences a maintainer has to know are listed next to each member.
#pragma once

#include <cuda_runtime.h>

#include <cuda_fp16.h>

#include <cstdint>
#include <stdexcept>
#include <unordered_map>
#include <vector>

#include "../../include/b200attn.h"

namespace qwen {
namespace cuda {

namespace detail {
// Plain fp32 DeltaNet path for sizes the library's kernels are not built for (qwen_cuda_compat_free.cu).
struct GenericLa;
GenericLa* generic_la_create(int hidden, int heads, int kd, int vd, int ck);
void generic_la_destroy(GenericLa* g);
void generic_la_set_weights(GenericLa* g, const std::vector<float>& qkv, const std::vector<float>& a, const std::vector<float>& b,
                            const std::vector<float>& z, const std::vector<float>& conv, const std::vector<float>& out,
                            const std::vector<float>& a_log, const std::vector<float>& dt_bias, const std::vector<float>& norm);
void generic_la_forward(GenericLa* g, const float* in, float* out, float* d_recurrent, float* d_conv, int rows, cudaStream_t s);
}  // namespace detail

// One sequence, `num_layers` layers, stored in the paged pool of the library.
struct CudaKVCache {
    // Kept for source compatibility. They point at the library's page arrays (K [page][head][64][256],
    // V [page][head][256][64], scales [page][head][64]), not at the reference's contiguous [layer][seq][head][dim].
    int8_t* d_k_cache = nullptr;
    int8_t* d_v_cache = nullptr;
    float* d_k_scale = nullptr;
    float* d_v_scale = nullptr;
    std::vector<int> layer_lengths;
    int num_layers = 0;
    int num_kv_heads = 0;
    int head_dim = 0;
    int max_seq_len = 0;
    int capacity_seq_len = 0;

    // init_capacity is rounded up to 8192 tokens (the reference's decode kernel attends to at most 8192 keys,
    // full_attention_cuda.cu:181,380-382); pages are reserved on demand inside that bound.
    void reset(int nl, int nkh, int hd, int init_capacity = 1024);
    void clear();
    int length(int layer_idx) const { return layer_lengths[layer_idx]; }
    void ensure_capacity(int required_seq_len);   // throws std::runtime_error beyond max_seq_len

    b200attn_kv_pool pool = nullptr;   // library handle (not in the reference)
    int slot = -1;
    int* d_slot = nullptr;             // device copy of `slot` for the decode entry point
};

class CudaFullAttention {
  public:
    CudaFullAttention(int hidden_size = 1024, int num_heads = 8, int num_kv_heads = 2, int q_head_dim = 256,
                      int kv_head_dim = 256);
    ~CudaFullAttention();
    void set_weights(const std::vector<float>& q_proj_weight, const std::vector<float>& k_proj_weight,
                     const std::vector<float>& v_proj_weight, const std::vector<float>& q_norm_weight,
                     const std::vector<float>& k_norm_weight, const std::vector<float>& o_proj_weight);
    // One token.  `position` must equal the layer's cache length (the reference's callers always pass that).
    void forward(const float* input, float* output, CudaKVCache& kv_cache, int layer_idx, int position) const;
    // batch_size consecutive tokens of the cache's sequence, causal.  `positions` (device) is not read: row i sits
    // at cache length + i.  (The reference kernel applies no causal mask, fused_kernels.cu:126-264; this follows
    // the CPU class, language_full_attn.cpp:227-252.)
    void forward_batch_prefill(const float* input, float* output, CudaKVCache& kv_cache, int layer_idx,
                               const int* positions, int batch_size, int max_seq = 0) const;
    int hidden_size() const { return hidden_size_; }
    int num_heads() const { return num_heads_; }

  private:
    int hidden_size_, num_heads_, num_kv_heads_, q_head_dim_, kv_head_dim_;
    b200attn_fa op_ = nullptr;
};

struct CudaLinearAttnState {
    // Reference-layout mirrors of the library's state ([heads][key_dim*value_dim] and [conv_dim][conv_kernel-1] with
    // index 0 = newest).  They are imported before and exported after every forward call, so code that reads or
    // writes them between calls (as tests/integration/v2_kernel_accuracy_validate.cu does) keeps working, and the
    // caller may cudaFree them by hand as the reference's tests do.
    float* d_recurrent_state = nullptr;
    float* d_conv_state = nullptr;
    int num_heads = 0;
    int key_dim = 0;
    int value_dim = 0;
    int conv_dim = 0;
    int conv_kernel = 0;
    void reset(int nh, int kd, int vd, int conv_k = 4);
    void clear();

    b200attn_la_state state = nullptr;    // library handle (not in the reference)
    int* d_slot = nullptr;
};

class CudaLinearAttention {
  public:
    CudaLinearAttention(int hidden_size = 1024, int num_heads = 16, int key_dim = 128, int value_dim = 128,
                        int conv_kernel = 4);
    ~CudaLinearAttention();
    // Note the order: out_proj comes before a_log (linear_attention_cuda.hpp:31-39).  Empty a_log / dt_bias mean
    // zeros, empty norm_weight means ones (linear_attention_cuda.cu:449-465).
    void set_weights(const std::vector<float>& in_proj_qkv_weight, const std::vector<float>& in_proj_a_weight,
                     const std::vector<float>& in_proj_b_weight, const std::vector<float>& in_proj_z_weight,
                     const std::vector<float>& conv1d_weight, const std::vector<float>& out_proj_weight,
                     const std::vector<float>& a_log = {}, const std::vector<float>& dt_bias = {},
                     const std::vector<float>& norm_weight = {});
    void forward(const float* input, float* output, CudaLinearAttnState& state) const;
    // batch_size consecutive tokens of the state's sequence (a true causal pass: every token sees the conv
    // history of the tokens before it, unlike linear_attention_cuda.cu:552-559).
    void forward_batch(const float* input, float* output, CudaLinearAttnState& state, int batch_size) const;
    void forward_fused(const float* input, float* output, CudaLinearAttnState& state) const;
    int hidden_size() const { return hidden_size_; }
    int num_heads() const { return num_heads_; }

  protected:
    int hidden_size_, num_heads_, key_dim_, value_dim_, conv_kernel_;
    b200attn_la op_ = nullptr;
    detail::GenericLa* generic_ = nullptr;      // used instead of op_ at sizes other than the model's
    int proj_precision_ = B200ATTN_PROJ_FP16;   // 16-bit weights (the reference rounds these weights to bf16 at load)
};

// Same operator with fp32 weights and an explicit stream on forward_batch (linear_attention_v2.cuh:10-33).
class CudaLinearAttentionV2 {
  public:
    CudaLinearAttentionV2(int hidden_size = 1024, int num_heads = 16, int key_dim = 128, int value_dim = 128,
                          int conv_kernel = 4);
    ~CudaLinearAttentionV2();
    void set_weights(const std::vector<float>& in_proj_qkv_weight, const std::vector<float>& in_proj_a_weight,
                     const std::vector<float>& in_proj_b_weight, const std::vector<float>& in_proj_z_weight,
                     const std::vector<float>& conv1d_weight, const std::vector<float>& out_proj_weight,
                     const std::vector<float>& a_log = {}, const std::vector<float>& dt_bias = {},
                     const std::vector<float>& norm_weight = {});
    void forward(const float* input, float* output, CudaLinearAttnState& state) const;
    void forward_batch(const float* input, float* output, CudaLinearAttnState& state, int batch_size,
                       cudaStream_t stream = 0) const;
    int hidden_size() const { return hidden_size_; }
    int num_heads() const { return num_heads_; }

  private:
    int hidden_size_, num_heads_, key_dim_, value_dim_, conv_kernel_;
    b200attn_la op_ = nullptr;
    detail::GenericLa* generic_ = nullptr;      // used instead of op_ at sizes other than the model's
};

// ---- free launchers (qwen_cuda_compat_free.cu) ---------------------------------------------------------------------------
// They stage the caller's contiguous caches into a private paged pool and run the library's attention cores; shapes
// other than 8 query heads / 2 kv heads / head_dim 256 throw std::invalid_argument.  Where the reference's CUDA kernels
// deviate from its CPU classes the CPU semantics are followed: prefill rows are causal (row i of a batch is the token
// at position seq_len - batch_size + i) and INT8 scales are read per (token, kv head), [layer][max_seq][kv_heads].

// flash_attention.cuh:25-27.  d_Q [8][256], caches [seq_len][2][256] fp32, d_output [8][256]; scale 0 = 1/sqrt(head_dim).
void flash_attention_decode(const float* d_Q, const float* d_K_cache, const float* d_V_cache, float* d_output, int num_heads,
                            int num_kv_heads, int q_head_dim, int kv_head_dim, int seq_len, float scale = 0.0f);
// flash_attention_int8.cuh:41-69.  Caches [layer][max_seq_len][2][256] codes, scales [layer][max_seq_len][2].
void flash_attention_decode_int8(const float* d_Q, const int8_t* d_K_cache, const int8_t* d_V_cache, const float* d_K_scale,
                                 const float* d_V_scale, float* d_output, int num_heads, int num_kv_heads, int q_head_dim,
                                 int kv_head_dim, int seq_len, int layer_idx, int max_seq_len, float scale = 0.0f);
void flash_attention_decode_int8_batched(const float* d_Q, const int8_t* d_K_cache, const int8_t* d_V_cache,
                                         const float* d_K_scale, const float* d_V_scale, float* d_output, int num_heads,
                                         int num_kv_heads, int q_head_dim, int kv_head_dim, int seq_len, int layer_idx,
                                         int max_seq_len, float scale = 0.0f);
// fused_kernels.cuh:37-82.  Q / output [batch_size][8][256]; caches indexed layer * max_seq_len * 512 + t * 512 + kvh * 256 + d.
void launch_flash_attn_v2_prefill(const float* Q, const float* K_cache, const float* V_cache, float* output, int num_heads,
                                  int num_kv_heads, int head_dim, int seq_len, int batch_size, int layer_idx, int max_seq_len,
                                  float scale, cudaStream_t stream = 0);
void launch_flash_attn_v2_prefill_fp16_cache(const float* Q, const half* K_cache, const half* V_cache, float* output,
                                             int num_heads, int num_kv_heads, int head_dim, int seq_len, int batch_size,
                                             int layer_idx, int max_seq_len, float scale, cudaStream_t stream = 0);
void launch_flash_attn_v2_prefill_int8_cache(const float* Q, const int8_t* K_cache, const int8_t* V_cache, const float* K_scale,
                                             const float* V_scale, float* output, int num_heads, int num_kv_heads, int head_dim,
                                             int seq_len, int batch_size, int layer_idx, int max_seq_len, float scale,
                                             cudaStream_t stream = 0);

// kv_int8_cuda.hpp:11-43.  Codes [layer][max_seq_len][kv_heads * head_dim]; scales [layer][max_seq_len][kv_heads] (one
// per token and kv head; the reference's append kernel lets two blocks race for one slot per token).
struct CudaKVCacheINT8 {
    int8_t* d_k_cache = nullptr;
    int8_t* d_v_cache = nullptr;
    float* d_k_scale = nullptr;
    float* d_v_scale = nullptr;
    std::vector<int> layer_lengths;
    int num_layers = 0;
    int num_kv_heads = 0;
    int head_dim = 0;
    int max_seq_len = 0;
    size_t bytes_allocated = 0;
    void reset(int nl, int nkh, int hd, int max_len);
    void clear();
    int length(int layer_idx) const { return layer_lengths[layer_idx]; }
    size_t memory_bytes() const { return bytes_allocated; }
};
// One scale per 256 consecutive values: scale = absmax / 127 (1 below 1e-8), code = roundf(x / scale).
void kv_quantize_fp32_to_int8(const float* d_input, int8_t* d_output, float* d_scale, int num_elements, cudaStream_t stream = 0);
void kv_dequantize_int8_to_fp32(const int8_t* d_input, const float* d_scale, float* d_output, int num_elements,
                                cudaStream_t stream = 0);
void kv_append_int8(CudaKVCacheINT8& cache, const float* d_k, const float* d_v, int layer_idx, cudaStream_t stream = 0);
void kv_get_int8(const CudaKVCacheINT8& cache, float* d_k_out, float* d_v_out, int layer_idx, cudaStream_t stream = 0);

// paged_kv.hpp:18-58: the reference's page bookkeeping interface on the library's page pool (pages of 64 tokens).
class PagedKVCache {
  public:
    PagedKVCache();
    ~PagedKVCache();
    void initialize(int num_layers, int num_kv_heads, int head_dim, int page_size, int max_pages);
    void clear();
    int allocate_sequence(int initial_len = 0);   // -1 when the pool cannot serve it (paged_kv.cpp:90-112)
    void append_tokens(int seq_id, int num_tokens);
    void release_sequence(int seq_id);
    void shrink_sequence(int seq_id, int new_len);
    size_t get_kv_bytes() const;
    size_t get_gpu_bytes() const;
    int get_allocated_pages() const;
    int get_used_pages() const;
    void print_status() const;
    b200attn_kv_pool pool() const { return pool_; }                 // library handle (not in the reference)
    int slot_of(int seq_id) const { auto it = seq_to_slot_.find(seq_id); return it == seq_to_slot_.end() ? -1 : it->second; }

  private:
    b200attn_kv_pool pool_ = nullptr;
    std::unordered_map<int, int> seq_to_slot_;
    std::unordered_map<int, int> seq_lengths_;
    int num_layers_ = 0, num_kv_heads_ = 0, head_dim_ = 0, page_size_ = 0, max_pages_ = 0, next_seq_id_ = 1;
    size_t gpu_bytes_ = 0;
};

// cuda_engine.hpp:166-169.
void set_fa_weights(CudaFullAttention* fa, const std::vector<float>& q_w, const std::vector<float>& k_w,
                    const std::vector<float>& v_w, const std::vector<float>& qn_w, const std::vector<float>& kn_w,
                    const std::vector<float>& o_w, int layer_idx);

}  // namespace cuda
}  // namespace qwen
