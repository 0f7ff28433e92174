// Implementation of the source-compatible operator classes on the b200attn C ABI.  Status codes map to the
// exception types the reference throws: std::invalid_argument for bad sizes
// (src/backend/cpu/core/attention/language_full_attn.cpp:30-79), std::runtime_error otherwise
// (src/backend/cuda/include/cuda_error_handling.cuh:19-27).
#include "qwen_cuda_compat.hpp"

#include <algorithm>
#include <string>

namespace qwen {
namespace cuda {
namespace {

void check(int status) {
    if (status == 0) return;
    const std::string msg = b200attn_last_error();
    if (status == B200ATTN_ERR_INVALID) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}
void check_cuda(cudaError_t e) {
    if (e != cudaSuccess) throw std::runtime_error(cudaGetErrorString(e));
}
int* device_int(int v) {
    int* d = nullptr;
    check_cuda(cudaMalloc(&d, sizeof(int)));
    check_cuda(cudaMemcpy(d, &v, sizeof(int), cudaMemcpyHostToDevice));
    return d;
}
constexpr int kMaxRows = 4096;   // rows per forward_batch* call the operator scratch is sized for

void check_size(const std::vector<float>& v, size_t want, const char* what) {
    if (v.size() != want)
        throw std::invalid_argument(std::string(what) + " weight size mismatch: expected " + std::to_string(want) + ", got " +
                                    std::to_string(v.size()));
}

}  // namespace

// ---- CudaKVCache ------------------------------------------------------------------------------------------------
void CudaKVCache::reset(int nl, int nkh, int hd, int init_capacity) {
    if (pool) { b200attn_kv_pool_destroy(pool); pool = nullptr; }
    num_layers = nl; num_kv_heads = nkh; head_dim = hd;
    max_seq_len = std::max(init_capacity, 8192);
    capacity_seq_len = 0;
    layer_lengths.assign(nl, 0);
    const int pages = (max_seq_len + 63) / 64;
    b200attn_kv_config cfg{nl, nkh, hd, 64, pages, 1, pages, B200ATTN_KV_INT8};
    check(b200attn_kv_pool_create(&cfg, &pool));
    check(b200attn_kv_seq_alloc(pool, init_capacity, &slot));
    capacity_seq_len = ((init_capacity + 63) / 64) * 64;
    if (!d_slot) d_slot = device_int(slot);
}
void CudaKVCache::clear() {
    if (!pool) return;
    check(b200attn_kv_clear(pool, nullptr));
    std::fill(layer_lengths.begin(), layer_lengths.end(), 0);
}
void CudaKVCache::ensure_capacity(int required_seq_len) {
    if (required_seq_len > max_seq_len) throw std::runtime_error("CudaKVCache: sequence longer than the pool");
    check(b200attn_kv_seq_reserve(pool, slot, required_seq_len));
    capacity_seq_len = std::max(capacity_seq_len, ((required_seq_len + 63) / 64) * 64);
}

// ---- CudaFullAttention ----------------------------------------------------------------------------------------------
CudaFullAttention::CudaFullAttention(int hidden_size, int num_heads, int num_kv_heads, int q_head_dim, int kv_head_dim)
    : hidden_size_(hidden_size), num_heads_(num_heads), num_kv_heads_(num_kv_heads), q_head_dim_(q_head_dim),
      kv_head_dim_(kv_head_dim) {
    if (hidden_size <= 0 || num_heads <= 0 || num_kv_heads <= 0) throw std::invalid_argument("All dimensions must be > 0");
    if (q_head_dim != kv_head_dim) throw std::invalid_argument("q_head_dim must equal kv_head_dim");
    b200attn_fa_config cfg{hidden_size, num_heads, num_kv_heads, kv_head_dim, kv_head_dim / 4, 10000000.0f, B200ATTN_PROJ_FP32, 1,
                           kMaxRows};
    check(b200attn_fa_create(&cfg, &op_));
}
CudaFullAttention::~CudaFullAttention() { b200attn_fa_destroy(op_); }

void CudaFullAttention::set_weights(const std::vector<float>& q, const std::vector<float>& k, const std::vector<float>& v,
                                    const std::vector<float>& qn, const std::vector<float>& kn, const std::vector<float>& o) {
    const size_t hid = hidden_size_;
    check_size(q, (size_t)num_heads_ * q_head_dim_ * 2 * hid, "q_proj");
    check_size(k, (size_t)num_kv_heads_ * kv_head_dim_ * hid, "k_proj");
    check_size(v, (size_t)num_kv_heads_ * kv_head_dim_ * hid, "v_proj");
    check_size(qn, (size_t)kv_head_dim_, "q_norm");
    check_size(kn, (size_t)kv_head_dim_, "k_norm");
    check_size(o, hid * num_heads_ * kv_head_dim_, "o_proj");
    b200attn_fa_weights w{q.data(), k.data(), v.data(), qn.data(), kn.data(), o.data()};
    check(b200attn_fa_set_weights(op_, &w));
}

void CudaFullAttention::forward(const float* input, float* output, CudaKVCache& kv, int layer_idx, int position) const {
    if (layer_idx < 0 || layer_idx >= kv.num_layers) throw std::invalid_argument("layer_idx out of range");
    if (position != kv.layer_lengths[layer_idx])
        throw std::invalid_argument("CudaFullAttention::forward: position must equal the layer's cache length");
    kv.ensure_capacity(position + 1);
    check(b200attn_fa_decode(op_, kv.pool, layer_idx, kv.d_slot, 1, input, output, nullptr));
    kv.layer_lengths[layer_idx] += 1;
}

void CudaFullAttention::forward_batch_prefill(const float* input, float* output, CudaKVCache& kv, int layer_idx,
                                              const int* /*positions*/, int batch_size, int /*max_seq*/) const {
    if (layer_idx < 0 || layer_idx >= kv.num_layers) throw std::invalid_argument("layer_idx out of range");
    if (batch_size <= 0) throw std::invalid_argument("batch_size must be > 0");
    kv.ensure_capacity(kv.layer_lengths[layer_idx] + batch_size);
    for (int done = 0; done < batch_size; done += kMaxRows) {
        const int n = std::min(kMaxRows, batch_size - done);
        check(b200attn_fa_prefill(op_, kv.pool, layer_idx, &kv.slot, &n, 1, input + (size_t)done * hidden_size_,
                                  output + (size_t)done * hidden_size_, nullptr));
    }
    kv.layer_lengths[layer_idx] += batch_size;
}

// ---- CudaLinearAttnState ------------------------------------------------------------------------------------------------
void CudaLinearAttnState::reset(int nh, int kd, int vd, int conv_k) {
    num_heads = nh; key_dim = kd; value_dim = vd; conv_kernel = conv_k;
    conv_dim = nh * (2 * kd + vd);
    if (nh == 16 && kd == 128 && vd == 128 && conv_k == 4) {     // the sizes the library's kernels are built for
        b200attn_la_state_config cfg{1, 1, nh, kd, vd, conv_k};
        check(b200attn_la_state_create(&cfg, &state));
    }
    check_cuda(cudaMalloc(&d_conv_state, (size_t)conv_dim * (conv_k - 1) * sizeof(float)));
    check_cuda(cudaMemset(d_conv_state, 0, (size_t)conv_dim * (conv_k - 1) * sizeof(float)));
    check_cuda(cudaMalloc(&d_recurrent_state, (size_t)nh * kd * vd * sizeof(float)));
    check_cuda(cudaMemset(d_recurrent_state, 0, (size_t)nh * kd * vd * sizeof(float)));
    if (!d_slot) d_slot = device_int(0);
}
void CudaLinearAttnState::clear() {
    if (!d_recurrent_state) return;
    if (state) check(b200attn_la_state_clear(state, -1, nullptr));
    check_cuda(cudaMemset(d_recurrent_state, 0, (size_t)num_heads * key_dim * value_dim * sizeof(float)));
    check_cuda(cudaMemset(d_conv_state, 0, (size_t)conv_dim * (conv_kernel - 1) * sizeof(float)));
}

namespace {
// The public d_recurrent_state / d_conv_state arrays are the reference-layout mirror of the library state: they are
// imported before and exported after every call, so code that reads or writes them between calls keeps working.
void sync_in(CudaLinearAttnState& s) { check(b200attn_la_state_import(s.state, 0, 0, s.d_recurrent_state, s.d_conv_state, nullptr)); }
void sync_out(CudaLinearAttnState& s) { check(b200attn_la_state_export(s.state, 0, 0, s.d_recurrent_state, s.d_conv_state, nullptr)); }

bool model_sizes(int hidden, int heads, int kd, int vd, int ck) { return hidden == 1024 && heads == 16 && kd == 128 && vd == 128 && ck == 4; }
void generic_set(detail::GenericLa* g, int hidden, int heads, int kd, int vd, int ck, const std::vector<float>& qkv, const std::vector<float>& a,
                 const std::vector<float>& b, const std::vector<float>& z, const std::vector<float>& conv, const std::vector<float>& out,
                 const std::vector<float>& a_log, const std::vector<float>& dt_bias, const std::vector<float>& norm) {
    const size_t conv_dim = (size_t)heads * (2 * kd + vd);
    check_size(qkv, conv_dim * hidden, "in_proj_qkv");
    check_size(a, (size_t)heads * hidden, "in_proj_a");
    check_size(b, (size_t)heads * hidden, "in_proj_b");
    check_size(z, (size_t)heads * vd * hidden, "in_proj_z");
    check_size(conv, conv_dim * ck, "conv1d");
    check_size(out, (size_t)hidden * heads * vd, "out_proj");
    detail::generic_la_set_weights(g, qkv, a, b, z, conv, out, a_log.empty() ? std::vector<float>(heads, 0.f) : a_log,
                                   dt_bias.empty() ? std::vector<float>(heads, 0.f) : dt_bias, norm.empty() ? std::vector<float>(vd, 1.f) : norm);
}
b200attn_la make_la(int hidden, int heads, int kd, int vd, int ck, int precision) {
    if (hidden <= 0 || heads <= 0 || kd <= 0 || vd <= 0) throw std::invalid_argument("All dimensions must be > 0");
    b200attn_la_config cfg{hidden, heads, kd, vd, ck, precision, 1, kMaxRows};
    b200attn_la op = nullptr;
    check(b200attn_la_create(&cfg, &op));
    return op;
}
void la_set(b200attn_la op, int hidden, int heads, int kd, int vd, int ck, const std::vector<float>& qkv,
            const std::vector<float>& a, const std::vector<float>& b, const std::vector<float>& z, const std::vector<float>& conv,
            const std::vector<float>& out, const std::vector<float>& a_log, const std::vector<float>& dt_bias,
            const std::vector<float>& norm) {
    const size_t conv_dim = (size_t)heads * (2 * kd + vd);
    check_size(qkv, conv_dim * hidden, "in_proj_qkv");
    check_size(a, (size_t)heads * hidden, "in_proj_a");
    check_size(b, (size_t)heads * hidden, "in_proj_b");
    check_size(z, (size_t)heads * vd * hidden, "in_proj_z");
    check_size(conv, conv_dim * ck, "conv1d");
    check_size(out, (size_t)hidden * heads * vd, "out_proj");
    const std::vector<float> zeros(heads, 0.0f), ones(vd, 1.0f);
    const std::vector<float>& al = a_log.empty() ? zeros : a_log;
    const std::vector<float>& dt = dt_bias.empty() ? zeros : dt_bias;
    const std::vector<float>& nw = norm.empty() ? ones : norm;
    check_size(al, (size_t)heads, "A_log");
    check_size(dt, (size_t)heads, "dt_bias");
    check_size(nw, (size_t)vd, "norm");
    b200attn_la_weights w{qkv.data(), a.data(), b.data(), z.data(), conv.data(), al.data(), dt.data(), nw.data(), out.data()};
    check(b200attn_la_set_weights(op, &w));
}
void la_forward(b200attn_la op, const float* in, float* out, CudaLinearAttnState& s, cudaStream_t stream) {
    sync_in(s);
    check(b200attn_la_decode(op, s.state, 0, s.d_slot, 1, in, out, stream));
    sync_out(s);
}
void la_forward_batch(b200attn_la op, int hidden, const float* in, float* out, CudaLinearAttnState& s, int rows, cudaStream_t stream) {
    if (rows <= 0) throw std::invalid_argument("batch_size must be > 0");
    sync_in(s);
    const int slot = 0;
    for (int done = 0; done < rows; done += kMaxRows) {
        const int n = std::min(kMaxRows, rows - done);
        check(b200attn_la_prefill(op, s.state, 0, &slot, &n, 1, in + (size_t)done * hidden, out + (size_t)done * hidden, stream));
    }
    sync_out(s);
}
}  // namespace

// ---- CudaLinearAttention / V2 ------------------------------------------------------------------------------------------
CudaLinearAttention::CudaLinearAttention(int hidden_size, int num_heads, int key_dim, int value_dim, int conv_kernel)
    : hidden_size_(hidden_size), num_heads_(num_heads), key_dim_(key_dim), value_dim_(value_dim), conv_kernel_(conv_kernel) {
    if (model_sizes(hidden_size, num_heads, key_dim, value_dim, conv_kernel)) op_ = make_la(hidden_size, num_heads, key_dim, value_dim, conv_kernel, proj_precision_);
    else generic_ = detail::generic_la_create(hidden_size, num_heads, key_dim, value_dim, conv_kernel);
}
CudaLinearAttention::~CudaLinearAttention() { b200attn_la_destroy(op_); detail::generic_la_destroy(generic_); }
void CudaLinearAttention::set_weights(const std::vector<float>& qkv, const std::vector<float>& a, const std::vector<float>& b,
                                      const std::vector<float>& z, const std::vector<float>& conv, const std::vector<float>& out,
                                      const std::vector<float>& a_log, const std::vector<float>& dt_bias,
                                      const std::vector<float>& norm) {
    if (generic_) return generic_set(generic_, hidden_size_, num_heads_, key_dim_, value_dim_, conv_kernel_, qkv, a, b, z, conv, out, a_log, dt_bias, norm);
    la_set(op_, hidden_size_, num_heads_, key_dim_, value_dim_, conv_kernel_, qkv, a, b, z, conv, out, a_log, dt_bias, norm);
}
void CudaLinearAttention::forward(const float* in, float* out, CudaLinearAttnState& s) const {
    if (generic_) return detail::generic_la_forward(generic_, in, out, s.d_recurrent_state, s.d_conv_state, 1, nullptr);
    la_forward(op_, in, out, s, nullptr);
}
void CudaLinearAttention::forward_batch(const float* in, float* out, CudaLinearAttnState& s, int rows) const {
    if (rows <= 0) throw std::invalid_argument("batch_size must be > 0");
    if (generic_) return detail::generic_la_forward(generic_, in, out, s.d_recurrent_state, s.d_conv_state, rows, nullptr);
    la_forward_batch(op_, hidden_size_, in, out, s, rows, nullptr);
}
void CudaLinearAttention::forward_fused(const float* in, float* out, CudaLinearAttnState& s) const { forward(in, out, s); }

CudaLinearAttentionV2::CudaLinearAttentionV2(int hidden_size, int num_heads, int key_dim, int value_dim, int conv_kernel)
    : hidden_size_(hidden_size), num_heads_(num_heads), key_dim_(key_dim), value_dim_(value_dim), conv_kernel_(conv_kernel) {
    if (model_sizes(hidden_size, num_heads, key_dim, value_dim, conv_kernel)) op_ = make_la(hidden_size, num_heads, key_dim, value_dim, conv_kernel, B200ATTN_PROJ_FP32);
    else generic_ = detail::generic_la_create(hidden_size, num_heads, key_dim, value_dim, conv_kernel);
}
CudaLinearAttentionV2::~CudaLinearAttentionV2() { b200attn_la_destroy(op_); detail::generic_la_destroy(generic_); }
void CudaLinearAttentionV2::set_weights(const std::vector<float>& qkv, const std::vector<float>& a, const std::vector<float>& b,
                                        const std::vector<float>& z, const std::vector<float>& conv, const std::vector<float>& out,
                                        const std::vector<float>& a_log, const std::vector<float>& dt_bias,
                                        const std::vector<float>& norm) {
    if (generic_) return generic_set(generic_, hidden_size_, num_heads_, key_dim_, value_dim_, conv_kernel_, qkv, a, b, z, conv, out, a_log, dt_bias, norm);
    la_set(op_, hidden_size_, num_heads_, key_dim_, value_dim_, conv_kernel_, qkv, a, b, z, conv, out, a_log, dt_bias, norm);
}
void CudaLinearAttentionV2::forward(const float* in, float* out, CudaLinearAttnState& s) const {
    if (generic_) return detail::generic_la_forward(generic_, in, out, s.d_recurrent_state, s.d_conv_state, 1, nullptr);
    la_forward(op_, in, out, s, nullptr);
}
void CudaLinearAttentionV2::forward_batch(const float* in, float* out, CudaLinearAttnState& s, int rows, cudaStream_t stream) const {
    if (rows <= 0) throw std::invalid_argument("batch_size must be > 0");
    if (generic_) return detail::generic_la_forward(generic_, in, out, s.d_recurrent_state, s.d_conv_state, rows, stream);
    la_forward_batch(op_, hidden_size_, in, out, s, rows, stream);
}

}  // namespace cuda
}  // namespace qwen
