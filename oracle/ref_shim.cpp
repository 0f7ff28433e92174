// TEST INFRASTRUCTURE ONLY — C shim over the reference's own CPU classes.
//
// This file is compiled together with the reference's unmodified sources
//   src/backend/cpu/core/attention/language_full_attn.cpp
//   src/backend/cpu/core/attention/language_linear_attn.cpp
//   src/backend/cpu/core/mlp/language_mlp.cpp
// (read in place from the reference checkout, never copied) into
// oracle/_ref/libqwen_ref.so.  It only forwards plain C calls to
// qwen::FullAttention / qwen::LinearAttention / qwen::MLP so that the Python
// tests and the CPU-baseline leg of the benchmark can drive the real reference.
// Nothing in the product library links or loads it.
#include <cstring>
#include <exception>
#include <vector>

#include "language_full_attn.hpp"
#include "language_linear_attn.hpp"
#include "language_mlp.hpp"

namespace {
thread_local char g_err[512];
template <class F> int guarded(F&& f) {
    try { f(); return 0; }
    catch (const std::exception& e) { std::strncpy(g_err, e.what(), sizeof(g_err) - 1); return -1; }
    catch (...) { std::strncpy(g_err, "unknown exception", sizeof(g_err) - 1); return -2; }
}
std::vector<float> vec(const float* p, size_t n) { return std::vector<float>(p, p + n); }

struct FullAttn {
    qwen::FullAttention op;
    qwen::KVCache cache;
    FullAttn(int hidden, int heads, int kv_heads, int q_dim, int kv_dim)
        : op(hidden, heads, kv_heads, q_dim, kv_dim) {}
};
struct LinAttn {
    qwen::LinearAttention op;
    qwen::LinearAttnState state;
    LinAttn(int hidden, int heads, int kd, int vd, int ck) : op(hidden, heads, kd, vd, ck) {
        state.reset(heads, kd, vd, ck);
    }
};
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err; }

// ---- qwen::FullAttention (language_full_attn.hpp:57-123) --------------------------------
void* ref_fa_create(int hidden, int heads, int kv_heads, int q_dim, int kv_dim, int num_layers,
                    int max_seq) {
    FullAttn* p = nullptr;
    if (guarded([&] {
            p = new FullAttn(hidden, heads, kv_heads, q_dim, kv_dim);
            p->cache.reset(num_layers, kv_heads, kv_dim, max_seq);
        }) != 0)
        return nullptr;
    return p;
}
void ref_fa_destroy(void* h) { delete static_cast<FullAttn*>(h); }
int ref_fa_set_weights(void* h, const float* wq, const float* wk, const float* wv,
                       const float* qn, const float* kn, const float* wo) {
    auto* p = static_cast<FullAttn*>(h);
    const size_t hid = p->op.hidden_size(), nh = p->op.num_heads(), nkv = p->op.num_kv_heads();
    const size_t qd = p->op.q_head_dim(), kd = p->op.kv_head_dim();
    return guarded([&] {
        p->op.set_weights(vec(wq, nh * qd * 2 * hid), vec(wk, nkv * kd * hid), vec(wv, nkv * kd * hid),
                          vec(qn, kd), vec(kn, kd), vec(wo, hid * nh * kd));
    });
}
// One token through FullAttention::forward (language_full_attn.cpp:115-225); appends to the cache.
int ref_fa_forward(void* h, const float* x, float* y, int layer_idx, int position) {
    auto* p = static_cast<FullAttn*>(h);
    return guarded([&] {
        std::vector<float> out = p->op.forward(vec(x, p->op.hidden_size()), p->cache, layer_idx, position);
        std::memcpy(y, out.data(), out.size() * sizeof(float));
    });
}
void ref_fa_cache_clear(void* h) { static_cast<FullAttn*>(h)->cache.clear(); }
int ref_fa_cache_len(void* h, int layer_idx) { return static_cast<FullAttn*>(h)->cache.length(layer_idx); }
// Copies the fp32 K / V rows [len, kv_heads*kv_dim] of one layer out of qwen::KVCache.
int ref_fa_cache_read(void* h, int layer_idx, float* k_out, float* v_out) {
    auto* p = static_cast<FullAttn*>(h);
    const size_t n = static_cast<size_t>(p->cache.length(layer_idx)) * p->cache.num_kv_heads * p->cache.head_dim;
    std::memcpy(k_out, p->cache.get_k(layer_idx), n * sizeof(float));
    std::memcpy(v_out, p->cache.get_v(layer_idx), n * sizeof(float));
    return 0;
}

// ---- qwen::LinearAttention (language_linear_attn.hpp:37-85) ------------------------------
void* ref_la_create(int hidden, int heads, int kd, int vd, int conv_k) {
    LinAttn* p = nullptr;
    if (guarded([&] { p = new LinAttn(hidden, heads, kd, vd, conv_k); }) != 0) return nullptr;
    return p;
}
void ref_la_destroy(void* h) { delete static_cast<LinAttn*>(h); }
// Argument order is the CPU class's: qkv, a, b, z, conv, A_log, dt_bias, norm, out.
int ref_la_set_weights(void* h, const float* qkv, const float* a, const float* b, const float* z,
                       const float* conv, const float* a_log, const float* dt_bias,
                       const float* norm, const float* out) {
    auto* p = static_cast<LinAttn*>(h);
    const size_t hid = p->op.hidden_size(), nh = p->op.num_heads(), kd = p->op.key_dim(), vd = p->op.value_dim();
    const size_t conv_dim = nh * (2 * kd + vd);
    const size_t ck = p->state.conv_kernel;
    return guarded([&] {
        p->op.set_weights(vec(qkv, conv_dim * hid), vec(a, nh * hid), vec(b, nh * hid),
                          vec(z, nh * vd * hid), vec(conv, conv_dim * ck), vec(a_log, nh),
                          vec(dt_bias, nh), vec(norm, vd), vec(out, hid * nh * vd));
    });
}
// One token through LinearAttention::forward (language_linear_attn.cpp:125-266).
int ref_la_forward(void* h, const float* x, float* y) {
    auto* p = static_cast<LinAttn*>(h);
    return guarded([&] {
        std::vector<float> out = p->op.forward(vec(x, p->op.hidden_size()), p->state);
        std::memcpy(y, out.data(), out.size() * sizeof(float));
    });
}
void ref_la_state_clear(void* h) { static_cast<LinAttn*>(h)->state.clear(); }
// recurrent [heads][kd*vd]; conv [conv_dim][conv_k-1] with index 0 = newest (language_linear_attn.cpp:154-159).
int ref_la_state_get(void* h, float* recurrent, float* conv) {
    auto* p = static_cast<LinAttn*>(h);
    size_t o = 0;
    for (auto& s : p->state.recurrent_state) { std::memcpy(recurrent + o, s.data(), s.size() * 4); o += s.size(); }
    o = 0;
    for (auto& s : p->state.conv_state) { std::memcpy(conv + o, s.data(), s.size() * 4); o += s.size(); }
    return 0;
}
int ref_la_state_set(void* h, const float* recurrent, const float* conv) {
    auto* p = static_cast<LinAttn*>(h);
    size_t o = 0;
    for (auto& s : p->state.recurrent_state) { std::memcpy(s.data(), recurrent + o, s.size() * 4); o += s.size(); }
    o = 0;
    for (auto& s : p->state.conv_state) { std::memcpy(s.data(), conv + o, s.size() * 4); o += s.size(); }
    return 0;
}

// ---- qwen::MLP (language_mlp.hpp) — used only by the whole-stack CPU baseline ---------------
void* ref_mlp_create(int hidden, int inter, const float* gate, const float* up, const float* down) {
    qwen::MLP* p = nullptr;
    if (guarded([&] {
            p = new qwen::MLP(hidden, inter);
            const size_t n = static_cast<size_t>(hidden) * inter;
            p->set_weights(vec(gate, n), vec(up, n), vec(down, n));
        }) != 0)
        return nullptr;
    return p;
}
void ref_mlp_destroy(void* h) { delete static_cast<qwen::MLP*>(h); }
int ref_mlp_forward(void* h, const float* x, float* y, int hidden) {
    auto* p = static_cast<qwen::MLP*>(h);
    return guarded([&] {
        std::vector<float> out = p->forward(vec(x, hidden));
        std::memcpy(y, out.data(), out.size() * sizeof(float));
    });
}

}  // extern "C"
