// Hybrid 24-layer stack around the attention operators, and the CUDA-graph-captured decode step.
//
// Layer wiring follows qwen::LanguageLayer::forward (src/backend/cpu/core/common/language_backbone.cpp:55-91
// in the reference): h1 = RMSNorm(x); a = attention(h1); h = x + a; h2 = RMSNorm(h); y = h + MLP(h2), with the
// (1 + w) RMSNorm of language_common.cpp:21-38 and the SwiGLU MLP of core/mlp/language_mlp.cpp:54-91.
// Engine-level behaviour mirrors qwen::cuda::CudaEngine (src/backend/cuda/kernels/cuda_engine.cu:158-519):
// per-layer weights, prefill over token batches, a decode step for the whole batch, reset_cache, and a
// graph-captured step (there: prefill, :391-479; here: decode with device-resident lengths and tokens).
// The residual stream is fp32; GEMM operands are fp16 with fp32 accumulation (cuBLAS).
#include "kernels.cuh"
#include "ptx_utils.cuh"

#include <algorithm>
#include <new>
#include <vector>

struct b200attn_stack_s {
    b200attn_stack_config cfg{};
    int n_fa = 0, n_la = 0;
    std::vector<int> layer_kind;      // 1 = full attention, 0 = DeltaNet
    std::vector<int> layer_sub;       // index inside the kv pool / state pool
    std::vector<b200attn_fa> fa;
    std::vector<b200attn_la> la;
    std::vector<float*> d_in_norm, d_post_norm;
    std::vector<__half*> d_wgu, d_wdown;   // [2*inter, hidden], [hidden, inter]
    std::vector<char> layer_ready;
    __half* d_embed = nullptr;  // [vocab, hidden]
    float* d_final_norm = nullptr;
    bool embed_ready = false;
    b200attn_kv_pool pool = nullptr;
    b200attn_la_state state = nullptr;
    b200::Scratch op_scratch;
    int max_rows = 0;
    float* d_h = nullptr;              // [max_rows, hidden] residual stream
    __half* d_xb = nullptr;     // [max_rows, hidden]
    __half* d_gu = nullptr;     // [max_rows, 2*inter]
    __half* d_act = nullptr;    // [max_rows, inter]
    float* d_last = nullptr;           // [max_seqs, hidden]
    float* d_logits = nullptr;         // [max_seqs, vocab]
    int* d_tokens = nullptr;           // [max_seqs] decode token buffer (in place)
    int* d_slots = nullptr;            // [max_seqs] identity slots
    __half* d_xh = nullptr;            // [128, hidden] fp16 copy of the residual stream in the fused decode step
    float* d_rowsq = nullptr;          // [128][kRowsqParts] partial sums of squares of the residual rows
    unsigned long long* d_packed = nullptr;   // [128] running argmax words of the LM head
    int* d_error = nullptr;            // device status word of the stack's own tcgen05 GEMMs
    int* d_last_idx = nullptr;         // [max_seqs] row of every sequence's last prompt token inside a prefill pass
    // Continuous batching: row r of a decode step is bound to slot row_slot[r] (its KV pages and DeltaNet state), -1 =
    // inactive.  Empty in the plain mode, where row r is slot r.
    bool batching = false;
    std::vector<int> row_slot;
    std::vector<int> free_slots;
    int n_active = 0;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
    int graph_nseqs = 0;
    long long graph_nodes = 0;
};

namespace b200 {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// h[row] = embed[token[row]] (fp16 -> fp32). grid rows, block 256 (4 elements per thread).
__global__ void embed_gather_kernel(const int* __restrict__ tokens, const __half* __restrict__ embed, int vocab,
                                    float* __restrict__ h) {
    pdl_enter();
    const int row = blockIdx.x;
    int tok = tokens[row];
    tok = min(max(tok, 0), vocab - 1);
    const uint2 raw = *reinterpret_cast<const uint2*>(embed + (size_t)tok * kHidden + 4 * threadIdx.x);
    const __half2* p = reinterpret_cast<const __half2*>(&raw);
    const float2 a = __half22float2(p[0]), b = __half22float2(p[1]);
    *reinterpret_cast<float4*>(h + (size_t)row * kHidden + 4 * threadIdx.x) = make_float4(a.x, a.y, b.x, b.y);
}

// The same gather for the fused decode step: besides h it leaves the fp16 copy of the row and the row's sum of squares
// (part 0 of kRowsqParts, the others zero), which the first input projection turns into the RMSNorm scale.
__global__ void __launch_bounds__(256)
embed_gather_fused_kernel(const int* __restrict__ tokens, const __half* __restrict__ embed, int vocab, float* __restrict__ h,
                          __half* __restrict__ xh, float* __restrict__ rowsq) {
    __shared__ float s_part[8];
    pdl_enter();
    const int row = blockIdx.x, t = threadIdx.x;
    int tok = tokens[row];
    tok = min(max(tok, 0), vocab - 1);
    const uint2 raw = *reinterpret_cast<const uint2*>(embed + (size_t)tok * kHidden + 4 * t);
    const __half2* p = reinterpret_cast<const __half2*>(&raw);
    const float2 a = __half22float2(p[0]), b = __half22float2(p[1]);
    *reinterpret_cast<float4*>(h + (size_t)row * kHidden + 4 * t) = make_float4(a.x, a.y, b.x, b.y);
    *reinterpret_cast<uint2*>(xh + (size_t)row * kHidden + 4 * t) = raw;
    float ss = wsum(a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y);
    if ((t & 31) == 0) s_part[t >> 5] = ss;
    __syncthreads();
    if (t < kRowsqParts) {
        float tot = 0.f;
        if (t == 0)
#pragma unroll
            for (int i = 0; i < 8; ++i) tot += s_part[i];
        rowsq[(size_t)row * kRowsqParts + t] = tot;
    }
}

// RMSNorm with (1 + w), fp32 in, fp16 out (and optional fp32 copy).  One 256-thread block per row, one float4 per
// thread; optional row gather.
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ row_index, const float* __restrict__ w, float eps,
               int rows, __half* __restrict__ out_fp16, float* __restrict__ out_f32) {
    __shared__ float s_part[8];
    const int row = blockIdx.x, t = threadIdx.x;
    const float4 ww = *reinterpret_cast<const float4*>(w + 4 * t);
    pdl_enter();
    const size_t srow = (size_t)(row_index ? row_index[row] : row);
    const float4 v = *(reinterpret_cast<const float4*>(x + srow * kHidden) + t);
    float ss = wsum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    if ((t & 31) == 0) s_part[t >> 5] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += s_part[i];
    const float rms = sqrtf(ss / (float)kHidden + eps);
    const float r0 = v.x / rms * (1.0f + ww.x), r1 = v.y / rms * (1.0f + ww.y);
    const float r2 = v.z / rms * (1.0f + ww.z), r3 = v.w / rms * (1.0f + ww.w);
    if (out_fp16) {
        __half2 a = __floats2half2_rn(r0, r1), b = __floats2half2_rn(r2, r3);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&a);
        pk.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(out_fp16 + (size_t)row * kHidden + 4 * t) = pk;
    }
    if (out_f32) *reinterpret_cast<float4*>(out_f32 + (size_t)row * kHidden + 4 * t) = make_float4(r0, r1, r2, r3);
}

// The same RMSNorm for many rows (prefill): one warp per row, 32 values per lane, four rows per
// block, so that a pass over 131072 rows is 32768 blocks of useful size instead of 131072 blocks of one float4 per thread.
__global__ void __launch_bounds__(128)
rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, int rows, __half* __restrict__ out_fp16) {
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)row * kHidden);
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[i] = src[32 * i + lane];
        ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
    ss = wsum(ss);
    const float rms = sqrtf(ss / (float)kHidden + eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 ww = *reinterpret_cast<const float4*>(w + 4 * (32 * i + lane));
        __half2 a = __floats2half2_rn(v[i].x / rms * (1.0f + ww.x), v[i].y / rms * (1.0f + ww.y));
        __half2 b = __floats2half2_rn(v[i].z / rms * (1.0f + ww.z), v[i].w / rms * (1.0f + ww.w));
        *reinterpret_cast<uint2*>(out_fp16 + (size_t)row * kHidden + 4 * (32 * i + lane)) =
            make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
    }
}

// act = silu(gate) * up.  gu rows hold tiles of 64 columns: 32 gate columns followed by the 32 matching up columns
// (the layout the decode-step GEMM epilogue consumes as well).  fp16.
__global__ void swiglu_kernel(const __half* __restrict__ gu, int inter, size_t n_oct, __half* __restrict__ act) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // index over (row, inter/8): eight outputs per thread
    if (i >= n_oct) return;
    const size_t per_row = inter / 8;
    const size_t row = i / per_row, c = (i % per_row) * 8;            // output channels c .. c+7 (inside one 32-channel tile)
    const size_t gcol = (c / 32) * 64 + (c % 32);
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + row * 2 * inter + gcol);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + row * 2 * inter + gcol + 32);
    const __half2* gp = reinterpret_cast<const __half2*>(&g4);
    const __half2* up = reinterpret_cast<const __half2*>(&u4);
    __half2 o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 g = __half22float2(gp[e]), u = __half22float2(up[e]);
        o[e] = __floats2half2_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(act + row * inter + c) = *reinterpret_cast<uint4*>(o);
}

// Greedy argmax over one row of logits (first maximum wins). grid rows, block 1024.
__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += 1024) {
        const float v = row[i];
        if (v > best) { best = v; idx = i; }
    }
    __shared__ float sb[32];
    __shared__ int si[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sb[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sb[threadIdx.x]; idx = si[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = idx;
    }
}

// Embedding ~ N(0, std) from a counter-based hash (Box-Muller), written as fp16.
__global__ void init_normal_fp16_kernel(__half* __restrict__ out, size_t n, uint64_t seed, float std_dev) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (i + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    const float u1 = ((uint32_t)(z & 0xffffffffu) + 1.0f) * (1.0f / 4294967296.0f);
    const float u2 = (uint32_t)(z >> 32) * (1.0f / 4294967296.0f);
    out[i] = __float2half_rn(std_dev * sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2));
}

__global__ void iota_kernel(int* p, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = i;
}
__global__ void last_row_index_kernel(int* idx, int n_seqs, int len) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_seqs) idx[i] = i * len + len - 1;
}

// Per-output-channel INT8 fake quantisation in place: scale = absmax/127 (1 if not > 1e-8),
// w <- clamp(roundf(w/scale)) * scale  (src/backend/cuda/kernels/mlp_cuda.cu:22-39).  One warp per row.
__global__ void quantize_rows_kernel(float* __restrict__ w, int rows, int cols) {
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (gw >= rows) return;
    float* r = w + (size_t)gw * cols;
    float amax = 0.f;
    for (int c = lane; c < cols; c += 32) amax = fmaxf(amax, fabsf(r[c]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float s = __fdiv_rn(amax, 127.0f);
    s = (s > 1e-8f) ? s : 1.0f;
    for (int c = lane; c < cols; c += 32) r[c] = fmaxf(-127.f, fminf(127.f, roundf(__fdiv_rn(r[c], s)))) * s;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Uploads a host fp32 matrix as fp16, optionally through the INT8 fake quantiser.
static int upload_matrix(const float* h, int rows, int cols, bool int8, __half** out) {
    float* tmp = nullptr;
    B2_TRY(upload_f32(h, &tmp, (size_t)rows * cols));
    if (int8) {
        quantize_rows_kernel<<<ceil_div(rows, 4), 128>>>(tmp, rows, cols);
        count_launch();
    }
    cudaError_t e = cudaMalloc(out, (size_t)rows * cols * 2);
    int st = 0;
    if (e != cudaSuccess) { set_error("cudaMalloc failed: %s", cudaGetErrorString(e)); st = B200ATTN_ERR_NOMEM; }
    if (st == 0) st = f32_to_f16(0, tmp, *out, (size_t)rows * cols);
    e = cudaDeviceSynchronize();
    cudaFree(tmp);
    if (st == 0 && e != cudaSuccess) { set_error("weight upload failed: %s", cudaGetErrorString(e)); st = B200ATTN_ERR_CUDA; }
    return st;
}

}  // namespace b200

using namespace b200;

extern "C" int b200attn_stack_destroy(b200attn_stack st) {
    if (!st) return 0;
    if (st->graph_exec) cudaGraphExecDestroy(st->graph_exec);
    if (st->graph) cudaGraphDestroy(st->graph);
    for (auto f : st->fa) b200attn_fa_destroy(f);
    for (auto l : st->la) b200attn_la_destroy(l);
    for (auto p : st->d_in_norm) cudaFree(p);
    for (auto p : st->d_post_norm) cudaFree(p);
    for (auto p : st->d_wgu) cudaFree(p);
    for (auto p : st->d_wdown) cudaFree(p);
    cudaFree(st->d_embed); cudaFree(st->d_final_norm);
    b200attn_kv_pool_destroy(st->pool);
    b200attn_la_state_destroy(st->state);
    cudaFree(st->op_scratch.base);
    cudaFree(st->d_h); cudaFree(st->d_xb); cudaFree(st->d_gu); cudaFree(st->d_act); cudaFree(st->d_last);
    cudaFree(st->d_logits); cudaFree(st->d_tokens); cudaFree(st->d_slots);
    cudaFree(st->d_xh); cudaFree(st->d_rowsq); cudaFree(st->d_packed); cudaFree(st->d_error); cudaFree(st->d_last_idx);
    delete st;
    return 0;
}

extern "C" int b200attn_stack_create(const b200attn_stack_config* cfg, b200attn_stack* out) {
    B2_CHECK_ARG(cfg && out, "stack_create: null argument");
    B2_CHECK_ARG(cfg->num_layers > 0 && cfg->intermediate_size > 0 && cfg->intermediate_size % 64 == 0 && cfg->vocab_size > 0 &&
                     cfg->max_seqs > 0 && cfg->max_seq_len > 0 && cfg->prefill_chunk_seqs > 0,
                 "stack_create: all sizes must be > 0");
    if (cfg->hidden_size != kHidden) B2_FAIL(B200ATTN_ERR_UNSUPPORTED, "stack_create: kernels are built for hidden=1024");
    refresh_runtime_flags();
    auto* st = new (std::nothrow) b200attn_stack_s();
    if (!st) B2_FAIL(B200ATTN_ERR_NOMEM, "stack_create: host allocation failed");
    st->cfg = *cfg;
    const int L = cfg->num_layers;
    st->layer_kind.resize(L); st->layer_sub.resize(L);
    for (int i = 0; i < L; ++i) {
        st->layer_kind[i] = (i % 4 == 3) ? 1 : 0;
        st->layer_sub[i] = st->layer_kind[i] ? st->n_fa++ : st->n_la++;
    }
    st->d_in_norm.assign(L, nullptr); st->d_post_norm.assign(L, nullptr);
    st->d_wgu.assign(L, nullptr); st->d_wdown.assign(L, nullptr);
    st->layer_ready.assign(L, 0);
    st->max_rows = std::max(cfg->max_seqs, cfg->prefill_chunk_seqs * cfg->max_seq_len);
    int rc = 0;
    auto fail = [&](int code) { b200attn_stack_destroy(st); return code; };
#define ST_CUDA(e) do { cudaError_t _e = (e); if (_e != cudaSuccess) { set_error("stack_create: %s: %s", #e, cudaGetErrorString(_e)); \
        return fail(_e == cudaErrorMemoryAllocation ? B200ATTN_ERR_NOMEM : B200ATTN_ERR_CUDA); } } while (0)
    const int pages_per_seq = ceil_div(cfg->max_seq_len, kPageTokens);
    if (st->n_fa > 0) {
        b200attn_kv_config kc{st->n_fa, kFaKvHeads, kHeadDim, kPageTokens, pages_per_seq * cfg->max_seqs, cfg->max_seqs,
                              pages_per_seq, cfg->kv_dtype};
        if ((rc = b200attn_kv_pool_create(&kc, &st->pool)) != 0) return fail(rc);
        for (int i = 0; i < cfg->max_seqs; ++i) {
            int slot = -1;
            if ((rc = b200attn_kv_seq_alloc(st->pool, cfg->max_seq_len, &slot)) != 0) return fail(rc);
        }
    }
    if (st->n_la > 0) {
        b200attn_la_state_config sc{st->n_la, cfg->max_seqs, kLaHeads, kLaKd, kLaVd, kLaConvK};
        if ((rc = b200attn_la_state_create(&sc, &st->state)) != 0) return fail(rc);
    }
    b200attn_fa_config fc{kHidden, kFaHeads, kFaKvHeads, kHeadDim, kRotaryDim, 1e7f, B200ATTN_PROJ_FP16, cfg->max_seqs, st->max_rows};
    b200attn_la_config lc{kHidden, kLaHeads, kLaKd, kLaVd, kLaConvK, B200ATTN_PROJ_FP16, cfg->max_seqs, st->max_rows};
    st->op_scratch.bytes = std::max(fa_scratch_bytes(fc), la_scratch_bytes(lc));
    ST_CUDA(cudaMalloc(&st->op_scratch.base, st->op_scratch.bytes));
    for (int i = 0; i < L; ++i) {
        if (st->layer_kind[i]) {
            b200attn_fa f = nullptr;
            if ((rc = fa_create_internal(&fc, &st->op_scratch, &f)) != 0) return fail(rc);
            st->fa.push_back(f);
        } else {
            b200attn_la l = nullptr;
            if ((rc = la_create_internal(&lc, &st->op_scratch, &l)) != 0) return fail(rc);
            st->la.push_back(l);
        }
    }
    const size_t R = st->max_rows;
    ST_CUDA(cudaMalloc(&st->d_h, R * kHidden * 4));
    ST_CUDA(cudaMalloc(&st->d_xb, R * kHidden * 2));
    ST_CUDA(cudaMalloc(&st->d_gu, R * 2 * cfg->intermediate_size * 2));
    ST_CUDA(cudaMalloc(&st->d_act, R * cfg->intermediate_size * 2));
    ST_CUDA(cudaMalloc(&st->d_last, (size_t)cfg->max_seqs * kHidden * 4));
    ST_CUDA(cudaMalloc(&st->d_logits, (size_t)cfg->max_seqs * cfg->vocab_size * 4));
    ST_CUDA(cudaMalloc(&st->d_tokens, (size_t)cfg->max_seqs * 4));
    ST_CUDA(cudaMalloc(&st->d_slots, (size_t)cfg->max_seqs * 4));
    ST_CUDA(cudaMemset(st->d_tokens, 0, (size_t)cfg->max_seqs * 4));
    ST_CUDA(cudaMalloc(&st->d_xh, (size_t)128 * kHidden * 2));
    ST_CUDA(cudaMalloc(&st->d_rowsq, (size_t)128 * kRowsqParts * 4));
    ST_CUDA(cudaMemset(st->d_rowsq, 0, (size_t)128 * kRowsqParts * 4));
    ST_CUDA(cudaMalloc(&st->d_packed, 128 * sizeof(unsigned long long)));
    ST_CUDA(cudaMemset(st->d_packed, 0, 128 * sizeof(unsigned long long)));
    ST_CUDA(cudaMalloc(&st->d_error, sizeof(int)));
    ST_CUDA(cudaMemset(st->d_error, 0, sizeof(int)));
    ST_CUDA(cudaMalloc(&st->d_last_idx, (size_t)cfg->max_seqs * 4));
    iota_kernel<<<ceil_div(cfg->max_seqs, 128), 128>>>(st->d_slots, cfg->max_seqs);
    ST_CUDA(cudaDeviceSynchronize());
#undef ST_CUDA
    *out = st;
    return 0;
}

extern "C" int b200attn_stack_set_layer_weights(b200attn_stack st, int layer, const b200attn_layer_weights* w) {
    B2_CHECK_ARG(st && w, "stack_set_layer_weights: null argument");
    B2_CHECK_ARG(layer >= 0 && layer < st->cfg.num_layers, "stack_set_layer_weights: layer %d out of range", layer);
    B2_CHECK_ARG(w->input_norm && w->post_norm && w->ffn_gate && w->ffn_up && w->ffn_down, "stack_set_layer_weights: null weight pointer");
    const bool q8 = st->cfg.int8_weights != 0;
    const int inter = st->cfg.intermediate_size;
    st->layer_ready[layer] = 0;
    cudaFree(st->d_in_norm[layer]); cudaFree(st->d_post_norm[layer]); cudaFree(st->d_wgu[layer]); cudaFree(st->d_wdown[layer]);
    st->d_in_norm[layer] = st->d_post_norm[layer] = nullptr; st->d_wgu[layer] = st->d_wdown[layer] = nullptr;
    // The (1 + w) factors of the two RMSNorms are folded into the columns of the matrices that consume the normalised
    // rows (after quantisation, so the INT8 codes are those of the original matrix): x / rms * (1 + w) W^T = x / rms W'^T.
    // The norm kernels of the unfused paths therefore run with zero weights, and the fused decode step needs no norm
    // launch at all: its projections scale their output rows by 1 / rms.
    const std::vector<float> zeros(kHidden, 0.f);
    B2_TRY(upload_f32(zeros.data(), &st->d_in_norm[layer], kHidden));
    B2_TRY(upload_f32(zeros.data(), &st->d_post_norm[layer], kHidden));
    // Per-output-channel INT8 fake quantisation on the host (the arithmetic of quantize_rows_kernel).
    auto q8_copy = [&](const float* src, int rows, int cols, std::vector<float>& dst) {
        dst.assign(src, src + (size_t)rows * cols);
        if (!q8) return;
        for (int r = 0; r < rows; ++r) {
            float* row = dst.data() + (size_t)r * cols;
            float amax = 0.f;
            for (int c = 0; c < cols; ++c) amax = std::max(amax, std::fabs(row[c]));
            float s = amax / 127.0f;
            s = (s > 1e-8f) ? s : 1.0f;
            for (int c = 0; c < cols; ++c) row[c] = std::max(-127.f, std::min(127.f, roundf(row[c] / s))) * s;
        }
    };
    auto fold = [&](std::vector<float>& m, int rows, const float* norm_w) {     // column k of an [rows, hidden] matrix *= 1 + w[k]
        for (int r = 0; r < rows; ++r) {
            float* row = m.data() + (size_t)r * kHidden;
            for (int c = 0; c < kHidden; ++c) row[c] *= 1.0f + norm_w[c];
        }
    };
    {
        // rows in tiles of 64: 32 gate rows then the 32 matching up rows (see swiglu_kernel)
        std::vector<float> gu_src((size_t)2 * inter * kHidden), gu;
        for (int c = 0; c < inter; ++c) {
            const size_t tile = c / 32, j = c % 32;
            std::memcpy(gu_src.data() + (tile * 64 + j) * kHidden, w->ffn_gate + (size_t)c * kHidden, (size_t)kHidden * 4);
            std::memcpy(gu_src.data() + (tile * 64 + 32 + j) * kHidden, w->ffn_up + (size_t)c * kHidden, (size_t)kHidden * 4);
        }
        q8_copy(gu_src.data(), 2 * inter, kHidden, gu);
        fold(gu, 2 * inter, w->post_norm);
        B2_TRY(upload_matrix(gu.data(), 2 * inter, kHidden, false, &st->d_wgu[layer]));
    }
    B2_TRY(upload_matrix(w->ffn_down, kHidden, inter, q8, &st->d_wdown[layer]));
    if (st->layer_kind[layer]) {
        B2_CHECK_ARG(w->fa, "stack_set_layer_weights: layer %d is full attention, fa weights missing", layer);
        std::vector<float> q, k, v, o;
        q8_copy(w->fa->q_proj, kFaHeads * kHeadDim * 2, kHidden, q);
        q8_copy(w->fa->k_proj, kFaKvHeads * kHeadDim, kHidden, k);
        q8_copy(w->fa->v_proj, kFaKvHeads * kHeadDim, kHidden, v);
        q8_copy(w->fa->o_proj, kHidden, kFaHeads * kHeadDim, o);
        fold(q, kFaHeads * kHeadDim * 2, w->input_norm);
        fold(k, kFaKvHeads * kHeadDim, w->input_norm);
        fold(v, kFaKvHeads * kHeadDim, w->input_norm);
        b200attn_fa_weights fw{q.data(), k.data(), v.data(), w->fa->q_norm, w->fa->k_norm, o.data()};
        B2_TRY(b200attn_fa_set_weights(st->fa[st->layer_sub[layer]], &fw));
    } else {
        B2_CHECK_ARG(w->la, "stack_set_layer_weights: layer %d is DeltaNet, la weights missing", layer);
        std::vector<float> qkv, a, b, z, o;
        q8_copy(w->la->in_proj_qkv, kLaConvDim, kHidden, qkv);
        q8_copy(w->la->in_proj_a, kLaHeads, kHidden, a);
        q8_copy(w->la->in_proj_b, kLaHeads, kHidden, b);
        q8_copy(w->la->in_proj_z, kLaHeads * kLaVd, kHidden, z);
        q8_copy(w->la->out_proj, kHidden, kLaHeads * kLaVd, o);
        fold(qkv, kLaConvDim, w->input_norm);
        fold(a, kLaHeads, w->input_norm);
        fold(b, kLaHeads, w->input_norm);
        fold(z, kLaHeads * kLaVd, w->input_norm);
        b200attn_la_weights lw{qkv.data(), a.data(), b.data(), z.data(), w->la->conv1d, w->la->a_log, w->la->dt_bias,
                               w->la->norm, o.data()};
        B2_TRY(b200attn_la_set_weights(st->la[st->layer_sub[layer]], &lw));
    }
    st->layer_ready[layer] = 1;
    return 0;
}

extern "C" int b200attn_stack_set_embedding(b200attn_stack st, const float* h_embed, const float* h_final_norm) {
    B2_CHECK_ARG(st && h_embed && h_final_norm, "stack_set_embedding: null argument");
    cudaFree(st->d_embed); cudaFree(st->d_final_norm);
    st->d_embed = nullptr; st->d_final_norm = nullptr; st->embed_ready = false;
    B2_TRY(upload_matrix(h_embed, st->cfg.vocab_size, kHidden, st->cfg.int8_weights != 0, &st->d_embed));
    B2_TRY(upload_f32(h_final_norm, &st->d_final_norm, kHidden));
    st->embed_ready = true;
    return 0;
}

extern "C" int b200attn_stack_init_embedding_random(b200attn_stack st, uint64_t seed, float std_dev, const float* h_final_norm) {
    B2_CHECK_ARG(st && h_final_norm, "stack_init_embedding_random: null argument");
    cudaFree(st->d_embed); cudaFree(st->d_final_norm);
    st->d_embed = nullptr; st->d_final_norm = nullptr; st->embed_ready = false;
    const size_t n = (size_t)st->cfg.vocab_size * kHidden;
    B2_CUDA(cudaMalloc(&st->d_embed, n * 2));
    init_normal_fp16_kernel<<<(unsigned)((n + 255) / 256), 256>>>(st->d_embed, n, seed, std_dev);
    B2_LAUNCH_CHECK();
    B2_CUDA(cudaDeviceSynchronize());
    B2_TRY(upload_f32(h_final_norm, &st->d_final_norm, kHidden));
    st->embed_ready = true;
    return 0;
}

extern "C" int b200attn_stack_device_status(b200attn_stack st, int* code_out) {
    B2_CHECK_ARG(st && code_out, "stack_device_status: null argument");
    *code_out = 0;
    int c = 0;
    if (st->pool) { B2_TRY(b200attn_kv_device_status(st->pool, &c)); if (c && !*code_out) *code_out = c; }
    for (auto l : st->la) { B2_TRY(b200attn_la_device_status(l, &c)); if (c && !*code_out) *code_out = c; }
    B2_CUDA(cudaDeviceSynchronize());
    B2_CUDA(cudaMemcpy(&c, st->d_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (c) { B2_CUDA(cudaMemset(st->d_error, 0, sizeof(int))); if (!*code_out) *code_out = c; }
    return 0;
}

extern "C" int b200attn_stack_reset(b200attn_stack st, b200attn_stream stream) {
    B2_CHECK_ARG(st, "stack_reset: null stack");
    if (st->pool) B2_TRY(b200attn_kv_clear(st->pool, stream));
    if (st->state) B2_TRY(b200attn_la_state_clear(st->state, -1, stream));
    if (st->batching) {     // back to the plain mode: row r is slot r, every slot holds pages for max_seq_len tokens
        st->batching = false;
        st->n_active = 0;
        if (st->pool)
            for (int i = 0; i < st->cfg.max_seqs; ++i) B2_TRY(b200attn_kv_seq_reserve(st->pool, i, st->cfg.max_seq_len));
        iota_kernel<<<ceil_div(st->cfg.max_seqs, 128), 128, 0, b200::as_stream(stream)>>>(st->d_slots, st->cfg.max_seqs);
        B2_LAUNCH_CHECK();
    }
    return 0;
}

namespace b200 {

static int stack_ready(b200attn_stack st) {
    B2_CHECK_ARG(st, "stack: null handle");
    if (!st->embed_ready) B2_FAIL(B200ATTN_ERR_NOT_READY, "stack: embedding not set");
    for (int i = 0; i < st->cfg.num_layers; ++i)
        if (!st->layer_ready[i]) B2_FAIL(B200ATTN_ERR_NOT_READY, "stack: weights of layer %d not set", i);
    return 0;
}

// All layers over `rows` rows already embedded in d_h (and, for the fused decode step, in d_xh / d_rowsq).
static int stack_layers(b200attn_stack st, int rows, const int* h_slots, const int* h_counts, int n_seqs, const int* d_slots,
                        bool decode, cudaStream_t s) {
    const int inter = st->cfg.intermediate_size;
    if (decode && rows <= 128 && gemm_tc_enabled()) {
        // Fused decode step, five launches per DeltaNet layer: input projection (RMSNorm scale in its epilogue, the norm's
        // (1 + w) folded into the weights at load), attention, output projection + residual, gate/up + SwiGLU, down +
        // residual.  The residual projections also leave the fp16 copy and the sums of squares the next projection needs.
        DecodeOut f{st->d_xh, st->d_rowsq, st->cfg.rms_eps};
        for (int i = 0; i < st->cfg.num_layers; ++i) {
            if (st->layer_kind[i])
                B2_TRY(fa_forward_rows(st->fa[st->layer_sub[i]], st->pool, st->layer_sub[i], h_slots, h_counts, n_seqs, d_slots, true,
                                       st->d_xh, true, st->d_h, 1.0f, &f, s));
            else
                B2_TRY(la_forward_rows(st->la[st->layer_sub[i]], st->state, st->layer_sub[i], h_slots, h_counts, n_seqs, d_slots, true,
                                       st->d_xh, true, st->d_h, 1.0f, &f, s));
            B2_TRY(gemm_tc_swiglu(s, st->d_xh, st->d_wgu[i], st->d_act, rows, 2 * inter, kHidden, st->d_rowsq, st->cfg.rms_eps, st->d_error));
            B2_TRY(gemm_tc_residual(s, st->d_act, st->d_wdown[i], st->d_h, st->d_xh, st->d_rowsq, rows, kHidden, inter, st->d_error));
        }
        return 0;
    }
    const bool many_rows = !decode && rows > 128;      // prefill: warp-per-row norm
    for (int i = 0; i < st->cfg.num_layers; ++i) {
        if (many_rows)
            rmsnorm_rows_kernel<<<ceil_div(rows, 4), 128, 0, s>>>(st->d_h, st->d_in_norm[i], st->cfg.rms_eps, rows, st->d_xb);
        else
            launch_pdl(rmsnorm_kernel, dim3(rows), dim3(256), 0, s, st->d_h, nullptr, st->d_in_norm[i], st->cfg.rms_eps, rows, st->d_xb, nullptr);
        B2_LAUNCH_CHECK();
        if (st->layer_kind[i])
            B2_TRY(fa_forward_rows(st->fa[st->layer_sub[i]], st->pool, st->layer_sub[i], h_slots, h_counts, n_seqs, d_slots,
                                   decode, st->d_xb, true, st->d_h, 1.0f, nullptr, s));
        else
            B2_TRY(la_forward_rows(st->la[st->layer_sub[i]], st->state, st->layer_sub[i], h_slots, h_counts, n_seqs, d_slots,
                                   decode, st->d_xb, true, st->d_h, 1.0f, nullptr, s));
        if (many_rows)
            rmsnorm_rows_kernel<<<ceil_div(rows, 4), 128, 0, s>>>(st->d_h, st->d_post_norm[i], st->cfg.rms_eps, rows, st->d_xb);
        else
            launch_pdl(rmsnorm_kernel, dim3(rows), dim3(256), 0, s, st->d_h, nullptr, st->d_post_norm[i], st->cfg.rms_eps, rows, st->d_xb, nullptr);
        B2_LAUNCH_CHECK();
        B2_TRY(gemm_xwT(s, st->d_xb, true, st->d_wgu[i], true, st->d_gu, true, rows, 2 * inter, kHidden));
        const size_t octs = (size_t)rows * inter / 8;
        swiglu_kernel<<<(unsigned)((octs + 255) / 256), 256, 0, s>>>(st->d_gu, inter, octs, st->d_act);
        B2_LAUNCH_CHECK();
        B2_TRY(gemm_xwT(s, st->d_act, true, st->d_wdown[i], true, st->d_h, false, rows, kHidden, inter, 1.0f));
    }
    return 0;
}

// Final norm of the selected rows, tied LM head, greedy argmax.
static int stack_head(b200attn_stack st, int n_seqs, const int* d_row_index, int* d_next, float* d_hidden_out, cudaStream_t s) {
    launch_pdl(rmsnorm_kernel, dim3(n_seqs), dim3(256), 0, s, st->d_h, d_row_index, st->d_final_norm, st->cfg.rms_eps, n_seqs, st->d_xb,
               d_hidden_out);
    B2_LAUNCH_CHECK();
    // LM head with the argmax in the GEMM epilogue (the logits never reach memory): 103 us per step against 112 + 31 us for
    // the cuBLAS GEMM and the argmax kernel.  B200ATTN_LM_HEAD=cublas (read at create time) selects the latter.
    if (n_seqs <= 128 && !g_flags.lm_head_cublas)
        return gemm_tc_argmax(s, st->d_xb, st->d_embed, st->d_packed, d_next, n_seqs, st->cfg.vocab_size, kHidden, st->d_error);
    B2_TRY(gemm_xwT(s, st->d_xb, true, st->d_embed, true, st->d_logits, false, n_seqs, st->cfg.vocab_size, kHidden));
    argmax_kernel<<<n_seqs, 1024, 0, s>>>(st->d_logits, st->cfg.vocab_size, d_next);
    B2_LAUNCH_CHECK();
    return 0;
}

static int stack_decode_step(b200attn_stack st, int n_seqs, const int* d_tokens_in, int* d_tokens_out, cudaStream_t s) {
    if (n_seqs <= 128 && gemm_tc_enabled())
        launch_pdl(embed_gather_fused_kernel, dim3(n_seqs), dim3(256), 0, s, d_tokens_in, st->d_embed, st->cfg.vocab_size, st->d_h, st->d_xh,
                   st->d_rowsq);
    else
        launch_pdl(embed_gather_kernel, dim3(n_seqs), dim3(256), 0, s, d_tokens_in, st->d_embed, st->cfg.vocab_size, st->d_h);
    B2_LAUNCH_CHECK();
    B2_TRY(stack_layers(st, n_seqs, nullptr, nullptr, n_seqs, st->d_slots, true, s));
    return stack_head(st, n_seqs, nullptr, d_tokens_out, nullptr, s);
}

}  // namespace b200

namespace b200 {
// Prefill of n_seqs prompts of prompt_len tokens into the given slots (host array); the greedy next token of sequence
// i goes to d_next[i].
static int stack_prefill_slots(b200attn_stack st, const int* h_slots, int n_seqs, int prompt_len, const int* d_tokens, int* d_next,
                               float* d_hidden_out, cudaStream_t s) {
    const int chunk = std::max(1, std::min(n_seqs, st->max_rows / prompt_len));
    std::vector<int> counts(chunk, prompt_len);
    int* d_idx = st->d_last_idx;   // row of each sequence's last token inside the pass
    int rc = 0;
    for (int s0 = 0; s0 < n_seqs && rc == 0; s0 += chunk) {
        const int n = std::min(chunk, n_seqs - s0);
        const int rows = n * prompt_len;
        launch_pdl(embed_gather_kernel, dim3(rows), dim3(256), 0, s, d_tokens + (size_t)s0 * prompt_len, st->d_embed, st->cfg.vocab_size, st->d_h);
        count_launch();
        rc = stack_layers(st, rows, h_slots + s0, counts.data(), n, nullptr, false, s);
        if (rc != 0) break;
        last_row_index_kernel<<<ceil_div(n, 128), 128, 0, s>>>(d_idx, n, prompt_len);
        count_launch();
        rc = stack_head(st, n, d_idx, d_next + s0, d_hidden_out ? d_hidden_out + (size_t)s0 * kHidden : nullptr, s);
    }
    return rc;
}
}  // namespace b200

extern "C" int b200attn_stack_prefill(b200attn_stack st, int n_seqs, int prompt_len, const int* d_tokens, int* d_next,
                                      float* d_hidden_out, b200attn_stream stream) {
    B2_TRY(stack_ready(st));
    B2_CHECK_ARG(d_tokens && d_next, "stack_prefill: null argument");
    B2_CHECK_ARG(n_seqs > 0 && n_seqs <= st->cfg.max_seqs, "stack_prefill: n_seqs %d outside (0, %d]", n_seqs, st->cfg.max_seqs);
    B2_CHECK_ARG(prompt_len > 0 && prompt_len <= st->cfg.max_seq_len, "stack_prefill: prompt_len %d outside (0, %d]", prompt_len, st->cfg.max_seq_len);
    if (st->batching) B2_FAIL(B200ATTN_ERR_INVALID, "stack_prefill: the stack is in continuous-batching mode (use b200attn_stack_admit, or b200attn_stack_reset first)");
    std::vector<int> slots(n_seqs);
    for (int i = 0; i < n_seqs; ++i) slots[i] = i;
    return stack_prefill_slots(st, slots.data(), n_seqs, prompt_len, d_tokens, d_next, d_hidden_out, as_stream(stream));
}

// ---- continuous batching ---------------------------------------------------------------------------------------------
namespace b200 {
static int push_row_slots(b200attn_stack st, cudaStream_t s) {
    B2_CUDA(cudaMemcpyAsync(st->d_slots, st->row_slot.data(), st->row_slot.size() * sizeof(int), cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaStreamSynchronize(s));      // the host vector may change right after
    return 0;
}
}  // namespace b200

extern "C" int b200attn_stack_begin_batching(b200attn_stack st, b200attn_stream stream) {
    B2_TRY(stack_ready(st));
    cudaStream_t s = as_stream(stream);
    B2_CUDA(cudaStreamSynchronize(s));
    B2_TRY(b200attn_stack_reset(st, stream));
    const int n = st->cfg.max_seqs;
    st->batching = true;
    st->row_slot.assign(n, -1);
    st->free_slots.clear();
    for (int i = n - 1; i >= 0; --i) st->free_slots.push_back(i);          // slot 0 is handed out first
    st->n_active = 0;
    if (st->pool)
        for (int i = 0; i < n; ++i) B2_TRY(b200attn_kv_seq_shrink(st->pool, i, 0));   // pages go back to the pool (one stays with the slot)
    return push_row_slots(st, s);
}

extern "C" int b200attn_stack_admit(b200attn_stack st, const int* d_prompt, int prompt_len, int reserve_tokens, int* row_out,
                                    b200attn_stream stream) {
    B2_TRY(stack_ready(st));
    B2_CHECK_ARG(d_prompt && row_out, "stack_admit: null argument");
    if (!st->batching) B2_FAIL(B200ATTN_ERR_INVALID, "stack_admit: call b200attn_stack_begin_batching first");
    B2_CHECK_ARG(prompt_len > 0 && prompt_len <= reserve_tokens && reserve_tokens <= st->cfg.max_seq_len,
                 "stack_admit: need 0 < prompt_len (%d) <= reserve_tokens (%d) <= max_seq_len (%d)", prompt_len, reserve_tokens, st->cfg.max_seq_len);
    B2_CHECK_ARG(prompt_len <= st->max_rows, "stack_admit: prompt of %d tokens exceeds the prefill scratch (%d rows)", prompt_len, st->max_rows);
    if (st->free_slots.empty()) B2_FAIL(B200ATTN_ERR_NOMEM, "stack_admit: all %d rows are in use", st->cfg.max_seqs);
    cudaStream_t s = as_stream(stream);
    const int slot = st->free_slots.back();
    if (st->pool) B2_TRY(b200attn_kv_seq_reserve(st->pool, slot, reserve_tokens));      // NOMEM when the page pool cannot hold it: nothing changed
    st->free_slots.pop_back();
    if (st->state) B2_TRY(b200attn_la_state_clear(st->state, slot, stream));
    const int row = st->n_active;
    B2_TRY(stack_prefill_slots(st, &slot, 1, prompt_len, d_prompt, st->d_tokens + row, nullptr, s));
    st->row_slot[row] = slot;
    st->n_active = row + 1;
    B2_TRY(push_row_slots(st, s));
    *row_out = row;
    return 0;
}

extern "C" int b200attn_stack_retire(b200attn_stack st, int row, b200attn_stream stream) {
    B2_CHECK_ARG(st, "stack_retire: null stack");
    if (!st->batching) B2_FAIL(B200ATTN_ERR_INVALID, "stack_retire: the stack is not in continuous-batching mode");
    B2_CHECK_ARG(row >= 0 && row < st->n_active, "stack_retire: row %d is not active (%d active rows)", row, st->n_active);
    cudaStream_t s = as_stream(stream);
    B2_CUDA(cudaStreamSynchronize(s));            // no step may be in flight while rows move
    const int slot = st->row_slot[row], last = st->n_active - 1;
    if (st->pool) B2_TRY(b200attn_kv_seq_shrink(st->pool, slot, 0));
    st->free_slots.push_back(slot);
    if (row != last) {                            // keep the rows dense: the last active row takes the freed place
        st->row_slot[row] = st->row_slot[last];
        B2_CUDA(cudaMemcpyAsync(st->d_tokens + row, st->d_tokens + last, sizeof(int), cudaMemcpyDeviceToDevice, s));
    }
    st->row_slot[last] = -1;
    st->n_active = last;
    return push_row_slots(st, s);
}

extern "C" int b200attn_stack_rows(b200attn_stack st, int* n_active_out, int* h_row_slots) {
    B2_CHECK_ARG(st && n_active_out, "stack_rows: null argument");
    *n_active_out = st->batching ? st->n_active : 0;
    if (h_row_slots && st->batching) std::memcpy(h_row_slots, st->row_slot.data(), st->row_slot.size() * sizeof(int));
    return 0;
}

extern "C" int b200attn_stack_step(b200attn_stack st, int n_rows, b200attn_stream stream) {
    B2_TRY(stack_ready(st));
    B2_CHECK_ARG(n_rows > 0 && n_rows <= st->cfg.max_seqs, "stack_step: n_rows %d outside (0, %d]", n_rows, st->cfg.max_seqs);
    if (st->graph_exec && st->graph_nseqs == n_rows) return b200attn_decode_graph_launch(st, 1, stream);
    return stack_decode_step(st, n_rows, st->d_tokens, st->d_tokens, as_stream(stream));
}

extern "C" int b200attn_stack_decode(b200attn_stack st, int n_seqs, const int* d_tokens_in, int* d_tokens_out,
                                     b200attn_stream stream) {
    B2_TRY(stack_ready(st));
    B2_CHECK_ARG(d_tokens_in && d_tokens_out, "stack_decode: null argument");
    B2_CHECK_ARG(n_seqs > 0 && n_seqs <= st->cfg.max_seqs, "stack_decode: n_seqs %d outside (0, %d]", n_seqs, st->cfg.max_seqs);
    return stack_decode_step(st, n_seqs, d_tokens_in, d_tokens_out, as_stream(stream));
}

extern "C" int b200attn_decode_graph_capture(b200attn_stack st, int n_seqs, b200attn_stream stream) {
    B2_TRY(stack_ready(st));
    B2_CHECK_ARG(n_seqs > 0 && n_seqs <= st->cfg.max_seqs, "decode_graph_capture: n_seqs %d outside (0, %d]", n_seqs, st->cfg.max_seqs);
    cudaStream_t s = as_stream(stream);
    B2_CHECK_ARG(s != nullptr, "decode_graph_capture: needs a non-default stream");
    if (st->graph_exec) { cudaGraphExecDestroy(st->graph_exec); st->graph_exec = nullptr; }
    if (st->graph) { cudaGraphDestroy(st->graph); st->graph = nullptr; }
    B2_TRY(cublas_init());
    B2_CUDA(cudaStreamSynchronize(s));
    B2_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    const long long before = g_launches;
    const int rc = stack_decode_step(st, n_seqs, st->d_tokens, st->d_tokens, s);
    g_launches = before;   // captured launches do not run now
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(s, &g);
    if (rc != 0) { if (g) cudaGraphDestroy(g); return rc; }
    if (e != cudaSuccess || !g) B2_FAIL(B200ATTN_ERR_CUDA, "decode_graph_capture: end capture failed: %s", cudaGetErrorString(e));
    st->graph = g;
    e = cudaGraphInstantiate(&st->graph_exec, g, 0);
    if (e != cudaSuccess) B2_FAIL(B200ATTN_ERR_CUDA, "decode_graph_capture: instantiate failed: %s", cudaGetErrorString(e));
    size_t nodes = 0;
    cudaGraphGetNodes(g, nullptr, &nodes);
    st->graph_nodes = (long long)nodes;
    st->graph_nseqs = n_seqs;
    return 0;
}

extern "C" int b200attn_decode_graph_launch(b200attn_stack st, int steps, b200attn_stream stream) {
    B2_CHECK_ARG(st, "decode_graph_launch: null stack");
    if (!st->graph_exec) B2_FAIL(B200ATTN_ERR_NOT_READY, "decode_graph_launch: no captured graph");
    B2_CHECK_ARG(steps > 0, "decode_graph_launch: steps must be > 0");
    for (int i = 0; i < steps; ++i) B2_CUDA(cudaGraphLaunch(st->graph_exec, as_stream(stream)));
    g_launches += st->graph_nodes * steps;
    if (st->pool) st->pool->lens_dirty = true;
    return 0;
}

extern "C" int b200attn_stack_set_tokens(b200attn_stack st, const int* d_tokens, int n_seqs, b200attn_stream stream) {
    B2_CHECK_ARG(st && d_tokens && n_seqs > 0 && n_seqs <= st->cfg.max_seqs, "stack_set_tokens: bad argument");
    B2_CUDA(cudaMemcpyAsync(st->d_tokens, d_tokens, (size_t)n_seqs * 4, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return 0;
}

extern "C" int b200attn_stack_get_tokens(b200attn_stack st, int* d_tokens, int n_seqs, b200attn_stream stream) {
    B2_CHECK_ARG(st && d_tokens && n_seqs > 0 && n_seqs <= st->cfg.max_seqs, "stack_get_tokens: bad argument");
    B2_CUDA(cudaMemcpyAsync(d_tokens, st->d_tokens, (size_t)n_seqs * 4, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return 0;
}
