// Gated full-attention operator: weights, scratch, and the prefill / decode sequencing of
// projection GEMM -> Q/K epilogues + quantise-on-append -> attention core -> output projection.
// Mirrors qwen::cuda::CudaFullAttention (src/backend/cuda/kernels/full_attention_cuda.cu:174-250,
// 369-449, 644-715 in the reference).
#include "kernels.cuh"

#include <algorithm>
#include <cmath>
#include <new>
#include <vector>

namespace b200 {

constexpr int kMaxSplitsCap = kFaDecodeParts;

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t fa_scratch_bytes(const b200attn_fa_config& c) {
    const size_t R = (size_t)std::max(c.max_batch, c.max_prefill_rows);
    const size_t B = (size_t)c.max_batch;
    size_t n = 0;
    n += align_up(R * kFaQkvCols * 4, 256);                 // qkv_raw
    n += 2 * align_up(R * kFaHeads * kHeadDim * 2, 256);    // q, gate
    n += 2 * align_up(R * kFaKvHeads * kHeadDim * 2, 256);  // kstage, vstage
    n += 2 * align_up(R * kHidden * 2, 256);                // xb, xlo
    n += align_up(R * kFaHeads * kHeadDim * 4, 256);        // attn
    n += align_up(B * kFaKvHeads * kMaxSplitsCap * 4 * kHeadDim * 4, 256);   // part_o
    n += align_up(B * kFaKvHeads * kMaxSplitsCap * 4 * 2 * 4, 256);          // part_ml
    n += align_up((4 * R + 65536) * 4, 256);                // meta
    return n;
}

void fa_carve_scratch(b200attn_fa fa) {
    const b200attn_fa_config& c = fa->cfg;
    const size_t R = (size_t)std::max(c.max_batch, c.max_prefill_rows);
    const size_t B = (size_t)c.max_batch;
    char* p = fa->scratch.base;
    auto take = [&](size_t bytes) { char* r = p; p += align_up(bytes, 256); return r; };
    fa->max_rows = (int)R;
    fa->d_qkv_raw = (float*)take(R * kFaQkvCols * 4);
    fa->d_q = (__half*)take(R * kFaHeads * kHeadDim * 2);
    fa->d_gate = (__half*)take(R * kFaHeads * kHeadDim * 2);
    fa->d_kstage = (__half*)take(R * kFaKvHeads * kHeadDim * 2);
    fa->d_vstage = (__half*)take(R * kFaKvHeads * kHeadDim * 2);
    fa->d_xb = (__half*)take(R * kHidden * 2);
    fa->d_xlo = (__half*)take(R * kHidden * 2);
    fa->d_attn = take(R * kFaHeads * kHeadDim * 4);
    fa->d_part_o = (float*)take(B * kFaKvHeads * kMaxSplitsCap * 4 * kHeadDim * 4);
    fa->d_part_ml = (float*)take(B * kFaKvHeads * kMaxSplitsCap * 4 * 2 * 4);
    fa->meta_cap = (int)(4 * R + 65536);
    fa->d_meta = (int*)take((size_t)fa->meta_cap * 4);
    fa->max_splits = kMaxSplitsCap;
}

int fa_create_internal(const b200attn_fa_config* cfg, const Scratch* shared, b200attn_fa* out) {
    B2_CHECK_ARG(cfg && out, "fa_create: null argument");
    if (cfg->hidden_size != kHidden || cfg->num_heads != kFaHeads || cfg->num_kv_heads != kFaKvHeads ||
        cfg->head_dim != kHeadDim || cfg->rotary_dim != kRotaryDim)
        B2_FAIL(B200ATTN_ERR_UNSUPPORTED,
                "fa_create: kernels are built for hidden=1024, heads=8, kv_heads=2, head_dim=256, rotary_dim=64");
    B2_CHECK_ARG(cfg->hidden_size > 0 && cfg->num_heads > 0 && cfg->num_kv_heads > 0, "All dimensions must be > 0");
    B2_CHECK_ARG(cfg->max_batch > 0 && cfg->max_prefill_rows >= 0, "fa_create: max_batch must be > 0");
    B2_CHECK_ARG(cfg->proj_precision == B200ATTN_PROJ_FP32 || cfg->proj_precision == B200ATTN_PROJ_FP16,
                 "fa_create: bad proj_precision");
    refresh_runtime_flags();
    auto* fa = new (std::nothrow) b200attn_fa_s();
    if (!fa) B2_FAIL(B200ATTN_ERR_NOMEM, "fa_create: host allocation failed");
    fa->cfg = *cfg;
    const size_t need = fa_scratch_bytes(*cfg);
    if (shared) {
        if (shared->bytes < need) { delete fa; B2_FAIL(B200ATTN_ERR_INVALID, "fa_create: shared scratch too small"); }
        fa->scratch = *shared;
        fa->scratch.owned = false;
    } else {
        cudaError_t e = cudaMalloc(&fa->scratch.base, need);
        if (e != cudaSuccess) { delete fa; B2_FAIL(B200ATTN_ERR_NOMEM, "fa_create: scratch cudaMalloc(%zu) failed: %s", need, cudaGetErrorString(e)); }
        fa->scratch.bytes = need;
        fa->scratch.owned = true;
    }
    fa_carve_scratch(fa);
    // The arrival counters must read zero at every launch, so they are an allocation of their own: operators of one stack
    // overlay their working buffers on one scratch area, and counters inside it would be overwritten by another
    // operator's data.
    if (cudaMalloc(&fa->d_counters, (size_t)cfg->max_batch * kFaKvHeads * 4) != cudaSuccess ||
        cudaMemset(fa->d_counters, 0, (size_t)cfg->max_batch * kFaKvHeads * 4) != cudaSuccess) {
        b200attn_fa_destroy(fa);
        B2_FAIL(B200ATTN_ERR_CUDA, "fa_create: clearing the split counters failed");
    }
    // inv_freq[i] = 1 / theta^(2i / rotary_dim), evaluated in fp32 exactly as the reference does
    // (language_full_attn.cpp:93-95).
    std::vector<float> inv(kRotaryDim / 2);
    for (int i = 0; i < kRotaryDim / 2; ++i)
        inv[i] = 1.0f / std::pow(cfg->rope_theta, static_cast<float>(2 * i) / kRotaryDim);
    int st = upload_f32(inv.data(), &fa->d_inv_freq, inv.size());
    if (st != 0) { b200attn_fa_destroy(fa); return st; }
    st = cublas_init();
    if (st != 0) { b200attn_fa_destroy(fa); return st; }
    *out = fa;
    return 0;
}

}  // namespace b200

using namespace b200;

extern "C" int b200attn_fa_create(const b200attn_fa_config* cfg, b200attn_fa* out) {
    return fa_create_internal(cfg, nullptr, out);
}

extern "C" int b200attn_fa_destroy(b200attn_fa fa) {
    if (!fa) return 0;
    cudaFree(fa->d_wqkv_f32); cudaFree(fa->d_wqkv_fp16); cudaFree(fa->d_wkv_lo); cudaFree(fa->d_wo_f32); cudaFree(fa->d_wo_fp16);
    cudaFree(fa->d_qnorm); cudaFree(fa->d_knorm); cudaFree(fa->d_inv_freq);
    if (fa->scratch.owned) cudaFree(fa->scratch.base);
    cudaFree(fa->d_counters);
    delete fa;
    return 0;
}

extern "C" int b200attn_fa_set_weights(b200attn_fa fa, const b200attn_fa_weights* w) {
    B2_CHECK_ARG(fa && w, "fa_set_weights: null argument");
    B2_CHECK_ARG(w->q_proj && w->k_proj && w->v_proj && w->q_norm && w->k_norm && w->o_proj, "fa_set_weights: null weight pointer");
    const size_t nq = (size_t)kFaHeads * kHeadDim * 2 * kHidden, nkv = (size_t)kFaKvHeads * kHeadDim * kHidden;
    std::vector<float> cat((size_t)kFaQkvCols * kHidden);
    std::memcpy(cat.data(), w->q_proj, nq * 4);
    std::memcpy(cat.data() + nq, w->k_proj, nkv * 4);
    std::memcpy(cat.data() + nq + nkv, w->v_proj, nkv * 4);
    cudaFree(fa->d_wqkv_f32); cudaFree(fa->d_wqkv_fp16); cudaFree(fa->d_wkv_lo); cudaFree(fa->d_wo_f32); cudaFree(fa->d_wo_fp16);
    cudaFree(fa->d_qnorm); cudaFree(fa->d_knorm);
    fa->d_wqkv_f32 = nullptr; fa->d_wqkv_fp16 = nullptr; fa->d_wkv_lo = nullptr; fa->d_wo_f32 = nullptr; fa->d_wo_fp16 = nullptr;
    fa->d_qnorm = nullptr; fa->d_knorm = nullptr;
    fa->ready = false;
    const size_t no = (size_t)kHidden * kFaHeads * kHeadDim;
    if (fa->cfg.proj_precision == B200ATTN_PROJ_FP16) {
        B2_TRY(upload_f16_from_f32(cat.data(), &fa->d_wqkv_fp16, cat.size()));
        B2_TRY(upload_f16_from_f32(w->o_proj, &fa->d_wo_fp16, no));
        // Low-order halves of the K and V rows, w = fp16(w) + lo / kLoScale: an INT8 cache quantises K and V, and a
        // projection error of 2^-12 would move about one code in two hundred across a rounding boundary (a change of a
        // whole quantisation step), so for such caches the K / V columns are computed with compensated operands.
        std::vector<float> lo(2 * nkv);
        for (size_t i = 0; i < 2 * nkv; ++i) {
            const float v = cat[nq + i];
            lo[i] = (v - __half2float(__float2half_rn(v))) * kLoScale;
        }
        B2_TRY(upload_f16_from_f32(lo.data(), &fa->d_wkv_lo, lo.size()));
    } else {
        B2_TRY(upload_f32(cat.data(), &fa->d_wqkv_f32, cat.size()));
        B2_TRY(upload_f32(w->o_proj, &fa->d_wo_f32, no));
    }
    B2_TRY(upload_f32(w->q_norm, &fa->d_qnorm, kHeadDim));
    B2_TRY(upload_f32(w->k_norm, &fa->d_knorm, kHeadDim));
    fa->ready = true;
    return 0;
}

namespace b200 {

static int fa_check(b200attn_fa fa, b200attn_kv_pool pool, int layer) {
    B2_CHECK_ARG(fa, "full attention: null operator");
    if (!fa->ready) B2_FAIL(B200ATTN_ERR_NOT_READY, "FullAttention weights not set");
    if (pool) B2_CHECK_ARG(layer >= 0 && layer < pool->cfg.num_layers, "full attention: layer %d out of range", layer);
    return 0;
}

static int fa_project_in(b200attn_fa fa, const void* d_x, bool x_is_fp16, int rows, bool kv_int8, DecodeOut* fused, int* d_error,
                         cudaStream_t s) {
    if (fa->cfg.proj_precision == B200ATTN_PROJ_FP16) {
        if (fused)   // decode step of a stack: d_x is the un-normalised residual stream, its RMSNorm scale is applied in the epilogue
            return gemm_tc_store(s, (const __half*)d_x, fa->d_wqkv_fp16, fa->d_qkv_raw, rows, kFaQkvCols, kHidden, kFaQkvCols, fused->rowsq,
                                 fused->eps, d_error);
        const void* xb = d_x;
        const bool compensate = kv_int8 && !x_is_fp16;      // fp32 activations at hand and a quantising cache behind K / V
        if (!x_is_fp16) {
            if (compensate) B2_TRY(f32_split_f16(s, (const float*)d_x, fa->d_xb, fa->d_xlo, (size_t)rows * kHidden));
            else B2_TRY(f32_to_f16(s, (const float*)d_x, fa->d_xb, (size_t)rows * kHidden));
            xb = fa->d_xb;
        }
        B2_TRY(gemm_xwT(s, xb, true, fa->d_wqkv_fp16, true, fa->d_qkv_raw, false, rows, kFaQkvCols, kHidden));
        if (compensate) {
            // K | V columns += (x_lo W_hi^T + x_hi W_lo^T) / kLoScale
            const int q_cols = kFaHeads * kHeadDim * 2, kv_cols = 2 * kFaKvHeads * kHeadDim;
            const __half* w_kv_hi = fa->d_wqkv_fp16 + (size_t)q_cols * kHidden;
            B2_TRY(gemm_xwT(s, fa->d_xlo, true, w_kv_hi, true, fa->d_qkv_raw + q_cols, false, rows, kv_cols, kHidden, 1.0f, 1.0f / kLoScale, kFaQkvCols));
            B2_TRY(gemm_xwT(s, xb, true, fa->d_wkv_lo, true, fa->d_qkv_raw + q_cols, false, rows, kv_cols, kHidden, 1.0f, 1.0f / kLoScale, kFaQkvCols));
        }
        return 0;
    }
    if (x_is_fp16) B2_FAIL(B200ATTN_ERR_INVALID, "full attention: fp16 activations need the fp16 projection mode");
    return gemm_xwT(s, d_x, false, fa->d_wqkv_f32, false, fa->d_qkv_raw, false, rows, kFaQkvCols, kHidden);
}

static int fa_project_out(b200attn_fa fa, float* d_y, float beta, int rows, DecodeOut* fused, int* d_error, cudaStream_t s) {
    if (fused)   // residual stream += attn W_o^T, with the fp16 copy and the sums of squares for the next projection
        return gemm_tc_residual(s, (const __half*)fa->d_attn, fa->d_wo_fp16, d_y, fused->xh, fused->rowsq, rows, kHidden, kFaHeads * kHeadDim, d_error);
    if (fa->cfg.proj_precision == B200ATTN_PROJ_FP16)
        return gemm_xwT(s, fa->d_attn, true, fa->d_wo_fp16, true, d_y, false, rows, kHidden, kFaHeads * kHeadDim, beta);
    return gemm_xwT(s, fa->d_attn, false, fa->d_wo_f32, false, d_y, false, rows, kHidden, kFaHeads * kHeadDim, beta);
}

// One pass of the layer over a batch of rows.  decode == false: host-described varlen batch (h_slots /
// h_counts), causal prefill through the tensor-core kernel.  decode == true: one row per sequence, slots
// on the device, no host synchronisation or allocation (capture-safe).  d_y = beta * d_y + attn W_o^T.
int fa_forward_rows(b200attn_fa fa, b200attn_kv_pool pool, int layer, const int* h_slots, const int* h_counts,
                    int n_seqs, const int* d_slots_in, bool decode, const void* d_x, bool x_is_fp16, float* d_y,
                    float y_beta, DecodeOut* dout, cudaStream_t s) {
    B2_CHECK_ARG(pool && d_x && d_y, "full attention: null argument");
    B2_TRY(fa_check(fa, pool, layer));
    const KvView kv = pool->view();
    const bool fp16 = fa->cfg.proj_precision == B200ATTN_PROJ_FP16;
    const float* k_in = fa->d_qkv_raw + kFaHeads * kHeadDim * 2;
    const float* v_in = k_in + kFaKvHeads * kHeadDim;
    if (decode) {
        B2_CHECK_ARG(d_slots_in, "fa_decode: null slots");
        B2_CHECK_ARG(n_seqs > 0 && n_seqs <= fa->cfg.max_batch, "fa_decode: n_seqs %d outside (0, max_batch %d]", n_seqs, fa->cfg.max_batch);
        B2_TRY(fa_project_in(fa, d_x, x_is_fp16, n_seqs, !kv.is_fp16, dout, pool->d_error, s));
        // q / gate epilogue, append of the new token's K and V, and the length increment in one launch; the attention
        // kernel then sees the new length already
        B2_TRY(launch_fa_decode_pre(kv, layer, d_slots_in, n_seqs, fa->d_qkv_raw, fa->d_qnorm, fa->d_knorm, fa->d_inv_freq, fa->d_q,
                                    fa->d_gate, s));
        B2_TRY(launch_fa_decode(kv, layer, d_slots_in, n_seqs, fa->d_q, fa->d_gate, kMaxSplitsCap, fa->d_part_o,
                                fa->d_part_ml, fa->d_counters, fa->d_attn, fp16, s));
        B2_TRY(fa_project_out(fa, d_y, y_beta, n_seqs, dout, pool->d_error, s));
        pool->lens_dirty = true;
        return 0;
    }
    std::vector<int> base;
    int rows = 0;
    B2_TRY(pool_prepare_append(pool, layer, h_slots, h_counts, n_seqs, base, &rows));
    if (rows == 0) return 0;
    B2_CHECK_ARG(rows <= fa->cfg.max_prefill_rows, "fa_prefill: %d rows exceed max_prefill_rows %d", rows, fa->cfg.max_prefill_rows);
    std::vector<int> ctx0(n_seqs);
    int ctx_rows = 0;
    for (int i = 0; i < n_seqs; ++i) { ctx0[i] = ctx_rows; ctx_rows += base[i] + h_counts[i]; }
    B2_CHECK_ARG(ctx_rows <= fa->max_rows, "fa_prefill: %d context rows exceed the staging capacity %d", ctx_rows, fa->max_rows);

    std::vector<AppendTile> atiles;
    build_append_tiles(base, h_counts, n_seqs, atiles);
    std::vector<PrefillTile> ptiles;
    build_prefill_tiles(base, h_counts, ctx0, n_seqs, ptiles);
    std::vector<int> row_pos(rows);
    for (int i = 0, r = 0; i < n_seqs; ++i)
        for (int j = 0; j < h_counts[i]; ++j) row_pos[r++] = base[i] + j;
    const int need = 3 * n_seqs + rows + 4 * (int)atiles.size() + 4 * (int)ptiles.size();
    B2_CHECK_ARG(need <= fa->meta_cap, "fa_prefill: metadata (%d ints) exceeds scratch", need);
    int* m = fa->d_meta;
    int* d_slots = m;            m += n_seqs;
    int* d_counts = m;           m += n_seqs;
    int* d_ctx0 = m;             m += n_seqs;
    int* d_row_pos = m;          m += rows;
    AppendTile* d_atiles = reinterpret_cast<AppendTile*>(m);  m += 4 * atiles.size();
    PrefillTile* d_ptiles = reinterpret_cast<PrefillTile*>(m);
    B2_CUDA(cudaMemcpyAsync(d_slots, h_slots, n_seqs * 4, cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaMemcpyAsync(d_counts, h_counts, n_seqs * 4, cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaMemcpyAsync(d_ctx0, ctx0.data(), n_seqs * 4, cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaMemcpyAsync(d_row_pos, row_pos.data(), (size_t)rows * 4, cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaMemcpyAsync(d_atiles, atiles.data(), atiles.size() * sizeof(AppendTile), cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaMemcpyAsync(d_ptiles, ptiles.data(), ptiles.size() * sizeof(PrefillTile), cudaMemcpyHostToDevice, s));

    B2_TRY(fa_project_in(fa, d_x, x_is_fp16, rows, !kv.is_fp16, nullptr, pool->d_error, s));
    B2_TRY(launch_fa_q_epilogue(fa->d_qkv_raw, rows, fa->d_qnorm, fa->d_inv_freq, d_row_pos, fa->d_q, fa->d_gate, s));
    for (int i = 0; i < n_seqs; ++i)
        B2_TRY(launch_kv_stage_gather(kv, layer, h_slots[i], base[i], ctx0[i], fa->d_kstage, fa->d_vstage, s));
    {
        ProfScope prof(PROF_KV_APPEND, s);
        B2_TRY(launch_kv_append(kv, layer, d_atiles, (int)atiles.size(), d_slots, k_in, kFaQkvCols, v_in, kFaQkvCols, true,
                                fa->d_knorm, fa->d_inv_freq, fa->d_kstage, fa->d_vstage, d_ctx0, s));
    }
    {
        ProfScope prof(PROF_FA_PREFILL, s);
        B2_TRY(launch_fa_prefill_tc(fa->d_q, rows, fa->d_kstage, fa->d_vstage, ctx_rows, d_ptiles, (int)ptiles.size(),
                                    fa->d_gate, fa->d_attn, fp16, pool->d_error, s));
    }
    B2_TRY(launch_kv_advance(kv, layer, d_slots, d_counts, n_seqs, s));
    B2_TRY(fa_project_out(fa, d_y, y_beta, rows, nullptr, pool->d_error, s));
    for (int i = 0; i < n_seqs; ++i) pool->h_lens[(size_t)layer * pool->cfg.max_seqs + h_slots[i]] += h_counts[i];
    return 0;
}

}  // namespace b200

extern "C" int b200attn_fa_prefill(b200attn_fa fa, b200attn_kv_pool pool, int layer, const int* h_slots,
                                   const int* h_counts, int n_seqs, const float* d_x, float* d_y, b200attn_stream stream) {
    return fa_forward_rows(fa, pool, layer, h_slots, h_counts, n_seqs, nullptr, false, d_x, false, d_y, 0.f, nullptr, as_stream(stream));
}

extern "C" int b200attn_fa_decode(b200attn_fa fa, b200attn_kv_pool pool, int layer, const int* d_slots, int n_seqs,
                                  const float* d_x, float* d_y, b200attn_stream stream) {
    return fa_forward_rows(fa, pool, layer, nullptr, nullptr, n_seqs, d_slots, true, d_x, false, d_y, 0.f, nullptr, as_stream(stream));
}

extern "C" int b200attn_fa_decode_core(b200attn_fa fa, b200attn_kv_pool pool, int layer, const int* d_slots, int n_seqs,
                                       const float* d_q, float* d_out, b200attn_stream stream) {
    B2_CHECK_ARG(fa && pool && d_slots && d_q && d_out, "fa_decode_core: null argument");
    B2_CHECK_ARG(layer >= 0 && layer < pool->cfg.num_layers, "fa_decode_core: layer out of range");
    B2_CHECK_ARG(n_seqs > 0 && n_seqs <= fa->cfg.max_batch, "fa_decode_core: n_seqs %d outside (0, max_batch %d]", n_seqs, fa->cfg.max_batch);
    cudaStream_t s = as_stream(stream);
    const KvView kv = pool->view();
    B2_TRY(f32_to_f16(s, d_q, fa->d_q, (size_t)n_seqs * kFaHeads * kHeadDim));
    return launch_fa_decode(kv, layer, d_slots, n_seqs, fa->d_q, nullptr, kMaxSplitsCap, fa->d_part_o, fa->d_part_ml, fa->d_counters,
                            d_out, false, s);
}

extern "C" int b200attn_fa_prefill_core(b200attn_fa fa, const int* h_counts, int n_seqs, const float* d_q,
                                        const float* d_k, const float* d_v, float* d_out, int use_tensor_cores,
                                        b200attn_stream stream) {
    B2_CHECK_ARG(fa && h_counts && d_q && d_k && d_v && d_out, "fa_prefill_core: null argument");
    B2_CHECK_ARG(n_seqs > 0, "fa_prefill_core: n_seqs must be > 0");
    int rows = 0;
    std::vector<int> base(n_seqs, 0), ctx0(n_seqs);
    for (int i = 0; i < n_seqs; ++i) { B2_CHECK_ARG(h_counts[i] >= 0, "fa_prefill_core: negative count"); ctx0[i] = rows; rows += h_counts[i]; }
    if (rows == 0) return 0;
    B2_CHECK_ARG(rows <= fa->max_rows, "fa_prefill_core: %d rows exceed scratch capacity %d", rows, fa->max_rows);
    cudaStream_t s = as_stream(stream);
    B2_TRY(f32_to_f16(s, d_q, fa->d_q, (size_t)rows * kFaHeads * kHeadDim));
    B2_TRY(f32_to_f16(s, d_k, fa->d_kstage, (size_t)rows * kFaKvHeads * kHeadDim));
    B2_TRY(f32_to_f16(s, d_v, fa->d_vstage, (size_t)rows * kFaKvHeads * kHeadDim));
    if (use_tensor_cores) {
        std::vector<PrefillTile> ptiles;
        build_prefill_tiles(base, h_counts, ctx0, n_seqs, ptiles);
        B2_CHECK_ARG((int)ptiles.size() * 4 + 1 <= fa->meta_cap, "fa_prefill_core: metadata exceeds scratch");
        PrefillTile* d_ptiles = reinterpret_cast<PrefillTile*>(fa->d_meta + 4);
        int* d_err = fa->d_meta;
        B2_CUDA(cudaMemsetAsync(d_err, 0, 4, s));
        B2_CUDA(cudaMemcpyAsync(d_ptiles, ptiles.data(), ptiles.size() * sizeof(PrefillTile), cudaMemcpyHostToDevice, s));
        B2_TRY(launch_fa_prefill_tc(fa->d_q, rows, fa->d_kstage, fa->d_vstage, rows, d_ptiles, (int)ptiles.size(), nullptr,
                                    d_out, false, d_err, s));
        int err = 0;
        B2_CUDA(cudaMemcpyAsync(&err, d_err, 4, cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaStreamSynchronize(s));
        if (err != 0) B2_FAIL(B200ATTN_ERR_DEVICE, "fa_prefill_core: kernel reported device status %d (bounded wait ran out)", err);
        return 0;
    }
    std::vector<int> row_pos(rows), row_ctx0(rows);
    for (int i = 0, r = 0; i < n_seqs; ++i)
        for (int j = 0; j < h_counts[i]; ++j, ++r) { row_pos[r] = j; row_ctx0[r] = ctx0[i]; }
    B2_CHECK_ARG(2 * rows <= fa->meta_cap, "fa_prefill_core: metadata exceeds scratch");
    B2_CUDA(cudaMemcpyAsync(fa->d_meta, row_pos.data(), (size_t)rows * 4, cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaMemcpyAsync(fa->d_meta + rows, row_ctx0.data(), (size_t)rows * 4, cudaMemcpyHostToDevice, s));
    return launch_fa_prefill_simt(fa->d_q, fa->d_kstage, fa->d_vstage, fa->d_meta, fa->d_meta + rows, rows, nullptr, d_out,
                                  false, s);
}
