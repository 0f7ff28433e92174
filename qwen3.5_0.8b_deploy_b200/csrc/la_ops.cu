// Gated DeltaNet operator and state pool: weights, scratch, and the prefill / decode sequencing of
// fused input projection -> conv/norm/gates -> delta-rule recurrence -> gated RMSNorm -> output projection.
// Mirrors qwen::cuda::CudaLinearAttention / CudaLinearAttentionV2 / CudaLinearAttnState
// (src/backend/cuda/kernels/linear_attention_cuda.cu:266-326,412-684, linear_attention_v2.cu:734-883 in
// the reference).
#include "kernels.cuh"

#include <algorithm>
#include <new>
#include <vector>

namespace b200 {

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t la_scratch_bytes(const b200attn_la_config& c) {
    const size_t R = (size_t)std::max(c.max_batch, c.max_prefill_rows);
    size_t n = 0;
    n += align_up(R * kLaProjCols * 4, 256);            // mixed
    n += 3 * align_up(R * kLaHeads * kLaKd * 4, 256);   // q, k, v
    n += 3 * align_up(R * kLaHeads * kLaKd * 2, 256);   // q, k, v as fp16
    n += 2 * align_up(R * kLaHeads * 4, 256);           // g, beta
    n += align_up(R * kLaHeads * kLaVd * 4, 256);       // core
    n += align_up(R * kHidden * 2, 256);                // xb
    n += align_up(R * kLaHeads * kLaVd * 4, 256);       // gated
    n += align_up((2 * R + 65536) * 4, 256);            // meta
    return n;
}

void la_carve_scratch(b200attn_la la) {
    const b200attn_la_config& c = la->cfg;
    const size_t R = (size_t)std::max(c.max_batch, c.max_prefill_rows);
    char* p = la->scratch.base;
    auto take = [&](size_t bytes) { char* r = p; p += align_up(bytes, 256); return r; };
    la->max_rows = (int)R;
    la->d_mixed = (float*)take(R * kLaProjCols * 4);
    la->d_q = (float*)take(R * kLaHeads * kLaKd * 4);
    la->d_k = (float*)take(R * kLaHeads * kLaKd * 4);
    la->d_v = (float*)take(R * kLaHeads * kLaKd * 4);
    la->d_qh = (__half*)take(R * kLaHeads * kLaKd * 2);
    la->d_kh = (__half*)take(R * kLaHeads * kLaKd * 2);
    la->d_vh = (__half*)take(R * kLaHeads * kLaVd * 2);
    la->d_g = (float*)take(R * kLaHeads * 4);
    la->d_beta = (float*)take(R * kLaHeads * 4);
    la->d_core = (float*)take(R * kLaHeads * kLaVd * 4);
    la->d_xb = (__half*)take(R * kHidden * 2);
    la->d_gated = take(R * kLaHeads * kLaVd * 4);
    la->meta_cap = (int)(2 * R + 65536);
    la->d_meta = (int*)take((size_t)la->meta_cap * 4);
}

int la_create_internal(const b200attn_la_config* cfg, const Scratch* shared, b200attn_la* out) {
    B2_CHECK_ARG(cfg && out, "la_create: null argument");
    B2_CHECK_ARG(cfg->hidden_size > 0 && cfg->num_heads > 0 && cfg->key_dim > 0 && cfg->value_dim > 0,
                 "All dimensions must be > 0");
    if (cfg->hidden_size != kHidden || cfg->num_heads != kLaHeads || cfg->key_dim != kLaKd || cfg->value_dim != kLaVd ||
        cfg->conv_kernel != kLaConvK)
        B2_FAIL(B200ATTN_ERR_UNSUPPORTED, "la_create: kernels are built for hidden=1024, heads=16, key_dim=value_dim=128, conv_kernel=4");
    B2_CHECK_ARG(cfg->max_batch > 0 && cfg->max_prefill_rows >= 0, "la_create: max_batch must be > 0");
    B2_CHECK_ARG(cfg->proj_precision == B200ATTN_PROJ_FP32 || cfg->proj_precision == B200ATTN_PROJ_FP16, "la_create: bad proj_precision");
    refresh_runtime_flags();
    auto* la = new (std::nothrow) b200attn_la_s();
    if (!la) B2_FAIL(B200ATTN_ERR_NOMEM, "la_create: host allocation failed");
    la->cfg = *cfg;
    const size_t need = la_scratch_bytes(*cfg);
    if (shared) {
        if (shared->bytes < need) { delete la; B2_FAIL(B200ATTN_ERR_INVALID, "la_create: shared scratch too small"); }
        la->scratch = *shared;
        la->scratch.owned = false;
    } else {
        cudaError_t e = cudaMalloc(&la->scratch.base, need);
        if (e != cudaSuccess) { delete la; B2_FAIL(B200ATTN_ERR_NOMEM, "la_create: scratch cudaMalloc(%zu) failed: %s", need, cudaGetErrorString(e)); }
        la->scratch.bytes = need;
        la->scratch.owned = true;
    }
    la_carve_scratch(la);
    // The status word is an allocation of its own: operators of one stack overlay their working buffers on one scratch
    // area, and a word inside it would be overwritten by another operator's data.
    if (cudaMalloc(&la->d_error, 256) != cudaSuccess || cudaMemset(la->d_error, 0, 256) != cudaSuccess) {
        b200attn_la_destroy(la);
        B2_FAIL(B200ATTN_ERR_CUDA, "la_create: clearing the status word failed");
    }
    int st = cublas_init();
    if (st != 0) { b200attn_la_destroy(la); return st; }
    *out = la;
    return 0;
}

}  // namespace b200

using namespace b200;

extern "C" int b200attn_la_create(const b200attn_la_config* cfg, b200attn_la* out) {
    return la_create_internal(cfg, nullptr, out);
}

extern "C" int b200attn_la_destroy(b200attn_la la) {
    if (!la) return 0;
    cudaFree(la->d_win_f32); cudaFree(la->d_win_fp16); cudaFree(la->d_wout_f32); cudaFree(la->d_wout_fp16);
    cudaFree(la->d_conv_w); cudaFree(la->d_a_log); cudaFree(la->d_dt_bias); cudaFree(la->d_norm);
    if (la->scratch.owned) cudaFree(la->scratch.base);
    cudaFree(la->d_error);
    delete la;
    return 0;
}

extern "C" int b200attn_la_set_weights(b200attn_la la, const b200attn_la_weights* w) {
    B2_CHECK_ARG(la && w, "la_set_weights: null argument");
    B2_CHECK_ARG(w->in_proj_qkv && w->in_proj_a && w->in_proj_b && w->in_proj_z && w->conv1d && w->a_log && w->dt_bias &&
                     w->norm && w->out_proj, "la_set_weights: null weight pointer");
    // One fused input projection: rows [qkv (6144) | z (2048) | a (16) | b (16)].
    std::vector<float> cat((size_t)kLaProjCols * kHidden);
    std::memcpy(cat.data(), w->in_proj_qkv, (size_t)kLaConvDim * kHidden * 4);
    std::memcpy(cat.data() + (size_t)kLaZOff * kHidden, w->in_proj_z, (size_t)kLaHeads * kLaVd * kHidden * 4);
    std::memcpy(cat.data() + (size_t)kLaAOff * kHidden, w->in_proj_a, (size_t)kLaHeads * kHidden * 4);
    std::memcpy(cat.data() + (size_t)kLaBOff * kHidden, w->in_proj_b, (size_t)kLaHeads * kHidden * 4);
    cudaFree(la->d_win_f32); cudaFree(la->d_win_fp16); cudaFree(la->d_wout_f32); cudaFree(la->d_wout_fp16);
    cudaFree(la->d_conv_w); cudaFree(la->d_a_log); cudaFree(la->d_dt_bias); cudaFree(la->d_norm);
    la->d_win_f32 = nullptr; la->d_win_fp16 = nullptr; la->d_wout_f32 = nullptr; la->d_wout_fp16 = nullptr;
    la->d_conv_w = nullptr; la->d_a_log = nullptr; la->d_dt_bias = nullptr; la->d_norm = nullptr;
    la->ready = false;
    const size_t no = (size_t)kHidden * kLaHeads * kLaVd;
    if (la->cfg.proj_precision == B200ATTN_PROJ_FP16) {
        B2_TRY(upload_f16_from_f32(cat.data(), &la->d_win_fp16, cat.size()));
        B2_TRY(upload_f16_from_f32(w->out_proj, &la->d_wout_fp16, no));
    } else {
        B2_TRY(upload_f32(cat.data(), &la->d_win_f32, cat.size()));
        B2_TRY(upload_f32(w->out_proj, &la->d_wout_f32, no));
    }
    B2_TRY(upload_f32(w->conv1d, &la->d_conv_w, (size_t)kLaConvDim * kLaConvK));
    B2_TRY(upload_f32(w->a_log, &la->d_a_log, kLaHeads));
    B2_TRY(upload_f32(w->dt_bias, &la->d_dt_bias, kLaHeads));
    B2_TRY(upload_f32(w->norm, &la->d_norm, kLaVd));
    la->ready = true;
    return 0;
}

extern "C" int b200attn_la_device_status(b200attn_la la, int* code_out) {
    B2_CHECK_ARG(la && code_out, "la_device_status: null argument");
    B2_CUDA(cudaDeviceSynchronize());
    B2_CUDA(cudaMemcpy(code_out, la->d_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (*code_out != 0) B2_CUDA(cudaMemset(la->d_error, 0, sizeof(int)));
    return 0;
}

// ---- state pool -------------------------------------------------------------------------------------------
extern "C" int b200attn_la_state_create(const b200attn_la_state_config* cfg, b200attn_la_state* out) {
    B2_CHECK_ARG(cfg && out, "la_state_create: null argument");
    B2_CHECK_ARG(cfg->num_layers > 0 && cfg->max_seqs > 0, "la_state_create: sizes must be > 0");
    if (cfg->num_heads != kLaHeads || cfg->key_dim != kLaKd || cfg->value_dim != kLaVd || cfg->conv_kernel != kLaConvK)
        B2_FAIL(B200ATTN_ERR_UNSUPPORTED, "la_state_create: kernels are built for heads=16, key_dim=value_dim=128, conv_kernel=4");
    auto* st = new (std::nothrow) b200attn_la_state_s();
    if (!st) B2_FAIL(B200ATTN_ERR_NOMEM, "la_state_create: host allocation failed");
    st->cfg = *cfg;
    const size_t nrec = (size_t)cfg->num_layers * cfg->max_seqs * st->rec_stride_slot();
    const size_t nconv = (size_t)cfg->num_layers * cfg->max_seqs * st->conv_stride_slot();
    cudaError_t e = cudaMalloc(&st->d_recurrent, nrec * 4);
    if (e == cudaSuccess) e = cudaMalloc(&st->d_conv, nconv * 4);
    if (e == cudaSuccess) e = cudaMemset(st->d_recurrent, 0, nrec * 4);
    if (e == cudaSuccess) e = cudaMemset(st->d_conv, 0, nconv * 4);
    if (e != cudaSuccess) {
        set_error("la_state_create: %s", cudaGetErrorString(e));
        b200attn_la_state_destroy(st);
        return e == cudaErrorMemoryAllocation ? B200ATTN_ERR_NOMEM : B200ATTN_ERR_CUDA;
    }
    *out = st;
    return 0;
}

extern "C" int b200attn_la_state_destroy(b200attn_la_state st) {
    if (!st) return 0;
    cudaFree(st->d_recurrent); cudaFree(st->d_conv);
    delete st;
    return 0;
}

extern "C" int b200attn_la_state_clear(b200attn_la_state st, int slot, b200attn_stream stream) {
    B2_CHECK_ARG(st, "la_state_clear: null state");
    B2_CHECK_ARG(slot < st->cfg.max_seqs, "la_state_clear: slot out of range");
    cudaStream_t s = as_stream(stream);
    if (slot < 0) {
        B2_CUDA(cudaMemsetAsync(st->d_recurrent, 0, (size_t)st->cfg.num_layers * st->cfg.max_seqs * st->rec_stride_slot() * 4, s));
        B2_CUDA(cudaMemsetAsync(st->d_conv, 0, (size_t)st->cfg.num_layers * st->cfg.max_seqs * st->conv_stride_slot() * 4, s));
        return 0;
    }
    for (int l = 0; l < st->cfg.num_layers; ++l) {
        const size_t idx = (size_t)l * st->cfg.max_seqs + slot;
        B2_CUDA(cudaMemsetAsync(st->d_recurrent + idx * st->rec_stride_slot(), 0, st->rec_stride_slot() * 4, s));
        B2_CUDA(cudaMemsetAsync(st->d_conv + idx * st->conv_stride_slot(), 0, st->conv_stride_slot() * 4, s));
    }
    return 0;
}

static int la_state_index(b200attn_la_state st, int layer, int slot, size_t* idx) {
    B2_CHECK_ARG(st, "la_state: null state");
    B2_CHECK_ARG(layer >= 0 && layer < st->cfg.num_layers, "la_state: layer %d out of range", layer);
    B2_CHECK_ARG(slot >= 0 && slot < st->cfg.max_seqs, "la_state: slot %d out of range", slot);
    *idx = (size_t)layer * st->cfg.max_seqs + slot;
    return 0;
}

extern "C" int b200attn_la_state_import(b200attn_la_state st, int layer, int slot, const float* d_recurrent,
                                        const float* d_conv, b200attn_stream stream) {
    size_t idx;
    B2_TRY(la_state_index(st, layer, slot, &idx));
    cudaStream_t s = as_stream(stream);
    if (d_recurrent)
        B2_CUDA(cudaMemcpyAsync(st->d_recurrent + idx * st->rec_stride_slot(), d_recurrent, st->rec_stride_slot() * 4,
                                cudaMemcpyDeviceToDevice, s));
    if (d_conv) B2_TRY(launch_la_conv_import(d_conv, st->d_conv + idx * st->conv_stride_slot(), s));
    return 0;
}

extern "C" int b200attn_la_state_export(b200attn_la_state st, int layer, int slot, float* d_recurrent, float* d_conv,
                                        b200attn_stream stream) {
    size_t idx;
    B2_TRY(la_state_index(st, layer, slot, &idx));
    cudaStream_t s = as_stream(stream);
    if (d_recurrent)
        B2_CUDA(cudaMemcpyAsync(d_recurrent, st->d_recurrent + idx * st->rec_stride_slot(), st->rec_stride_slot() * 4,
                                cudaMemcpyDeviceToDevice, s));
    if (d_conv) B2_TRY(launch_la_conv_export(st->d_conv + idx * st->conv_stride_slot(), d_conv, s));
    return 0;
}

// ---- forward ---------------------------------------------------------------------------------------------------
namespace b200 {

static bool la_use_tensor_cores() { return !g_flags.la_prefill_serial; }

static int la_build_meta(b200attn_la la, b200attn_la_state st, const int* h_slots, const int* h_counts, int n_seqs,
                         int* rows_out, std::vector<LaSeqMeta>& seqs, LaSeqMeta** d_seqs, int** d_row_seq, bool need_row_seq,
                         cudaStream_t s) {
    B2_CHECK_ARG(h_slots && h_counts && n_seqs > 0, "linear attention: bad batch description");
    seqs.resize(n_seqs);
    int rows = 0;
    for (int i = 0; i < n_seqs; ++i) {
        B2_CHECK_ARG(h_slots[i] >= 0 && h_slots[i] < st->cfg.max_seqs, "linear attention: slot %d out of range", h_slots[i]);
        B2_CHECK_ARG(h_counts[i] >= 0, "linear attention: negative count");
        for (int j = 0; j < i; ++j) B2_CHECK_ARG(h_slots[j] != h_slots[i], "linear attention: slot %d listed twice", h_slots[i]);
        seqs[i] = LaSeqMeta{h_slots[i], rows, h_counts[i]};
        rows += h_counts[i];
    }
    *rows_out = rows;
    B2_CHECK_ARG(rows <= la->max_rows, "linear attention: %d rows exceed scratch capacity %d", rows, la->max_rows);
    const int need = 3 * n_seqs + (need_row_seq ? rows : 0);
    B2_CHECK_ARG(need <= la->meta_cap, "linear attention: metadata exceeds scratch");
    *d_seqs = reinterpret_cast<LaSeqMeta*>(la->d_meta);
    *d_row_seq = la->d_meta + 3 * n_seqs;
    B2_CUDA(cudaMemcpyAsync(*d_seqs, seqs.data(), (size_t)n_seqs * sizeof(LaSeqMeta), cudaMemcpyHostToDevice, s));
    if (need_row_seq && rows > 0) {
        std::vector<int> row_seq(rows);
        for (int i = 0, r = 0; i < n_seqs; ++i)
            for (int j = 0; j < h_counts[i]; ++j) row_seq[r++] = i;
        B2_CUDA(cudaMemcpyAsync(*d_row_seq, row_seq.data(), (size_t)rows * 4, cudaMemcpyHostToDevice, s));
    }
    return 0;
}

// Runs the delta-rule recurrence over the batch.  tensor_cores: q, k and v must already be in la->d_qh / d_kh / d_vh.
static int la_recurrence(b200attn_la la, b200attn_la_state st, int layer, const float* q, const float* k, const float* v,
                         const float* g, const float* beta, const LaSeqMeta* d_seqs, int n_seqs, int rows, float* out,
                         bool tensor_cores, cudaStream_t s) {
    float* rec_layer = st->d_recurrent + (size_t)layer * st->cfg.max_seqs * st->rec_stride_slot();
    ProfScope prof(PROF_LA_PREFILL, s);
    if (tensor_cores)
        return launch_la_chunk_tc(la->d_qh, la->d_kh, la->d_vh, g, beta, d_seqs, n_seqs, rows, rec_layer, st->rec_stride_slot(), out,
                                  la->d_error, s);
    return launch_la_recurrent_serial(q, k, v, g, beta, d_seqs, n_seqs, rec_layer, st->rec_stride_slot(), out, s);
}

int la_forward_rows(b200attn_la la, b200attn_la_state st, int layer, const int* h_slots, const int* h_counts, int n_seqs,
                    const int* d_slots, bool decode, const void* d_x, bool x_is_fp16, float* d_y, float y_beta,
                    DecodeOut* dout, cudaStream_t s) {
    B2_CHECK_ARG(la && st && d_x && d_y, "linear attention: null argument");
    if (!la->ready) B2_FAIL(B200ATTN_ERR_NOT_READY, "LinearAttention weights not set");
    B2_CHECK_ARG(layer >= 0 && layer < st->cfg.num_layers, "linear attention: layer %d out of range", layer);
    const bool fp16 = la->cfg.proj_precision == B200ATTN_PROJ_FP16;
    if (x_is_fp16 && !fp16) B2_FAIL(B200ATTN_ERR_INVALID, "linear attention: fp16 activations need the fp16 projection mode");
    float* rec_layer = st->d_recurrent + (size_t)layer * st->cfg.max_seqs * st->rec_stride_slot();
    float* conv_layer = st->d_conv + (size_t)layer * st->cfg.max_seqs * st->conv_stride_slot();
    auto project_in = [&](int rows) -> int {
        if (fp16) {
            if (decode && dout)   // decode step of a stack: d_x is the un-normalised residual stream, its RMSNorm scale is applied in the epilogue
                return gemm_tc_store(s, (const __half*)d_x, la->d_win_fp16, la->d_mixed, rows, kLaProjCols, kHidden, kLaProjCols, dout->rowsq,
                                     dout->eps, la->d_error);
            const void* xb = d_x;
            if (!x_is_fp16) { B2_TRY(f32_to_f16(s, (const float*)d_x, la->d_xb, (size_t)rows * kHidden)); xb = la->d_xb; }
            return gemm_xwT(s, xb, true, la->d_win_fp16, true, la->d_mixed, false, rows, kLaProjCols, kHidden);
        }
        return gemm_xwT(s, d_x, false, la->d_win_f32, false, la->d_mixed, false, rows, kLaProjCols, kHidden);
    };
    auto project_out = [&](int rows) -> int {
        if (decode && dout)   // residual stream += gated W_out^T, with the fp16 copy and the sums of squares for the next projection
            return gemm_tc_residual(s, (const __half*)la->d_gated, la->d_wout_fp16, d_y, dout->xh, dout->rowsq, rows, kHidden, kLaHeads * kLaVd,
                                    la->d_error);
        if (fp16) return gemm_xwT(s, la->d_gated, true, la->d_wout_fp16, true, d_y, false, rows, kHidden, kLaHeads * kLaVd, y_beta);
        return gemm_xwT(s, la->d_gated, false, la->d_wout_f32, false, d_y, false, rows, kHidden, kLaHeads * kLaVd, y_beta);
    };
    if (decode) {
        B2_CHECK_ARG(d_slots, "la_decode: null slots");
        B2_CHECK_ARG(n_seqs > 0 && n_seqs <= la->cfg.max_batch, "la_decode: n_seqs %d outside (0, max_batch %d]", n_seqs, la->cfg.max_batch);
        B2_TRY(project_in(n_seqs));
        B2_TRY(launch_la_decode(la->d_mixed, d_slots, n_seqs, st->cfg.max_seqs, rec_layer, st->rec_stride_slot(), conv_layer,
                                st->conv_stride_slot(), la->d_conv_w, la->d_a_log, la->d_dt_bias, la->d_norm, la->d_gated,
                                fp16, true, s));
        return project_out(n_seqs);
    }
    int rows = 0;
    std::vector<LaSeqMeta> seqs;
    LaSeqMeta* d_seqs = nullptr;
    int* d_row_seq = nullptr;
    B2_TRY(la_build_meta(la, st, h_slots, h_counts, n_seqs, &rows, seqs, &d_seqs, &d_row_seq, true, s));
    if (rows == 0) return 0;
    B2_CHECK_ARG(rows <= la->cfg.max_prefill_rows, "la_prefill: %d rows exceed max_prefill_rows %d", rows, la->cfg.max_prefill_rows);
    const bool tc = la_use_tensor_cores();
    B2_TRY(project_in(rows));
    B2_TRY(launch_la_conv_seq(la->d_mixed, d_row_seq, d_seqs, conv_layer, st->conv_stride_slot(), la->d_conv_w, la->d_a_log,
                              la->d_dt_bias, rows, tc ? nullptr : la->d_q, tc ? nullptr : la->d_k, tc ? la->d_qh : nullptr,
                              tc ? la->d_kh : nullptr, tc ? nullptr : la->d_v, tc ? la->d_vh : nullptr, la->d_g, la->d_beta, s));
    B2_TRY(la_recurrence(la, st, layer, la->d_q, la->d_k, la->d_v, la->d_g, la->d_beta, d_seqs, n_seqs, rows, la->d_core, tc, s));
    B2_TRY(launch_la_conv_state_update(la->d_mixed, d_seqs, n_seqs, conv_layer, st->conv_stride_slot(), s));
    B2_TRY(launch_la_gated_norm(la->d_core, la->d_mixed, la->d_norm, rows, la->d_gated, fp16, s));
    return project_out(rows);
}

}  // namespace b200

extern "C" int b200attn_la_prefill(b200attn_la la, b200attn_la_state st, int layer, const int* h_slots, const int* h_counts,
                                   int n_seqs, const float* d_x, float* d_y, b200attn_stream stream) {
    return la_forward_rows(la, st, layer, h_slots, h_counts, n_seqs, nullptr, false, d_x, false, d_y, 0.f, nullptr, as_stream(stream));
}

extern "C" int b200attn_la_decode(b200attn_la la, b200attn_la_state st, int layer, const int* d_slots, int n_seqs,
                                  const float* d_x, float* d_y, b200attn_stream stream) {
    return la_forward_rows(la, st, layer, nullptr, nullptr, n_seqs, d_slots, true, d_x, false, d_y, 0.f, nullptr, as_stream(stream));
}

extern "C" int b200attn_la_prefill_core(b200attn_la la, b200attn_la_state st, int layer, const int* h_slots,
                                        const int* h_counts, int n_seqs, const float* d_q, const float* d_k,
                                        const float* d_v, const float* d_g, const float* d_beta, float* d_out,
                                        int use_tensor_cores, b200attn_stream stream) {
    B2_CHECK_ARG(la && st && d_q && d_k && d_v && d_g && d_beta && d_out, "la_prefill_core: null argument");
    B2_CHECK_ARG(layer >= 0 && layer < st->cfg.num_layers, "la_prefill_core: layer %d out of range", layer);
    cudaStream_t s = as_stream(stream);
    int rows = 0;
    std::vector<LaSeqMeta> seqs;
    LaSeqMeta* d_seqs = nullptr;
    int* d_row_seq = nullptr;
    B2_TRY(la_build_meta(la, st, h_slots, h_counts, n_seqs, &rows, seqs, &d_seqs, &d_row_seq, false, s));
    if (rows == 0) return 0;
    if (use_tensor_cores) {
        B2_TRY(f32_to_f16(s, d_q, la->d_qh, (size_t)rows * kLaHeads * kLaKd));
        B2_TRY(f32_to_f16(s, d_k, la->d_kh, (size_t)rows * kLaHeads * kLaKd));
        B2_TRY(f32_to_f16(s, d_v, la->d_vh, (size_t)rows * kLaHeads * kLaVd));
        B2_CUDA(cudaMemsetAsync(la->d_error, 0, 4, s));
    }
    B2_TRY(la_recurrence(la, st, layer, d_q, d_k, d_v, d_g, d_beta, d_seqs, n_seqs, rows, d_out, use_tensor_cores != 0, s));
    if (use_tensor_cores) {
        int err = 0;
        B2_CUDA(cudaMemcpyAsync(&err, la->d_error, 4, cudaMemcpyDeviceToHost, s));
        B2_CUDA(cudaStreamSynchronize(s));
        if (err != 0) B2_FAIL(B200ATTN_ERR_DEVICE, "la_prefill_core: kernel reported device status %d (bounded wait ran out)", err);
    }
    return 0;
}

extern "C" int b200attn_la_decode_core(b200attn_la la, b200attn_la_state st, int layer, const int* d_slots, int n_seqs,
                                       const float* d_mixed, float* d_out, b200attn_stream stream) {
    B2_CHECK_ARG(la && st && d_slots && d_mixed && d_out, "la_decode_core: null argument");
    if (!la->ready) B2_FAIL(B200ATTN_ERR_NOT_READY, "LinearAttention weights not set");
    B2_CHECK_ARG(layer >= 0 && layer < st->cfg.num_layers, "la_decode_core: layer %d out of range", layer);
    B2_CHECK_ARG(n_seqs > 0, "la_decode_core: n_seqs must be > 0");
    cudaStream_t s = as_stream(stream);
    float* rec_layer = st->d_recurrent + (size_t)layer * st->cfg.max_seqs * st->rec_stride_slot();
    float* conv_layer = st->d_conv + (size_t)layer * st->cfg.max_seqs * st->conv_stride_slot();
    return launch_la_decode(d_mixed, d_slots, n_seqs, st->cfg.max_seqs, rec_layer, st->rec_stride_slot(), conv_layer,
                            st->conv_stride_slot(), la->d_conv_w, la->d_a_log, la->d_dt_bias, la->d_norm, d_out, false,
                            false, s);
}
