// Internal declarations shared between the kernel files and the operator files.
#pragma once

#include "common.cuh"

#include <vector>

namespace b200 {

// ---- paged KV cache (kv_cache.cu) ----------------------------------------------------------------------
struct AppendTile {  // the tokens of one sequence that land in one cache page
    int seq;         // index into slots[]
    int first_row;   // first input row of the tile
    int first_pos;   // cache position of that row
    int ntok;        // 1..64, never crosses a page boundary
};
int launch_kv_append(const KvView& kv, int layer, const AppendTile* d_tiles, int n_tiles, const int* d_slots,
                     const float* kin, int k_stride, const float* vin, int v_stride, bool do_norm_rope,
                     const float* k_norm_w, const float* inv_freq, __half* kstage, __half* vstage,
                     const int* d_stage_row0, cudaStream_t s);
int launch_fa_decode_pre(const KvView& kv, int layer, const int* d_slots, int n_seqs, const float* qkv_raw, const float* q_norm_w,
                         const float* k_norm_w, const float* inv_freq, __half* q_out, __half* gate_out, cudaStream_t s);
int launch_kv_advance(const KvView& kv, int layer, const int* d_slots, const int* d_counts, int n_seqs, cudaStream_t s);
int launch_fa_q_epilogue(const float* qkv_raw, int rows, const float* q_norm_w, const float* inv_freq,
                         const int* d_row_pos, __half* q_out, __half* gate_out, cudaStream_t s);
int launch_kv_stage_gather(const KvView& kv, int layer, int slot, int base, int stage_row0, __half* kstage,
                           __half* vstage, cudaStream_t s);
void build_append_tiles(const std::vector<int>& base, const int* h_counts, int n_seqs, std::vector<AppendTile>& tiles);
int pool_prepare_append(b200attn_kv_pool p, int layer, const int* h_slots, const int* h_counts, int n_seqs,
                        std::vector<int>& base, int* total_rows);
int ensure_meta(int** d_meta, int* cap, int need);

// ---- decode attention (fa_decode.cu) -----------------------------------------------------------------------
constexpr int kFaDecodeParts = 16;      // partial slots per (sequence, kv head) pair the decode kernel may use; sizes part_o / part_ml
int launch_fa_decode(const KvView& kv, int layer, const int* d_slots, int n_seqs, const __half* q,
                     const __half* gate, int max_splits, float* part_o, float* part_ml, int* counters,
                     void* out, bool out_fp16, cudaStream_t s);

// ---- prefill attention (fa_prefill.cu) -----------------------------------------------------------------------
struct PrefillTile {
    int q_row0;    // first global row of the tile (rows of Q / out)
    int q_pos0;    // position of that row inside its sequence's context
    int n_rows;    // valid rows (<= 128)
    int ctx_row0;  // staging row of the sequence's context position 0
};
int launch_fa_prefill_tc(const __half* q, int rows, const __half* kstage, const __half* vstage, int ctx_rows,
                         const PrefillTile* d_tiles, int n_tiles, const __half* gate, void* out, bool out_fp16,
                         int* d_error, cudaStream_t s);
int launch_fa_prefill_simt(const __half* q, const __half* kstage, const __half* vstage, const int* d_row_pos,
                           const int* d_row_ctx0, int rows, const __half* gate, void* out, bool out_fp16, cudaStream_t s);
void build_prefill_tiles(const std::vector<int>& base, const int* counts, const std::vector<int>& ctx0, int n_seqs,
                         std::vector<PrefillTile>& tiles);

// ---- Gated DeltaNet (la_kernels.cu, la_chunk.cu) -----------------------------------------------------------------
struct LaSeqMeta {  // per sequence, device array
    int slot;
    int row0;
    int count;
};
int launch_la_conv_seq(const float* mixed, const int* d_row_seq, const LaSeqMeta* d_seqs, const float* conv_layer,
                       size_t conv_stride, const float* conv_w, const float* a_log, const float* dt_bias, int rows,
                       float* q, float* k, __half* qh, __half* kh, float* v, __half* vh, float* g, float* beta, cudaStream_t s);
int launch_la_chunk_tc(const __half* q_h, const __half* k_h, const __half* v_h, const float* g, const float* beta,
                       const LaSeqMeta* d_seqs, int n_seqs, int rows, float* rec_layer, size_t rec_stride, float* out,
                       int* d_error, cudaStream_t s);
int launch_la_conv_state_update(const float* mixed, const LaSeqMeta* d_seqs, int n_seqs, float* conv_layer,
                                size_t conv_stride, cudaStream_t s);
int launch_la_recurrent_serial(const float* q, const float* k, const float* v, const float* g, const float* beta,
                               const LaSeqMeta* d_seqs, int n_seqs, float* rec_layer, size_t rec_stride, float* out,
                               cudaStream_t s);
int launch_la_gated_norm(const float* core, const float* mixed, const float* norm_w, int rows, void* out, bool out_fp16,
                         cudaStream_t s);
int launch_la_decode(const float* mixed, const int* d_slots, int n_seqs, int max_seqs, float* rec_layer,
                     size_t rec_stride, float* conv_layer, size_t conv_stride, const float* conv_w, const float* a_log,
                     const float* dt_bias, const float* norm_w, void* out, bool out_fp16, bool early_state_loads, cudaStream_t s);
int launch_la_conv_import(const float* ref_conv, float* mine, cudaStream_t s);
int launch_la_conv_export(const float* mine, float* ref_conv, cudaStream_t s);

// ---- tcgen05 skinny GEMMs for the decode step (gemm_tc.cu) ---------------------------------------------------------
constexpr int kRowsqParts = 16;   // partial sums of squares per row of the residual stream, one per 64-column tile of its producer
bool gemm_tc_enabled();
int gemm_tc_store(cudaStream_t s, const __half* X, const __half* W, float* Y, int M, int N, int K, int ld_out, const float* rowsq,
                  float rs_eps, int* d_error);
int gemm_tc_swiglu(cudaStream_t s, const __half* X, const __half* W, __half* act, int M, int N, int K, const float* rowsq, float rs_eps,
                   int* d_error);
int gemm_tc_residual(cudaStream_t s, const __half* X, const __half* W, float* h, __half* xh, float* rowsq, int M, int N, int K,
                     int* d_error);
int gemm_tc_argmax(cudaStream_t s, const __half* X, const __half* W, unsigned long long* d_packed, int* tokens,
                   int M, int N, int K, int* d_error);
void gemm_tc_forget(const void* ptr);
int gemm_tc_map(const void* ptr, int rows, int cols, int box_rows, void* tensor_map_out);   // cached CUtensorMap of a fp16 matrix
// The fused form of a decode step (tcgen05 projections): the operator's input is the UN-normalised residual stream as
// fp16 (`d_x`), whose RMSNorm scale the input projection applies in its epilogue from `rowsq`; the output projection
// adds into the residual stream `d_y` and refreshes `xh` and `rowsq` for the next projection.
struct DecodeOut {
    __half* xh;        // [rows, hidden] fp16 copy of the residual stream (read as d_x, rewritten by the output projection)
    float* rowsq;      // [128][kRowsqParts] partial sums of squares of the residual rows
    float eps;         // RMSNorm epsilon
};

// ---- operator internals shared with the stack ------------------------------------------------------------------------
size_t fa_scratch_bytes(const b200attn_fa_config& c);
int fa_create_internal(const b200attn_fa_config* cfg, const Scratch* shared, b200attn_fa* out);
size_t la_scratch_bytes(const b200attn_la_config& c);
int la_create_internal(const b200attn_la_config* cfg, const Scratch* shared, b200attn_la* out);
// Point the operator's working buffers into its `scratch` (sized by *_scratch_bytes of its cfg).
void fa_carve_scratch(b200attn_fa fa);
void la_carve_scratch(b200attn_la la);
// Operator bodies that take activations in the stack's own formats (see stack.cu).
int fa_forward_rows(b200attn_fa fa, b200attn_kv_pool pool, int layer, const int* h_slots, const int* h_counts,
                    int n_seqs, const int* d_slots, bool decode, const void* d_x, bool x_is_fp16, float* d_y,
                    float y_beta, DecodeOut* dout, cudaStream_t s);
int la_forward_rows(b200attn_la la, b200attn_la_state st, int layer, const int* h_slots, const int* h_counts,
                    int n_seqs, const int* d_slots, bool decode, const void* d_x, bool x_is_fp16, float* d_y,
                    float y_beta, DecodeOut* dout, cudaStream_t s);

}  // namespace b200
