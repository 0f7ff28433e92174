// Shared internals of libb200attn: status plumbing, handle structs, launch counter.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cublas_v2.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "../../include/b200attn.h"

namespace b200 {

// ---- model constants the kernels are compiled for -------------------------------------------------
constexpr int kHidden = 1024;
constexpr int kFaHeads = 8, kFaKvHeads = 2, kHeadDim = 256, kRotaryDim = 64;
constexpr int kFaQkvCols = kFaHeads * kHeadDim * 2 + 2 * kFaKvHeads * kHeadDim;  // 5120
constexpr int kPageTokens = 64;
constexpr int kLaHeads = 16, kLaKd = 128, kLaVd = 128, kLaConvK = 4;
constexpr int kLaConvDim = kLaHeads * (2 * kLaKd + kLaVd);                       // 6144
constexpr int kLaZOff = kLaConvDim;                                              // 6144
constexpr int kLaAOff = kLaConvDim + kLaHeads * kLaVd;                           // 8192
constexpr int kLaBOff = kLaAOff + kLaHeads;                                      // 8208
constexpr int kLaProjCols = kLaBOff + kLaHeads;                                  // 8224

// ---- error plumbing ------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
extern thread_local long long g_launches;
inline void count_launch(int n = 1) { g_launches += n; }

#define B2_FAIL(code, ...)            \
    do {                              \
        ::b200::set_error(__VA_ARGS__); \
        return (code);                \
    } while (0)

#define B2_CHECK_ARG(cond, ...)                                   \
    do {                                                          \
        if (!(cond)) B2_FAIL(B200ATTN_ERR_INVALID, __VA_ARGS__);  \
    } while (0)

#define B2_CUDA(expr)                                                                          \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess)                                                                 \
            B2_FAIL(_e == cudaErrorMemoryAllocation ? B200ATTN_ERR_NOMEM : B200ATTN_ERR_CUDA,  \
                    "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
    } while (0)

#define B2_LAUNCH_CHECK()                                                                      \
    do {                                                                                       \
        ::b200::count_launch();                                                                \
        cudaError_t _e = cudaGetLastError();                                                   \
        if (_e != cudaSuccess)                                                                 \
            B2_FAIL(B200ATTN_ERR_CUDA, "kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), \
                    __FILE__, __LINE__);                                                       \
    } while (0)

#define B2_TRY(expr)             \
    do {                         \
        int _s = (expr);         \
        if (_s != 0) return _s;  \
    } while (0)

// ---- per-kernel event timing (gemm.cu) ------------------------------------------------------------------
enum ProfKind { PROF_FA_PREFILL = 0, PROF_FA_DECODE, PROF_LA_PREFILL, PROF_LA_DECODE, PROF_KV_APPEND, PROF_COUNT };
extern bool g_prof_on;
void prof_begin(ProfKind k, cudaStream_t s);
void prof_end(ProfKind k, cudaStream_t s);
struct ProfScope {   // brackets the launches issued during its lifetime when profiling is enabled
    ProfKind k; cudaStream_t s;
    ProfScope(ProfKind kind, cudaStream_t st) : k(kind), s(st) { if (g_prof_on) prof_begin(k, s); }
    ~ProfScope() { if (g_prof_on) prof_end(k, s); }
};

// Launch with the programmatic-stream-serialization attribute: the kernel may become resident while the previous
// kernel of the stream drains; it must call pdl_wait() before touching anything that kernel produced or still reads.
// B200ATTN_PDL=0 turns the attribute off (ordinary stream order).
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline cudaStream_t as_stream(b200attn_stream s) { return reinterpret_cast<cudaStream_t>(s); }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- GEMM (cuBLAS) --------------------------------------------------------------------------------
// Y[rows, out] = X[rows, in] * W[out, in]^T, row-major.  x_bf16/w_bf16/y_bf16 select the storage
// types; accumulation is fp32.  fp32 inputs use full fp32 math (no TF32).
int gemm_xwT(cudaStream_t stream, const void* X, bool x_bf16, const void* W, bool w_bf16, void* Y,
             bool y_bf16, int rows, int out, int in, float beta = 0.f);
int cublas_init();   // creates the per-process handle and its capture-safe workspace
constexpr int kGemmLanes = 4;
int cublas_init_lanes(int n);      // handles 0..n-1, one per concurrent stream of GEMMs
void gemm_set_lane(int lane);      // handle the calling thread's next gemm_xwT calls use

// ---- small elementwise helpers (elementwise.cu) ----------------------------------------------------
int f32_to_bf16(cudaStream_t s, const float* in, __nv_bfloat16* out, size_t n);
int upload_f32(const float* h, float** d_out, size_t n);                       // cudaMalloc + H2D
int upload_bf16_from_f32(const float* h, __nv_bfloat16** d_out, size_t n);      // cudaMalloc + convert

// ---- paged KV pool ---------------------------------------------------------------------------------
struct KvView {            // what kernels need, passed by value
    void* k;               // [layer][page][kvh][64][256]
    void* v;               // [layer][page][kvh][256][64]
    float* ks;             // [layer][page][kvh][64]
    float* vs;
    const int* block_table;  // [max_seqs][max_pages_per_seq]
    int* lens;               // [layers][max_seqs]
    const int* capacity;     // [max_seqs] tokens reserved
    int* error;              // device error word
    int num_pages, max_seqs, max_pages_per_seq, is_fp16;
};

}  // namespace b200

struct b200attn_kv_pool_s {
    b200attn_kv_config cfg{};
    int elem_bytes = 1;
    void* d_k = nullptr;
    void* d_v = nullptr;
    float* d_ks = nullptr;
    float* d_vs = nullptr;
    int* d_block_table = nullptr;
    int* d_lens = nullptr;
    int* d_capacity = nullptr;
    int* d_error = nullptr;
    int* d_meta = nullptr;          // scratch for slots / cu_rows of append & export calls
    int meta_cap = 0;
    std::vector<int> h_lens;        // [layers][max_seqs] mirror
    bool lens_dirty = false;        // device lengths advanced without the host (decode / graph replay)
    std::vector<std::vector<int>> seq_pages;
    std::vector<char> slot_used;
    std::vector<int> free_pages;
    std::vector<int> h_block_table;
    std::vector<int> h_capacity;
    b200::KvView view() const;
    int sync_lens();                // refresh h_lens from the device when dirty
    size_t layer_stride_elems() const {
        return (size_t)cfg.num_pages * cfg.num_kv_heads * b200::kPageTokens * cfg.head_dim;
    }
};

namespace b200 {

// ---- scratch shared by the operators of one stack (or owned by a standalone operator) ------------------
struct Scratch {
    size_t bytes = 0;
    char* base = nullptr;
    bool owned = false;
};

}  // namespace b200

struct b200attn_fa_s {
    b200attn_fa_config cfg{};
    bool ready = false;
    float* d_wqkv_f32 = nullptr;           // [5120, 1024]  (fp32 mode)
    __nv_bfloat16* d_wqkv_bf16 = nullptr;  //               (bf16 mode)
    float* d_wo_f32 = nullptr;             // [1024, 2048]
    __nv_bfloat16* d_wo_bf16 = nullptr;
    float* d_qnorm = nullptr;
    float* d_knorm = nullptr;
    float* d_inv_freq = nullptr;           // [rotary_dim/2]
    // scratch (views into `scratch`)
    b200::Scratch scratch;
    int max_rows = 0;
    float* d_qkv_raw = nullptr;            // [max_rows, 5120]
    __half* d_q = nullptr;                 // [max_rows, 8, 256]
    __half* d_gate = nullptr;              // [max_rows, 8, 256]  sigmoid(gate)
    __half* d_kstage = nullptr;            // [max_rows, 2, 256]
    __half* d_vstage = nullptr;
    __nv_bfloat16* d_xb = nullptr;         // [max_rows, 1024]
    void* d_attn = nullptr;                // [max_rows, 2048] fp32 or bf16
    float* d_part_o = nullptr;             // split-KV partials
    float* d_part_ml = nullptr;
    int* d_counters = nullptr;             // split arrival counters [max_batch][kv_heads], zero between launches
    int* d_meta = nullptr;                 // slots / cu_rows / row->seq for prefill
    int meta_cap = 0;
    int max_splits = 0;
};

struct b200attn_la_state_s {
    b200attn_la_state_config cfg{};
    float* d_recurrent = nullptr;   // [layer][slot][16][128][128]
    float* d_conv = nullptr;        // [layer][slot][3][6144]
    size_t rec_stride_slot() const { return (size_t)cfg.num_heads * cfg.key_dim * cfg.value_dim; }
    size_t conv_stride_slot() const {
        return (size_t)(cfg.conv_kernel - 1) * cfg.num_heads * (2 * cfg.key_dim + cfg.value_dim);
    }
};

struct b200attn_la_s {
    b200attn_la_config cfg{};
    bool ready = false;
    float* d_win_f32 = nullptr;            // [8224, 1024] rows: qkv | z | a | b
    __nv_bfloat16* d_win_bf16 = nullptr;
    float* d_wout_f32 = nullptr;           // [1024, 2048]
    __nv_bfloat16* d_wout_bf16 = nullptr;
    float* d_conv_w = nullptr;             // [6144, 4]
    float* d_a_log = nullptr;
    float* d_dt_bias = nullptr;
    float* d_norm = nullptr;
    b200::Scratch scratch;
    int max_rows = 0;
    float* d_mixed = nullptr;              // [max_rows, 8224]
    float* d_q = nullptr;                  // [max_rows, 16, 128]
    float* d_k = nullptr;
    __half* d_qh = nullptr;                // fp16 copies for the tensor-core recurrence
    __half* d_kh = nullptr;
    float* d_v = nullptr;
    int* d_error = nullptr;                // device status word of the tensor-core recurrence
    float* d_g = nullptr;                  // [max_rows, 16]
    float* d_beta = nullptr;
    float* d_core = nullptr;               // [max_rows, 16, 128]
    __nv_bfloat16* d_xb = nullptr;
    void* d_gated = nullptr;               // [max_rows, 2048] fp32 or bf16
    int* d_meta = nullptr;
    int meta_cap = 0;
};
