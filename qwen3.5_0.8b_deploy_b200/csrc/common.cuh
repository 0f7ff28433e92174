// Shared internals of libb200attn: status plumbing, handle structs, launch counter.
#pragma once

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
enum ProfKind { PROF_FA_PREFILL = 0, PROF_FA_DECODE, PROF_LA_PREFILL, PROF_LA_DECODE, PROF_KV_APPEND, PROF_GEMM_IN, PROF_GEMM_FFN, PROF_GEMM_RES,
                PROF_LM_HEAD, PROF_COUNT };
extern bool g_prof_on;
void prof_begin(ProfKind k, cudaStream_t s);
void prof_end(ProfKind k, cudaStream_t s);
// Device-side stamps for kernels that carry a stamp argument (the decode kernels): while profiling is on, every launch
// gets a two-word slot [first CTA past its dependency wait, last CTA done] in a device buffer; works for eager
// launches and for launches captured into a graph (every replay overwrites its slots).  nullptr when profiling is off.
unsigned long long* prof_stamp_slot(ProfKind k);
struct ProfScope {   // brackets the launches issued during its lifetime when profiling is enabled
    ProfKind k; cudaStream_t s;
    ProfScope(ProfKind kind, cudaStream_t st) : k(kind), s(st) { if (g_prof_on) prof_begin(k, s); }
    ~ProfScope() { if (g_prof_on) prof_end(k, s); }
};

// ---- process-wide switches -------------------------------------------------------------------------------
// Read from the environment by refresh_runtime_flags(), which every *_create entry calls: a process picks its variants
// before it builds its operators, and no launch path touches the environment.
struct RuntimeFlags {
    bool pdl = true;                 // B200ATTN_PDL=0: ordinary stream order instead of programmatic dependent launch
    bool decode_gemm_tc = false;     // B200ATTN_DECODE_GEMM=tc: the fused decode step on the tcgen05 skinny GEMMs (default: library GEMMs + norm / SwiGLU kernels)
    bool lm_head_cublas = false;     // B200ATTN_LM_HEAD=cublas: library GEMM + argmax kernel instead of the fused epilogue
    bool la_prefill_serial = false;  // B200ATTN_LA_PREFILL=serial: token-serial fp32 recurrence instead of the chunked tensor-core kernels
    unsigned la_stagger_ns = 2750;   // B200ATTN_LA_DECODE_STAGGER_NS
    unsigned la_l2_ahead = 185;      // B200ATTN_LA_DECODE_L2_AHEAD
};
extern RuntimeFlags g_flags;
void refresh_runtime_flags();

// ---- per-device facts and one-time set-up -------------------------------------------------------------------
constexpr int kMaxDevices = 64;
int device_sm_count(int* out);          // multiprocessor count of the current device (cached per device)
// Runs `fn` (returning 0 or a status) once per device for the call site that owns `done`: kernel attributes such as the
// opt-in shared-memory size belong to the device's context, so a second GPU in the same process needs its own call.
struct PerDeviceOnce { bool done[kMaxDevices] = {}; };
int per_device_once_begin(PerDeviceOnce& o, int* dev_out, bool* need_out);
void per_device_once_end(PerDeviceOnce& o, int dev);
#define B2_PER_DEVICE_ONCE(once, ...)                                   \
    do {                                                                \
        int _dev = 0; bool _need = false;                               \
        B2_TRY(::b200::per_device_once_begin(once, &_dev, &_need));     \
        if (_need) { __VA_ARGS__; ::b200::per_device_once_end(once, _dev); } \
    } while (0)

// Launch with the programmatic-stream-serialization attribute: the kernel may become resident while the previous
// kernel of the stream drains; it must call pdl_wait() before touching anything that kernel produced or still reads.
// `on` = false (or B200ATTN_PDL=0) gives the ordinary stream order.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_if(bool on, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (on && g_flags.pdl) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    return launch_pdl_if(true, kernel, grid, block, smem, s, static_cast<Args&&>(args)...);
}

inline cudaStream_t as_stream(b200attn_stream s) { return reinterpret_cast<cudaStream_t>(s); }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- GEMM (cuBLAS) --------------------------------------------------------------------------------
// Y[rows, out] = X[rows, in] * W[out, in]^T, row-major.  x_fp16/w_fp16/y_fp16 select the storage
// types; accumulation is fp32.  fp32 inputs use full fp32 math (no TF32).
// Y = alpha * X W^T + beta * Y; ld_out > 0 gives the row pitch of Y (elements) when it is a column block of a wider matrix.
int gemm_xwT(cudaStream_t stream, const void* X, bool x_fp16, const void* W, bool w_fp16, void* Y,
             bool y_fp16, int rows, int out, int in, float beta = 0.f, float alpha = 1.f, int ld_out = 0);
int cublas_init();   // creates the current device's handle and its capture-safe workspace (call outside stream capture)

// ---- small elementwise helpers (elementwise.cu) ----------------------------------------------------
int f32_to_f16(cudaStream_t s, const float* in, __half* out, size_t n);
constexpr float kLoScale = 2048.0f;     // low-order fp16 terms are stored times 2^11 to stay clear of fp16 subnormals
int f32_split_f16(cudaStream_t s, const float* in, __half* hi, __half* lo, size_t n);   // hi = fp16(x), lo = fp16((x - hi) * kLoScale)
int upload_f32(const float* h, float** d_out, size_t n);                       // cudaMalloc + H2D
int upload_f16_from_f32(const float* h, __half** d_out, size_t n);      // cudaMalloc + convert

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
    __half* d_wqkv_fp16 = nullptr;  //               (fp16 mode)
    __half* d_wkv_lo = nullptr;     // [1024, 1024] low-order halves of the K | V rows, times kLoScale (fp16 mode)
    float* d_wo_f32 = nullptr;             // [1024, 2048]
    __half* d_wo_fp16 = nullptr;
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
    __half* d_xb = nullptr;         // [max_rows, 1024]
    __half* d_xlo = nullptr;        // [max_rows, 1024] low-order halves of the activations, times kLoScale
    void* d_attn = nullptr;                // [max_rows, 2048] fp32 or fp16
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
    __half* d_win_fp16 = nullptr;
    float* d_wout_f32 = nullptr;           // [1024, 2048]
    __half* d_wout_fp16 = nullptr;
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
    __half* d_vh = nullptr;
    float* d_v = nullptr;
    int* d_error = nullptr;                // device status word of the tensor-core recurrence
    float* d_g = nullptr;                  // [max_rows, 16]
    float* d_beta = nullptr;
    float* d_core = nullptr;               // [max_rows, 16, 128]
    __half* d_xb = nullptr;
    void* d_gated = nullptr;               // [max_rows, 2048] fp32 or fp16
    int* d_meta = nullptr;
    int meta_cap = 0;
};
