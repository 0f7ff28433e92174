// Library GEMMs (cuBLAS) for the projections around the attention cores, error text, launch counter and
// small conversion helpers.
#include "common.cuh"
#include <cstdlib>

#include <mutex>
#include <utility>
#include <vector>

namespace b200 {

thread_local char g_error[512] = "";
thread_local long long g_launches = 0;
bool pdl_enabled() {     // read on every launch so one process can compare both modes
    const char* e = std::getenv("B200ATTN_PDL");
    return !(e && e[0] == '0');
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// ---- per-kernel event timing ------------------------------------------------------------------------------
bool g_prof_on = false;
namespace {
struct ProfRec { std::vector<std::pair<cudaEvent_t, cudaEvent_t>> ev; cudaEvent_t open = nullptr; };
ProfRec g_prof[PROF_COUNT];
const char* kProfNames[PROF_COUNT] = {"fa_prefill", "fa_decode", "la_prefill", "la_decode", "kv_append"};
}  // namespace
void prof_begin(ProfKind k, cudaStream_t s) {
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) return;
    cudaEventRecord(e, s);
    g_prof[k].open = e;
}
void prof_end(ProfKind k, cudaStream_t s) {
    if (!g_prof[k].open) return;
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) return;
    cudaEventRecord(e, s);
    g_prof[k].ev.emplace_back(g_prof[k].open, e);
    g_prof[k].open = nullptr;
}

// One handle per lane, each with its own fixed workspace: GEMMs issued on different lanes may run at the same time
// (the decode step's branches), and two cuBLAS kernels must never share split-K workspace.  Lane 0 serves everything else.
static cublasHandle_t g_handle[kGemmLanes] = {};
static void* g_workspace[kGemmLanes] = {};
static constexpr size_t kWorkspaceBytes = 64ull << 20, kLaneWorkspaceBytes = 16ull << 20;
static std::mutex g_mu;
thread_local int g_gemm_lane = 0;

void gemm_set_lane(int lane) { g_gemm_lane = (lane >= 0 && lane < kGemmLanes) ? lane : 0; }

static int cublas_init_lane(int lane) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_handle[lane]) return 0;
    cublasStatus_t st = cublasCreate(&g_handle[lane]);
    if (st != CUBLAS_STATUS_SUCCESS) {
        g_handle[lane] = nullptr;
        B2_FAIL(B200ATTN_ERR_CUDA, "cublasCreate failed with status %d", (int)st);
    }
    const size_t bytes = lane == 0 ? kWorkspaceBytes : kLaneWorkspaceBytes;
    B2_CUDA(cudaMalloc(&g_workspace[lane], bytes));
    // A fixed workspace keeps cuBLAS from allocating inside stream capture.
    st = cublasSetWorkspace(g_handle[lane], g_workspace[lane], bytes);
    if (st != CUBLAS_STATUS_SUCCESS) B2_FAIL(B200ATTN_ERR_CUDA, "cublasSetWorkspace failed with status %d", (int)st);
    cublasSetMathMode(g_handle[lane], CUBLAS_DEFAULT_MATH);
    return 0;
}

int cublas_init() { return cublas_init_lane(0); }
int cublas_init_lanes(int n) {
    for (int i = 0; i < n && i < kGemmLanes; ++i) B2_TRY(cublas_init_lane(i));
    return 0;
}

int gemm_xwT(cudaStream_t stream, const void* X, bool x_bf16, const void* W, bool w_bf16, void* Y, bool y_bf16, int rows,
             int out, int in, float beta) {
    if (rows <= 0) return 0;
    const int lane = g_gemm_lane;
    B2_TRY(cublas_init_lane(lane));
    cublasHandle_t handle = g_handle[lane];
    if (x_bf16 != w_bf16) B2_FAIL(B200ATTN_ERR_INVALID, "gemm: activation and weight types must match");
    cublasStatus_t st = cublasSetStream(handle, stream);
    if (st != CUBLAS_STATUS_SUCCESS) B2_FAIL(B200ATTN_ERR_CUDA, "cublasSetStream failed with status %d", (int)st);
    const float alpha = 1.0f;
    const cudaDataType_t in_t = x_bf16 ? CUDA_R_16BF : CUDA_R_32F;
    const cudaDataType_t out_t = y_bf16 ? CUDA_R_16BF : CUDA_R_32F;
    // Row-major Y[rows,out] = X[rows,in] W[out,in]^T  ==  column-major Y^T[out,rows] = W^T(op T) X^T.
    st = cublasGemmEx(handle, CUBLAS_OP_T, CUBLAS_OP_N, out, rows, in, &alpha, W, in_t, in, X, in_t, in, &beta, Y, out_t,
                      out, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    if (st != CUBLAS_STATUS_SUCCESS) B2_FAIL(B200ATTN_ERR_CUDA, "cublasGemmEx(%d,%d,%d) failed with status %d", rows, out, in, (int)st);
    count_launch();
    return 0;
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = *reinterpret_cast<const float4*>(in + i);
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&a);
        pk.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(out + i) = pk;
    } else {
        for (size_t j = i; j < n; ++j) out[j] = __float2bfloat16_rn(in[j]);
    }
}

int f32_to_bf16(cudaStream_t s, const float* in, __nv_bfloat16* out, size_t n) {
    if (n == 0) return 0;
    const size_t threads = (n + 3) / 4;
    f32_to_bf16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(in, out, n);
    B2_LAUNCH_CHECK();
    return 0;
}

int upload_f32(const float* h, float** d_out, size_t n) {
    B2_CUDA(cudaMalloc(d_out, n * sizeof(float)));
    B2_CUDA(cudaMemcpy(*d_out, h, n * sizeof(float), cudaMemcpyHostToDevice));
    return 0;
}

int upload_bf16_from_f32(const float* h, __nv_bfloat16** d_out, size_t n) {
    float* tmp = nullptr;
    B2_TRY(upload_f32(h, &tmp, n));
    cudaError_t e = cudaMalloc(d_out, n * sizeof(__nv_bfloat16));
    if (e != cudaSuccess) { cudaFree(tmp); B2_FAIL(B200ATTN_ERR_NOMEM, "cudaMalloc failed: %s", cudaGetErrorString(e)); }
    int st = f32_to_bf16(0, tmp, *d_out, n);
    cudaError_t e2 = cudaDeviceSynchronize();
    cudaFree(tmp);
    if (st != 0) return st;
    if (e2 != cudaSuccess) B2_FAIL(B200ATTN_ERR_CUDA, "bf16 conversion failed: %s", cudaGetErrorString(e2));
    return 0;
}

}  // namespace b200

extern "C" const char* b200attn_last_error(void) { return b200::g_error; }
extern "C" int b200attn_abi_version(void) { return B200ATTN_ABI_VERSION; }
extern "C" long long b200attn_launch_count(int reset) {
    const long long v = b200::g_launches;
    if (reset) b200::g_launches = 0;
    return v;
}

extern "C" int b200attn_profile_enable(int on) { b200::g_prof_on = on != 0; return 0; }
extern "C" int b200attn_profile_reset(void) {
    using namespace b200;
    cudaDeviceSynchronize();
    for (auto& r : g_prof) {
        for (auto& p : r.ev) { cudaEventDestroy(p.first); cudaEventDestroy(p.second); }
        r.ev.clear();
        if (r.open) { cudaEventDestroy(r.open); r.open = nullptr; }
    }
    (void)cudaGetLastError();
    return 0;
}
extern "C" int b200attn_profile_read(const char* name, double* total_ms_out, long long* launches_out) {
    using namespace b200;
    B2_CHECK_ARG(name && total_ms_out && launches_out, "profile_read: null argument");
    int k = -1;
    for (int i = 0; i < PROF_COUNT; ++i) if (std::strcmp(name, kProfNames[i]) == 0) k = i;
    B2_CHECK_ARG(k >= 0, "profile_read: unknown kernel class '%s'", name);
    B2_CUDA(cudaDeviceSynchronize());
    double total = 0.0;
    long long timed = 0;
    for (auto& p : g_prof[k].ev) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, p.first, p.second) == cudaSuccess) { total += ms; ++timed; }
    }
    (void)cudaGetLastError();      // a pair that could not be timed must not surface as the next launch's error
    *total_ms_out = total;
    *launches_out = timed;         // pairs that produced a time
    return 0;
}
