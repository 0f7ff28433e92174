// Library GEMMs (cuBLAS) for the projections around the attention cores, error text, launch counter and
// small conversion helpers.
#include "common.cuh"
#include <cstdlib>

#include <algorithm>
#include <mutex>
#include <utility>
#include <vector>

namespace b200 {

thread_local char g_error[512] = "";
thread_local long long g_launches = 0;
RuntimeFlags g_flags;

static std::mutex g_dev_mu;
static int g_sm_count[kMaxDevices] = {};

void refresh_runtime_flags() {
    auto env = [](const char* name) { const char* e = std::getenv(name); return e ? e : ""; };
    auto env_uint = [&](const char* name, unsigned dflt, unsigned cap) {
        const char* e = std::getenv(name);
        return e ? (unsigned)std::min<long>(cap, std::max<long>(0, std::atol(e))) : dflt;
    };
    RuntimeFlags f;
    f.pdl = env("B200ATTN_PDL")[0] != '0';
    f.decode_gemm_tc = env("B200ATTN_DECODE_GEMM")[0] == 't';
    f.lm_head_cublas = env("B200ATTN_LM_HEAD")[0] == 'c';
    f.la_prefill_serial = env("B200ATTN_LA_PREFILL")[0] == 's';
    f.la_stagger_ns = env_uint("B200ATTN_LA_DECODE_STAGGER_NS", 2750u, 20000u);
    f.la_l2_ahead = env_uint("B200ATTN_LA_DECODE_L2_AHEAD", 185u, 4096u);
    g_flags = f;
}

int device_sm_count(int* out) {
    int dev = 0;
    B2_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) B2_FAIL(B200ATTN_ERR_UNSUPPORTED, "device index %d not supported", dev);
    std::lock_guard<std::mutex> lk(g_dev_mu);
    if (g_sm_count[dev] == 0) B2_CUDA(cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
    *out = g_sm_count[dev];
    return 0;
}

int per_device_once_begin(PerDeviceOnce& o, int* dev_out, bool* need_out) {
    int dev = 0;
    B2_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) B2_FAIL(B200ATTN_ERR_UNSUPPORTED, "device index %d not supported", dev);
    std::lock_guard<std::mutex> lk(g_dev_mu);
    *dev_out = dev;
    *need_out = !o.done[dev];
    return 0;
}
void per_device_once_end(PerDeviceOnce& o, int dev) {
    std::lock_guard<std::mutex> lk(g_dev_mu);
    o.done[dev] = true;
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
struct ProfRec { std::vector<std::pair<cudaEvent_t, cudaEvent_t>> ev; cudaEvent_t open = nullptr; std::vector<int> slots; };
constexpr int kMaxStampSlots = 4096;
unsigned long long* g_stamps = nullptr;     // [kMaxStampSlots][2] on the device
int g_stamp_next = 0;
ProfRec g_prof[PROF_COUNT];
const char* kProfNames[PROF_COUNT] = {"fa_prefill", "fa_decode", "la_prefill", "la_decode", "kv_append", "gemm_in", "gemm_ffn", "gemm_res", "lm_head"};
}  // namespace
unsigned long long* prof_stamp_slot(ProfKind k) {
    if (!g_prof_on || !g_stamps || g_stamp_next >= kMaxStampSlots) return nullptr;
    g_prof[k].slots.push_back(g_stamp_next);
    return g_stamps + 2 * (size_t)g_stamp_next++;
}
static int stamps_arm_all() {
    std::vector<unsigned long long> arm(2 * (size_t)kMaxStampSlots);
    for (int i = 0; i < kMaxStampSlots; ++i) { arm[2 * i] = ~0ull; arm[2 * i + 1] = 0ull; }
    B2_CUDA(cudaMemcpy(g_stamps, arm.data(), arm.size() * sizeof(unsigned long long), cudaMemcpyHostToDevice));
    return 0;
}

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

// One handle per device with a fixed workspace, which keeps cuBLAS from allocating inside stream capture.
static cublasHandle_t g_handle[kMaxDevices] = {};
static void* g_workspace[kMaxDevices] = {};
static constexpr size_t kWorkspaceBytes = 64ull << 20;
static std::mutex g_mu;

static int cublas_for_current_device(cublasHandle_t* out) {
    int dev = 0;
    B2_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) B2_FAIL(B200ATTN_ERR_UNSUPPORTED, "device index %d not supported", dev);
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_handle[dev]) {
        cublasHandle_t h = nullptr;
        cublasStatus_t st = cublasCreate(&h);
        if (st != CUBLAS_STATUS_SUCCESS) B2_FAIL(B200ATTN_ERR_CUDA, "cublasCreate failed with status %d", (int)st);
        void* ws = nullptr;
        if (cudaMalloc(&ws, kWorkspaceBytes) != cudaSuccess) {
            cublasDestroy(h);
            B2_FAIL(B200ATTN_ERR_NOMEM, "cudaMalloc of the cuBLAS workspace failed");
        }
        st = cublasSetWorkspace(h, ws, kWorkspaceBytes);
        if (st != CUBLAS_STATUS_SUCCESS) {
            cublasDestroy(h);
            cudaFree(ws);
            B2_FAIL(B200ATTN_ERR_CUDA, "cublasSetWorkspace failed with status %d", (int)st);
        }
        cublasSetMathMode(h, CUBLAS_DEFAULT_MATH);
        g_handle[dev] = h;
        g_workspace[dev] = ws;
    }
    if (out) *out = g_handle[dev];
    return 0;
}

int cublas_init() { return cublas_for_current_device(nullptr); }

int gemm_xwT(cudaStream_t stream, const void* X, bool x_fp16, const void* W, bool w_fp16, void* Y, bool y_fp16, int rows,
             int out, int in, float beta, float alpha, int ld_out) {
    if (rows <= 0) return 0;
    cublasHandle_t handle = nullptr;
    B2_TRY(cublas_for_current_device(&handle));
    if (x_fp16 != w_fp16) B2_FAIL(B200ATTN_ERR_INVALID, "gemm: activation and weight types must match");
    cublasStatus_t st = cublasSetStream(handle, stream);
    if (st != CUBLAS_STATUS_SUCCESS) B2_FAIL(B200ATTN_ERR_CUDA, "cublasSetStream failed with status %d", (int)st);
    const cudaDataType_t in_t = x_fp16 ? CUDA_R_16F : CUDA_R_32F;
    const cudaDataType_t out_t = y_fp16 ? CUDA_R_16F : CUDA_R_32F;
    // Row-major Y[rows,out] = X[rows,in] W[out,in]^T  ==  column-major Y^T[out,rows] = W^T(op T) X^T.
    st = cublasGemmEx(handle, CUBLAS_OP_T, CUBLAS_OP_N, out, rows, in, &alpha, W, in_t, in, X, in_t, in, &beta, Y, out_t,
                      ld_out > 0 ? ld_out : out, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    if (st != CUBLAS_STATUS_SUCCESS) B2_FAIL(B200ATTN_ERR_CUDA, "cublasGemmEx(%d,%d,%d) failed with status %d", rows, out, in, (int)st);
    count_launch();
    return 0;
}

// x -> hi = fp16(x), lo = fp16((x - hi) * 2^11): hi + lo * 2^-11 carries about 22 significant bits of x.
__global__ void f32_split_f16_kernel(const float* __restrict__ in, __half* __restrict__ hi, __half* __restrict__ lo, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i + 1 < n) {
        const float2 v = *reinterpret_cast<const float2*>(in + i);
        const __half2 h = __floats2half2_rn(v.x, v.y);
        const float2 hf = __half22float2(h);
        *reinterpret_cast<__half2*>(hi + i) = h;
        *reinterpret_cast<__half2*>(lo + i) = __floats2half2_rn((v.x - hf.x) * kLoScale, (v.y - hf.y) * kLoScale);
    } else if (i < n) {
        const __half h = __float2half_rn(in[i]);
        hi[i] = h;
        lo[i] = __float2half_rn((in[i] - __half2float(h)) * kLoScale);
    }
}
int f32_split_f16(cudaStream_t s, const float* in, __half* hi, __half* lo, size_t n) {
    if (n == 0) return 0;
    const size_t threads = (n + 1) / 2;
    f32_split_f16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(in, hi, lo, n);
    B2_LAUNCH_CHECK();
    return 0;
}

__global__ void f32_to_f16_kernel(const float* __restrict__ in, __half* __restrict__ out, size_t n) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = *reinterpret_cast<const float4*>(in + i);
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&a);
        pk.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(out + i) = pk;
    } else {
        for (size_t j = i; j < n; ++j) out[j] = __float2half_rn(in[j]);
    }
}

int f32_to_f16(cudaStream_t s, const float* in, __half* out, size_t n) {
    if (n == 0) return 0;
    const size_t threads = (n + 3) / 4;
    f32_to_f16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(in, out, n);
    B2_LAUNCH_CHECK();
    return 0;
}

int upload_f32(const float* h, float** d_out, size_t n) {
    B2_CUDA(cudaMalloc(d_out, n * sizeof(float)));
    B2_CUDA(cudaMemcpy(*d_out, h, n * sizeof(float), cudaMemcpyHostToDevice));
    return 0;
}

int upload_f16_from_f32(const float* h, __half** d_out, size_t n) {
    float* tmp = nullptr;
    B2_TRY(upload_f32(h, &tmp, n));
    cudaError_t e = cudaMalloc(d_out, n * sizeof(__half));
    if (e != cudaSuccess) { cudaFree(tmp); B2_FAIL(B200ATTN_ERR_NOMEM, "cudaMalloc failed: %s", cudaGetErrorString(e)); }
    int st = f32_to_f16(0, tmp, *d_out, n);
    cudaError_t e2 = cudaDeviceSynchronize();
    cudaFree(tmp);
    if (st != 0) return st;
    if (e2 != cudaSuccess) B2_FAIL(B200ATTN_ERR_CUDA, "fp16 conversion failed: %s", cudaGetErrorString(e2));
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

extern "C" int b200attn_profile_enable(int on) {
    using namespace b200;
    if (on && !g_stamps) {
        B2_CUDA(cudaMalloc(&g_stamps, 2 * (size_t)kMaxStampSlots * sizeof(unsigned long long)));
        B2_TRY(stamps_arm_all());
    }
    g_prof_on = on != 0;
    return 0;
}
extern "C" int b200attn_profile_reset(void) {
    using namespace b200;
    cudaDeviceSynchronize();
    for (auto& r : g_prof) {
        for (auto& p : r.ev) { cudaEventDestroy(p.first); cudaEventDestroy(p.second); }
        r.ev.clear();
        if (r.open) { cudaEventDestroy(r.open); r.open = nullptr; }
        r.slots.clear();
    }
    g_stamp_next = 0;
    if (g_stamps) B2_TRY(stamps_arm_all());
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
    // stamped launches of this class: read the slots, then arm them again for the next replay
    if (!g_prof[k].slots.empty() && g_stamps) {
        std::vector<unsigned long long> all(2 * (size_t)kMaxStampSlots);
        B2_CUDA(cudaMemcpy(all.data(), g_stamps, all.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        for (int sl : g_prof[k].slots) {
            const unsigned long long t0 = all[2 * (size_t)sl], t1 = all[2 * (size_t)sl + 1];
            if (t1 != 0ull && t0 != ~0ull && t1 > t0) { total += (double)(t1 - t0) * 1e-6; ++timed; }
            const unsigned long long arm[2] = {~0ull, 0ull};
            B2_CUDA(cudaMemcpy(g_stamps + 2 * (size_t)sl, arm, sizeof(arm), cudaMemcpyHostToDevice));
        }
    }
    *total_ms_out = total;
    *launches_out = timed;         // pairs that produced a time
    return 0;
}
