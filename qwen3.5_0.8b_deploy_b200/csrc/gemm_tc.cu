// Skinny GEMM for the decode step on tcgen05: Y[M <= 128, N] = X[M, K] W[N, K]^T with fp16 operands and fp32
// accumulation in TMEM.  At 128 rows the projections are pure weight streaming (every weight byte is used once),
// so the kernel is a TMA -> shared-memory ring -> tcgen05.mma pipeline with one 128 x BN output tile per CTA and
// optional split-K, sized so a launch puts about one CTA on every SM.  Epilogues:
//   kEpiStore   fp32 tile store (also used for split-K partials, which the following norm kernel sums);
//   kEpiSwiglu  the tile holds BN/2 gate columns then the BN/2 matching up columns: act = silu(gate) * up, fp16;
//   kEpiArgmax  running per-row argmax over all tiles (64-bit atomicMax on {ordered value, ~index}).
// Replaces the reference's thread-per-output projection kernels at decode (linear_proj_fp16_kernel,
// src/backend/cuda/kernels/linear_attention_cuda.cu:33-45; fused_q_path_kernel's GEMV loop,
// full_attention_cuda.cu:31-76; output_proj_kernel :161-172) and the 128 sequential LM-head GEMVs plus host
// argmax of the benchmark driver (src/backend/cuda/performance_test.cu:313-319).
#include "kernels.cuh"
#include "tc05.cuh"

#include <map>
#include <string>
#include <mutex>
#include <tuple>

namespace b200 {

enum { kEpiStore = 0, kEpiSwiglu = 1, kEpiArgmax = 2 };

template <int BN>
struct GemmCfg {
    static constexpr uint32_t kABytes = 128 * 128;          // 128 rows x 64 fp16
    static constexpr uint32_t kBBytes = BN * 128;
    static constexpr uint32_t kStage = kABytes + kBBytes;
    static constexpr int kStages = (8 * kStage <= 200 * 1024) ? 8 : (int)(200 * 1024 / kStage);   // ring depth
    static constexpr uint32_t kSmem = kStages * kStage + 256 + 1024;
};

__device__ __forceinline__ unsigned long long pack_argmax(float v, int idx) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);                        // order-preserving map of fp32 to uint32
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)idx);   // ties: smallest index wins
}

// grid (ceil(N / BN), splits), block 192: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2-5 = epilogue.
// Launched as a programmatic dependent: barriers, TMEM and the first ring of WEIGHT tiles (which no kernel of the
// step writes) are set up before the wait on the preceding kernel; activations are loaded and results written after.
// Every CTA walks its k tiles from a different starting tile so that the CTAs of a wave do not all pull the same
// activation tile from the same L2 slice at once.
template <int BN, int EPI>
__global__ void __launch_bounds__(192)
gemm_small_m_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, int M, int N,
                    int k_steps_per_split, int k_steps_total, float* __restrict__ out_f32, int ld_out, size_t split_stride,
                    __half* __restrict__ out_fp16, unsigned long long* __restrict__ argmax_out,
                    int* __restrict__ error_word) {
    using Cfg = GemmCfg<BN>;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = smem_raw + (base - raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kStages * Cfg::kStage);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = base + kStages * Cfg::kStage;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
    const uint32_t acc_done = bar0 + 8u * (2 * kStages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN, split = blockIdx.y;
    const int ks0 = split * k_steps_per_split;
    const int nk = min(k_steps_per_split, k_steps_total - ks0);
    if (nk <= 0 || *reinterpret_cast<volatile int*>(error_word) != 0) { pdl_enter(); return; }

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2 * kStages + 1; ++i) mbar_init(bar0 + 8u * i, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), BN < 32 ? 32 : BN);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) { tma_prefetch_desc(&map_x); tma_prefetch_desc(&map_w); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0 && lane == 0) {
        const int rot = (int)((blockIdx.x * 3u + blockIdx.y * 7u) % (unsigned)nk);
        auto ktile = [&](int ks) { int k = ks + rot; if (k >= nk) k -= nk; return (ks0 + k) * 64; };
        const int pre = min(nk, kStages);
        for (int ks = 0; ks < pre; ++ks) {
            mbar_arrive_expect_tx(full(ks), Cfg::kStage);
            tma_load_2d(base + ks * Cfg::kStage + Cfg::kABytes, &map_w, full(ks), ktile(ks), n0);
        }
        pdl_enter();
        for (int ks = 0; ks < pre; ++ks) tma_load_2d(base + ks * Cfg::kStage, &map_x, full(ks), ktile(ks), 0);
        for (int ks = pre; ks < nk; ++ks) {
            const int st = ks % kStages;
            if (!mbar_wait(empty(st), ((ks / kStages) - 1) & 1, abort_flag)) break;
            const uint32_t dst = base + st * Cfg::kStage;
            mbar_arrive_expect_tx(full(st), Cfg::kStage);
            tma_load_2d(dst, &map_x, full(st), ktile(ks), 0);
            tma_load_2d(dst + Cfg::kABytes, &map_w, full(st), ktile(ks), n0);
        }
    } else {
        pdl_enter();
    }
    if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(kFmtF16, 128, BN, 0, 0);
            bool ok = true;
            for (int ks = 0; ks < nk; ++ks) {
                const int st = ks % kStages;
                if (!mbar_wait(full(st), (ks / kStages) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a = base + st * Cfg::kStage, b = a + Cfg::kABytes;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_f16(tmem, umma_smem_desc(a + kk * 32, 16, 1024), umma_smem_desc(b + kk * 32, 16, 1024), idesc,
                             (ks > 0 || kk > 0) ? 1u : 0u);
                umma_commit(empty(st));
            }
            if (ok) umma_commit(acc_done);
        }
    } else if (warp >= 2) {
        const int q = warp & 3;                       // TMEM lane quadrant this warp may read
        const int m = 32 * q + lane;                  // output row
        if (mbar_wait_warp(acc_done, 0, abort_flag)) {
            tc_fence_after();
            const uint32_t lane_base = (uint32_t)(32 * q) << 16;
            const int n_valid = min(BN, N - n0);
            if constexpr (EPI == kEpiStore) {
#pragma unroll 1
                for (int ch = 0; ch < BN / 32; ++ch) {
                    uint32_t v[32];
                    tmem_ld32(tmem + lane_base + ch * 32, v);
                    tmem_wait_ld();
                    if (m < M) {
                        float* dst = out_f32 + (size_t)split * split_stride + (size_t)m * ld_out + n0 + ch * 32;
                        if (n_valid == BN) {
#pragma unroll
                            for (int c4 = 0; c4 < 8; ++c4)
                                *reinterpret_cast<uint4*>(dst + 4 * c4) = make_uint4(v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
                        } else {
#pragma unroll
                            for (int c = 0; c < 32; ++c) if (ch * 32 + c < n_valid) dst[c] = __uint_as_float(v[c]);
                        }
                    }
                }
            } else if constexpr (EPI == kEpiSwiglu) {
                static_assert(EPI != kEpiSwiglu || BN % 64 == 0, "SwiGLU tiles are groups of 32 gate + 32 up columns");
#pragma unroll 1
                for (int grp = 0; grp < BN / 64; ++grp) {       // each 64-column group: 32 gate columns, then the 32 matching up columns
                    uint32_t gt[32], up[32];
                    tmem_ld32(tmem + lane_base + grp * 64, gt);
                    tmem_ld32(tmem + lane_base + grp * 64 + 32, up);
                    tmem_wait_ld();
                    if (m < M && n0 + grp * 64 < N) {
                        __half* dst = out_fp16 + (size_t)m * ld_out + (n0 >> 1) + grp * 32;
#pragma unroll
                        for (int c8 = 0; c8 < 4; ++c8) {
                            __half2 h[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float g0 = __uint_as_float(gt[8 * c8 + 2 * e]), g1 = __uint_as_float(gt[8 * c8 + 2 * e + 1]);
                                const float u0 = __uint_as_float(up[8 * c8 + 2 * e]), u1 = __uint_as_float(up[8 * c8 + 2 * e + 1]);
                                h[e] = __floats2half2_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
                            }
                            *reinterpret_cast<uint4*>(dst + 8 * c8) = *reinterpret_cast<uint4*>(h);
                        }
                    }
                }
            } else {
                float best = -INFINITY;
                int bi = 0;
#pragma unroll 1
                for (int ch = 0; ch < BN / 32; ++ch) {
                    uint32_t v[32];
                    tmem_ld32(tmem + lane_base + ch * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const float x = __uint_as_float(v[c]);
                        if (ch * 32 + c < n_valid && x > best) { best = x; bi = ch * 32 + c; }
                    }
                }
                if (m < M) atomicMax(argmax_out + m, pack_argmax(best, n0 + bi));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, BN < 32 ? 32 : BN);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(error_word, 7);
}

// packed running argmax -> token ids; leaves the packed words at zero for the next step.
__global__ void argmax_unpack_kernel(unsigned long long* __restrict__ packed, int n, int* __restrict__ tokens) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned long long p = packed[i];
    tokens[i] = (int)(0xFFFFFFFFu - (uint32_t)(p & 0xFFFFFFFFull));
    packed[i] = 0ull;
}

// ---- host ----------------------------------------------------------------------------------------------------
namespace {
std::mutex g_map_mu;
std::map<std::tuple<const void*, int, int, int>, CUtensorMap> g_maps;

// Tensor map of a row-major fp16 matrix [rows, cols] with a {64 cols, box_rows} box (128-byte swizzle); cached per
// (pointer, shape) since weights and activation buffers keep their addresses.
int fp16_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> lk(g_map_mu);
    const auto key = std::make_tuple(ptr, rows, cols, box_rows);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return 0; }
    const uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
    const uint64_t str[1] = {(uint64_t)cols * 2};
    const uint32_t box[2] = {64, (uint32_t)box_rows};
    B2_TRY(make_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ptr, dims, str, box));
    g_maps[key] = *out;
    return 0;
}

template <int BN, int EPI>
int launch_one(const CUtensorMap& mx, const CUtensorMap& mw, int M, int N, int K, int splits, float* out_f32, int ld_out,
               size_t split_stride, __half* out_fp16, unsigned long long* argmax_out, int* d_error, cudaStream_t s) {
    static PerDeviceOnce once;
    B2_PER_DEVICE_ONCE(once, B2_CUDA(cudaFuncSetAttribute(gemm_small_m_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::kSmem)));
    const int k_steps = K / 64;
    const int per = ceil_div(k_steps, splits);
    dim3 grid(ceil_div(N, BN), ceil_div(k_steps, per));
    launch_pdl(gemm_small_m_kernel<BN, EPI>, grid, dim3(192), GemmCfg<BN>::kSmem, s, mx, mw, M, N, per, k_steps, out_f32, ld_out,
               split_stride, out_fp16, argmax_out, d_error);
    B2_LAUNCH_CHECK();
    return 0;
}
}  // namespace

int gemm_tc_map(const void* ptr, int rows, int cols, int box_rows, void* tensor_map_out) {
    return fp16_map(ptr, rows, cols, box_rows, static_cast<CUtensorMap*>(tensor_map_out));
}

void gemm_tc_forget(const void* ptr) {     // drop cached maps of a buffer that is being freed
    std::lock_guard<std::mutex> lk(g_map_mu);
    for (auto it = g_maps.begin(); it != g_maps.end();)
        it = (std::get<0>(it->first) == ptr) ? g_maps.erase(it) : std::next(it);
}

// B200ATTN_DECODE_GEMM=tc selects this kernel with its fused epilogues for the projections of the decode step; the
// default is cuBLAS with separate SwiGLU / argmax kernels.
bool gemm_tc_enabled() { return g_flags.decode_gemm_tc; }

// Number of split-K slices a [M<=128, N] x K product is cut into when the caller can sum partial tiles.
int gemm_tc_splits(int N, int K, int bn) {
    const int tiles = ceil_div(N, bn);
    int s = std::max(1, 148 / std::max(tiles, 1));
    s = std::min(s, std::max(1, K / 256));         // at least four 64-wide k-steps per slice
    return s;
}

// Y tile store (fp32).  splits > 1 writes `splits` partial matrices split_stride floats apart.
int gemm_tc_store(cudaStream_t s, const __half* X, const __half* W, float* Y, int M, int N, int K, int ld_out,
                  int splits, size_t split_stride, int* d_error) {
    B2_CHECK_ARG(M > 0 && M <= 128 && K % 64 == 0 && N > 0, "gemm_tc: unsupported shape %d x %d x %d", M, N, K);
    CUtensorMap mx, mw;
    B2_TRY(fp16_map(X, M, K, 128, &mx));
    // Without split-K every CTA reads all of X from L2, so wide N (the input projections) takes 128-column tiles:
    // half as many CTAs pull the activations, and 40-65 SMs still stream the weights faster than HBM delivers them.
    if (splits <= 1 && N >= 2048) {
        B2_TRY(fp16_map(W, N, K, 128, &mw));
        return launch_one<128, kEpiStore>(mx, mw, M, N, K, 1, Y, ld_out, split_stride, nullptr, nullptr, d_error, s);
    }
    B2_TRY(fp16_map(W, N, K, 64, &mw));
    return launch_one<64, kEpiStore>(mx, mw, M, N, K, splits, Y, ld_out, split_stride, nullptr, nullptr, d_error, s);
}

// act[M, N/2] = silu(gate) * up with W rows arranged in tiles of 32 gate rows followed by the 32 matching up rows.
int gemm_tc_swiglu(cudaStream_t s, const __half* X, const __half* W, __half* act, int M, int N, int K,
                   int* d_error) {
    B2_CHECK_ARG(M > 0 && M <= 128 && K % 64 == 0 && N % 64 == 0, "gemm_tc_swiglu: unsupported shape %d x %d x %d", M, N, K);
    CUtensorMap mx, mw;
    B2_TRY(fp16_map(X, M, K, 128, &mx));
    // 128-column tiles (two gate/up groups): half as many CTAs re-read the activations, and 56 SMs still stream the
    // 14.7 MB of gate/up weights of the model's FFN faster than HBM delivers them
    B2_TRY(fp16_map(W, N, K, 128, &mw));
    return launch_one<128, kEpiSwiglu>(mx, mw, M, N, K, 1, nullptr, N / 2, 0, act, nullptr, d_error, s);
}

// tokens[m] = argmax_n X[m] . W[n]   (d_packed: M zeroed 64-bit words, left zeroed again).
int gemm_tc_argmax(cudaStream_t s, const __half* X, const __half* W, unsigned long long* d_packed, int* tokens,
                   int M, int N, int K, int* d_error) {
    B2_CHECK_ARG(M > 0 && M <= 128 && K % 64 == 0 && N > 0, "gemm_tc_argmax: unsupported shape %d x %d x %d", M, N, K);
    CUtensorMap mx, mw;
    B2_TRY(fp16_map(X, M, K, 128, &mx));
    B2_TRY(fp16_map(W, N, K, 256, &mw));
    B2_TRY((launch_one<256, kEpiArgmax>(mx, mw, M, N, K, 1, nullptr, 0, 0, nullptr, d_packed, d_error, s)));
    launch_pdl(argmax_unpack_kernel, dim3(ceil_div(M, 128)), dim3(128), 0, s, d_packed, M, tokens);
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200
