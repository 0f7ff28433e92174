// Decode-step layer chain: the projections and RMSNorms that sit between two attention kernels of the decode step,
//     out-proj(l) -> +residual, RMSNorm -> gate/up + SwiGLU -> down -> +residual, RMSNorm(l+1) -> in-proj(l+1),
// as ONE persistent cooperative kernel (one CTA per SM) instead of eight launches.  At 128 rows every one of these
// steps is a few microseconds of weight streaming, so a launch boundary (drain, launch, ramp) costs as much as the
// work; here the phases are separated by grid barriers and the TMA ring of weight tiles keeps running across them:
// while a CTA waits for a barrier its producer has already requested the next phase's weights.
//
// Phases are skinny GEMMs (Y[rows <= 128, N] = X W^T, one 128 x 64 tile and one k-slice per CTA, tcgen05.mma with the
// accumulator in this phase's own 64 TMEM columns; epilogues: fp32 store / split-K partials, or SwiGLU -> bf16) and
// RMSNorms (one row per CTA: adds the split-K partials of the preceding GEMM to the residual stream, writes it back,
// normalises to bf16).  Replaces, per layer, output_proj_kernel / linear_proj_bf16_kernel calls and the norm + MLP
// launches of CudaLayer::forward_batch_decode (src/backend/cuda/kernels/cuda_engine.cu:109-156 in the reference).
// Every wait (mbarrier, grid barrier) is bounded; after a failed wait a CTA keeps arriving at barriers but stops
// storing, and raises the device status word.
#include "kernels.cuh"
#include "tc05.cuh"

namespace b200 {

constexpr int kChainStages = 8;
constexpr uint32_t kChainABytes = 128 * 128;              // 128 rows x 64 bf16 of activations
constexpr uint32_t kChainBBytes = 64 * 128;               // 64 rows x 64 bf16 of weights
constexpr uint32_t kChainStage = kChainABytes + kChainBBytes;
constexpr int kChainMaxGemm = 4, kChainMaxNorm = 2, kChainMaxPhases = 6;
constexpr uint32_t kChainSmem = kChainStages * kChainStage + 512 + 1024;
constexpr int kChainThreads = 192;

struct alignas(64) ChainGemm {
    CUtensorMap map_x, map_w;
    float* out_f32;
    __nv_bfloat16* out_bf16;
    size_t split_stride;
    int N, k_steps, k_per_split, n_tiles, ld_out, epi;
};
struct ChainNorm {
    float* h;
    const float* w;
    const float* partials;
    __nv_bfloat16* out;
    size_t split_stride;
    int n_splits;
    float eps;
};
struct alignas(64) ChainParams {
    ChainGemm g[kChainMaxGemm];
    ChainNorm n[kChainMaxNorm];
    int kind[kChainMaxPhases];     // 1 = GEMM, 0 = norm
    int idx[kChainMaxPhases];
    int n_phases, rows;
    unsigned* sync;                // [0] arrivals, [1] generation
    int* error_word;
};

// All CTAs of the (co-resident) grid meet here.  The generation is read before arriving; the last arriver resets
// the count and bumps the generation.  Bounded: on time-out the CTA raises its abort flag and goes on.
__device__ __forceinline__ bool chain_grid_barrier(unsigned* sync, unsigned n_cta, volatile int* abort_flag) {
    unsigned gen;
    asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(gen) : "l"(sync + 1) : "memory");
    __threadfence();
    const unsigned prev = atomicAdd(sync, 1u);
    if (prev == n_cta - 1) {
        atomicExch(sync, 0u);
        __threadfence();
        atomicAdd(sync + 1, 1u);
        return true;
    }
    if (*abort_flag) return false;
    const uint64_t t0 = global_timer_ns();
    uint32_t it = 0;
    while (true) {
        unsigned g2;
        asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(g2) : "l"(sync + 1) : "memory");
        if (g2 != gen) return true;
        if ((++it & 63u) == 0u && global_timer_ns() - t0 > 500000000ull) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// grid = number of SMs (cooperative), block 192: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2-5 = norm rows, epilogues and the grid barriers.
__global__ void __launch_bounds__(kChainThreads, 1) decode_chain_kernel(const __grid_constant__ ChainParams P) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ float s_red[4];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = smem_raw + (base - raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kChainStages * kChainStage);
    const uint32_t bar0 = base + kChainStages * kChainStage;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kChainStages + s); };
    auto acc_done = [&](int g) { return bar0 + 8u * (2 * kChainStages + g); };
    auto go = [&](int p) { return bar0 + 8u * (2 * kChainStages + kChainMaxGemm + p); };
    constexpr int kBars = 2 * kChainStages + kChainMaxGemm + kChainMaxPhases;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, n_cta = gridDim.x;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kBars; ++i) mbar_init(bar0 + 8u * i, 1);
        *abort_flag = (*reinterpret_cast<volatile int*>(P.error_word) != 0) ? 1 : 0;   // an earlier launch gave up: wait for nothing
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 64 * kChainMaxGemm);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0)
        for (int p = 0; p < P.n_phases; ++p)
            if (P.kind[p]) { tma_prefetch_desc(&P.g[P.idx[p]].map_x); tma_prefetch_desc(&P.g[P.idx[p]].map_w); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // this CTA's work item of GEMM phase G: one 64-column tile, one k-slice
    auto job = [&](const ChainGemm& G, int& n0, int& split, int& ks0, int& nk) -> bool {
        const int splits = (G.k_steps + G.k_per_split - 1) / G.k_per_split;
        if (cta >= G.n_tiles * splits) return false;
        n0 = (cta % G.n_tiles) * 64;
        split = cta / G.n_tiles;
        ks0 = split * G.k_per_split;
        nk = min(G.k_per_split, G.k_steps - ks0);
        return nk > 0;
    };

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int it = 0;     // k-steps issued so far, over all phases: stage = it % kChainStages
            bool ok = true;
            for (int p = 0; p < P.n_phases && ok; ++p) {
                if (!P.kind[p]) continue;
                const ChainGemm& G = P.g[P.idx[p]];
                int n0, split, ks0, nk;
                if (!job(G, n0, split, ks0, nk)) continue;
                // weights first: nothing in the chain writes them, so they may be requested before the barrier in front
                // of this phase has been passed
                const int pre = min(nk, kChainStages);
                for (int ks = 0; ks < pre && ok; ++ks) {
                    const int i = it + ks, st = i % kChainStages;
                    if (i >= kChainStages && !mbar_wait(empty(st), ((i / kChainStages) - 1) & 1, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(full(st), kChainStage);
                    tma_load_2d(base + st * kChainStage + kChainABytes, &G.map_w, full(st), (ks0 + ks) * 64, n0);
                }
                if (!ok) break;
                if (p > 0 && !mbar_wait(go(p), 0, abort_flag)) break;
                fence_proxy_async_all();     // other CTAs' generic-proxy writes of X, acquired at the barrier, before async-proxy reads
                for (int ks = 0; ks < pre; ++ks)
                    tma_load_2d(base + ((it + ks) % kChainStages) * kChainStage, &G.map_x, full((it + ks) % kChainStages), (ks0 + ks) * 64, 0);
                for (int ks = pre; ks < nk; ++ks) {
                    const int i = it + ks, st = i % kChainStages;
                    if (!mbar_wait(empty(st), ((i / kChainStages) - 1) & 1, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(full(st), kChainStage);
                    tma_load_2d(base + st * kChainStage, &G.map_x, full(st), (ks0 + ks) * 64, 0);
                    tma_load_2d(base + st * kChainStage + kChainABytes, &G.map_w, full(st), (ks0 + ks) * 64, n0);
                }
                it += nk;
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(kFmtBF16, 128, 64, 0, 0);
            int it = 0;
            bool ok = true;
            for (int p = 0; p < P.n_phases && ok; ++p) {
                if (!P.kind[p]) continue;
                const int gi = P.idx[p];
                int n0, split, ks0, nk;
                if (!job(P.g[gi], n0, split, ks0, nk)) continue;
                for (int ks = 0; ks < nk; ++ks, ++it) {
                    const int st = it % kChainStages;
                    if (!mbar_wait(full(st), (it / kChainStages) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a = base + st * kChainStage, b = a + kChainABytes;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_f16(tmem + 64 * gi, umma_smem_desc(a + kk * 32, 16, 1024), umma_smem_desc(b + kk * 32, 16, 1024), idesc,
                                 (ks > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(empty(st));
                }
                if (ok) umma_commit(acc_done(gi));
            }
        }
    } else {
        // ------------------------------ workers: norms, epilogues, grid barriers ------------------------------
        const int wt = threadIdx.x - 64;              // 0..127
        const int q = warp & 3;                       // TMEM lane quadrant this warp may read
        const int m = 32 * q + lane;                  // output row of the epilogues
        bool ok = true;
        for (int p = 0; p < P.n_phases; ++p) {
            if (p > 0) {
                // everything this CTA wrote in the previous phase is made visible, then the whole grid meets
                __threadfence();
                fence_proxy_async_all();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (wt == 0) {
                    if (!chain_grid_barrier(P.sync, (unsigned)n_cta, abort_flag)) ok = false;
                    mbar_arrive(go(p));
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (!P.kind[p]) {
                const ChainNorm& Nn = P.n[P.idx[p]];
                const bool mine = cta < P.rows;
                float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
                float4* src = reinterpret_cast<float4*>(Nn.h + (size_t)cta * kHidden);
                if (mine) {
                    v0 = __ldcg(src + wt);
                    v1 = __ldcg(src + wt + 128);
                    if (Nn.n_splits > 0) {
                        const float4* pp = reinterpret_cast<const float4*>(Nn.partials + (size_t)cta * kHidden);
                        const size_t step = Nn.split_stride / 4;
                        for (int sp = 0; sp < Nn.n_splits; sp += 4) {
                            float4 a[4], b[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const bool in = sp + e < Nn.n_splits;
                                a[e] = in ? __ldcg(pp + (size_t)(sp + e) * step + wt) : make_float4(0.f, 0.f, 0.f, 0.f);
                                b[e] = in ? __ldcg(pp + (size_t)(sp + e) * step + wt + 128) : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                v0.x += a[e].x; v0.y += a[e].y; v0.z += a[e].z; v0.w += a[e].w;
                                v1.x += b[e].x; v1.y += b[e].y; v1.z += b[e].z; v1.w += b[e].w;
                            }
                        }
                        if (ok) { src[wt] = v0; src[wt + 128] = v1; }
                    }
                }
                float ss = v0.x * v0.x + v0.y * v0.y + v0.z * v0.z + v0.w * v0.w + v1.x * v1.x + v1.y * v1.y + v1.z * v1.z + v1.w * v1.w;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) s_red[q] = ss;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (mine && ok) {
                    const float rms = sqrtf((s_red[0] + s_red[1] + s_red[2] + s_red[3]) / (float)kHidden + Nn.eps);
                    const float4 w0 = *reinterpret_cast<const float4*>(Nn.w + 4 * wt);
                    const float4 w1 = *reinterpret_cast<const float4*>(Nn.w + 4 * (wt + 128));
                    __nv_bfloat162 a0 = __floats2bfloat162_rn(v0.x / rms * (1.0f + w0.x), v0.y / rms * (1.0f + w0.y));
                    __nv_bfloat162 a1 = __floats2bfloat162_rn(v0.z / rms * (1.0f + w0.z), v0.w / rms * (1.0f + w0.w));
                    __nv_bfloat162 b0 = __floats2bfloat162_rn(v1.x / rms * (1.0f + w1.x), v1.y / rms * (1.0f + w1.y));
                    __nv_bfloat162 b1 = __floats2bfloat162_rn(v1.z / rms * (1.0f + w1.z), v1.w / rms * (1.0f + w1.w));
                    __nv_bfloat16* dst = Nn.out + (size_t)cta * kHidden;
                    *reinterpret_cast<uint2*>(dst + 4 * wt) = make_uint2(*reinterpret_cast<uint32_t*>(&a0), *reinterpret_cast<uint32_t*>(&a1));
                    *reinterpret_cast<uint2*>(dst + 4 * (wt + 128)) = make_uint2(*reinterpret_cast<uint32_t*>(&b0), *reinterpret_cast<uint32_t*>(&b1));
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");     // s_red is reused by the next norm phase
            } else {
                const int gi = P.idx[p];
                const ChainGemm& G = P.g[gi];
                int n0, split, ks0, nk;
                if (!job(G, n0, split, ks0, nk)) continue;
                if (!mbar_wait_warp(acc_done(gi), 0, abort_flag)) ok = false;
                tc_fence_after();
                const uint32_t taddr = tmem + 64 * gi + ((uint32_t)(32 * q) << 16);
                const int n_valid = min(64, G.N - n0);
                uint32_t c0[32], c1[32];
                tmem_ld32(taddr, c0);
                tmem_ld32(taddr + 32, c1);
                tmem_wait_ld();
                if (ok && m < P.rows) {
                    if (G.epi == 0) {
                        float* dst = G.out_f32 + (size_t)split * G.split_stride + (size_t)m * G.ld_out + n0;
                        if (n_valid == 64) {
#pragma unroll
                            for (int c4 = 0; c4 < 8; ++c4) {
                                *reinterpret_cast<uint4*>(dst + 4 * c4) = make_uint4(c0[4 * c4], c0[4 * c4 + 1], c0[4 * c4 + 2], c0[4 * c4 + 3]);
                                *reinterpret_cast<uint4*>(dst + 32 + 4 * c4) = make_uint4(c1[4 * c4], c1[4 * c4 + 1], c1[4 * c4 + 2], c1[4 * c4 + 3]);
                            }
                        } else {
#pragma unroll
                            for (int c = 0; c < 32; ++c) {
                                if (c < n_valid) dst[c] = __uint_as_float(c0[c]);
                                if (32 + c < n_valid) dst[32 + c] = __uint_as_float(c1[c]);
                            }
                        }
                    } else {
                        __nv_bfloat16* dst = G.out_bf16 + (size_t)m * G.ld_out + (n0 >> 1);
#pragma unroll
                        for (int c8 = 0; c8 < 4; ++c8) {
                            __nv_bfloat162 hh[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float g0 = __uint_as_float(c0[8 * c8 + 2 * e]), g1 = __uint_as_float(c0[8 * c8 + 2 * e + 1]);
                                const float u0 = __uint_as_float(c1[8 * c8 + 2 * e]), u1 = __uint_as_float(c1[8 * c8 + 2 * e + 1]);
                                hh[e] = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
                            }
                            *reinterpret_cast<uint4*>(dst + 8 * c8) = *reinterpret_cast<uint4*>(hh);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 64 * kChainMaxGemm);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(P.error_word, 7);
}

int launch_decode_chain(cudaStream_t s, int rows, const ChainPhaseDesc* phases, int n_phases, unsigned* d_sync, int* d_error) {
    B2_CHECK_ARG(rows > 0 && rows <= 128 && n_phases > 0 && n_phases <= kChainMaxPhases, "decode chain: %d rows, %d phases", rows, n_phases);
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        B2_CUDA(cudaGetDevice(&dev));
        B2_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
        B2_CUDA(cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kChainSmem));
    }
    ChainParams P;
    memset(&P, 0, sizeof(P));
    int ng = 0, nn = 0;
    for (int p = 0; p < n_phases; ++p) {
        P.kind[p] = phases[p].is_gemm;
        if (phases[p].is_gemm) {
            B2_CHECK_ARG(ng < kChainMaxGemm, "decode chain: more than %d GEMM phases", kChainMaxGemm);
            const ChainGemmDesc& d = phases[p].g;
            B2_CHECK_ARG(d.K % 64 == 0 && d.N > 0 && d.splits >= 1, "decode chain: unsupported GEMM %d x %d", d.N, d.K);
            ChainGemm& G = P.g[ng];
            B2_TRY(gemm_tc_map(d.X, rows, d.K, 128, &G.map_x));
            B2_TRY(gemm_tc_map(d.W, d.N, d.K, 64, &G.map_w));
            G.out_f32 = d.out_f32;
            G.out_bf16 = d.out_bf16;
            G.split_stride = d.split_stride;
            G.N = d.N;
            G.k_steps = d.K / 64;
            G.k_per_split = ceil_div(G.k_steps, d.splits);
            G.n_tiles = ceil_div(d.N, 64);
            G.ld_out = d.ld_out;
            G.epi = d.epi;
            const int items = G.n_tiles * ceil_div(G.k_steps, G.k_per_split);
            B2_CHECK_ARG(items <= n_sm, "decode chain: %d work items of one phase exceed the %d CTAs of the grid", items, n_sm);
            B2_CHECK_ARG(d.epi == 0 || (d.N % 64 == 0 && d.splits == 1), "decode chain: SwiGLU needs whole tiles and no split");
            P.idx[p] = ng++;
        } else {
            B2_CHECK_ARG(nn < kChainMaxNorm, "decode chain: more than %d norm phases", kChainMaxNorm);
            const ChainNormDesc& d = phases[p].n;
            P.n[nn] = ChainNorm{d.h, d.w, d.partials, d.out, d.split_stride, d.n_splits, d.eps};
            P.idx[p] = nn++;
        }
    }
    P.n_phases = n_phases;
    P.rows = rows;
    P.sync = d_sync;
    P.error_word = d_error;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_sm);
    cfg.blockDim = dim3(kChainThreads);
    cfg.dynamicSmemBytes = kChainSmem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;     // all CTAs resident at once: they wait for one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, decode_chain_kernel, P);
    if (e != cudaSuccess) B2_FAIL(B200ATTN_ERR_CUDA, "decode chain: launch failed: %s", cudaGetErrorString(e));
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200
