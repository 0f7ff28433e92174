// Skinny GEMM for the decode step on tcgen05: Y[M <= 128, N] = X[M, K] W[N, K]^T with fp16 operands and fp32
// accumulation in TMEM.  At 128 rows the projections are pure weight streaming (every weight byte is used once),
// so the kernel is a TMA -> shared-memory ring -> tcgen05.mma pipeline with one 128 x BN output tile per CTA and
// optional split-K, sized so a launch puts about one CTA on every SM.  Epilogues:
//   kEpiStore   fp32 tile store (also used for split-K partials, which the following norm kernel sums);
//   kEpiSwiglu  the tile holds BN/2 gate columns then the BN/2 matching up columns: act = silu(gate) * up, fp16;
//   kEpiArgmax  running per-row argmax over all tiles (64-bit atomicMax on {ordered value, ~index}).
// With `rowsq` the store and SwiGLU epilogues first scale row m by 1 / sqrt(mean(x_m^2) + eps), taken from the sums of
// squares the producer of X left behind: the RMSNorm in front of the projection then costs no launch (its (1 + w)
// factor is folded into the weight columns when the weights are loaded).
// gemm_residual_kernel is the matching producer: h += X W^T for the 1024-wide output projections, cut along K over
// the CTAs of a thread-block cluster, reduced through distributed shared memory in a fixed order, and written back
// as fp32 h, an fp16 copy and the per-row sums of squares for the next projection.
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
                    const float* __restrict__ rowsq, float rs_eps, int* __restrict__ error_word, unsigned long long* stamp) {
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
        stamp_begin(stamp);
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
            float rs = 1.0f;                          // RMSNorm scale of row m (the producer of X left kRowsqParts partial sums)
            if (rowsq && m < M) {
                float ss = 0.f;
#pragma unroll
                for (int p4 = 0; p4 < kRowsqParts / 4; ++p4) {
                    const float4 v4 = __ldcg(reinterpret_cast<const float4*>(rowsq + (size_t)m * kRowsqParts) + p4);
                    ss += (v4.x + v4.y) + (v4.z + v4.w);
                }
                rs = 1.0f / sqrtf(ss / (float)kHidden + rs_eps);
            }
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
                                *reinterpret_cast<float4*>(dst + 4 * c4) = make_float4(__uint_as_float(v[4 * c4]) * rs, __uint_as_float(v[4 * c4 + 1]) * rs,
                                                                                        __uint_as_float(v[4 * c4 + 2]) * rs, __uint_as_float(v[4 * c4 + 3]) * rs);
                        } else {
#pragma unroll
                            for (int c = 0; c < 32; ++c) if (ch * 32 + c < n_valid) dst[c] = __uint_as_float(v[c]) * rs;
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
                                const float g0 = __uint_as_float(gt[8 * c8 + 2 * e]) * rs, g1 = __uint_as_float(gt[8 * c8 + 2 * e + 1]) * rs;
                                const float u0 = __uint_as_float(up[8 * c8 + 2 * e]) * rs, u1 = __uint_as_float(up[8 * c8 + 2 * e + 1]) * rs;
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
    stamp_end(stamp);
    if (threadIdx.x == 0 && *abort_flag) atomicExch(error_word, 7);
}

// ---- h += X W^T for the two 1024-wide output projections of a layer (attention output, FFN down) ------------------------
// grid (N / 64, S) with clusters (1, S, 1): the S CTAs of a cluster share one 64-column output tile and cut K between
// them (S = 4 or 8, at most kResStages k-steps of 64 each, all in flight at once).  Every CTA leaves its partial tile in its
// own shared memory; after a cluster barrier CTA r adds up rows [128 r / S, 128 (r + 1) / S) over all S partials through
// distributed shared memory, always in the order s = 0 .. S-1, adds the residual stream and writes back:
//   h      fp32 [M, N]   the residual stream, in place;
//   xh     fp16 [M, N]   the same rows as the A operand of the next projection;
//   rowsq  fp32 [128][kRowsqParts]  column blockIdx.x of it: the sum of squares of the row over this tile's 64 columns.
// No partial ever reaches global memory and nothing depends on arrival order.  Block 192 as in gemm_small_m_kernel.
constexpr int kResBN = 64;
constexpr int kResStages = 8;
constexpr uint32_t kResStage = 128 * 128 + kResBN * 128;      // X tile + W tile of one k-step
constexpr int kResLd = 68;                                    // pitch (floats) of a partial row: no bank conflicts for row-per-lane float4
constexpr uint32_t kResSmem = kResStages * kResStage + 256 + 1024;
static_assert(128 * kResLd * 4 <= kResStages * kResStage, "the partial tile reuses the operand ring");
static_assert(kHidden / kResBN == kRowsqParts, "one sum-of-squares part per output tile of the residual GEMM");

__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_smem_addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ float4 dsmem_ld_f4(uint32_t addr) {
    float4 v;
    // not volatile: the loads of one thread are independent and may be issued as a batch; they cannot move above the
    // cluster barrier because their address comes out of mapa, which is ordered after it
    asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
// Every thread of every CTA of the cluster (threads that have exited do not count).
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int S>
__global__ void __launch_bounds__(192)
gemm_residual_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, int M, int N, int nk,
                     float* __restrict__ h, __half* __restrict__ xh, float* __restrict__ rowsq, int* __restrict__ error_word,
                     unsigned long long* stamp) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = smem_raw + (base - raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kResStages * kResStage);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kResStages + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = base + kResStages * kResStage;
    auto full = [&](int st) { return bar0 + 8u * st; };
    const uint32_t acc_done = bar0 + 8u * kResStages;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kResBN;
    const uint32_t rank = blockIdx.y;              // rank inside the cluster: the grid is exactly one cluster high
    const int ks0 = (int)rank * nk;
    // No CTA may leave before its peers have read its partial tile, so a failure seen earlier does not end the kernel
    // here: the CTA skips its work and still meets both cluster barriers.
    const bool dead = *reinterpret_cast<volatile int*>(error_word) != 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kResStages + 1; ++i) mbar_init(bar0 + 8u * i, 1);
        *abort_flag = dead ? 1 : 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), kResBN);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) { tma_prefetch_desc(&map_x); tma_prefetch_desc(&map_w); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0 && lane == 0 && !dead) {
        for (int ks = 0; ks < nk; ++ks) {           // the weights are never written during a step: request them before the wait
            mbar_arrive_expect_tx(full(ks), kResStage);
            tma_load_2d(base + ks * kResStage + 128 * 128, &map_w, full(ks), (ks0 + ks) * 64, n0);
        }
        pdl_enter();
        stamp_begin(stamp);
        for (int ks = 0; ks < nk; ++ks) tma_load_2d(base + ks * kResStage, &map_x, full(ks), (ks0 + ks) * 64, 0);
    } else {
        pdl_enter();
    }
    if (warp == 1 && lane == 0 && !dead) {
        constexpr uint32_t idesc = umma_idesc(kFmtF16, 128, kResBN, 0, 0);
        bool ok = true;
        for (int ks = 0; ks < nk; ++ks) {
            if (!mbar_wait(full(ks), 0, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a = base + ks * kResStage, b = a + 128 * 128;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_f16(tmem, umma_smem_desc(a + kk * 32, 16, 1024), umma_smem_desc(b + kk * 32, 16, 1024), idesc, (ks > 0 || kk > 0) ? 1u : 0u);
        }
        if (ok) umma_commit(acc_done);
    }
    float* part = reinterpret_cast<float*>(sm);     // [128][kResLd] over the operand ring once every product has completed
    // Reduction roles of the epilogue threads: 128 / S rows per CTA, S threads per row, 64 / S columns per thread.  The
    // residual values they will add to are requested right after the dependency wait, long before they are needed.
    constexpr int kCols = kResBN / S, kV4 = kCols / 4;
    const int rt = (int)threadIdx.x - 64;
    const int rrow = (int)rank * (128 / S) + (rt >= 0 ? rt / S : 0), rseg = rt >= 0 ? rt % S : 0;
    const bool ract = warp >= 2 && rrow < M && !dead;
    float* hrow = h + (size_t)rrow * N + n0 + rseg * kCols;
    float4 acc[kV4];
    if (ract) {
#pragma unroll
        for (int c4 = 0; c4 < kV4; ++c4) acc[c4] = __ldcg(reinterpret_cast<const float4*>(hrow) + c4);
    }
    if (warp >= 2) {
        const int q = warp & 3, m = 32 * q + lane;
        if (mbar_wait_warp(acc_done, 0, abort_flag)) {
            tc_fence_after();
            const uint32_t lane_base = (uint32_t)(32 * q) << 16;
#pragma unroll 1
            for (int ch = 0; ch < kResBN / 32; ++ch) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + ch * 32, v);
                tmem_wait_ld();
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4)
                    *reinterpret_cast<uint4*>(part + m * kResLd + ch * 32 + 4 * c4) = make_uint4(v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
            }
        }
    }
    tc_fence_before();
    cluster_sync_all();                              // every partial tile of the cluster is in place (or its CTA has flagged a failure)
    const bool reduce = warp >= 2 && !*abort_flag;
    float4 pv[S][kV4];
    if (reduce) {
        // sixteen 16-byte remote loads per thread, all requested before the first one is used
        const uint32_t local = smem_u32(part + rrow * kResLd + rseg * kCols);
#pragma unroll
        for (int sp = 0; sp < S; ++sp) {
            const uint32_t remote = dsmem_addr(local, (uint32_t)sp);
#pragma unroll
            for (int c4 = 0; c4 < kV4; ++c4) pv[sp][c4] = dsmem_ld_f4(remote + 16 * c4);
        }
        // touch every loaded value so that all remote reads of this thread have completed before it reports to the peers
        float touch = 0.f;
#pragma unroll
        for (int sp = 0; sp < S; ++sp)
#pragma unroll
            for (int c4 = 0; c4 < kV4; ++c4) touch += pv[sp][c4].x;
        asm volatile("" ::"f"(touch));
    }
    // This CTA has finished reading its peers' shared memory: tell them now, wait for them only before leaving, so the
    // write-back below runs under the barrier's latency.
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    if (reduce) {
        float ss = 0.f;
        if (ract) {
#pragma unroll
            for (int sp = 0; sp < S; ++sp)             // fixed order: the sum does not depend on which CTA finished first
#pragma unroll
                for (int c4 = 0; c4 < kV4; ++c4) {
                    acc[c4].x += pv[sp][c4].x; acc[c4].y += pv[sp][c4].y; acc[c4].z += pv[sp][c4].z; acc[c4].w += pv[sp][c4].w;
                }
            uint32_t pk[2 * kV4];
#pragma unroll
            for (int c4 = 0; c4 < kV4; ++c4) {
                reinterpret_cast<float4*>(hrow)[c4] = acc[c4];
                pk[2 * c4] = pack_half2(acc[c4].x, acc[c4].y);
                pk[2 * c4 + 1] = pack_half2(acc[c4].z, acc[c4].w);
                ss += acc[c4].x * acc[c4].x + acc[c4].y * acc[c4].y + acc[c4].z * acc[c4].z + acc[c4].w * acc[c4].w;
            }
            uint4* xrow = reinterpret_cast<uint4*>(xh + (size_t)rrow * N + n0 + rseg * kCols);
#pragma unroll
            for (int c8 = 0; c8 < kV4 / 2; ++c8) xrow[c8] = make_uint4(pk[4 * c8], pk[4 * c8 + 1], pk[4 * c8 + 2], pk[4 * c8 + 3]);
        }
#pragma unroll
        for (int o = 1; o < S; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (ract && rseg == 0) rowsq[(size_t)rrow * kRowsqParts + blockIdx.x] = ss;
    }
    __syncwarp();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // nobody reads this CTA's shared memory any more
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kResBN);
    }
    stamp_end(stamp);
    if (threadIdx.x == 0 && *abort_flag && !dead) atomicExch(error_word, 7);
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
               size_t split_stride, __half* out_fp16, unsigned long long* argmax_out, const float* rowsq, float rs_eps, int* d_error,
               cudaStream_t s) {
    unsigned long long* stamp = prof_stamp_slot(EPI == kEpiStore ? PROF_GEMM_IN : EPI == kEpiSwiglu ? PROF_GEMM_FFN : PROF_LM_HEAD);
    static PerDeviceOnce once;
    B2_PER_DEVICE_ONCE(once, B2_CUDA(cudaFuncSetAttribute(gemm_small_m_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::kSmem)));
    const int k_steps = K / 64;
    const int per = ceil_div(k_steps, splits);
    dim3 grid(ceil_div(N, BN), ceil_div(k_steps, per));
    launch_pdl(gemm_small_m_kernel<BN, EPI>, grid, dim3(192), GemmCfg<BN>::kSmem, s, mx, mw, M, N, per, k_steps, out_f32, ld_out,
               split_stride, out_fp16, argmax_out, rowsq, rs_eps, d_error, stamp);
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

// B200ATTN_DECODE_GEMM=tc selects the kernels of this file for the projections of the decode step (five launches per
// DeltaNet layer instead of eight).  The default is library GEMMs with separate norm / SwiGLU kernels, which is still
// the faster step as a whole: measured at 128 rows inside the captured step, an input or gate / up projection here
// takes 8.5 us and a residual projection 11 us (2.5 us from the dependency wait to the accumulators, then the cluster
// barrier, the remote reads and the write-back), 2.27 ms per step against 2.13 ms at a cache length of 256.  Asking
// L2 for the coming weights from inside the attention kernels made it worse (2.60 ms): the state stream evicts them.
bool gemm_tc_enabled() { return g_flags.decode_gemm_tc; }

// Y[M, N] = rs[m] * X W^T (fp32 store).  rowsq == nullptr: no row scale.
int gemm_tc_store(cudaStream_t s, const __half* X, const __half* W, float* Y, int M, int N, int K, int ld_out, const float* rowsq,
                  float rs_eps, int* d_error) {
    B2_CHECK_ARG(M > 0 && M <= 128 && K % 64 == 0 && N > 0, "gemm_tc: unsupported shape %d x %d x %d", M, N, K);
    CUtensorMap mx, mw;
    B2_TRY(fp16_map(X, M, K, 128, &mx));
    // 64-column tiles: 129 CTAs for the 8224-wide input projection.  Every CTA reads all of X from L2, so 128-column
    // tiles would halve that traffic, but with half as many CTAs there are too few weight bytes in flight to keep HBM
    // busy: measured 12.5 us per launch against 8.5 us inside the captured step.
    B2_TRY(fp16_map(W, N, K, 64, &mw));
    return launch_one<64, kEpiStore>(mx, mw, M, N, K, 1, Y, ld_out, 0, nullptr, nullptr, rowsq, rs_eps, d_error, s);
}

// act[M, N/2] = silu(gate) * up of rs[m] * X W^T, with W rows arranged in tiles of 32 gate rows followed by the 32 matching
// up rows.
int gemm_tc_swiglu(cudaStream_t s, const __half* X, const __half* W, __half* act, int M, int N, int K, const float* rowsq,
                   float rs_eps, int* d_error) {
    B2_CHECK_ARG(M > 0 && M <= 128 && K % 64 == 0 && N % 64 == 0, "gemm_tc_swiglu: unsupported shape %d x %d x %d", M, N, K);
    CUtensorMap mx, mw;
    B2_TRY(fp16_map(X, M, K, 128, &mx));
    B2_TRY(fp16_map(W, N, K, 64, &mw));      // one gate / up group of 32 + 32 columns per CTA, 112 CTAs for the model's FFN
    return launch_one<64, kEpiSwiglu>(mx, mw, M, N, K, 1, nullptr, N / 2, 0, act, nullptr, rowsq, rs_eps, d_error, s);
}

// h[M, N] += X[M, K] W[N, K]^T; also xh = fp16(h) and the per-row sums of squares (see gemm_residual_kernel).  N must be
// kHidden; K / 64 must split into at most 8 CTAs of at most kResStages k-steps.
int gemm_tc_residual(cudaStream_t s, const __half* X, const __half* W, float* h, __half* xh, float* rowsq, int M, int N, int K,
                     int* d_error) {
    B2_CHECK_ARG(M > 0 && M <= 128 && K % 64 == 0 && N == kHidden, "gemm_tc_residual: unsupported shape %d x %d x %d", M, N, K);
    const int k_steps = K / 64;
    int S = 0;
    // the smaller cluster where the slice still fits the ring: clusters of four start sooner than clusters of eight
    // (measured 10.9 against 13.7 us per launch for the 2048-deep attention output projection)
    for (int cand : {4, 8}) if (k_steps % cand == 0 && k_steps / cand <= kResStages) { S = cand; break; }
    B2_CHECK_ARG(S != 0, "gemm_tc_residual: K = %d does not split into 4 or 8 slices of at most %d k-steps", K, kResStages);
    CUtensorMap mx, mw;
    B2_TRY(fp16_map(X, M, K, 128, &mx));
    B2_TRY(fp16_map(W, N, K, 64, &mw));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(N / kResBN, S);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = kResSmem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = S; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_flags.pdl ? 2 : 1;
    const int nk = k_steps / S;
    unsigned long long* stamp = prof_stamp_slot(PROF_GEMM_RES);
#define RES_LAUNCH(SS)                                                                                                              \
    do {                                                                                                                            \
        static PerDeviceOnce once;                                                                                                  \
        B2_PER_DEVICE_ONCE(once, B2_CUDA(cudaFuncSetAttribute(gemm_residual_kernel<SS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kResSmem))); \
        B2_CUDA(cudaLaunchKernelEx(&cfg, gemm_residual_kernel<SS>, mx, mw, M, N, nk, h, xh, rowsq, d_error, stamp));                       \
    } while (0)
    if (S == 8) RES_LAUNCH(8); else RES_LAUNCH(4);
#undef RES_LAUNCH
    count_launch();
    return 0;
}

// tokens[m] = argmax_n X[m] . W[n]   (d_packed: M zeroed 64-bit words, left zeroed again).
int gemm_tc_argmax(cudaStream_t s, const __half* X, const __half* W, unsigned long long* d_packed, int* tokens,
                   int M, int N, int K, int* d_error) {
    B2_CHECK_ARG(M > 0 && M <= 128 && K % 64 == 0 && N > 0, "gemm_tc_argmax: unsupported shape %d x %d x %d", M, N, K);
    CUtensorMap mx, mw;
    B2_TRY(fp16_map(X, M, K, 128, &mx));
    B2_TRY(fp16_map(W, N, K, 256, &mw));
    B2_TRY((launch_one<256, kEpiArgmax>(mx, mw, M, N, K, 1, nullptr, 0, 0, nullptr, d_packed, nullptr, 0.f, d_error, s)));
    launch_pdl(argmax_unpack_kernel, dim3(ceil_div(M, 128)), dim3(128), 0, s, d_packed, M, tokens);
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200
