// G1: chunk-64 gated delta rule (WY / UT form) on tcgen05 tensor cores.
//
// One CTA per (sequence, head) walks the sequence in chunks of C = 64 tokens.  With b_i the running sum of
// the log decays g inside the chunk and S0 the state at the chunk start, the serial recurrence
//     S_i = e^{g_i} S_{i-1} + k_i (x) beta_i (v_i - (e^{g_i} S_{i-1})^T k_i),   o_i = S_i^T q_i
// (src/backend/cpu/core/attention/language_linear_attn.cpp:206-240 in the reference; its CUDA form is the
// token-serial gated_delta_batch_fused_v2_kernel, linear_attention_v2.cu:492-595) is equivalent to
//     A_ij   = beta_i e^{b_i-b_j} (k_i.k_j)  (j < i),      (I + A) [U | W] = [beta V | beta e^{b} K]
//     V_new  = U - W S0
//     O      = (Q e^{b}) S0 + tril(e^{b_i-b_j} (q_i.k_j)) V_new
//     S_C    = e^{b_C} S0 + K^T (e^{b_C-b} V_new)
// Every decay factor is formed as exp(b_i - b_j) with i >= j, never as a quotient of products.
//
// Contractions on the tensor cores (tcgen05.mma kind::f16, fp16 operands = the same 10-bit mantissa as tf32,
// fp32 accumulation in TMEM; all operand tiles use the 128-byte swizzle):
//   (a) D1[128x64]  = [K ; Q] K^T                      rows 0-63: K K^T, rows 64-127: Q K^T
//   (b) D2[128x128] = [W ; Q e^{b}] S0                 rows 0-63: W S0,  rows 64-127: inter-chunk output
//   (d) D2         += [0 ; Mq] V_new                   adds the intra-chunk output to rows 64-127
//   (u) D3[128x128] = e^{b_C} D3 + (e^{b_C-b} V_new)^T K    D3 holds S^T (lane = value dim) for the whole sequence
// The unit-lower-triangular solve runs in fp32 on the CUDA cores (thread t owns column t of U and of W).
// Warps 0-3 compute, warp 4 issues TMA loads and MMAs.  All waits are bounded.
#include "kernels.cuh"
#include "tc05.cuh"

namespace b200 {

constexpr int kC = 64;
constexpr uint32_t kOffKQ = 0;                 // [2 blocks][128 rows][128 B]: rows 0-63 K chunk, rows 64-127 Q chunk
constexpr uint32_t kOffWQ = 32768;             // A of (b): [2 blocks][128 rows][128 B]
constexpr uint32_t kOffST = 65536;             // B of (b): S^T, [2 blocks (64 kd)][128 vd rows][128 B]
constexpr uint32_t kOffVN = 98304;             // B of (d): V_new, [2 blocks (64 vd)][64 token rows][128 B]
constexpr uint32_t kOffVT = 114688;            // A of (u): (e^{b_C-b} V_new)^T, [128 vd rows][128 B = 64 tokens]
constexpr uint32_t kOffMQ = 131072;            // A of (d): [128 rows][128 B]; rows 0-63 zero, rows 64-127 Mq
constexpr uint32_t kOffAM = 147456;            // fp32 A matrix [64][64]
constexpr uint32_t kOffUS = 163840;            // fp32 U [64][kUSStride] (row stride 129 floats: conflict-free column and row access)
constexpr int kUSStride = 129;
constexpr uint32_t kOffSC = 197632;            // scalars: b[64], beta[64], eb[64], ebc[64]   (US ends at 163840 + 64*129*4 = 196864)
constexpr uint32_t kOffBarG = 198656;
constexpr uint32_t kG1Smem = kOffBarG + 128 + 1024;
enum { G_KQ_FULL = 0, G_A_DONE, G_B_READY, G_B_DONE, G_V_READY, G_D_DONE, G_KQ_FREE, G_BAR_COUNT };

__device__ __forceinline__ void named_sync_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ uint16_t f2h_bits(float x) {
    const __half h = __float2half_rn(x);
    return *reinterpret_cast<const uint16_t*>(&h);
}

// grid (heads, n_seqs), block 160
__global__ void __launch_bounds__(160, 1)
la_chunk_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const float* __restrict__ v, const float* __restrict__ g, const float* __restrict__ beta,
                   const LaSeqMeta* __restrict__ seqs, float* __restrict__ rec_layer, size_t rec_stride_slot,
                   float* __restrict__ out, int* __restrict__ error_word) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = smem_raw + (base - raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffBarG);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + G_BAR_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    auto bar = [&](int i) { return base + kOffBarG + 8u * i; };
    float* s_b = reinterpret_cast<float*>(sm + kOffSC);
    float* s_beta = s_b + 64;
    float* s_eb = s_b + 128;
    float* s_ebc = s_b + 192;
    float* AM = reinterpret_cast<float*>(sm + kOffAM);
    float* US = reinterpret_cast<float*>(sm + kOffUS);

    const int h = blockIdx.x;
    const LaSeqMeta sq = seqs[blockIdx.y];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int n_chunks = (sq.count + kC - 1) / kC;
    if (n_chunks == 0) return;
    if (*reinterpret_cast<volatile int*>(error_word) != 0) return;   // an earlier CTA gave up: do not queue more bounded waits
    float* Sg = rec_layer + (size_t)sq.slot * rec_stride_slot + (size_t)h * kLaKd * kLaVd;

    if (tid == 0) {
        for (int i = 0; i < G_BAR_COUNT; ++i)
            mbar_init(bar(i), (i == G_B_READY || i == G_V_READY || i == G_KQ_FREE) ? 128 : 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
        if (lane == 0) { tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tm_d1 = tmem, tm_d2 = tmem + 64, tm_d3 = tmem + 192;

    if (warp == 4) {
        // ------------------------------ TMA + MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t id_a = umma_idesc(kFmtF16, 128, 64, 0, 0);
            constexpr uint32_t id_b = umma_idesc(kFmtF16, 128, 128, 0, 0);
            constexpr uint32_t id_mn = umma_idesc(kFmtF16, 128, 128, 0, 1);
            for (int c = 0; c < n_chunks; ++c) {
                const uint32_t par = c & 1, prev = (c - 1) & 1;
                if (c > 0) {
                    if (!mbar_wait(bar(G_D_DONE), prev, abort_flag)) break;
                    if (!mbar_wait(bar(G_KQ_FREE), prev, abort_flag)) break;
                }
                const int row = sq.row0 + c * kC;
                mbar_arrive_expect_tx(bar(G_KQ_FULL), 32768);
                for (int blk = 0; blk < 2; ++blk) {
                    tma_load_3d(base + kOffKQ + blk * 16384, &map_k, bar(G_KQ_FULL), blk * 64, h, row);
                    tma_load_3d(base + kOffKQ + blk * 16384 + 8192, &map_q, bar(G_KQ_FULL), blk * 64, h, row);
                }
                if (!mbar_wait(bar(G_KQ_FULL), par, abort_flag)) break;
                tc_fence_after();
                // (a) D1 = [K;Q] K^T
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    umma_f16(tm_d1, umma_smem_desc(base + kOffKQ + off, 16, 1024), umma_smem_desc(base + kOffKQ + off, 16, 1024),
                             id_a, ks > 0 ? 1u : 0u);
                }
                umma_commit(bar(G_A_DONE));
                // (b) D2 = [W;Qe^b] S0
                if (!mbar_wait(bar(G_B_READY), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    umma_f16(tm_d2, umma_smem_desc(base + kOffWQ + off, 16, 1024), umma_smem_desc(base + kOffST + off, 16, 1024),
                             id_b, ks > 0 ? 1u : 0u);
                }
                umma_commit(bar(G_B_DONE));
                // (d) D2 += [0;Mq] V_new     (u) D3 += (e^{b_C-b} V_new)^T K
                if (!mbar_wait(bar(G_V_READY), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma_f16(tm_d2, umma_smem_desc(base + kOffMQ + ks * 32, 16, 1024),
                             umma_smem_desc(base + kOffVN + ks * 2048, 8192, 1024), id_mn, 1u);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma_f16(tm_d3, umma_smem_desc(base + kOffVT + ks * 32, 16, 1024),
                             umma_smem_desc(base + kOffKQ + ks * 2048, 16384, 1024), id_mn, 1u);
                umma_commit(bar(G_D_DONE));
            }
        }
    } else {
        // ------------------------------ compute warps ------------------------------
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const int r = tid;                      // TMEM lane: D1/D2 row, D3 value dim, and the solve column
        // MQ rows 0-63 stay zero for the whole kernel
        for (int i = tid; i < 64 * 8; i += 128) *reinterpret_cast<uint4*>(sm + kOffMQ + i * 16) = make_uint4(0, 0, 0, 0);
        // D3 <- S^T from the state pool: lane vd = r, column kd
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
            uint32_t sv[32];
#pragma unroll
            for (int c2 = 0; c2 < 32; ++c2) sv[c2] = __float_as_uint(Sg[(size_t)(ch * 32 + c2) * kLaVd + r]);
            tmem_st32(tm_d3 + lane_base + ch * 32, sv);
        }
        tmem_wait_st();
        bool ok = true;
        for (int c = 0; c < n_chunks && ok; ++c) {
            const uint32_t par = c & 1, prev = (c - 1) & 1;
            const int tok0 = c * kC;
            const int n_valid = min(kC, sq.count - tok0);
            // ---- per-chunk scalars: b = cumsum(g), beta; padded tokens get g = 0, beta = 0 ----
            if (warp < 2) {
                const int i = tid;
                const bool val = i < n_valid;
                const size_t gi = (size_t)(sq.row0 + tok0 + i) * kLaHeads + h;
                float gv = val ? g[gi] : 0.f;
                const float bv = val ? beta[gi] : 0.f;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float t2 = __shfl_up_sync(0xffffffffu, gv, o);
                    if (lane >= o) gv += t2;
                }
                s_b[i] = gv;
                s_beta[i] = bv;
            }
            named_sync_128();
            if (warp == 1) s_b[tid] += s_b[31];
            named_sync_128();
            if (tid < 64) {
                s_eb[tid] = expf(s_b[tid]);
                s_ebc[tid] = expf(s_b[63] - s_b[tid]);
            }
            named_sync_128();
            const float e_bc = expf(s_b[63]);
            // ---- S prep: D3 (S^T of the chunk start) -> fp16 tile for (b), and back to TMEM scaled by e^{b_C} ----
            if (c > 0 && !mbar_wait_warp(bar(G_D_DONE), prev, abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t sv[32];
                tmem_ld32(tm_d3 + lane_base + ch * 32, sv);
                tmem_wait_ld();
                unsigned char* row_ptr = sm + kOffST + (ch >> 1) * 16384 + r * 128;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {     // 8 halves = 16 bytes per store
                    uint32_t pk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        pk[e] = pack_half2(__uint_as_float(sv[q4 * 8 + 2 * e]), __uint_as_float(sv[q4 * 8 + 2 * e + 1]));
                    const int chunk16 = (ch & 1) * 4 + q4;
                    *reinterpret_cast<uint4*>(row_ptr + ((chunk16 ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
#pragma unroll
                for (int c2 = 0; c2 < 32; ++c2) sv[c2] = __float_as_uint(__uint_as_float(sv[c2]) * e_bc);
                tmem_st32(tm_d3 + lane_base + ch * 32, sv);
            }
            tmem_wait_st();
            // ---- right-hand sides: xu = beta V[:, t], xw = beta e^{b} K[:, t]  (t = tid) ----
            float xu[64], xw[64];
#pragma unroll
            for (int i = 0; i < 64; ++i)
                xu[i] = (i < n_valid) ? s_beta[i] * v[((size_t)(sq.row0 + tok0 + i) * kLaHeads + h) * kLaVd + tid] : 0.f;
            if (!mbar_wait_warp(bar(G_KQ_FULL), par, abort_flag)) { ok = false; break; }
            const unsigned char* kq_blk = sm + kOffKQ + (tid >> 6) * 16384;
            const int tcol = tid & 63;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                const __half kh = *reinterpret_cast<const __half*>(kq_blk + i * 128 + (((tcol >> 3) ^ (i & 7)) << 4) + (tcol & 7) * 2);
                xw[i] = s_beta[i] * s_eb[i] * __half2float(kh);
            }
            // ---- D1 -> A matrix (rows 0-63) and masked, decayed Q K^T (rows 64-127) ----
            if (!mbar_wait_warp(bar(G_A_DONE), par, abort_flag)) { ok = false; break; }
            tc_fence_after();
            {
                uint32_t d1[2][32];
                tmem_ld32(tm_d1 + lane_base, d1[0]);
                tmem_ld32(tm_d1 + lane_base + 32, d1[1]);
                tmem_wait_ld();
                if (r < 64) {
                    const float bi = s_b[r], be = s_beta[r];
#pragma unroll
                    for (int j4 = 0; j4 < 16; ++j4) {
                        float a4[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = j4 * 4 + e;
                            a4[e] = (j < r) ? be * expf(bi - s_b[j]) * __uint_as_float(d1[j >> 5][j & 31]) : 0.f;
                        }
                        *reinterpret_cast<float4*>(AM + r * 64 + j4 * 4) = make_float4(a4[0], a4[1], a4[2], a4[3]);
                    }
                } else {
                    const int i = r - 64;
                    const float bi = s_b[i];
                    unsigned char* row_ptr = sm + kOffMQ + r * 128;
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j0 = c8 * 8 + 2 * e, j1 = j0 + 1;
                            const float m0 = (j0 <= i) ? expf(bi - s_b[j0]) * __uint_as_float(d1[j0 >> 5][j0 & 31]) : 0.f;
                            const float m1 = (j1 <= i) ? expf(bi - s_b[j1]) * __uint_as_float(d1[j1 >> 5][j1 & 31]) : 0.f;
                            pk[e] = pack_half2(m0, m1);
                        }
                        *reinterpret_cast<uint4*>(row_ptr + ((c8 ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
            }
            named_sync_128();
            // ---- forward substitution (I + A) x = rhs, two columns per thread, fp32; four partial sums per
            //      column keep the FMA chains short ----
            {
                const float4* AM4 = reinterpret_cast<const float4*>(AM);
#pragma unroll
                for (int i = 1; i < 64; ++i) {
                    float u0 = 0.f, u1 = 0.f, u2 = 0.f, u3 = 0.f, w0 = 0.f, w1 = 0.f, w2 = 0.f, w3 = 0.f;
#pragma unroll
                    for (int j4 = 0; j4 * 4 < i; ++j4) {
                        const float4 a = AM4[i * 16 + j4];     // entries with j >= i are exact zeros
                        u0 += a.x * xu[j4 * 4];     w0 += a.x * xw[j4 * 4];
                        u1 += a.y * xu[j4 * 4 + 1]; w1 += a.y * xw[j4 * 4 + 1];
                        u2 += a.z * xu[j4 * 4 + 2]; w2 += a.z * xw[j4 * 4 + 2];
                        u3 += a.w * xu[j4 * 4 + 3]; w3 += a.w * xw[j4 * 4 + 3];
                    }
                    xu[i] -= (u0 + u1) + (u2 + u3);
                    xw[i] -= (w0 + w1) + (w2 + w3);
                }
            }
            // ---- publish U (fp32, row-major), W and Q e^{b} (fp16, swizzled K-major A tile of (b)) ----
            {
                unsigned char* wq_blk = sm + kOffWQ + (tid >> 6) * 16384;
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    US[i * kUSStride + tid] = xu[i];
                    const uint32_t sw = (((tcol >> 3) ^ (i & 7)) << 4) + (tcol & 7) * 2;      // (64 + i) & 7 == i & 7
                    *reinterpret_cast<uint16_t*>(wq_blk + i * 128 + sw) = f2h_bits(xw[i]);
                    const __half qh = *reinterpret_cast<const __half*>(kq_blk + (64 + i) * 128 + sw);
                    *reinterpret_cast<uint16_t*>(wq_blk + (64 + i) * 128 + sw) = f2h_bits(s_eb[i] * __half2float(qh));
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(G_B_READY));
            // ---- V_new = U - W S0 (threads 0-63, one token each) ----
            if (!mbar_wait_warp(bar(G_B_DONE), par, abort_flag)) { ok = false; break; }
            tc_fence_after();
            if (r < 64) {
                const float ebc = s_ebc[r];
#pragma unroll 1
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t d2[32];
                    tmem_ld32(tm_d2 + lane_base + ch * 32, d2);
                    tmem_wait_ld();
                    float vn[32];
#pragma unroll
                    for (int c2 = 0; c2 < 32; ++c2) vn[c2] = US[r * kUSStride + ch * 32 + c2] - __uint_as_float(d2[c2]);
                    unsigned char* vn_row = sm + kOffVN + (ch >> 1) * 8192 + r * 128;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) pk[e] = pack_half2(vn[q4 * 8 + 2 * e], vn[q4 * 8 + 2 * e + 1]);
                        const int chunk16 = (ch & 1) * 4 + q4;
                        *reinterpret_cast<uint4*>(vn_row + ((chunk16 ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
#pragma unroll
                    for (int c2 = 0; c2 < 32; ++c2) {
                        const int vd = ch * 32 + c2;
                        *reinterpret_cast<uint16_t*>(sm + kOffVT + vd * 128 + (((r >> 3) ^ (vd & 7)) << 4) + (r & 7) * 2) =
                            f2h_bits(ebc * vn[c2]);
                    }
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(G_V_READY));
            mbar_arrive(bar(G_KQ_FREE));       // no thread reads the K/Q tile after this point
            // ---- outputs: D2 rows 64-127 once (d) has been added ----
            if (r >= 64) {
                if (!mbar_wait_warp(bar(G_D_DONE), par, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const int i = r - 64;
                float* orow = out + ((size_t)(sq.row0 + tok0 + i) * kLaHeads + h) * kLaVd;
#pragma unroll 1
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t d2[32];
                    tmem_ld32(tm_d2 + lane_base + ch * 32, d2);
                    tmem_wait_ld();
                    if (i < n_valid) {
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4)
                            *reinterpret_cast<float4*>(orow + ch * 32 + q4 * 4) =
                                make_float4(__uint_as_float(d2[q4 * 4]), __uint_as_float(d2[q4 * 4 + 1]),
                                            __uint_as_float(d2[q4 * 4 + 2]), __uint_as_float(d2[q4 * 4 + 3]));
                    }
                }
                tc_fence_before();
            }
        }
        // ---- final state: D3 (S^T) -> state pool ----
        if (ok && mbar_wait_warp(bar(G_D_DONE), (n_chunks - 1) & 1, abort_flag)) {
            tc_fence_after();
#pragma unroll 1
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t sv[32];
                tmem_ld32(tm_d3 + lane_base + ch * 32, sv);
                tmem_wait_ld();
#pragma unroll
                for (int c2 = 0; c2 < 32; ++c2) Sg[(size_t)(ch * 32 + c2) * kLaVd + r] = __uint_as_float(sv[c2]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
    if (tid == 0 && *abort_flag) atomicExch(error_word, 6);
}

// q_h, k_h: fp16 [rows][16][128]; v fp32 [rows][16][128]; g, beta fp32 [rows][16].
int launch_la_chunk_tc(const __half* q_h, const __half* k_h, const float* v, const float* g, const float* beta,
                       const LaSeqMeta* d_seqs, int n_seqs, int rows, float* rec_layer, size_t rec_stride, float* out,
                       int* d_error, cudaStream_t s) {
    CUtensorMap mq, mk;
    const uint64_t dims[3] = {(uint64_t)kLaKd, (uint64_t)kLaHeads, (uint64_t)rows};
    const uint64_t str[2] = {(uint64_t)kLaKd * 2, (uint64_t)kLaHeads * kLaKd * 2};
    const uint32_t box[3] = {64, 1, (uint32_t)kC};
    B2_TRY(make_tensor_map(&mq, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, q_h, dims, str, box));
    B2_TRY(make_tensor_map(&mk, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, k_h, dims, str, box));
    static bool attr_done = false;
    if (!attr_done) {
        B2_CUDA(cudaFuncSetAttribute(la_chunk_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kG1Smem));
        attr_done = true;
    }
    dim3 grid(kLaHeads, n_seqs);
    la_chunk_tc_kernel<<<grid, 160, kG1Smem, s>>>(mq, mk, v, g, beta, d_seqs, rec_layer, rec_stride, out, d_error);
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200
