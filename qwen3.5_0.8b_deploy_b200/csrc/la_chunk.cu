// G1: chunk-64 gated delta rule (WY / UT form) on tcgen05 tensor cores.
//
// One CTA per (sequence, head) walks the sequence in chunks of C = 64 tokens; two CTAs share an SM (106 KB of shared
// memory and 256 TMEM columns each), so one CTA's CUDA-core phases run under the other's tensor-core phases.  With b_i
// the running sum of the log decays g inside the chunk and S0 the state at the chunk start, the serial recurrence
//     S_i = e^{g_i} S_{i-1} + k_i (x) beta_i (v_i - (e^{g_i} S_{i-1})^T k_i),   o_i = S_i^T q_i
// (src/backend/cpu/core/attention/language_linear_attn.cpp:206-240 in the reference; its CUDA form is the
// token-serial gated_delta_batch_fused_v2_kernel, linear_attention_v2.cu:492-595) is equivalent to
//     A_ij  = beta_i e^{b_i-b_j} (k_i.k_j)  (j < i),     T = (I + A)^-1
//     U     = T (beta V),   W = T (beta e^{b} K),        V_new = U - W S0
//     O     = (Q e^{b}) S0 + tril(e^{b_i-b_j} (q_i.k_j)) V_new
//     S_C   = e^{b_C} S0 + (e^{b_C-b} K)^T V_new
// Every decay factor is formed as exp(b_i - b_j) with i >= j, never as a quotient of products.
//
// All state-sized objects are kept TRANSPOSED in TMEM (lane = value dim or key dim, column = token), so every
// tensor-core product has M = 128 and every tile a thread writes is one of its own rows.  The row scalings by beta and
// beta e^b are folded into the columns of T, so that the K and V tiles go to the tensor core exactly as TMA delivered
// them (as MN-major operands) and no transposed operand is ever built by scattered stores:
//   (a)  D1  [128 x 64] = [K ; Q] K^T                         rows 0-63: K K^T, rows 64-127: Q K^T
//   (uw) Ut  [vd x 64]  = V^T (T diag(beta))^T,   Wt [kd x 64] = K^T (T diag(beta e^b))^T     (T as an fp16 hi + lo pair)
//   (ws) Ut -= S0^T W^T                                        -> V_new^T, accumulated in place (negated A operand)
//   (o)  Ot  [vd x 64]  = S0^T (Q e^b)^T + V_new^T Mq^T       (Q is scaled in place in its TMA tile)
//   (u)  D3  [vd x kd]  = e^{b_C} D3 + V_new^T (e^{b_C-b} K)  D3 holds S^T for the whole sequence; K is scaled in place
// tcgen05.mma kind::f16: fp16 operands (the same 10-bit mantissa as tf32), fp32 accumulation; 128-byte swizzle.
// T itself is built in fp32 in shared memory by a blocked inverse (16 x 16 blocks) on the CUDA cores, each warp
// solving its own columns of T from top to bottom.
//
// Eight compute warps (two threads per TMEM lane, each owning half of the 64 token columns) and one warp that
// issues TMA loads and MMAs.  All waits are bounded.
#include "kernels.cuh"
#include "tc05.cuh"

namespace b200 {

constexpr int kC = 64;
// shared-memory map (bytes from a 1024-aligned base); regions are reused as their contents die during a chunk
constexpr uint32_t kOffKQ = 0;        // [2 blocks of 64 key dims][rows 0-63 K chunk, rows 64-127 Q chunk][128 B]
constexpr uint32_t kOffV = 32768;     // V chunk [2 blocks of 64 value dims][64 tokens][128 B]; after (uw): V_new^T [128 vd][64 tokens]
constexpr uint32_t kOffR = 49152;     // 32 KB: fp32 A and T ([64][68] each, 34 KB: the tail lies in the W tile, dead at that time)
                                      //        ->  T diag(beta) hi, lo, T diag(beta e^b) hi, lo (four [64][64] fp16 tiles)
                                      //        ->  S0^T fp16 [2 blocks of 64 kd][128 vd rows][128 B]
constexpr uint32_t kOffW = 81920;     // W^T [128 kd rows][64 tokens] fp16                B of (ws), MN-major
constexpr uint32_t kOffMQ = 98304;    // Mq [64][64] fp16                                 B of (o)
constexpr uint32_t kOffSC = 106496;   // scalars: b[64], beta[64], eb[64], ebc[64]
constexpr uint32_t kOffBarG = 107520;
constexpr uint32_t kG1Smem = kOffBarG + 128 + 1024;
constexpr int kG1Threads = 288;
enum { G_FULL = 0, G_A_DONE, G_B1, G_C1, G_B2, G_C2, G_B3, G_C3, G_OT_FREE, G_BAR_COUNT };

__device__ __forceinline__ void named_sync_256() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// 2^x on the special-function unit (about 2 ulp); the decay matrices need 64 x 64 of them per chunk and head.
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr float kLog2e = 1.4426950408889634f;

// Row pitch (floats) of the fp32 A and T matrices in shared memory: 68 keeps 16-byte alignment and moves consecutive
// rows by four banks, so a warp's row-per-lane float4 accesses do not collide.
constexpr int kLd = 68;

// Columns [c0, c0 + NC) of the blocks below the diagonal block J of T = (I + A)^-1, given the inverted diagonal blocks
// D_I (already in T):  T_IJ = -D_I sum_{K=J}^{I-1} A_IK T_KJ  for I = J+1 .. 3.  A column of T depends only on the same
// column of the block rows above it, so one warp owns its columns from top to bottom and never meets another warp.
// Lane (rg, c): RPL = NC / 2 rows rg*RPL .. of the 16-row block, column c0 + c.  The inner sums P are passed from the
// accumulating lanes to the lanes that multiply by D_I through A's block (J, I), which lies above the diagonal, is
// zero and not otherwise used.
template <int NC>
__device__ __forceinline__ void solve_column_group(float* AM, float* TF, int J, int c0, int lane) {
    constexpr int RPL = NC / 2;
    const int rg = lane / NC, c = lane % NC;
    const int r0 = rg * RPL;
    for (int I = J + 1; I < 4; ++I) {
        float p[RPL];
#pragma unroll
        for (int i = 0; i < RPL; ++i) p[i] = 0.f;
        for (int K = J; K < I; ++K) {
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
                float t[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) t[e] = TF[(16 * K + 4 * k4 + e) * kLd + c0 + c];
#pragma unroll
                for (int i = 0; i < RPL; ++i) {
                    const float4 a = *reinterpret_cast<const float4*>(&AM[(16 * I + r0 + i) * kLd + 16 * K + 4 * k4]);
                    p[i] += a.x * t[0] + a.y * t[1] + a.z * t[2] + a.w * t[3];
                }
            }
        }
        float* P = AM + (16 * J) * kLd + 16 * I + (c0 - 16 * J);      // 16 x NC scratch in the zero block (J, I)
#pragma unroll
        for (int i = 0; i < RPL; ++i) P[(r0 + i) * kLd + c] = p[i];
        __syncwarp();
        float o[RPL];
#pragma unroll
        for (int i = 0; i < RPL; ++i) o[i] = 0.f;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
            float t[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) t[e] = P[(4 * k4 + e) * kLd + c];
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const float4 d = *reinterpret_cast<const float4*>(&TF[(16 * I + r0 + i) * kLd + 16 * I + 4 * k4]);
                o[i] += d.x * t[0] + d.y * t[1] + d.z * t[2] + d.w * t[3];
            }
        }
#pragma unroll
        for (int i = 0; i < RPL; ++i) TF[(16 * I + r0 + i) * kLd + c0 + c] = -o[i];
        __syncwarp();
    }
}

// grid (heads, n_seqs), block 288, two CTAs per SM
__global__ void __launch_bounds__(kG1Threads, 2)
la_chunk_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const float* __restrict__ g, const float* __restrict__ beta,
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
    float* AM = reinterpret_cast<float*>(sm + kOffR);                      // fp32 A, [64][kLd]
    float* TF = reinterpret_cast<float*>(sm + kOffR + 64 * kLd * 4);       // fp32 T, [64][kLd]; its tail reaches into the W tile, which is dead then

    const int h = blockIdx.x;
    const LaSeqMeta sq = seqs[blockIdx.y];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int n_chunks = (sq.count + kC - 1) / kC;
    if (n_chunks == 0) return;
    if (*reinterpret_cast<volatile int*>(error_word) != 0) return;   // an earlier CTA gave up: do not queue more bounded waits
    float* Sg = rec_layer + (size_t)sq.slot * rec_stride_slot + (size_t)h * kLaKd * kLaVd;

    if (tid == 0) {
        for (int i = 0; i < G_BAR_COUNT; ++i)
            mbar_init(bar(i), (i == G_B1 || i == G_B2 || i == G_B3 || i == G_OT_FREE) ? 256 : 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(smem_u32(tmem_slot), 256);
        tmem_relinquish();
        if (lane == 0) { tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v); }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // D3 = S^T (128 columns); X = D1, then W^T, then O^T (64 columns); Ut = U^T, then V_new^T (64 columns)
    const uint32_t tm_d3 = tmem, tm_x = tmem + 128, tm_ut = tmem + 192;

    if (warp == 8) {
        // ------------------------------ TMA + MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t id64 = umma_idesc(kFmtF16, 128, 64, 0, 0);
            constexpr uint32_t id64_amn = umma_idesc(kFmtF16, 128, 64, 1, 0);                    // A MN-major (a TMA tile as it came)
            constexpr uint32_t id64_bmn_neg = umma_idesc(kFmtF16, 128, 64, 0, 1) | (1u << 13);   // B MN-major, negated A
            constexpr uint32_t id_u = umma_idesc(kFmtF16, 128, 128, 0, 1);                       // B MN-major, N = 128
            auto load_chunk = [&](int c) {
                const int row = sq.row0 + c * kC;
                mbar_arrive_expect_tx(bar(G_FULL), 49152);
                for (int blk = 0; blk < 2; ++blk) {
                    tma_load_3d(base + kOffKQ + blk * 16384, &map_k, bar(G_FULL), blk * 64, h, row);
                    tma_load_3d(base + kOffKQ + blk * 16384 + 8192, &map_q, bar(G_FULL), blk * 64, h, row);
                    tma_load_3d(base + kOffV + blk * 8192, &map_v, bar(G_FULL), blk * 64, h, row);
                }
            };
            const uint32_t kq = base + kOffKQ;
            load_chunk(0);
            for (int c = 0; c < n_chunks; ++c) {
                const uint32_t par = c & 1;
                if (!mbar_wait(bar(G_FULL), par, abort_flag)) break;
                if (c > 0 && !mbar_wait(bar(G_OT_FREE), (c - 1) & 1, abort_flag)) break;   // O^T of chunk c-1 has left TMEM
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {   // (a) D1 = [K;Q] K^T
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    umma_f16(tm_x, umma_smem_desc(kq + off, 16, 1024), umma_smem_desc(kq + off, 16, 1024), id64, ks > 0 ? 1u : 0u);
                }
                umma_commit(bar(G_A_DONE));
                if (c + 1 < n_chunks) {            // the next chunk's tiles can only land after this chunk's last product: ask L2 for them now
                    const int row = sq.row0 + (c + 1) * kC;
                    for (int blk = 0; blk < 2; ++blk) {
                        tma_prefetch_l2_3d(&map_k, blk * 64, h, row);
                        tma_prefetch_l2_3d(&map_q, blk * 64, h, row);
                        tma_prefetch_l2_3d(&map_v, blk * 64, h, row);
                    }
                }
                if (!mbar_wait(bar(G_B1), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int hl = 0; hl < 2; ++hl)    // (uw): T diag(beta) and T diag(beta e^b) as hi + lo pairs
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint32_t acc = (hl > 0 || ks > 0) ? 1u : 0u;
                        umma_f16(tm_ut, umma_smem_desc(base + kOffV + ks * 2048, 8192, 1024),
                                 umma_smem_desc(base + kOffR + hl * 8192 + ks * 32, 16, 1024), id64_amn, acc);
                        umma_f16(tm_x, umma_smem_desc(kq + ks * 2048, 16384, 1024),
                                 umma_smem_desc(base + kOffR + 16384 + hl * 8192 + ks * 32, 16, 1024), id64_amn, acc);
                    }
                umma_commit(bar(G_C1));
                if (!mbar_wait(bar(G_B2), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {   // (ws) Ut -= S0^T W^T ; (o) Ot = S0^T (Q e^b)^T
                    const uint64_t a = umma_smem_desc(base + kOffR + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
                    umma_f16(tm_ut, a, umma_smem_desc(base + kOffW + ks * 2048, 8192, 1024), id64_bmn_neg, 1u);
                    umma_f16(tm_x, a, umma_smem_desc(kq + 8192 + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024), id64, ks > 0 ? 1u : 0u);
                }
                umma_commit(bar(G_C2));
                if (!mbar_wait(bar(G_B3), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {   // (o) Ot += V_new^T Mq^T ; (u) D3 += V_new^T (e^{b_C-b} K)
                    const uint64_t a = umma_smem_desc(base + kOffV + ks * 32, 16, 1024);
                    umma_f16(tm_x, a, umma_smem_desc(base + kOffMQ + ks * 32, 16, 1024), id64, 1u);
                    umma_f16(tm_d3, a, umma_smem_desc(kq + ks * 2048, 16384, 1024), id_u, 1u);
                }
                umma_commit(bar(G_C3));
                if (c + 1 < n_chunks) {            // every tile of this chunk has been read: fetch the next one
                    if (!mbar_wait(bar(G_C3), par, abort_flag)) break;
                    load_chunk(c + 1);
                }
            }
        }
    } else {
        // ------------------------------ compute warps ------------------------------
        const int r = tid & 127;     // TMEM lane: D1 row, value dim of Ut/Ot/D3, key dim of Wt; also this thread's tile row
        const int hf = tid >> 7;     // which 32 of the 64 token columns (or which half of the state columns) it handles
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        float* s_b = reinterpret_cast<float*>(sm + kOffSC);
        float* s_beta = s_b + 64;
        float* s_eb = s_b + 128;
        float* s_ebc = s_b + 192;
        unsigned char* kq = sm + kOffKQ;
        // D3 <- S^T from the state pool: lane vd = r, column kd
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
            const int ch = hf * 2 + cc;
            uint32_t sv[32];
#pragma unroll
            for (int c2 = 0; c2 < 32; ++c2) sv[c2] = __float_as_uint(Sg[(size_t)(ch * 32 + c2) * kLaVd + r]);
            tmem_st32(tm_d3 + lane_base + ch * 32, sv);
        }
        tmem_wait_st();
        bool ok = true;
        // Outputs of chunk cp: O^T (lane = value dim) -> out[token][head][vd]; the TMEM columns are released as soon as
        // they are in registers.
        auto store_out = [&](int cp, bool do_store) {
            const int tok0 = cp * kC;
            const int n_valid = min(kC, sq.count - tok0);
            uint32_t ov[32];
            tmem_ld32(tm_x + lane_base + hf * 32, ov);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(bar(G_OT_FREE));
            if (!do_store) return;
            float* obase = out + ((size_t)(sq.row0 + tok0 + hf * 32) * kLaHeads + h) * kLaVd + r;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (hf * 32 + j < n_valid) obase[(size_t)j * kLaHeads * kLaVd] = __uint_as_float(ov[j]);
        };
        for (int c = 0; c < n_chunks; ++c) {   // after a failed wait the warp keeps the barrier protocol going, without waiting or storing
            const uint32_t par = c & 1;
            const int tok0 = c * kC;
            const int n_valid = min(kC, sq.count - tok0);
            // this chunk's decay and beta values are requested before the wait on the previous chunk's tensor-core work:
            // warp 0, two consecutive tokens per lane
            float g0 = 0.f, g1 = 0.f, bt0 = 0.f, bt1 = 0.f;
            if (warp == 0) {
                const size_t gi = (size_t)(sq.row0 + tok0 + 2 * lane) * kLaHeads + h;
                if (2 * lane < n_valid) { g0 = g[gi]; bt0 = beta[gi]; }
                if (2 * lane + 1 < n_valid) { g1 = g[gi + kLaHeads]; bt1 = beta[gi + kLaHeads]; }
            }
            if (c > 0) {
                if (!mbar_wait_warp(bar(G_C3), (c - 1) & 1, abort_flag)) ok = false;
                tc_fence_after();
                store_out(c - 1, ok);
            }
            // ---- per-chunk scalars: b = cumsum(g), beta, e^b, e^{b_C - b}; padded tokens get g = 0, beta = 0 ----
            if (warp == 0) {
                float run = g0 + g1;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float t2 = __shfl_up_sync(0xffffffffu, run, o);
                    if (lane >= o) run += t2;
                }
                const float b1 = run, b0 = run - g1, b_last = __shfl_sync(0xffffffffu, run, 31);
                s_b[2 * lane] = b0; s_b[2 * lane + 1] = b1;
                s_beta[2 * lane] = bt0; s_beta[2 * lane + 1] = bt1;
                s_eb[2 * lane] = ex2_approx(b0 * kLog2e); s_eb[2 * lane + 1] = ex2_approx(b1 * kLog2e);
                s_ebc[2 * lane] = ex2_approx((b_last - b0) * kLog2e); s_ebc[2 * lane + 1] = ex2_approx((b_last - b1) * kLog2e);
            }
            named_sync_256();
            const float e_bc = ex2_approx(s_b[63] * kLog2e);
            // ---- D1 -> A matrix (rows 0-63) and masked, decayed Q K^T (rows 64-127); then Q *= e^b in place ----
            if (!mbar_wait_warp(bar(G_FULL), par, abort_flag)) ok = false;
            if (!mbar_wait_warp(bar(G_A_DONE), par, abort_flag)) ok = false;
            tc_fence_after();
            {
                uint32_t d1[32];
                tmem_ld32(tm_x + lane_base + hf * 32, d1);
                tmem_wait_ld();
                if (r < 64) {
                    const float bi = s_b[r], be = s_beta[r];
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) {
                        float a4[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = hf * 32 + j4 * 4 + e;
                            a4[e] = (j < r) ? be * ex2_approx((bi - s_b[j]) * kLog2e) * __uint_as_float(d1[j4 * 4 + e]) : 0.f;
                        }
                        *reinterpret_cast<float4*>(AM + r * kLd + hf * 32 + j4 * 4) = make_float4(a4[0], a4[1], a4[2], a4[3]);
                    }
                } else {
                    const int i = r - 64;
                    const float bi = s_b[i];
                    unsigned char* row_ptr = sm + kOffMQ + i * 128;
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j0 = hf * 32 + cc * 8 + 2 * e, j1 = j0 + 1;
                            const float m0 = (j0 <= i) ? ex2_approx((bi - s_b[j0]) * kLog2e) * __uint_as_float(d1[cc * 8 + 2 * e]) : 0.f;
                            const float m1 = (j1 <= i) ? ex2_approx((bi - s_b[j1]) * kLog2e) * __uint_as_float(d1[cc * 8 + 2 * e + 1]) : 0.f;
                            pk[e] = pack_half2(m0, m1);
                        }
                        *reinterpret_cast<uint4*>(row_ptr + (((hf * 4 + cc) ^ (i & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
                {   // Q tile rows (token i): every element times e^{b_i}; the swizzle only permutes 16-byte pieces inside a row
                    const int i = tid >> 2;
                    const float sc = s_eb[i];
#pragma unroll
                    for (int blk = 0; blk < 2; ++blk)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            uint4* p4 = reinterpret_cast<uint4*>(kq + blk * 16384 + 8192 + i * 128 + (((tid & 3) * 2 + e) << 4));
                            uint4 x = *p4;
                            __half2* hx = reinterpret_cast<__half2*>(&x);
#pragma unroll
                            for (int w2 = 0; w2 < 4; ++w2) {
                                const float2 f = __half22float2(hx[w2]);
                                hx[w2] = __floats2half2_rn(f.x * sc, f.y * sc);
                            }
                            *p4 = x;
                        }
                }
            }
            named_sync_256();
            // ---- T = (I + A)^-1, blocked 16 x 16.  Diagonal blocks by forward substitution (one thread per column); then
            //      every warp takes a group of columns of T and works down its block rows (solve_column_group): the four
            //      leftmost groups of 4 columns have the longest way (nine 16 x 16 x 4 products), the others less. ----
            if (tid < 64) {
                const int b0 = (tid >> 4) * 16, col = tid & 15;      // column `col` of diagonal block b0 / 16
                float t[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) t[i] = (i == col) ? 1.f : 0.f;
#pragma unroll
                for (int i = 1; i < 16; ++i) {
                    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                    for (int j = 0; j + 1 < i; j += 2) {
                        acc0 += AM[(b0 + i) * kLd + b0 + j] * t[j];
                        acc1 += AM[(b0 + i) * kLd + b0 + j + 1] * t[j + 1];
                    }
                    if (i & 1) acc0 += AM[(b0 + i) * kLd + b0 + i - 1] * t[i - 1];
                    t[i] -= acc0 + acc1;   // rows <= col keep their start value: A is strictly lower and t[j < col] = 0
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) TF[(b0 + i) * kLd + b0 + col] = t[i];
            }
            named_sync_256();
            if (warp < 4) solve_column_group<4>(AM, TF, 0, 4 * warp, lane);
            else if (warp < 6) solve_column_group<8>(AM, TF, 1, 16 + 8 * (warp - 4), lane);
            else solve_column_group<8>(AM, TF, 2, 32 + 8 * (warp - 6), lane);
            named_sync_256();
            {   // T diag(beta) and T diag(beta e^b) -> fp16 hi + lo tiles (row = i, K = j), written over A and T
                const int i = tid >> 2, qd = tid & 3;
                float tv[16];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float4 t4 = *reinterpret_cast<const float4*>(&TF[i * kLd + qd * 16 + 4 * e]);
                    if (qd > (i >> 4)) t4 = make_float4(0.f, 0.f, 0.f, 0.f);      // blocks above the diagonal are never written
                    tv[4 * e] = t4.x; tv[4 * e + 1] = t4.y; tv[4 * e + 2] = t4.z; tv[4 * e + 3] = t4.w;
                }
                named_sync_256();     // every thread holds its part of T: the tiles may overwrite it
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t uh[4], ul[4], wh[4], wl[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j0 = qd * 16 + cc * 8 + 2 * e, j1 = j0 + 1;
                        const float u0 = tv[cc * 8 + 2 * e] * s_beta[j0], u1 = tv[cc * 8 + 2 * e + 1] * s_beta[j1];
                        const float w0 = u0 * s_eb[j0], w1 = u1 * s_eb[j1];
                        const float uh0 = __half2float(__float2half_rn(u0)), uh1 = __half2float(__float2half_rn(u1));
                        const float wh0 = __half2float(__float2half_rn(w0)), wh1 = __half2float(__float2half_rn(w1));
                        uh[e] = pack_half2(uh0, uh1); ul[e] = pack_half2(u0 - uh0, u1 - uh1);
                        wh[e] = pack_half2(wh0, wh1); wl[e] = pack_half2(w0 - wh0, w1 - wh1);
                    }
                    const uint32_t o16 = i * 128 + (((qd * 2 + cc) ^ (i & 7)) << 4);
                    *reinterpret_cast<uint4*>(sm + kOffR + o16) = make_uint4(uh[0], uh[1], uh[2], uh[3]);
                    *reinterpret_cast<uint4*>(sm + kOffR + 8192 + o16) = make_uint4(ul[0], ul[1], ul[2], ul[3]);
                    *reinterpret_cast<uint4*>(sm + kOffR + 16384 + o16) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                    *reinterpret_cast<uint4*>(sm + kOffR + 24576 + o16) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(G_B1));
            // ======================= the part that needs the state of the chunk start =======================
            if (!mbar_wait_warp(bar(G_C1), par, abort_flag)) ok = false;    // (uw) is done: the T tiles are dead, W^T is in TMEM
            tc_fence_after();
            // ---- D3 (S^T of the chunk start) -> fp16 tile over the T tiles, and back to TMEM scaled by e^{b_C} ----
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                const int ch = hf * 2 + cc;
                uint32_t sv[32];
                tmem_ld32(tm_d3 + lane_base + ch * 32, sv);
                tmem_wait_ld();
                unsigned char* row_ptr = sm + kOffR + (ch >> 1) * 16384 + r * 128;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
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
            // ---- W^T (lane = key dim): row r of the W tile, this thread's 32 tokens ----
            {
                uint32_t wv[32];
                tmem_ld32(tm_x + lane_base + hf * 32, wv);
                tmem_wait_ld();
                unsigned char* w_row = sm + kOffW + r * 128;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t pk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        pk[e] = pack_half2(__uint_as_float(wv[cc * 8 + 2 * e]), __uint_as_float(wv[cc * 8 + 2 * e + 1]));
                    *reinterpret_cast<uint4*>(w_row + (((hf * 4 + cc) ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            }
            {   // K tile rows (token j): every element times e^{b_C - b_j} for the state update
                const int j = tid >> 2;
                const float sc = s_ebc[j];
#pragma unroll
                for (int blk = 0; blk < 2; ++blk)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        uint4* p4 = reinterpret_cast<uint4*>(kq + blk * 16384 + j * 128 + (((tid & 3) * 2 + e) << 4));
                        uint4 x = *p4;
                        __half2* hx = reinterpret_cast<__half2*>(&x);
#pragma unroll
                        for (int w2 = 0; w2 < 4; ++w2) {
                            const float2 f = __half22float2(hx[w2]);
                            hx[w2] = __floats2half2_rn(f.x * sc, f.y * sc);
                        }
                        *p4 = x;
                    }
            }
            tmem_wait_st();
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(G_B2));
            // ---- V_new^T (lane = value dim) -> fp16 rows over the V tile ----
            if (!mbar_wait_warp(bar(G_C2), par, abort_flag)) ok = false;
            tc_fence_after();
            {
                uint32_t uv[32];
                tmem_ld32(tm_ut + lane_base + hf * 32, uv);
                tmem_wait_ld();
                unsigned char* vn_row = sm + kOffV + r * 128;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t pa[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        pa[e] = pack_half2(__uint_as_float(uv[cc * 8 + 2 * e]), __uint_as_float(uv[cc * 8 + 2 * e + 1]));
                    *reinterpret_cast<uint4*>(vn_row + (((hf * 4 + cc) ^ (r & 7)) << 4)) = make_uint4(pa[0], pa[1], pa[2], pa[3]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(G_B3));
        }
        // ---- last chunk's outputs and the final state: D3 (S^T) -> state pool ----
        if (ok && mbar_wait_warp(bar(G_C3), (n_chunks - 1) & 1, abort_flag)) {
            tc_fence_after();
            store_out(n_chunks - 1, true);
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                const int ch = hf * 2 + cc;
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
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
    if (tid == 0 && *abort_flag) atomicExch(error_word, 6);
}

// q_h, k_h, v_h: fp16 [rows][16][128]; g, beta fp32 [rows][16].
int launch_la_chunk_tc(const __half* q_h, const __half* k_h, const __half* v_h, const float* g, const float* beta,
                       const LaSeqMeta* d_seqs, int n_seqs, int rows, float* rec_layer, size_t rec_stride, float* out,
                       int* d_error, cudaStream_t s) {
    CUtensorMap mq, mk, mv;
    const uint64_t dims[3] = {(uint64_t)kLaKd, (uint64_t)kLaHeads, (uint64_t)rows};
    const uint64_t str[2] = {(uint64_t)kLaKd * 2, (uint64_t)kLaHeads * kLaKd * 2};
    const uint32_t box[3] = {64, 1, (uint32_t)kC};
    B2_TRY(make_tensor_map(&mq, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, q_h, dims, str, box));
    B2_TRY(make_tensor_map(&mk, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, k_h, dims, str, box));
    B2_TRY(make_tensor_map(&mv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, v_h, dims, str, box));
    static PerDeviceOnce once;
    B2_PER_DEVICE_ONCE(once, B2_CUDA(cudaFuncSetAttribute(la_chunk_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kG1Smem)));
    dim3 grid(kLaHeads, n_seqs);
    la_chunk_tc_kernel<<<grid, kG1Threads, kG1Smem, s>>>(mq, mk, mv, g, beta, d_seqs, rec_layer, rec_stride, out, d_error);
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200
