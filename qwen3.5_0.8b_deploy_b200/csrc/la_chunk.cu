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
//
// The K / Q tiles and the 32 KB work region (fp32 A and T, then the T tiles, then the fp16 state tile) swap places from
// chunk to chunk: the work region of chunk c is dead once the products that read the state tile are done, long before
// the chunk ends, so the K and Q tiles of chunk c+1 are loaded into it then, and their product (a) is queued right
// behind the last product of chunk c (into the accumulator that held V_new, which is free by then).  A chunk therefore
// starts with (a) already computed.
#include "kernels.cuh"
#include "tc05.cuh"

namespace b200 {

constexpr int kC = 64;
// shared-memory map (bytes from a 1024-aligned base); regions are reused as their contents die during a chunk
constexpr uint32_t kOffX = 2048;      // 32 KB: K/Q tiles of even chunks, work region of odd chunks (whose fp32 part starts at 0)
constexpr uint32_t kOffV = 34816;     // 16 KB: V chunk [2 blocks of 64 value dims][64 tokens][128 B]
                                      //        -> after (uw): W^T [128 kd rows][64 tokens] fp16, B of (ws), MN-major
                                      //        -> after (ws): V_new^T [128 vd][64 tokens]
constexpr uint32_t kOffY = 51200;     // 32 KB + 2 KB: work region of even chunks, K/Q tiles of odd chunks
// K/Q tiles: [2 blocks of 64 key dims][rows 0-63 K chunk, rows 64-127 Q chunk][128 B]
// work region: fp32 A and T ([64][68] each, 34 KB: the odd chunks' copy starts 2 KB in front of X, the even chunks' copy
//              ends 2 KB behind Y)
//          ->  T diag(beta) hi, lo, T diag(beta e^b) hi, lo (four [64][64] fp16 tiles, in the 1024-aligned 32 KB)
//          ->  S0^T fp16 [2 blocks of 64 kd][128 vd rows][128 B]
constexpr uint32_t kOffMQ = 86016;    // Mq [64][64] fp16                                 B of (o)
constexpr uint32_t kOffSC = 94208;    // scalars: b[64], beta[64], eb[64], ebc[64]
constexpr uint32_t kOffBarG = 95232;
constexpr uint32_t kG1Smem = kOffBarG + 128 + 1024;
constexpr int kG1Threads = 288;
enum { G_FULL_KQ = 0, G_FULL_V, G_A_DONE, G_B1, G_C1, G_B2, G_C2, G_B3, G_C3, G_BAR_COUNT };

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

// Blocked inverse of the unit lower triangular I + A (64 x 64, blocks of 16).  With D_I the inverted diagonal blocks,
//     T_II = D_I,      T_IJ = - sum_{K=J}^{I-1} (D_I A_IK) T_KJ     (I > J).
// scale_blocks forms B_IK = D_I A_IK in place of A_IK (six independent 16 x 16 x 16 products, one warp each); then a
// column of T depends only on the same column of the block rows above it, so solve_column_group lets one warp own NC
// columns of block column J from top to bottom: it never meets another warp and needs one product per block row.

// warp w < 6 takes block (I, K) = (1,0) (2,0) (2,1) (3,0) (3,1) (3,2); lane = (half of the rows, column)
__device__ __forceinline__ void scale_blocks(float* AM, const float* TF, int w, int lane) {
    const int I = (w == 0) ? 1 : (w < 3 ? 2 : 3);
    const int K = (w == 0) ? 0 : (w < 3 ? w - 1 : w - 3);
    const int rh = lane >> 4, col = lane & 15;        // rows rh, rh + 2, ..: the two halves' D rows lie four banks apart
    float a[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) a[k] = AM[(16 * I + k) * kLd + 16 * K + col];
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float* drow = TF + (16 * I + 2 * i + rh) * kLd + 16 * I;
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
            const float4 d = *reinterpret_cast<const float4*>(drow + 4 * k4);    // entries above the diagonal are zero
            acc0 += d.x * a[4 * k4] + d.z * a[4 * k4 + 2];
            acc1 += d.y * a[4 * k4 + 1] + d.w * a[4 * k4 + 3];
        }
        o[i] = acc0 + acc1;
    }
    __syncwarp();                 // every lane holds its column of A_IK: the block may be overwritten
#pragma unroll
    for (int i = 0; i < 8; ++i) AM[(16 * I + 2 * i + rh) * kLd + 16 * K + col] = o[i];
}

// Lane (rg, c): rows rg, rg + 32 / NC, .. of a 16-row block (RPL = NC / 2 of them: neighbouring lanes' rows lie four
// banks apart), column c0 + c of block column J.
template <int NC, int J>
__device__ __forceinline__ void solve_column_group(const float* BM, float* TF, int c0, int lane) {
    constexpr int RPL = NC / 2, RS = 32 / NC;
    const int rg = lane / NC, c = lane % NC;
#pragma unroll
    for (int I = J + 1; I < 4; ++I) {
        float p[RPL];
#pragma unroll
        for (int i = 0; i < RPL; ++i) p[i] = 0.f;
#pragma unroll
        for (int K = J; K < I; ++K) {
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
                float t[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) t[e] = TF[(16 * K + 4 * k4 + e) * kLd + c0 + c];
#pragma unroll
                for (int i = 0; i < RPL; ++i) {
                    const float4 bq = *reinterpret_cast<const float4*>(&BM[(16 * I + rg + RS * i) * kLd + 16 * K + 4 * k4]);
                    p[i] += bq.x * t[0] + bq.y * t[1] + bq.z * t[2] + bq.w * t[3];
                }
            }
        }
#pragma unroll
        for (int i = 0; i < RPL; ++i) TF[(16 * I + rg + RS * i) * kLd + c0 + c] = -p[i];
        __syncwarp();             // the next block row reads these entries from other lanes of this warp
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

    const int h = blockIdx.x;
    const LaSeqMeta sq = seqs[blockIdx.y];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int n_chunks = (sq.count + kC - 1) / kC;
    if (n_chunks == 0) return;
    if (*reinterpret_cast<volatile int*>(error_word) != 0) return;   // an earlier CTA gave up: do not queue more bounded waits
    float* Sg = rec_layer + (size_t)sq.slot * rec_stride_slot + (size_t)h * kLaKd * kLaVd;

    if (tid == 0) {
        for (int i = 0; i < G_BAR_COUNT; ++i)
            mbar_init(bar(i), (i == G_B1 || i == G_B2 || i == G_B3) ? 256 : 1);
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
    // D3 = S^T (128 columns); X = W^T, then O^T (64 columns); Ut = D1, then U^T, then V_new^T (64 columns)
    const uint32_t tm_d3 = tmem, tm_x = tmem + 128, tm_ut = tmem + 192;

    if (warp == 8) {
        // ------------------------------ TMA + MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t id64 = umma_idesc(kFmtF16, 128, 64, 0, 0);
            constexpr uint32_t id64_amn = umma_idesc(kFmtF16, 128, 64, 1, 0);                    // A MN-major (a TMA tile as it came)
            constexpr uint32_t id64_bmn_neg = umma_idesc(kFmtF16, 128, 64, 0, 1) | (1u << 13);   // B MN-major, negated A
            constexpr uint32_t id_u = umma_idesc(kFmtF16, 128, 128, 0, 1);                       // B MN-major, N = 128
            auto load_kq = [&](int c) {
                const int row = sq.row0 + c * kC;
                const uint32_t dst = base + ((c & 1) ? kOffY : kOffX);
                mbar_arrive_expect_tx(bar(G_FULL_KQ), 32768);
                for (int blk = 0; blk < 2; ++blk) {
                    tma_load_3d(dst + blk * 16384, &map_k, bar(G_FULL_KQ), blk * 64, h, row);
                    tma_load_3d(dst + blk * 16384 + 8192, &map_q, bar(G_FULL_KQ), blk * 64, h, row);
                }
            };
            auto load_v = [&](int c) {
                const int row = sq.row0 + c * kC;
                mbar_arrive_expect_tx(bar(G_FULL_V), 16384);
                for (int blk = 0; blk < 2; ++blk) tma_load_3d(base + kOffV + blk * 8192, &map_v, bar(G_FULL_V), blk * 64, h, row);
            };
            auto issue_a = [&](int c) {            // (a) D1 = [K;Q] K^T of chunk c, into the Ut columns
                const uint32_t kq = base + ((c & 1) ? kOffY : kOffX);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    umma_f16(tm_ut, umma_smem_desc(kq + off, 16, 1024), umma_smem_desc(kq + off, 16, 1024), id64, ks > 0 ? 1u : 0u);
                }
                umma_commit(bar(G_A_DONE));
            };
            load_kq(0);
            load_v(0);
            bool ok = mbar_wait(bar(G_FULL_KQ), 0, abort_flag);
            if (ok) { tc_fence_after(); issue_a(0); }
            for (int c = 0; ok && c < n_chunks; ++c) {
                const uint32_t par = c & 1;
                const uint32_t kq = base + (par ? kOffY : kOffX);       // this chunk's K/Q tiles
                const uint32_t wr = base + (par ? kOffX : kOffY);       // this chunk's T tiles, then its state tile
                if (c > 0) {                        // V_new of chunk c-1 has been read by its last products: the V tile may land
                    if (!mbar_wait(bar(G_C3), (c - 1) & 1, abort_flag)) break;
                    load_v(c);
                }
                if (c + 1 < n_chunks) {             // ask L2 for the next chunk's tiles well ahead of their loads
                    const int row = sq.row0 + (c + 1) * kC;
                    for (int blk = 0; blk < 2; ++blk) {
                        tma_prefetch_l2_3d(&map_k, blk * 64, h, row);
                        tma_prefetch_l2_3d(&map_q, blk * 64, h, row);
                        tma_prefetch_l2_3d(&map_v, blk * 64, h, row);
                    }
                }
                if (!mbar_wait(bar(G_B1), par, abort_flag)) break;
                if (!mbar_wait(bar(G_FULL_V), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int hl = 0; hl < 2; ++hl)    // (uw): T diag(beta) and T diag(beta e^b) as hi + lo pairs
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint32_t acc = (hl > 0 || ks > 0) ? 1u : 0u;
                        umma_f16(tm_ut, umma_smem_desc(base + kOffV + ks * 2048, 8192, 1024),
                                 umma_smem_desc(wr + hl * 8192 + ks * 32, 16, 1024), id64_amn, acc);
                        umma_f16(tm_x, umma_smem_desc(kq + ks * 2048, 16384, 1024),
                                 umma_smem_desc(wr + 16384 + hl * 8192 + ks * 32, 16, 1024), id64_amn, acc);
                    }
                umma_commit(bar(G_C1));
                if (!mbar_wait(bar(G_B2), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {   // (ws) Ut -= S0^T W^T ; (o) Ot = S0^T (Q e^b)^T
                    const uint64_t a = umma_smem_desc(wr + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
                    umma_f16(tm_ut, a, umma_smem_desc(base + kOffV + ks * 2048, 8192, 1024), id64_bmn_neg, 1u);
                    umma_f16(tm_x, a, umma_smem_desc(kq + 8192 + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024), id64, ks > 0 ? 1u : 0u);
                }
                umma_commit(bar(G_C2));
                if (c + 1 < n_chunks) {            // the state tile is dead once these products are done: the next K/Q tiles go there
                    if (!mbar_wait(bar(G_C2), par, abort_flag)) break;
                    load_kq(c + 1);
                }
                if (!mbar_wait(bar(G_B3), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {   // (o) Ot += V_new^T Mq^T ; (u) D3 += V_new^T (e^{b_C-b} K)
                    const uint64_t a = umma_smem_desc(base + kOffV + ks * 32, 16, 1024);
                    umma_f16(tm_x, a, umma_smem_desc(base + kOffMQ + ks * 32, 16, 1024), id64, 1u);
                    umma_f16(tm_d3, a, umma_smem_desc(kq + ks * 2048, 16384, 1024), id_u, 1u);
                }
                umma_commit(bar(G_C3));
                if (c + 1 < n_chunks) {            // (a) of the next chunk runs right behind; V_new has left the Ut columns
                    if (!mbar_wait(bar(G_FULL_KQ), (c + 1) & 1, abort_flag)) break;
                    tc_fence_after();
                    issue_a(c + 1);
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
        // Outputs of chunk cp: O^T (lane = value dim) -> out[token][head][vd]
        auto store_out = [&](int cp, bool do_store) {
            const int tok0 = cp * kC;
            const int n_valid = min(kC, sq.count - tok0);
            uint32_t ov[32];
            tmem_ld32(tm_x + lane_base + hf * 32, ov);
            tmem_wait_ld();
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
            unsigned char* kq = sm + (par ? kOffY : kOffX);                        // K/Q tiles of this chunk
            float* AM = reinterpret_cast<float*>(sm + (par ? 0u : kOffY));         // fp32 A, [64][kLd]
            float* TF = AM + 64 * kLd;                                             // fp32 T, [64][kLd]
            unsigned char* wr = sm + (par ? kOffX : kOffY);                        // T tiles, then the state tile
            // this chunk's decay and beta values are requested before the wait on the previous chunk's tensor-core work:
            // warp 0, two consecutive tokens per lane
            float g0 = 0.f, g1 = 0.f, bt0 = 0.f, bt1 = 0.f;
            if (warp == 0) {
                const size_t gi = (size_t)(sq.row0 + tok0 + 2 * lane) * kLaHeads + h;
                if (2 * lane < n_valid) { g0 = g[gi]; bt0 = beta[gi]; }
                if (2 * lane + 1 < n_valid) { g1 = g[gi + kLaHeads]; bt1 = beta[gi + kLaHeads]; }
            }
            if (c > 0) {      // the previous chunk's last products: its outputs are complete, its K/Q tiles and Mq are dead
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
            // ---- D1 -> A matrix (rows 0-63) and masked, decayed Q K^T (rows 64-127) ----
            if (!mbar_wait_warp(bar(G_FULL_KQ), par, abort_flag)) ok = false;      // the tiles are visible to this thread too
            if (!mbar_wait_warp(bar(G_A_DONE), par, abort_flag)) ok = false;
            tc_fence_after();
            {
                uint32_t d1[32];
                tmem_ld32(tm_ut + lane_base + hf * 32, d1);
                tmem_wait_ld();
                if (r < 64) {
                    const float bi = s_b[r], be = s_beta[r];
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) {
                        float a4[4];
                        const float4 bj4 = *reinterpret_cast<const float4*>(&s_b[hf * 32 + j4 * 4]);
                        const float bj[4] = {bj4.x, bj4.y, bj4.z, bj4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = hf * 32 + j4 * 4 + e;
                            a4[e] = (j < r) ? be * ex2_approx((bi - bj[e]) * kLog2e) * __uint_as_float(d1[j4 * 4 + e]) : 0.f;
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
                        const float4 bl = *reinterpret_cast<const float4*>(&s_b[hf * 32 + cc * 8]);
                        const float4 bh = *reinterpret_cast<const float4*>(&s_b[hf * 32 + cc * 8 + 4]);
                        const float bj[8] = {bl.x, bl.y, bl.z, bl.w, bh.x, bh.y, bh.z, bh.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j0 = hf * 32 + cc * 8 + 2 * e, j1 = j0 + 1;
                            const float m0 = (j0 <= i) ? ex2_approx((bi - bj[2 * e]) * kLog2e) * __uint_as_float(d1[cc * 8 + 2 * e]) : 0.f;
                            const float m1 = (j1 <= i) ? ex2_approx((bi - bj[2 * e + 1]) * kLog2e) * __uint_as_float(d1[cc * 8 + 2 * e + 1]) : 0.f;
                            pk[e] = pack_half2(m0, m1);
                        }
                        *reinterpret_cast<uint4*>(row_ptr + (((hf * 4 + cc) ^ (i & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
            }
            named_sync_256();
            // ---- T = (I + A)^-1, blocked 16 x 16.  Two warps invert the diagonal blocks by forward substitution (one
            //      thread per column); meanwhile the other six scale the Q tile: every element of row i times e^{b_i}
            //      (the swizzle only permutes 16-byte pieces inside a row). ----
            if (tid < 64) {
                const int b0 = (tid >> 4) * 16, col = tid & 15;      // column `col` of diagonal block b0 / 16
                float t[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) t[i] = (i == col) ? 1.f : 0.f;
#pragma unroll
                for (int i = 1; i < 16; ++i) {
                    const float* arow = AM + (b0 + i) * kLd + b0;
                    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                    for (int j4 = 0; 4 * j4 < i; ++j4) {
                        const float4 a4 = *reinterpret_cast<const float4*>(arow + 4 * j4);   // entries at and above the diagonal are zero
                        acc0 += a4.x * t[4 * j4] + a4.z * t[4 * j4 + 2];
                        acc1 += a4.y * t[4 * j4 + 1] + a4.w * t[4 * j4 + 3];
                    }
                    t[i] -= acc0 + acc1;   // rows <= col keep their start value: A is strictly lower and t[j < col] = 0
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) TF[(b0 + i) * kLd + b0 + col] = t[i];
            } else {
                for (int idx = tid - 64; idx < 1024; idx += 192) {
                    const int blk = idx >> 9, i = (idx >> 3) & 63;
                    const float sc = s_eb[i];
                    uint4* p4 = reinterpret_cast<uint4*>(kq + blk * 16384 + 8192 + i * 128 + ((idx & 7) << 4));
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
            named_sync_256();
            if (warp < 6) scale_blocks(AM, TF, warp, lane);
            named_sync_256();
            // every warp takes a group of columns of T and works down its block rows: the four leftmost groups of 4 columns
            // have the longest way (six 16 x 16 x 4 products), the others less
            if (warp < 4) solve_column_group<4, 0>(AM, TF, 4 * warp, lane);
            else if (warp < 6) solve_column_group<8, 1>(AM, TF, 16 + 8 * (warp - 4), lane);
            else solve_column_group<8, 2>(AM, TF, 32 + 8 * (warp - 6), lane);
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
                float bt[16], ebv[16];       // beta_j and e^{b_j} of this thread's 16 columns
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float4 b4 = *reinterpret_cast<const float4*>(&s_beta[qd * 16 + 4 * e]);
                    const float4 e4 = *reinterpret_cast<const float4*>(&s_eb[qd * 16 + 4 * e]);
                    bt[4 * e] = b4.x; bt[4 * e + 1] = b4.y; bt[4 * e + 2] = b4.z; bt[4 * e + 3] = b4.w;
                    ebv[4 * e] = e4.x; ebv[4 * e + 1] = e4.y; ebv[4 * e + 2] = e4.z; ebv[4 * e + 3] = e4.w;
                }
                named_sync_256();     // every thread holds its part of T: the tiles may overwrite it
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t uh[4], ul[4], wh[4], wl[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float u0 = tv[cc * 8 + 2 * e] * bt[cc * 8 + 2 * e], u1 = tv[cc * 8 + 2 * e + 1] * bt[cc * 8 + 2 * e + 1];
                        const float w0 = u0 * ebv[cc * 8 + 2 * e], w1 = u1 * ebv[cc * 8 + 2 * e + 1];
                        const float uh0 = __half2float(__float2half_rn(u0)), uh1 = __half2float(__float2half_rn(u1));
                        const float wh0 = __half2float(__float2half_rn(w0)), wh1 = __half2float(__float2half_rn(w1));
                        uh[e] = pack_half2(uh0, uh1); ul[e] = pack_half2(u0 - uh0, u1 - uh1);
                        wh[e] = pack_half2(wh0, wh1); wl[e] = pack_half2(w0 - wh0, w1 - wh1);
                    }
                    const uint32_t o16 = i * 128 + (((qd * 2 + cc) ^ (i & 7)) << 4);
                    *reinterpret_cast<uint4*>(wr + o16) = make_uint4(uh[0], uh[1], uh[2], uh[3]);
                    *reinterpret_cast<uint4*>(wr + 8192 + o16) = make_uint4(ul[0], ul[1], ul[2], ul[3]);
                    *reinterpret_cast<uint4*>(wr + 16384 + o16) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                    *reinterpret_cast<uint4*>(wr + 24576 + o16) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(G_B1));
            // ======================= the part that needs the state of the chunk start =======================
            if (!mbar_wait_warp(bar(G_C1), par, abort_flag)) ok = false;    // (uw) is done: the T tiles and the V chunk are dead, W^T is in TMEM
            tc_fence_after();
            // ---- D3 (S^T of the chunk start) -> fp16 tile over the T tiles, and back to TMEM scaled by e^{b_C} ----
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                const int ch = hf * 2 + cc;
                uint32_t sv[32];
                tmem_ld32(tm_d3 + lane_base + ch * 32, sv);
                tmem_wait_ld();
                unsigned char* row_ptr = wr + (ch >> 1) * 16384 + r * 128;
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
            // ---- W^T (lane = key dim): row r of the W tile (over the V chunk), this thread's 32 tokens ----
            {
                uint32_t wv[32];
                tmem_ld32(tm_x + lane_base + hf * 32, wv);
                tmem_wait_ld();
                unsigned char* w_row = sm + kOffV + r * 128;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t pk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        pk[e] = pack_half2(__uint_as_float(wv[cc * 8 + 2 * e]), __uint_as_float(wv[cc * 8 + 2 * e + 1]));
                    *reinterpret_cast<uint4*>(w_row + (((hf * 4 + cc) ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            }
            // K tile rows (token j): every element times e^{b_C - b_j} for the state update; consecutive threads take
            // consecutive 16-byte pieces
            for (int idx = tid; idx < 1024; idx += 256) {
                const int blk = idx >> 9, j = (idx >> 3) & 63;
                const float sc = s_ebc[j];
                uint4* p4 = reinterpret_cast<uint4*>(kq + blk * 16384 + j * 128 + ((idx & 7) << 4));
                uint4 x = *p4;
                __half2* hx = reinterpret_cast<__half2*>(&x);
#pragma unroll
                for (int w2 = 0; w2 < 4; ++w2) {
                    const float2 f = __half22float2(hx[w2]);
                    hx[w2] = __floats2half2_rn(f.x * sc, f.y * sc);
                }
                *p4 = x;
            }
            tmem_wait_st();
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(G_B2));
            // ---- V_new^T (lane = value dim) -> fp16 rows over the W tile ----
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
