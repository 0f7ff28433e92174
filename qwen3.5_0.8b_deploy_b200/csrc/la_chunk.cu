// G1: chunk-64 gated delta rule (WY / UT form) on tcgen05 tensor cores.
//
// One CTA per (sequence, head) walks the sequence in chunks of C = 64 tokens.  With b_i the running sum of
// the log decays g inside the chunk and S0 the state at the chunk start, the serial recurrence
//     S_i = e^{g_i} S_{i-1} + k_i (x) beta_i (v_i - (e^{g_i} S_{i-1})^T k_i),   o_i = S_i^T q_i
// (src/backend/cpu/core/attention/language_linear_attn.cpp:206-240 in the reference; its CUDA form is the
// token-serial gated_delta_batch_fused_v2_kernel, linear_attention_v2.cu:492-595) is equivalent to
//     A_ij  = beta_i e^{b_i-b_j} (k_i.k_j)  (j < i),     T = (I + A)^-1
//     U     = T (beta V),   W = T (beta e^{b} K),        V_new = U - W S0
//     O     = (Q e^{b}) S0 + tril(e^{b_i-b_j} (q_i.k_j)) V_new
//     S_C   = e^{b_C} S0 + K^T (e^{b_C-b} V_new)
// Every decay factor is formed as exp(b_i - b_j) with i >= j, never as a quotient of products.
//
// All state-sized objects are kept TRANSPOSED in TMEM (lane = value dim or key dim, column = token), so every
// tensor-core product has M = 128 and every tile a thread writes is one of its own rows:
//   (a)  D1  [128 x 64] = [K ; Q] K^T                         rows 0-63: K K^T, rows 64-127: Q K^T
//   (uw) Ut  [vd x 64]  = (beta V)^T T^T,   Wt [kd x 64] = (beta e^b K)^T T^T     (T as an fp16 hi + lo pair)
//   (ws) Ut -= S0^T W^T                                        -> V_new^T, accumulated in place (negated A operand)
//   (o)  Ot  [vd x 64]  = S0^T (Q e^b)^T + V_new^T Mq^T       (Q is scaled in place in its TMA tile)
//   (u)  D3  [vd x kd]  = e^{b_C} D3 + (e^{b_C-b} V_new)^T K  D3 holds S^T for the whole sequence
// tcgen05.mma kind::f16: fp16 operands (the same 10-bit mantissa as tf32), fp32 accumulation; 128-byte swizzle.
// T itself is built in fp32 in shared memory by a blocked inverse (16 x 16 blocks) on the CUDA cores.
//
// Eight compute warps (two threads per TMEM lane, each owning half of the 64 token columns) and one warp that
// issues TMA loads (K/Q tiles double-buffered) and MMAs.  The chunk is split in a front half that does not need
// the state (scalars, A, T, operand tiles -> B1) and a back half (S0 tile, W, V_new -> B2, B3); the front half of
// chunk c+1 runs while the tensor core finishes (o) and (u) of chunk c, whose outputs are stored one chunk late.
// All waits are bounded.
#include "kernels.cuh"
#include "tc05.cuh"

namespace b200 {

constexpr int kC = 64;
// shared-memory map (bytes from a 1024-aligned base)
constexpr uint32_t kOffKQ = 0;        // 2 buffers x [2 blocks][128 rows][128 B]: rows 0-63 K chunk, rows 64-127 Q chunk
constexpr uint32_t kOffAM = 65536;    // fp32 A [64][64]; its (zero) upper blocks double as scratch of the inverse
constexpr uint32_t kOffTF = 81920;    // fp32 T [64][64]
constexpr uint32_t kOffST = 65536;    // S0^T fp16 [2 blocks (64 kd)][128 vd rows][128 B], over A / T once T is converted
constexpr uint32_t kOffRV = 98304;    // (beta V)^T [128 vd rows][64 tokens]            A of (uw)
constexpr uint32_t kOffRK = 114688;   // (beta e^b K)^T [128 kd rows][64 tokens]        A of (uw)
constexpr uint32_t kOffVN = 131072;   // V_new^T [128 vd rows][64 tokens]               A of (o)
constexpr uint32_t kOffVS = 147456;   // (e^{b_C-b} V_new)^T                            A of (u)
constexpr uint32_t kOffTT = 163840;   // T hi [64][64] fp16, then T lo                  B of (uw)
constexpr uint32_t kOffWT = 163840;   // W [2 blocks][64 token rows][128 B], over T     B of (ws)
constexpr uint32_t kOffMQ = 180224;   // 2 buffers x Mq [64][64] fp16                   B of (o)
constexpr uint32_t kOffSC = 196608;   // 2 buffers x scalars: b[64], beta[64], eb[64], ebc[64]
constexpr uint32_t kOffBarG = 198656;
constexpr uint32_t kG1Smem = kOffBarG + 128 + 1024;
constexpr int kG1Threads = 288;
enum { G_KQ_FULL0 = 0, G_KQ_FULL1, G_A_DONE, G_B1, G_C1, G_B2, G_C2, G_B3, G_C3, G_BAR_COUNT };

__device__ __forceinline__ void named_sync_256() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// 2^x on the special-function unit (about 2 ulp); the decay matrices need 64 x 64 of them per chunk and head.
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr float kLog2e = 1.4426950408889634f;

// dst(16x16 block at dr,dc) (+)= sign * A(16x16 at ar,ac) * B(16x16 at br,bc); matrices 64x64 fp32 row-major in
// shared memory; 256 threads, one output each.
__device__ __forceinline__ void block_product(float* dst, int dr, int dc, const float* A, int ar, int ac, const float* B,
                                              int br, int bc, float sign, bool accumulate, int tid) {
    const int r = tid >> 4, c = tid & 15;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int k = 0; k < 16; k += 2) {
        s0 += A[(ar + r) * 64 + ac + k] * B[(br + k) * 64 + bc + c];
        s1 += A[(ar + r) * 64 + ac + k + 1] * B[(br + k + 1) * 64 + bc + c];
    }
    float* d = &dst[(dr + r) * 64 + dc + c];
    const float v = sign * (s0 + s1);
    *d = accumulate ? *d + v : v;
}

// grid (heads, n_seqs), block 288
__global__ void __launch_bounds__(kG1Threads, 1)
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
    float* AM = reinterpret_cast<float*>(sm + kOffAM);
    float* TF = reinterpret_cast<float*>(sm + kOffTF);

    const int h = blockIdx.x;
    const LaSeqMeta sq = seqs[blockIdx.y];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int n_chunks = (sq.count + kC - 1) / kC;
    if (n_chunks == 0) return;
    if (*reinterpret_cast<volatile int*>(error_word) != 0) return;   // an earlier CTA gave up: do not queue more bounded waits
    float* Sg = rec_layer + (size_t)sq.slot * rec_stride_slot + (size_t)h * kLaKd * kLaVd;

    if (tid == 0) {
        for (int i = 0; i < G_BAR_COUNT; ++i) mbar_init(bar(i), (i == G_B1 || i == G_B2 || i == G_B3) ? 256 : 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
        if (lane == 0) { tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tm_d1 = tmem, tm_ut = tmem + 64, tm_wt = tmem + 128, tm_ot = tmem + 192, tm_d3 = tmem + 256;

    if (warp == 8) {
        // ------------------------------ TMA + MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t id64 = umma_idesc(kFmtF16, 128, 64, 0, 0);
            constexpr uint32_t id64_neg = id64 | (1u << 13);                  // negated A operand
            constexpr uint32_t id_u = umma_idesc(kFmtF16, 128, 128, 0, 1);    // B MN-major, N = 128
            auto load_kq = [&](int c) {
                const uint32_t dst = base + kOffKQ + (c & 1) * 32768;
                const uint32_t fb = bar(G_KQ_FULL0 + (c & 1));
                const int row = sq.row0 + c * kC;
                mbar_arrive_expect_tx(fb, 32768);
                for (int blk = 0; blk < 2; ++blk) {
                    tma_load_3d(dst + blk * 16384, &map_k, fb, blk * 64, h, row);
                    tma_load_3d(dst + blk * 16384 + 8192, &map_q, fb, blk * 64, h, row);
                }
            };
            load_kq(0);
            for (int c = 0; c < n_chunks; ++c) {
                const uint32_t par = c & 1;
                const uint32_t kq = base + kOffKQ + (c & 1) * 32768;
                if (!mbar_wait(bar(G_KQ_FULL0 + (c & 1)), (c >> 1) & 1, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {   // (a) D1 = [K;Q] K^T
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    umma_f16(tm_d1, umma_smem_desc(kq + off, 16, 1024), umma_smem_desc(kq + off, 16, 1024), id64, ks > 0 ? 1u : 0u);
                }
                umma_commit(bar(G_A_DONE));
                // the other K/Q buffer was last read by (o) and (u) of chunk c-1 (its threads were done with it before B2)
                if (c + 1 < n_chunks) {
                    if (c >= 1 && !mbar_wait(bar(G_C3), (c - 1) & 1, abort_flag)) break;
                    load_kq(c + 1);
                }
                if (!mbar_wait(bar(G_B1), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int hl = 0; hl < 2; ++hl)    // (uw) with T = hi + lo
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t bt = umma_smem_desc(base + kOffTT + hl * 8192 + ks * 32, 16, 1024);
                        umma_f16(tm_ut, umma_smem_desc(base + kOffRV + ks * 32, 16, 1024), bt, id64, (hl > 0 || ks > 0) ? 1u : 0u);
                        umma_f16(tm_wt, umma_smem_desc(base + kOffRK + ks * 32, 16, 1024), bt, id64, (hl > 0 || ks > 0) ? 1u : 0u);
                    }
                umma_commit(bar(G_C1));
                if (!mbar_wait(bar(G_B2), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {   // (ws) Ut -= S0^T W^T ; (o) Ot = S0^T (Q e^b)^T
                    const uint64_t a = umma_smem_desc(base + kOffST + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
                    umma_f16(tm_ut, a, umma_smem_desc(base + kOffWT + (ks >> 2) * 8192 + (ks & 3) * 32, 16, 1024), id64_neg, 1u);
                    umma_f16(tm_ot, a, umma_smem_desc(kq + 8192 + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024), id64, ks > 0 ? 1u : 0u);
                }
                umma_commit(bar(G_C2));
                if (!mbar_wait(bar(G_B3), par, abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {   // (o) Ot += V_new^T Mq^T ; (u) D3 += (e^{b_C-b} V_new)^T K
                    umma_f16(tm_ot, umma_smem_desc(base + kOffVN + ks * 32, 16, 1024),
                             umma_smem_desc(base + kOffMQ + (c & 1) * 8192 + ks * 32, 16, 1024), id64, 1u);
                    umma_f16(tm_d3, umma_smem_desc(base + kOffVS + ks * 32, 16, 1024), umma_smem_desc(kq + ks * 2048, 16384, 1024),
                             id_u, 1u);
                }
                umma_commit(bar(G_C3));
            }
        }
    } else {
        // ------------------------------ compute warps ------------------------------
        const int r = tid & 127;     // TMEM lane: D1 row, value dim of Ut/Ot/D3, key dim of Wt; also this thread's tile row
        const int hf = tid >> 7;     // which 32 of the 64 token columns (or which half of the state columns) it handles
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
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
        // stores the outputs of chunk cp (Ot, lane = value dim) -> out[token][head][vd]
        auto store_out = [&](int cp) {
            const int tok0 = cp * kC;
            const int n_valid = min(kC, sq.count - tok0);
            uint32_t ov[32];
            tmem_ld32(tm_ot + lane_base + hf * 32, ov);
            tmem_wait_ld();
            float* obase = out + ((size_t)(sq.row0 + tok0 + hf * 32) * kLaHeads + h) * kLaVd + r;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (hf * 32 + j < n_valid) obase[(size_t)j * kLaHeads * kLaVd] = __uint_as_float(ov[j]);
        };
        bool ok = true;
        for (int c = 0; c < n_chunks; ++c) {   // after a failed wait the warp keeps the barrier protocol going, without waiting or storing
            const uint32_t par = c & 1, prev = (c - 1) & 1;
            const int tok0 = c * kC;
            const int n_valid = min(kC, sq.count - tok0);
            unsigned char* kq = sm + kOffKQ + (c & 1) * 32768;
            float* s_b = reinterpret_cast<float*>(sm + kOffSC) + (c & 1) * 256;
            float* s_beta = s_b + 64;
            float* s_eb = s_b + 128;
            float* s_ebc = s_b + 192;
            // ======================= front half: needs nothing of the state =======================
            // ---- per-chunk scalars: b = cumsum(g), beta; padded tokens get g = 0, beta = 0 ----
            if (tid < 64) {
                const bool val = tid < n_valid;
                const size_t gi = (size_t)(sq.row0 + tok0 + tid) * kLaHeads + h;
                float gv = val ? g[gi] : 0.f;
                const float bv = val ? beta[gi] : 0.f;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float t2 = __shfl_up_sync(0xffffffffu, gv, o);
                    if (lane >= o) gv += t2;
                }
                s_b[tid] = gv;
                s_beta[tid] = bv;
            }
            named_sync_256();
            if (warp == 1) s_b[tid] += s_b[31];
            named_sync_256();
            if (tid < 64) {
                s_eb[tid] = ex2_approx(s_b[tid] * kLog2e);
                s_ebc[tid] = ex2_approx((s_b[63] - s_b[tid]) * kLog2e);
            }
            named_sync_256();
            const float e_bc = ex2_approx(s_b[63] * kLog2e);
            // ---- this thread's half column of beta V ----
            float vcol[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int tk = hf * 32 + i;
                vcol[i] = (tk < n_valid) ? s_beta[tk] * v[((size_t)(sq.row0 + tok0 + tk) * kLaHeads + h) * kLaVd + r] : 0.f;
            }
            // ---- (beta V)^T row r and (beta e^b K)^T row r, tokens of this half ----
            if (!mbar_wait_warp(bar(G_KQ_FULL0 + (c & 1)), (c >> 1) & 1, abort_flag)) ok = false;
            {
                const unsigned char* kq_blk = kq + (r >> 6) * 16384;
                const int tcol = r & 63;
                unsigned char* rv_row = sm + kOffRV + r * 128;
                unsigned char* rk_row = sm + kOffRK + r * 128;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const int c8 = hf * 4 + cc;
                    uint32_t pv[4], pk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int l0 = cc * 8 + 2 * e;                 // index into vcol
                        const int i0 = c8 * 8 + 2 * e, i1 = i0 + 1;    // token
                        const uint32_t sw0 = (((tcol >> 3) ^ (i0 & 7)) << 4) + (tcol & 7) * 2;
                        const uint32_t sw1 = (((tcol >> 3) ^ (i1 & 7)) << 4) + (tcol & 7) * 2;
                        const float k0 = __half2float(*reinterpret_cast<const __half*>(kq_blk + i0 * 128 + sw0));
                        const float k1 = __half2float(*reinterpret_cast<const __half*>(kq_blk + i1 * 128 + sw1));
                        pv[e] = pack_half2(vcol[l0], vcol[l0 + 1]);
                        pk[e] = pack_half2(s_beta[i0] * s_eb[i0] * k0, s_beta[i1] * s_eb[i1] * k1);
                    }
                    *reinterpret_cast<uint4*>(rv_row + ((c8 ^ (r & 7)) << 4)) = make_uint4(pv[0], pv[1], pv[2], pv[3]);
                    *reinterpret_cast<uint4*>(rk_row + ((c8 ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            }
            // ---- D1 -> A matrix (rows 0-63) and masked, decayed Q K^T (rows 64-127); then Q *= e^b in place ----
            if (!mbar_wait_warp(bar(G_A_DONE), par, abort_flag)) ok = false;
            tc_fence_after();
            {
                uint32_t d1[32];
                tmem_ld32(tm_d1 + lane_base + hf * 32, d1);
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
                        *reinterpret_cast<float4*>(AM + r * 64 + hf * 32 + j4 * 4) = make_float4(a4[0], a4[1], a4[2], a4[3]);
                    }
                } else {
                    const int i = r - 64;
                    const float bi = s_b[i];
                    unsigned char* row_ptr = sm + kOffMQ + (c & 1) * 8192 + i * 128;
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
            // ---- T = (I + A)^-1, blocked 16 x 16: diagonal blocks by forward substitution, the rest by block products
            //      T_ij = -T_ii sum_{k=j}^{i-1} A_ik T_kj.  The inner sums are staged in A's upper blocks, which are zero
            //      and not otherwise used. ----
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
                        acc0 += AM[(b0 + i) * 64 + b0 + j] * t[j];
                        acc1 += AM[(b0 + i) * 64 + b0 + j + 1] * t[j + 1];
                    }
                    if (i & 1) acc0 += AM[(b0 + i) * 64 + b0 + i - 1] * t[i - 1];
                    t[i] -= acc0 + acc1;   // rows <= col keep their start value: A is strictly lower and t[j < col] = 0
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) TF[(b0 + i) * 64 + b0 + col] = t[i];
            } else {
                for (int idx = tid - 64; idx < 6 * 256; idx += 192) {   // the other threads clear T's six upper blocks
                    const int blk = idx >> 8, e = idx & 255;
                    const int bi = (blk < 3) ? 0 : (blk < 5 ? 1 : 2);
                    const int bj = (blk < 3) ? blk + 1 : (blk < 5 ? blk - 1 : 3);
                    TF[(bi * 16 + (e >> 4)) * 64 + bj * 16 + (e & 15)] = 0.f;
                }
            }
            named_sync_256();
            for (int i = 1; i < 4; ++i)   // first sub-diagonal
                block_product(AM, (i - 1) * 16, i * 16, AM, i * 16, (i - 1) * 16, TF, (i - 1) * 16, (i - 1) * 16, 1.f, false, tid);
            named_sync_256();
            for (int i = 1; i < 4; ++i)
                block_product(TF, i * 16, (i - 1) * 16, TF, i * 16, i * 16, AM, (i - 1) * 16, i * 16, -1.f, false, tid);
            named_sync_256();
            for (int i = 2; i < 4; ++i) {   // second sub-diagonal
                block_product(AM, (i - 2) * 16, i * 16, AM, i * 16, (i - 2) * 16, TF, (i - 2) * 16, (i - 2) * 16, 1.f, false, tid);
                block_product(AM, (i - 2) * 16, i * 16, AM, i * 16, (i - 1) * 16, TF, (i - 1) * 16, (i - 2) * 16, 1.f, true, tid);
            }
            named_sync_256();
            for (int i = 2; i < 4; ++i)
                block_product(TF, i * 16, (i - 2) * 16, TF, i * 16, i * 16, AM, (i - 2) * 16, i * 16, -1.f, false, tid);
            named_sync_256();
            block_product(AM, 0, 48, AM, 48, 0, TF, 0, 0, 1.f, false, tid);      // corner block
            block_product(AM, 0, 48, AM, 48, 16, TF, 16, 0, 1.f, true, tid);
            block_product(AM, 0, 48, AM, 48, 32, TF, 32, 0, 1.f, true, tid);
            named_sync_256();
            block_product(TF, 48, 0, TF, 48, 48, AM, 0, 48, -1.f, false, tid);
            named_sync_256();
            {   // T -> fp16 hi + lo tiles (row = i, K = j)
                const int i = tid >> 2, qd = tid & 3;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t ph[4], pl[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 t2 = *reinterpret_cast<const float2*>(&TF[i * 64 + qd * 16 + cc * 8 + 2 * e]);
                        const float h0 = __half2float(__float2half_rn(t2.x)), h1 = __half2float(__float2half_rn(t2.y));
                        ph[e] = pack_half2(h0, h1);
                        pl[e] = pack_half2(t2.x - h0, t2.y - h1);
                    }
                    const int chunk16 = qd * 2 + cc;
                    *reinterpret_cast<uint4*>(sm + kOffTT + i * 128 + ((chunk16 ^ (i & 7)) << 4)) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
                    *reinterpret_cast<uint4*>(sm + kOffTT + 8192 + i * 128 + ((chunk16 ^ (i & 7)) << 4)) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(G_B1));
            named_sync_256();     // every thread is done reading A / T: their space becomes the S0 tile below
            // ======================= back half: needs the state of the chunk start =======================
            if (c > 0) {
                if (!mbar_wait_warp(bar(G_C3), prev, abort_flag)) ok = false;
                tc_fence_after();
                if (ok) store_out(c - 1);
            }
            // ---- D3 (S^T of the chunk start) -> fp16 tile, and back to TMEM scaled by e^{b_C} ----
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                const int ch = hf * 2 + cc;
                uint32_t sv[32];
                tmem_ld32(tm_d3 + lane_base + ch * 32, sv);
                tmem_wait_ld();
                unsigned char* row_ptr = sm + kOffST + (ch >> 1) * 16384 + r * 128;
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
            tmem_wait_st();
            // ---- W^T (lane = key dim) -> column r of the W tile (over T, which (uw) has finished reading) ----
            if (!mbar_wait_warp(bar(G_C1), par, abort_flag)) ok = false;
            tc_fence_after();
            {
                uint32_t wv[32];
                tmem_ld32(tm_wt + lane_base + hf * 32, wv);
                tmem_wait_ld();
                unsigned char* wt_blk = sm + kOffWT + (r >> 6) * 8192;
                const int tcol = r & 63;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int i = hf * 32 + j;
                    const __half hv = __float2half_rn(__uint_as_float(wv[j]));
                    *reinterpret_cast<__half*>(wt_blk + i * 128 + (((tcol >> 3) ^ (i & 7)) << 4) + (tcol & 7) * 2) = hv;
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(G_B2));
            // ---- V_new^T (lane = value dim): plain and decayed fp16 rows ----
            if (!mbar_wait_warp(bar(G_C2), par, abort_flag)) ok = false;
            tc_fence_after();
            {
                uint32_t uv[32];
                tmem_ld32(tm_ut + lane_base + hf * 32, uv);
                tmem_wait_ld();
                unsigned char* vn_row = sm + kOffVN + r * 128;
                unsigned char* vs_row = sm + kOffVS + r * 128;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t pa[4], pb[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int l0 = cc * 8 + 2 * e, j0 = hf * 32 + l0;
                        const float x0 = __uint_as_float(uv[l0]), x1 = __uint_as_float(uv[l0 + 1]);
                        pa[e] = pack_half2(x0, x1);
                        pb[e] = pack_half2(x0 * s_ebc[j0], x1 * s_ebc[j0 + 1]);
                    }
                    const int c8 = hf * 4 + cc;
                    *reinterpret_cast<uint4*>(vn_row + ((c8 ^ (r & 7)) << 4)) = make_uint4(pa[0], pa[1], pa[2], pa[3]);
                    *reinterpret_cast<uint4*>(vs_row + ((c8 ^ (r & 7)) << 4)) = make_uint4(pb[0], pb[1], pb[2], pb[3]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(G_B3));
        }
        // ---- last chunk's outputs and the final state: D3 (S^T) -> state pool ----
        if (ok && mbar_wait_warp(bar(G_C3), (n_chunks - 1) & 1, abort_flag)) {
            tc_fence_after();
            store_out(n_chunks - 1);
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
    la_chunk_tc_kernel<<<grid, kG1Threads, kG1Smem, s>>>(mq, mk, v, g, beta, d_seqs, rec_layer, rec_stride, out, d_error);
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200
