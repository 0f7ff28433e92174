// D1: split-KV decode attention over the paged INT8 / FP16 cache.
//
// Persistent kernel, one CTA per SM.  The pages of all (sequence, kv head) pairs of the batch form one linear
// list; it is cut into equal contiguous ranges, one per consumer WARP of the grid, so every SM streams the same
// number of bytes whatever the sequence lengths are.  A producer warp streams whole cache pages (K block,
// token-minor V block and the two scale rows of one page and kv head are each contiguous) into shared memory with
// 1-D bulk (TMA) copies; each consumer warp owns a K buffer and a V buffer and runs the four query heads of the
// GQA group against its pages on mma.sync m16n8k16 (fp16 operands, fp32 accumulation), so every K/V byte leaves
// HBM once for all four heads.  INT8 codes are widened to fp16 in registers (exact); K scales multiply the
// logits, V scales are folded into P.  A range that ends inside a (sequence, kv head) pair leaves a partial
// (m, l, O) in global memory; the warp that delivers the last partial of a pair combines them, applies the gate
// and writes the output (arrival counter in `counters`, left at zero again).
//
// Orientation: S^T[key, head] = K[key, dim] Q^T[dim, head] and O^T[dim, head] = V^T[dim, key] P^T[key, head],
// so the big operands (K rows, token-minor V rows) are the row-major A fragments and load straight
// from the page layout; P^T moves from accumulator to B-fragment layout with movmatrix.
// The contraction indices are permuted (the same permutation on both operands) so each lane reads
// 16 contiguous bytes.
//
// Replaces flash_attn_v2_decode_kernel (src/backend/cuda/kernels/flash_attention.cu:30-181) and
// flash_attn_decode_int8_kernel (src/backend/cuda/kernels/flash_attention_int8.cu:25-238) of the
// reference, plus gate_sigmoid_kernel (full_attention_cuda.cu:150-159) in the combine step.
// Each consumer warp's K buffer and V buffer are released separately, so the next page's K streams in while the
// warp is still multiplying by V, and the next V while it computes the next logits.
#include "kernels.cuh"
#include "ptx_utils.cuh"

namespace b200 {

template <bool kFp16>
struct DecodeCfg {
    static constexpr int kElem = kFp16 ? 2 : 1;
    static constexpr int kBlockBytes = kPageTokens * kHeadDim * kElem;       // K or V of one (page, kv head)
    static constexpr int kScaleBytes = kFp16 ? 0 : kPageTokens * 4;
    static constexpr int kHalfBytes = kBlockBytes + kScaleBytes;              // one K (or V) buffer with its scale row
    static constexpr int kStageBytes = 2 * kHalfBytes;
    static constexpr int kWarps = kFp16 ? 3 : 4;                              // consumer warps, each with a K and a V buffer (INT8: 4 measured 43.2 us, 5: 42.8, 6: 47.7, 3: 44.4 at 128 x 1280)
    static constexpr int kSmemBytes = kWarps * kStageBytes + 4 * kWarps * 8 + 16;
    static constexpr int kThreads = (kWarps + 1) * 32;
    static constexpr float kVBoost = kFp16 ? 1.0f : 256.0f;                   // keeps P * v_scale out of fp16 subnormals
};

constexpr float kLog2e = 1.4426950408889634f;

constexpr int kDecodeMaxSeqs = 2048;      // sequences per launch (prefix table in shared memory)

// Position of linear page x: sequence (searched from `seq`, which must not be past it), kv head, page in sequence.
__device__ __forceinline__ void locate_page(const int* s_pref, int n_seqs, int x, int& seq, int& kvh, int& page) {
    while (seq + 1 < n_seqs && x >= 2 * s_pref[seq + 1]) ++seq;
    const int pages = s_pref[seq + 1] - s_pref[seq];
    const int rem = x - 2 * s_pref[seq];
    kvh = rem >= pages ? 1 : 0;
    page = rem - kvh * pages;
}
__device__ __forceinline__ int find_seq(const int* s_pref, int n_seqs, int x) {   // largest seq with 2 * pref[seq] <= x
    int lo = 0, hi = n_seqs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (2 * s_pref[mid] <= x) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// grid (number of SMs).  max_parts = partial slots per (sequence, kv head) in part_o / part_ml (>= 3).
template <bool kFp16, typename OutT>
__global__ void __launch_bounds__(DecodeCfg<kFp16>::kThreads, 1)
fa_decode_split_kernel(KvView kv, int layer, const int* __restrict__ slots, int n_seqs,
                       const __half* __restrict__ q, const __half* __restrict__ gate, int max_parts,
                       float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                       OutT* __restrict__ out, unsigned long long* stamp) {
    using Cfg = DecodeCfg<kFp16>;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_pref[kDecodeMaxSeqs + 1];      // s_pref[i] = pages of the sequences before i
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    unsigned char* stage_base = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kWarps * Cfg::kStageBytes);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 4 * Cfg::kWarps);
    const uint32_t full_k0 = smem_u32(bars), full_v0 = full_k0 + 8 * Cfg::kWarps;
    const uint32_t empty_k0 = full_v0 + 8 * Cfg::kWarps, empty_v0 = empty_k0 + 8 * Cfg::kWarps;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 4 * Cfg::kWarps; ++i) mbar_init(full_k0 + 8 * i, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    pdl_enter();
    stamp_begin(stamp);
    __shared__ int s_stop;
    if (threadIdx.x == 0) s_stop = (*reinterpret_cast<volatile int*>(kv.error) == 3);   // an earlier launch gave up: queue no more bounded waits

    // ---- pages per sequence and their prefix sums ----
    for (int i = threadIdx.x; i < n_seqs; i += Cfg::kThreads) {
        const int slot = slots[i];
        int pages = 0;
        if (slot >= 0 && slot < kv.max_seqs) pages = (kv.lens[layer * kv.max_seqs + slot] + kPageTokens - 1) / kPageTokens;
        s_pref[i + 1] = pages;
        if (pages == 0 && blockIdx.x == 0 && slot >= 0 && slot < kv.max_seqs)    // no cached token: the output is defined as zero
            for (int idx = 0; idx < kFaHeads * kHeadDim; ++idx) out[(size_t)i * kFaHeads * kHeadDim + idx] = (OutT)0.f;
    }
    if (threadIdx.x == 0) s_pref[0] = 0;
    __syncthreads();
    if (s_stop) return;
    if (warp == 0) {
        const int per = (n_seqs + 31) / 32;
        const int b0 = min(n_seqs, lane * per), b1 = min(n_seqs, b0 + per);
        int sum = 0;
        for (int i = b0; i < b1; ++i) sum += s_pref[i + 1];
        int incl = sum;
#pragma unroll
        for (int o2 = 1; o2 < 32; o2 <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o2);
            if (lane >= o2) incl += v;
        }
        int off = incl - sum;
        for (int i = b0; i < b1; ++i) { off += s_pref[i + 1]; s_pref[i + 1] = off; }
    }
    __syncthreads();
    const int P = 2 * s_pref[n_seqs];                 // linear page list: sequence-major, then kv head, then page
    if (P == 0) return;
    // Equal contiguous ranges, one per consumer warp of the grid; a floor on the range length bounds the number of
    // ranges that can touch one (sequence, kv head) pair to max_parts.
    const int W = gridDim.x * Cfg::kWarps;
    const int r_min = max(1, (kv.max_pages_per_seq + max_parts - 3) / (max_parts - 2));
    const int W_eff = min(W, max(1, P / r_min));
    auto range_start = [&](int w) { return (int)(((long long)w * P) / W_eff); };
    auto owner_of = [&](int x) { return (int)((((long long)(x + 1)) * W_eff - 1) / P); };   // worker whose range holds page x

    if (warp == Cfg::kWarps) {
        // ---------------- producer warp: lane w keeps the K and the V buffer of consumer warp w refilled ----------------
        // One lane per consumer: the look-ups in front of a copy (sequence, block table) are a chain of dependent loads,
        // and a single lane serving every buffer could not start copies faster than the memory system delivers them.
        // The page number of a buffer's next fill is fetched right after the current one is issued.
        if (lane < Cfg::kWarps) {
            const int w = lane;
            const int wid = blockIdx.x + gridDim.x * w;
            int x[2] = {0, 0}, seq[2] = {0, 0}, rounds[2] = {0, 0}, next_page[2] = {0, 0}, next_kvh[2] = {0, 0};
            int xe = 0;
            if (wid < W_eff) {
                x[0] = x[1] = range_start(wid);
                xe = range_start(wid + 1);
            }
            auto look_up = [&](int is_v) {     // sequence, kv head and physical page of linear page x[is_v]
                int kvh, pg;
                locate_page(s_pref, n_seqs, x[is_v], seq[is_v], kvh, pg);
                next_kvh[is_v] = kvh;
                next_page[is_v] = kv.block_table[(size_t)slots[seq[is_v]] * kv.max_pages_per_seq + pg];
            };
            if (x[0] < xe) {
                seq[0] = seq[1] = find_seq(s_pref, n_seqs, x[0]);
                look_up(0);
                seq[1] = seq[0];
                next_page[1] = next_page[0]; next_kvh[1] = next_kvh[0];
            }
            const uint64_t t0 = global_timer_ns();
            uint32_t idle = 0;
            while (x[0] < xe || x[1] < xe) {
                bool progressed = false;
#pragma unroll
                for (int is_v = 0; is_v < 2; ++is_v) {
                    if (x[is_v] >= xe) continue;
                    const int r = rounds[is_v];
                    const uint32_t eb = (is_v ? empty_v0 : empty_k0) + 8 * w;
                    if (r > 0 && !mbar_test_wait(eb, (r - 1) & 1)) continue;
                    const size_t head_base = (size_t)(layer * kv.num_pages + next_page[is_v]) * kFaKvHeads + next_kvh[is_v];
                    const unsigned char* src = reinterpret_cast<const unsigned char*>(is_v ? kv.v : kv.k) + head_base * Cfg::kBlockBytes;
                    const uint32_t dst = smem_u32(stage_base + w * Cfg::kStageBytes + is_v * Cfg::kHalfBytes);
                    const uint32_t fb = (is_v ? full_v0 : full_k0) + 8 * w;
                    mbar_arrive_expect_tx(fb, Cfg::kHalfBytes);
                    bulk_g2s(dst, src, Cfg::kBlockBytes, fb);
                    if constexpr (!kFp16)
                        bulk_g2s(dst + Cfg::kBlockBytes, (is_v ? kv.vs : kv.ks) + head_base * kPageTokens, Cfg::kScaleBytes, fb);
                    ++rounds[is_v];
                    if (++x[is_v] < xe) look_up(is_v);
                    progressed = true;
                }
                if (!progressed && ((++idle & 255u) == 0u)) {
                    if (*abort_flag) break;
                    if (global_timer_ns() - t0 > 500000000ull) { *abort_flag = 1; break; }
                }
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int wid = blockIdx.x + gridDim.x * warp;
        int x = 0, x_end = 0;
        if (wid < W_eff) { x = range_start(wid); x_end = range_start(wid + 1); }
        const float sm_scale = kLog2e / 16.0f;   // 1/sqrt(256), logits kept in log2 units
        const unsigned char* sK = stage_base + warp * Cfg::kStageBytes;
        const float* sKs = reinterpret_cast<const float*>(sK + Cfg::kBlockBytes);
        const unsigned char* sV = sK + Cfg::kHalfBytes;
        const float* sVs = reinterpret_cast<const float*>(sV + Cfg::kBlockBytes);
        const uint32_t my_full_k = full_k0 + 8 * warp, my_full_v = full_v0 + 8 * warp;
        const uint32_t my_empty_k = empty_k0 + 8 * warp, my_empty_v = empty_v0 + 8 * warp;
        int round = 0;
        int seq = (x < x_end) ? find_seq(s_pref, n_seqs, x) : 0;
        bool alive = true;
        while (x < x_end && alive) {
        // ---- one (sequence, kv head) pair, pages [pg0, pg0 + n_my) of it ----
        int kvh, pg0;
        locate_page(s_pref, n_seqs, x, seq, kvh, pg0);
        const int seg_pages = s_pref[seq + 1] - s_pref[seq];
        const int seg_begin = 2 * s_pref[seq] + kvh * seg_pages;
        const int n_my = min(x_end, seg_begin + seg_pages) - x;
        const int L = kv.lens[layer * kv.max_seqs + slots[seq]];
        // Q^T B-fragments: k-step ks = 4*blk + s covers dims 64*blk + 16*t + 4*s + {0,1 | 2,3}; head = g (< 4).
        uint32_t qf[16][2];
        {
            const __half* qrow = q + ((size_t)seq * kFaHeads + kvh * 4 + (g & 3)) * kHeadDim;
#pragma unroll
            for (int ks = 0; ks < 16; ++ks) {
                const int p0 = 64 * (ks >> 2) + 16 * t + 4 * (ks & 3);
                const uint2 v = *reinterpret_cast<const uint2*>(qrow + p0);
                qf[ks][0] = (g < 4) ? v.x : 0u;
                qf[ks][1] = (g < 4) ? v.y : 0u;
            }
        }
        // INT8 cache: the K codes enter the MMA as code + 1152 (one instruction less per pair of values); the logits are
        // corrected by 1152 * sum_dim q[dim, head], which is computed here once per (sequence, kv head) pair
        float corr0 = 0.f, corr1 = 0.f;
        if constexpr (!kFp16) {
            float qs = 0.f;
#pragma unroll
            for (int ks = 0; ks < 16; ++ks) {
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&qf[ks][0]));
                const float2 b2 = __half22float2(*reinterpret_cast<const __half2*>(&qf[ks][1]));
                qs += (a.x + a.y) + (b2.x + b2.y);
            }
            qs += __shfl_xor_sync(0xffffffffu, qs, 1);
            qs += __shfl_xor_sync(0xffffffffu, qs, 2);           // lanes of one g now hold the sum over all 256 dims of head g
            corr0 = 1152.0f * __shfl_sync(0xffffffffu, qs, (2 * t) * 4);
            corr1 = 1152.0f * __shfl_sync(0xffffffffu, qs, (2 * t + 1) * 4);
        }
        float o[16][4];
#pragma unroll
        for (int j = 0; j < 16; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
        float c0 = 0.f, c1 = 0.f;       // INT8 cache: sums of the fp16 weights that multiplied V codes carrying the +1152 bias

        for (int i = 0; i < n_my; ++i, ++round) {
            if (!mbar_wait_warp(my_full_k, round & 1, abort_flag)) { alive = false; break; }
            const int page_pos0 = (pg0 + i) * kPageTokens;

            // ---- S^T = K Q^T for the four 16-token tiles of the page ----
            float s[4][4];
            float kl[4], kh[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                s[w][0] = s[w][1] = s[w][2] = s[w][3] = 0.f;
                const int tok_lo = 16 * (g >> 1) + 4 * w + (g & 1);
                const int tok_hi = tok_lo + 2;
                kl[w] = sm_scale; kh[w] = sm_scale;
                if constexpr (!kFp16) { kl[w] *= sKs[tok_lo]; kh[w] *= sKs[tok_hi]; }
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
                    if constexpr (kFp16) {
                        const unsigned char* pl = sK + tok_lo * 512 + 128 * blk + 32 * t;
                        const unsigned char* ph = sK + tok_hi * 512 + 128 * blk + 32 * t;
                        const uint4 l0v = *reinterpret_cast<const uint4*>(pl);
                        const uint4 l1v = *reinterpret_cast<const uint4*>(pl + 16);
                        const uint4 h0v = *reinterpret_cast<const uint4*>(ph);
                        const uint4 h1v = *reinterpret_cast<const uint4*>(ph + 16);
                        mma_16816(s[w], l0v.x, h0v.x, l0v.y, h0v.y, qf[4 * blk + 0][0], qf[4 * blk + 0][1]);
                        mma_16816(s[w], l0v.z, h0v.z, l0v.w, h0v.w, qf[4 * blk + 1][0], qf[4 * blk + 1][1]);
                        mma_16816(s[w], l1v.x, h1v.x, l1v.y, h1v.y, qf[4 * blk + 2][0], qf[4 * blk + 2][1]);
                        mma_16816(s[w], l1v.z, h1v.z, l1v.w, h1v.w, qf[4 * blk + 3][0], qf[4 * blk + 3][1]);
                    } else {
                        const uint4 xl = *reinterpret_cast<const uint4*>(sK + tok_lo * 256 + 64 * blk + 16 * t);
                        const uint4 xh = *reinterpret_cast<const uint4*>(sK + tok_hi * 256 + 64 * blk + 16 * t);
                        const uint32_t wl[4] = {xl.x, xl.y, xl.z, xl.w};
                        const uint32_t wh[4] = {xh.x, xh.y, xh.z, xh.w};
#pragma unroll
                        for (int ss = 0; ss < 4; ++ss) {
                            uint32_t r0, r2, r1, r3;
                            cvt_s8x4_half2x2_biased(wl[ss], r0, r2);
                            cvt_s8x4_half2x2_biased(wh[ss], r1, r3);
                            mma_16816(s[w], r0, r1, r2, r3, qf[4 * blk + ss][0], qf[4 * blk + ss][1]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(my_empty_k);       // the K buffer (and its scale row, already in registers) is free again
            // ---- scale, mask, online softmax (log2 domain); this lane sees heads 2t, 2t+1 ----
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const int tok_lo = 16 * (g >> 1) + 4 * w + (g & 1);
                const int tok_hi = tok_lo + 2;
                const bool val_lo = page_pos0 + tok_lo < L, val_hi = page_pos0 + tok_hi < L;
                s[w][0] = val_lo ? (s[w][0] - corr0) * kl[w] : -INFINITY;      // corr = 0 for the FP16 cache
                s[w][1] = val_lo ? (s[w][1] - corr1) * kl[w] : -INFINITY;
                s[w][2] = val_hi ? (s[w][2] - corr0) * kh[w] : -INFINITY;
                s[w][3] = val_hi ? (s[w][3] - corr1) * kh[w] : -INFINITY;
                mx0 = fmaxf(mx0, fmaxf(s[w][0], s[w][2]));
                mx1 = fmaxf(mx1, fmaxf(s[w][1], s[w][3]));
            }
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
            }
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: every page holds a valid token
            const float a0 = exp2f(m0 - mn0), a1 = exp2f(m1 - mn1);
            m0 = mn0; m1 = mn1;
            l0 *= a0; l1 *= a1;
            if constexpr (!kFp16) { c0 *= a0; c1 *= a1; }
#pragma unroll
            for (int j = 0; j < 16; ++j) { o[j][0] *= a0; o[j][2] *= a0; o[j][1] *= a1; o[j][3] *= a1; }
            float p[4][4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                p[w][0] = exp2f(s[w][0] - mn0); p[w][1] = exp2f(s[w][1] - mn1);
                p[w][2] = exp2f(s[w][2] - mn0); p[w][3] = exp2f(s[w][3] - mn1);
                l0 += p[w][0] + p[w][2]; l1 += p[w][1] + p[w][3];
            }
            // ---- O^T += V^T P^T ----
            if (!mbar_wait_warp(my_full_v, round & 1, abort_flag)) { alive = false; break; }
            uint32_t pb[4][2];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                float vl = 1.f, vh = 1.f;
                if constexpr (!kFp16) {
                    const int tok_lo = 16 * (g >> 1) + 4 * w + (g & 1);
                    vl = sVs[tok_lo] * Cfg::kVBoost; vh = sVs[tok_lo + 2] * Cfg::kVBoost;
                }
                const uint32_t plo = pack_half2(p[w][0] * vl, p[w][1] * vl), phi = pack_half2(p[w][2] * vh, p[w][3] * vh);
                if constexpr (!kFp16) {         // the rounded weights, exactly as the tensor core sees them
                    const float2 fl = __half22float2(*reinterpret_cast<const __half2*>(&plo));
                    const float2 fh = __half22float2(*reinterpret_cast<const __half2*>(&phi));
                    c0 += fl.x + fh.x; c1 += fl.y + fh.y;
                }
                pb[w][0] = movmatrix_trans(plo);
                pb[w][1] = movmatrix_trans(phi);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int dim_lo = 16 * j + g, dim_hi = dim_lo + 8;
                if constexpr (kFp16) {
                    const unsigned char* pl = sV + dim_lo * 128 + 32 * t;
                    const unsigned char* ph = sV + dim_hi * 128 + 32 * t;
                    const uint4 l0v = *reinterpret_cast<const uint4*>(pl);
                    const uint4 l1v = *reinterpret_cast<const uint4*>(pl + 16);
                    const uint4 h0v = *reinterpret_cast<const uint4*>(ph);
                    const uint4 h1v = *reinterpret_cast<const uint4*>(ph + 16);
                    mma_16816(o[j], l0v.x, h0v.x, l0v.y, h0v.y, pb[0][0], pb[0][1]);
                    mma_16816(o[j], l0v.z, h0v.z, l0v.w, h0v.w, pb[1][0], pb[1][1]);
                    mma_16816(o[j], l1v.x, h1v.x, l1v.y, h1v.y, pb[2][0], pb[2][1]);
                    mma_16816(o[j], l1v.z, h1v.z, l1v.w, h1v.w, pb[3][0], pb[3][1]);
                } else {
                    const uint4 vl4 = *reinterpret_cast<const uint4*>(sV + dim_lo * 64 + 16 * t);
                    const uint4 vh4 = *reinterpret_cast<const uint4*>(sV + dim_hi * 64 + 16 * t);
                    const uint32_t wl[4] = {vl4.x, vl4.y, vl4.z, vl4.w};
                    const uint32_t wh[4] = {vh4.x, vh4.y, vh4.z, vh4.w};
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        uint32_t r0, r2, r1, r3;
                        cvt_s8x4_half2x2_biased(wl[w], r0, r2);
                        cvt_s8x4_half2x2_biased(wh[w], r1, r3);
                        mma_16816(o[j], r0, r1, r2, r3, pb[w][0], pb[w][1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(my_empty_v);
        }
        if (!alive) break;
        // ---- this range's share of the pair is done: write the output, or a partial for the combine ----
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, off);
            l1 += __shfl_xor_sync(0xffffffffu, l1, off);
            if constexpr (!kFp16) {
                c0 += __shfl_xor_sync(0xffffffffu, c0, off);
                c1 += __shfl_xor_sync(0xffffffffu, c1, off);
            }
        }
        if constexpr (!kFp16) {                  // take the bias of the V codes back out: 1152 * sum of weights, per head
            const float b0 = 1152.0f * c0, b1 = 1152.0f * c1;
#pragma unroll
            for (int j = 0; j < 16; ++j) { o[j][0] -= b0; o[j][2] -= b0; o[j][1] -= b1; o[j][3] -= b1; }
        }
        constexpr float inv_boost = 1.0f / Cfg::kVBoost;
        const int pair = seq * kFaKvHeads + kvh;
        const int w_first = owner_of(seg_begin), w_last = owner_of(seg_begin + seg_pages - 1);
        const int n_parts = w_last - w_first + 1;
        const size_t obase = ((size_t)seq * kFaHeads + kvh * 4) * kHeadDim;
        if (n_parts == 1) {
            if (t < 2) {
                const float i0 = inv_boost / l0, i1 = inv_boost / l1;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const size_t a0 = obase + (size_t)(2 * t) * kHeadDim + 16 * j + g, a1 = a0 + kHeadDim;
                    float r0 = o[j][0] * i0, r1 = o[j][1] * i1, r2 = o[j][2] * i0, r3 = o[j][3] * i1;
                    if (gate) {
                        r0 *= __half2float(gate[a0]); r1 *= __half2float(gate[a1]);
                        r2 *= __half2float(gate[a0 + 8]); r3 *= __half2float(gate[a1 + 8]);
                    }
                    out[a0] = (OutT)r0; out[a1] = (OutT)r1; out[a0 + 8] = (OutT)r2; out[a1 + 8] = (OutT)r3;
                }
            }
        } else {
            // A partial is stored in the order the accumulators lie in the registers (lane (g, t < 2): its 64 values as
            // sixteen 16-byte pieces), so writing it takes 16 stores per lane and reading it back 16-byte loads as well.
            const size_t pbase = ((size_t)pair * max_parts) * 4;
            const int part = wid - w_first;
            if (t < 2) {
                float4* po = reinterpret_cast<float4*>(part_o + (pbase + part * 4) * kHeadDim) + (g * 2 + t) * 16;
#pragma unroll
                for (int j = 0; j < 16; ++j) po[j] = make_float4(o[j][0], o[j][1], o[j][2], o[j][3]);
                if (g == 0)
                    *reinterpret_cast<float4*>(part_ml + (pbase + part * 4 + 2 * t) * 2) = make_float4(m0, l0, m1, l1);
            }
            // One release / acquire atomic per warp instead of a fence on either side of a relaxed one: the warp barrier
            // orders the lanes' stores before lane 0's release, the shuffle orders its acquire before the lanes' loads
            // (which go to L2).  The gate values do not depend on the partials and are requested before the atomic.
            const int tt = t & 1, half = t >> 1;
            __half gv[32];
            if (gate) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const size_t a0 = obase + (size_t)(2 * tt) * kHeadDim + 16 * (8 * half + k) + g, a1 = a0 + kHeadDim;
                    gv[4 * k] = gate[a0]; gv[4 * k + 1] = gate[a1]; gv[4 * k + 2] = gate[a0 + 8]; gv[4 * k + 3] = gate[a1 + 8];
                }
            }
            __syncwarp();
            int last = 0;
            if (lane == 0) {
                int old;
                asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(counters + pair) : "memory");
                last = (old == n_parts - 1);
                if (last) counters[pair] = 0;          // ready for the next launch
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {                                // the last partial of the pair to arrive: combine them all
                // The warp that combines is usually among the last of the launch to finish, so this is on the kernel's
                // critical path: every lane takes half of a (g, t) fragment (heads 2tt, 2tt + 1; eight of the sixteen
                // 16-dim tiles), and the loads of up to four parts, their (m, l) included, are issued together - one L2
                // round trip for the usual case.  More parts are folded in with the running-maximum rule.
                float4 acc[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                float rm0 = -INFINITY, rm1 = -INFINITY, ls0 = 0.f, ls1 = 0.f;
                for (int sp0 = 0; sp0 < n_parts; sp0 += 4) {
                    float4 ml[4], pv[4][8];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int sp = min(sp0 + u, n_parts - 1);      // parts past the end are loaded again and weighted zero
                        ml[u] = __ldcg(reinterpret_cast<const float4*>(part_ml + (pbase + sp * 4 + 2 * tt) * 2));
                        const float4* po = reinterpret_cast<const float4*>(part_o + (pbase + sp * 4) * kHeadDim) + (g * 2 + tt) * 16 + 8 * half;
#pragma unroll
                        for (int k = 0; k < 8; ++k) pv[u][k] = __ldcg(po + k);
                    }
                    float nm0 = rm0, nm1 = rm1;
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (sp0 + u < n_parts) { nm0 = fmaxf(nm0, ml[u].x); nm1 = fmaxf(nm1, ml[u].z); }
                    const float s0 = exp2f(rm0 - nm0), s1 = exp2f(rm1 - nm1);     // 0 for the first group
                    rm0 = nm0; rm1 = nm1;
                    ls0 *= s0; ls1 *= s1;
#pragma unroll
                    for (int k = 0; k < 8; ++k) { acc[k].x *= s0; acc[k].z *= s0; acc[k].y *= s1; acc[k].w *= s1; }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const bool valid = sp0 + u < n_parts;
                        const float w0 = valid ? exp2f(ml[u].x - nm0) : 0.f, w1 = valid ? exp2f(ml[u].z - nm1) : 0.f;
                        ls0 += ml[u].y * w0; ls1 += ml[u].w * w1;
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            acc[k].x += pv[u][k].x * w0; acc[k].z += pv[u][k].z * w0;
                            acc[k].y += pv[u][k].y * w1; acc[k].w += pv[u][k].w * w1;
                        }
                    }
                }
                const float i0 = inv_boost / ls0, i1 = inv_boost / ls1;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const size_t a0 = obase + (size_t)(2 * tt) * kHeadDim + 16 * (8 * half + k) + g, a1 = a0 + kHeadDim;
                    float r0 = acc[k].x * i0, r1 = acc[k].y * i1, r2 = acc[k].z * i0, r3 = acc[k].w * i1;
                    if (gate) {
                        r0 *= __half2float(gv[4 * k]); r1 *= __half2float(gv[4 * k + 1]);
                        r2 *= __half2float(gv[4 * k + 2]); r3 *= __half2float(gv[4 * k + 3]);
                    }
                    out[a0] = (OutT)r0; out[a1] = (OutT)r1; out[a0 + 8] = (OutT)r2; out[a1 + 8] = (OutT)r3;
                }
            }
        }
        x += n_my;
        }   // pairs of this range
    }
    __syncthreads();
    stamp_end(stamp);
    if (*abort_flag && threadIdx.x == 0) atomicExch(kv.error, 3);
}

// max_splits = partial slots per (sequence, kv head) pair in part_o / part_ml (kFaDecodeParts in the callers' scratch).
int launch_fa_decode(const KvView& kv, int layer, const int* d_slots, int n_seqs, const __half* q,
                     const __half* gate, int max_splits, float* part_o, float* part_ml, int* counters,
                     void* out, bool out_fp16, cudaStream_t s) {
    B2_CHECK_ARG(n_seqs > 0 && n_seqs <= kDecodeMaxSeqs, "decode attention: %d sequences outside (0, %d]", n_seqs, kDecodeMaxSeqs);
    B2_CHECK_ARG(max_splits >= 3, "decode attention: scratch for %d partials per head group, need >= 3", max_splits);
    int n_sm = 0;
    B2_TRY(device_sm_count(&n_sm));
    static PerDeviceOnce once;
    B2_PER_DEVICE_ONCE(once,
        B2_CUDA(cudaFuncSetAttribute(fa_decode_split_kernel<true, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<true>::kSmemBytes));
        B2_CUDA(cudaFuncSetAttribute(fa_decode_split_kernel<true, __half>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<true>::kSmemBytes));
        B2_CUDA(cudaFuncSetAttribute(fa_decode_split_kernel<false, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<false>::kSmemBytes));
        B2_CUDA(cudaFuncSetAttribute(fa_decode_split_kernel<false, __half>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<false>::kSmemBytes)));
    dim3 grid(n_sm);
    unsigned long long* stamp = prof_stamp_slot(PROF_FA_DECODE);
#define FA_DEC_LAUNCH(F16, T)                                                                                          \
    launch_pdl(fa_decode_split_kernel<F16, T>, grid, dim3(DecodeCfg<F16>::kThreads), DecodeCfg<F16>::kSmemBytes, s,    \
               kv, layer, d_slots, n_seqs, q, gate, max_splits, part_o, part_ml, counters, (T*)out, stamp)
    if (kv.is_fp16) { if (out_fp16) FA_DEC_LAUNCH(true, __half); else FA_DEC_LAUNCH(true, float); }
    else            { if (out_fp16) FA_DEC_LAUNCH(false, __half); else FA_DEC_LAUNCH(false, float); }
#undef FA_DEC_LAUNCH
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200
