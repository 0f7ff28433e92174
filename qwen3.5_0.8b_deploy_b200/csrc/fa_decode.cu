// D1: split-KV decode attention over the paged INT8 / FP16 cache.
//
// One CTA per (sequence, kv head, split).  A producer warp streams whole cache pages (K block,
// token-minor V block and the two scale rows of one page and kv head are each contiguous) into a
// shared-memory ring with 1-D bulk (TMA) copies; each consumer warp owns one ring stage and runs
// the four query heads of the GQA group against its page on mma.sync m16n8k16 (fp16 operands, fp32
// accumulation), so every K/V byte leaves HBM once for all four heads.  INT8 codes are widened to
// fp16 in registers (exact); K scales multiply the logits, V scales are folded into P.
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
    static constexpr int kWarps = kFp16 ? 3 : 6;                              // consumer warps, each with a K and a V buffer
    static constexpr int kMergeBytes = 4 * kHeadDim * 4 + 32;                 // per warp: O^T [4][256] + m[4] + l[4]
    static constexpr int kSmemBytes = kWarps * (kStageBytes + kMergeBytes) + 4 * kWarps * 8 + 16;
    static constexpr int kThreads = (kWarps + 1) * 32;
    static constexpr float kVBoost = kFp16 ? 1.0f : 256.0f;                   // keeps P * v_scale out of fp16 subnormals
};

constexpr float kLog2e = 1.4426950408889634f;

// grid (max_splits, kv_heads, n_seqs).  The CTA that finishes last for a (sequence, kv head) combines the splits,
// applies the gate and writes the output (arrival counter in `counters`, left at zero again).
template <bool kFp16, typename OutT>
__global__ void __launch_bounds__(DecodeCfg<kFp16>::kThreads, 1)
fa_decode_split_kernel(KvView kv, int layer, const int* __restrict__ slots, int len_add,
                       const __half* __restrict__ q, const __half* __restrict__ gate, int pages_per_warp,
                       int max_splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                       int* __restrict__ counters, OutT* __restrict__ out) {
    using Cfg = DecodeCfg<kFp16>;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_last;
    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    pdl_enter();

    const int slot = slots[seq];
    if (slot < 0 || slot >= kv.max_seqs) return;
    if (*reinterpret_cast<volatile int*>(kv.error) == 3) return;     // an earlier CTA gave up: do not queue more bounded waits
    const int L = kv.lens[layer * kv.max_seqs + slot] + len_add;
    const int n_pages = (L + kPageTokens - 1) / kPageTokens;
    const int pages_per_cta = pages_per_warp * Cfg::kWarps;
    const int p_begin = split * pages_per_cta;
    if (p_begin >= n_pages) {
        // A sequence without cached tokens has no split at all: split 0 writes zeros so the output is defined.
        if (n_pages == 0 && split == 0)
            for (int idx = threadIdx.x; idx < 4 * kHeadDim; idx += Cfg::kThreads)
                out[((size_t)seq * kFaHeads + kvh * 4) * kHeadDim + idx] = (OutT)0.f;
        return;
    }
    const int p_end = min(n_pages, p_begin + pages_per_cta);
    const int n_my = p_end - p_begin;
    const int n_splits = (n_pages + pages_per_cta - 1) / pages_per_cta;

    unsigned char* stage_base = smem;
    float* merge_base = reinterpret_cast<float*>(smem + Cfg::kWarps * Cfg::kStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kWarps * (Cfg::kStageBytes + Cfg::kMergeBytes));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 4 * Cfg::kWarps);
    const uint32_t full_k0 = smem_u32(bars), full_v0 = full_k0 + 8 * Cfg::kWarps;
    const uint32_t empty_k0 = full_v0 + 8 * Cfg::kWarps, empty_v0 = empty_k0 + 8 * Cfg::kWarps;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 4 * Cfg::kWarps; ++i) mbar_init(full_k0 + 8 * i, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == Cfg::kWarps) {
        // ---------------- producer: one lane keeps every warp's K and V buffer refilled ----------------
        if (lane == 0) {
            const int* bt = kv.block_table + (size_t)slot * kv.max_pages_per_seq;
            int rk[Cfg::kWarps], rv[Cfg::kWarps];      // rounds issued per warp
#pragma unroll
            for (int w = 0; w < Cfg::kWarps; ++w) { rk[w] = 0; rv[w] = 0; }
            int remaining = 2 * n_my;
            const uint64_t t0 = global_timer_ns();
            uint32_t idle = 0;
            while (remaining > 0) {
                bool progressed = false;
#pragma unroll
                for (int w = 0; w < Cfg::kWarps; ++w) {
#pragma unroll
                    for (int is_v = 0; is_v < 2; ++is_v) {
                        const int r = is_v ? rv[w] : rk[w];
                        const int i = w + r * Cfg::kWarps;
                        if (i >= n_my) continue;
                        const uint32_t eb = (is_v ? empty_v0 : empty_k0) + 8 * w;
                        if (r > 0 && !mbar_test_wait(eb, (r - 1) & 1)) continue;
                        const int page = bt[p_begin + i];
                        const size_t head_base = (size_t)(layer * kv.num_pages + page) * kFaKvHeads + kvh;
                        const unsigned char* src = reinterpret_cast<const unsigned char*>(is_v ? kv.v : kv.k) + head_base * Cfg::kBlockBytes;
                        const uint32_t dst = smem_u32(stage_base + w * Cfg::kStageBytes + is_v * Cfg::kHalfBytes);
                        const uint32_t fb = (is_v ? full_v0 : full_k0) + 8 * w;
                        mbar_arrive_expect_tx(fb, Cfg::kHalfBytes);
                        bulk_g2s(dst, src, Cfg::kBlockBytes, fb);
                        if constexpr (!kFp16)
                            bulk_g2s(dst + Cfg::kBlockBytes, (is_v ? kv.vs : kv.ks) + head_base * kPageTokens, Cfg::kScaleBytes, fb);
                        if (is_v) ++rv[w]; else ++rk[w];
                        --remaining;
                        progressed = true;
                    }
                }
                if (!progressed && ((++idle & 255u) == 0u)) {
                    if (*abort_flag) break;
                    if (global_timer_ns() - t0 > 500000000ull) { *abort_flag = 1; break; }
                }
            }
        }
    } else {
        // ---------------- consumers ----------------
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
        float o[16][4];
#pragma unroll
        for (int j = 0; j < 16; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
        const float sm_scale = kLog2e / 16.0f;   // 1/sqrt(256), logits kept in log2 units

        const unsigned char* sK = stage_base + warp * Cfg::kStageBytes;
        const float* sKs = reinterpret_cast<const float*>(sK + Cfg::kBlockBytes);
        const unsigned char* sV = sK + Cfg::kHalfBytes;
        const float* sVs = reinterpret_cast<const float*>(sV + Cfg::kBlockBytes);
        const uint32_t my_full_k = full_k0 + 8 * warp, my_full_v = full_v0 + 8 * warp;
        const uint32_t my_empty_k = empty_k0 + 8 * warp, my_empty_v = empty_v0 + 8 * warp;

        for (int i = warp, round = 0; i < n_my; i += Cfg::kWarps, ++round) {
            if (!mbar_wait_warp(my_full_k, round & 1, abort_flag)) break;
            const int page_pos0 = (p_begin + i) * kPageTokens;

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
                            cvt_s8x4_half2x2(wl[ss], r0, r2);
                            cvt_s8x4_half2x2(wh[ss], r1, r3);
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
                s[w][0] = val_lo ? s[w][0] * kl[w] : -INFINITY;
                s[w][1] = val_lo ? s[w][1] * kl[w] : -INFINITY;
                s[w][2] = val_hi ? s[w][2] * kh[w] : -INFINITY;
                s[w][3] = val_hi ? s[w][3] * kh[w] : -INFINITY;
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
            if (!mbar_wait_warp(my_full_v, round & 1, abort_flag)) break;
            uint32_t pb[4][2];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                float vl = 1.f, vh = 1.f;
                if constexpr (!kFp16) {
                    const int tok_lo = 16 * (g >> 1) + 4 * w + (g & 1);
                    vl = sVs[tok_lo] * Cfg::kVBoost; vh = sVs[tok_lo + 2] * Cfg::kVBoost;
                }
                pb[w][0] = movmatrix_trans(pack_half2(p[w][0] * vl, p[w][1] * vl));
                pb[w][1] = movmatrix_trans(pack_half2(p[w][2] * vh, p[w][3] * vh));
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
                        cvt_s8x4_half2x2(wl[w], r0, r2);
                        cvt_s8x4_half2x2(wh[w], r1, r3);
                        mma_16816(o[j], r0, r1, r2, r3, pb[w][0], pb[w][1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(my_empty_v);
        }
        // ---- publish this warp's (m, l, O^T) for the CTA merge ----
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, off);
            l1 += __shfl_xor_sync(0xffffffffu, l1, off);
        }
        float* mO = merge_base + warp * (Cfg::kMergeBytes / 4);
        float* mM = mO + 4 * kHeadDim;
        float* mL = mM + 4;
        if (t < 2) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                mO[(2 * t) * kHeadDim + 16 * j + g] = o[j][0];
                mO[(2 * t + 1) * kHeadDim + 16 * j + g] = o[j][1];
                mO[(2 * t) * kHeadDim + 16 * j + 8 + g] = o[j][2];
                mO[(2 * t + 1) * kHeadDim + 16 * j + 8 + g] = o[j][3];
            }
            if (g == 0) { mM[2 * t] = m0; mM[2 * t + 1] = m1; mL[2 * t] = l0; mL[2 * t + 1] = l1; }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(kv.error, 3);
        return;
    }
    // ---- merge the consumer warps and write this split's partial ----
    const size_t pbase = ((size_t)(seq * kFaKvHeads + kvh) * max_splits) * 4;
    for (int idx = threadIdx.x; idx < 4 * kHeadDim; idx += Cfg::kThreads) {
        const int head = idx / kHeadDim, dim = idx % kHeadDim;
        float mmax = -INFINITY;
#pragma unroll
        for (int w = 0; w < Cfg::kWarps; ++w) mmax = fmaxf(mmax, merge_base[w * (Cfg::kMergeBytes / 4) + 4 * kHeadDim + head]);
        float acc = 0.f, lsum = 0.f;
#pragma unroll
        for (int w = 0; w < Cfg::kWarps; ++w) {
            const float* mw = merge_base + w * (Cfg::kMergeBytes / 4);
            const float wgt = exp2f(mw[4 * kHeadDim + head] - mmax);   // a warp without pages has m = -inf -> weight 0
            acc += mw[head * kHeadDim + dim] * wgt;
            lsum += mw[4 * kHeadDim + 4 + head] * wgt;
        }
        part_o[(pbase + split * 4 + head) * kHeadDim + dim] = acc;
        if (dim == 0) { part_ml[(pbase + split * 4 + head) * 2] = mmax; part_ml[(pbase + split * 4 + head) * 2 + 1] = lsum; }
    }
    // ---- the last split to arrive combines all of them ----
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int old = atomicAdd(&counters[seq * kFaKvHeads + kvh], 1);
        s_last = (old == n_splits - 1);
        if (s_last) counters[seq * kFaKvHeads + kvh] = 0;   // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    constexpr float inv_boost = 1.0f / Cfg::kVBoost;
    for (int idx = threadIdx.x; idx < 4 * kHeadDim; idx += Cfg::kThreads) {
        const int head = idx / kHeadDim, dim = idx % kHeadDim;
        float mmax = -INFINITY;
        for (int sp = 0; sp < n_splits; ++sp) mmax = fmaxf(mmax, __ldcg(&part_ml[(pbase + sp * 4 + head) * 2]));
        float acc = 0.f, lsum = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const float wgt = exp2f(__ldcg(&part_ml[(pbase + sp * 4 + head) * 2]) - mmax);
            acc += __ldcg(&part_o[(pbase + sp * 4 + head) * kHeadDim + dim]) * wgt;
            lsum += __ldcg(&part_ml[(pbase + sp * 4 + head) * 2 + 1]) * wgt;
        }
        float r = acc / lsum * inv_boost;
        const size_t oo = ((size_t)seq * kFaHeads + kvh * 4 + head) * kHeadDim + dim;
        if (gate) r *= __half2float(gate[oo]);
        out[oo] = (OutT)r;
    }
}

int fa_decode_max_splits(bool fp16, int max_pages_per_seq, int pages_per_warp) {
    const int per_cta = pages_per_warp * (fp16 ? DecodeCfg<true>::kWarps : DecodeCfg<false>::kWarps);
    return ceil_div(max_pages_per_seq, per_cta);
}

int launch_fa_decode(const KvView& kv, int layer, const int* d_slots, int n_seqs, int len_add, const __half* q,
                     const __half* gate, int pages_per_warp, int max_splits, float* part_o, float* part_ml, int* counters,
                     void* out, bool out_bf16, cudaStream_t s) {
    dim3 grid(max_splits, kFaKvHeads, n_seqs);
    static bool attr_done = false;
    if (!attr_done) {
        B2_CUDA(cudaFuncSetAttribute(fa_decode_split_kernel<true, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<true>::kSmemBytes));
        B2_CUDA(cudaFuncSetAttribute(fa_decode_split_kernel<true, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<true>::kSmemBytes));
        B2_CUDA(cudaFuncSetAttribute(fa_decode_split_kernel<false, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<false>::kSmemBytes));
        B2_CUDA(cudaFuncSetAttribute(fa_decode_split_kernel<false, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<false>::kSmemBytes));
        attr_done = true;
    }
#define FA_DEC_LAUNCH(F16, T)                                                                                          \
    launch_pdl(fa_decode_split_kernel<F16, T>, grid, dim3(DecodeCfg<F16>::kThreads), DecodeCfg<F16>::kSmemBytes, s,    \
               kv, layer, d_slots, len_add, q, gate, pages_per_warp, max_splits, part_o, part_ml, counters, (T*)out)
    if (kv.is_fp16) { if (out_bf16) FA_DEC_LAUNCH(true, __nv_bfloat16); else FA_DEC_LAUNCH(true, float); }
    else            { if (out_bf16) FA_DEC_LAUNCH(false, __nv_bfloat16); else FA_DEC_LAUNCH(false, float); }
#undef FA_DEC_LAUNCH
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200
