// F1: causal flash-attention prefill for head_dim 256 on tcgen05 tensor cores.
//
// Persistent CTAs, each walking (128-query tile of one sequence, q head) work items.  Warp roles: warps 0-7 = softmax (two threads per query
// row = TMEM lane, each owning 32 of the 64 key columns of a tile and half of the output columns; the pair
// exchanges its row maxima through shared memory), warp 8 = TMA producer, warp 9 = MMA issuer and TMEM owner.
//   S[128x64]  = Q[128x256] K_j^T      tcgen05.mma kind::f16 (fp16 operands), A and B K-major, TMEM cols [0,128) double-buffered
//   O[128x256] += P_j[128x64] V_j      A = P (written by the softmax warps, K-major), B = V tile MN-major, TMEM cols [128,384)
// Q / K / V tiles arrive through tiled TMA with 128-byte swizzle; K and V are double-buffered.  The softmax
// keeps logits in log2 units and rescales O only when a row maximum grows by more than 2^8.
// Every mbarrier wait is bounded: on give-up the CTA raises an error word and leaves through the common exit.
//
// Replaces flash_attn_v2_prefill_kernel (src/backend/cuda/kernels/fused_kernels.cu:126-264 in the reference;
// that kernel applies no causal mask, this one does, as the CPU reference's token loop implies) and
// gate_sigmoid_kernel (full_attention_cuda.cu:602-614) in the epilogue.
#include "kernels.cuh"
#include "tc05.cuh"

#include <algorithm>
#include <vector>

namespace b200 {

constexpr int kBM = 128, kBN = 64;
constexpr uint32_t kQBytes = 4 * kBM * 128;     // 65536
constexpr uint32_t kKVBytes = 4 * kBN * 128;    // 32768
constexpr uint32_t kPBytes = kBM * 128;         // 16384
constexpr uint32_t kOffQ = 0, kOffK = kQBytes, kOffV = kOffK + 2 * kKVBytes, kOffP = kOffV + 2 * kKVBytes;
constexpr uint32_t kOffBar = kOffP + 2 * kPBytes;
constexpr uint32_t kOffXch = kOffBar + 256;          // row-maximum exchange [2 tiles][2 halves][128]; row sums reuse the idle tile slot
constexpr uint32_t kF1Smem = kOffXch + 2048;         // no alignment slack: the kernel checks its base instead
constexpr int kF1Threads = 320;
constexpr float kLog2eF = 1.4426950408889634f;
__device__ __forceinline__ float ex2_fast(float x) {     // 2^x, one MUFU op; -inf -> 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

enum { BAR_Q = 0, BAR_QE = 1, BAR_KF = 2, BAR_KE = 4, BAR_VF = 6, BAR_VE = 8, BAR_SF = 10, BAR_SE = 12, BAR_PF = 14, BAR_PV = 16,
       BAR_OF = 18, BAR_OD = 19, BAR_COUNT = 20 };

// Persistent: grid = min(number of SMs, tiles x heads); CTA c walks the work items c, c + grid, ... (item w = tile w / 8,
// head w % 8; the tile list is sorted longest context first, so the round-robin is balanced).  All ring barriers run on a
// step counter that continues across items, so the K / V / Q loads and the first S products of the next item are under
// way while the softmax warps still read the finished item's output out of TMEM.
template <typename OutT>
__global__ void __launch_bounds__(kF1Threads, 1)
fa_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                     const PrefillTile* __restrict__ tiles, int n_items, const __half* __restrict__ gate, OutT* __restrict__ out,
                     int* __restrict__ error_word) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    unsigned char* sm = smem_raw;
    if (base & 1023u) {            // the 128-byte swizzle needs 1024-byte aligned tiles
        if (threadIdx.x == 0) atomicExch(error_word, 8);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = base + kOffBar;
    auto bar = [&](int i) { return bar0 + 8u * i; };

    if (*reinterpret_cast<volatile int*>(error_word) != 0) return;   // an earlier launch gave up: do not queue more bounded waits
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, n_cta = gridDim.x;
    const int n_my = (cta < n_items) ? (n_items - cta + n_cta - 1) / n_cta : 0;
    auto item_tile = [&](int i, int& head) -> PrefillTile {
        const int w = cta + i * n_cta;
        head = w & 7;
        return tiles[w >> 3];
    };
    auto key_tiles = [](const PrefillTile& t) { return (t.q_pos0 + t.n_rows + kBN - 1) / kBN; };   // tiles 0..n-1 cover positions <= last query

    if (threadIdx.x == 0) {
        for (int i = 0; i < BAR_COUNT; ++i) {
            const bool many = (i == BAR_SE || i == BAR_SE + 1 || i == BAR_PF || i == BAR_PF + 1 || i == BAR_OD);
            mbar_init(bar(i), many ? 256 : 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    if (warp == 8 && lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        if constexpr (sizeof(OutT) == 2) tma_prefetch_desc(&map_o);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_o = tmem + 128;

    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        // Three independent streams, each advanced as soon as its consumer has released the buffer: Q (one tile per item),
        // K and V (one tile per key step, double-buffered, steps counted across items).
        if (lane == 0) {
            int iq = 0;
            int ik = 0, jk = 0, gk = 0, iv = 0, jv = 0, gv = 0;
            int hk = 0, hv = 0;
            PrefillTile tk = {}, tv = {};
            int nk = 0, nv = 0;
            if (n_my > 0) { tk = item_tile(0, hk); tv = tk; hv = hk; nk = nv = key_tiles(tk); }
            const uint64_t t0 = global_timer_ns();
            uint32_t idle = 0;
            while (iq < n_my || ik < n_my || iv < n_my) {
                bool progressed = false;
                if (iq < n_my && (iq == 0 || mbar_test_wait(bar(BAR_QE), (iq - 1) & 1))) {
                    int hq;
                    const PrefillTile tq = item_tile(iq, hq);
                    mbar_arrive_expect_tx(bar(BAR_Q), kQBytes);
                    for (int blk = 0; blk < 4; ++blk)
                        tma_load_3d(base + kOffQ + blk * (kBM * 128), &map_q, bar(BAR_Q), blk * 64, hq, tq.q_row0);
                    ++iq;
                    progressed = true;
                }
                if (ik < n_my && (gk < 2 || mbar_test_wait(bar(BAR_KE + (gk & 1)), ((gk >> 1) - 1) & 1))) {
                    const int b = gk & 1, row = tk.ctx_row0 + jk * kBN;
                    mbar_arrive_expect_tx(bar(BAR_KF + b), kKVBytes);
                    for (int blk = 0; blk < 4; ++blk)
                        tma_load_3d(base + kOffK + b * kKVBytes + blk * (kBN * 128), &map_k, bar(BAR_KF + b), blk * 64, hk >> 2, row);
                    ++gk;
                    if (++jk == nk) { jk = 0; if (++ik < n_my) { tk = item_tile(ik, hk); nk = key_tiles(tk); } }
                    progressed = true;
                }
                if (iv < n_my && (gv < 2 || mbar_test_wait(bar(BAR_VE + (gv & 1)), ((gv >> 1) - 1) & 1))) {
                    const int b = gv & 1, row = tv.ctx_row0 + jv * kBN;
                    mbar_arrive_expect_tx(bar(BAR_VF + b), kKVBytes);
                    for (int blk = 0; blk < 4; ++blk)
                        tma_load_3d(base + kOffV + b * kKVBytes + blk * (kBN * 128), &map_v, bar(BAR_VF + b), blk * 64, hv >> 2, row);
                    ++gv;
                    if (++jv == nv) { jv = 0; if (++iv < n_my) { tv = item_tile(iv, hv); nv = key_tiles(tv); } }
                    progressed = true;
                }
                if (!progressed && ((++idle & 255u) == 0u)) {
                    if (*abort_flag) break;
                    if (global_timer_ns() - t0 > 4000000000ull) { *abort_flag = 1; break; }
                }
            }
        }
    } else if (warp == 9) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(kFmtF16, kBM, kBN, 0, 0);
            constexpr uint32_t idesc_pv = umma_idesc(kFmtF16, kBM, kHeadDim, 0, 1);
            // PV product of global step g; `first`: first key step of its item (overwrites O, which the previous item's
            // epilogue must have read), `last`: last key step of its item (O is final afterwards)
            auto issue_pv = [&](int g, bool first, bool last, int item) -> bool {
                const int b = g & 1;
                const uint32_t par = (g >> 1) & 1;
                if (!mbar_wait(bar(BAR_VF + b), par, abort_flag)) return false;
                if (!mbar_wait(bar(BAR_PF + b), par, abort_flag)) return false;
                if (first && item > 0 && !mbar_wait(bar(BAR_OD), (item - 1) & 1, abort_flag)) return false;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint64_t a = umma_smem_desc(base + kOffP + b * kPBytes + ks * 32, 16, 1024);
                    const uint64_t bd = umma_smem_desc(base + kOffV + b * kKVBytes + ks * 2048, kBN * 128, 1024);
                    umma_f16(tmem_o, a, bd, idesc_pv, (!first || ks > 0) ? 1u : 0u);
                }
                umma_commit(bar(BAR_PV + b));
                umma_commit(bar(BAR_VE + b));
                if (last) umma_commit(bar(BAR_OF));
                return true;
            };
            bool ok = true, pending = false;
            int pg = 0, pitem = 0;
            bool pfirst = false, plast = false;
            int gs = 0;
            for (int i = 0; ok && i < n_my; ++i) {
                int head;
                const PrefillTile tile = item_tile(i, head);
                const int n_kt = key_tiles(tile);
                // the previous item's last PV product goes out before the wait for this item's Q tile, so that its
                // epilogue runs while Q and the first S product are on their way
                if (pending) {
                    if (!issue_pv(pg, pfirst, plast, pitem)) { ok = false; break; }
                    pending = false;
                }
                if (!mbar_wait(bar(BAR_Q), i & 1, abort_flag)) { ok = false; break; }
                for (int j = 0; j < n_kt; ++j, ++gs) {
                    const int b = gs & 1;
                    if (!mbar_wait(bar(BAR_KF + b), (gs >> 1) & 1, abort_flag)) { ok = false; break; }
                    if (gs >= 2 && !mbar_wait(bar(BAR_SE + b), ((gs >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 16; ++ks) {
                        const uint32_t off = (ks & 3) * 32;
                        const uint64_t a = umma_smem_desc(base + kOffQ + (ks >> 2) * (kBM * 128) + off, 16, 1024);
                        const uint64_t bd = umma_smem_desc(base + kOffK + b * kKVBytes + (ks >> 2) * (kBN * 128) + off, 16, 1024);
                        umma_f16(tmem + b * kBN, a, bd, idesc_s, ks > 0 ? 1u : 0u);
                    }
                    umma_commit(bar(BAR_SF + b));
                    umma_commit(bar(BAR_KE + b));
                    if (j == n_kt - 1) umma_commit(bar(BAR_QE));      // the Q tile is free once this item's S products are done
                    if (pending && !issue_pv(pg, pfirst, plast, pitem)) { ok = false; break; }
                    pending = true; pg = gs; pfirst = (j == 0); plast = (j == n_kt - 1); pitem = i;
                }
            }
            if (ok && pending) issue_pv(pg, pfirst, plast, pitem);
        }
    } else {
        // ------------------------------ softmax / correction / epilogue ------------------------------
        const int r = threadIdx.x & 127;                 // query row == TMEM lane
        const int hf = threadIdx.x >> 7;                 // which 32 of a tile's 64 key columns / which half of the output columns
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const int pair_bar = 1 + (warp & 3);             // named barrier shared by the two warps that cover the same rows
        float* x_mx = reinterpret_cast<float*>(sm + kOffXch);          // [2][2][128]
        const float sc = kLog2eF / 16.0f;
        bool ok = true;
        int gs = 0;
        for (int it = 0; it < n_my; ++it) {
            int head;
            const PrefillTile tile = item_tile(it, head);
            const int n_kt = key_tiles(tile);
            const int q_pos = tile.q_pos0 + r;
            float m_ref = -INFINITY, l = 0.f;
            // this row's gate values (512 bytes, read in the epilogue) start their way from DRAM to L2 now
            if (gate && r < tile.n_rows) {
                const __half* grow = gate + ((size_t)(tile.q_row0 + r) * kFaHeads + head) * kHeadDim + hf * 128;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(grow));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(grow + 64));
            }
            for (int j = 0; j < n_kt; ++j, ++gs) {
                const int b = gs & 1;
                if (!mbar_wait_warp(bar(BAR_SF + b), (gs >> 1) & 1, abort_flag)) ok = false;
                tc_fence_after();
                uint32_t sr[32];
                tmem_ld32(tmem + lane_base + b * kBN + hf * 32, sr);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(bar(BAR_SE + b));
                const int col0 = j * kBN + hf * 32;
                const bool diag = (col0 + 31 > tile.q_pos0);   // warp-uniform: this half tile may cross a diagonal
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four short chains instead of one long one
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    float v = __uint_as_float(sr[c]);
                    if (diag && (col0 + c > q_pos)) v = -INFINITY;
                    sr[c] = __float_as_uint(v);
                    mx4[c & 3] = fmaxf(mx4[c & 3], v);
                }
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                x_mx[(b * 2 + hf) * 128 + r] = mx;
                asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
                mx = fmaxf(mx, x_mx[(b * 2 + (hf ^ 1)) * 128 + r]) * sc;
                const float m_new = fmaxf(m_ref, mx);            // finite: key 0 is visible to every row
                const bool need = (m_new - m_ref > 8.0f);        // also true on the first tile (m_ref = -inf)
                if (__any_sync(0xffffffffu, need)) {             // same decision in both warps of the pair: same rows, same values
                    if (j > 0) {
                        if (!mbar_wait_warp(bar(BAR_PV + ((gs - 1) & 1)), ((gs - 1) >> 1) & 1, abort_flag)) ok = false;
                        tc_fence_after();
                        const float alpha = exp2f(m_ref - m_new);
                        l *= alpha;
#pragma unroll 1
                        for (int cc = 0; cc < 4; ++cc) {
                            const int ch = hf * 4 + cc;
                            uint32_t orr[32];
                            tmem_ld32(tmem_o + lane_base + ch * 32, orr);
                            tmem_wait_ld();
#pragma unroll
                            for (int c = 0; c < 32; ++c) orr[c] = __float_as_uint(__uint_as_float(orr[c]) * alpha);
                            tmem_st32(tmem_o + lane_base + ch * 32, orr);
                        }
                        tmem_wait_st();
                    }
                    m_ref = m_new;
                }
                // P = 2^(s * scale - m_ref) as fp16 into the swizzled K-major A tile
                if (gs >= 2 && !mbar_wait_warp(bar(BAR_PV + b), ((gs >> 1) - 1) & 1, abort_flag)) ok = false;
                unsigned char* prow = sm + kOffP + b * kPBytes + r * 128;
                float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c8 = 0; c8 < 4; ++c8) {
                    uint32_t pk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float p0 = ex2_fast(fmaf(__uint_as_float(sr[c8 * 8 + 2 * e]), sc, -m_ref));
                        const float p1 = ex2_fast(fmaf(__uint_as_float(sr[c8 * 8 + 2 * e + 1]), sc, -m_ref));
                        ls4[e] += p0 + p1;
                        pk[e] = pack_half2(p0, p1);
                    }
                    *reinterpret_cast<uint4*>(prow + (((hf * 4 + c8) ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
                l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
                fence_proxy_async_smem();
                tc_fence_before();
                mbar_arrive(bar(BAR_PF + b));
            }
            // row sums of the two halves: through the exchange slot the next step will use, hence the second barrier
            float* x_l = x_mx + (gs & 1) * 256;
            x_l[hf * 128 + r] = l;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            l += x_l[(hf ^ 1) * 128 + r];
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            const bool valid = r < tile.n_rows;
            const size_t orow = ((size_t)(tile.q_row0 + r) * kFaHeads + head) * kHeadDim;
            // fp16 output of a full tile leaves through shared memory and tiled TMA stores (the P buffers are idle between
            // the last PV product and the next item's first P tile); anything else is stored from registers.
            const bool via_tma = (sizeof(OutT) == 2) && (tile.n_rows == kBM);
            if (!via_tma) {
                // columns [32 ch, 32 ch + 32) of this thread's row, ch = 2 cc + hf
                if (!mbar_wait_warp(bar(BAR_OF), it & 1, abort_flag)) ok = false;
                tc_fence_after();
                const float inv_l = 1.0f / l;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const int ch = 2 * cc + hf;
                    uint32_t orr[32];
                    tmem_ld32(tmem_o + lane_base + ch * 32, orr);
                    tmem_wait_ld();
                    float vals[32];
#pragma unroll
                    for (int c = 0; c < 32; ++c) vals[c] = __uint_as_float(orr[c]) * inv_l;
                    if (gate && valid) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            const uint4 gv = *reinterpret_cast<const uint4*>(gate + orow + ch * 32 + q4 * 8);
                            const __half2* gh = reinterpret_cast<const __half2*>(&gv);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 gf = __half22float2(gh[e]);
                                vals[q4 * 8 + 2 * e] *= gf.x;
                                vals[q4 * 8 + 2 * e + 1] *= gf.y;
                            }
                        }
                    }
                    if (valid && ok) {
                        OutT* dst = out + orow + ch * 32;          // 32 consecutive outputs of this row: 16-byte stores
                        if constexpr (sizeof(OutT) == 2) {
#pragma unroll
                            for (int q8 = 0; q8 < 4; ++q8) {
                                __half2 h[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(vals[8 * q8 + 2 * e], vals[8 * q8 + 2 * e + 1]);
                                *reinterpret_cast<uint4*>(dst + 8 * q8) = *reinterpret_cast<uint4*>(h);
                            }
                        } else {
#pragma unroll
                            for (int q4 = 0; q4 < 8; ++q4)
                                *reinterpret_cast<float4*>(dst + 4 * q4) =
                                    make_float4(vals[4 * q4], vals[4 * q4 + 1], vals[4 * q4 + 2], vals[4 * q4 + 3]);
                        }
                    }
                }
            } else {
                // Four rounds of 64 columns, alternating between the two P buffers: while the TMA store of one round
                // reads its buffer, the next round is read out of TMEM, converted and staged into the other one.  In a
                // round the thread owns columns [64 k + 32 hf, +32) of its row.
                // The gate: a thread's own row of it lies a 4 KB stride away from its neighbour's, so fetched per row
                // every 16-byte load of a warp touches 32 lines.  It is applied to the staged tile instead, where
                // consecutive threads take consecutive 16-byte pieces of a row (four pieces per thread and round) and
                // the loads coalesce; each round's pieces are requested one round ahead.
                uint4 gst[4];
                const size_t gate_tile = ((size_t)tile.q_row0 * kFaHeads + head) * kHeadDim;
                auto load_gate_round = [&](int k) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int idx = (int)threadIdx.x + 256 * i, grow = idx >> 3, c16 = idx & 7;
                        gst[i] = *reinterpret_cast<const uint4*>(gate + gate_tile + (size_t)grow * kFaHeads * kHeadDim + k * 64 + c16 * 8);
                    }
                };
                if (gate) load_gate_round(0);
                if (!mbar_wait_warp(bar(BAR_OF), it & 1, abort_flag)) ok = false;
                tc_fence_after();
                const float inv_l = 1.0f / l;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    uint32_t orr[32];
                    tmem_ld32(tmem_o + lane_base + (2 * k + hf) * 32, orr);
                    tmem_wait_ld();
                    if (k == 3) {          // this thread has read its part of O: the next item's first PV may overwrite it
                        tc_fence_before();
                        mbar_arrive(bar(BAR_OD));
                    }
                    uint32_t hv[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c)
                        hv[c] = pack_half2(__uint_as_float(orr[2 * c]) * inv_l, __uint_as_float(orr[2 * c + 1]) * inv_l);
                    unsigned char* buf = sm + kOffP + (k & 1) * kPBytes;
                    if (k >= 2) {          // the store of round k - 2 must have read this buffer
                        if (threadIdx.x == 0) bulk_wait_group_read1();
                        asm volatile("bar.sync 5, 256;" ::: "memory");
                    }
                    unsigned char* srow = buf + r * 128;
#pragma unroll
                    for (int q8 = 0; q8 < 4; ++q8)
                        *reinterpret_cast<uint4*>(srow + (((hf * 4 + q8) ^ (r & 7)) << 4)) =
                            make_uint4(hv[4 * q8], hv[4 * q8 + 1], hv[4 * q8 + 2], hv[4 * q8 + 3]);
                    if (gate) {
                        asm volatile("bar.sync 5, 256;" ::: "memory");       // the round's tile is complete
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int idx = (int)threadIdx.x + 256 * i, grow = idx >> 3, c16 = idx & 7;
                            uint4* p4 = reinterpret_cast<uint4*>(buf + grow * 128 + ((c16 ^ (grow & 7)) << 4));
                            uint4 ov = *p4;
                            __half2* oh = reinterpret_cast<__half2*>(&ov);
                            const __half2* gh = reinterpret_cast<const __half2*>(&gst[i]);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 of = __half22float2(oh[e]), gf = __half22float2(gh[e]);
                                oh[e] = __floats2half2_rn(of.x * gf.x, of.y * gf.y);
                            }
                            *p4 = ov;
                        }
                        if (k < 3) load_gate_round(k + 1);
                    }
                    fence_proxy_async_smem();
                    asm volatile("bar.sync 5, 256;" ::: "memory");
                    if (threadIdx.x == 0 && ok) {
                        tma_store_3d(&map_o, base + kOffP + (k & 1) * kPBytes, k * 64, head, tile.q_row0);
                        bulk_commit_group();
                    }
                }
                // the P buffers go back to the softmax of the next item: both stores must have read them
                if (threadIdx.x == 0) bulk_wait_group_read0();
                asm volatile("bar.sync 5, 256;" ::: "memory");
                continue;
            }
            tc_fence_before();
            mbar_arrive(bar(BAR_OD));      // this thread has read its part of O: the next item's first PV may overwrite it
        }
    }
    if (threadIdx.x == 0) bulk_wait_group0();      // this thread's TMA stores have reached global memory
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(error_word, 4);
}

// ---- plain SIMT causal attention (cross-check at sizes the CPU checker cannot reach) ---------------------------
// One warp per (row, head); lane owns dims 8*lane..8*lane+7.  Same inputs / outputs as the tensor-core kernel.
template <typename OutT>
__global__ void __launch_bounds__(128)
fa_prefill_simt_kernel(const __half* __restrict__ q, const __half* __restrict__ ks, const __half* __restrict__ vs,
                       const int* __restrict__ row_pos, const int* __restrict__ row_ctx0, int rows,
                       const __half* __restrict__ gate, OutT* __restrict__ out) {
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (gw >= rows * kFaHeads) return;
    const int row = gw / kFaHeads, head = gw % kFaHeads, kvh = head >> 2;
    const int pos = row_pos[row], ctx0 = row_ctx0[row];
    float qv[8];
    {
        const uint4 raw = *reinterpret_cast<const uint4*>(q + ((size_t)row * kFaHeads + head) * kHeadDim + 8 * lane);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); qv[2 * e] = f.x; qv[2 * e + 1] = f.y; }
    }
    float m = -INFINITY, l = 0.f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int t = 0; t <= pos; ++t) {
        const size_t o = ((size_t)(ctx0 + t) * kFaKvHeads + kvh) * kHeadDim + 8 * lane;
        const uint4 kr = *reinterpret_cast<const uint4*>(ks + o);
        const __half2* kh = reinterpret_cast<const __half2*>(&kr);
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(kh[e]); d += qv[2 * e] * f.x + qv[2 * e + 1] * f.y; }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        d *= 1.0f / 16.0f;
        const float mn = fmaxf(m, d);
        const float a = expf(m - mn), p = expf(d - mn);
        const uint4 vr = *reinterpret_cast<const uint4*>(vs + o);
        const __half2* vh = reinterpret_cast<const __half2*>(&vr);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(vh[e]);
            acc[2 * e] = acc[2 * e] * a + p * f.x;
            acc[2 * e + 1] = acc[2 * e + 1] * a + p * f.y;
        }
        l = l * a + p;
        m = mn;
    }
    const size_t oo = ((size_t)row * kFaHeads + head) * kHeadDim + 8 * lane;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        float r = acc[e] / l;
        if (gate) r *= __half2float(gate[oo + e]);
        out[oo + e] = (OutT)r;
    }
}


// ---- host: tensor maps + launch -------------------------------------------------------------------------------
int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !p)
            B2_FAIL(B200ATTN_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
        fn = reinterpret_cast<EncodeFn>(p);
    }
    cuuint64_t gdims[5], gstr[5];
    cuuint32_t gbox[5], estr[5];
    for (int i = 0; i < rank; ++i) { gdims[i] = dims[i]; gbox[i] = box[i]; estr[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
    CUresult r = fn(out, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstr, gbox, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) B2_FAIL(B200ATTN_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return 0;
}

// q [rows][8][256], kstage/vstage [ctx_rows][2][256] fp16.  d_tiles: device copy of the tile list.
int launch_fa_prefill_tc(const __half* q, int rows, const __half* kstage, const __half* vstage, int ctx_rows,
                         const PrefillTile* d_tiles, int n_tiles, const __half* gate, void* out, bool out_fp16,
                         int* d_error, cudaStream_t s) {
    if (n_tiles <= 0) return 0;
    CUtensorMap mq, mk, mv;
    {
        const uint64_t dims[3] = {(uint64_t)kHeadDim, (uint64_t)kFaHeads, (uint64_t)rows};
        const uint64_t str[2] = {(uint64_t)kHeadDim * 2, (uint64_t)kFaHeads * kHeadDim * 2};
        const uint32_t box[3] = {64, 1, (uint32_t)kBM};
        B2_TRY(make_tensor_map(&mq, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, q, dims, str, box));
    }
    {
        const uint64_t dims[3] = {(uint64_t)kHeadDim, (uint64_t)kFaKvHeads, (uint64_t)ctx_rows};
        const uint64_t str[2] = {(uint64_t)kHeadDim * 2, (uint64_t)kFaKvHeads * kHeadDim * 2};
        const uint32_t box[3] = {64, 1, (uint32_t)kBN};
        B2_TRY(make_tensor_map(&mk, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, kstage, dims, str, box));
        B2_TRY(make_tensor_map(&mv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, vstage, dims, str, box));
    }
    CUtensorMap mo = mq;      // only the fp16 kernel uses it
    if (out_fp16) {
        const uint64_t dims[3] = {(uint64_t)kHeadDim, (uint64_t)kFaHeads, (uint64_t)rows};
        const uint64_t str[2] = {(uint64_t)kHeadDim * 2, (uint64_t)kFaHeads * kHeadDim * 2};
        const uint32_t box[3] = {64, 1, (uint32_t)kBM};
        B2_TRY(make_tensor_map(&mo, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, out, dims, str, box));
    }
    static PerDeviceOnce once;
    B2_PER_DEVICE_ONCE(once,
        B2_CUDA(cudaFuncSetAttribute(fa_prefill_tc_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, kF1Smem));
        B2_CUDA(cudaFuncSetAttribute(fa_prefill_tc_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kF1Smem)));
    int n_sm = 0;
    B2_TRY(device_sm_count(&n_sm));
    const int n_items = n_tiles * kFaHeads;
    dim3 grid(std::min(n_items, n_sm));
    if (out_fp16)
        fa_prefill_tc_kernel<__half><<<grid, kF1Threads, kF1Smem, s>>>(mq, mk, mv, mo, d_tiles, n_items, gate, (__half*)out, d_error);
    else
        fa_prefill_tc_kernel<float><<<grid, kF1Threads, kF1Smem, s>>>(mq, mk, mv, mo, d_tiles, n_items, gate, (float*)out, d_error);
    B2_LAUNCH_CHECK();
    return 0;
}

int launch_fa_prefill_simt(const __half* q, const __half* kstage, const __half* vstage, const int* d_row_pos,
                           const int* d_row_ctx0, int rows, const __half* gate, void* out, bool out_fp16,
                           cudaStream_t s) {
    const int blocks = ceil_div(rows * kFaHeads, 4);
    if (out_fp16)
        fa_prefill_simt_kernel<__half><<<blocks, 128, 0, s>>>(q, kstage, vstage, d_row_pos, d_row_ctx0, rows, gate,
                                                                    (__half*)out);
    else
        fa_prefill_simt_kernel<float><<<blocks, 128, 0, s>>>(q, kstage, vstage, d_row_pos, d_row_ctx0, rows, gate, (float*)out);
    B2_LAUNCH_CHECK();
    return 0;
}

// Tile list for a batch: sequence i has base[i] cached tokens and counts[i] new rows; its context
// occupies staging rows [ctx0[i], ctx0[i] + base[i] + counts[i]).  Longest contexts first.
void build_prefill_tiles(const std::vector<int>& base, const int* counts, const std::vector<int>& ctx0, int n_seqs,
                         std::vector<PrefillTile>& tiles) {
    tiles.clear();
    int row = 0;
    for (int i = 0; i < n_seqs; ++i) {
        for (int r0 = 0; r0 < counts[i]; r0 += kBM)
            tiles.push_back(PrefillTile{row + r0, base[i] + r0, std::min(kBM, counts[i] - r0), ctx0[i]});
        row += counts[i];
    }
    std::stable_sort(tiles.begin(), tiles.end(),
                     [](const PrefillTile& a, const PrefillTile& b) { return a.q_pos0 + a.n_rows > b.q_pos0 + b.n_rows; });
}

}  // namespace b200
