// Paged KV cache: host page bookkeeping, quantise-on-append kernels (standalone and fused with the
// K norm + RoPE epilogue of the qkv projection), Q/gate epilogue, export and staging gather.
//
// Arithmetic of the INT8 path follows fused_kv_cache_int8_kernel
// (src/backend/cuda/kernels/full_attention_cuda.cu:78-148 in the reference): per (token, kv head)
// scale = absmax / 127 (IEEE division), 1.0 if not > 1e-8, code = clamp(roundf(x / scale), +-127).
#include "kernels.cuh"
#include "ptx_utils.cuh"

#include <algorithm>
#include <cmath>

namespace b200 {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void load8(const float* p, float (&x)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

// Per-head RMSNorm with (1 + w) and interleaved-pair RoPE on the first rotary_dim dims.
// Lane l owns dims 8l..8l+7 of a 256-wide head.
// (src/backend/cpu/core/attention/language_full_attn.cpp:81-113 in the reference.)
__device__ __forceinline__ void norm_rope8(float (&x)[8], const float* __restrict__ norm_w,
                                           const float* __restrict__ inv_freq, int pos, int lane) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float rms = sqrtf(ss / (float)kHeadDim + 1e-6f);
    float w[8];
    load8(norm_w + 8 * lane, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = __fdiv_rn(x[i], rms) * (1.0f + w[i]);
    if (lane < kRotaryDim / 8) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            const float ang = (float)pos * inv_freq[(8 * lane + i) >> 1];
            float s, c;
            sincosf(ang, &s, &c);
            const float a = x[i], b = x[i + 1];
            x[i] = a * c - b * s;
            x[i + 1] = a * s + b * c;
        }
    }
}

// INT8 quantisation of one 256-wide head held 8 per lane.
__device__ __forceinline__ float quantize8(const float (&x)[8], int (&code)[8]) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
    amax = warp_max(amax);
    float scale = __fdiv_rn(amax, 127.0f);
    scale = (scale > 1e-8f) ? scale : 1.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float q = roundf(__fdiv_rn(x[i], scale));
        code[i] = (int)fmaxf(-127.0f, fminf(127.0f, q));
    }
    return scale;
}

// grid (n_tiles, kv_heads), block 256.
// Input rows: K from kin[row*k_stride + kvh*256 ..], V from vin[row*v_stride + kvh*256 ..].
template <bool kFp16>
__global__ void __launch_bounds__(256)
kv_append_kernel(KvView kv, int layer, const AppendTile* __restrict__ tiles, const int* __restrict__ slots,
                 const float* __restrict__ kin, int k_stride, const float* __restrict__ vin, int v_stride,
                 int do_norm_rope, const float* __restrict__ k_norm_w, const float* __restrict__ inv_freq,
                 __half* __restrict__ kstage, __half* __restrict__ vstage, const int* __restrict__ stage_row0) {
    using VT = typename std::conditional<kFp16, __half, int8_t>::type;
    __shared__ __align__(16) VT sV[kHeadDim][kPageTokens + (kFp16 ? 8 : 16)];
    const int kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_enter();
    const AppendTile tile = tiles[blockIdx.x];
    const int slot = slots[tile.seq];
    if (slot < 0 || slot >= kv.max_seqs) {
        if (threadIdx.x == 0) atomicExch(kv.error, 1);
        return;
    }
    if (tile.first_pos + tile.ntok > kv.capacity[slot]) {
        if (threadIdx.x == 0) atomicExch(kv.error, 2);   // page not reserved: skip the write
        return;
    }
    const int page_idx = tile.first_pos / kPageTokens;
    const int t0 = tile.first_pos % kPageTokens;
    const int page = kv.block_table[slot * kv.max_pages_per_seq + page_idx];
    const size_t head_base = ((size_t)(layer * kv.num_pages + page) * kFaKvHeads + kvh);
    VT* kpage = reinterpret_cast<VT*>(kv.k) + head_base * (kPageTokens * kHeadDim);
    VT* vpage = reinterpret_cast<VT*>(kv.v) + head_base * (kPageTokens * kHeadDim);
    float* ks = kv.ks ? kv.ks + head_base * kPageTokens : nullptr;
    float* vs = kv.vs ? kv.vs + head_base * kPageTokens : nullptr;
    const int srow0 = (kstage && stage_row0) ? stage_row0[tile.seq] : 0;

    for (int j = warp; j < tile.ntok; j += 8) {
        const int row = tile.first_row + j;
        const int pos = tile.first_pos + j;
        const int t = t0 + j;
        float xk[8], xv[8];
        load8(kin + (size_t)row * k_stride + kvh * kHeadDim + 8 * lane, xk);
        load8(vin + (size_t)row * v_stride + kvh * kHeadDim + 8 * lane, xv);
        if (do_norm_rope) norm_rope8(xk, k_norm_w, inv_freq, pos, lane);
        __half hk[8], hv[8];
        if constexpr (kFp16) {
#pragma unroll
            for (int i = 0; i < 8; ++i) { hk[i] = __float2half_rn(xk[i]); hv[i] = __float2half_rn(xv[i]); }
            *reinterpret_cast<uint4*>(kpage + t * kHeadDim + 8 * lane) = *reinterpret_cast<uint4*>(hk);
#pragma unroll
            for (int i = 0; i < 8; ++i) sV[8 * lane + i][t] = hv[i];
        } else {
            int ck[8], cv[8];
            const float sk = quantize8(xk, ck);
            const float sv = quantize8(xv, cv);
            if (lane == 0) { ks[t] = sk; vs[t] = sv; }
            int8_t bk[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                bk[i] = (int8_t)ck[i];
                sV[8 * lane + i][t] = (int8_t)cv[i];
                hk[i] = __float2half_rn((float)ck[i] * sk);
                hv[i] = __float2half_rn((float)cv[i] * sv);
            }
            *reinterpret_cast<uint2*>(kpage + t * kHeadDim + 8 * lane) = *reinterpret_cast<uint2*>(bk);
        }
        if (kstage) {
            const size_t so = ((size_t)(srow0 + pos) * kFaKvHeads + kvh) * kHeadDim + 8 * lane;
            *reinterpret_cast<uint4*>(kstage + so) = *reinterpret_cast<uint4*>(hk);
            *reinterpret_cast<uint4*>(vstage + so) = *reinterpret_cast<uint4*>(hv);
        }
    }
    __syncthreads();
    // V is stored token-minor: [dim][64 tokens].  Full aligned tiles go out as 16-byte chunks.
    if (tile.ntok == kPageTokens && t0 == 0) {
        constexpr int kChunks = kPageTokens * (int)sizeof(VT) / 16;   // 4 (int8) or 8 (half)
        for (int i = threadIdx.x; i < kHeadDim * kChunks; i += 256) {
            const int d = i / kChunks, c = i % kChunks;
            const uint4 val = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(&sV[d][0]) + 16 * c);
            *reinterpret_cast<uint4*>(reinterpret_cast<char*>(vpage + d * kPageTokens) + 16 * c) = val;
        }
    } else {
        for (int i = threadIdx.x; i < kHeadDim * tile.ntok; i += 256) {
            const int d = i / tile.ntok, j = i % tile.ntok;
            vpage[d * kPageTokens + t0 + j] = sV[d][t0 + j];
        }
    }
}

// After all tiles of a call were written: lens[layer][slot] += count (one thread per sequence).
__global__ void kv_advance_kernel(KvView kv, int layer, const int* __restrict__ slots,
                                  const int* __restrict__ counts, int n_seqs) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_seqs) return;
    const int slot = slots[i];
    if (slot < 0 || slot >= kv.max_seqs) return;
    const int c = counts ? counts[i] : 1;
    const int cur = kv.lens[layer * kv.max_seqs + slot];
    if (cur + c <= kv.capacity[slot]) kv.lens[layer * kv.max_seqs + slot] = cur + c;
}

// Q / gate epilogue of the fused qkv projection: one warp per (row, q head).
// qkv_raw row layout: head h -> [h*512, h*512+256) q, [h*512+256, h*512+512) gate
// (language_full_attn.cpp:133-140).  Writes q (normalised, rotated) and sigmoid(gate) as half.
// pos = row_pos[row].  (The decode step does this work inside fa_decode_pre_kernel.)
__global__ void __launch_bounds__(128)
fa_q_epilogue_kernel(const float* __restrict__ qkv_raw, int rows, const float* __restrict__ q_norm_w,
                     const float* __restrict__ inv_freq, const int* __restrict__ row_pos,
                     __half* __restrict__ q_out, __half* __restrict__ gate_out) {
    pdl_enter();
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (gw >= rows * kFaHeads) return;
    const int row = gw / kFaHeads, h = gw % kFaHeads;
    const int pos = row_pos[row];
    const float* src = qkv_raw + (size_t)row * kFaQkvCols + h * 2 * kHeadDim + 8 * lane;
    float x[8], g[8];
    load8(src, x);
    load8(src + kHeadDim, g);
    norm_rope8(x, q_norm_w, inv_freq, pos, lane);
    __half hq[8], hg[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        hq[i] = __float2half_rn(x[i]);
        hg[i] = __float2half_rn(1.0f / (1.0f + expf(-g[i])));
    }
    const size_t o = ((size_t)row * kFaHeads + h) * kHeadDim + 8 * lane;
    *reinterpret_cast<uint4*>(q_out + o) = *reinterpret_cast<uint4*>(hq);
    *reinterpret_cast<uint4*>(gate_out + o) = *reinterpret_cast<uint4*>(hg);
}

// Decode step, everything between the fused qkv projection and the attention kernel in ONE launch: one CTA per sequence,
// twelve warps = 8 q heads (norm, RoPE, gate: fa_q_epilogue_kernel's work), 2 K heads and 2 V heads of the new token
// (norm / RoPE / quantise-on-append: kv_append_kernel's work for one token), then the sequence's length on this layer
// goes up by one (kv_advance_kernel's work) -- after every warp of the CTA has read the old length, and no other CTA
// touches this sequence.  The attention kernel that follows therefore sees the new length.
template <bool kFp16>
__global__ void __launch_bounds__(384)
fa_decode_pre_kernel(KvView kv, int layer, const int* __restrict__ slots, const float* __restrict__ qkv_raw,
                     const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, const float* __restrict__ inv_freq,
                     __half* __restrict__ q_out, __half* __restrict__ gate_out) {
    using VT = typename std::conditional<kFp16, __half, int8_t>::type;
    pdl_enter();
    const int seq = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = slots[seq];
    if (slot == -1) return;                 // inactive row of a decode batch: nothing is read or written for it
    if (slot < 0 || slot >= kv.max_seqs) {
        if (threadIdx.x == 0) atomicExch(kv.error, 1);
        return;
    }
    const int pos = kv.lens[layer * kv.max_seqs + slot];
    const bool room = pos + 1 <= kv.capacity[slot];
    const float* rowp = qkv_raw + (size_t)seq * kFaQkvCols;
    if (warp < kFaHeads) {
        const int h = warp;
        const float* src = rowp + h * 2 * kHeadDim + 8 * lane;
        float x[8], g[8];
        load8(src, x);
        load8(src + kHeadDim, g);
        norm_rope8(x, q_norm_w, inv_freq, pos, lane);
        __half hq[8], hg[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            hq[i] = __float2half_rn(x[i]);
            hg[i] = __float2half_rn(1.0f / (1.0f + expf(-g[i])));
        }
        const size_t o = ((size_t)seq * kFaHeads + h) * kHeadDim + 8 * lane;
        *reinterpret_cast<uint4*>(q_out + o) = *reinterpret_cast<uint4*>(hq);
        *reinterpret_cast<uint4*>(gate_out + o) = *reinterpret_cast<uint4*>(hg);
    } else if (room) {
        const bool is_v = warp >= kFaHeads + kFaKvHeads;
        const int kvh = (warp - kFaHeads) % kFaKvHeads;
        const int page = kv.block_table[slot * kv.max_pages_per_seq + pos / kPageTokens];
        const int t = pos % kPageTokens;
        const size_t head_base = ((size_t)(layer * kv.num_pages + page) * kFaKvHeads + kvh);
        float x[8];
        load8(rowp + kFaHeads * kHeadDim * 2 + (is_v ? kFaKvHeads * kHeadDim : 0) + kvh * kHeadDim + 8 * lane, x);
        if (!is_v) norm_rope8(x, k_norm_w, inv_freq, pos, lane);
        VT* pg = reinterpret_cast<VT*>(is_v ? kv.v : kv.k) + head_base * (kPageTokens * kHeadDim);
        if constexpr (kFp16) {
            __half hx[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) hx[i] = __float2half_rn(x[i]);
            if (!is_v) {
                *reinterpret_cast<uint4*>(pg + t * kHeadDim + 8 * lane) = *reinterpret_cast<uint4*>(hx);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) pg[(8 * lane + i) * kPageTokens + t] = hx[i];     // token-minor V
            }
        } else {
            int c[8];
            const float sc = quantize8(x, c);
            if (lane == 0) (is_v ? kv.vs : kv.ks)[head_base * kPageTokens + t] = sc;
            if (!is_v) {
                int8_t b[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) b[i] = (int8_t)c[i];
                *reinterpret_cast<uint2*>(pg + t * kHeadDim + 8 * lane) = *reinterpret_cast<uint2*>(b);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) pg[(8 * lane + i) * kPageTokens + t] = (int8_t)c[i];
            }
        }
    }
    __syncthreads();      // every warp has used the old length
    if (threadIdx.x == 0) {
        if (room) kv.lens[layer * kv.max_seqs + slot] = pos + 1;
        else atomicExch(kv.error, 2);               // page not reserved: nothing was written, the length stays
    }
}

// Export one sequence's cache on one layer as token-major arrays. grid (len, kv_heads), block 256.
template <bool kFp16>
__global__ void kv_export_kernel(KvView kv, int layer, int slot, int len, void* k_out, void* v_out,
                                 float* ks_out, float* vs_out) {
    using VT = typename std::conditional<kFp16, __half, int8_t>::type;
    const int tok = blockIdx.x, kvh = blockIdx.y, d = threadIdx.x;
    if (tok >= len) return;
    const int page = kv.block_table[slot * kv.max_pages_per_seq + tok / kPageTokens];
    const int t = tok % kPageTokens;
    const size_t head_base = ((size_t)(layer * kv.num_pages + page) * kFaKvHeads + kvh);
    const VT* kpage = reinterpret_cast<const VT*>(kv.k) + head_base * (kPageTokens * kHeadDim);
    const VT* vpage = reinterpret_cast<const VT*>(kv.v) + head_base * (kPageTokens * kHeadDim);
    const size_t o = ((size_t)tok * kFaKvHeads + kvh) * kHeadDim + d;
    reinterpret_cast<VT*>(k_out)[o] = kpage[t * kHeadDim + d];
    reinterpret_cast<VT*>(v_out)[o] = vpage[d * kPageTokens + t];
    if (!kFp16 && d == 0 && ks_out) {
        ks_out[tok * kFaKvHeads + kvh] = kv.ks[head_base * kPageTokens + t];
        vs_out[tok * kFaKvHeads + kvh] = kv.vs[head_base * kPageTokens + t];
    }
}

// Dequantise the first `base` cached tokens of a sequence into the fp16 staging rows the prefill
// kernel reads (only used when a prefill continues a non-empty cache). grid (base, kv_heads), block 256.
template <bool kFp16>
__global__ void kv_stage_gather_kernel(KvView kv, int layer, int slot, int base, int stage_row0,
                                       __half* kstage, __half* vstage) {
    using VT = typename std::conditional<kFp16, __half, int8_t>::type;
    const int tok = blockIdx.x, kvh = blockIdx.y, d = threadIdx.x;
    if (tok >= base) return;
    const int page = kv.block_table[slot * kv.max_pages_per_seq + tok / kPageTokens];
    const int t = tok % kPageTokens;
    const size_t head_base = ((size_t)(layer * kv.num_pages + page) * kFaKvHeads + kvh);
    const VT* kpage = reinterpret_cast<const VT*>(kv.k) + head_base * (kPageTokens * kHeadDim);
    const VT* vpage = reinterpret_cast<const VT*>(kv.v) + head_base * (kPageTokens * kHeadDim);
    const size_t o = ((size_t)(stage_row0 + tok) * kFaKvHeads + kvh) * kHeadDim + d;
    if constexpr (kFp16) {
        kstage[o] = kpage[t * kHeadDim + d];
        vstage[o] = vpage[d * kPageTokens + t];
    } else {
        kstage[o] = __float2half_rn((float)kpage[t * kHeadDim + d] * kv.ks[head_base * kPageTokens + t]);
        vstage[o] = __float2half_rn((float)vpage[d * kPageTokens + t] * kv.vs[head_base * kPageTokens + t]);
    }
}

// ---- launch helpers used by the operators ------------------------------------------------------------
int launch_kv_append(const KvView& kv, int layer, const AppendTile* d_tiles, int n_tiles, const int* d_slots,
                     const float* kin, int k_stride, const float* vin, int v_stride, bool do_norm_rope,
                     const float* k_norm_w, const float* inv_freq, __half* kstage, __half* vstage,
                     const int* d_stage_row0, cudaStream_t s) {
    if (n_tiles <= 0) return 0;
    dim3 grid(n_tiles, kFaKvHeads);
    if (kv.is_fp16)
        launch_pdl(kv_append_kernel<true>, grid, dim3(256), 0, s, kv, layer, d_tiles, d_slots, kin, k_stride, vin, v_stride,
                   do_norm_rope, k_norm_w, inv_freq, kstage, vstage, d_stage_row0);
    else
        launch_pdl(kv_append_kernel<false>, grid, dim3(256), 0, s, kv, layer, d_tiles, d_slots, kin, k_stride, vin, v_stride,
                   do_norm_rope, k_norm_w, inv_freq, kstage, vstage, d_stage_row0);
    B2_LAUNCH_CHECK();
    return 0;
}

int launch_fa_decode_pre(const KvView& kv, int layer, const int* d_slots, int n_seqs, const float* qkv_raw, const float* q_norm_w,
                         const float* k_norm_w, const float* inv_freq, __half* q_out, __half* gate_out, cudaStream_t s) {
    if (kv.is_fp16)
        launch_pdl(fa_decode_pre_kernel<true>, dim3(n_seqs), dim3(384), 0, s, kv, layer, d_slots, qkv_raw, q_norm_w, k_norm_w, inv_freq,
                   q_out, gate_out);
    else
        launch_pdl(fa_decode_pre_kernel<false>, dim3(n_seqs), dim3(384), 0, s, kv, layer, d_slots, qkv_raw, q_norm_w, k_norm_w, inv_freq,
                   q_out, gate_out);
    B2_LAUNCH_CHECK();
    return 0;
}

int launch_kv_advance(const KvView& kv, int layer, const int* d_slots, const int* d_counts, int n_seqs,
                      cudaStream_t s) {
    launch_pdl(kv_advance_kernel, dim3(ceil_div(n_seqs, 128)), dim3(128), 0, s, kv, layer, d_slots, d_counts, n_seqs);
    B2_LAUNCH_CHECK();
    return 0;
}

int launch_fa_q_epilogue(const float* qkv_raw, int rows, const float* q_norm_w, const float* inv_freq,
                         const int* d_row_pos, __half* q_out, __half* gate_out, cudaStream_t s) {
    const int warps = rows * kFaHeads;
    launch_pdl(fa_q_epilogue_kernel, dim3(ceil_div(warps, 4)), dim3(128), 0, s, qkv_raw, rows, q_norm_w, inv_freq, d_row_pos,
               q_out, gate_out);
    B2_LAUNCH_CHECK();
    return 0;
}

int launch_kv_stage_gather(const KvView& kv, int layer, int slot, int base, int stage_row0, __half* kstage,
                           __half* vstage, cudaStream_t s) {
    if (base <= 0) return 0;
    dim3 grid(base, kFaKvHeads);
    if (kv.is_fp16)
        kv_stage_gather_kernel<true><<<grid, 256, 0, s>>>(kv, layer, slot, base, stage_row0, kstage, vstage);
    else
        kv_stage_gather_kernel<false><<<grid, 256, 0, s>>>(kv, layer, slot, base, stage_row0, kstage, vstage);
    B2_LAUNCH_CHECK();
    return 0;
}

// Builds the per-page tile list of an append on the host. Returns tiles and per-sequence base lengths.
void build_append_tiles(const std::vector<int>& base, const int* h_counts, int n_seqs,
                        std::vector<AppendTile>& tiles) {
    tiles.clear();
    int row = 0;
    for (int i = 0; i < n_seqs; ++i) {
        int pos = base[i], left = h_counts[i];
        while (left > 0) {
            const int room = kPageTokens - pos % kPageTokens;
            const int n = std::min(room, left);
            tiles.push_back(AppendTile{i, row, pos, n});
            row += n; pos += n; left -= n;
        }
    }
}

}  // namespace b200

using namespace b200;

// ---- host side of the pool -------------------------------------------------------------------------------
b200::KvView b200attn_kv_pool_s::view() const {
    KvView v;
    v.k = d_k; v.v = d_v; v.ks = d_ks; v.vs = d_vs;
    v.block_table = d_block_table; v.lens = d_lens; v.capacity = d_capacity; v.error = d_error;
    v.num_pages = cfg.num_pages; v.max_seqs = cfg.max_seqs; v.max_pages_per_seq = cfg.max_pages_per_seq;
    v.is_fp16 = cfg.kv_dtype == B200ATTN_KV_FP16;
    return v;
}

int b200attn_kv_pool_s::sync_lens() {
    if (!lens_dirty) return 0;
    // Decode steps and graph replays advance the lengths on streams the pool does not know (non-blocking streams do not
    // order against the legacy stream a plain cudaMemcpy uses), so wait for the whole device first.
    B2_CUDA(cudaDeviceSynchronize());
    B2_CUDA(cudaMemcpy(h_lens.data(), d_lens, h_lens.size() * sizeof(int), cudaMemcpyDeviceToHost));
    lens_dirty = false;
    return 0;
}

extern "C" int b200attn_kv_pool_create(const b200attn_kv_config* cfg, b200attn_kv_pool* out) {
    B2_CHECK_ARG(cfg && out, "kv_pool_create: null argument");
    B2_CHECK_ARG(cfg->num_layers > 0 && cfg->num_pages > 0 && cfg->max_seqs > 0 && cfg->max_pages_per_seq > 0,
                 "kv_pool_create: all sizes must be > 0");
    if (cfg->num_kv_heads != kFaKvHeads || cfg->head_dim != kHeadDim || cfg->page_tokens != kPageTokens)
        B2_FAIL(B200ATTN_ERR_UNSUPPORTED, "kv_pool_create: kernels are built for kv_heads=2, head_dim=256, page_tokens=64");
    B2_CHECK_ARG(cfg->kv_dtype == B200ATTN_KV_INT8 || cfg->kv_dtype == B200ATTN_KV_FP16, "kv_pool_create: bad kv_dtype");
    auto* p = new (std::nothrow) b200attn_kv_pool_s();
    if (!p) B2_FAIL(B200ATTN_ERR_NOMEM, "kv_pool_create: host allocation failed");
    p->cfg = *cfg;
    p->elem_bytes = cfg->kv_dtype == B200ATTN_KV_FP16 ? 2 : 1;
    const size_t elems = (size_t)cfg->num_layers * p->layer_stride_elems();
    const size_t nscale = elems / kHeadDim;
    int st = 0;
    auto fail = [&](int code) { b200attn_kv_pool_destroy(p); return code; };
#define POOL_CUDA(e) do { cudaError_t _e = (e); if (_e != cudaSuccess) { set_error("%s: %s", #e, cudaGetErrorString(_e)); \
        return fail(_e == cudaErrorMemoryAllocation ? B200ATTN_ERR_NOMEM : B200ATTN_ERR_CUDA); } } while (0)
    POOL_CUDA(cudaMalloc(&p->d_k, elems * p->elem_bytes));
    POOL_CUDA(cudaMalloc(&p->d_v, elems * p->elem_bytes));
    POOL_CUDA(cudaMemset(p->d_k, 0, elems * p->elem_bytes));
    POOL_CUDA(cudaMemset(p->d_v, 0, elems * p->elem_bytes));
    if (cfg->kv_dtype == B200ATTN_KV_INT8) {
        POOL_CUDA(cudaMalloc(&p->d_ks, nscale * sizeof(float)));
        POOL_CUDA(cudaMalloc(&p->d_vs, nscale * sizeof(float)));
        POOL_CUDA(cudaMemset(p->d_ks, 0, nscale * sizeof(float)));
        POOL_CUDA(cudaMemset(p->d_vs, 0, nscale * sizeof(float)));
    }
    const size_t bt = (size_t)cfg->max_seqs * cfg->max_pages_per_seq;
    POOL_CUDA(cudaMalloc(&p->d_block_table, bt * sizeof(int)));
    POOL_CUDA(cudaMemset(p->d_block_table, 0, bt * sizeof(int)));
    POOL_CUDA(cudaMalloc(&p->d_lens, (size_t)cfg->num_layers * cfg->max_seqs * sizeof(int)));
    POOL_CUDA(cudaMemset(p->d_lens, 0, (size_t)cfg->num_layers * cfg->max_seqs * sizeof(int)));
    POOL_CUDA(cudaMalloc(&p->d_capacity, cfg->max_seqs * sizeof(int)));
    POOL_CUDA(cudaMemset(p->d_capacity, 0, cfg->max_seqs * sizeof(int)));
    POOL_CUDA(cudaMalloc(&p->d_error, sizeof(int)));
    POOL_CUDA(cudaMemset(p->d_error, 0, sizeof(int)));
#undef POOL_CUDA
    (void)st;
    p->h_lens.assign((size_t)cfg->num_layers * cfg->max_seqs, 0);
    p->seq_pages.assign(cfg->max_seqs, {});
    p->slot_used.assign(cfg->max_seqs, 0);
    p->h_block_table.assign(bt, 0);
    p->h_capacity.assign(cfg->max_seqs, 0);
    p->free_pages.reserve(cfg->num_pages);
    for (int i = cfg->num_pages - 1; i >= 0; --i) p->free_pages.push_back(i);   // pop_back hands out page 0 first
    *out = p;
    return 0;
}

extern "C" int b200attn_kv_pool_destroy(b200attn_kv_pool p) {
    if (!p) return 0;
    cudaFree(p->d_k); cudaFree(p->d_v); cudaFree(p->d_ks); cudaFree(p->d_vs);
    cudaFree(p->d_block_table); cudaFree(p->d_lens); cudaFree(p->d_capacity); cudaFree(p->d_error);
    cudaFree(p->d_meta);
    delete p;
    return 0;
}

// Host -> device copy of small bookkeeping data that kernels on ANY stream may read next: a pageable cudaMemcpy may
// return while its DMA is still in flight on the legacy stream, which non-blocking streams do not wait for, so the
// copy is followed by a wait on that stream.
static int push_ints(int* d_dst, const int* h_src, size_t n) {
    B2_CUDA(cudaMemcpy(d_dst, h_src, n * sizeof(int), cudaMemcpyHostToDevice));
    B2_CUDA(cudaStreamSynchronize(cudaStreamLegacy));
    return 0;
}

static int pool_push_tables(b200attn_kv_pool p, int slot) {
    const int w = p->cfg.max_pages_per_seq;
    B2_TRY(push_ints(p->d_block_table + (size_t)slot * w, p->h_block_table.data() + (size_t)slot * w, w));
    return push_ints(p->d_capacity + slot, p->h_capacity.data() + slot, 1);
}

// Sets the slot's length to zero on every layer, on the host mirror and on the device.
static int pool_zero_lens(b200attn_kv_pool p, int slot) {
    B2_TRY(p->sync_lens());
    const int zero = 0;
    for (int l = 0; l < p->cfg.num_layers; ++l) {
        p->h_lens[(size_t)l * p->cfg.max_seqs + slot] = 0;
        B2_TRY(push_ints(p->d_lens + (size_t)l * p->cfg.max_seqs + slot, &zero, 1));
    }
    return 0;
}

extern "C" int b200attn_kv_seq_reserve(b200attn_kv_pool p, int slot, int total_tokens) {
    B2_CHECK_ARG(p, "kv_seq_reserve: null pool");
    B2_CHECK_ARG(slot >= 0 && slot < p->cfg.max_seqs && p->slot_used[slot], "kv_seq_reserve: slot %d is not allocated", slot);
    B2_CHECK_ARG(total_tokens >= 0, "kv_seq_reserve: negative token count");
    const int need = ceil_div(total_tokens, kPageTokens);
    auto& pages = p->seq_pages[slot];
    if (need <= (int)pages.size()) return 0;
    if (need > p->cfg.max_pages_per_seq)
        B2_FAIL(B200ATTN_ERR_NOMEM, "kv_seq_reserve: %d tokens need %d pages, block table holds %d", total_tokens,
                need, p->cfg.max_pages_per_seq);
    if (need - (int)pages.size() > (int)p->free_pages.size())
        B2_FAIL(B200ATTN_ERR_NOMEM, "kv_seq_reserve: page pool exhausted (%zu free, %d needed)", p->free_pages.size(),
                need - (int)pages.size());
    while ((int)pages.size() < need) {
        const int pg = p->free_pages.back();
        p->free_pages.pop_back();
        p->h_block_table[(size_t)slot * p->cfg.max_pages_per_seq + pages.size()] = pg;
        pages.push_back(pg);
    }
    p->h_capacity[slot] = (int)pages.size() * kPageTokens;
    return pool_push_tables(p, slot);
}

extern "C" int b200attn_kv_seq_alloc(b200attn_kv_pool p, int reserve_tokens, int* slot_out) {
    B2_CHECK_ARG(p && slot_out, "kv_seq_alloc: null argument");
    int slot = -1;
    for (int i = 0; i < p->cfg.max_seqs; ++i)
        if (!p->slot_used[i]) { slot = i; break; }
    if (slot < 0) B2_FAIL(B200ATTN_ERR_NOMEM, "kv_seq_alloc: all %d slots in use", p->cfg.max_seqs);
    p->slot_used[slot] = 1;
    p->seq_pages[slot].clear();
    p->h_capacity[slot] = 0;
    B2_TRY(pool_zero_lens(p, slot));
    int st = b200attn_kv_seq_reserve(p, slot, reserve_tokens);
    if (st != 0) { p->slot_used[slot] = 0; return st; }
    if (reserve_tokens == 0) B2_TRY(pool_push_tables(p, slot));
    *slot_out = slot;
    return 0;
}

extern "C" int b200attn_kv_seq_free(b200attn_kv_pool p, int slot) {
    B2_CHECK_ARG(p, "kv_seq_free: null pool");
    B2_CHECK_ARG(slot >= 0 && slot < p->cfg.max_seqs && p->slot_used[slot], "kv_seq_free: slot %d is not allocated", slot);
    // The slot's lengths go to zero first: a decode launch that still names the slot then writes its defined zero output
    // instead of attending over pages that may already belong to another sequence.
    B2_TRY(pool_zero_lens(p, slot));
    for (int pg : p->seq_pages[slot]) p->free_pages.push_back(pg);
    p->seq_pages[slot].clear();
    p->slot_used[slot] = 0;
    p->h_capacity[slot] = 0;
    return pool_push_tables(p, slot);
}

extern "C" int b200attn_kv_seq_shrink(b200attn_kv_pool p, int slot, int new_len) {
    B2_CHECK_ARG(p, "kv_seq_shrink: null pool");
    B2_CHECK_ARG(slot >= 0 && slot < p->cfg.max_seqs && p->slot_used[slot], "kv_seq_shrink: slot %d is not allocated", slot);
    B2_CHECK_ARG(new_len >= 0, "kv_seq_shrink: negative length");
    B2_TRY(p->sync_lens());
    // every layer's length drops to new_len (layers that hold fewer tokens keep theirs)
    for (int l = 0; l < p->cfg.num_layers; ++l) {
        int& len = p->h_lens[(size_t)l * p->cfg.max_seqs + slot];
        if (new_len < len) {
            len = new_len;
            B2_TRY(push_ints(p->d_lens + (size_t)l * p->cfg.max_seqs + slot, &len, 1));
        }
    }
    // pages wholly behind the new end go back to the pool; like the reference, a sequence keeps at least one page
    auto& pages = p->seq_pages[slot];
    const int keep = std::max(1, ceil_div(new_len, kPageTokens));
    if ((int)pages.size() <= keep) return 0;
    while ((int)pages.size() > keep) {
        p->free_pages.push_back(pages.back());
        pages.pop_back();
    }
    p->h_capacity[slot] = (int)pages.size() * kPageTokens;
    return pool_push_tables(p, slot);
}

extern "C" int b200attn_kv_clear(b200attn_kv_pool p, b200attn_stream stream) {
    B2_CHECK_ARG(p, "kv_clear: null pool");
    B2_CUDA(cudaMemsetAsync(p->d_lens, 0, p->h_lens.size() * sizeof(int), as_stream(stream)));
    std::fill(p->h_lens.begin(), p->h_lens.end(), 0);
    p->lens_dirty = false;
    return 0;
}

extern "C" int b200attn_kv_seq_len(b200attn_kv_pool p, int layer, int slot, int* len_out) {
    B2_CHECK_ARG(p && len_out, "kv_seq_len: null argument");
    B2_CHECK_ARG(layer >= 0 && layer < p->cfg.num_layers && slot >= 0 && slot < p->cfg.max_seqs, "kv_seq_len: index out of range");
    B2_TRY(p->sync_lens());
    *len_out = p->h_lens[(size_t)layer * p->cfg.max_seqs + slot];
    return 0;
}

extern "C" int b200attn_kv_pages(b200attn_kv_pool p, int* total_out, int* used_out) {
    B2_CHECK_ARG(p, "kv_pages: null pool");
    if (total_out) *total_out = p->cfg.num_pages;
    if (used_out) *used_out = p->cfg.num_pages - (int)p->free_pages.size();
    return 0;
}

extern "C" int b200attn_kv_device_status(b200attn_kv_pool p, int* code_out) {
    B2_CHECK_ARG(p && code_out, "kv_device_status: null argument");
    B2_CUDA(cudaDeviceSynchronize());
    B2_CUDA(cudaMemcpy(code_out, p->d_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (*code_out != 0) B2_CUDA(cudaMemset(p->d_error, 0, sizeof(int)));
    return 0;
}

namespace b200 {
// Grows a device int scratch buffer (never shrinks).  Not capture-safe; callers on captured paths
// size their buffers at create time instead.
int ensure_meta(int** d_meta, int* cap, int need) {
    if (need <= *cap) return 0;
    if (*d_meta) B2_CUDA(cudaFree(*d_meta));
    *d_meta = nullptr;
    int n = std::max(need, 1024);
    B2_CUDA(cudaMalloc(d_meta, (size_t)n * sizeof(int)));
    *cap = n;
    return 0;
}

// Validates slots/counts of a host-described batch against the pool, reserves pages and returns the
// per-sequence base lengths on `layer`.
int pool_prepare_append(b200attn_kv_pool p, int layer, const int* h_slots, const int* h_counts, int n_seqs,
                        std::vector<int>& base, int* total_rows) {
    B2_CHECK_ARG(p && h_slots && h_counts, "append: null argument");
    B2_CHECK_ARG(layer >= 0 && layer < p->cfg.num_layers, "append: layer %d out of range", layer);
    B2_CHECK_ARG(n_seqs > 0, "append: n_seqs must be > 0");
    B2_TRY(p->sync_lens());
    base.resize(n_seqs);
    int rows = 0;
    for (int i = 0; i < n_seqs; ++i) {
        const int s = h_slots[i];
        B2_CHECK_ARG(s >= 0 && s < p->cfg.max_seqs && p->slot_used[s], "append: slot %d is not allocated", s);
        B2_CHECK_ARG(h_counts[i] >= 0, "append: negative count");
        for (int j = 0; j < i; ++j) B2_CHECK_ARG(h_slots[j] != s, "append: slot %d listed twice", s);
        base[i] = p->h_lens[(size_t)layer * p->cfg.max_seqs + s];
        B2_TRY(b200attn_kv_seq_reserve(p, s, base[i] + h_counts[i]));
        rows += h_counts[i];
    }
    *total_rows = rows;
    return 0;
}
}  // namespace b200

extern "C" int b200attn_kv_append(b200attn_kv_pool p, int layer, const int* h_slots, const int* h_counts, int n_seqs,
                                  const float* d_k, const float* d_v, b200attn_stream stream) {
    B2_CHECK_ARG(d_k && d_v, "kv_append: null K/V");
    std::vector<int> base;
    int rows = 0;
    B2_TRY(pool_prepare_append(p, layer, h_slots, h_counts, n_seqs, base, &rows));
    if (rows == 0) return 0;
    std::vector<AppendTile> tiles;
    build_append_tiles(base, h_counts, n_seqs, tiles);
    const int need = 2 * n_seqs + 4 * (int)tiles.size();
    cudaStream_t s = as_stream(stream);
    B2_CUDA(cudaStreamSynchronize(s));   // previous users of the meta buffer
    B2_TRY(ensure_meta(&p->d_meta, &p->meta_cap, need));
    int* d_slots = p->d_meta;
    int* d_counts = p->d_meta + n_seqs;
    AppendTile* d_tiles = reinterpret_cast<AppendTile*>(p->d_meta + 2 * n_seqs);
    B2_CUDA(cudaMemcpyAsync(d_slots, h_slots, n_seqs * sizeof(int), cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaMemcpyAsync(d_counts, h_counts, n_seqs * sizeof(int), cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaMemcpyAsync(d_tiles, tiles.data(), tiles.size() * sizeof(AppendTile), cudaMemcpyHostToDevice, s));
    B2_CUDA(cudaStreamSynchronize(s));   // host vectors go out of scope
    const int w = kFaKvHeads * kHeadDim;
    B2_TRY(launch_kv_append(p->view(), layer, d_tiles, (int)tiles.size(), d_slots, d_k, w, d_v, w, false, nullptr,
                            nullptr, nullptr, nullptr, nullptr, s));
    B2_TRY(launch_kv_advance(p->view(), layer, d_slots, d_counts, n_seqs, s));
    for (int i = 0; i < n_seqs; ++i) p->h_lens[(size_t)layer * p->cfg.max_seqs + h_slots[i]] += h_counts[i];
    return 0;
}

extern "C" int b200attn_kv_export(b200attn_kv_pool p, int layer, int slot, void* d_k_codes, void* d_v_codes,
                                  float* d_k_scale, float* d_v_scale, int max_tokens, b200attn_stream stream) {
    B2_CHECK_ARG(p && d_k_codes && d_v_codes, "kv_export: null argument");
    B2_CHECK_ARG(layer >= 0 && layer < p->cfg.num_layers, "kv_export: layer out of range");
    B2_CHECK_ARG(slot >= 0 && slot < p->cfg.max_seqs && p->slot_used[slot], "kv_export: slot %d is not allocated", slot);
    B2_TRY(p->sync_lens());
    const int len = p->h_lens[(size_t)layer * p->cfg.max_seqs + slot];
    B2_CHECK_ARG(len <= max_tokens, "kv_export: sequence holds %d tokens, buffer %d", len, max_tokens);
    if (len == 0) return 0;
    const bool fp16 = p->cfg.kv_dtype == B200ATTN_KV_FP16;
    B2_CHECK_ARG(fp16 || (d_k_scale && d_v_scale), "kv_export: INT8 pool needs scale buffers");
    dim3 grid(len, kFaKvHeads);
    if (fp16)
        kv_export_kernel<true><<<grid, 256, 0, as_stream(stream)>>>(p->view(), layer, slot, len, d_k_codes, d_v_codes, nullptr, nullptr);
    else
        kv_export_kernel<false><<<grid, 256, 0, as_stream(stream)>>>(p->view(), layer, slot, len, d_k_codes, d_v_codes, d_k_scale, d_v_scale);
    B2_LAUNCH_CHECK();
    return 0;
}
