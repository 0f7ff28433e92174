// Gated DeltaNet kernels: causal conv1d + SiLU + L2 norm + gates (sequence form), the fused
// recurrent decode step (conv update + delta rule + gated RMSNorm, one read and one write of the
// state), the token-serial fp32 recurrence used as prefill cross-check, and the gated RMSNorm.
//
// Math follows qwen::LinearAttention::forward
// (src/backend/cpu/core/attention/language_linear_attn.cpp:125-266 in the reference).
// Projection row layout ("mixed"): [0,6144) q|k|v pre-conv, [6144,8192) z, [8192,8208) a, [8208,8224) b.
// Conv state here: [3][6144] with row 0 = oldest (t-3) ... row 2 = newest (t-1); the reference keeps
// [6144][3] with index 0 = newest.  Conv taps: w[d][3] * x_t + w[d][0] * x_{t-1} + w[d][1] * x_{t-2}
// + w[d][2] * x_{t-3} (language_linear_attn.cpp:145-152).
#include "kernels.cuh"
#include "ptx_utils.cuh"

#include <algorithm>
#include <cstdlib>

namespace b200 {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
// SiLU on the special-function unit (ex2.approx + rcp.approx, about 2 ulp): the sequence-form conv kernel evaluates it
// 6144 times per token and is otherwise bound by these instructions, not by memory.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : logf(1.0f + expf(x)); }

// ---- C1, sequence form -------------------------------------------------------------------------------
// One warp per (run of kConvRun consecutive rows, head, part) with part = q, k or v channels of the head: conv +
// SiLU, L2 norm of q and k (eps inside the sqrt), q * 1/sqrt(128); the v warps also produce beta and the log-decay g.
// A warp requests its whole input window (the run's rows plus three rows of history, 16 bytes per lane and row) before
// it computes anything, so every input row leaves HBM once and enough loads are in flight to cover the latency.
// q, k and v are written as fp32 (q_out, k_out, v_out) and / or fp16 (qh_out, kh_out, vh_out, the operand format of the
// tensor-core recurrence); null pointers are skipped.
constexpr int kConvRun = 16;
__global__ void __launch_bounds__(128)
la_conv_seq_kernel(const float* __restrict__ mixed, const int* __restrict__ row_seq,
                   const LaSeqMeta* __restrict__ seqs, const float* __restrict__ conv_state_layer,
                   size_t conv_stride_slot, const float* __restrict__ conv_w, const float* __restrict__ a_log,
                   const float* __restrict__ dt_bias, int rows, float* __restrict__ q_out,
                   float* __restrict__ k_out, __half* __restrict__ qh_out, __half* __restrict__ kh_out,
                   float* __restrict__ v_out, __half* __restrict__ vh_out, float* __restrict__ g_out,
                   float* __restrict__ beta_out) {
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int n_runs = (rows + kConvRun - 1) / kConvRun;
    if (gw >= n_runs * kLaHeads * 3) return;
    const int part = gw % 3, h = (gw / 3) % kLaHeads, run = gw / (3 * kLaHeads);
    const int row_begin = run * kConvRun, n = min(rows - row_begin, kConvRun);
    const int ch = part * (kLaHeads * kLaKd) + h * kLaKd + 4 * lane;   // kd == vd == 128
    float4 w[4];             // tap weights of this lane's four channels
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = *reinterpret_cast<const float4*>(conv_w + (size_t)(ch + i) * kLaConvK);
    const float q_scale = 1.0f / sqrtf((float)kLaKd);
    const int s_first = row_seq[row_begin], s_last = row_seq[row_begin + n - 1];
    float4 x[kConvRun + 3];  // the window: x[i] = input at (first row of the run) - 3 + i
    LaSeqMeta sm = seqs[s_first];
    if (s_first == s_last && n == kConvRun) {
        const int t0 = row_begin - sm.row0;             // index of the run's first row inside this call's chunk of the sequence
        const float* st = conv_state_layer + (size_t)sm.slot * conv_stride_slot;
#pragma unroll
        for (int i = 0; i < kConvRun + 3; ++i) {
            const int tt = t0 - 3 + i;
            const float* src = (tt >= 0) ? mixed + (size_t)(sm.row0 + tt) * kLaProjCols + ch
                                         : st + (size_t)(tt + 3) * kLaConvDim + ch;
            x[i] = *reinterpret_cast<const float4*>(src);
        }
    }
    // conv + SiLU of this lane's four channels for one row, from the four taps oldest .. newest
    auto conv_row = [&](const float4& x0, const float4& x1, const float4& x2, const float4& x3, float (&res)[4]) {
        const float a0[4] = {x0.x, x0.y, x0.z, x0.w}, a1[4] = {x1.x, x1.y, x1.z, x1.w};
        const float a2[4] = {x2.x, x2.y, x2.z, x2.w}, a3[4] = {x3.x, x3.y, x3.z, x3.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float s2 = w[i].w * a3[i];
            s2 += w[i].x * a2[i];
            s2 += w[i].y * a1[i];
            s2 += w[i].z * a0[i];
            res[i] = silu_fast(s2);
        }
    };
    auto store_row = [&](int row, const float (&res)[4], float ss_total) {
        const size_t o = ((size_t)row * kLaHeads + h) * kLaKd + 4 * lane;
        if (part == 2) {
            if (v_out) *reinterpret_cast<float4*>(v_out + o) = make_float4(res[0], res[1], res[2], res[3]);
            if (vh_out) {
                __half2 a = __floats2half2_rn(res[0], res[1]), b = __floats2half2_rn(res[2], res[3]);
                *reinterpret_cast<uint2*>(vh_out + o) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
            }
            return;
        }
        const float inv = ((part == 0) ? q_scale : 1.0f) / sqrtf(ss_total + 1e-6f);     // one division per row, not per channel
        const float4 r4 = make_float4(res[0] * inv, res[1] * inv, res[2] * inv, res[3] * inv);
        float* o32 = (part == 0) ? q_out : k_out;
        __half* o16 = (part == 0) ? qh_out : kh_out;
        if (o32) *reinterpret_cast<float4*>(o32 + o) = r4;
        if (o16) {
            __half2 a = __floats2half2_rn(r4.x, r4.y), b = __floats2half2_rn(r4.z, r4.w);
            *reinterpret_cast<uint2*>(o16 + o) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
        }
    };
    if (s_first == s_last && n == kConvRun) {
        // whole run inside one sequence: straight-line code, eight rows at a time so that the eight row-norm reductions
        // (five shuffle steps each) interleave instead of forming eight serial chains
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float res[8][4], ss[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                const int j = half * 8 + jj;
                conv_row(x[j], x[j + 1], x[j + 2], x[j + 3], res[jj]);
                ss[jj] = res[jj][0] * res[jj][0] + res[jj][1] * res[jj][1] + res[jj][2] * res[jj][2] + res[jj][3] * res[jj][3];
            }
            if (part != 2) {
#pragma unroll
                for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) ss[jj] += __shfl_xor_sync(0xffffffffu, ss[jj], off);
            }
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) store_row(row_begin + half * 8 + jj, res[jj], ss[jj]);
        }
    } else {
        for (int j = 0; j < n; ++j) {
            // short run or a run that crosses into another sequence (a length that is not a multiple of the run): four taps per row
            const int row = row_begin + j;
            sm = seqs[row_seq[row]];
            const int t = row - sm.row0;
            const float* st = conv_state_layer + (size_t)sm.slot * conv_stride_slot;
            float4 xs[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int tt = t - 3 + b;
                const float* src = (tt >= 0) ? mixed + (size_t)(sm.row0 + tt) * kLaProjCols + ch
                                             : st + (size_t)(tt + 3) * kLaConvDim + ch;
                xs[b] = *reinterpret_cast<const float4*>(src);
            }
            float res[4];
            conv_row(xs[0], xs[1], xs[2], xs[3], res);
            float ss = res[0] * res[0] + res[1] * res[1] + res[2] * res[2] + res[3] * res[3];
            if (part != 2) ss = warp_sum_f(ss);
            store_row(row, res, ss);
        }
    }
    if (part == 2 && lane < n) {      // beta and log-decay of the run's rows, one row per lane
        const int row = row_begin + lane;
        const float a = mixed[(size_t)row * kLaProjCols + kLaAOff + h];
        const float b = mixed[(size_t)row * kLaProjCols + kLaBOff + h];
        beta_out[row * kLaHeads + h] = sigmoid_f(b);
        g_out[row * kLaHeads + h] = -expf(a_log[h]) * softplus_f(a + dt_bias[h]);
    }
}

// Conv state after a chunk: the last three inputs of the sequence. grid (n_seqs, 6144/256), block 256.
__global__ void la_conv_state_update_kernel(const float* __restrict__ mixed, const LaSeqMeta* __restrict__ seqs,
                                            float* __restrict__ conv_state_layer, size_t conv_stride_slot) {
    const LaSeqMeta sm = seqs[blockIdx.x];
    const int d = blockIdx.y * blockDim.x + threadIdx.x;
    if (d >= kLaConvDim || sm.count <= 0) return;
    float* st = conv_state_layer + (size_t)sm.slot * conv_stride_slot;
    float old[3] = {st[d], st[kLaConvDim + d], st[2 * kLaConvDim + d]};
    float nw[3];
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        const int tt = sm.count - 3 + j;
        nw[j] = (tt >= 0) ? mixed[(size_t)(sm.row0 + tt) * kLaProjCols + d] : old[tt + 3];
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) st[(size_t)j * kLaConvDim + d] = nw[j];
}

// ---- recurrence, token-serial fp32 (cross-check and small-batch path) ----------------------------------
// grid (heads, n_seqs), block 128: thread vd keeps column S[:, vd] in registers.
__global__ void __launch_bounds__(128)
la_recurrent_serial_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                           const float* __restrict__ g, const float* __restrict__ beta,
                           const LaSeqMeta* __restrict__ seqs, float* __restrict__ rec_layer,
                           size_t rec_stride_slot, float* __restrict__ out) {
    const int h = blockIdx.x;
    const LaSeqMeta sm = seqs[blockIdx.y];
    const int vd = threadIdx.x;
    __shared__ __align__(16) float sq[2][kLaKd];
    __shared__ __align__(16) float sk[2][kLaKd];
    float* Sg = rec_layer + (size_t)sm.slot * rec_stride_slot + (size_t)h * kLaKd * kLaVd;
    float S[kLaKd];
#pragma unroll
    for (int kd = 0; kd < kLaKd; ++kd) S[kd] = Sg[kd * kLaVd + vd];
    if (sm.count > 0) {
        const size_t o = ((size_t)sm.row0 * kLaHeads + h) * kLaKd + vd;
        sq[0][vd] = q[o];
        sk[0][vd] = k[o];
    }
    __syncthreads();
    for (int t = 0; t < sm.count; ++t) {
        const int cur = t & 1;
        const int row = sm.row0 + t;
        const size_t o = ((size_t)row * kLaHeads + h) * kLaKd + vd;
        const float vv = v[o];
        const float gt = expf(g[row * kLaHeads + h]);
        const float bt = beta[row * kLaHeads + h];
        float nq = 0.f, nk = 0.f;
        if (t + 1 < sm.count) { nq = q[o + kLaHeads * kLaKd]; nk = k[o + kLaHeads * kLaKd]; }
        float kv = 0.f;
#pragma unroll
        for (int kd = 0; kd < kLaKd; kd += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(&sk[cur][kd]);
            kv += S[kd] * k4.x; kv += S[kd + 1] * k4.y; kv += S[kd + 2] * k4.z; kv += S[kd + 3] * k4.w;
        }
        const float delta = (vv - gt * kv) * bt;
        float acc = 0.f;
#pragma unroll
        for (int kd = 0; kd < kLaKd; kd += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(&sk[cur][kd]);
            const float4 q4 = *reinterpret_cast<const float4*>(&sq[cur][kd]);
            S[kd] = S[kd] * gt + k4.x * delta;         acc += S[kd] * q4.x;
            S[kd + 1] = S[kd + 1] * gt + k4.y * delta; acc += S[kd + 1] * q4.y;
            S[kd + 2] = S[kd + 2] * gt + k4.z * delta; acc += S[kd + 2] * q4.z;
            S[kd + 3] = S[kd + 3] * gt + k4.w * delta; acc += S[kd + 3] * q4.w;
        }
        out[o] = acc;
        sq[cur ^ 1][vd] = nq;
        sk[cur ^ 1][vd] = nk;
        __syncthreads();
    }
#pragma unroll
    for (int kd = 0; kd < kLaKd; ++kd) Sg[kd * kLaVd + vd] = S[kd];
}

// ---- gated RMSNorm epilogue: o * rsqrt(mean(o^2)+1e-6) * w * silu(z), one warp per (row, head) ------------
template <typename OutT>
__global__ void __launch_bounds__(128)
la_gated_norm_kernel(const float* __restrict__ core, const float* __restrict__ mixed, const float* __restrict__ norm_w,
                     int rows, OutT* __restrict__ out) {
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (gw >= rows * kLaHeads) return;
    const int row = gw / kLaHeads, h = gw % kLaHeads;
    const float4 o4 = *reinterpret_cast<const float4*>(core + ((size_t)row * kLaHeads + h) * kLaVd + 4 * lane);
    const float4 z4 = *reinterpret_cast<const float4*>(mixed + (size_t)row * kLaProjCols + kLaZOff + h * kLaVd + 4 * lane);
    const float4 w4 = *reinterpret_cast<const float4*>(norm_w + 4 * lane);
    float var = o4.x * o4.x + o4.y * o4.y + o4.z * o4.z + o4.w * o4.w;
    var = warp_sum_f(var) / (float)kLaVd;
    const float inv = 1.0f / sqrtf(var + 1e-6f);
    const float r[4] = {o4.x * inv * w4.x * silu_f(z4.x), o4.y * inv * w4.y * silu_f(z4.y),
                        o4.z * inv * w4.z * silu_f(z4.z), o4.w * inv * w4.w * silu_f(z4.w)};
    OutT* dst = out + (size_t)row * (kLaHeads * kLaVd) + h * kLaVd + 4 * lane;
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = (OutT)r[i];
}

// ---- R1: fused recurrent decode step ---------------------------------------------------------------------
// grid (heads, n_seqs), block 32 * 128 / kRows.  Per (sequence, head): conv update of the head's 384 channels,
// L2 norms, gates, then ONE pass over the 128x128 fp32 state: thread (warp r, lane c) keeps rows
// kRows * r .. kRows * r + kRows - 1 of columns 4c..4c+3 in registers between the read (kv = S^T k) and the write
// (S' = g S + k (x) delta, o = S'^T q), followed by the gated RMSNorm.
// kRows = 16: 256 threads, three CTAs per SM.
template <typename OutT, int kMinBlocks, int kRows>
__global__ void __launch_bounds__(32 * 128 / kRows, kMinBlocks)
la_decode_kernel(const float* __restrict__ mixed, const int* __restrict__ slots, int max_seqs,
                 float* __restrict__ rec_layer, size_t rec_stride_slot, float* __restrict__ conv_layer,
                 size_t conv_stride_slot, const float* __restrict__ conv_w, const float* __restrict__ a_log,
                 const float* __restrict__ dt_bias, const float* __restrict__ norm_w, OutT* __restrict__ out,
                 unsigned stagger_ns, unsigned n_sms, unsigned l2_ahead, unsigned long long* stamp) {
    const int h = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slot = slots[b];
    if (slot < 0 || slot >= max_seqs) return;
    __shared__ __align__(16) float s_qkv[3][kLaKd];
    constexpr int kWarpsR = 128 / kRows, kThreadsR = 32 * kWarpsR;
    if (stagger_ns) {
        // The CTAs of the first wave start together and would keep reading, computing and writing in step, so that the
        // memory system sees a burst of reads, a pause, a burst of writes.  The second and third CTA of every SM start a
        // fraction of a CTA's lifetime later; their successors inherit the offset, and the three phases interleave.
        const unsigned k = (blockIdx.y * gridDim.x + blockIdx.x) / n_sms;
        if (k > 0 && k < (unsigned)kMinBlocks) {
            const unsigned long long t0 = global_timer_ns(), span = (unsigned long long)k * stagger_ns;
            while (global_timer_ns() - t0 < span) __nanosleep(100);
        }
    }
    __shared__ __align__(16) float s_part[kWarpsR][kLaVd];
    __shared__ float s_gb[2];
    __shared__ float s_red[4];
    const float* mrow = mixed + (size_t)b * kLaProjCols;
    float* cst = conv_layer + (size_t)slot * conv_stride_slot;
    float* Sg = rec_layer + (size_t)slot * rec_stride_slot + (size_t)h * kLaKd * kLaVd;

    // Issue the state loads first: they are the long pole and do not depend on anything below.
    float4 S[kRows];
    const float* Sp = Sg + (size_t)(warp * kRows) * kLaVd + 4 * lane;
#pragma unroll
    for (int i = 0; i < kRows; ++i) S[i] = __ldcs(reinterpret_cast<const float4*>(Sp + (size_t)i * kLaVd));
    if (l2_ahead && tid == 0) {
        // Ask L2 for the state of the unit that will run `l2_ahead` units later (about one wave): its CTA then finds the
        // state in L2, and HBM keeps streaming while the resident CTAs compute.
        const unsigned nxt = blockIdx.y * gridDim.x + blockIdx.x + l2_ahead;
        if (nxt < gridDim.x * gridDim.y) {
            const int slot2 = slots[nxt / gridDim.x];
            if (slot2 >= 0 && slot2 < max_seqs)
                bulk_prefetch_l2(rec_layer + (size_t)slot2 * rec_stride_slot + (size_t)(nxt % gridDim.x) * kLaKd * kLaVd, kLaKd * kLaVd * 4);
        }
    }
    // The state was last written by this layer's previous step; everything read below comes from the preceding kernel.
    pdl_enter();
    stamp_begin(stamp);

    // conv + SiLU + state shift for the head's q, k, v channels (384 values, 256 threads)
    for (int i = tid; i < 3 * kLaKd; i += kThreadsR) {
        const int part = i / kLaKd, d = i % kLaKd;
        const int ch = part * (kLaHeads * kLaKd) + h * kLaKd + d;
        const float x = mrow[ch];
        const float s0 = cst[ch], s1 = cst[kLaConvDim + ch], s2 = cst[2 * kLaConvDim + ch];
        const float4 w = *reinterpret_cast<const float4*>(conv_w + (size_t)ch * kLaConvK);
        float s = w.w * x;
        s += w.x * s2;
        s += w.y * s1;
        s += w.z * s0;
        s_qkv[part][d] = silu_f(s);
        cst[ch] = s1;
        cst[kLaConvDim + ch] = s2;
        cst[2 * kLaConvDim + ch] = x;
    }
    __syncthreads();
    if (warp < 2) {   // warp 0: q, warp 1: k
        float4 x4 = *reinterpret_cast<float4*>(&s_qkv[warp][4 * lane]);
        float ss = x4.x * x4.x + x4.y * x4.y + x4.z * x4.z + x4.w * x4.w;
        ss = sqrtf(warp_sum_f(ss) + 1e-6f);
        const float sc = (warp == 0) ? 1.0f / sqrtf((float)kLaKd) : 1.0f;
        x4.x = __fdiv_rn(x4.x, ss) * sc; x4.y = __fdiv_rn(x4.y, ss) * sc;
        x4.z = __fdiv_rn(x4.z, ss) * sc; x4.w = __fdiv_rn(x4.w, ss) * sc;
        *reinterpret_cast<float4*>(&s_qkv[warp][4 * lane]) = x4;
    } else if (tid == 64) {
        const float a = mrow[kLaAOff + h], bb = mrow[kLaBOff + h];
        s_gb[0] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
        s_gb[1] = sigmoid_f(bb);
    }
    __syncthreads();
    const float gt = s_gb[0], bt = s_gb[1];

    // pass 1 (registers): partial kv over this warp's rows
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
        const float kk = s_qkv[1][warp * kRows + i];
        acc.x += S[i].x * kk; acc.y += S[i].y * kk; acc.z += S[i].z * kk; acc.w += S[i].w * kk;
    }
    *reinterpret_cast<float4*>(&s_part[warp][4 * lane]) = acc;
    __syncthreads();
    float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < kWarpsR; ++w) {
        const float4 p = *reinterpret_cast<const float4*>(&s_part[w][4 * lane]);
        kv.x += p.x; kv.y += p.y; kv.z += p.z; kv.w += p.w;
    }
    const float4 v4 = *reinterpret_cast<const float4*>(&s_qkv[2][4 * lane]);
    float4 dl;
    dl.x = (v4.x - gt * kv.x) * bt; dl.y = (v4.y - gt * kv.y) * bt;
    dl.z = (v4.z - gt * kv.z) * bt; dl.w = (v4.w - gt * kv.w) * bt;
    __syncthreads();   // s_part is reused below

    // pass 2 (registers): update, write back, partial o
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float* Sw = Sg + (size_t)(warp * kRows) * kLaVd + 4 * lane;
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
        const float kk = s_qkv[1][warp * kRows + i];
        const float qq = s_qkv[0][warp * kRows + i];
        float4 s = S[i];
        s.x = s.x * gt + kk * dl.x; s.y = s.y * gt + kk * dl.y;
        s.z = s.z * gt + kk * dl.z; s.w = s.w * gt + kk * dl.w;
        __stcs(reinterpret_cast<float4*>(Sw + (size_t)i * kLaVd), s);   // (write-through stores measured no better: 57.2 vs 53.5 us)
        acc.x += s.x * qq; acc.y += s.y * qq; acc.z += s.z * qq; acc.w += s.w * qq;
    }
    *reinterpret_cast<float4*>(&s_part[warp][4 * lane]) = acc;
    __syncthreads();

    // o[vd], gated RMSNorm over the head's 128 values
    if (tid < kLaVd) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kWarpsR; ++w) o += s_part[w][tid];
        float ss = warp_sum_f(o * o);
        if (lane == 0) s_red[warp] = ss;
        // warps 0..3 all take this branch, so a named barrier over 128 threads is enough
        asm volatile("bar.sync 1, 128;");
        const float var = (s_red[0] + s_red[1] + s_red[2] + s_red[3]) / (float)kLaVd;
        const float inv = 1.0f / sqrtf(var + 1e-6f);
        const float z = mrow[kLaZOff + h * kLaVd + tid];
        out[(size_t)b * (kLaHeads * kLaVd) + h * kLaVd + tid] = (OutT)(o * inv * norm_w[tid] * silu_f(z));
    }
    if (stamp) {
        __syncthreads();
        stamp_end(stamp);
    }
}

// ---- state import / export in the reference's layouts ------------------------------------------------------
__global__ void la_conv_import_kernel(const float* __restrict__ ref_conv, float* __restrict__ mine) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= kLaConvDim) return;
#pragma unroll
    for (int j = 0; j < 3; ++j) mine[(size_t)j * kLaConvDim + d] = ref_conv[d * 3 + (2 - j)];
}
__global__ void la_conv_export_kernel(const float* __restrict__ mine, float* __restrict__ ref_conv) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= kLaConvDim) return;
#pragma unroll
    for (int j = 0; j < 3; ++j) ref_conv[d * 3 + (2 - j)] = mine[(size_t)j * kLaConvDim + d];
}

// ---- launchers ------------------------------------------------------------------------------------------
int launch_la_conv_seq(const float* mixed, const int* d_row_seq, const LaSeqMeta* d_seqs, const float* conv_layer,
                       size_t conv_stride, const float* conv_w, const float* a_log, const float* dt_bias, int rows,
                       float* q, float* k, __half* qh, __half* kh, float* v, __half* vh, float* g, float* beta, cudaStream_t s) {
    la_conv_seq_kernel<<<ceil_div(ceil_div(rows, kConvRun) * kLaHeads * 3, 4), 128, 0, s>>>(mixed, d_row_seq, d_seqs, conv_layer, conv_stride,
                                                                  conv_w, a_log, dt_bias, rows, q, k, qh, kh, v, vh, g, beta);
    B2_LAUNCH_CHECK();
    return 0;
}
int launch_la_conv_state_update(const float* mixed, const LaSeqMeta* d_seqs, int n_seqs, float* conv_layer,
                                size_t conv_stride, cudaStream_t s) {
    dim3 grid(n_seqs, kLaConvDim / 256);
    la_conv_state_update_kernel<<<grid, 256, 0, s>>>(mixed, d_seqs, conv_layer, conv_stride);
    B2_LAUNCH_CHECK();
    return 0;
}
int launch_la_recurrent_serial(const float* q, const float* k, const float* v, const float* g, const float* beta,
                               const LaSeqMeta* d_seqs, int n_seqs, float* rec_layer, size_t rec_stride, float* out,
                               cudaStream_t s) {
    dim3 grid(kLaHeads, n_seqs);
    la_recurrent_serial_kernel<<<grid, 128, 0, s>>>(q, k, v, g, beta, d_seqs, rec_layer, rec_stride, out);
    B2_LAUNCH_CHECK();
    return 0;
}
int launch_la_gated_norm(const float* core, const float* mixed, const float* norm_w, int rows, void* out,
                         bool out_fp16, cudaStream_t s) {
    const int blocks = ceil_div(rows * kLaHeads, 4);
    if (out_fp16)
        la_gated_norm_kernel<__half><<<blocks, 128, 0, s>>>(core, mixed, norm_w, rows, (__half*)out);
    else
        la_gated_norm_kernel<float><<<blocks, 128, 0, s>>>(core, mixed, norm_w, rows, (float*)out);
    B2_LAUNCH_CHECK();
    return 0;
}
int launch_la_decode(const float* mixed, const int* d_slots, int n_seqs, int max_seqs, float* rec_layer,
                     size_t rec_stride, float* conv_layer, size_t conv_stride, const float* conv_w, const float* a_log,
                     const float* dt_bias, const float* norm_w, void* out, bool out_fp16, bool early_state_loads, cudaStream_t s) {
    dim3 grid(kLaHeads, n_seqs);
    unsigned long long* stamp = prof_stamp_slot(PROF_LA_DECODE);
    int n_sm = 0;
    B2_TRY(device_sm_count(&n_sm));
    // Start offset between the CTAs that share an SM in the first wave (B200ATTN_LA_DECODE_STAGGER_NS, 0 = none).
    // Measured at 128 sequences inside the decode step: 2.317 ms per step without, 2.254 / 2.240 / 2.242 / 2.261 / 2.282
    // with 2000 / 2500 / 3000 / 3500 / 5000 ns; alone 52.8 -> 50.9 us per launch.  Only for launches of at least two
    // full waves: a smaller launch is latency-bound and a delayed start would only lengthen it.
    unsigned stagger_ns = g_flags.la_stagger_ns;
    if (n_seqs * kLaHeads < 2 * 3 * n_sm) stagger_ns = 0;
    // How many units ahead of itself a CTA asks L2 for a state (B200ATTN_LA_DECODE_L2_AHEAD, 0 = off).  Measured at 128
    // sequences with the start offset: 51.7 us without, 48.5 / 48.2 / 48.7 / 49.5 / 51.8 / 54.4 us at 148 / 222 / 296 /
    // 444 / 592 / 888 units.
    const unsigned l2_ahead = g_flags.la_l2_ahead;
    // The kernel requests its state before the programmatic-launch wait.  That is only sound when another kernel that
    // executes the wait runs between two writers of the same state (the decode step of a stack).  A caller that may
    // launch this kernel twice in a row on one layer (the core entry) takes the ordinary stream order instead.
#define LA_DEC(T) launch_pdl_if(early_state_loads, la_decode_kernel<T, 3, 16>, grid, dim3(256), 0, s, mixed, d_slots, max_seqs, rec_layer, \
                                rec_stride, conv_layer, conv_stride, conv_w, a_log, dt_bias, norm_w, (T*)out, stagger_ns, (unsigned)n_sm, l2_ahead, stamp)
    if (out_fp16) LA_DEC(__half); else LA_DEC(float);
#undef LA_DEC
    B2_LAUNCH_CHECK();
    return 0;
}
int launch_la_conv_import(const float* ref_conv, float* mine, cudaStream_t s) {
    la_conv_import_kernel<<<kLaConvDim / 256, 256, 0, s>>>(ref_conv, mine);
    B2_LAUNCH_CHECK();
    return 0;
}
int launch_la_conv_export(const float* mine, float* ref_conv, cudaStream_t s) {
    la_conv_export_kernel<<<kLaConvDim / 256, 256, 0, s>>>(mine, ref_conv);
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200
