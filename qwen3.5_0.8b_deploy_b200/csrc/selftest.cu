// Self-test of the tcgen05 / TMA building blocks: one CTA computes D[128,N] = A[128,K] * B^T with the
// operand formats the prefill kernels rely on (fp16 or tf32 operands, A K-major, B K-major or MN-major,
// 128-byte swizzle, fp32 accumulation in TMEM).  Exposed through the C ABI so a test can localise a
// descriptor problem without going through a full attention kernel.
#include "kernels.cuh"
#include "tc05.cuh"

namespace b200 {

// variant bit0: B is MN-major ([K][N] in memory); bit1: tf32 (else fp16).
// smem: A blocks [K/KB][128 rows][128 B], then B blocks.  KB = elements per 128 bytes (64 fp16 / 32 tf32).
template <bool kTf32, bool kBMn>
__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, int N, int K,
                     float* __restrict__ d_out, int* __restrict__ error_word) {
    constexpr int kElem = kTf32 ? 4 : 2;
    constexpr int kKB = 128 / kElem;            // K (or N) elements per 128-byte swizzle row
    constexpr int kUmmaK = kTf32 ? 8 : 16;      // K per instruction
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = smem_raw + (base - raw);
    const uint32_t a_bytes = 128u * K * kElem, b_bytes = (uint32_t)N * K * kElem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + a_bytes + b_bytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar_load = base + a_bytes + b_bytes, bar_mma = bar_load + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bar_load, 1);
        mbar_init(bar_mma, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(tmem_slot), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (threadIdx.x == 0) {
        mbar_arrive_expect_tx(bar_load, a_bytes + b_bytes);
        for (int kb = 0; kb < K / kKB; ++kb) tma_load_2d(base + kb * (128 * 128), &map_a, bar_load, kb * kKB, 0);
        if (!kBMn) {
            for (int kb = 0; kb < K / kKB; ++kb) tma_load_2d(base + a_bytes + kb * (N * 128), &map_b, bar_load, kb * kKB, 0);
        } else {
            for (int nb = 0; nb < N / kKB; ++nb) tma_load_2d(base + a_bytes + nb * (K * 128), &map_b, bar_load, nb * kKB, 0);
        }
        if (mbar_wait(bar_load, 0, abort_flag)) {
            tc_fence_after();
            const uint32_t idesc = umma_idesc(kTf32 ? kFmtTF32 : kFmtF16, 128, (uint32_t)N, 0, kBMn ? 1 : 0);
            for (int ks = 0; ks < K / kUmmaK; ++ks) {
                const int kb = (ks * kUmmaK) / kKB, kin = (ks * kUmmaK) % kKB;
                const uint64_t a = umma_smem_desc(base + kb * (128 * 128) + kin * kElem, 16, 1024);
                uint64_t b;
                if (!kBMn)
                    b = umma_smem_desc(base + a_bytes + kb * (N * 128) + kin * kElem, 16, 1024);
                else   // K rows are 128 B apart, 8-row groups 1024 B apart, 128-byte runs along N are K*128 B apart
                    b = umma_smem_desc(base + a_bytes + (ks * kUmmaK) * 128, (uint32_t)K * 128, 1024);
                if (kTf32) umma_tf32(tmem, a, b, idesc, ks > 0 ? 1u : 0u);
                else       umma_f16(tmem, a, b, idesc, ks > 0 ? 1u : 0u);
            }
            umma_commit(bar_mma);
        }
    }
    __syncwarp();
    if (mbar_wait_warp(bar_mma, 0, abort_flag)) {
        tc_fence_after();
        const int r = threadIdx.x;
        for (int ch = 0; ch < N / 32; ++ch) {
            uint32_t v[32];
            tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + ch * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; ++c) d_out[(size_t)r * N + ch * 32 + c] = __uint_as_float(v[c]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(error_word, 5);
    (void)lane;
}

}  // namespace b200

using namespace b200;

extern "C" int b200attn_selftest_umma(int variant, int n, int k, const float* d_a, const float* d_b, float* d_d,
                                      b200attn_stream stream) {
    B2_CHECK_ARG(variant >= 0 && variant < 4, "selftest_umma: variant must be 0..3");
    // An MN-major tf32 operand needs the 32-byte-atom form of the 128-byte swizzle, which none of the kernels
    // here use (their MN-major operands are fp16).
    if (variant == 3) B2_FAIL(B200ATTN_ERR_UNSUPPORTED, "selftest_umma: tf32 with an MN-major operand is not built");
    B2_CHECK_ARG(d_a && d_b && d_d, "selftest_umma: null argument");
    const bool tf32 = (variant & 2) != 0, bmn = (variant & 1) != 0;
    const int kb = tf32 ? 32 : 64;
    B2_CHECK_ARG(n == 64 || n == 128 || n == 256, "selftest_umma: N must be 64, 128 or 256");
    B2_CHECK_ARG(k > 0 && k % kb == 0, "selftest_umma: K must be a multiple of %d", kb);
    const int elem = tf32 ? 4 : 2;
    const size_t smem = (size_t)(128 + n) * k * elem + 64 + 1024;
    B2_CHECK_ARG(smem <= 227 * 1024, "selftest_umma: operands (%zu bytes) do not fit shared memory", smem);
    cudaStream_t s = as_stream(stream);
    const void* pa = d_a;
    const void* pb = d_b;
    __half* ha = nullptr;
    __half* hb = nullptr;
    int* d_err = nullptr;
    B2_CUDA(cudaMalloc(&d_err, 4));
    B2_CUDA(cudaMemsetAsync(d_err, 0, 4, s));
    if (!tf32) {
        B2_CUDA(cudaMalloc(&ha, (size_t)128 * k * 2));
        B2_CUDA(cudaMalloc(&hb, (size_t)n * k * 2));
        B2_TRY(f32_to_f16(s, d_a, ha, (size_t)128 * k));
        B2_TRY(f32_to_f16(s, d_b, hb, (size_t)n * k));
        pa = ha; pb = hb;
    }
    const CUtensorMapDataType dt = tf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap ma, mb;
    int st = 0;
    {
        const uint64_t dims[2] = {(uint64_t)k, 128};
        const uint64_t str[1] = {(uint64_t)k * elem};
        const uint32_t box[2] = {(uint32_t)kb, 128};
        st = make_tensor_map(&ma, dt, 2, pa, dims, str, box);
    }
    if (st == 0) {
        if (!bmn) {   // B [N][K]
            const uint64_t dims[2] = {(uint64_t)k, (uint64_t)n};
            const uint64_t str[1] = {(uint64_t)k * elem};
            const uint32_t box[2] = {(uint32_t)kb, (uint32_t)n};
            st = make_tensor_map(&mb, dt, 2, pb, dims, str, box);
        } else {      // B [K][N]
            const uint64_t dims[2] = {(uint64_t)n, (uint64_t)k};
            const uint64_t str[1] = {(uint64_t)n * elem};
            const uint32_t box[2] = {(uint32_t)kb, (uint32_t)k};
            st = make_tensor_map(&mb, dt, 2, pb, dims, str, box);
        }
    }
    if (st == 0) {
        cudaError_t e = cudaSuccess;
#define ST_LAUNCH(T, B)                                                                                              \
    do {                                                                                                             \
        e = cudaFuncSetAttribute(umma_selftest_kernel<T, B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e == cudaSuccess) umma_selftest_kernel<T, B><<<1, 128, smem, s>>>(ma, mb, n, k, d_d, d_err);             \
    } while (0)
        if (tf32 && bmn) ST_LAUNCH(true, true);
        else if (tf32) ST_LAUNCH(true, false);
        else if (bmn) ST_LAUNCH(false, true);
        else ST_LAUNCH(false, false);
#undef ST_LAUNCH
        count_launch();
        if (e == cudaSuccess) e = cudaGetLastError();
        int err = 0;
        if (e == cudaSuccess) e = cudaMemcpyAsync(&err, d_err, 4, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) { set_error("selftest_umma: %s", cudaGetErrorString(e)); st = B200ATTN_ERR_CUDA; }
        else if (err != 0) { set_error("selftest_umma: device status %d (bounded wait ran out)", err); st = B200ATTN_ERR_DEVICE; }
    }
    cudaFree(ha); cudaFree(hb); cudaFree(d_err);
    return st;
}
