// Thin inline-PTX helpers shared by the kernels: mbarrier with bounded waits, bulk (TMA) copies,
// warp-level mma.sync for the decode path.  tcgen05 helpers live in tc05.cuh.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace b200 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---- in-kernel time stamps ------------------------------------------------------------------------------
// slot[0] = earliest time a CTA of the launch passed its dependency wait, slot[1] = latest time a CTA finished
// (armed as ~0 / 0 by the host).  slot == nullptr: off.  stamp_end must follow a CTA-wide barrier.
__device__ __forceinline__ void stamp_begin(unsigned long long* slot) {
    if (slot && threadIdx.x == 0) atomicMin(slot, (unsigned long long)global_timer_ns());
}
__device__ __forceinline__ void stamp_end(unsigned long long* slot) {
    if (slot && threadIdx.x == 0) atomicMax(slot + 1, (unsigned long long)global_timer_ns());
}

// ---- mbarrier ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe (try_wait may park the thread for a while when the phase is not complete; a producer that
// polls several barriers must not).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit_ns` or as soon as another thread of the CTA raised *abort_flag.
// Returns false on give-up (and raises the flag), so every role can fall through to the common exit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t limit_ns = 500000000ull) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t it = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++it & 63u) == 0u) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// Warp-uniform form for roles whose next instruction is warp-collective (.sync.aligned): either every
// lane proceeds or every lane gives up.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    const bool r = mbar_wait(bar, parity, abort_flag);
    return __all_sync(0xffffffffu, r);
}

// ---- programmatic dependent launch ---------------------------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may start while its predecessor in the
// stream is still running.  pdl_wait() blocks until the predecessor has completed and its writes are visible: it
// must precede every global read of produced data and every global write.  pdl_launch_dependents() lets the next
// kernel of the stream begin its own prologue.  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() { pdl_wait(); pdl_launch_dependents(); }

// Hint: bring `bytes` (a multiple of 16, 16-byte aligned source) into L2; nothing waits for it.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// ---- bulk async copy global -> shared, completion on an mbarrier (1-D TMA) -----------------------------------
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// shared -> global bulk copy, tracked by the issuing thread's bulk groups.  Both addresses 16-byte aligned, bytes a
// multiple of 16.  The source must have been made visible to the async proxy (fence_proxy_async_smem by the writers).
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }   // sources may be overwritten
__device__ __forceinline__ void bulk_wait_group_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }   // all but the newest group
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }             // writes are complete
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- mma.sync m16n8k16 f16 x f16 -> f32 ------------------------------------------------------------------------
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Transposes an 8x8 matrix of 16-bit elements held one row-pair per lane (lane l: row l/4, columns
// 2(l%4), 2(l%4)+1); afterwards lane l holds elements (2(l%4), l/4) and (2(l%4)+1, l/4).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
// Four signed bytes -> two half2 (b0,b1) and (b2,b3) holding b + 1152 (exact integers 1024..1279): the sign bit is
// flipped and each byte dropped into the mantissa of 1024.0.  For a dot product with a vector q the caller subtracts
// 1152 * sum(q) once instead of subtracting the bias from every element.
__device__ __forceinline__ void cvt_s8x4_half2x2_biased(uint32_t x, uint32_t& lo, uint32_t& hi) {
    x ^= 0x80808080u;
    lo = __byte_perm(x, 0x64646464u, 0x4140);
    hi = __byte_perm(x, 0x64646464u, 0x4342);
}

}  // namespace b200
