// Decode attention core for callers that must not allocate.
//
// b200attn_fa_decode_core needs an operator handle because the split-KV kernel works through scratch memory
// (the fp16 copy of q and the per-split partial outputs).  Some hosts cannot provide that: a serving loop that
// has been told to stay off cudaMalloc / cudaFree once it is warm (both synchronise the whole device), or a
// plugin that runs under a fixed device-memory budget handed out at load time.  For them this file keeps the
// scratch in a file-scope __device__ array that is part of the loaded module, so the entry point below runs the
// same kernels without creating or freeing anything.
//
// Limits and rules
//   * at most kStaticMaxSeqs sequences per call and a block table of at most kStaticMaxPages pages per sequence;
//     larger requests are refused with B200ATTN_ERR_INVALID;
//   * the array (about 4.3 MB) exists once per GPU that loads the library and stays until the process exits;
//   * every call uses the same array and leaves its intermediate data there.  Only the split arrival counters
//     have to start at zero; the entry point clears them (cudaMemsetAsync on the caller's stream) before each
//     launch.  Two calls that overlap on the GPU (different streams, or different host threads) overwrite each
//     other's partials and counters: serialise them;
//   * the device address of the array is looked up with cudaGetSymbolAddress on the first call made on each
//     device.  Make that first call outside any stream capture.
#include "kernels.cuh"

#include <cstdlib>
#include <mutex>

namespace b200 {

constexpr int kStaticMaxSeqs = 32;
constexpr int kStaticMaxSplits = 16;
constexpr int kStaticMaxPages = 512;     // block-table width the split heuristics are sized for (32768 tokens)
constexpr size_t kStaticQBytes = (size_t)kStaticMaxSeqs * kFaHeads * kHeadDim * sizeof(__half);                         // 128 KB
constexpr size_t kStaticPartOBytes = (size_t)kStaticMaxSeqs * kFaKvHeads * kStaticMaxSplits * 4 * kHeadDim * sizeof(float);  // 4 MB
constexpr size_t kStaticPartMlBytes = (size_t)kStaticMaxSeqs * kFaKvHeads * kStaticMaxSplits * 4 * 2 * sizeof(float);        // 32 KB
constexpr size_t kStaticCounterBytes = (size_t)kStaticMaxSeqs * kFaKvHeads * sizeof(int);                                     // 256 B
constexpr size_t kStaticBytes = kStaticQBytes + kStaticPartOBytes + kStaticPartMlBytes + kStaticCounterBytes;

// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to hand to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

static unsigned char* g_static_ptr[kMaxDevices] = {};
static std::mutex g_static_mu;

// Device address of the scratch array on the current device (looked up once per device).
static int static_scratch_ptr(unsigned char** out) {
    int dev = -1;
    B2_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) B2_FAIL(B200ATTN_ERR_UNSUPPORTED, "fa_decode_core_static: device index %d not supported", dev);
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        B2_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) B2_FAIL(B200ATTN_ERR_CUDA, "fa_decode_core_static: cudaGetSymbolAddress returned a null address");
        g_static_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_static_ptr[dev];
    return 0;
}

}  // namespace b200

using namespace b200;

extern "C" int b200attn_fa_decode_core_static(b200attn_kv_pool pool, int layer, const int* d_slots, int n_seqs,
                                              const float* d_q, float* d_out, b200attn_stream stream) {
    B2_CHECK_ARG(pool && d_slots && d_q && d_out, "fa_decode_core_static: null argument");
    B2_CHECK_ARG(layer >= 0 && layer < pool->cfg.num_layers, "fa_decode_core_static: layer %d out of range", layer);
    B2_CHECK_ARG(n_seqs > 0 && n_seqs <= kStaticMaxSeqs,
                 "fa_decode_core_static: %d sequences, the built-in scratch holds at most %d per call", n_seqs, kStaticMaxSeqs);
    B2_CHECK_ARG(pool->cfg.max_pages_per_seq <= kStaticMaxPages,
                 "fa_decode_core_static: block table of %d pages per sequence, the built-in scratch is sized for %d",
                 pool->cfg.max_pages_per_seq, kStaticMaxPages);
    const KvView kv = pool->view();
    unsigned char* base = nullptr;
    B2_TRY(static_scratch_ptr(&base));
    __half* q16 = reinterpret_cast<__half*>(base);
    float* part_o = reinterpret_cast<float*>(base + kStaticQBytes);
    float* part_ml = reinterpret_cast<float*>(base + kStaticQBytes + kStaticPartOBytes);
    int* counters = reinterpret_cast<int*>(base + kStaticQBytes + kStaticPartOBytes + kStaticPartMlBytes);
    cudaStream_t s = as_stream(stream);
    B2_CUDA(cudaMemsetAsync(counters, 0, kStaticCounterBytes, s));
    B2_TRY(f32_to_f16(s, d_q, q16, (size_t)n_seqs * kFaHeads * kHeadDim));
    return launch_fa_decode(kv, layer, d_slots, n_seqs, q16, nullptr, kStaticMaxSplits, part_o, part_ml, counters, d_out, false, s);
}
