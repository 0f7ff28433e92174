// Exercises the source-compatible classes the way the reference's layer code drives them
// (src/backend/cuda/kernels/cuda_engine.cu:109-156): token-by-token forward against the token-batch entry
// points on the same seeded inputs, for both operators, plus the error conventions.  Exit code 0 = pass.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

#include "qwen_cuda_compat.hpp"

using namespace qwen::cuda;

static std::vector<float> rnd(std::mt19937& g, size_t n, float sd) {
    std::normal_distribution<float> d(0.f, sd);
    std::vector<float> v(n);
    for (auto& x : v) x = d(g);
    return v;
}
static float max_diff(const std::vector<float>& a, const std::vector<float>& b) {
    float m = 0.f;
    for (size_t i = 0; i < a.size(); ++i) m = std::fmax(m, std::fabs(a[i] - b[i]));
    return m;
}

// softmax(q K^T / 16) V for 8 query heads over 2 kv heads in double: q [8][256], k / v [L][2][256].
static std::vector<float> attention_ref(const float* q, const std::vector<float>& k, const std::vector<float>& v, int L) {
    std::vector<float> out(8 * 256);
    std::vector<double> p(L);
    for (int h = 0; h < 8; ++h) {
        const int g = h / 4;
        double mx = -1e300;
        for (int t = 0; t < L; ++t) {
            double s = 0;
            for (int d = 0; d < 256; ++d) s += (double)q[h * 256 + d] * k[((size_t)t * 2 + g) * 256 + d];
            p[t] = s / 16.0;
            mx = std::max(mx, p[t]);
        }
        double den = 0;
        for (int t = 0; t < L; ++t) { p[t] = std::exp(p[t] - mx); den += p[t]; }
        for (int d = 0; d < 256; ++d) {
            double acc = 0;
            for (int t = 0; t < L; ++t) acc += p[t] * v[((size_t)t * 2 + g) * 256 + d];
            out[h * 256 + d] = (float)(acc / den);
        }
    }
    return out;
}
template <typename T>
static T* to_device(const std::vector<T>& h) {
    T* d = nullptr;
    cudaMalloc(&d, h.size() * sizeof(T));
    cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d;
}

// The free launchers and cache types that take raw pointers in the reference's layouts.
static int check_free_functions(std::mt19937& gen) {
    int fails = 0;
    const int L = 150, B = 6, MAXS = 256, LAYER = 1;                 // cache of 2 layers x 256 positions, layer 1 in use
    std::vector<float> k = rnd(gen, (size_t)L * 512, 1.0f), v = rnd(gen, (size_t)L * 512, 0.6f), q = rnd(gen, (size_t)B * 8 * 256, 1.0f);
    std::vector<float> kc((size_t)2 * MAXS * 512, 0.f), vc(kc.size(), 0.f);
    std::copy(k.begin(), k.end(), kc.begin() + (size_t)LAYER * MAXS * 512);
    std::copy(v.begin(), v.end(), vc.begin() + (size_t)LAYER * MAXS * 512);
    float *d_k = to_device(k), *d_v = to_device(v), *d_q = to_device(q), *d_kc = to_device(kc), *d_vc = to_device(vc), *d_o = nullptr;
    cudaMalloc(&d_o, (size_t)B * 8 * 256 * 4);
    std::vector<float> got(8 * 256), gotb((size_t)B * 8 * 256);
    // decode, fp32 cache: the last query against all L keys
    flash_attention_decode(d_q + (size_t)(B - 1) * 2048, d_k, d_v, d_o, 8, 2, 256, 256, L);
    cudaMemcpy(got.data(), d_o, got.size() * 4, cudaMemcpyDeviceToHost);
    float d = max_diff(got, attention_ref(q.data() + (size_t)(B - 1) * 2048, k, v, L));
    std::printf("flash_attention_decode: max diff %.3e\n", d);
    if (!(d < 2e-3f)) { ++fails; std::printf("FAIL\n"); }
    // INT8 cache built with the compat quantiser (one scale per token and kv head), decode and prefill over it
    int8_t *d_kq = nullptr, *d_vq = nullptr;
    float *d_ks = nullptr, *d_vs = nullptr, *d_kd = nullptr, *d_vd = nullptr;
    cudaMalloc(&d_kq, kc.size()); cudaMalloc(&d_vq, kc.size());
    cudaMalloc(&d_ks, kc.size() / 256 * 4); cudaMalloc(&d_vs, kc.size() / 256 * 4);
    cudaMalloc(&d_kd, kc.size() * 4); cudaMalloc(&d_vd, kc.size() * 4);
    kv_quantize_fp32_to_int8(d_kc, d_kq, d_ks, (int)kc.size());
    kv_quantize_fp32_to_int8(d_vc, d_vq, d_vs, (int)vc.size());
    kv_dequantize_int8_to_fp32(d_kq, d_ks, d_kd, (int)kc.size());
    kv_dequantize_int8_to_fp32(d_vq, d_vs, d_vd, (int)vc.size());
    std::vector<float> kd(kc.size()), vd(vc.size());
    cudaMemcpy(kd.data(), d_kd, kd.size() * 4, cudaMemcpyDeviceToHost);
    cudaMemcpy(vd.data(), d_vd, vd.size() * 4, cudaMemcpyDeviceToHost);
    float qerr = 0.f;
    for (size_t i = 0; i < kc.size(); ++i) qerr = std::fmax(qerr, std::fabs(kd[i] - kc[i]));
    std::printf("kv_quantize / kv_dequantize round trip: max abs err %.3e\n", qerr);
    if (!(qerr < 0.03f)) { ++fails; std::printf("FAIL\n"); }
    std::vector<float> kdl(kd.begin() + (size_t)LAYER * MAXS * 512, kd.begin() + (size_t)LAYER * MAXS * 512 + (size_t)L * 512);
    std::vector<float> vdl(vd.begin() + (size_t)LAYER * MAXS * 512, vd.begin() + (size_t)LAYER * MAXS * 512 + (size_t)L * 512);
    flash_attention_decode_int8(d_q + (size_t)(B - 1) * 2048, d_kq, d_vq, d_ks, d_vs, d_o, 8, 2, 256, 256, L, LAYER, MAXS);
    cudaMemcpy(got.data(), d_o, got.size() * 4, cudaMemcpyDeviceToHost);
    d = max_diff(got, attention_ref(q.data() + (size_t)(B - 1) * 2048, kdl, vdl, L));
    std::printf("flash_attention_decode_int8: max diff %.3e\n", d);
    if (!(d < 2e-3f)) { ++fails; std::printf("FAIL\n"); }
    // prefill launchers: the B query rows are the last B of the L cached tokens, causal
    auto prefill_ref = [&](const std::vector<float>& kk, const std::vector<float>& vv) {
        std::vector<float> want((size_t)B * 2048);
        for (int i = 0; i < B; ++i) {
            const std::vector<float> o = attention_ref(q.data() + (size_t)i * 2048, kk, vv, L - B + i + 1);
            std::copy(o.begin(), o.end(), want.begin() + (size_t)i * 2048);
        }
        return want;
    };
    launch_flash_attn_v2_prefill(d_q, d_kc, d_vc, d_o, 8, 2, 256, L, B, LAYER, MAXS, 0.0625f);
    cudaDeviceSynchronize();
    cudaMemcpy(gotb.data(), d_o, gotb.size() * 4, cudaMemcpyDeviceToHost);
    d = max_diff(gotb, prefill_ref(k, v));
    std::printf("launch_flash_attn_v2_prefill: max diff %.3e\n", d);
    if (!(d < 2e-3f)) { ++fails; std::printf("FAIL\n"); }
    launch_flash_attn_v2_prefill_int8_cache(d_q, d_kq, d_vq, d_ks, d_vs, d_o, 8, 2, 256, L, B, LAYER, MAXS, 0.0625f);
    cudaDeviceSynchronize();
    cudaMemcpy(gotb.data(), d_o, gotb.size() * 4, cudaMemcpyDeviceToHost);
    d = max_diff(gotb, prefill_ref(kdl, vdl));
    std::printf("launch_flash_attn_v2_prefill_int8_cache: max diff %.3e\n", d);
    if (!(d < 2e-3f)) { ++fails; std::printf("FAIL\n"); }
    {   // half cache
        std::vector<half> kh(kc.size()), vh(vc.size());
        std::vector<float> khf((size_t)L * 512), vhf((size_t)L * 512);
        for (size_t i = 0; i < kc.size(); ++i) { kh[i] = __float2half(kc[i]); vh[i] = __float2half(vc[i]); }
        for (size_t i = 0; i < khf.size(); ++i) {
            khf[i] = __half2float(kh[(size_t)LAYER * MAXS * 512 + i]);
            vhf[i] = __half2float(vh[(size_t)LAYER * MAXS * 512 + i]);
        }
        half *d_kh = to_device(kh), *d_vh = to_device(vh);
        launch_flash_attn_v2_prefill_fp16_cache(d_q, d_kh, d_vh, d_o, 8, 2, 256, L, B, LAYER, MAXS, 0.0625f);
        cudaDeviceSynchronize();
        cudaMemcpy(gotb.data(), d_o, gotb.size() * 4, cudaMemcpyDeviceToHost);
        d = max_diff(gotb, prefill_ref(khf, vhf));
        std::printf("launch_flash_attn_v2_prefill_fp16_cache: max diff %.3e\n", d);
        if (!(d < 2e-3f)) { ++fails; std::printf("FAIL\n"); }
        cudaFree(d_kh); cudaFree(d_vh);
    }
    try { flash_attention_decode(d_q, d_k, d_v, d_o, 4, 2, 256, 256, L); ++fails; std::printf("FAIL: unsupported head count accepted\n"); }
    catch (const std::invalid_argument&) {}
    {   // CudaKVCacheINT8: append three tokens on layer 1, read the last one back
        CudaKVCacheINT8 c;
        c.reset(2, 2, 256, 16);
        for (int t = 0; t < 3; ++t) kv_append_int8(c, d_k + (size_t)t * 512, d_v + (size_t)t * 512, 1);
        kv_get_int8(c, d_kd, d_vd, 1);
        std::vector<float> k2(512), v2(512);
        cudaMemcpy(k2.data(), d_kd, 512 * 4, cudaMemcpyDeviceToHost);
        cudaMemcpy(v2.data(), d_vd, 512 * 4, cudaMemcpyDeviceToHost);
        float e = 0.f;
        for (int i = 0; i < 512; ++i) e = std::fmax(e, std::fmax(std::fabs(k2[i] - k[2 * 512 + i]), std::fabs(v2[i] - v[2 * 512 + i])));
        std::printf("kv_append_int8 / kv_get_int8: lengths %d/%d, max abs err %.3e\n", c.length(0), c.length(1), e);
        if (c.length(1) != 3 || c.length(0) != 0 || !(e < 0.03f) || c.memory_bytes() == 0) { ++fails; std::printf("FAIL\n"); }
        c.clear();
    }
    {   // PagedKVCache bookkeeping (paged_kv.cpp:90-192)
        PagedKVCache pk;
        pk.initialize(6, 2, 256, 64, 8);
        const int a = pk.allocate_sequence(65), b = pk.allocate_sequence(0);
        bool ok = a > 0 && b > 0 && a != b && pk.get_allocated_pages() == 8 && pk.get_used_pages() == 3;
        pk.append_tokens(b, 200);                                    // 1 -> 4 pages
        ok = ok && pk.get_used_pages() == 6;
        pk.shrink_sequence(b, 70);                                   // back to 2 pages
        ok = ok && pk.get_used_pages() == 4;
        const int c = pk.allocate_sequence(64 * 5);                  // 5 pages do not fit any more
        ok = ok && c == -1 && pk.get_used_pages() == 4;
        pk.release_sequence(a);
        ok = ok && pk.get_used_pages() == 2 && pk.get_kv_bytes() > 0 && pk.get_gpu_bytes() >= pk.get_kv_bytes();
        pk.release_sequence(a);                                      // unknown id: ignored, as in the reference
        pk.clear();
        ok = ok && pk.get_used_pages() == 0;
        std::printf("PagedKVCache bookkeeping: %s\n", ok ? "ok" : "FAIL");
        if (!ok) ++fails;
    }
    cudaFree(d_k); cudaFree(d_v); cudaFree(d_q); cudaFree(d_kc); cudaFree(d_vc); cudaFree(d_o);
    cudaFree(d_kq); cudaFree(d_vq); cudaFree(d_ks); cudaFree(d_vs); cudaFree(d_kd); cudaFree(d_vd);
    return fails;
}

int main() {
    const int H = 1024, T = 70;
    std::mt19937 gen(42);
    int fails = 0;
    float *d_in = nullptr, *d_out = nullptr;
    cudaMalloc(&d_in, (size_t)T * H * 4);
    cudaMalloc(&d_out, (size_t)T * H * 4);
    std::vector<float> x = rnd(gen, (size_t)T * H, 1.0f), serial((size_t)T * H), batch((size_t)T * H);
    cudaMemcpy(d_in, x.data(), x.size() * 4, cudaMemcpyHostToDevice);
    {   // gated full attention: 70 x forward == forward_batch_prefill(64) + 6 x forward
        CudaFullAttention fa;
        try { fa.set_weights({}, {}, {}, {}, {}, {}); ++fails; std::printf("FAIL: empty weights accepted\n"); }
        catch (const std::invalid_argument&) {}
        fa.set_weights(rnd(gen, 4096 * 1024, 0.02f), rnd(gen, 512 * 1024, 0.02f), rnd(gen, 512 * 1024, 0.02f),
                       std::vector<float>(256, 0.f), std::vector<float>(256, 0.f), rnd(gen, 1024 * 2048, 0.02f));
        CudaKVCache c1, c2;
        c1.reset(2, 2, 256);
        c2.reset(2, 2, 256);
        for (int t = 0; t < T; ++t) fa.forward(d_in + (size_t)t * H, d_out + (size_t)t * H, c1, 1, t);
        cudaMemcpy(serial.data(), d_out, serial.size() * 4, cudaMemcpyDeviceToHost);
        fa.forward_batch_prefill(d_in, d_out, c2, 1, nullptr, 64);
        for (int t = 64; t < T; ++t) fa.forward(d_in + (size_t)t * H, d_out + (size_t)t * H, c2, 1, t);
        cudaMemcpy(batch.data(), d_out, batch.size() * 4, cudaMemcpyDeviceToHost);
        const float d = max_diff(serial, batch);
        std::printf("CudaFullAttention serial vs batch: max diff %.3e, lengths %d/%d\n", d, c1.length(1), c2.length(1));
        if (!(d < 2e-3f) || c1.length(1) != T || c2.length(1) != T || c1.length(0) != 0) { ++fails; std::printf("FAIL\n"); }
        try { fa.forward(d_in, d_out, c1, 1, 3); ++fails; std::printf("FAIL: stale position accepted\n"); }
        catch (const std::invalid_argument&) {}
        c1.clear();
        if (c1.length(1) != 0) { ++fails; std::printf("FAIL: clear\n"); }
    }
    {   // Gated DeltaNet (fp32-weight V2 class): 70 x forward == forward_batch(70)
        CudaLinearAttentionV2 la;
        la.set_weights(rnd(gen, 6144 * 1024, 0.02f), rnd(gen, 16 * 1024, 0.02f), rnd(gen, 16 * 1024, 0.02f),
                       rnd(gen, 2048 * 1024, 0.02f), rnd(gen, 6144 * 4, 0.02f), rnd(gen, 1024 * 2048, 0.02f),
                       std::vector<float>(16, 1.0f), std::vector<float>(16, 0.1f));
        CudaLinearAttnState s1, s2;
        s1.reset(16, 128, 128);
        s2.reset(16, 128, 128);
        for (int t = 0; t < T; ++t) la.forward(d_in + (size_t)t * H, d_out + (size_t)t * H, s1);
        cudaMemcpy(serial.data(), d_out, serial.size() * 4, cudaMemcpyDeviceToHost);
        la.forward_batch(d_in, d_out, s2, T);
        cudaMemcpy(batch.data(), d_out, batch.size() * 4, cudaMemcpyDeviceToHost);
        const float d = max_diff(serial, batch);
        std::vector<float> r1(16 * 128 * 128), r2(r1.size());
        cudaMemcpy(r1.data(), s1.d_recurrent_state, r1.size() * 4, cudaMemcpyDeviceToHost);
        cudaMemcpy(r2.data(), s2.d_recurrent_state, r2.size() * 4, cudaMemcpyDeviceToHost);
        double num = 0, den = 0;
        for (size_t i = 0; i < r1.size(); ++i) { num += (double)(r1[i] - r2[i]) * (r1[i] - r2[i]); den += (double)r1[i] * r1[i]; }
        std::printf("CudaLinearAttentionV2 serial vs batch: max diff %.3e, state rel %.3e\n", d, std::sqrt(num / den));
        if (!(d < 1e-3f) || !(std::sqrt(num / den) < 1e-3)) { ++fails; std::printf("FAIL\n"); }
        cudaFree(s1.d_recurrent_state); cudaFree(s1.d_conv_state);     // the reference's tests free these by hand
        cudaFree(s2.d_recurrent_state); cudaFree(s2.d_conv_state);
    }
    {   // set_fa_weights forwards to the operator (cuda_engine.hpp:166-169)
        CudaFullAttention fa;
        try { set_fa_weights(&fa, {}, {}, {}, {}, {}, {}, 3); ++fails; std::printf("FAIL: set_fa_weights accepted empty weights\n"); }
        catch (const std::invalid_argument&) {}
    }
    fails += check_free_functions(gen);
    std::printf(fails ? "compat_check: %d FAILED\n" : "compat_check: PASS\n", fails);
    return fails ? 1 : 0;
}
