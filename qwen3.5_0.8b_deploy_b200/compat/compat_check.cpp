// Exercises the source-compatible classes the way the reference's layer code drives them
// (src/backend/cuda/kernels/cuda_engine.cu:109-156): token-by-token forward against the token-batch entry
// points on the same seeded inputs, for both operators, plus the error conventions.  Exit code 0 = pass.
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
    std::printf(fails ? "compat_check: %d FAILED\n" : "compat_check: PASS\n", fails);
    return fails ? 1 : 0;
}
