// C++ parity test of the operator classes (operators.hpp over libsdfl.so) against the CPU
// oracle (oracle/libsdfl_oracle.so, linked here as the checker).  Run on a machine with a GPU:
//     tests/cpp/test_operators      -> prints "ok" and exits 0, or the first mismatch and 1.
// Tolerance: |got - want| <= tol + tol * |want| with tol = 1e-5 (fp32 storage).
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <random>
#include <stdexcept>
#include <vector>

#include "../../mobile-stable-diffusion_b200/csrc/operators.hpp"

extern "C" {
int oracle_group_norm(const float *in, float *out, const float *w, const float *b, size_t batch, size_t C,
                      size_t hw, size_t G, float eps, int apply_silu, float *mean_out, float *var_out);
int oracle_layer_norm(const float *in, float *out, const float *w, const float *b, size_t rows, size_t D,
                      float eps, float *mean_out, float *var_out);
void oracle_gelu_multiply(const float *AB, float *dst, size_t rows, size_t D);
}

static std::vector<float> randn(size_t n, unsigned seed, float mean, float std) {
    std::mt19937 gen(seed);
    std::normal_distribution<float> d(mean, std);
    std::vector<float> v(n);
    for (auto &x : v) x = d(gen);
    return v;
}

static bool close(const std::vector<float> &got, const std::vector<float> &want, float tol, const char *what) {
    double worst = 0;
    for (size_t i = 0; i < got.size(); ++i) {
        const double e = std::fabs(double(got[i]) - want[i]) / (tol + tol * std::fabs(double(want[i])));
        if (!(e <= worst)) worst = e;
    }
    std::printf("%-28s worst error %.3f x tolerance\n", what, worst);
    return worst <= 1.0;
}

int main() {
    using namespace sdfl_ops;
    bool ok = true;
    // GroupNorm(32, 320, 1e-5) + SiLU on [2, 320, 32, 32], in place like nn/ResBlock.cpp:222
    {
        const size_t B = 2, C = 320, HW = 32 * 32;
        auto x = randn(B * C * HW, 1, 0.2f, 1.3f), w = randn(C, 2, 1.f, 0.1f), b = randn(C, 3, 0.f, 0.1f);
        std::vector<float> want(x.size()), got(x.size());
        oracle_group_norm(x.data(), want.data(), w.data(), b.data(), B, C, HW, 32, 1e-5f, 1, nullptr, nullptr);
        GroupNorm gn(32, C, 1e-5f, w, b, /*fuse_silu=*/true);
        gn.init();
        gn.init();
        DeviceBuffer d;
        d.upload(x);
        if (gn.forward(d.get(), d.get(), B, HW, SDFL_F32) != 0) return 1;
        cuda_check(cudaMemcpy(got.data(), d.get(), got.size() * 4, cudaMemcpyDeviceToHost), "D2H");
        ok &= close(got, want, 1e-5f, "GroupNorm+SiLU in place");
        bool threw = false;
        try { GroupNorm(32, 640, 1e-5f, w, b).init(); } catch (const std::runtime_error &) { threw = true; }
        ok &= threw;
        threw = false;
        try { GroupNorm bad(32, 30, 1e-5f, std::vector<float>(30, 1.f), std::vector<float>(30, 0.f));
              bad.init(); bad.forward(d.get(), d.get(), 1, 64, SDFL_F32); }
        catch (const std::runtime_error &) { threw = true; }
        ok &= threw;
    }
    // LayerNorm(768) on [154, 768]
    {
        const size_t R = 154, D = 768;
        auto x = randn(R * D, 4, -0.3f, 2.f), w = randn(D, 5, 1.f, 0.1f), b = randn(D, 6, 0.f, 0.1f);
        std::vector<float> want(x.size()), got(x.size());
        oracle_layer_norm(x.data(), want.data(), w.data(), b.data(), R, D, 1e-5f, nullptr, nullptr);
        LayerNorm ln(D, w, b);
        ln.init();
        DeviceBuffer din, dout;
        din.upload(x);
        dout.reserve(x.size() * 4);
        if (ln.forward(din.get(), dout.get(), R, SDFL_F32) != 0) return 1;
        cuda_check(cudaMemcpy(got.data(), dout.get(), got.size() * 4, cudaMemcpyDeviceToHost), "D2H");
        ok &= close(got, want, 1e-5f, "LayerNorm");
    }
    // GEGLU gate on [64, 2 * 1280]
    {
        const size_t R = 64, D = 1280;
        auto ab = randn(R * 2 * D, 7, 0.f, 1.5f);
        std::vector<float> want(R * D), got(R * D);
        oracle_gelu_multiply(ab.data(), want.data(), R, D);
        GEGLU ge(320, D);
        DeviceBuffer din, dout;
        din.upload(ab);
        dout.reserve(got.size() * 4);
        if (ge.forward(din.get(), dout.get(), R, SDFL_F32) != 0) return 1;
        cuda_check(cudaMemcpy(got.data(), dout.get(), got.size() * 4, cudaMemcpyDeviceToHost), "D2H");
        ok &= close(got, want, 1e-5f, "GEGLU gate");
        ok &= ge.weightShape[0] == 2 * D && ge.weightShape[1] == 320;
    }
    std::printf(ok ? "ok\n" : "FAILED\n");
    return ok ? 0 : 1;
}
