// C++ parity test of the operator classes (include/sdfl_operators.hpp) and of the C operator handles
// they wrap (sdfl_groupnorm_create / _op_forward / _destroy ... of include/sdfl.h) against the CPU
// oracle (oracle/libsdfl_oracle.so, linked here as the checker).  Run on a machine with a GPU:
//     tests/cpp/test_operators      -> prints "ok" and exits 0, or the first mismatch and 1.
// Tolerance: |got - want| <= tol + tol * |want| with tol = 1e-5 (fp32 storage).
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <random>
#include <stdexcept>
#include <vector>

#include "../../include/sdfl_operators.hpp"

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
    // The C handles directly: an unaligned fp32 tensor (the path that needs scratch) inside and outside
    // the maximum shape stated at create time; forward must not allocate.
    {
        const size_t B = 2, C = 64, HW = 15 * 15;            // 225 elements per channel: not a multiple of 4
        auto x = randn(B * C * HW + 1, 8, 0.f, 1.f), w = randn(C, 9, 1.f, 0.1f), b = randn(C, 10, 0.f, 0.1f);
        std::vector<float> want(B * C * HW), got(B * C * HW);
        oracle_group_norm(x.data() + 1, want.data(), w.data(), b.data(), B, C, HW, 32, 1e-5f, 0, nullptr, nullptr);
        DeviceBuffer dx, dw, db, dy;
        dx.upload(x); dw.upload(w); db.upload(b);
        dy.reserve(got.size() * 4);
        sdfl_groupnorm *op = nullptr;
        ok &= sdfl_groupnorm_create(&op, 32, 30, 1e-5f, (const float *)dw.get(), (const float *)db.get(), 0, 2, 225, SDFL_F32) == SDFL_ERR_INVALID_VALUE;
        ok &= op == nullptr;
        ok &= sdfl_groupnorm_create(&op, 32, C, 1e-5f, (const float *)dw.get(), (const float *)db.get(), 0, B, HW, SDFL_F32) == SDFL_OK;
        size_t free0 = 0, free1 = 0, total = 0;
        const float *xin = static_cast<const float *>(dx.get()) + 1;      // 4-byte aligned only
        // first call: the driver loads the kernels' code on first use; the second call is measured
        int rc = sdfl_groupnorm_op_forward(op, xin, dy.get(), B, HW, SDFL_F32, nullptr);
        cuda_check(cudaDeviceSynchronize(), "sync");
        ok &= rc == SDFL_OK;
        cuda_check(cudaMemGetInfo(&free0, &total), "cudaMemGetInfo");
        rc = sdfl_groupnorm_op_forward(op, xin, dy.get(), B, HW, SDFL_F32, nullptr);
        cuda_check(cudaDeviceSynchronize(), "sync");
        cuda_check(cudaMemGetInfo(&free1, &total), "cudaMemGetInfo");
        ok &= rc == SDFL_OK && free0 == free1;
        if (free0 != free1) std::printf("forward changed free device memory: %zu -> %zu\n", free0, free1);
        cuda_check(cudaMemcpy(got.data(), dy.get(), got.size() * 4, cudaMemcpyDeviceToHost), "D2H");
        ok &= close(got, want, 1e-5f, "GroupNorm handle, unaligned");
        // beyond the stated maximum on the scratch path (300 images: 9600 slabs need 75 KB of pairs, the
        // handle reserved 64 KB for its 2-image maximum): refused, nothing launched, nothing allocated
        {
            const size_t B2 = 300;
            DeviceBuffer big_in, big_out;
            big_in.reserve((B2 * C * HW + 1) * 4);
            big_out.reserve(B2 * C * HW * 4);
            rc = sdfl_groupnorm_op_forward(op, static_cast<const float *>(big_in.get()) + 1, big_out.get(), B2, HW,
                                           SDFL_F32, nullptr);
            if (rc != SDFL_ERR_WORKSPACE) std::printf("beyond the maximum shape: status %d\n", rc);
            ok &= rc == SDFL_ERR_WORKSPACE;
        }
        ok &= sdfl_groupnorm_destroy(op) == SDFL_OK && sdfl_groupnorm_destroy(nullptr) == SDFL_OK;

        sdfl_geglu *ge = nullptr;
        int64_t shape[2] = {0, 0};
        ok &= sdfl_geglu_create(&ge, 320, 1280) == SDFL_OK && sdfl_geglu_weight_shape(ge, shape) == SDFL_OK;
        ok &= shape[0] == 2560 && shape[1] == 320;
        ok &= sdfl_geglu_destroy(ge) == SDFL_OK;
        sdfl_layernorm *ln = nullptr;
        ok &= sdfl_layernorm_create(&ln, 0, 1e-5f, (const float *)dw.get(), (const float *)db.get()) == SDFL_ERR_INVALID_VALUE;
        ok &= sdfl_layernorm_create(&ln, 64, 1e-5f, (const float *)dw.get(), nullptr) == SDFL_ERR_INVALID_POINTER;
        ok &= sdfl_layernorm_create(&ln, 64, 1e-5f, (const float *)dw.get(), (const float *)db.get()) == SDFL_OK;
        ok &= sdfl_layernorm_destroy(ln) == SDFL_OK;
        std::printf("%-28s %s\n", "C operator handles", ok ? "ok" : "FAILED");
    }
    std::printf(ok ? "ok\n" : "FAILED\n");
    return ok ? 0 : 1;
}
