// LayerNorm over the last dimension of a row-major [rows, D] tensor; fp32 or fp16 I/O, fp32
// arithmetic.  One launch replaces the reference's three (layer_norm.cl:1-78:
// local_reduction_mean, local_reduction_variance, layer_norm).  Semantics kept: biased variance,
// y = fma((x - mean) / sqrt(var + eps), w[k], b[k]); eps is an argument (the reference fixes it
// at 1e-5, layer_norm.cl:58).
//
// Row-in-registers kernel: one warp owns a row, each lane keeps its 16-byte vectors of the row
// in registers, so mean, exact two-pass variance and the normalised write cost one read and
// one write of the row.  Rows that do not meet the alignment rules, or are too long for the
// register budget, go to a block-per-row kernel that re-reads the row from L1/L2.
#include "common.cuh"
#include "kernels.h"

namespace sdfl {

namespace {

constexpr int kLnThreads = 256;
constexpr int kLnWarps = kLnThreads / 32;

// PREFETCH: the next row of the warp is already on its way into a second register set while
// the current one is reduced and written, so two rows per warp are in flight (the kernel is
// bound by load latency otherwise).  Only for short rows, where the registers allow it.
// Register budget: the more row vectors a lane holds, the fewer CTAs share an SM.
constexpr int ln_min_blocks(int maxv) { return maxv <= 3 ? 6 : maxv <= 6 ? 4 : maxv <= 8 ? 3 : 2; }

template <typename T, int MAXV, bool PREFETCH>
__global__ void __launch_bounds__(kLnThreads, ln_min_blocks(MAXV))
ln_warp_kernel(const T *__restrict__ in, T *__restrict__ out, const float *__restrict__ w,
               const float *__restrict__ b, long long rows, int nvec, int dim, float eps) {
    constexpr int VEC = VecOf<T>::N;
    const int lane = threadIdx.x & 31;
    const long long warp0 = static_cast<long long>(blockIdx.x) * kLnWarps + (threadIdx.x >> 5);
    const long long nwarps = static_cast<long long>(gridDim.x) * kLnWarps;
    const float inv_d = 1.0f / static_cast<float>(dim);
    uint4 v[MAXV], nxt[PREFETCH ? MAXV : 1];

    auto load_row = [&](uint4 (&dst)[MAXV], long long row) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(in + row * dim);
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < nvec) dst[i] = ld_stream(xr + idx);
        }
    };

    if (warp0 < rows) load_row(v, warp0);
    for (long long row = warp0; row < rows; row += nwarps) {
        if (PREFETCH) {
            if (row + nwarps < rows) {
                const uint4 *xr = reinterpret_cast<const uint4 *>(in + (row + nwarps) * dim);
#pragma unroll
                for (int i = 0; i < MAXV; ++i) {
                    const int idx = lane + 32 * i;
                    if (idx < nvec) nxt[i] = ld_stream(xr + idx);
                }
            }
        } else if (row != warp0) {
            load_row(v, row);
        }
        uint4 *yr = reinterpret_cast<uint4 *>(out + row * dim);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            if (lane + 32 * i < nvec) {
                float f[VEC];
                unpack<T>(v[i], f);
#pragma unroll
                for (int j = 0; j < VEC; ++j) s += f[j];
            }
        }
        const float mean = warp_sum(s) * inv_d;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            if (lane + 32 * i < nvec) {
                float f[VEC];
                unpack<T>(v[i], f);
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    const float d = f[j] - mean;
                    q = fmaf(d, d, q);
                }
            }
        }
        const float var = warp_sum(q) * inv_d;
        const float rstd = 1.0f / sqrtf(var + eps);
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < nvec) {
                float f[VEC];
                unpack<T>(v[i], f);
                const float4 *wv = reinterpret_cast<const float4 *>(w + idx * VEC);
                const float4 *bv = reinterpret_cast<const float4 *>(b + idx * VEC);
#pragma unroll
                for (int h = 0; h < VEC / 4; ++h) {
                    const float4 ww = __ldg(wv + h), bb = __ldg(bv + h);
                    f[4 * h + 0] = fmaf((f[4 * h + 0] - mean) * rstd, ww.x, bb.x);
                    f[4 * h + 1] = fmaf((f[4 * h + 1] - mean) * rstd, ww.y, bb.y);
                    f[4 * h + 2] = fmaf((f[4 * h + 2] - mean) * rstd, ww.z, bb.z);
                    f[4 * h + 3] = fmaf((f[4 * h + 3] - mean) * rstd, ww.w, bb.w);
                }
                st_stream(yr + idx, pack<T>(f));
            }
        }
        if (PREFETCH) {
#pragma unroll
            for (int i = 0; i < MAXV; ++i) v[i] = nxt[i];
        }
    }
}

// Any D, any alignment: one CTA per row (grid-stride), three reads of the row.
template <typename T>
__global__ void __launch_bounds__(kLnThreads)
ln_block_kernel(const T *__restrict__ in, T *__restrict__ out, const float *__restrict__ w,
                const float *__restrict__ b, long long rows, long long dim, float eps) {
    __shared__ float red[33];
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *x = in + row * dim;
        T *y = out + row * dim;
        float s = 0.f;
        for (long long i = threadIdx.x; i < dim; i += kLnThreads) s += to_float<T>(x[i]);
        const float mean = block_sum(s, red) / static_cast<float>(dim);
        float q = 0.f;
        for (long long i = threadIdx.x; i < dim; i += kLnThreads) {
            const float d = to_float<T>(x[i]) - mean;
            q = fmaf(d, d, q);
        }
        const float var = block_sum(q, red) / static_cast<float>(dim);
        const float rstd = 1.0f / sqrtf(var + eps);
        for (long long i = threadIdx.x; i < dim; i += kLnThreads)
            y[i] = from_float<T>(fmaf((to_float<T>(x[i]) - mean) * rstd, w[i], b[i]));
        __syncthreads();
    }
}

template <typename T, int MAXV>
void launch_warp(const void *in, void *out, const float *w, const float *b, int64_t rows,
                 int nvec, int dim, float eps, cudaStream_t stream) {
    int64_t blocks = (rows + kLnWarps - 1) / kLnWarps;
    const int64_t cap = 148 * 8 * 4;
    if (blocks > cap) blocks = cap;
    ln_warp_kernel<T, MAXV, false><<<static_cast<unsigned>(blocks), kLnThreads, 0, stream>>>(
        static_cast<const T *>(in), static_cast<T *>(out), w, b, rows, nvec, dim, eps);
}

template <typename T>
cudaError_t ln_dispatch(const void *in, void *out, const float *w, const float *b, int64_t rows,
                        int64_t dim, float eps, cudaStream_t stream) {
    constexpr int VEC = VecOf<T>::N;
    const bool vec_ok = dim % VEC == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0 &&
                        (reinterpret_cast<uintptr_t>(out) & 15u) == 0 &&
                        (reinterpret_cast<uintptr_t>(w) & 15u) == 0 &&
                        (reinterpret_cast<uintptr_t>(b) & 15u) == 0;
    const int64_t nvec = dim / VEC;
    if (vec_ok && nvec <= 32 * 16) {
        const int need = static_cast<int>((nvec + 31) / 32);
        const int nv = static_cast<int>(nvec), d = static_cast<int>(dim);
        if (need <= 1) launch_warp<T, 1>(in, out, w, b, rows, nv, d, eps, stream);
        else if (need <= 2) launch_warp<T, 2>(in, out, w, b, rows, nv, d, eps, stream);
        else if (need <= 3) launch_warp<T, 3>(in, out, w, b, rows, nv, d, eps, stream);
        else if (need <= 4) launch_warp<T, 4>(in, out, w, b, rows, nv, d, eps, stream);
        else if (need <= 5) launch_warp<T, 5>(in, out, w, b, rows, nv, d, eps, stream);
        else if (need <= 6) launch_warp<T, 6>(in, out, w, b, rows, nv, d, eps, stream);
        else if (need <= 8) launch_warp<T, 8>(in, out, w, b, rows, nv, d, eps, stream);
        else if (need <= 10) launch_warp<T, 10>(in, out, w, b, rows, nv, d, eps, stream);
        else if (need <= 12) launch_warp<T, 12>(in, out, w, b, rows, nv, d, eps, stream);
        else launch_warp<T, 16>(in, out, w, b, rows, nv, d, eps, stream);
    } else {
        int64_t blocks = rows < 148 * 8 ? rows : 148 * 8;
        ln_block_kernel<T><<<static_cast<unsigned>(blocks), kLnThreads, 0, stream>>>(
            static_cast<const T *>(in), static_cast<T *>(out), w, b, rows, dim, eps);
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

}  // namespace

cudaError_t ln_launch(const void *in, void *out, const float *w, const float *b, int64_t rows,
                      int64_t dim, float eps, int dtype, cudaStream_t stream) {
    if (rows == 0 || dim == 0) return cudaSuccess;
    return dtype == kF16 ? ln_dispatch<__half>(in, out, w, b, rows, dim, eps, stream)
                         : ln_dispatch<float>(in, out, w, b, rows, dim, eps, stream);
}

}  // namespace sdfl
