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

// Per-vector arithmetic.  For fp16 storage the mixed-precision add / sub (f16 operand, f32
// result) widens and combines in one instruction, so no separate conversions are issued.
template <typename T> struct LnVec;

template <> struct LnVec<float> {
    static __device__ __forceinline__ void sum(const uint4 &v, float (&s)[2]) {
        s[0] += __uint_as_float(v.x); s[1] += __uint_as_float(v.y);
        s[0] += __uint_as_float(v.z); s[1] += __uint_as_float(v.w);
    }
    static __device__ __forceinline__ void sq(const uint4 &v, float mean, float (&q)[2]) {
        const float d0 = __uint_as_float(v.x) - mean, d1 = __uint_as_float(v.y) - mean;
        const float d2 = __uint_as_float(v.z) - mean, d3 = __uint_as_float(v.w) - mean;
        q[0] = fmaf(d0, d0, q[0]); q[1] = fmaf(d1, d1, q[1]);
        q[0] = fmaf(d2, d2, q[0]); q[1] = fmaf(d3, d3, q[1]);
    }
    struct WB { float4 ww, bb; };
    static __device__ __forceinline__ WB load_wb(const float *w, const float *b) {
        return WB{*reinterpret_cast<const float4 *>(w), *reinterpret_cast<const float4 *>(b)};
    }
    static __device__ __forceinline__ uint4 norm(const uint4 &v, float mean, float rstd, const WB &k) {
        const float4 ww = k.ww, bb = k.bb;
        uint4 o;
        o.x = __float_as_uint(fmaf((__uint_as_float(v.x) - mean) * rstd, ww.x, bb.x));
        o.y = __float_as_uint(fmaf((__uint_as_float(v.y) - mean) * rstd, ww.y, bb.y));
        o.z = __float_as_uint(fmaf((__uint_as_float(v.z) - mean) * rstd, ww.z, bb.z));
        o.w = __float_as_uint(fmaf((__uint_as_float(v.w) - mean) * rstd, ww.w, bb.w));
        return o;
    }
};

__device__ __forceinline__ void ln_sum_half2(uint32_t packed, float (&s)[2]) {
    asm("{\n .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %2;\n"
        " add.rn.f32.f16 %0, lo, %0;\n add.rn.f32.f16 %1, hi, %1;\n}\n"
        : "+f"(s[0]), "+f"(s[1]) : "r"(packed));
}
__device__ __forceinline__ void ln_sq_half2(uint32_t packed, float mean, float (&q)[2]) {
    asm("{\n .reg .b16 lo, hi;\n .reg .f32 d0, d1;\n mov.b32 {lo, hi}, %2;\n"
        " sub.rn.f32.f16 d0, lo, %3;\n sub.rn.f32.f16 d1, hi, %3;\n"
        " fma.rn.f32 %0, d0, d0, %0;\n fma.rn.f32 %1, d1, d1, %1;\n}\n"
        : "+f"(q[0]), "+f"(q[1]) : "r"(packed), "f"(mean));
}
// (x - mean) for both halves of a packed pair
__device__ __forceinline__ void ln_center_half2(uint32_t packed, float mean, float &d0, float &d1) {
    asm("{\n .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %2;\n"
        " sub.rn.f32.f16 %0, lo, %3;\n sub.rn.f32.f16 %1, hi, %3;\n}\n"
        : "=f"(d0), "=f"(d1) : "r"(packed), "f"(mean));
}

template <> struct LnVec<__half> {
    static __device__ __forceinline__ void sum(const uint4 &v, float (&s)[2]) {
        ln_sum_half2(v.x, s); ln_sum_half2(v.y, s); ln_sum_half2(v.z, s); ln_sum_half2(v.w, s);
    }
    static __device__ __forceinline__ void sq(const uint4 &v, float mean, float (&q)[2]) {
        ln_sq_half2(v.x, mean, q); ln_sq_half2(v.y, mean, q);
        ln_sq_half2(v.z, mean, q); ln_sq_half2(v.w, mean, q);
    }
    struct WB { float4 w0, w1, b0, b1; };
    static __device__ __forceinline__ WB load_wb(const float *w, const float *b) {
        return WB{*reinterpret_cast<const float4 *>(w), *(reinterpret_cast<const float4 *>(w) + 1),
                  *reinterpret_cast<const float4 *>(b), *(reinterpret_cast<const float4 *>(b) + 1)};
    }
    static __device__ __forceinline__ uint4 norm(const uint4 &v, float mean, float rstd, const WB &k) {
        const float4 w0 = k.w0, w1 = k.w1, b0 = k.b0, b1 = k.b1;
        float d[8];
        ln_center_half2(v.x, mean, d[0], d[1]);
        ln_center_half2(v.y, mean, d[2], d[3]);
        ln_center_half2(v.z, mean, d[4], d[5]);
        ln_center_half2(v.w, mean, d[6], d[7]);
        uint4 o;
        __half2 *h = reinterpret_cast<__half2 *>(&o);
        h[0] = __floats2half2_rn(fmaf(d[0] * rstd, w0.x, b0.x), fmaf(d[1] * rstd, w0.y, b0.y));
        h[1] = __floats2half2_rn(fmaf(d[2] * rstd, w0.z, b0.z), fmaf(d[3] * rstd, w0.w, b0.w));
        h[2] = __floats2half2_rn(fmaf(d[4] * rstd, w1.x, b1.x), fmaf(d[5] * rstd, w1.y, b1.y));
        h[3] = __floats2half2_rn(fmaf(d[6] * rstd, w1.z, b1.z), fmaf(d[7] * rstd, w1.w, b1.w));
        return o;
    }
};

// Register budget: the more row vectors a lane holds, the fewer CTAs share an SM.
constexpr int ln_min_blocks(int maxv) { return maxv <= 3 ? 6 : maxv <= 6 ? 4 : maxv <= 8 ? 3 : 2; }
// Rows a warp takes per iteration: two while the row vectors of both still fit the registers, so
// that every shared-memory load of scale / shift serves two rows (those loads, four times the
// bytes of an fp16 row, made the L1 / shared-memory pipe the kernel's limit at 84 %).
// (Used for plain LayerNorm with enough rows to fill the SMs; the add variant keeps one row.)
constexpr int ln_min_blocks_r(int maxv, int rows_per_warp) {
    return rows_per_warp == 2 ? (ln_min_blocks(2 * maxv) > 4 ? 4 : ln_min_blocks(2 * maxv)) : ln_min_blocks(maxv);
}

// One warp per row; lane l keeps vectors l, l+32, ... of the row in registers, so the mean,
// the exact two-pass variance and the normalised write cost one read and one write of the row.
//
// ADD: the row normalised is in + in2 (the residual add that precedes the norm in the
// reference's transformer block, BasicTransformerBlock.cpp:126-136); the sum itself is also
// written to `sum_out`, rounded to the storage type first, so the result equals the
// reference's two steps (elemwise_add, then layer_norm on what was stored).
// Scale and shift are fp32 (2 x 4 bytes per element against 2 bytes of fp16 data): read through
// L1 for every row they saturate the L1 data path, so each CTA first copies them to shared
// memory (dynamic, 2 * dim floats) and every row reads them from there.  The copy is plain loads
// and stores followed by one CTA barrier before the first row: a barrier placed behind the first
// rows' loads instead makes every warp wait for the slowest.
template <typename T, int MAXV, bool ADD, int R>
__global__ void __launch_bounds__(kLnThreads, ln_min_blocks_r(MAXV, R))
ln_warp_kernel(const T *in, const T *in2, T *sum_out, T *out, const float *__restrict__ gw,
               const float *__restrict__ gb, long long rows, int nvec, int dim, float eps) {
    constexpr int VEC = VecOf<T>::N;
    extern __shared__ __align__(16) float s_wb[];
    float *w = s_wb, *b = s_wb + dim;
    for (int i = threadIdx.x; i < dim / 4; i += kLnThreads) {
        reinterpret_cast<float4 *>(w)[i] = __ldg(reinterpret_cast<const float4 *>(gw) + i);
        reinterpret_cast<float4 *>(b)[i] = __ldg(reinterpret_cast<const float4 *>(gb) + i);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const long long warp0 = static_cast<long long>(blockIdx.x) * kLnWarps + (threadIdx.x >> 5);
    const long long nwarps = static_cast<long long>(gridDim.x) * kLnWarps;
    const float inv_d = 1.0f / static_cast<float>(dim);
    for (long long row0 = warp0 * R; row0 < rows; row0 += nwarps * R) {
        uint4 v[R][MAXV];
        float mean[R], rstd[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const long long row = row0 + r;
            if (row >= rows) break;
            const uint4 *xr = reinterpret_cast<const uint4 *>(in + row * dim);
#pragma unroll
            for (int i = 0; i < MAXV; ++i) {
                const int idx = lane + 32 * i;
                if (idx < nvec) {
                    v[r][i] = ld_stream(xr + idx);
                    if (ADD) {
                        float fa[VEC], fb[VEC];
                        unpack<T>(v[r][i], fa);
                        unpack<T>(ld_stream(reinterpret_cast<const uint4 *>(in2 + row * dim) + idx), fb);
#pragma unroll
                        for (int j = 0; j < VEC; ++j) fa[j] += fb[j];
                        v[r][i] = pack<T>(fa);
                        st_stream(reinterpret_cast<uint4 *>(sum_out + row * dim) + idx, v[r][i]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (row0 + r >= rows) break;
            float s[2] = {0.f, 0.f};
#pragma unroll
            for (int i = 0; i < MAXV; ++i)
                if (lane + 32 * i < nvec) LnVec<T>::sum(v[r][i], s);
            mean[r] = warp_sum(s[0] + s[1]) * inv_d;
            float q[2] = {0.f, 0.f};
#pragma unroll
            for (int i = 0; i < MAXV; ++i)
                if (lane + 32 * i < nvec) LnVec<T>::sq(v[r][i], mean[r], q);
            const float var = warp_sum(q[0] + q[1]) * inv_d;
            rstd[r] = 1.0f / sqrtf(var + eps);
        }
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < nvec) {
                const typename LnVec<T>::WB k = LnVec<T>::load_wb(w + idx * VEC, b + idx * VEC);
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (row0 + r < rows)
                        st_stream(reinterpret_cast<uint4 *>(out + (row0 + r) * dim) + idx,
                                  LnVec<T>::norm(v[r][i], mean[r], rstd[r], k));
            }
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
void launch_warp(const void *in, const void *in2, void *sum_out, void *out, const float *w,
                 const float *b, int64_t rows, int nvec, int dim, float eps, cudaStream_t stream) {
    // persistent grid: as many CTAs as fit the SMs at once, so the staged scale / shift are
    // reused for many rows.  Two rows per warp when the pairs still give every SM its warps.
    const bool two = in2 == nullptr && MAXV <= 6 && rows >= sm_count() * kLnWarps * 4;
    const int64_t rows_per_cta = kLnWarps * (two ? 2 : 1);
    int64_t blocks = (rows + rows_per_cta - 1) / rows_per_cta;
    const int64_t cap = sm_count() * ln_min_blocks_r(MAXV, two ? 2 : 1);
    if (blocks > cap) blocks = cap;
    const size_t smem = 2 * static_cast<size_t>(dim) * sizeof(float);
    const unsigned grid = static_cast<unsigned>(blocks);
    if (in2)
        ln_warp_kernel<T, MAXV, true, 1><<<grid, kLnThreads, smem, stream>>>(
            static_cast<const T *>(in), static_cast<const T *>(in2), static_cast<T *>(sum_out),
            static_cast<T *>(out), w, b, rows, nvec, dim, eps);
    else if (two)
        ln_warp_kernel<T, (MAXV <= 6 ? MAXV : 1), false, 2><<<grid, kLnThreads, smem, stream>>>(
            static_cast<const T *>(in), nullptr, nullptr, static_cast<T *>(out), w, b, rows, nvec, dim, eps);
    else
        ln_warp_kernel<T, MAXV, false, 1><<<grid, kLnThreads, smem, stream>>>(
            static_cast<const T *>(in), nullptr, nullptr, static_cast<T *>(out), w, b, rows, nvec, dim, eps);
}

inline bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Returns cudaErrorNotSupported when the row-in-registers kernel cannot take the shape.
template <typename T>
cudaError_t ln_warp_dispatch(const void *in, const void *in2, void *sum_out, void *out, const float *w,
                             const float *b, int64_t rows, int64_t dim, float eps, cudaStream_t stream) {
    constexpr int VEC = VecOf<T>::N;
    const bool vec_ok = dim % VEC == 0 && al16(in) && al16(out) && al16(w) && al16(b) &&
                        (!in2 || (al16(in2) && al16(sum_out)));
    const int64_t nvec = dim / VEC;
    if (!vec_ok || nvec > 32 * 16) return cudaErrorNotSupported;
    const int need = static_cast<int>((nvec + 31) / 32);
    const int nv = static_cast<int>(nvec), d = static_cast<int>(dim);
    if (need <= 1) launch_warp<T, 1>(in, in2, sum_out, out, w, b, rows, nv, d, eps, stream);
    else if (need <= 2) launch_warp<T, 2>(in, in2, sum_out, out, w, b, rows, nv, d, eps, stream);
    else if (need <= 3) launch_warp<T, 3>(in, in2, sum_out, out, w, b, rows, nv, d, eps, stream);
    else if (need <= 4) launch_warp<T, 4>(in, in2, sum_out, out, w, b, rows, nv, d, eps, stream);
    else if (need <= 5) launch_warp<T, 5>(in, in2, sum_out, out, w, b, rows, nv, d, eps, stream);
    else if (need <= 6) launch_warp<T, 6>(in, in2, sum_out, out, w, b, rows, nv, d, eps, stream);
    else if (need <= 8) launch_warp<T, 8>(in, in2, sum_out, out, w, b, rows, nv, d, eps, stream);
    else if (need <= 10) launch_warp<T, 10>(in, in2, sum_out, out, w, b, rows, nv, d, eps, stream);
    else if (need <= 12) launch_warp<T, 12>(in, in2, sum_out, out, w, b, rows, nv, d, eps, stream);
    else launch_warp<T, 16>(in, in2, sum_out, out, w, b, rows, nv, d, eps, stream);
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

template <typename T>
cudaError_t ln_dispatch(const void *in, void *out, const float *w, const float *b, int64_t rows,
                        int64_t dim, float eps, cudaStream_t stream) {
    cudaError_t err = ln_warp_dispatch<T>(in, nullptr, nullptr, out, w, b, rows, dim, eps, stream);
    if (err != cudaErrorNotSupported) return err;
    int64_t blocks = rows < sm_count() * 8 ? rows : sm_count() * 8;
    ln_block_kernel<T><<<static_cast<unsigned>(blocks), kLnThreads, 0, stream>>>(
        static_cast<const T *>(in), static_cast<T *>(out), w, b, rows, dim, eps);
    err = cudaGetLastError();
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

// sum_out = a + b, out = LayerNorm(sum_out).  One launch when the row-in-registers kernel takes
// the shape; otherwise the add kernel followed by the LayerNorm fallback (same results).
cudaError_t add_ln_launch(const void *a, const void *b2, void *sum_out, void *out, const float *w,
                          const float *b, int64_t rows, int64_t dim, float eps, int dtype,
                          cudaStream_t stream) {
    if (rows == 0 || dim == 0) return cudaSuccess;
    cudaError_t err = dtype == kF16
                          ? ln_warp_dispatch<__half>(a, b2, sum_out, out, w, b, rows, dim, eps, stream)
                          : ln_warp_dispatch<float>(a, b2, sum_out, out, w, b, rows, dim, eps, stream);
    if (err != cudaErrorNotSupported) return err;
    err = add_launch(a, b2, sum_out, rows * dim, dtype, stream);
    if (err != cudaSuccess) return err;
    return ln_launch(sum_out, out, w, b, rows, dim, eps, dtype, stream);
}

}  // namespace sdfl
