// Row softmax over the last dimension of a row-major [rows, D] tensor (util.cl:150-187 `softmax`,
// launched on the attention scores at nn/CrossAttention.cpp:365-378 with one 64-item work-group
// per row; rows are 77 keys for cross-attention, 64-4096 for self-attention).  fp32 or fp16 I/O,
// fp32 arithmetic, out == in allowed (the reference runs it in place).
//
// The reference computes exp(x) / sum(exp(x)) without subtracting the row maximum
// (util.cl:164-169) and overflows for x > 88.  Here the maximum is subtracted: the quotient is
// the same number, the result stays finite for any finite input, and on the reference's working
// range the two agree to a few ulp (the parity tests run there).
//
// Rows whose bytes are a multiple of 16 and fit 16 vectors per lane live in one warp's
// registers: one read, one write.  Other rows take a CTA each, with the row's exponentials
// cached in shared memory as the reference does (`cache`), or re-read when too long for that.
#include "common.cuh"
#include "kernels.h"

namespace sdfl {

namespace {

constexpr int kSmThreads = 256;
constexpr int kSmWarps = kSmThreads / 32;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

constexpr int sm_min_blocks(int maxv) { return maxv <= 2 ? 6 : maxv <= 4 ? 4 : maxv <= 8 ? 3 : 2; }

template <typename T, int MAXV>
__global__ void __launch_bounds__(kSmThreads, sm_min_blocks(MAXV))
softmax_warp_kernel(const T *__restrict__ in, T *out, long long rows, int dim) {
    constexpr int VEC = VecOf<T>::N;
    const int nvec = dim / VEC;
    const int lane = threadIdx.x & 31;
    const long long warp0 = static_cast<long long>(blockIdx.x) * kSmWarps + (threadIdx.x >> 5);
    const long long nwarps = static_cast<long long>(gridDim.x) * kSmWarps;
    for (long long row = warp0; row < rows; row += nwarps) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(in + row * dim);
        uint4 *yr = reinterpret_cast<uint4 *>(out + row * dim);
        // fp32 rows are kept as floats and exponentiated in place.  fp16 rows stay packed (16
        // vectors of 8 would be 128 float registers) and exp is evaluated in both later passes:
        // two SFU operations per element still fit under the HBM time of 4 bytes per element.
        constexpr bool PACKED = sizeof(T) == 2;
        uint4 v[MAXV];
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < nvec) {
                v[i] = ld_stream(xr + idx);
                float f[VEC];
                unpack<T>(v[i], f);
#pragma unroll
                for (int j = 0; j < VEC; ++j) m = fmaxf(m, f[j]);
            }
        }
        m = warp_max(m);
        const float shift = m * kLog2e;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            if (lane + 32 * i < nvec) {
                float f[VEC];
                unpack<T>(v[i], f);
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    f[j] = ex2_approx(fmaf(f[j], kLog2e, -shift));     // exp(x - max)
                    s += f[j];
                }
                if (!PACKED) v[i] = pack<T>(f);
            }
        }
        s = warp_sum(s);
        const float inv = 1.0f / s;
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < nvec) {
                float f[VEC];
                unpack<T>(v[i], f);
#pragma unroll
                for (int j = 0; j < VEC; ++j)
                    f[j] = (PACKED ? ex2_approx(fmaf(f[j], kLog2e, -shift)) : f[j]) * inv;
                st_stream(yr + idx, pack<T>(f));
            }
        }
    }
}

// Short rows of any length and alignment (the 77 keys of cross-attention: 154- or 308-byte rows):
// one warp per row, lane l holds elements l, l+32, ... (up to MAXE), element-wise accesses that
// are consecutive across the lanes.  (Four rows per warp iteration, all loads issued first, was
// slower: 15.2 against 9.4 us on 65536 fp16 rows of 77; blocks of 64 rows staged in shared memory
// with 16-byte global accesses on both sides: 11.8 us.)
template <typename T, int MAXE>
__global__ void __launch_bounds__(kSmThreads)
softmax_warp_scalar_kernel(const T *__restrict__ in, T *out, long long rows, int dim) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = static_cast<long long>(blockIdx.x) * kSmWarps + (threadIdx.x >> 5);
    const long long nwarps = static_cast<long long>(gridDim.x) * kSmWarps;
    for (long long row = warp0; row < rows; row += nwarps) {
        const T *x = in + row * dim;
        T *y = out + row * dim;
        float f[MAXE];
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < MAXE; ++i) {
            const int idx = lane + 32 * i;
            f[i] = idx < dim ? to_float<T>(x[idx]) : -INFINITY;
            m = fmaxf(m, f[i]);
        }
        m = warp_max(m);
        const float shift = m * kLog2e;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < MAXE; ++i) {
            f[i] = ex2_approx(fmaf(f[i], kLog2e, -shift));       // exp(-inf) = 0 past the row's end
            s += f[i];
        }
        s = warp_sum(s);
        const float inv = 1.0f / s;
#pragma unroll
        for (int i = 0; i < MAXE; ++i) {
            const int idx = lane + 32 * i;
            if (idx < dim) y[idx] = from_float<T>(f[i] * inv);
        }
    }
}

// One CTA per row for rows too long for a warp (up to 256 * 4 vectors: 4096 fp32 or 8192 fp16
// elements): same scheme as the warp kernel with the two reductions going through shared memory.
template <typename T>
__global__ void __launch_bounds__(kSmThreads, 4)
softmax_cta_kernel(const T *__restrict__ in, T *out, long long rows, int dim) {
    constexpr int VEC = VecOf<T>::N;
    constexpr int MAXV = 4;
    constexpr bool PACKED = sizeof(T) == 2;
    __shared__ float red[2][kSmWarps];
    const int nvec = dim / VEC;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(in + row * dim);
        uint4 *yr = reinterpret_cast<uint4 *>(out + row * dim);
        uint4 v[MAXV];
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int idx = tid + kSmThreads * i;
            if (idx < nvec) {
                v[i] = ld_stream(xr + idx);
                float f[VEC];
                unpack<T>(v[i], f);
#pragma unroll
                for (int j = 0; j < VEC; ++j) m = fmaxf(m, f[j]);
            }
        }
        m = warp_max(m);
        if (lane == 0) red[0][warp] = m;
        __syncthreads();
        m = warp_max(lane < kSmWarps ? red[0][lane] : -INFINITY);
        const float shift = m * kLog2e;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            if (tid + kSmThreads * i < nvec) {
                float f[VEC];
                unpack<T>(v[i], f);
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    f[j] = ex2_approx(fmaf(f[j], kLog2e, -shift));
                    s += f[j];
                }
                if (!PACKED) v[i] = pack<T>(f);
            }
        }
        s = warp_sum(s);
        if (lane == 0) red[1][warp] = s;
        __syncthreads();
        s = warp_sum(lane < kSmWarps ? red[1][lane] : 0.f);
        const float inv = 1.0f / s;
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int idx = tid + kSmThreads * i;
            if (idx < nvec) {
                float f[VEC];
                unpack<T>(v[i], f);
#pragma unroll
                for (int j = 0; j < VEC; ++j)
                    f[j] = (PACKED ? ex2_approx(fmaf(f[j], kLog2e, -shift)) : f[j]) * inv;
                st_stream(yr + idx, pack<T>(f));
            }
        }
        __syncthreads();                       // red is reused by the next row
    }
}

// One CTA per row, any length and alignment.  CACHE: the row's exponentials are kept in dynamic
// shared memory (dim floats) between the passes; otherwise the row is read three times.
template <typename T, bool CACHE>
__global__ void __launch_bounds__(kSmThreads)
softmax_block_kernel(const T *in, T *out, long long rows, int dim) {
    extern __shared__ float cache[];
    __shared__ float red[kSmWarps];
    __shared__ float bcast;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *x = in + row * dim;
        T *y = out + row * dim;
        float m = -INFINITY;
        for (int i = tid; i < dim; i += kSmThreads) {
            const float v = to_float<T>(x[i]);
            if (CACHE) cache[i] = v;
            m = fmaxf(m, v);
        }
        m = warp_max(m);
        if (lane == 0) red[warp] = m;
        __syncthreads();
        if (warp == 0) {
            float t = lane < kSmWarps ? red[lane] : -INFINITY;
            t = warp_max(t);
            if (lane == 0) bcast = t;
        }
        __syncthreads();
        const float shift = bcast * kLog2e;
        float s = 0.f;
        for (int i = tid; i < dim; i += kSmThreads) {
            const float e = ex2_approx(fmaf(CACHE ? cache[i] : to_float<T>(x[i]), kLog2e, -shift));
            if (CACHE) cache[i] = e;
            s += e;
        }
        s = warp_sum(s);
        __syncthreads();                       // everyone has read bcast (the maximum)
        if (lane == 0) red[warp] = s;
        __syncthreads();
        if (warp == 0) {
            float t = lane < kSmWarps ? red[lane] : 0.f;
            t = warp_sum(t);
            if (lane == 0) bcast = t;
        }
        __syncthreads();
        const float inv = 1.0f / bcast;
        for (int i = tid; i < dim; i += kSmThreads) {
            const float e = CACHE ? cache[i] : ex2_approx(fmaf(to_float<T>(x[i]), kLog2e, -shift));
            y[i] = from_float<T>(e * inv);
        }
        __syncthreads();                       // red / bcast / cache are reused by the next row
    }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T>
cudaError_t softmax_dispatch(const void *in, void *out, int64_t rows, int64_t dim, cudaStream_t stream) {
    constexpr int VEC = VecOf<T>::N;
    const T *x = static_cast<const T *>(in);
    T *y = static_cast<T *>(out);
    const int d = static_cast<int>(dim);
    const int64_t nvec = dim / VEC;
    if (dim % VEC == 0 && aligned16(in) && aligned16(out) && nvec <= 32 * 16) {
        const int per_lane = static_cast<int>((nvec + 31) / 32);
        const int64_t want = (rows + kSmWarps - 1) / kSmWarps;
        auto grid_for = [&](int min_blocks) {
            const int64_t cap = static_cast<int64_t>(sm_count()) * min_blocks;
            return static_cast<unsigned>(want < cap ? want : cap);
        };
        if (per_lane <= 1) softmax_warp_kernel<T, 1><<<grid_for(sm_min_blocks(1)), kSmThreads, 0, stream>>>(x, y, rows, d);
        else if (per_lane <= 2) softmax_warp_kernel<T, 2><<<grid_for(sm_min_blocks(2)), kSmThreads, 0, stream>>>(x, y, rows, d);
        else if (per_lane <= 4) softmax_warp_kernel<T, 4><<<grid_for(sm_min_blocks(4)), kSmThreads, 0, stream>>>(x, y, rows, d);
        else if (per_lane <= 8) softmax_warp_kernel<T, 8><<<grid_for(sm_min_blocks(8)), kSmThreads, 0, stream>>>(x, y, rows, d);
        else softmax_warp_kernel<T, 16><<<grid_for(sm_min_blocks(16)), kSmThreads, 0, stream>>>(x, y, rows, d);
    } else if (dim % VEC == 0 && aligned16(in) && aligned16(out) && nvec <= kSmThreads * 4) {
        const unsigned grid = static_cast<unsigned>(rows < sm_count() * 4 ? rows : sm_count() * 4);
        softmax_cta_kernel<T><<<grid, kSmThreads, 0, stream>>>(x, y, rows, d);
    } else if (dim <= 256) {
        const int64_t want = (rows + kSmWarps - 1) / kSmWarps;
        const unsigned grid = static_cast<unsigned>(want < sm_count() * 8 ? want : sm_count() * 8);
        if (dim <= 32) softmax_warp_scalar_kernel<T, 1><<<grid, kSmThreads, 0, stream>>>(x, y, rows, d);
        else if (dim <= 96) softmax_warp_scalar_kernel<T, 3><<<grid, kSmThreads, 0, stream>>>(x, y, rows, d);
        else softmax_warp_scalar_kernel<T, 8><<<grid, kSmThreads, 0, stream>>>(x, y, rows, d);
    } else {
        const unsigned grid = static_cast<unsigned>(rows < sm_count() * 8 ? rows : sm_count() * 8);
        const size_t smem = static_cast<size_t>(dim) * sizeof(float);
        if (smem <= 40 * 1024)
            softmax_block_kernel<T, true><<<grid, kSmThreads, smem, stream>>>(x, y, rows, d);
        else
            softmax_block_kernel<T, false><<<grid, kSmThreads, 0, stream>>>(x, y, rows, d);
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

}  // namespace

cudaError_t softmax_launch(const void *in, void *out, int64_t rows, int64_t dim, int dtype,
                           cudaStream_t stream) {
    if (rows == 0 || dim == 0) return cudaSuccess;
    return dtype == kF16 ? softmax_dispatch<__half>(in, out, rows, dim, stream)
                         : softmax_dispatch<float>(in, out, rows, dim, stream);
}

}  // namespace sdfl
