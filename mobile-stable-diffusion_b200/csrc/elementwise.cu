// Flat elementwise kernels: GEGLU gate (geglu.cl:1-25), gelu (util.cl:104-122), silu
// (util.cl:124-134), quick_gelu (no reference kernel; silu's form with slope 1.702) and
// elemwise_add (util.cl:1-12), chunkwise_add (util.cl:136-148).  fp32 or fp16 I/O, fp32 arithmetic, 16-byte accesses when the
// pointers and extents allow it, scalar otherwise.  src == dst is allowed for the unary ops.
#include "common.cuh"
#include "kernels.h"

namespace sdfl {

namespace {

constexpr int kEwThreads = 256;

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline unsigned ew_grid(int64_t work_items) {
    int64_t blocks = (work_items + kEwThreads - 1) / kEwThreads;
    const int64_t cap = sm_count() * 8 * 4;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<unsigned>(blocks);
}

// ---- unary activations ------------------------------------------------------------------------
template <typename T, int ACT>
__global__ void __launch_bounds__(kEwThreads)
act_vec_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, long long nvec) {
    constexpr int VEC = VecOf<T>::N;
    constexpr bool HALF = sizeof(T) == 2;
    const long long stride = static_cast<long long>(gridDim.x) * kEwThreads;
    for (long long i = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x; i < nvec;
         i += stride) {
        float f[VEC];
        unpack<T>(ld_stream(src + i), f);
#pragma unroll
        for (int j = 0; j < VEC; ++j) f[j] = activate<ACT, HALF>(f[j]);
        st_stream(dst + i, pack<T>(f));
    }
}

template <typename T, int ACT>
__global__ void __launch_bounds__(kEwThreads)
act_scalar_kernel(const T *src, T *dst, long long first, long long n) {
    constexpr bool HALF = sizeof(T) == 2;
    const long long stride = static_cast<long long>(gridDim.x) * kEwThreads;
    for (long long i = first + static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x; i < n;
         i += stride)
        dst[i] = from_float<T>(activate<ACT, HALF>(to_float<T>(src[i])));
}

template <typename T, int ACT>
cudaError_t act_dispatch(const void *src, void *dst, int64_t n, cudaStream_t stream) {
    constexpr int VEC = VecOf<T>::N;
    int launches = 0;
    int64_t done = 0;
    if (aligned16(src) && aligned16(dst) && n >= VEC) {
        const int64_t nvec = n / VEC;
        act_vec_kernel<T, ACT><<<ew_grid(nvec), kEwThreads, 0, stream>>>(
            static_cast<const uint4 *>(src), static_cast<uint4 *>(dst), nvec);
        done = nvec * VEC;
        ++launches;
    }
    if (done < n) {
        act_scalar_kernel<T, ACT><<<ew_grid(n - done), kEwThreads, 0, stream>>>(
            static_cast<const T *>(src), static_cast<T *>(dst), done, n);
        ++launches;
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(launches);
    return err;
}

// ---- GEGLU gate: dst[r, j] = AB[r, j] * gelu(AB[r, D + j]) -----------------------------------
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
geglu_vec_kernel(const uint4 *__restrict__ ab, uint4 *__restrict__ dst, long long total_vecs,
                 FastDiv dvec_div, uint32_t dvec) {
    constexpr int VEC = VecOf<T>::N;
    constexpr bool HALF = sizeof(T) == 2;
    const long long stride = static_cast<long long>(gridDim.x) * kEwThreads;
    for (long long i = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x; i < total_vecs;
         i += stride) {
        const uint32_t r = dvec_div.div(static_cast<uint32_t>(i));
        const uint32_t j = static_cast<uint32_t>(i) - r * dvec;
        const uint4 *row = ab + static_cast<size_t>(r) * 2 * dvec;
        float a[VEC], g[VEC];
        unpack<T>(ld_stream(row + j), a);
        unpack<T>(ld_stream(row + dvec + j), g);
#pragma unroll
        for (int k = 0; k < VEC; ++k) a[k] = a[k] * gelu_erf<HALF>(g[k]);
        st_stream(dst + i, pack<T>(a));
    }
}

template <typename T>
__global__ void __launch_bounds__(kEwThreads)
geglu_scalar_kernel(const T *__restrict__ ab, T *__restrict__ dst, long long rows, long long d) {
    constexpr bool HALF = sizeof(T) == 2;
    const long long total = rows * d;
    const long long stride = static_cast<long long>(gridDim.x) * kEwThreads;
    for (long long i = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x; i < total;
         i += stride) {
        const long long r = i / d, j = i - r * d;
        const float a = to_float<T>(ab[r * 2 * d + j]);
        const float g = to_float<T>(ab[r * 2 * d + d + j]);
        dst[i] = from_float<T>(a * gelu_erf<HALF>(g));
    }
}

template <typename T>
cudaError_t geglu_dispatch(const void *ab, void *dst, int64_t rows, int64_t d, cudaStream_t stream) {
    constexpr int VEC = VecOf<T>::N;
    const int64_t total_vecs = rows * (d / VEC);
    if (d % VEC == 0 && aligned16(ab) && aligned16(dst) && total_vecs < (1ll << 31)) {
        const uint32_t dvec = static_cast<uint32_t>(d / VEC);
        geglu_vec_kernel<T><<<ew_grid(total_vecs), kEwThreads, 0, stream>>>(
            static_cast<const uint4 *>(ab), static_cast<uint4 *>(dst), total_vecs,
            FastDiv::make(dvec), dvec);
    } else {
        geglu_scalar_kernel<T><<<ew_grid(rows * d), kEwThreads, 0, stream>>>(
            static_cast<const T *>(ab), static_cast<T *>(dst), rows, d);
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

// ---- C = A + B ----------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
add_vec_kernel(const uint4 *a, const uint4 *b, uint4 *c, long long nvec) {
    constexpr int VEC = VecOf<T>::N;
    const long long stride = static_cast<long long>(gridDim.x) * kEwThreads;
    for (long long i = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x; i < nvec;
         i += stride) {
        float x[VEC], y[VEC];
        unpack<T>(ld_stream(a + i), x);
        unpack<T>(ld_stream(b + i), y);
#pragma unroll
        for (int j = 0; j < VEC; ++j) x[j] = x[j] + y[j];
        st_stream(c + i, pack<T>(x));
    }
}

template <typename T>
__global__ void __launch_bounds__(kEwThreads)
add_scalar_kernel(const T *a, const T *b, T *c, long long first, long long n) {
    const long long stride = static_cast<long long>(gridDim.x) * kEwThreads;
    for (long long i = first + static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x; i < n;
         i += stride)
        c[i] = from_float<T>(to_float<T>(a[i]) + to_float<T>(b[i]));
}

template <typename T>
cudaError_t add_dispatch(const void *a, const void *b, void *c, int64_t n, cudaStream_t stream) {
    constexpr int VEC = VecOf<T>::N;
    int launches = 0;
    int64_t done = 0;
    if (aligned16(a) && aligned16(b) && aligned16(c) && n >= VEC) {
        const int64_t nvec = n / VEC;
        add_vec_kernel<T><<<ew_grid(nvec), kEwThreads, 0, stream>>>(
            static_cast<const uint4 *>(a), static_cast<const uint4 *>(b), static_cast<uint4 *>(c), nvec);
        done = nvec * VEC;
        ++launches;
    }
    if (done < n) {
        add_scalar_kernel<T><<<ew_grid(n - done), kEwThreads, 0, stream>>>(
            static_cast<const T *>(a), static_cast<const T *>(b), static_cast<T *>(c), done, n);
        ++launches;
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(launches);
    return err;
}

// ---- C[i] = A[i] + chunk[i / chunk_size]  (util.cl:136-148) -----------------------------------
// Vector form: chunk_size is a multiple of the vector width, so a 16-byte vector lies inside one
// chunk and its addend index is one division of the vector index (multiply-high while the vector
// count fits 31 bits, a 64-bit division per vector beyond that).
template <typename T, bool WIDE>
__global__ void __launch_bounds__(kEwThreads)
chunkwise_add_vec_kernel(const uint4 *a, const T *__restrict__ chunk, uint4 *c, long long nvec,
                         FastDiv chunk_div, unsigned long long chunk_vecs) {
    constexpr int VEC = VecOf<T>::N;
    const long long stride = static_cast<long long>(gridDim.x) * kEwThreads;
    for (long long i = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x; i < nvec;
         i += stride) {
        const unsigned long long k = WIDE ? static_cast<unsigned long long>(i) / chunk_vecs
                                          : chunk_div.div(static_cast<uint32_t>(i));
        const float e = to_float<T>(__ldg(chunk + k));
        float x[VEC];
        unpack<T>(ld_stream(a + i), x);
#pragma unroll
        for (int j = 0; j < VEC; ++j) x[j] = x[j] + e;
        st_stream(c + i, pack<T>(x));
    }
}

template <typename T>
__global__ void __launch_bounds__(kEwThreads)
chunkwise_add_kernel(const T *a, const T *__restrict__ chunk, T *c, unsigned long long first,
                     unsigned long long n, unsigned long long chunk_size) {
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kEwThreads;
    for (unsigned long long i = first + static_cast<unsigned long long>(blockIdx.x) * kEwThreads + threadIdx.x;
         i < n; i += stride)
        c[i] = from_float<T>(to_float<T>(a[i]) + to_float<T>(chunk[i / chunk_size]));
}

template <typename T>
cudaError_t chunkwise_add_dispatch(const void *a, const void *chunk, void *c, int64_t n,
                                   int64_t chunk_size, cudaStream_t stream) {
    constexpr int VEC = VecOf<T>::N;
    int launches = 0;
    int64_t done = 0;
    if (aligned16(a) && aligned16(c) && chunk_size % VEC == 0 && n >= VEC) {
        const int64_t nvec = n / VEC, chunk_vecs = chunk_size / VEC;
        const bool wide = nvec >= (1ll << 31) || chunk_vecs >= (1ll << 31);
        const FastDiv cdiv = FastDiv::make(static_cast<uint32_t>(wide ? 1 : chunk_vecs));
        if (wide)
            chunkwise_add_vec_kernel<T, true><<<ew_grid(nvec), kEwThreads, 0, stream>>>(
                static_cast<const uint4 *>(a), static_cast<const T *>(chunk), static_cast<uint4 *>(c), nvec, cdiv,
                static_cast<unsigned long long>(chunk_vecs));
        else
            chunkwise_add_vec_kernel<T, false><<<ew_grid(nvec), kEwThreads, 0, stream>>>(
                static_cast<const uint4 *>(a), static_cast<const T *>(chunk), static_cast<uint4 *>(c), nvec, cdiv,
                static_cast<unsigned long long>(chunk_vecs));
        done = nvec * VEC;
        ++launches;
    }
    if (done < n) {
        chunkwise_add_kernel<T><<<ew_grid(n - done), kEwThreads, 0, stream>>>(
            static_cast<const T *>(a), static_cast<const T *>(chunk), static_cast<T *>(c),
            static_cast<unsigned long long>(done), static_cast<unsigned long long>(n),
            static_cast<unsigned long long>(chunk_size));
        ++launches;
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(launches);
    return err;
}

}  // namespace

cudaError_t chunkwise_add_launch(const void *a, const void *chunk, void *c, int64_t n,
                                 int64_t chunk_size, int dtype, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    return dtype == kF16 ? chunkwise_add_dispatch<__half>(a, chunk, c, n, chunk_size, stream)
                         : chunkwise_add_dispatch<float>(a, chunk, c, n, chunk_size, stream);
}

cudaError_t act_launch(int act, const void *src, void *dst, int64_t n, int dtype, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    if (dtype == kF16) {
        switch (act) {
            case kActSilu: return act_dispatch<__half, kActSilu>(src, dst, n, stream);
            case kActGelu: return act_dispatch<__half, kActGelu>(src, dst, n, stream);
            case kActQuickGelu: return act_dispatch<__half, kActQuickGelu>(src, dst, n, stream);
            default: return cudaErrorInvalidValue;
        }
    }
    switch (act) {
        case kActSilu: return act_dispatch<float, kActSilu>(src, dst, n, stream);
        case kActGelu: return act_dispatch<float, kActGelu>(src, dst, n, stream);
        case kActQuickGelu: return act_dispatch<float, kActQuickGelu>(src, dst, n, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t geglu_launch(const void *ab, void *dst, int64_t rows, int64_t d, int dtype,
                         cudaStream_t stream) {
    if (rows == 0 || d == 0) return cudaSuccess;
    return dtype == kF16 ? geglu_dispatch<__half>(ab, dst, rows, d, stream)
                         : geglu_dispatch<float>(ab, dst, rows, d, stream);
}

cudaError_t add_launch(const void *a, const void *b, void *c, int64_t n, int dtype, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    return dtype == kF16 ? add_dispatch<__half>(a, b, c, n, stream)
                         : add_dispatch<float>(a, b, c, n, stream);
}

}  // namespace sdfl
