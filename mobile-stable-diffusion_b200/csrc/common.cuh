// Shared device helpers for the fused-layer kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sdfl {

constexpr int kF32 = 0;
constexpr int kF16 = 1;

enum Act : int { kActNone = 0, kActSilu = 1, kActGelu = 2, kActQuickGelu = 3 };

// Number of SMs of the current device, asked of the driver once per device (grids are sized in
// multiples of it).  Without a usable device -- planning calls made on a machine that has none --
// the answer is the B200's 148.
inline int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return 148;
    }
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = 148;
        }
        cached[dev] = n;        // racing threads write the same value
    }
    return cached[dev];
}

// ---------------------------------------------------------------------------------------------
// 16-byte vectors of T <-> float lanes
// ---------------------------------------------------------------------------------------------
template <typename T> struct VecOf;
template <> struct VecOf<float> { static constexpr int N = 4; };
template <> struct VecOf<__half> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void unpack(const uint4 &v, float (&f)[VecOf<T>::N]);

template <> __device__ __forceinline__ void unpack<float>(const uint4 &v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}

template <> __device__ __forceinline__ void unpack<__half>(const uint4 &v, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

template <typename T> __device__ __forceinline__ uint4 pack(const float (&f)[VecOf<T>::N]);

template <> __device__ __forceinline__ uint4 pack<float>(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
}

template <> __device__ __forceinline__ uint4 pack<__half>(const float (&f)[8]) {
    uint4 v;
    __half2 *h = reinterpret_cast<__half2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);   // RNE
    return v;
}

template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }

// Streaming 16-byte global accesses: the tensors here are touched once per launch.
__device__ __forceinline__ uint4 ld_stream(const void *p) {
    return __ldcs(reinterpret_cast<const uint4 *>(p));
}
__device__ __forceinline__ void st_stream(void *p, const uint4 &v) {
    __stcs(reinterpret_cast<uint4 *>(p), v);
}

// ---------------------------------------------------------------------------------------------
// Activations.  exp2 / reciprocal use the SFU approximations (relative error ~2^-22), which is
// two orders of magnitude inside the fp32 parity tolerance and keeps the kernels HBM-bound.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// x * 1/(1 + exp(-k x)); k = 1 is SiLU, k = 1.702 is quick_gelu.
__device__ __forceinline__ float sigmoid_mul(float x, float k_log2e) {
    float t = ex2_approx(-k_log2e * x);
    return x * rcp_approx(1.0f + t);
}

// erf for half-precision outputs: Abramowitz-Stegun 7.1.26, |error| <= 1.5e-7 in exact
// arithmetic; with the SFU exp2/rcp the result stays within ~1e-6 absolute.
__device__ __forceinline__ float erf_fast(float x) {
    const float ax = fabsf(x);
    const float t = rcp_approx(fmaf(0.3275911f, ax, 1.0f));
    float p = fmaf(1.061405429f, t, -1.453152027f);
    p = fmaf(p, t, 1.421413741f);
    p = fmaf(p, t, -0.284496736f);
    p = fmaf(p, t, 0.254829592f);
    p *= t;
    const float e = ex2_approx(-1.4426950408889634f * ax * ax);
    return copysignf(1.0f - p * e, x);
}

template <bool HALF_OUT> __device__ __forceinline__ float gelu_erf(float x) {
    const float e = HALF_OUT ? erf_fast(x * 0.70710678118654752440f)
                             : erff(x * 0.70710678118654752440f);
    return x * 0.5f * (1.0f + e);
}

template <int ACT, bool HALF_OUT> __device__ __forceinline__ float activate(float x) {
    if (ACT == kActSilu) return sigmoid_mul(x, 1.4426950408889634f);
    if (ACT == kActQuickGelu) return sigmoid_mul(x, 1.702f * 1.4426950408889634f);
    if (ACT == kActGelu) return gelu_erf<HALF_OUT>(x);
    return x;
}

// ---------------------------------------------------------------------------------------------
// Division of a 31-bit index by a launch-constant divisor (multiply-high + shift).
// ---------------------------------------------------------------------------------------------
struct FastDiv {
    uint32_t d, m, s;
    __host__ __device__ static FastDiv make(uint32_t d) {
        FastDiv f;
        f.d = d ? d : 1;
        uint32_t s = 0;
        while ((1ull << s) < f.d) ++s;
        f.s = s;
        f.m = static_cast<uint32_t>(((1ull << 32) * ((1ull << s) - f.d)) / f.d + 1);
        return f;
    }
    __device__ __forceinline__ uint32_t div(uint32_t n) const {   // n < 2^31
        return (__umulhi(n, m) + n) >> s;
    }
};

// ---------------------------------------------------------------------------------------------
// Block-wide sum, result broadcast to every thread.  `scratch` holds >= 33 floats.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float block_sum(float v, float *scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                 // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace sdfl
