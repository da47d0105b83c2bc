// The two bandwidth movers that feed the skip-connection GroupNorms of the UNet's output blocks:
//   up_sample_nearest (up_sample.cl:1-18, launched at nn/UpSample.cpp:93-102 with global size
//     {channels, height, height}): every input element is written to a scale x scale block;
//   concat_buffer (UNetModel.cpp:1960-1990): two buffer copies, input1 then input2 -- for a batch
//     that is a concatenation along the channels of each image.
// fp32 or fp16, 16-byte stores where the extents allow it, element-wise otherwise.
#include "common.cuh"
#include "kernels.h"

namespace sdfl {

namespace {

constexpr int kRsThreads = 256;

inline bool aligned_to(const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

inline unsigned rs_grid(int64_t items) {
    int64_t blocks = (items + kRsThreads - 1) / kRsThreads;
    const int64_t cap = sm_count() * 8 * 4;
    return static_cast<unsigned>(blocks < 1 ? 1 : blocks > cap ? cap : blocks);
}

// scale 2, rows of a multiple of 8 bytes: a thread reads 8 bytes of an input row (4 fp16 or 2 fp32
// values) and writes the two 16-byte vectors they become in output rows 2i and 2i+1.
template <typename T>
__global__ void __launch_bounds__(kRsThreads)
upsample2_vec_kernel(const uint2 *__restrict__ in, uint4 *__restrict__ out, long long total, FastDiv wq_div,
                     uint32_t wq) {
    // total = planes * H * wq items, wq = 8-byte pieces per input row; item -> (row r, piece q)
    const long long stride = static_cast<long long>(gridDim.x) * kRsThreads;
    for (long long it = static_cast<long long>(blockIdx.x) * kRsThreads + threadIdx.x; it < total; it += stride) {
        const uint32_t r = wq_div.div(static_cast<uint32_t>(it));      // plane * H + i
        const uint32_t q = static_cast<uint32_t>(it) - r * wq;
        const uint2 v = __ldg(in + it);
        uint4 o;
        if (sizeof(T) == 2) {
            o.x = __byte_perm(v.x, 0, 0x1010); o.y = __byte_perm(v.x, 0, 0x3232);
            o.z = __byte_perm(v.y, 0, 0x1010); o.w = __byte_perm(v.y, 0, 0x3232);
        } else {
            o.x = v.x; o.y = v.x; o.z = v.y; o.w = v.y;
        }
        uint4 *row0 = out + (static_cast<size_t>(r) * 2) * wq + q;      // output row 2r has wq vectors too
        st_stream(row0, o);
        st_stream(row0 + wq, o);
    }
}

template <typename T>
__global__ void __launch_bounds__(kRsThreads)
upsample_scalar_kernel(const T *__restrict__ in, T *__restrict__ out, long long planes, int H, int W, int scale) {
    const long long ow = static_cast<long long>(W) * scale, oh = static_cast<long long>(H) * scale;
    const long long total = planes * oh * ow;
    const long long stride = static_cast<long long>(gridDim.x) * kRsThreads;
    for (long long o = static_cast<long long>(blockIdx.x) * kRsThreads + threadIdx.x; o < total; o += stride) {
        const long long x = o % ow, y = (o / ow) % oh, p = o / (ow * oh);
        out[o] = in[(p * H + y / scale) * W + x / scale];
    }
}

// out[n] = [in1[n] | in2[n]] with n1 and n2 elements (or 16-byte vectors) per image.
template <typename V>
__global__ void __launch_bounds__(kRsThreads)
concat_kernel(const V *__restrict__ in1, const V *__restrict__ in2, V *__restrict__ out, long long batch,
              long long n1, long long n2) {
    const long long per = n1 + n2, total = batch * per;
    const long long stride = static_cast<long long>(gridDim.x) * kRsThreads;
    for (long long o = static_cast<long long>(blockIdx.x) * kRsThreads + threadIdx.x; o < total; o += stride) {
        const long long n = o / per, r = o - n * per;
        out[o] = r < n1 ? in1[n * n1 + r] : in2[n * n2 + (r - n1)];
    }
}

}  // namespace

cudaError_t upsample_nearest_launch(const void *in, void *out, int64_t planes, int64_t H, int64_t W,
                                    int64_t scale, int dtype, cudaStream_t stream) {
    if (planes == 0 || H == 0 || W == 0) return cudaSuccess;
    const int64_t esz = dtype == kF16 ? 2 : 4;
    const int64_t rows = planes * H;
    if (scale == 2 && (W * esz) % 8 == 0 && aligned_to(in, 8) && aligned_to(out, 16) &&
        rows * (W * esz / 8) < (1ll << 32)) {
        const uint32_t wq = static_cast<uint32_t>(W * esz / 8);
        const long long total = rows * wq;
        if (dtype == kF16)
            upsample2_vec_kernel<__half><<<rs_grid(total), kRsThreads, 0, stream>>>(
                static_cast<const uint2 *>(in), static_cast<uint4 *>(out), total, FastDiv::make(wq), wq);
        else
            upsample2_vec_kernel<float><<<rs_grid(total), kRsThreads, 0, stream>>>(
                static_cast<const uint2 *>(in), static_cast<uint4 *>(out), total, FastDiv::make(wq), wq);
    } else {
        const long long total = planes * H * W * scale * scale;
        if (dtype == kF16)
            upsample_scalar_kernel<__half><<<rs_grid(total), kRsThreads, 0, stream>>>(
                static_cast<const __half *>(in), static_cast<__half *>(out), planes, static_cast<int>(H),
                static_cast<int>(W), static_cast<int>(scale));
        else
            upsample_scalar_kernel<float><<<rs_grid(total), kRsThreads, 0, stream>>>(
                static_cast<const float *>(in), static_cast<float *>(out), planes, static_cast<int>(H),
                static_cast<int>(W), static_cast<int>(scale));
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

cudaError_t concat_launch(const void *in1, const void *in2, void *out, int64_t batch, int64_t n1,
                          int64_t n2, int dtype, cudaStream_t stream) {
    if (batch == 0 || n1 + n2 == 0) return cudaSuccess;
    const int64_t esz = dtype == kF16 ? 2 : 4;
    if ((n1 * esz) % 16 == 0 && (n2 * esz) % 16 == 0 && aligned_to(in1, 16) && aligned_to(in2, 16) &&
        aligned_to(out, 16)) {
        const long long v1 = n1 * esz / 16, v2 = n2 * esz / 16;
        concat_kernel<uint4><<<rs_grid(batch * (v1 + v2)), kRsThreads, 0, stream>>>(
            static_cast<const uint4 *>(in1), static_cast<const uint4 *>(in2), static_cast<uint4 *>(out), batch, v1, v2);
    } else if (dtype == kF16) {
        concat_kernel<unsigned short><<<rs_grid(batch * (n1 + n2)), kRsThreads, 0, stream>>>(
            static_cast<const unsigned short *>(in1), static_cast<const unsigned short *>(in2),
            static_cast<unsigned short *>(out), batch, n1, n2);
    } else {
        concat_kernel<uint32_t><<<rs_grid(batch * (n1 + n2)), kRsThreads, 0, stream>>>(
            static_cast<const uint32_t *>(in1), static_cast<const uint32_t *>(in2),
            static_cast<uint32_t *>(out), batch, n1, n2);
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

}  // namespace sdfl
