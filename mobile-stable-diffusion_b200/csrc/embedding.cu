// Token + position embedding gather, and the sinusoidal timestep embedding.
//
// Token path: the reference gathers rows on the HOST (TextEncoder.cpp:105-125: one std::copy
// per token from the table) and then runs elemwise_add with the positional table on the device
// (TextEncoder.cpp:141-151, util.cl:1-12).  Here both are one kernel:
//     out[b, t, :] = table[ids[b, t], :] + pos[t, :]
// A gather is a copy and an fp32 add is exactly rounded, so the result is bit-identical to the
// reference's two steps.  The reference does not check ids; this kernel never reads outside
// the table: a bad id zeroes its output row and raises bit 0 of *d_status.
//
// Timestep path: UNetModel::createTimestepEmbedding (UNetModel.cpp:1935-1958) is host float
// math: freq = exp(-log(max_period) * i / half), arg = t * freq, out = [cos(arg) | sin(arg)].
// arg reaches ~1000 rad, so one ulp of freq moves cos/sin by ~1e-4: freq is therefore formed
// in double and rounded once (correctly rounded, like glibc's expf), and sincos uses the
// full-range single-precision functions, never the SFU approximations.
#include "common.cuh"
#include "kernels.h"

namespace sdfl {

namespace {

constexpr int kEmbThreads = 128;

template <typename T, bool VECTORIZED>
__global__ void __launch_bounds__(kEmbThreads)
token_embedding_kernel(const long long *__restrict__ ids, const T *__restrict__ table,
                       const T *__restrict__ pos, T *__restrict__ out, long long tokens,
                       long long seq, long long d, long long vocab, int *status) {
    constexpr int VEC = VecOf<T>::N;
    for (long long tok = blockIdx.x; tok < tokens; tok += gridDim.x) {
        const long long id = ids[tok];
        const long long t = tok % seq;
        const bool ok = id >= 0 && id < vocab;
        if (!ok && threadIdx.x == 0 && status) atomicOr(status, 1);
        if (VECTORIZED) {
            const long long nvec = d / VEC;
            const uint4 *src = reinterpret_cast<const uint4 *>(table + (ok ? id : 0) * d);
            const uint4 *pv = reinterpret_cast<const uint4 *>(pos + t * d);
            uint4 *dst = reinterpret_cast<uint4 *>(out + tok * d);
            for (long long i = threadIdx.x; i < nvec; i += kEmbThreads) {
                if (!ok) { dst[i] = make_uint4(0, 0, 0, 0); continue; }
                float x[VEC], p[VEC];
                unpack<T>(__ldg(src + i), x);
                unpack<T>(__ldg(pv + i), p);
#pragma unroll
                for (int j = 0; j < VEC; ++j) x[j] = x[j] + p[j];
                dst[i] = pack<T>(x);
            }
        } else {
            for (long long i = threadIdx.x; i < d; i += kEmbThreads) {
                const float v = ok ? to_float<T>(table[id * d + i]) + to_float<T>(pos[t * d + i]) : 0.f;
                out[tok * d + i] = from_float<T>(v);
            }
        }
    }
}

template <typename T>
__global__ void timestep_embedding_kernel(const long long *__restrict__ t, T *__restrict__ out,
                                          int batch, int dim, float max_period) {
    const int half = dim / 2;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= batch * half) return;
    const int n = i / half, k = i - n * half;
    // (-log(max_period)) * (float)k / (float)half, each step rounded to float as in the
    // reference; log and exp themselves are evaluated in double and rounded once.
    const float neg_log = -static_cast<float>(log(static_cast<double>(max_period)));
    const float e = __fdiv_rn(__fmul_rn(neg_log, static_cast<float>(k)), static_cast<float>(half));
    const float freq = static_cast<float>(exp(static_cast<double>(e)));
    const float arg = __fmul_rn(static_cast<float>(t[n]), freq);
    out[static_cast<size_t>(n) * dim + k] = from_float<T>(cosf(arg));
    out[static_cast<size_t>(n) * dim + half + k] = from_float<T>(sinf(arg));
    if (k == 0 && (dim & 1)) out[static_cast<size_t>(n) * dim + dim - 1] = from_float<T>(0.f);
}

}  // namespace

cudaError_t token_embedding_launch(const int64_t *ids, const void *table, const void *pos,
                                   void *out, int64_t batch, int64_t t, int64_t d, int64_t vocab,
                                   int dtype, int *d_status, cudaStream_t stream) {
    const int64_t tokens = batch * t;
    if (tokens == 0 || d == 0) return cudaSuccess;
    const unsigned grid = static_cast<unsigned>(tokens < sm_count() * 16 ? tokens : sm_count() * 16);
    const int64_t esz = dtype == kF16 ? 2 : 4;
    const bool vec_ok = (d * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(table) & 15u) == 0 &&
                        (reinterpret_cast<uintptr_t>(pos) & 15u) == 0 &&
                        (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
    const long long *lids = reinterpret_cast<const long long *>(ids);
    if (dtype == kF16) {
        auto *tb = static_cast<const __half *>(table);
        auto *pp = static_cast<const __half *>(pos);
        auto *oo = static_cast<__half *>(out);
        if (vec_ok) token_embedding_kernel<__half, true><<<grid, kEmbThreads, 0, stream>>>(lids, tb, pp, oo, tokens, t, d, vocab, d_status);
        else token_embedding_kernel<__half, false><<<grid, kEmbThreads, 0, stream>>>(lids, tb, pp, oo, tokens, t, d, vocab, d_status);
    } else {
        auto *tb = static_cast<const float *>(table);
        auto *pp = static_cast<const float *>(pos);
        auto *oo = static_cast<float *>(out);
        if (vec_ok) token_embedding_kernel<float, true><<<grid, kEmbThreads, 0, stream>>>(lids, tb, pp, oo, tokens, t, d, vocab, d_status);
        else token_embedding_kernel<float, false><<<grid, kEmbThreads, 0, stream>>>(lids, tb, pp, oo, tokens, t, d, vocab, d_status);
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

cudaError_t timestep_embedding_launch(const int64_t *t, void *out, int64_t batch, int64_t dim,
                                      float max_period, int dtype, cudaStream_t stream) {
    const int64_t work = batch * (dim / 2);
    if (work == 0) return cudaSuccess;
    const unsigned grid = static_cast<unsigned>((work + 127) / 128);
    const long long *lt = reinterpret_cast<const long long *>(t);
    if (dtype == kF16)
        timestep_embedding_kernel<__half><<<grid, 128, 0, stream>>>(
            lt, static_cast<__half *>(out), static_cast<int>(batch), static_cast<int>(dim), max_period);
    else
        timestep_embedding_kernel<float><<<grid, 128, 0, stream>>>(
            lt, static_cast<float *>(out), static_cast<int>(batch), static_cast<int>(dim), max_period);
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

}  // namespace sdfl
