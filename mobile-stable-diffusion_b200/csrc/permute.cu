// permute3D__0_2_1 (util.cl:47-64): dst[i][k][j] = src[i][j][k], the [C, HW] <-> [HW, C] transposes
// around the transformer of a SpatialTransformer block (SpatialTransformer.cpp:127-140 and
// :154-162), and the same fused with the residual add that follows the second one
// (elemwise_add, SpatialTransformer.cpp:163-171): dst[i][k][j] = src[i][j][k] + res[i][k][j].
//
// The reference moves one element per work-item with one side of the copy strided by a whole
// row.  Here a CTA moves a 64 x 64 tile through shared memory: both the global reads (along k)
// and the global writes (along j) are pairs of elements in consecutive lanes, i.e. full 128- or
// 256-byte segments per warp.  Odd extents or unaligned pointers take the scalar 32 x 32 tiles.
#include "common.cuh"
#include "kernels.h"


namespace sdfl {

namespace {

template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<__half> { using type = __half2; };

template <typename T>
__device__ __forceinline__ typename Pair<T>::type pair_add(typename Pair<T>::type a, typename Pair<T>::type b);
template <>
__device__ __forceinline__ float2 pair_add<float>(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
template <>
__device__ __forceinline__ __half2 pair_add<__half>(__half2 a, __half2 b) {
    // fp32 add, one rounding: the same value as the reference's float add of the widened halves
    const float2 x = __half22float2(a), y = __half22float2(b);
    return __floats2half2_rn(x.x + y.x, x.y + y.y);
}

constexpr int kTile = 64;

// Persistent CTAs walk over 64 x 64 tiles (tile id = (i * tiles_j + jt) * tiles_k + kt).  A tile
// is fetched with asynchronous 4- or 8-byte copies straight into shared memory (cp.async: no
// registers hold data in flight) while the previous tile is written out, so every CTA always has
// a tile's worth of loads outstanding: with 8 KB tiles and plain loads the kernel was bound by
// bytes in flight per SM (1.2-1.5 TB/s fp16), not by HBM.  J and K even, pointers 2-element aligned.
// NS buffers per CTA: NS - 1 tiles are in flight while one is written out.  Two are enough: with
// four, fp16 (8 KB tiles) stayed at 4.2-4.3 TB/s -- there the 2-byte column reads and 4-byte
// stores of the write-out are the limit, not the bytes in flight.
template <typename T> struct Stages { static constexpr int N = 2; };

template <typename T, bool ADD>
__global__ void __launch_bounds__(256, 6)
transpose_pairs_kernel(const T *__restrict__ src, const T *res, T *dst, int J, int K, unsigned tiles_j,
                       unsigned tiles_k, unsigned long long total_tiles) {
    using P = typename Pair<T>::type;
    // odd row stride in 32-bit words (33 fp16, 65 fp32): the column reads of the write-out fall
    // on 16 different banks (two lanes per bank, the best this pairing allows)
    constexpr int kPad = sizeof(T) == 2 ? 2 : 1;
    using Tile = T[kTile][kTile + kPad];
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int NS = Stages<T>::N;
    Tile *tile = reinterpret_cast<Tile *>(smem_raw);              // [NS] source tiles
    Tile *rtile = tile + NS;                                      // [NS] residual tiles in dst layout (ADD only)
    const int tx = threadIdx.x, ty = threadIdx.y;
    const long long slice = static_cast<long long>(J) * K;

    // one commit group per call, empty past the last tile, so that "all but the newest NS - 1
    // groups are complete" always means "the tile about to be written out has landed"
    auto issue = [&](unsigned long long id, int buf) {
        if (id >= total_tiles) {
            asm volatile("cp.async.commit_group;" ::: "memory");
            return;
        }
        const unsigned kt = static_cast<unsigned>(id % tiles_k);
        const unsigned long long q = id / tiles_k;
        const unsigned jt = static_cast<unsigned>(q % tiles_j);
        const T *s = src + (q / tiles_j) * slice;
        const int k = kt * kTile + 2 * tx;
#pragma unroll
        for (int r = ty; r < kTile; r += 8) {
            const int j = jt * kTile + r;
            if (j < J && k < K) {
                const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(&tile[buf][r][2 * tx]));
                const T *g = s + static_cast<long long>(j) * K + k;
                // fp16: one 4-byte copy (rows are 132 bytes, so the pair is 4-byte aligned).  fp32: the
                // rows are 260 bytes, a pair is only 4-byte aligned in odd rows: two 4-byte copies.
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(g) : "memory");
                if (sizeof(T) == 4)
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d + 4u), "l"(g + 1) : "memory");
            }
        }
        if (ADD) {
            const T *a = res + (q / tiles_j) * slice;
            const int j = jt * kTile + 2 * tx;
#pragma unroll
            for (int r = ty; r < kTile; r += 8) {
                const int kk = kt * kTile + r;
                if (kk < K && j < J) {
                    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(&rtile[buf][r][2 * tx]));
                    const T *g = a + static_cast<long long>(kk) * J + j;
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(g) : "memory");
                    if (sizeof(T) == 4)
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d + 4u), "l"(g + 1) : "memory");
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    unsigned long long id = blockIdx.x;
#pragma unroll
    for (int s = 0; s < NS - 1; ++s) issue(id + static_cast<unsigned long long>(s) * gridDim.x, s);
    for (int buf = 0; id < total_tiles; id += gridDim.x, buf = buf + 1 == NS ? 0 : buf + 1) {
        issue(id + static_cast<unsigned long long>(NS - 1) * gridDim.x, buf == 0 ? NS - 1 : buf - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(NS - 1) : "memory");
        __syncthreads();
        const unsigned kt = static_cast<unsigned>(id % tiles_k);
        const unsigned long long q = id / tiles_k;
        const unsigned jt = static_cast<unsigned>(q % tiles_j);
        const long long base = (q / tiles_j) * slice;
        T *d = dst + base;
        const int j = jt * kTile + 2 * tx;
        if constexpr (sizeof(T) == 2) {
            // fp16: 2 x 2 blocks.  One 32-bit word of source row 2tx and one of row 2tx+1 (two
            // consecutive k each) give the pairs of output rows k and k+1: half as many
            // shared-memory loads as element-wise column reads.
#pragma unroll
            for (int pr = ty; pr < kTile / 2; pr += 8) {
                const int r0 = 2 * pr, k = kt * kTile + r0;
                if (k < K && j < J) {               // K is even: row k + 1 exists too
                    const uint32_t a = *reinterpret_cast<const uint32_t *>(&tile[buf][2 * tx][r0]);
                    const uint32_t b = *reinterpret_cast<const uint32_t *>(&tile[buf][2 * tx + 1][r0]);
                    uint32_t o0 = __byte_perm(a, b, 0x5410), o1 = __byte_perm(a, b, 0x7632);
                    const long long o = static_cast<long long>(k) * J + j;
                    if (ADD) {
                        const uint32_t w0 = *reinterpret_cast<const uint32_t *>(&rtile[buf][r0][2 * tx]);
                        const uint32_t w1 = *reinterpret_cast<const uint32_t *>(&rtile[buf][r0 + 1][2 * tx]);
                        P v0 = pair_add<T>(*reinterpret_cast<const P *>(&o0), *reinterpret_cast<const P *>(&w0));
                        P v1 = pair_add<T>(*reinterpret_cast<const P *>(&o1), *reinterpret_cast<const P *>(&w1));
                        o0 = *reinterpret_cast<const uint32_t *>(&v0);
                        o1 = *reinterpret_cast<const uint32_t *>(&v1);
                    }
                    *reinterpret_cast<uint32_t *>(d + o) = o0;
                    *reinterpret_cast<uint32_t *>(d + o + J) = o1;
                }
            }
        } else {
#pragma unroll
        for (int r = ty; r < kTile; r += 8) {
            const int k = kt * kTile + r;
            if (k < K && j < J) {
                P v;
                v.x = tile[buf][2 * tx][r];
                v.y = tile[buf][2 * tx + 1][r];
                const long long o = static_cast<long long>(k) * J + j;
                if (ADD) {
                    P w;
                    w.x = rtile[buf][r][2 * tx];
                    w.y = rtile[buf][r][2 * tx + 1];
                    v = pair_add<T>(v, w);
                }
                *reinterpret_cast<P *>(d + o) = v;
            }
        }
        }
        __syncthreads();      // this buffer is the target of the copies issued next time round
    }
}

// Any extents and alignment: 32 x 32 tiles, one element per access.
template <typename T, bool ADD>
__global__ void __launch_bounds__(256)
transpose_scalar_kernel(const T *__restrict__ src, const T *res, T *dst, long long I, int J, int K) {
    __shared__ T tile[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int k0 = blockIdx.x * 32, j0 = blockIdx.y * 32;
    for (long long i = blockIdx.z; i < I; i += gridDim.z) {
        const T *s = src + i * J * K;
#pragma unroll
        for (int r = ty; r < 32; r += 8) {
            const int j = j0 + r, k = k0 + tx;
            if (j < J && k < K) tile[r][tx] = s[static_cast<long long>(j) * K + k];
        }
        __syncthreads();
        T *d = dst + i * J * K;
#pragma unroll
        for (int r = ty; r < 32; r += 8) {
            const int k = k0 + r, j = j0 + tx;
            if (k < K && j < J) {
                const long long o = static_cast<long long>(k) * J + j;
                T v = tile[tx][r];
                if (ADD) v = from_float<T>(to_float<T>(v) + to_float<T>(res[i * J * K + o]));
                d[o] = v;
            }
        }
        __syncthreads();
    }
}

template <typename T, bool ADD>
constexpr size_t transpose_smem_bytes() {
    return (ADD ? 2 : 1) * Stages<T>::N * sizeof(T) * kTile * (kTile + (sizeof(T) == 2 ? 2 : 1));
}

template <typename T, bool ADD>
cudaError_t transpose_dispatch(const void *src, const void *res, void *dst, int64_t I, int64_t J,
                               int64_t K, cudaStream_t stream) {
    const uintptr_t align = 2 * sizeof(T) - 1;
    const bool pairs = J % 2 == 0 && K % 2 == 0 && (reinterpret_cast<uintptr_t>(src) & align) == 0 &&
                       (reinterpret_cast<uintptr_t>(dst) & align) == 0 &&
                       (!ADD || (reinterpret_cast<uintptr_t>(res) & align) == 0);
    const T *s = static_cast<const T *>(src), *r = static_cast<const T *>(res);
    T *d = static_cast<T *>(dst);
    if (pairs) {
        const unsigned tiles_j = static_cast<unsigned>((J + kTile - 1) / kTile);
        const unsigned tiles_k = static_cast<unsigned>((K + kTile - 1) / kTile);
        const unsigned long long total = static_cast<unsigned long long>(I) * tiles_j * tiles_k;
        constexpr size_t smem = transpose_smem_bytes<T, ADD>();
        if (smem > 48 * 1024) {
            static std::atomic<bool> done[64];
            int dev = 0;
            cudaError_t e = cudaGetDevice(&dev);
            if (e != cudaSuccess) return e;
            if (!(dev >= 0 && dev < 64 && done[dev].load(std::memory_order_acquire))) {
                e = cudaFuncSetAttribute(transpose_pairs_kernel<T, ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
                if (e != cudaSuccess) return e;
                if (dev >= 0 && dev < 64) done[dev].store(true, std::memory_order_release);
            }
        }
        const unsigned long long ctas = 148ull * (200 * 1024 / smem < 6 ? 200 * 1024 / smem : 6);
        const unsigned grid = static_cast<unsigned>(total < ctas ? total : ctas);
        transpose_pairs_kernel<T, ADD><<<grid, dim3(32, 8), smem, stream>>>(s, r, d, static_cast<int>(J),
                                                                        static_cast<int>(K), tiles_j, tiles_k, total);
    } else {
        const dim3 grid(static_cast<unsigned>((K + 31) / 32), static_cast<unsigned>((J + 31) / 32),
                        static_cast<unsigned>(I < 65535 ? I : 65535));
        if (grid.y > 65535) return cudaErrorInvalidValue;
        transpose_scalar_kernel<T, ADD><<<grid, dim3(32, 8), 0, stream>>>(s, r, d, I, static_cast<int>(J),
                                                                         static_cast<int>(K));
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

}  // namespace

cudaError_t permute_021_launch(const void *src, const void *res, void *dst, int64_t I, int64_t J,
                               int64_t K, int dtype, cudaStream_t stream) {
    if (I == 0 || J == 0 || K == 0) return cudaSuccess;
    if (dtype == kF16)
        return res ? transpose_dispatch<__half, true>(src, res, dst, I, J, K, stream)
                   : transpose_dispatch<__half, false>(src, nullptr, dst, I, J, K, stream);
    return res ? transpose_dispatch<float, true>(src, res, dst, I, J, K, stream)
               : transpose_dispatch<float, false>(src, nullptr, dst, I, J, K, stream);
}

}  // namespace sdfl
