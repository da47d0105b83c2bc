// permute3D__0_2_1 (util.cl:47-64): dst[i][k][j] = src[i][j][k], the [C, HW] <-> [HW, C] transposes
// around the transformer of a SpatialTransformer block (SpatialTransformer.cpp:127-140 and
// :154-162), and the same fused with the residual add that follows the second one
// (elemwise_add, SpatialTransformer.cpp:163-171): dst[i][k][j] = src[i][j][k] + res[i][k][j].
//
// The reference moves one element per work-item with one side of the copy strided by a whole
// row.  Here a CTA moves a 64 x 64 tile through shared memory: both the global reads (along k)
// and the global writes (along j) are pairs of elements in consecutive lanes, i.e. full 128- or
// 256-byte segments per warp (fp16 with extents that are multiples of 8: 16-byte accesses and an
// ldmatrix.trans write-out, transpose_h8_kernel).  Odd extents or unaligned pointers take the
// scalar 32 x 32 tiles.
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

// fp16 with J and K multiples of 8 and 16-byte aligned pointers: the same persistent double-buffered
// walk over tiles, but every access is 16 bytes wide.  A tile arrives by 16-byte cp.async into rows
// padded by 16 bytes (eight consecutive rows start in eight different groups of four banks).  It
// leaves through ldmatrix.trans: one x4 instruction hands a warp four transposed 8 x 8 blocks
// (source rows j0 .. j0+31, columns k0 .. k0+7), lane (r, q) holding the pairs (j0 + 8m + 2q, +1)
// of output row k0 + r for m = 0 .. 3; a 4 x 4 exchange inside each quad of lanes turns that into
// the eight consecutive j of block q, one 16-byte store per lane.  The 2-byte column reads that
// capped the pair kernel at 4.5 TB/s are gone.
__device__ __forceinline__ uint32_t quad_pick(const uint32_t (&v)[4], uint32_t i) {
    return i == 0 ? v[0] : i == 1 ? v[1] : i == 2 ? v[2] : v[3];
}

// TJ x TK: tile extents along the source's rows (j) and columns (k), multiples of 32 and 8.
template <bool ADD, int TJ, int TK>
__global__ void __launch_bounds__(256)
transpose_h8_kernel(const __half *__restrict__ src, const __half *res, __half *dst, int J, int K, unsigned tiles_j,
                    unsigned tiles_k, unsigned long long total_tiles) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kSrcRow = TK * 2 + 16, kResRow = TJ * 2 + 16;       // bytes; 16 mod 128 either way
    constexpr int kSrcTile = TJ * kSrcRow, kResTile = TK * kResRow;
    unsigned char *tile = smem_raw;                       // [2] source tiles, rows along k
    unsigned char *rtile = smem_raw + 2 * kSrcTile;       // [2] residual tiles, rows along j (ADD only)
    const int tid = threadIdx.y * 32 + threadIdx.x, lane = threadIdx.x, warp = threadIdx.y;
    const long long slice = static_cast<long long>(J) * K;

    auto issue = [&](unsigned long long id, int buf) {
        if (id < total_tiles) {
            const unsigned kt = static_cast<unsigned>(id % tiles_k);
            const unsigned long long q = id / tiles_k;
            const unsigned jt = static_cast<unsigned>(q % tiles_j);
            const __half *s = src + (q / tiles_j) * slice;
#pragma unroll
            for (int t = tid; t < TJ * (TK / 8); t += 256) {          // TJ rows x TK/8 segments of 16 bytes
                const int r = t / (TK / 8), seg = t % (TK / 8);
                const int j = jt * TJ + r, k = kt * TK + seg * 8;
                if (j < J && k < K) {
                    const uint32_t d = static_cast<uint32_t>(
                        __cvta_generic_to_shared(tile + buf * kSrcTile + r * kSrcRow + seg * 16));
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(s + static_cast<long long>(j) * K + k) : "memory");
                }
            }
            if (ADD) {
                const __half *a = res + (q / tiles_j) * slice;
#pragma unroll
                for (int t = tid; t < TK * (TJ / 8); t += 256) {
                    const int r = t / (TJ / 8), seg = t % (TJ / 8);
                    const int kk = kt * TK + r, jj = jt * TJ + seg * 8;
                    if (kk < K && jj < J) {
                        const uint32_t d = static_cast<uint32_t>(
                            __cvta_generic_to_shared(rtile + buf * kResTile + r * kResRow + seg * 16));
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(a + static_cast<long long>(kk) * J + jj) : "memory");
                    }
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");      // one group per call, empty past the end
    };

    unsigned long long id = blockIdx.x;
    issue(id, 0);
    for (int buf = 0; id < total_tiles; id += gridDim.x, buf ^= 1) {
        issue(id + gridDim.x, buf ^ 1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const unsigned kt = static_cast<unsigned>(id % tiles_k);
        const unsigned long long q = id / tiles_k;
        const unsigned jt = static_cast<unsigned>(q % tiles_j);
        __half *d = dst + (q / tiles_j) * slice;
        const uint32_t rr = lane >> 2, qq = lane & 3;
#pragma unroll
        for (int kb = warp; kb < TK / 8; kb += 8) {
            const int k = kt * TK + kb * 8 + rr;                  // this lane's output row
#pragma unroll
            for (int jg = 0; jg < TJ / 32; ++jg) {
                // four 8 x 8 blocks: source rows jg*32 + 8m .. +7 (lane l gives the address of row
                // jg*32 + l), columns kb*8 .. +7
                const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(
                    tile + buf * kSrcTile + (jg * 32 + lane) * kSrcRow + kb * 16));
                uint32_t in[4];
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                             : "=r"(in[0]), "=r"(in[1]), "=r"(in[2]), "=r"(in[3]) : "r"(addr));
                // exchange inside the quad: lane q ends up with word q of lanes 0 .. 3
                uint32_t out[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (uint32_t s = 0; s < 4; ++s) {
                    const uint32_t send = quad_pick(in, (qq - s) & 3u);
                    const uint32_t got = __shfl_sync(0xffffffffu, send, (lane & ~3u) | ((qq + s) & 3u));
                    const uint32_t slot = (qq + s) & 3u;
                    out[0] = slot == 0 ? got : out[0];
                    out[1] = slot == 1 ? got : out[1];
                    out[2] = slot == 2 ? got : out[2];
                    out[3] = slot == 3 ? got : out[3];
                }
                const int j = jt * TJ + jg * 32 + qq * 8;
                if (k < K && j < J) {
                    uint4 v = make_uint4(out[0], out[1], out[2], out[3]);
                    if (ADD) {
                        const uint4 w = *reinterpret_cast<const uint4 *>(
                            rtile + buf * kResTile + (kb * 8 + rr) * kResRow + (jg * 32 + qq * 8) * 2);
                        float x[8], y[8];
                        unpack<__half>(v, x);
                        unpack<__half>(w, y);
#pragma unroll
                        for (int e = 0; e < 8; ++e) x[e] += y[e];       // fp32 add, one rounding, as the reference
                        v = pack<__half>(x);
                    }
                    st_stream(d + static_cast<long long>(k) * J + j, v);
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

template <bool ADD, int TJ, int TK>
cudaError_t launch_h8(const __half *s, const __half *r, __half *d, int64_t I, int64_t J, int64_t K, cudaStream_t stream) {
    constexpr size_t smem = 2 * (TJ * (TK * 2 + 16) + (ADD ? TK * (TJ * 2 + 16) : 0));
    if (smem > 48 * 1024) {      // once per device and instantiation, not per launch
        static std::atomic<bool> done[64];
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (!(dev >= 0 && dev < 64 && done[dev].load(std::memory_order_acquire))) {
            e = cudaFuncSetAttribute(transpose_h8_kernel<ADD, TJ, TK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem));
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) done[dev].store(true, std::memory_order_release);
        }
    }
    const unsigned tiles_j = static_cast<unsigned>((J + TJ - 1) / TJ), tiles_k = static_cast<unsigned>((K + TK - 1) / TK);
    const unsigned long long total = static_cast<unsigned long long>(I) * tiles_j * tiles_k;
    const unsigned long long per_sm = 220 * 1024 / (smem + 1024) < 6 ? 220 * 1024 / (smem + 1024) : 6;
    const unsigned long long ctas = static_cast<unsigned long long>(sm_count()) * per_sm;
    const unsigned grid = static_cast<unsigned>(total < ctas ? total : ctas);
    transpose_h8_kernel<ADD, TJ, TK><<<grid, dim3(32, 8), smem, stream>>>(s, r, d, static_cast<int>(J), static_cast<int>(K),
                                                                         tiles_j, tiles_k, total);
    return cudaGetLastError();
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
    if constexpr (sizeof(T) == 2) {
        const bool wide = J % 8 == 0 && K % 8 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                          (reinterpret_cast<uintptr_t>(dst) & 15) == 0 &&
                          (!ADD || (reinterpret_cast<uintptr_t>(res) & 15) == 0);
        if (wide) {
            // 64 x 128 tiles, the long side (256-byte row segments) along a dimension that is a
            // multiple of 128, the longer one if both are: on [64,320,4096] 80 % of the HBM peak
            // against 71 % with 64 x 64 tiles, on [64,4096,320] with the residual 86 % against 82 %
            // (128 x 128 tiles: 71 % and 40 %).
            // Small tensors keep 64 x 64 tiles: with fewer tiles than two rounds of the persistent
            // grid the larger tiles leave SMs idle ([2,320,4096]: 5.5 against 5.0 us).
            const bool enough = I * ((J + 63) / 64) * ((K + 63) / 64) >= 4 * sm_count() * 6;
            const bool k_wide = enough && K % 128 == 0 && (J % 128 != 0 || K >= J);
            const bool j_wide = enough && !k_wide && J % 128 == 0;
            cudaError_t err = k_wide   ? launch_h8<ADD, 64, 128>(s, r, d, I, J, K, stream)
                              : j_wide ? launch_h8<ADD, 128, 64>(s, r, d, I, J, K, stream)
                                       : launch_h8<ADD, 64, 64>(s, r, d, I, J, K, stream);
            if (err == cudaSuccess) g_launches.fetch_add(1);
            return err;
        }
    }
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
        const unsigned long long ctas = static_cast<unsigned long long>(sm_count()) * (200 * 1024 / smem < 6 ? 200 * 1024 / smem : 6);
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
