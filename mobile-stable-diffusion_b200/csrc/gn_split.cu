// GroupNorm (+SiLU), split path and the reference's kernels by name.
//
// Split path: any shape and alignment.  Kernel 1 writes one (mean, M2) pair per chunk to a scratch
// buffer; kernel 2 merges the chunk pairs of its slab in a fixed order and normalises (or, for the
// channels-last form, normalises and transposes tile by tile).  Also the stand-alone
// local_reduction_mean / local_reduction_variance / group_norm / layer_norm kernels that keep the
// reference's three-launch call sequence (group_norm.cl:1-76, layer_norm.cl:58-78).
#include "gn_device.cuh"

namespace sdfl {

namespace {

// ---------------------------------------------------------------------------------------------
// Split path
// ---------------------------------------------------------------------------------------------
constexpr int kSplitThreads = 512;

struct SplitArgs {
    const void *in;
    void *out;
    const float *w;
    const float *b;
    const void *bias;      // [batch, C] addend of the storage type, or nullptr
    uint32_t channels;     // C
    float *partial;        // [units * splits * 2]  (mean, M2) per chunk
    uint32_t slab_elems;
    uint32_t chunk_elems;  // multiple of the vector width when `vec` is set
    uint32_t splits;
    uint32_t cpg, groups;
    uint32_t vec;          // 16-byte accesses allowed (alignment and divisibility hold)
    uint32_t vec_uniform;  // and a vector never straddles a channel
    float eps;
    FastDiv hw_div;
};

template <typename T>
__global__ void __launch_bounds__(kSplitThreads) gn_split_stats_kernel(const SplitArgs a) {
    constexpr int VEC = VecOf<T>::N;
    __shared__ Moments warp_m[kSplitThreads / 32];
    const uint32_t unit = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
    const uint32_t e0 = split * a.chunk_elems;
    const uint32_t e1 = min(a.slab_elems, e0 + a.chunk_elems);
    const T *x = static_cast<const T *>(a.in) + static_cast<size_t>(unit) * a.slab_elems;
    const T *erow = a.bias ? static_cast<const T *>(a.bias) +
                                 static_cast<size_t>(unit / a.groups) * a.channels + (unit % a.groups) * a.cpg
                           : nullptr;
    Shifted sh{0.f, 0.f, 0.f, 0.f};
    Moments m{0.f, 0.f, 0.f};
    if (a.vec && !erow) {
        // Shifted sums with the thread's first value as pivot, four independent 16-byte loads in
        // flight per thread, as in the cluster kernel.
        const uint4 *xv = reinterpret_cast<const uint4 *>(x);
        const uint32_t i1 = e1 / VEC;
        float shift = 0.f;
        float s[2] = {0.f, 0.f}, q[2] = {0.f, 0.f};
        uint32_t mine = 0, i = e0 / VEC + threadIdx.x;
        if (i < i1) shift = to_float<T>(reinterpret_cast<const T *>(xv + i)[0]);
        for (; i + 3 * kSplitThreads < i1; i += 4 * kSplitThreads) {
            const uint4 v0 = __ldg(xv + i), v1 = __ldg(xv + i + kSplitThreads);
            const uint4 v2 = __ldg(xv + i + 2 * kSplitThreads), v3 = __ldg(xv + i + 3 * kSplitThreads);
            stats_vec<T>(v0, shift, s, q);
            stats_vec<T>(v1, shift, s, q);
            stats_vec<T>(v2, shift, s, q);
            stats_vec<T>(v3, shift, s, q);
            mine += 4;
        }
        for (; i < i1; i += kSplitThreads) {
            stats_vec<T>(__ldg(xv + i), shift, s, q);
            ++mine;
        }
        const float cnt = static_cast<float>(mine * VEC);
        const float ss = s[0] + s[1], qq = q[0] + q[1];
        m.n = cnt;
        m.mean = mine ? shift + ss / cnt : 0.f;
        m.m2 = mine ? fmaxf(qq - ss * ss / cnt, 0.f) : 0.f;
    } else if (a.vec) {
        const uint4 *xv = reinterpret_cast<const uint4 *>(x);
        for (uint32_t i = e0 / VEC + threadIdx.x; i < e1 / VEC; i += kSplitThreads) {
            float f[VEC];
            unpack<T>(__ldg(xv + i), f);
            if (erow) {
#pragma unroll
                for (int j = 0; j < VEC; ++j) f[j] += to_float<T>(erow[a.hw_div.div(i * VEC + j)]);
            }
#pragma unroll
            for (int j = 0; j < VEC; ++j) sh.add(f[j]);
        }
    } else {
        for (uint32_t i = e0 + threadIdx.x; i < e1; i += kSplitThreads)
            sh.add(to_float<T>(x[i]) + (erow ? to_float<T>(erow[a.hw_div.div(i)]) : 0.f));
    }
    if (!(a.vec && !erow)) m = sh.done();
    m = warp_merge(m);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) warp_m[warp] = m;
    __syncthreads();
    if (warp == 0) {
        Moments t = lane < kSplitThreads / 32 ? warp_m[lane] : Moments{0.f, 0.f, 0.f};
        t = warp_merge(t);
        if (lane == 0) {
            a.partial[2 * static_cast<size_t>(blockIdx.x)] = t.mean;
            a.partial[2 * static_cast<size_t>(blockIdx.x) + 1] = t.m2;
        }
    }
}

template <typename T, int ACT>
__global__ void __launch_bounds__(kSplitThreads) gn_split_apply_kernel(const SplitArgs a) {
    constexpr int VEC = VecOf<T>::N;
    constexpr bool HALF = sizeof(T) == 2;
    __shared__ float s_stats[2];
    const uint32_t unit = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
    if (threadIdx.x < 32) {
        // lane l folds chunks l, l+32, ... in order; lanes are then folded by shuffles.
        Moments m{0.f, 0.f, 0.f};
        for (uint32_t s = threadIdx.x; s < a.splits; s += 32) {
            const uint32_t c0 = s * a.chunk_elems;
            const uint32_t c1 = min(a.slab_elems, c0 + a.chunk_elems);
            Moments y;
            y.n = c1 > c0 ? static_cast<float>(c1 - c0) : 0.f;
            const size_t p = 2 * (static_cast<size_t>(unit) * a.splits + s);
            y.mean = a.partial[p];
            y.m2 = a.partial[p + 1];
            m = merge(m, y);
        }
        m = warp_merge(m);
        if (threadIdx.x == 0) {
            s_stats[0] = m.mean;
            s_stats[1] = m.m2 / static_cast<float>(a.slab_elems);
        }
    }
    __syncthreads();
    const float mean = s_stats[0];
    const float rstd = 1.0f / sqrtf(s_stats[1] + a.eps);
    const uint32_t ch0 = (unit % a.groups) * a.cpg;
    const uint32_t e0 = split * a.chunk_elems;
    const uint32_t e1 = min(a.slab_elems, e0 + a.chunk_elems);
    const size_t base = static_cast<size_t>(unit) * a.slab_elems;
    const T *x = static_cast<const T *>(a.in) + base;
    T *y = static_cast<T *>(a.out) + base;
    const T *erow = a.bias ? static_cast<const T *>(a.bias) +
                                 static_cast<size_t>(unit / a.groups) * a.channels + ch0
                           : nullptr;
    if (a.vec) {
        const uint4 *xv = reinterpret_cast<const uint4 *>(x);
        uint4 *yv = reinterpret_cast<uint4 *>(y);
#pragma unroll 4
        for (uint32_t i = e0 / VEC + threadIdx.x; i < e1 / VEC; i += kSplitThreads) {
            float f[VEC];
            unpack<T>(ld_stream(xv + i), f);
            if (a.vec_uniform) {
                const uint32_t cl = a.hw_div.div(i * VEC), c = ch0 + cl;
                const float wv = __ldg(a.w + c), bv = __ldg(a.b + c);
                const float mc = erow ? mean - to_float<T>(erow[cl]) : mean;
#pragma unroll
                for (int j = 0; j < VEC; ++j)
                    f[j] = activate<ACT, HALF>(fmaf((f[j] - mc) * rstd, wv, bv));
            } else {
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    const uint32_t cl = a.hw_div.div(i * VEC + j), c = ch0 + cl;
                    const float mc = erow ? mean - to_float<T>(erow[cl]) : mean;
                    f[j] = activate<ACT, HALF>(
                        fmaf((f[j] - mc) * rstd, __ldg(a.w + c), __ldg(a.b + c)));
                }
            }
            st_stream(yv + i, pack<T>(f));
        }
    } else {
        for (uint32_t i = e0 + threadIdx.x; i < e1; i += kSplitThreads) {
            const uint32_t cl = a.hw_div.div(i), c = ch0 + cl;
            const float mc = erow ? mean - to_float<T>(erow[cl]) : mean;
            const float v = fmaf((to_float<T>(x[i]) - mc) * rstd, __ldg(a.w + c), __ldg(a.b + c));
            y[i] = from_float<T>(activate<ACT, HALF>(v));
        }
    }
}

// Second kernel of the split path with a channels-last store: out[n][p][c] = act(norm(in[n][c][p])).
// A CTA takes a tile of TS channels x TS pixels (TS = 64 with two elements per access, 32 with one),
// folds the per-chunk moments of the groups its channels belong to, applies the affine while
// loading (rows along the pixels: coalesced) and writes through shared memory with rows along
// the channels (coalesced again).  grid (ceil(hw / TS), ceil(C / TS), batch), block (32, 8).
template <typename T, int ACT, bool PAIRS>
__global__ void __launch_bounds__(256) gn_apply_nhwc_kernel(const SplitArgs a, uint32_t hw) {
    constexpr bool HALF = sizeof(T) == 2;
    constexpr int TS = PAIRS ? 64 : 32, E = PAIRS ? 2 : 1;
    constexpr int PAD = PAIRS ? (HALF ? 2 : 1) : 1;
    __shared__ __align__(8) T tile[TS][TS + PAD];
    __shared__ float4 coef[TS];        // per channel of the tile: mean, rstd, scale, shift
    const uint32_t tx = threadIdx.x, ty = threadIdx.y, tid = ty * 32 + tx;
    const uint32_t p0 = blockIdx.x * TS, c0 = blockIdx.y * TS, n = blockIdx.z;
    if (tid < TS && c0 + tid < a.channels) {
        const uint32_t c = c0 + tid;
        const size_t unit = static_cast<size_t>(n) * a.groups + c / a.cpg;
        Moments m{0.f, 0.f, 0.f};
        for (uint32_t s = 0; s < a.splits; ++s) {      // chunks in order: every CTA gets the same bits
            const uint32_t e0 = s * a.chunk_elems, e1 = min(a.slab_elems, e0 + a.chunk_elems);
            Moments y;
            y.n = e1 > e0 ? static_cast<float>(e1 - e0) : 0.f;
            y.mean = a.partial[2 * (unit * a.splits + s)];
            y.m2 = a.partial[2 * (unit * a.splits + s) + 1];
            m = merge(m, y);
        }
        const float var = m.m2 / static_cast<float>(a.slab_elems);
        coef[tid] = make_float4(m.mean, 1.0f / sqrtf(var + a.eps), __ldg(a.w + c), __ldg(a.b + c));
    }
    __syncthreads();
    const T *x = static_cast<const T *>(a.in) + static_cast<size_t>(n) * a.channels * hw;
    T *y = static_cast<T *>(a.out) + static_cast<size_t>(n) * a.channels * hw;
#pragma unroll
    for (int r = ty; r < TS; r += 8) {
        const uint32_t c = c0 + r, p = p0 + E * tx;
        if (c < a.channels && p < hw) {
            const float4 k = coef[r];
            const T *src = x + static_cast<size_t>(c) * hw + p;
            if (PAIRS) {
                float f0, f1;
                if (HALF) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(src));
                    f0 = f.x; f1 = f.y;
                } else {
                    const float2 f = *reinterpret_cast<const float2 *>(src);
                    f0 = f.x; f1 = f.y;
                }
                tile[r][2 * tx] = from_float<T>(activate<ACT, HALF>(fmaf((f0 - k.x) * k.y, k.z, k.w)));
                tile[r][2 * tx + 1] = from_float<T>(activate<ACT, HALF>(fmaf((f1 - k.x) * k.y, k.z, k.w)));
            } else {
                tile[r][tx] = from_float<T>(activate<ACT, HALF>(fmaf((to_float<T>(*src) - k.x) * k.y, k.z, k.w)));
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = ty; r < TS; r += 8) {
        const uint32_t p = p0 + r, c = c0 + E * tx;
        if (p < hw && c < a.channels) {
            T *dst = y + static_cast<size_t>(p) * a.channels + c;
            if (PAIRS) {
                const T v0 = tile[2 * tx][r], v1 = tile[2 * tx + 1][r];
                if (HALF) {
                    *reinterpret_cast<uint32_t *>(dst) =
                        static_cast<uint32_t>(*reinterpret_cast<const unsigned short *>(&v0)) |
                        (static_cast<uint32_t>(*reinterpret_cast<const unsigned short *>(&v1)) << 16);
                } else {
                    *reinterpret_cast<float2 *>(dst) = make_float2(to_float<T>(v0), to_float<T>(v1));
                }
            } else {
                *dst = tile[tx][r];
            }
        }
    }
}

// The same for tensors whose extents and alignment allow two elements per access, as a persistent
// kernel: CTAs walk over 64-channel x 64-pixel tiles (tile id = (n * tiles_c + ct) * tiles_p + pt,
// pixels fastest, so consecutive tiles of a CTA mostly share their channels and the folded
// moments are recomputed only when (n, ct) changes).  A tile is fetched with cp.async 4-byte
// copies straight into shared memory while the previous one is normalised and written out
// (double buffer): the loads in flight per SM no longer depend on registers.
template <typename T, int ACT>
__global__ void __launch_bounds__(256, 6)
gn_apply_nhwc_async_kernel(const SplitArgs a, uint32_t hw, unsigned tiles_c, unsigned tiles_p,
                           unsigned long long total_tiles) {
    constexpr bool HALF = sizeof(T) == 2;
    constexpr int TS = 64, PAD = HALF ? 2 : 1;
    using Tile = T[TS][TS + PAD];
    extern __shared__ __align__(16) unsigned char nhwc_smem[];
    Tile *tile = reinterpret_cast<Tile *>(nhwc_smem);                       // [2]
    float4 *coef = reinterpret_cast<float4 *>(nhwc_smem + 2 * sizeof(Tile)); // [TS]: mean, rstd, scale, shift
    const uint32_t tx = threadIdx.x, ty = threadIdx.y, tid = ty * 32 + tx;
    const size_t image = static_cast<size_t>(a.channels) * hw;

    auto issue = [&](unsigned long long id, int buf) {
        if (id < total_tiles) {
            const unsigned pt = static_cast<unsigned>(id % tiles_p);
            const unsigned long long q = id / tiles_p;
            const unsigned ct = static_cast<unsigned>(q % tiles_c);
            const T *x = static_cast<const T *>(a.in) + (q / tiles_c) * image;
            const uint32_t p = pt * TS + 2 * tx;
#pragma unroll
            for (int r = ty; r < TS; r += 8) {
                const uint32_t c = ct * TS + r;
                if (c < a.channels && p < hw) {
                    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(&tile[buf][r][2 * tx]));
                    const T *g = x + static_cast<size_t>(c) * hw + p;
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(g) : "memory");
                    if (!HALF) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d + 4u), "l"(g + 1) : "memory");
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");      // one group per call, empty past the end
    };

    unsigned long long id = blockIdx.x, coef_of = ~0ull;
    issue(id, 0);
    for (int buf = 0; id < total_tiles; id += gridDim.x, buf ^= 1) {
        issue(id + gridDim.x, buf ^ 1);
        const unsigned pt = static_cast<unsigned>(id % tiles_p);
        const unsigned long long q = id / tiles_p;              // n * tiles_c + ct
        const unsigned ct = static_cast<unsigned>(q % tiles_c);
        const unsigned long long n = q / tiles_c;
        if (q != coef_of) {                                      // uniform over the CTA
            if (tid < TS && ct * TS + tid < a.channels) {
                const uint32_t c = ct * TS + tid;
                const size_t unit = static_cast<size_t>(n) * a.groups + c / a.cpg;
                Moments m{0.f, 0.f, 0.f};
                for (uint32_t s = 0; s < a.splits; ++s) {        // chunks in order: every CTA gets the same bits
                    const uint32_t e0 = s * a.chunk_elems, e1 = min(a.slab_elems, e0 + a.chunk_elems);
                    Moments y;
                    y.n = e1 > e0 ? static_cast<float>(e1 - e0) : 0.f;
                    y.mean = a.partial[2 * (unit * a.splits + s)];
                    y.m2 = a.partial[2 * (unit * a.splits + s) + 1];
                    m = merge(m, y);
                }
                const float var = m.m2 / static_cast<float>(a.slab_elems);
                coef[tid] = make_float4(m.mean, 1.0f / sqrtf(var + a.eps), __ldg(a.w + c), __ldg(a.b + c));
            }
            coef_of = q;
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();                                         // the tile has landed; coef is written
        const uint32_t c = ct * TS + 2 * tx;
        const float4 k0 = coef[2 * tx], k1 = coef[2 * tx + 1];   // this thread's two channels
        T *y = static_cast<T *>(a.out) + n * image;
#pragma unroll
        for (int r = ty; r < TS; r += 8) {
            const uint32_t p = pt * TS + r;
            if (p < hw && c < a.channels) {
                const float v0 = activate<ACT, HALF>(fmaf((to_float<T>(tile[buf][2 * tx][r]) - k0.x) * k0.y, k0.z, k0.w));
                const float v1 = activate<ACT, HALF>(fmaf((to_float<T>(tile[buf][2 * tx + 1][r]) - k1.x) * k1.y, k1.z, k1.w));
                T *dst = y + static_cast<size_t>(p) * a.channels + c;
                if (HALF) *reinterpret_cast<__half2 *>(dst) = __floats2half2_rn(v0, v1);
                else *reinterpret_cast<float2 *>(dst) = make_float2(v0, v1);
            }
        }
        __syncthreads();      // tile[buf] is the target of the copies issued next time round; coef may change
    }
}

// fp16 with hw and C multiples of 8 and 16-byte aligned tensors: the same persistent walk with
// 16-byte accesses on both sides.  A TJ-channel x TK-pixel tile arrives by 16-byte cp.async into rows
// padded by 16 bytes; ldmatrix.trans hands each lane the pairs (channel c, c+1) of one pixel, the
// affine (+ SiLU) is applied there, and a 4 x 4 exchange inside each quad of lanes gives every lane
// eight consecutive channels of its pixel: one 16-byte store.
__device__ __forceinline__ uint32_t nhwc_quad_pick(const uint32_t (&v)[4], uint32_t i) {
    return i == 0 ? v[0] : i == 1 ? v[1] : i == 2 ? v[2] : v[3];
}

template <int ACT, int TJ, int TK>
__global__ void __launch_bounds__(256)
gn_apply_nhwc_h8_kernel(const SplitArgs a, uint32_t hw, unsigned tiles_c, unsigned tiles_p,
                        unsigned long long total_tiles) {
    extern __shared__ __align__(16) unsigned char nhwc_smem[];
    constexpr int kRow = TK * 2 + 16, kTileBytes = TJ * kRow;
    unsigned char *tile = nhwc_smem;                                          // [2]
    float2 *coef = reinterpret_cast<float2 *>(nhwc_smem + 2 * kTileBytes);    // [TJ]: folded scale, shift
    const int tid = threadIdx.y * 32 + threadIdx.x, lane = threadIdx.x, warp = threadIdx.y;
    const size_t image = static_cast<size_t>(a.channels) * hw;
    const __half *in = static_cast<const __half *>(a.in);
    __half *out = static_cast<__half *>(a.out);

    auto issue = [&](unsigned long long id, int buf) {
        if (id < total_tiles) {
            const unsigned pt = static_cast<unsigned>(id % tiles_p);
            const unsigned long long q = id / tiles_p;
            const unsigned ct = static_cast<unsigned>(q % tiles_c);
            const __half *x = in + (q / tiles_c) * image;
#pragma unroll
            for (int t = tid; t < TJ * (TK / 8); t += 256) {
                const int r = t / (TK / 8), seg = t % (TK / 8);
                const uint32_t c = ct * TJ + r, p = pt * TK + seg * 8;
                if (c < a.channels && p < hw) {
                    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(tile + buf * kTileBytes + r * kRow + seg * 16));
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(x + static_cast<size_t>(c) * hw + p) : "memory");
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");      // one group per call, empty past the end
    };

    unsigned long long id = blockIdx.x, coef_of = ~0ull;
    issue(id, 0);
    for (int buf = 0; id < total_tiles; id += gridDim.x, buf ^= 1) {
        issue(id + gridDim.x, buf ^ 1);
        const unsigned pt = static_cast<unsigned>(id % tiles_p);
        const unsigned long long q = id / tiles_p;              // n * tiles_c + ct
        const unsigned ct = static_cast<unsigned>(q % tiles_c);
        const unsigned long long n = q / tiles_c;
        if (q != coef_of) {                                      // uniform over the CTA
            if (tid < TJ && ct * TJ + tid < a.channels) {
                const uint32_t c = ct * TJ + tid;
                const size_t unit = static_cast<size_t>(n) * a.groups + c / a.cpg;
                Moments m{0.f, 0.f, 0.f};
                for (uint32_t s = 0; s < a.splits; ++s) {        // chunks in order: every CTA gets the same bits
                    const uint32_t e0 = s * a.chunk_elems, e1 = min(a.slab_elems, e0 + a.chunk_elems);
                    Moments y;
                    y.n = e1 > e0 ? static_cast<float>(e1 - e0) : 0.f;
                    y.mean = a.partial[2 * (unit * a.splits + s)];
                    y.m2 = a.partial[2 * (unit * a.splits + s) + 1];
                    m = merge(m, y);
                }
                const float var = m.m2 / static_cast<float>(a.slab_elems);
                const Affine<__half> af = make_affine<__half, ACT>(m.mean, 1.0f / sqrtf(var + a.eps), __ldg(a.w + c), __ldg(a.b + c));
                coef[tid] = make_float2(af.p0, af.p1);
            }
            coef_of = q;
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();                                         // the tile has landed; coef is written
        __half *y = out + n * image;
        const uint32_t rr = lane >> 2, qq = lane & 3;
#pragma unroll
        for (int kb = warp; kb < TK / 8; kb += 8) {
            const uint32_t p = pt * TK + kb * 8 + rr;            // this lane's pixel
#pragma unroll
            for (int jg = 0; jg < TJ / 32; ++jg) {
                const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(
                    tile + buf * kTileBytes + (jg * 32 + lane) * kRow + kb * 16));
                uint32_t v[4];
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr));
#pragma unroll
                for (int m = 0; m < 4; ++m) {                    // channels jg*32 + 8m + 2q, +1 of pixel p
                    const float2 k0 = coef[jg * 32 + 8 * m + 2 * qq], k1 = coef[jg * 32 + 8 * m + 2 * qq + 1];
                    const float2 x = __half22float2(*reinterpret_cast<const __half2 *>(&v[m]));
                    const float h0 = fmaf(x.x, k0.x, k0.y), h1 = fmaf(x.y, k1.x, k1.y);
                    const __half2 r = __floats2half2_rn(ACT == kActSilu ? fmaf(h0, tanh_approx(h0), h0) : h0,
                                                        ACT == kActSilu ? fmaf(h1, tanh_approx(h1), h1) : h1);
                    v[m] = *reinterpret_cast<const uint32_t *>(&r);
                }
                uint32_t o[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (uint32_t s = 0; s < 4; ++s) {               // lane q ends up with word q of lanes 0 .. 3
                    const uint32_t send = nhwc_quad_pick(v, (qq - s) & 3u);
                    const uint32_t got = __shfl_sync(0xffffffffu, send, (lane & ~3u) | ((qq + s) & 3u));
                    const uint32_t slot = (qq + s) & 3u;
                    o[0] = slot == 0 ? got : o[0];
                    o[1] = slot == 1 ? got : o[1];
                    o[2] = slot == 2 ? got : o[2];
                    o[3] = slot == 3 ? got : o[3];
                }
                const uint32_t c = ct * TJ + jg * 32 + qq * 8;
                if (p < hw && c < a.channels)
                    st_stream(y + static_cast<size_t>(p) * a.channels + c, make_uint4(o[0], o[1], o[2], o[3]));
            }
        }
        __syncthreads();      // tile[buf] is the target of the copies issued next time round; coef may change
    }
}

template <int ACT, int TJ, int TK>
cudaError_t launch_nhwc_h8(const SplitArgs &a, const GnShape &s, cudaStream_t stream) {
    constexpr size_t smem = 2 * TJ * (TK * 2 + 16) + TJ * sizeof(float2);
    const unsigned tiles_c = static_cast<unsigned>((s.channels + TJ - 1) / TJ), tiles_p = static_cast<unsigned>((s.hw + TK - 1) / TK);
    const unsigned long long total = static_cast<unsigned long long>(s.batch) * tiles_c * tiles_p;
    const unsigned long long ctas = static_cast<unsigned long long>(sm_count()) * 6;
    const unsigned grid = static_cast<unsigned>(total < ctas ? total : ctas);
    gn_apply_nhwc_h8_kernel<ACT, TJ, TK><<<grid, dim3(32, 8), smem, stream>>>(a, static_cast<uint32_t>(s.hw), tiles_c, tiles_p, total);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Stand-alone kernels for the reference's three-launch sequence
// ---------------------------------------------------------------------------------------------
constexpr int kStatsThreads = 256;

// out[g] = sum(in[g*n .. (g+1)*n)) / n                      (group_norm.cl:1-27)
// out[g] = sum((in - mean[g])^2) / n  when `mean` is given   (group_norm.cl:29-57)
template <typename T>
__global__ void __launch_bounds__(kStatsThreads)
stats_kernel(const T *__restrict__ in, const float *__restrict__ mean, float *__restrict__ out,
             long long n) {
    __shared__ float red[33];
    const T *x = in + static_cast<size_t>(blockIdx.x) * n;
    const float m = mean ? mean[blockIdx.x] : 0.f;
    float acc = 0.f;
    for (long long i = threadIdx.x; i < n; i += kStatsThreads) {
        const float v = to_float<T>(x[i]);
        if (mean) {
            const float d = v - m;
            acc = fmaf(d, d, acc);
        } else {
            acc += v;
        }
    }
    const float t = block_sum(acc, red);
    if (threadIdx.x == 0) out[blockIdx.x] = t / static_cast<float>(n);
}

// The same for 16-byte aligned groups whose length is a multiple of the vector width: a thread-block
// cluster of S CTAs per group (S = 1, 2, 4 or 8, chosen so that the grid fills the SMs even with 32
// groups), each CTA sums its share with four 16-byte loads in flight per thread, and rank 0 folds
// the S partial sums in rank order through distributed shared memory -- no scratch buffer, no
// atomics, the same bits on every run.
template <typename T>
__global__ void __launch_bounds__(kStatsThreads)
stats_vec_kernel(const uint4 *__restrict__ in, const float *__restrict__ mean, float *__restrict__ out,
                 unsigned long long nvec) {
    constexpr int VEC = VecOf<T>::N;
    __shared__ float red[33];
    __shared__ float cta_sum;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned S = cluster.num_blocks(), rank = cluster.block_rank();
    const unsigned long long group = blockIdx.x / S;
    const uint4 *x = in + group * nvec;
    const unsigned long long v0 = nvec * rank / S, v1 = nvec * (rank + 1) / S;
    const bool var = mean != nullptr;
    const float m = var ? mean[group] : 0.f;
    float acc[2] = {0.f, 0.f};
    auto fold = [&](const uint4 &v) {
        float f[VEC];
        unpack<T>(v, f);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const float d = f[j] - m;              // m = 0 for the mean
            acc[j & 1] = var ? fmaf(d, d, acc[j & 1]) : acc[j & 1] + d;
        }
    };
    unsigned long long i = v0 + threadIdx.x;
    for (; i + 3ull * kStatsThreads < v1; i += 4ull * kStatsThreads) {
        const uint4 a0 = ld_stream(x + i), a1 = ld_stream(x + i + kStatsThreads);
        const uint4 a2 = ld_stream(x + i + 2 * kStatsThreads), a3 = ld_stream(x + i + 3 * kStatsThreads);
        fold(a0); fold(a1); fold(a2); fold(a3);
    }
    for (; i < v1; i += kStatsThreads) fold(ld_stream(x + i));
    const float t = block_sum(acc[0] + acc[1], red);
    if (S == 1) {
        if (threadIdx.x == 0) out[group] = t / static_cast<float>(nvec * VEC);
        return;
    }
    if (threadIdx.x == 0) cta_sum = t;
    cluster.sync();                                  // every CTA's partial sum is in its shared memory
    if (rank == 0 && threadIdx.x == 0) {
        float total = 0.f;
        for (unsigned r = 0; r < S; ++r) total += *cluster.map_shared_rank(&cta_sum, r);
        out[group] = total / static_cast<float>(nvec * VEC);
    }
    cluster.sync();                                  // nobody leaves while rank 0 still reads
}

// group_norm.cl:59-76 with the weight index wrapped per image: c = (i / channelSize) % C.
// Vector form (16-byte aligned, group and channel sizes multiples of the vector width, fewer than
// 2^31 vectors): the group and channel of a vector by multiply-high divisions, one reciprocal
// square root per vector.
template <typename T>
__global__ void __launch_bounds__(256)
gn_apply_vec_kernel(const uint4 *__restrict__ in, const float *__restrict__ mean, const float *__restrict__ var,
                    const float *__restrict__ w, const float *__restrict__ b, FastDiv group_div, FastDiv chan_div,
                    FastDiv wrap_div, float eps, uint4 *__restrict__ out, uint32_t nvec) {
    constexpr int VEC = VecOf<T>::N;
    for (uint32_t i = blockIdx.x * 256u + threadIdx.x; i < nvec; i += gridDim.x * 256u) {
        const uint32_t g = group_div.div(i);
        const uint32_t q = chan_div.div(i);
        const uint32_t c = q - wrap_div.div(q) * wrap_div.d;
        const float mu = __ldg(mean + g), inv = 1.0f / sqrtf(__ldg(var + g) + eps);
        const float wc = __ldg(w + c), bc = __ldg(b + c);
        float f[VEC];
        unpack<T>(ld_stream(in + i), f);
#pragma unroll
        for (int j = 0; j < VEC; ++j) f[j] = fmaf((f[j] - mu) * inv, wc, bc);
        st_stream(out + i, pack<T>(f));
    }
}

// layer_norm.cl:63-78, vector form: dim a multiple of the vector width, everything 16-byte aligned.
template <typename T>
__global__ void __launch_bounds__(256)
ln_apply_vec_kernel(const uint4 *__restrict__ in, const float *__restrict__ mean, const float *__restrict__ var,
                    const float *__restrict__ w, const float *__restrict__ b, FastDiv row_div, float eps,
                    uint4 *__restrict__ out, uint32_t nvec) {
    constexpr int VEC = VecOf<T>::N;
    for (uint32_t i = blockIdx.x * 256u + threadIdx.x; i < nvec; i += gridDim.x * 256u) {
        const uint32_t r = row_div.div(i);
        const uint32_t k = (i - r * row_div.d) * VEC;
        const float mu = __ldg(mean + r), inv = 1.0f / sqrtf(__ldg(var + r) + eps);
        float f[VEC], wk[VEC], bk[VEC];
        unpack<T>(ld_stream(in + i), f);
#pragma unroll
        for (int j = 0; j < VEC; j += 4) {
            const float4 w4 = __ldg(reinterpret_cast<const float4 *>(w + k + j));
            const float4 b4 = __ldg(reinterpret_cast<const float4 *>(b + k + j));
            wk[j] = w4.x; wk[j + 1] = w4.y; wk[j + 2] = w4.z; wk[j + 3] = w4.w;
            bk[j] = b4.x; bk[j + 1] = b4.y; bk[j + 2] = b4.z; bk[j + 3] = b4.w;
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) f[j] = fmaf((f[j] - mu) * inv, wk[j], bk[j]);
        st_stream(out + i, pack<T>(f));
    }
}

template <typename T>
__global__ void gn_apply_kernel(const T *__restrict__ in, const float *__restrict__ mean,
                                const float *__restrict__ var, const float *__restrict__ w,
                                const float *__restrict__ b, unsigned long long group_size,
                                unsigned long long channel_size, float eps, T *__restrict__ out,
                                unsigned long long n, unsigned long long channels) {
    for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
         i < n; i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
        const unsigned long long g = i / group_size;
        const unsigned long long c = (i / channel_size) % channels;
        float t = to_float<T>(in[i]) - mean[g];
        t /= sqrtf(var[g] + eps);
        out[i] = from_float<T>(fmaf(t, w[c], b[c]));
    }
}

// layer_norm.cl:63-78 (eps as an argument instead of the file-scope constant at :58).
template <typename T>
__global__ void ln_apply_kernel(const T *__restrict__ in, const float *__restrict__ mean,
                                const float *__restrict__ var, const float *__restrict__ w,
                                const float *__restrict__ b, unsigned long long dim, float eps,
                                T *__restrict__ out, unsigned long long n) {
    for (unsigned long long i = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
         i < n; i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
        const unsigned long long k = i % dim;
        const unsigned long long r = i / dim;
        float t = to_float<T>(in[i]) - mean[r];
        t /= sqrtf(var[r] + eps);
        out[i] = from_float<T>(fmaf(t, w[k], b[k]));
    }
}

}  // namespace

cudaError_t gn_split_launch(const GnShape &s, const GnPlan &plan, const void *in, void *out, const float *w,
                            const float *b, void *workspace, cudaStream_t stream, const void *bias) {
    const int64_t esz = s.dtype == kF16 ? 2 : 4;
    const int64_t vec = 16 / esz;
    const int64_t cpg = s.channels / s.groups;
    const int64_t slab_elems = cpg * s.hw;
    const int64_t units = s.batch * s.groups;
    if (units == 0 || slab_elems == 0) return cudaSuccess;
    if (workspace == nullptr) return cudaErrorInvalidValue;
    SplitArgs a;
    a.in = in; a.out = out; a.w = w; a.b = b;
    a.partial = static_cast<float *>(workspace);
    a.bias = bias;
    a.channels = static_cast<uint32_t>(s.channels);
    a.slab_elems = static_cast<uint32_t>(slab_elems);
    a.splits = static_cast<uint32_t>(plan.splits);
    int64_t chunk = (slab_elems + plan.splits - 1) / plan.splits;
    chunk = ((chunk + vec - 1) / vec) * vec;
    a.chunk_elems = static_cast<uint32_t>(chunk);
    a.cpg = static_cast<uint32_t>(cpg);
    a.groups = static_cast<uint32_t>(s.groups);
    a.vec = aligned16(in) && aligned16(out) && slab_elems % vec == 0;
    a.vec_uniform = a.vec && s.hw % vec == 0;
    a.eps = s.eps;
    a.hw_div = FastDiv::make(static_cast<uint32_t>(s.hw));
    const unsigned grid = static_cast<unsigned>(units * plan.splits);
    if (plan.nhwc) {
        // statistics as usual, then the tiled apply that writes channels-last
        if (bias != nullptr || s.batch > 65535) return cudaErrorInvalidValue;
        const uintptr_t pa = esz == 2 ? 3 : 7;
        const bool pairs = s.hw % 2 == 0 && s.channels % 2 == 0 &&
                           (reinterpret_cast<uintptr_t>(in) & pa) == 0 && (reinterpret_cast<uintptr_t>(out) & pa) == 0;
        const int ts = pairs ? 64 : 32;
        const dim3 tgrid(static_cast<unsigned>((s.hw + ts - 1) / ts), static_cast<unsigned>((s.channels + ts - 1) / ts),
                         static_cast<unsigned>(s.batch));
        if (tgrid.y > 65535) return cudaErrorInvalidValue;
        const dim3 tblock(32, 8);
        const uint32_t hw32 = static_cast<uint32_t>(s.hw);
        const unsigned tiles_c = static_cast<unsigned>((s.channels + 63) / 64), tiles_p = static_cast<unsigned>((s.hw + 63) / 64);
        const unsigned long long total = static_cast<unsigned long long>(s.batch) * tiles_c * tiles_p;
        const size_t asmem = 2 * esz * 64 * (64 + (esz == 2 ? 2 : 1)) + 64 * sizeof(float4);
        const unsigned agrid = static_cast<unsigned>(total < static_cast<unsigned long long>(sm_count()) * 6 ? total : static_cast<unsigned long long>(sm_count()) * 6);
#define SDFL_NHWC_APPLY(T, ACT)                                                              \
        do {                                                                                 \
            if (pairs) gn_apply_nhwc_async_kernel<T, ACT><<<agrid, tblock, asmem, stream>>>(a, hw32, tiles_c, tiles_p, total); \
            else gn_apply_nhwc_kernel<T, ACT, false><<<tgrid, tblock, 0, stream>>>(a, hw32);        \
        } while (0)
        const bool wide = s.dtype == kF16 && s.hw % 8 == 0 && s.channels % 8 == 0 && aligned16(in) && aligned16(out);
        if (wide) {
            // tile shape as in the fp16 transpose: the long side along a dimension that is a multiple of 128
            gn_split_stats_kernel<__half><<<grid, kSplitThreads, 0, stream>>>(a);
            const bool p_wide = s.hw % 128 == 0 && (s.channels % 128 != 0 || s.hw >= s.channels);
            const bool c_wide = !p_wide && s.channels % 128 == 0;
            cudaError_t herr;
            if (s.act == kActSilu)
                herr = p_wide ? launch_nhwc_h8<kActSilu, 64, 128>(a, s, stream)
                       : c_wide ? launch_nhwc_h8<kActSilu, 128, 64>(a, s, stream)
                                : launch_nhwc_h8<kActSilu, 64, 64>(a, s, stream);
            else
                herr = p_wide ? launch_nhwc_h8<kActNone, 64, 128>(a, s, stream)
                       : c_wide ? launch_nhwc_h8<kActNone, 128, 64>(a, s, stream)
                                : launch_nhwc_h8<kActNone, 64, 64>(a, s, stream);
            if (herr == cudaSuccess) g_launches.fetch_add(2);
            return herr;
        }
        if (s.dtype == kF16) {
            gn_split_stats_kernel<__half><<<grid, kSplitThreads, 0, stream>>>(a);
            if (s.act == kActSilu) SDFL_NHWC_APPLY(__half, kActSilu); else SDFL_NHWC_APPLY(__half, kActNone);
        } else {
            gn_split_stats_kernel<float><<<grid, kSplitThreads, 0, stream>>>(a);
            if (s.act == kActSilu) SDFL_NHWC_APPLY(float, kActSilu); else SDFL_NHWC_APPLY(float, kActNone);
        }
#undef SDFL_NHWC_APPLY
        cudaError_t err = cudaGetLastError();
        if (err == cudaSuccess) g_launches.fetch_add(2);
        return err;
    }
    if (s.dtype == kF16) {
        gn_split_stats_kernel<__half><<<grid, kSplitThreads, 0, stream>>>(a);
        if (s.act == kActSilu) gn_split_apply_kernel<__half, kActSilu><<<grid, kSplitThreads, 0, stream>>>(a);
        else gn_split_apply_kernel<__half, kActNone><<<grid, kSplitThreads, 0, stream>>>(a);
    } else {
        gn_split_stats_kernel<float><<<grid, kSplitThreads, 0, stream>>>(a);
        if (s.act == kActSilu) gn_split_apply_kernel<float, kActSilu><<<grid, kSplitThreads, 0, stream>>>(a);
        else gn_split_apply_kernel<float, kActNone><<<grid, kSplitThreads, 0, stream>>>(a);
    }
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(2);
    return err;
}

// ---------------------------------------------------------------------------------------------
// Split path with its scratch inside the library image (no allocation anywhere)
// ---------------------------------------------------------------------------------------------
// Some callers cannot give the split path a workspace because they are not allowed to call an
// allocator at all: a host that pre-commits every byte of device memory to its own pools at
// start-up and treats any later cudaMalloc as a bug, a plugin loaded into such a host, or code
// on a latency-critical thread where an allocator's implicit device synchronisation is not
// acceptable.  For them the (mean, M2) pairs of the split path live in this fixed array, which
// every device that loads the library carries until the process exits.
//
// g_static_scratch names device memory only inside device code.  On the host the symbol is a
// stand-in; its device address has to be asked for (cudaGetSymbolAddress) with the right device
// current, once per device, and that address is what the kernels get.
static __device__ __align__(256) unsigned char g_static_scratch[kGnStaticScratchBytes];

cudaError_t gn_launch_static_scratch(const GnShape &s, const GnPlan &plan, const void *in, void *out,
                                     const float *w, const float *b, cudaStream_t stream) {
    static std::mutex mu;
    static void *address[kMaxDevices] = {};       // device address of g_static_scratch, per device
    if (plan.path != kGnSplit || plan.workspace > kGnStaticScratchBytes) return cudaErrorInvalidValue;
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    void *ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (address[dev] == nullptr) {
            // first call on this device: resolve the symbol while this device is current
            err = cudaGetSymbolAddress(&address[dev], g_static_scratch);
            if (err != cudaSuccess) { address[dev] = nullptr; return err; }
        }
        ptr = address[dev];
    }
    // Nothing in the scratch has to start at zero: the statistics kernel overwrites every
    // (mean, M2) pair the apply kernel reads, and the two run in stream order.
    return gn_launch(s, plan, in, out, w, b, ptr, stream, nullptr);
}

namespace {
// mean (mean == nullptr) or variance of `groups` runs of n elements.
template <typename T>
cudaError_t stats_launch(const void *in, const float *mean, float *out, int64_t groups, int64_t n,
                         cudaStream_t stream) {
    constexpr int VEC = VecOf<T>::N;
    cudaError_t err;
    if (gn_aligned16(in) && n % VEC == 0 && n >= VEC) {
        // cluster size: up to eight CTAs of 256 threads per SM, at least 8 vectors per thread
        int S = 1;
        while (S < 8 && groups * S * 2 <= 8 * sm_count() && n / VEC / (S * 2) >= 8 * kStatsThreads) S *= 2;
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        cluster_config(&cfg, attr, static_cast<unsigned>(groups * S), S, kStatsThreads, 0, stream);
        err = cudaLaunchKernelEx(&cfg, stats_vec_kernel<T>, static_cast<const uint4 *>(in), mean, out,
                                 static_cast<unsigned long long>(n / VEC));
    } else {
        stats_kernel<T><<<static_cast<unsigned>(groups), kStatsThreads, 0, stream>>>(
            static_cast<const T *>(in), mean, out, n);
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}
}  // namespace

cudaError_t stats_mean_launch(const void *in, float *out, int64_t groups, int64_t n, int dtype,
                              cudaStream_t stream) {
    if (groups == 0) return cudaSuccess;
    return dtype == kF16 ? stats_launch<__half>(in, nullptr, out, groups, n, stream)
                         : stats_launch<float>(in, nullptr, out, groups, n, stream);
}

cudaError_t stats_var_launch(const void *in, const float *mean, float *out, int64_t groups,
                             int64_t n, int dtype, cudaStream_t stream) {
    if (groups == 0) return cudaSuccess;
    return dtype == kF16 ? stats_launch<__half>(in, mean, out, groups, n, stream)
                         : stats_launch<float>(in, mean, out, groups, n, stream);
}

static unsigned flat_grid(int64_t n, int threads) {
    int64_t blocks = (n + threads - 1) / threads;
    const int64_t cap = sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<unsigned>(blocks);
}

cudaError_t gn_apply_launch(const void *in, const float *mean, const float *var, const float *w,
                            const float *b, int64_t group_size, int64_t channel_size, float eps,
                            void *out, int64_t n, int64_t channels, int dtype, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    const int64_t vec = dtype == kF16 ? 8 : 4;
    if (gn_aligned16(in) && gn_aligned16(out) && n % vec == 0 && group_size % vec == 0 &&
        channel_size % vec == 0 && n / vec < (1ll << 31) && channels < (1ll << 31)) {
        const uint32_t nvec = static_cast<uint32_t>(n / vec);
        const FastDiv gd = FastDiv::make(static_cast<uint32_t>(group_size / vec));
        const FastDiv cd = FastDiv::make(static_cast<uint32_t>(channel_size / vec));
        const FastDiv wd = FastDiv::make(static_cast<uint32_t>(channels));
        const unsigned vgrid = flat_grid(nvec, 256);
        if (dtype == kF16)
            gn_apply_vec_kernel<__half><<<vgrid, 256, 0, stream>>>(static_cast<const uint4 *>(in), mean, var, w, b, gd,
                                                                  cd, wd, eps, static_cast<uint4 *>(out), nvec);
        else
            gn_apply_vec_kernel<float><<<vgrid, 256, 0, stream>>>(static_cast<const uint4 *>(in), mean, var, w, b, gd,
                                                                 cd, wd, eps, static_cast<uint4 *>(out), nvec);
        cudaError_t verr = cudaGetLastError();
        if (verr == cudaSuccess) g_launches.fetch_add(1);
        return verr;
    }
    const unsigned grid = flat_grid(n, 256);
    if (dtype == kF16)
        gn_apply_kernel<__half><<<grid, 256, 0, stream>>>(
            static_cast<const __half *>(in), mean, var, w, b, group_size, channel_size, eps,
            static_cast<__half *>(out), n, channels);
    else
        gn_apply_kernel<float><<<grid, 256, 0, stream>>>(
            static_cast<const float *>(in), mean, var, w, b, group_size, channel_size, eps,
            static_cast<float *>(out), n, channels);
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

cudaError_t ln_apply_launch(const void *in, const float *mean, const float *var, const float *w,
                            const float *b, int64_t dim, float eps, void *out, int64_t n, int dtype,
                            cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    const int64_t vec = dtype == kF16 ? 8 : 4;
    if (gn_aligned16(in) && gn_aligned16(out) && gn_aligned16(w) && gn_aligned16(b) && n % vec == 0 &&
        dim % vec == 0 && n / vec < (1ll << 31)) {
        const uint32_t nvec = static_cast<uint32_t>(n / vec);
        const FastDiv rd = FastDiv::make(static_cast<uint32_t>(dim / vec));
        const unsigned vgrid = flat_grid(nvec, 256);
        if (dtype == kF16)
            ln_apply_vec_kernel<__half><<<vgrid, 256, 0, stream>>>(static_cast<const uint4 *>(in), mean, var, w, b, rd,
                                                                  eps, static_cast<uint4 *>(out), nvec);
        else
            ln_apply_vec_kernel<float><<<vgrid, 256, 0, stream>>>(static_cast<const uint4 *>(in), mean, var, w, b, rd,
                                                                 eps, static_cast<uint4 *>(out), nvec);
        cudaError_t verr = cudaGetLastError();
        if (verr == cudaSuccess) g_launches.fetch_add(1);
        return verr;
    }
    const unsigned grid = flat_grid(n, 256);
    if (dtype == kF16)
        ln_apply_kernel<__half><<<grid, 256, 0, stream>>>(
            static_cast<const __half *>(in), mean, var, w, b, dim, eps, static_cast<__half *>(out), n);
    else
        ln_apply_kernel<float><<<grid, 256, 0, stream>>>(
            static_cast<const float *>(in), mean, var, w, b, dim, eps, static_cast<float *>(out), n);
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

}  // namespace sdfl
