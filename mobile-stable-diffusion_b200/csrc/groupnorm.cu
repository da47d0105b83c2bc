// GroupNorm with optional fused SiLU for NCHW tensors, fp32 or fp16 I/O, fp32 arithmetic.
//
// Replaces the reference's four launches / six tensor passes (group_norm.cl:1-76 =
// local_reduction_mean, local_reduction_variance, group_norm; then util.cl:124-134 silu) by
// one launch with one HBM read and one HBM write.  Semantics kept from the reference: biased
// variance (group_norm.cl:53-55), y = fma((x - mean) / sqrt(var + eps), w[c], b[c])
// (group_norm.cl:73-75), silu(y) = y / (1 + exp(-y)) (util.cl:130-133).  Added over the
// reference: a batch dimension (slab = one (image, group) pair; weight index wraps per image)
// and fp16 storage.
//
// Resident path: the slab of one (image, group) is contiguous in NCHW (C/G * H*W elements).
// A thread-block cluster of 1..16 CTAs splits it; each CTA pulls its part into shared memory
// with cp.async.bulk (bulk-copy engine, mbarrier completion), sums chunks as they land,
// exchanges partial sums through distributed shared memory, takes the exact two-pass variance
// from the resident copy, then normalises from shared memory straight to global memory.
// Because nothing is written before the whole slab is resident, out == in is safe.
//
// Split path: any shape.  Kernel 1 writes one (mean, M2) pair per chunk to a scratch buffer
// (per-thread shifted sums merged pairwise with Chan's update through warp shuffles and a
// block merge); kernel 2 merges the chunk pairs of its slab in a fixed order and normalises.
#include "common.cuh"
#include "kernels.h"

#include <cooperative_groups.h>

#include <map>
#include <mutex>

namespace cg = cooperative_groups;

namespace sdfl {

namespace {

__device__ unsigned int g_gn_status;   // sticky; bit 0: a bounded mbarrier wait ran out

constexpr int kResidentThreads = 512;
constexpr int kMaxChunks = 16;
constexpr uint32_t kHeaderBytes = 512;             // mbarriers + reduction scratch + published sums
constexpr uint32_t kMaxPartBytes = 200 * 1024;     // per-CTA resident part (227 KB minus headroom)
constexpr long long kWaitCycles = 2000000000LL;    // ~1 s: far beyond any healthy bulk copy

// ---------------------------------------------------------------------------------------------
// mbarrier / bulk-copy primitives
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait for phase `parity` of `bar`, at most `limit` clock cycles.  Returns false on time-out;
// the caller records it and carries on (every CTA must still reach the cluster barriers).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > limit) return false;
    }
    return true;
}

// 1-D bulk copy global -> this CTA's shared memory; completion counted in bytes on `bar`.
// dst, src and bytes are multiples of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

struct ResidentArgs {
    const void *in;
    void *out;
    const float *w;
    const float *b;
    uint32_t slab_vecs;    // 16-byte vectors per slab
    uint32_t slab_elems;
    uint32_t cpg;          // channels per group
    uint32_t groups;
    uint32_t chunk_bytes;  // bulk-copy granule, multiple of 16
    uint32_t vec_uniform;  // hw % lanes-per-vector == 0
    float eps;
    FastDiv hw_div;
};

template <typename T, int ACT>
__global__ void __launch_bounds__(kResidentThreads)
gn_resident_kernel(const ResidentArgs a) {
    constexpr int VEC = VecOf<T>::N;
    constexpr bool HALF = sizeof(T) == 2;
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t csize = cluster.num_blocks();
    const uint32_t rank = cluster.block_rank();
    const uint32_t unit = blockIdx.x / csize;
    const uint32_t tid = threadIdx.x;

    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);           // [16]
    float *red = reinterpret_cast<float *>(smem + 128);            // [33]
    float *pub = reinterpret_cast<float *>(smem + 320);            // [2] read by cluster peers
    unsigned char *data = smem + kHeaderBytes;

    const uint32_t v0 = static_cast<uint32_t>((static_cast<uint64_t>(a.slab_vecs) * rank) / csize);
    const uint32_t v1 = static_cast<uint32_t>((static_cast<uint64_t>(a.slab_vecs) * (rank + 1)) / csize);
    const uint32_t nv = v1 - v0;
    const uint32_t part_bytes = nv * 16u;
    const size_t part_off = (static_cast<size_t>(unit) * a.slab_vecs + v0) * 16u;
    const unsigned char *gsrc = static_cast<const unsigned char *>(a.in) + part_off;
    unsigned char *gdst = static_cast<unsigned char *>(a.out) + part_off;
    const uint32_t nchunks = (part_bytes + a.chunk_bytes - 1) / a.chunk_bytes;   // <= kMaxChunks

    if (tid == 0) {
        for (uint32_t k = 0; k < nchunks; ++k) mbar_init(smem_addr(&bars[k]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0) {
        for (uint32_t k = 0; k < nchunks; ++k) {
            const uint32_t off = k * a.chunk_bytes;
            const uint32_t bytes = min(a.chunk_bytes, part_bytes - off);
            const uint32_t bar = smem_addr(&bars[k]);
            mbar_expect_tx(bar, bytes);
            bulk_load(smem_addr(data + off), gsrc + off, bytes, bar);
        }
    }

    // ---- pass 1: sum, chunk by chunk as the copies land --------------------------------------
    const uint4 *sv = reinterpret_cast<const uint4 *>(data);
    const uint32_t vpc = a.chunk_bytes / 16u;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    bool timed_out = false;
    for (uint32_t k = 0; k < nchunks; ++k) {
        if (!mbar_wait_bounded(smem_addr(&bars[k]), 0, timed_out ? 2000000LL : kWaitCycles))
            timed_out = true;
        const uint32_t hi = min(nv, (k + 1) * vpc);
        for (uint32_t i = k * vpc + tid; i < hi; i += kResidentThreads) {
            float f[VEC];
            unpack<T>(sv[i], f);
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[j & 3] += f[j];
        }
    }
    if (timed_out && tid == 0) atomicOr(&g_gn_status, 1u);

    float part = block_sum((acc[0] + acc[1]) + (acc[2] + acc[3]), red);
    if (tid == 0) pub[0] = part;
    cluster.sync();
    float total = 0.f;
    for (uint32_t r = 0; r < csize; ++r) total += *cluster.map_shared_rank(&pub[0], r);
    const float mean = total / static_cast<float>(a.slab_elems);

    // ---- pass 2: exact centred sum of squares from the resident copy -------------------------
    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
    for (uint32_t i = tid; i < nv; i += kResidentThreads) {
        float f[VEC];
        unpack<T>(sv[i], f);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const float d = f[j] - mean;
            acc[j & 3] = fmaf(d, d, acc[j & 3]);
        }
    }
    part = block_sum((acc[0] + acc[1]) + (acc[2] + acc[3]), red);
    if (tid == 0) pub[1] = part;
    cluster.sync();
    total = 0.f;
    for (uint32_t r = 0; r < csize; ++r) total += *cluster.map_shared_rank(&pub[1], r);
    cluster.barrier_arrive();     // peers may exit only after everyone has read their sums
    const float var = total / static_cast<float>(a.slab_elems);   // biased: group_norm.cl:53-55
    const float rstd = 1.0f / sqrtf(var + a.eps);

    // ---- pass 3: normalise + affine (+ activation) from shared memory to global --------------
    const uint32_t ch0 = (unit % a.groups) * a.cpg;
    uint4 *gv = reinterpret_cast<uint4 *>(gdst);
    for (uint32_t i = tid; i < nv; i += kResidentThreads) {
        float f[VEC];
        unpack<T>(sv[i], f);
        const uint32_t e = (v0 + i) * VEC;
        if (a.vec_uniform) {
            const uint32_t c = ch0 + a.hw_div.div(e);
            const float wv = __ldg(a.w + c), bv = __ldg(a.b + c);
            if (HALF) {
                const float sc = wv * rstd;
                const float sh = fmaf(-mean, sc, bv);
#pragma unroll
                for (int j = 0; j < VEC; ++j) f[j] = activate<ACT, HALF>(fmaf(f[j], sc, sh));
            } else {
#pragma unroll
                for (int j = 0; j < VEC; ++j)
                    f[j] = activate<ACT, HALF>(fmaf((f[j] - mean) * rstd, wv, bv));
            }
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
                const uint32_t c = ch0 + a.hw_div.div(e + j);
                f[j] = activate<ACT, HALF>(fmaf((f[j] - mean) * rstd, __ldg(a.w + c), __ldg(a.b + c)));
            }
        }
        st_stream(&gv[i], pack<T>(f));
    }
    cluster.barrier_wait();
}

// ---------------------------------------------------------------------------------------------
// Split path
// ---------------------------------------------------------------------------------------------
constexpr int kSplitThreads = 512;

struct Moments { float n, mean, m2; };

// Chan et al. pairwise update of (count, mean, sum of squared deviations).
__device__ __forceinline__ Moments merge(const Moments &x, const Moments &y) {
    if (y.n == 0.f) return x;
    if (x.n == 0.f) return y;
    Moments r;
    r.n = x.n + y.n;
    const float d = y.mean - x.mean;
    const float f = y.n / r.n;
    r.mean = fmaf(d, f, x.mean);
    r.m2 = x.m2 + y.m2 + d * d * x.n * f;
    return r;
}

__device__ __forceinline__ Moments warp_merge(Moments m) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Moments y;
        y.n = __shfl_down_sync(0xffffffffu, m.n, o);
        y.mean = __shfl_down_sync(0xffffffffu, m.mean, o);
        y.m2 = __shfl_down_sync(0xffffffffu, m.m2, o);
        m = merge(m, y);
    }
    return m;   // valid in lane 0
}

struct SplitArgs {
    const void *in;
    void *out;
    const float *w;
    const float *b;
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

// Shifted single-pass moments of a thread's elements: d = x - first, sum d and d*d.
struct Shifted {
    float k, s, q, n;
    __device__ __forceinline__ void add(float x) {
        if (n == 0.f) k = x;
        const float d = x - k;
        s += d;
        q = fmaf(d, d, q);
        n += 1.f;
    }
    __device__ __forceinline__ Moments done() const {
        Moments m;
        m.n = n;
        m.mean = n > 0.f ? k + s / n : 0.f;
        m.m2 = n > 0.f ? fmaxf(q - s * s / n, 0.f) : 0.f;
        return m;
    }
};

template <typename T>
__global__ void __launch_bounds__(kSplitThreads) gn_split_stats_kernel(const SplitArgs a) {
    constexpr int VEC = VecOf<T>::N;
    __shared__ Moments warp_m[kSplitThreads / 32];
    const uint32_t unit = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
    const uint32_t e0 = split * a.chunk_elems;
    const uint32_t e1 = min(a.slab_elems, e0 + a.chunk_elems);
    const T *x = static_cast<const T *>(a.in) + static_cast<size_t>(unit) * a.slab_elems;
    Shifted sh{0.f, 0.f, 0.f, 0.f};
    if (a.vec) {
        const uint4 *xv = reinterpret_cast<const uint4 *>(x);
        for (uint32_t i = e0 / VEC + threadIdx.x; i < e1 / VEC; i += kSplitThreads) {
            float f[VEC];
            unpack<T>(__ldg(xv + i), f);
#pragma unroll
            for (int j = 0; j < VEC; ++j) sh.add(f[j]);
        }
    } else {
        for (uint32_t i = e0 + threadIdx.x; i < e1; i += kSplitThreads) sh.add(to_float<T>(x[i]));
    }
    Moments m = warp_merge(sh.done());
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
    if (a.vec) {
        const uint4 *xv = reinterpret_cast<const uint4 *>(x);
        uint4 *yv = reinterpret_cast<uint4 *>(y);
        for (uint32_t i = e0 / VEC + threadIdx.x; i < e1 / VEC; i += kSplitThreads) {
            float f[VEC];
            unpack<T>(ld_stream(xv + i), f);
            if (a.vec_uniform) {
                const uint32_t c = ch0 + a.hw_div.div(i * VEC);
                const float wv = __ldg(a.w + c), bv = __ldg(a.b + c);
#pragma unroll
                for (int j = 0; j < VEC; ++j)
                    f[j] = activate<ACT, HALF>(fmaf((f[j] - mean) * rstd, wv, bv));
            } else {
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    const uint32_t c = ch0 + a.hw_div.div(i * VEC + j);
                    f[j] = activate<ACT, HALF>(
                        fmaf((f[j] - mean) * rstd, __ldg(a.w + c), __ldg(a.b + c)));
                }
            }
            st_stream(yv + i, pack<T>(f));
        }
    } else {
        for (uint32_t i = e0 + threadIdx.x; i < e1; i += kSplitThreads) {
            const uint32_t c = ch0 + a.hw_div.div(i);
            const float v = fmaf((to_float<T>(x[i]) - mean) * rstd, __ldg(a.w + c), __ldg(a.b + c));
            y[i] = from_float<T>(activate<ACT, HALF>(v));
        }
    }
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

// group_norm.cl:59-76 with the weight index wrapped per image: c = (i / channelSize) % C.
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

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int pow2_at_least(double x) {
    int c = 1;
    while (c < x) c <<= 1;
    return c;
}

// Per-device, per-kernel-instance one-time attribute set-up (maximum dynamic shared memory and
// the opt-in for 16-CTA clusters), so that launches themselves make no attribute calls.
constexpr int kMaxDevices = 64;

template <typename T, int ACT>
cudaError_t ensure_resident_attrs() {
    static std::atomic<bool> done[kMaxDevices];
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < kMaxDevices && done[dev].load(std::memory_order_acquire)) return cudaSuccess;
    auto kernel = gn_resident_kernel<T, ACT>;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kHeaderBytes + kMaxPartBytes));
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < kMaxDevices) done[dev].store(true, std::memory_order_release);
    return cudaSuccess;
}

inline void cluster_config(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attr, unsigned grid,
                           int cluster, size_t smem, cudaStream_t stream) {
    *cfg = cudaLaunchConfig_t{};
    cfg->gridDim = dim3(grid);
    cfg->blockDim = dim3(kResidentThreads);
    cfg->dynamicSmemBytes = smem;
    cfg->stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg->attrs = attr;
    cfg->numAttrs = 1;
}

template <typename T, int ACT>
cudaError_t launch_resident(const ResidentArgs &a, int64_t units, const GnPlan &plan,
                            cudaStream_t stream) {
    cudaError_t err = ensure_resident_attrs<T, ACT>();
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cluster_config(&cfg, attr, static_cast<unsigned>(units * plan.cluster), plan.cluster, plan.smem,
                   stream);
    err = cudaLaunchKernelEx(&cfg, gn_resident_kernel<T, ACT>, a);
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

// Can at least one cluster of this size and shared-memory footprint be resident (a 16-CTA
// cluster needs a GPC with 16 free SMs)?  Asked of the driver once per (device, dtype,
// cluster, shared-memory size in KiB) and remembered.
template <typename T>
cudaError_t resident_clusters_fit(const GnPlan &plan, int *fits) {
    static std::mutex mu;
    static std::map<uint64_t, int> cache;
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    const uint64_t key = (static_cast<uint64_t>(dev) << 40) | (static_cast<uint64_t>(sizeof(T)) << 32) |
                         (static_cast<uint64_t>(plan.cluster) << 24) | ((plan.smem + 1023) / 1024);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *fits = it->second; return cudaSuccess; }
    }
    err = ensure_resident_attrs<T, kActSilu>();
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cluster_config(&cfg, attr, static_cast<unsigned>(plan.cluster), plan.cluster,
                   ((plan.smem + 1023) / 1024) * 1024, nullptr);
    int n = 0;
    err = cudaOccupancyMaxActiveClusters(&n, gn_resident_kernel<T, kActSilu>, &cfg);
    if (err != cudaSuccess) return err;
    *fits = n;
    std::lock_guard<std::mutex> lock(mu);
    cache[key] = n;
    return cudaSuccess;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Planning
// ---------------------------------------------------------------------------------------------
cudaError_t gn_make_plan(const GnShape &s, const void *in, const void *out, int force_path,
                         int force_cluster, GnPlan *plan) {
    const int64_t esz = s.dtype == kF16 ? 2 : 4;
    const int64_t vec = 16 / esz;
    const int64_t cpg = s.channels / s.groups;
    const int64_t slab_elems = cpg * s.hw;
    const int64_t slab_bytes = slab_elems * esz;
    const int64_t units = s.batch * s.groups;
    *plan = GnPlan{};
    plan->threads = kResidentThreads;

    bool resident_ok = aligned16(in) && aligned16(out) && slab_bytes % 16 == 0 && slab_bytes >= 16 &&
                       slab_bytes <= 16 * static_cast<int64_t>(kMaxPartBytes) &&
                       units * 16 < (1ll << 31);
    if (force_path == kGnSplit) resident_ok = false;

    if (resident_ok) {
        const double sb = static_cast<double>(slab_bytes);
        int c_min = pow2_at_least(sb / kMaxPartBytes);             // must fit
        int c_occ = pow2_at_least(sb / (72.0 * 1024.0));           // three CTAs per SM
        int c_fill = pow2_at_least(296.0 / static_cast<double>(units));   // two waves of 148 SMs
        int c_cap = 1;                                              // parts of at least 8 KB
        while (c_cap < 16 && sb / (2.0 * c_cap) >= 8192.0) c_cap <<= 1;
        int c = c_occ > c_fill ? c_occ : c_fill;
        if (c > c_cap) c = c_cap;
        if (c > 8 && c_min <= 8) c = 8;      // keep to portable cluster sizes unless forced by size
        if (c < c_min) c = c_min;
        if (c > 16) c = 16;
        if (force_cluster > 0) c = force_cluster;
        const int64_t slab_vecs = slab_bytes / 16;
        if (c > slab_vecs) c = 1;
        const int64_t max_part = ((slab_vecs + c - 1) / c) * 16;
        if (max_part <= kMaxPartBytes && c >= 1 && c <= 16 && (c & (c - 1)) == 0) {
            plan->path = kGnResident;
            plan->cluster = c;
            plan->smem = kHeaderBytes + static_cast<size_t>(max_part);
            int fits = 0;
            cudaError_t err = s.dtype == kF16 ? resident_clusters_fit<__half>(*plan, &fits)
                                              : resident_clusters_fit<float>(*plan, &fits);
            if (err != cudaSuccess) { (void)cudaGetLastError(); fits = 0; }
            if (fits > 0) return cudaSuccess;
        }
        if (force_path == kGnResident) return cudaErrorInvalidConfiguration;
    } else if (force_path == kGnResident) {
        return cudaErrorInvalidConfiguration;
    }

    // split path
    if (slab_elems >= (1ll << 31)) return cudaErrorInvalidValue;
    plan->path = kGnSplit;
    plan->cluster = 1;
    plan->smem = 0;
    plan->threads = kSplitThreads;
    // enough chunks for ~4 CTAs per SM across all slabs, at least 16K elements per chunk.
    int64_t splits = (148 * 4 + units - 1) / units;
    const int64_t max_splits = (slab_elems + 16383) / 16384;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > 1024) splits = 1024;
    if (force_cluster > 0) splits = force_cluster;
    int64_t chunk = (slab_elems + splits - 1) / splits;
    chunk = ((chunk + vec - 1) / vec) * vec;
    splits = (slab_elems + chunk - 1) / chunk;
    plan->splits = static_cast<int>(splits);
    plan->workspace = static_cast<size_t>(units * splits * 2) * sizeof(float);
    return cudaSuccess;
}

cudaError_t gn_launch(const GnShape &s, const GnPlan &plan, const void *in, void *out,
                      const float *w, const float *b, void *workspace, cudaStream_t stream) {
    const int64_t esz = s.dtype == kF16 ? 2 : 4;
    const int64_t vec = 16 / esz;
    const int64_t cpg = s.channels / s.groups;
    const int64_t slab_elems = cpg * s.hw;
    const int64_t units = s.batch * s.groups;
    if (units == 0 || slab_elems == 0) return cudaSuccess;

    if (plan.path == kGnResident) {
        ResidentArgs a;
        a.in = in; a.out = out; a.w = w; a.b = b;
        a.slab_vecs = static_cast<uint32_t>(slab_elems * esz / 16);
        a.slab_elems = static_cast<uint32_t>(slab_elems);
        a.cpg = static_cast<uint32_t>(cpg);
        a.groups = static_cast<uint32_t>(s.groups);
        const uint32_t max_part = static_cast<uint32_t>(plan.smem - kHeaderBytes);
        uint32_t chunk = 16 * 1024;
        while ((max_part + chunk - 1) / chunk > kMaxChunks) chunk *= 2;
        a.chunk_bytes = chunk;
        a.vec_uniform = s.hw % vec == 0;
        a.eps = s.eps;
        a.hw_div = FastDiv::make(static_cast<uint32_t>(s.hw));
        if (s.dtype == kF16)
            return s.act == kActSilu ? launch_resident<__half, kActSilu>(a, units, plan, stream)
                                     : launch_resident<__half, kActNone>(a, units, plan, stream);
        return s.act == kActSilu ? launch_resident<float, kActSilu>(a, units, plan, stream)
                                 : launch_resident<float, kActNone>(a, units, plan, stream);
    }

    if (workspace == nullptr) return cudaErrorInvalidValue;
    SplitArgs a;
    a.in = in; a.out = out; a.w = w; a.b = b;
    a.partial = static_cast<float *>(workspace);
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

cudaError_t gn_read_status(unsigned int *value, bool clear, cudaStream_t stream) {
    cudaError_t err = cudaMemcpyFromSymbolAsync(value, g_gn_status, sizeof(unsigned int), 0,
                                                cudaMemcpyDeviceToHost, stream);
    if (err != cudaSuccess) return err;
    err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) return err;
    if (clear && *value != 0) {
        const unsigned int zero = 0;
        err = cudaMemcpyToSymbolAsync(g_gn_status, &zero, sizeof(unsigned int), 0,
                                      cudaMemcpyHostToDevice, stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    }
    return err;
}

cudaError_t stats_mean_launch(const void *in, float *out, int64_t groups, int64_t n, int dtype,
                              cudaStream_t stream) {
    if (groups == 0) return cudaSuccess;
    if (dtype == kF16)
        stats_kernel<__half><<<static_cast<unsigned>(groups), kStatsThreads, 0, stream>>>(
            static_cast<const __half *>(in), nullptr, out, n);
    else
        stats_kernel<float><<<static_cast<unsigned>(groups), kStatsThreads, 0, stream>>>(
            static_cast<const float *>(in), nullptr, out, n);
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

cudaError_t stats_var_launch(const void *in, const float *mean, float *out, int64_t groups,
                             int64_t n, int dtype, cudaStream_t stream) {
    if (groups == 0) return cudaSuccess;
    if (dtype == kF16)
        stats_kernel<__half><<<static_cast<unsigned>(groups), kStatsThreads, 0, stream>>>(
            static_cast<const __half *>(in), mean, out, n);
    else
        stats_kernel<float><<<static_cast<unsigned>(groups), kStatsThreads, 0, stream>>>(
            static_cast<const float *>(in), mean, out, n);
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

static unsigned flat_grid(int64_t n, int threads) {
    int64_t blocks = (n + threads - 1) / threads;
    const int64_t cap = 148 * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<unsigned>(blocks);
}

cudaError_t gn_apply_launch(const void *in, const float *mean, const float *var, const float *w,
                            const float *b, int64_t group_size, int64_t channel_size, float eps,
                            void *out, int64_t n, int64_t channels, int dtype, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
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
