// Device-side building blocks shared by the GroupNorm kernels: mbarrier / bulk-copy / cluster
// exchange primitives, (n, mean, M2) moments with Chan's merge, and the per-vector statistics and
// normalise arithmetic.  Everything here has internal linkage (one copy per translation unit).
#pragma once

#include "common.cuh"
#include "gn_internal.h"

#include <cooperative_groups.h>

#include <atomic>
#include <map>
#include <mutex>

namespace cg = cooperative_groups;

namespace sdfl {

namespace {

constexpr int kMaxSlots = kGnMaxSlots;
constexpr uint32_t kHeaderBytes = kGnHeaderBytes;
constexpr uint32_t kMaxPartBytes = kGnMaxPartBytes;
constexpr long long kWaitCycles = 2000000000LL;    // ~1 s: far beyond any healthy bulk copy
constexpr long long kWaitCyclesAfterTimeout = 2000000LL;

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

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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

__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}

// Wait for phase `parity` of `bar`, at most about `limit` clock cycles.  The hardware parks the
// warp inside try_wait (suspend-time hint), so a waiting warp takes almost no issue slots from
// the warps that have work; the clock is only looked at every few wake-ups.  Returns false on
// time-out; the caller records it and carries on (every thread must still reach the cluster
// barriers).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 8; ++i)
            if (mbar_try_wait_hint(bar, parity, 4000u)) return true;
        if (clock64() - t0 > limit) return false;
    }
}

// 1-D bulk copy global -> this CTA's shared memory; completion counted in bytes on `bar`.
// dst, src and bytes are multiples of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// Same with an L2 eviction-priority hint: evict_last for data that will be read again soon
// (the first read of the re-read mode), evict_first for data that is dead after this read.
__device__ __forceinline__ void bulk_load_hint(uint32_t dst, const void *src, uint32_t bytes,
                                               uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// ---- cluster exchange primitives: write into a peer CTA's shared memory and signal its mbarrier
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void st_peer_f32x2(uint32_t peer_addr, float a, float b) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(peer_addr), "f"(a), "f"(b) : "memory");
}

// Release at cluster scope: the stores above are visible to whoever acquires this arrival.
__device__ __forceinline__ void mbar_arrive_peer(uint32_t peer_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(peer_bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}

// Bounded wait on a barrier that PEER CTAs arrive on (acquire at cluster scope).
__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint32_t bar, uint32_t parity, long long limit) {
    if (mbar_try_wait_cluster(bar, parity, 0u)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 8; ++i)
            if (mbar_try_wait_cluster(bar, parity, 4000u)) return true;
        if (clock64() - t0 > limit) return false;
    }
}

// Barrier among the consumer warps only (the producer warp never joins it).
__device__ __forceinline__ void consumer_sync(uint32_t consumers) {
    asm volatile("bar.sync 1, %0;" ::"r"(consumers) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Moments: (count, mean, sum of squared deviations) with Chan et al.'s pairwise update
// ---------------------------------------------------------------------------------------------
struct Moments { float n, mean, m2; };

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

// ---------------------------------------------------------------------------------------------
// Per-vector work of the resident kernel
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// s += x - shift, q += (x - shift)^2 over the lanes of one 16-byte vector.
template <typename T>
__device__ __forceinline__ void stats_vec(const uint4 &v, float shift, float (&s)[2], float (&q)[2]);

template <>
__device__ __forceinline__ void stats_vec<float>(const uint4 &v, float shift, float (&s)[2], float (&q)[2]) {
    const float d0 = __uint_as_float(v.x) - shift, d1 = __uint_as_float(v.y) - shift;
    const float d2 = __uint_as_float(v.z) - shift, d3 = __uint_as_float(v.w) - shift;
    s[0] += d0; s[1] += d1; s[0] += d2; s[1] += d3;
    q[0] = fmaf(d0, d0, q[0]); q[1] = fmaf(d1, d1, q[1]);
    q[0] = fmaf(d2, d2, q[0]); q[1] = fmaf(d3, d3, q[1]);
}

// fp16 lanes: the mixed-precision subtract (f16 operand, f32 result) widens and shifts in one
// instruction, so a lane costs three instructions instead of four.
__device__ __forceinline__ void stats_half2(uint32_t packed, float shift, float (&s)[2], float (&q)[2]) {
    asm("{\n"
        " .reg .b16 lo, hi;\n"
        " .reg .f32 d0, d1;\n"
        " mov.b32 {lo, hi}, %4;\n"
        " sub.rn.f32.f16 d0, lo, %5;\n"
        " sub.rn.f32.f16 d1, hi, %5;\n"
        " add.rn.f32 %0, %0, d0;\n"
        " add.rn.f32 %1, %1, d1;\n"
        " fma.rn.f32 %2, d0, d0, %2;\n"
        " fma.rn.f32 %3, d1, d1, %3;\n"
        "}\n"
        : "+f"(s[0]), "+f"(s[1]), "+f"(q[0]), "+f"(q[1])
        : "r"(packed), "f"(shift));
}

template <>
__device__ __forceinline__ void stats_vec<__half>(const uint4 &v, float shift, float (&s)[2], float (&q)[2]) {
    stats_half2(v.x, shift, s, q);
    stats_half2(v.y, shift, s, q);
    stats_half2(v.z, shift, s, q);
    stats_half2(v.w, shift, s, q);
}

// Per-channel constants of the normalise pass.
//   fp32 storage: the reference's operation order, y = fma((x - mean) * rstd, w, b).
//   fp16 storage: folded, y = fma(x, sc, sh) with sc = w * rstd, sh = b - mean * sc; with SiLU
//   the fold goes one step further to h = y / 2, because silu(y) = h + h * tanh(h) needs one
//   SFU operation where y / (1 + exp(-y)) needs two.  tanh.approx on h keeps the fp16 result
//   within a quarter of the 2e-3 tolerance over the whole range (the error is dominated by
//   the final fp16 rounding).
template <typename T> struct Affine { float p0, p1, p2, p3; };

template <typename T, int ACT>
__device__ __forceinline__ Affine<T> make_affine(float mean, float rstd, float w, float b) {
    Affine<T> a;
    if (sizeof(T) == 2) {
        const float sc = w * rstd;
        const float sh = fmaf(-mean, sc, b);
        const float half = ACT == kActSilu ? 0.5f : 1.0f;
        a.p0 = sc * half; a.p1 = sh * half; a.p2 = 0.f; a.p3 = 0.f;
    } else {
        a.p0 = mean; a.p1 = rstd; a.p2 = w; a.p3 = b;
    }
    return a;
}

template <typename T, int ACT>
__device__ __forceinline__ uint4 norm_vec(const uint4 &v, const Affine<T> &a) {
    constexpr int VEC = VecOf<T>::N;
    float f[VEC];
    unpack<T>(v, f);
    if (sizeof(T) == 2) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const float h = fmaf(f[j], a.p0, a.p1);
            f[j] = ACT == kActSilu ? fmaf(h, tanh_approx(h), h) : h;
        }
    } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j)
            f[j] = activate<ACT, false>(fmaf((f[j] - a.p0) * a.p1, a.p2, a.p3));
    }
    return pack<T>(f);
}

inline bool aligned16(const void *p) { return gn_aligned16(p); }

constexpr int kMaxDevices = 64;

inline void cluster_config(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attr, unsigned grid,
                           int cluster, int threads, size_t smem, cudaStream_t stream) {
    *cfg = cudaLaunchConfig_t{};
    cfg->gridDim = dim3(grid);
    cfg->blockDim = dim3(static_cast<unsigned>(threads));
    cfg->dynamicSmemBytes = smem;
    cfg->stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg->attrs = attr;
    cfg->numAttrs = 1;
}

}  // namespace

}  // namespace sdfl
