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
// Cluster path (gn_resident_kernel).  The slab of one (image, group) is contiguous in NCHW
// (C/G * H*W elements).  A persistent thread-block cluster of 1..16 CTAs walks over slabs; each
// CTA owns a fixed share of every slab and moves it through a small shared-memory ring of
// chunk slots:
//   producer warp : cp.async.bulk (bulk-copy engine) global -> shared, one "full" mbarrier per
//                   slot; a slot is refilled as soon as the consumer warps have released it
//                   ("empty" mbarrier), also across slab boundaries, so loads never drain.
//   consumer warps: (1) as chunks land, one pass of shifted sums -> per-thread (n, mean, M2),
//                   merged with Chan's update through warp shuffles, a block merge, and a
//                   cluster merge over distributed shared memory; (2) normalise + affine
//                   (+ SiLU) from shared memory straight to global, 16-byte streaming stores.
// If a CTA's share fits the ring it stays resident between (1) and (2).  Otherwise -- the
// normal case for large slabs, and the faster one on B200 because several CTAs then share an
// SM -- the chunks are loaded a second time for (2): the first load carries an L2 evict_last
// hint, the clusters in flight hold a few tens of MB, and the second load is served by L2
// (measured: DRAM reads = 1.00-1.07x the tensor).  HBM therefore sees one read and one write.
// Every output chunk is written only after the whole slab has been read for (1) and the chunk
// itself has been read again for (2), so out == in is safe.
//
// Split path: any shape.  Kernel 1 writes one (mean, M2) pair per chunk to a scratch buffer;
// kernel 2 merges the chunk pairs of its slab in a fixed order and normalises.
#include "common.cuh"
#include "kernels.h"

#include <cooperative_groups.h>

#include <map>
#include <mutex>

namespace cg = cooperative_groups;

namespace sdfl {

namespace {

__device__ unsigned int g_gn_status;   // sticky; bit 0: a bounded mbarrier wait ran out

constexpr int kMaxSlots = 16;
constexpr uint32_t kHeaderBytes = 1024;            // mbarriers, merge scratch, published moments
constexpr uint32_t kMaxPartBytes = 226 * 1024;     // per-CTA resident part (227 KB less the header)
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

struct ResidentArgs {
    const void *in;
    void *out;
    const float *w;
    const float *b;
    uint32_t units;        // slabs = batch * groups
    uint32_t slab_vecs;    // 16-byte vectors per slab
    uint32_t slab_elems;
    uint32_t cpg;          // channels per group
    uint32_t groups;
    uint32_t chunk_vecs;   // vectors per ring chunk
    uint32_t nslots;       // chunk slots in the shared-memory ring
    uint32_t hold;         // chunks kept in their slots between the two passes (re-read mode)
    uint32_t vec_uniform;  // hw % lanes-per-vector == 0
    uint32_t hw_vecs;      // hw / lanes-per-vector (when vec_uniform)
    uint32_t channels;     // C (row length of `bias`)
    const void *bias;      // [batch, C] addend of the storage type, or nullptr
    // Input given as two tensors concatenated along the channels (in: [B, c1, hw], in2: [B, C - c1, hw]):
    // the skip-connection concat in front of a ResBlock's first norm (UNetModel.cpp:1960-1990).
    const void *in2;       // nullptr: `in` is the whole [B, C, hw] tensor
    uint32_t c1;
    float eps;
    FastDiv hw_div;        // element offset -> channel
    FastDiv hwv_div;       // vector offset -> channel (when vec_uniform)
};

// blockDim.x = consumer threads (a multiple of 32, at most 480) + one producer warp; at least
// two CTAs per SM, i.e. up to 64 registers per thread.
// BIAS: a per-(image, channel) addend is applied before the statistics (the reference's
// chunkwise_add in front of the out-norm of a ResBlock, ResBlock.cpp:188-231).  x + e only
// moves the shift of the shifted sums and the mean of the normalise pass, so it costs no
// instruction per element.
//
// Shared memory is a ring of `nslots` chunk slots.  The producer numbers its chunk loads
// n = 0, 1, 2, ... across slabs; load n goes to slot n % nslots and completes phase
// (n / nslots) & 1 of that slot's "full" barrier; it may start once the consumers have released
// the slot's previous occupant (phase ((n / nslots) - 1) & 1 of the "empty" barrier).
//   resident  (a part has at most nslots chunks): a slab's chunks are loaded once, read for the
//             moments, read again for the normalise pass, then released; free slots are filled
//             with the next slab's chunks meanwhile.
//   otherwise the chunks are released after the moments pass and loaded a second time for the
//             normalise pass (this second read is served by L2 when the clusters' slabs fit it).
//
// NV > 0: the launch has exactly 256 consumer threads and chunks of 256 * NV vectors, so a full
// chunk that lies inside one channel is NV vectors per thread at compile-time offsets: the
// loads are issued together and the loop, index and channel arithmetic disappear (they were
// about 40 % of the instructions issued, and the consumer warps are issue-bound).
template <typename T, int ACT, bool BIAS, int NV>
__global__ void __launch_bounds__(NV == 4 ? 288 : 512, NV == 4 ? 4 : 2)
gn_resident_kernel(const ResidentArgs a) {
    constexpr int VEC = VecOf<T>::N;
    constexpr bool HALF = sizeof(T) == 2;
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t csize = cluster.num_blocks();
    const uint32_t rank = cluster.block_rank();
    const uint32_t cluster_id = blockIdx.x / csize;
    const uint32_t nclusters = gridDim.x / csize;
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    const uint32_t consumers = blockDim.x - 32u;
    const uint32_t cwarps = consumers >> 5;

    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);                  // [kMaxSlots]
    uint64_t *empty = reinterpret_cast<uint64_t *>(smem + 128);           // [kMaxSlots]
    Moments *warp_m = reinterpret_cast<Moments *>(smem + 256);            // [31]
    uint64_t *stat_bar = reinterpret_cast<uint64_t *>(smem + 640);        // [2] peers arrive here
    float *peer_stats = reinterpret_cast<float *>(smem + 704);            // [2][16][2] written by peers
    unsigned char *data = smem + kHeaderBytes;

    // This CTA's share of every slab: vectors [v0, v0 + nv), cut into P chunks that move through
    // a ring of S slots.  Loads are numbered 0, 1, 2, ... over the whole kernel ("positions");
    // position p uses slot p % S, phase (p / S) & 1 of that slot's barriers.  Per slab:
    //   positions p0 .. p0+P-1        first read of chunks 0 .. P-1        (moments pass)
    //   positions p0+P .. p0+2P-H-1   second read of chunks 0 .. P-H-1     (normalise pass)
    // The last H = min(S-1, P) chunks of the first read are not released after the moments
    // pass: they are still in their slots when the normalise pass starts, which therefore
    // begins without waiting and reads P-H instead of P chunks again.  P <= S means H = P:
    // the share is resident and nothing is read twice.
    const uint32_t v0 = static_cast<uint32_t>((static_cast<uint64_t>(a.slab_vecs) * rank) / csize);
    const uint32_t v1 = static_cast<uint32_t>((static_cast<uint64_t>(a.slab_vecs) * (rank + 1)) / csize);
    const uint32_t nv = v1 - v0;
    const uint32_t cv = a.chunk_vecs;
    const uint32_t P = (nv + cv - 1) / cv;
    const uint32_t S = a.nslots;
    const uint32_t H = P <= S ? P : min(a.hold, S - 1u);
    const uint32_t loads_per_slab = 2u * P - H;
    const uint32_t chunk_bytes = cv * 16u;

    if (warp == cwarps) {
        // ---------------- producer warp ----------------------------------------------------------
        bool timed_out = false;
        const uint64_t keep = policy_evict_last(), drop = policy_evict_first();
        uint32_t unit = cluster_id, l = 0, slot = 0, round = 0;
        // Issue the next load of the sequence; false when all slabs are done.
        auto issue_next = [&]() -> bool {
            if (unit >= a.units) return false;
            const uint32_t j = l < P ? l : l - P;
            if (round > 0) {       // the slot's previous occupant must have been released
                if (!mbar_wait_bounded(smem_addr(&empty[slot]), (round - 1) & 1u,
                                       timed_out ? kWaitCyclesAfterTimeout : kWaitCycles))
                    timed_out = true;
            }
            const uint32_t lo = j * cv;
            const uint32_t bytes = (min(nv, lo + cv) - lo) * 16u;
            const uint32_t bar = smem_addr(&full[slot]);
            const uint64_t policy = (l < P && j + H < P) ? keep : drop;
            mbar_expect_tx(bar, bytes);
            // a chunk that will be read a second time should stay in L2; a last read need not
            if (a.in2 == nullptr) {
                const unsigned char *gsrc = static_cast<const unsigned char *>(a.in) +
                                            (static_cast<size_t>(unit) * a.slab_vecs + v0) * 16u;
                bulk_load_hint(smem_addr(data + slot * chunk_bytes), gsrc + lo * 16u, bytes, bar, policy);
            } else {
                // the slab's first k1 channels come from `in`, the rest from `in2`: the chunk
                // [b0, b1) of the slab (in bytes) is one or two bulk copies
                const uint32_t n = unit / a.groups, c_first = (unit % a.groups) * a.cpg;
                const uint32_t k1 = c_first >= a.c1 ? 0u : min(a.cpg, a.c1 - c_first);
                const size_t row = static_cast<size_t>(a.hw_vecs) * 16u;            // bytes of one channel
                const size_t split = k1 * row;
                const size_t b0 = (static_cast<size_t>(v0) + lo) * 16u, b1 = b0 + bytes;
                const unsigned char *s1 = static_cast<const unsigned char *>(a.in) +
                                          (static_cast<size_t>(n) * a.c1 + c_first) * row;
                const unsigned char *s2 = static_cast<const unsigned char *>(a.in2) +
                                          (static_cast<size_t>(n) * (a.channels - a.c1) + (max(c_first, a.c1) - a.c1)) * row;
                const uint32_t dst = smem_addr(data + slot * chunk_bytes);
                if (b0 < split) {
                    const uint32_t part = static_cast<uint32_t>(min(b1, split) - b0);
                    bulk_load_hint(dst, s1 + b0, part, bar, policy);
                    if (b1 > split) bulk_load_hint(dst + part, s2, static_cast<uint32_t>(b1 - split), bar, policy);
                } else {
                    bulk_load_hint(dst, s2 + (b0 - split), bytes, bar, policy);
                }
            }
            if (++slot == S) { slot = 0; ++round; }
            if (++l == loads_per_slab) { l = 0; unit += nclusters; }
            return true;
        };
        if (lane == 0) {
            for (uint32_t k = 0; k < S; ++k) {
                mbar_init(smem_addr(&full[k]), 1);
                mbar_init(smem_addr(&empty[k]), cwarps);
            }
            mbar_init(smem_addr(&stat_bar[0]), csize);
            mbar_init(smem_addr(&stat_bar[1]), csize);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // inits before the copy engine's arrivals
            // The first S loads need no release: start them before the barrier below, so the
            // first HBM round trip overlaps the cluster's start-up.
            for (uint32_t k = 0; k < S; ++k)
                if (!issue_next()) break;
        }
        __syncwarp();
        cluster.sync();            // see the consumers' side
        if (lane == 0) {
            while (issue_next()) {}
            if (timed_out) atomicOr(&g_gn_status, 1u);
        }
        return;
    }

    // ---------------- consumer warps -------------------------------------------------------------
    const uint32_t hwv = a.hw_vecs;          // vectors per channel (valid when vec_uniform)
    {
        // warm L2 with the first slab's scale and shift while the first chunks are in flight
        const uint32_t g0 = (cluster_id % a.groups) * a.cpg;
        const uint32_t c_lo = a.hw_div.div(v0 * VEC), c_hi = a.hw_div.div((v0 + nv) * VEC - 1u);
        for (uint32_t c = c_lo + tid; c <= c_hi && c < a.cpg; c += consumers) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(a.w + g0 + c));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(a.b + g0 + c));
        }
    }
    // Peers signal this CTA's stat barriers and the consumers use the barriers the producer
    // initialised: one full cluster barrier, the only one of the kernel.
    cluster.sync();

    bool timed_out = false;
    uint32_t pos = 0, it = 0;                // position of the slab's first load
    for (uint32_t unit = cluster_id; unit < a.units; unit += nclusters, ++it) {
        const uint32_t par = it & 1u;
        const uint32_t p0 = pos;
        // this slab's addends: bias[image, group's first channel ...]
        const T *erow = BIAS ? static_cast<const T *>(a.bias) +
                                   static_cast<size_t>(unit / a.groups) * a.channels + (unit % a.groups) * a.cpg
                             : nullptr;

        // pass 1: shifted sums, chunk by chunk as the copies land
        float s[2] = {0.f, 0.f}, q[2] = {0.f, 0.f};
        float shift = 0.f;
        uint32_t nvec_mine = 0;
        for (uint32_t j = 0; j < P; ++j) {
            const uint32_t p = p0 + j, slot = p % S, round = p / S;
            if (!mbar_wait_bounded(smem_addr(&full[slot]), round & 1u,
                                   timed_out ? kWaitCyclesAfterTimeout : kWaitCycles))
                timed_out = true;
            const uint4 *sv = reinterpret_cast<const uint4 *>(data + slot * chunk_bytes);
            if (j == 0) shift = to_float<T>(reinterpret_cast<const T *>(sv)[0]);
            const uint32_t cnt = min(cv, nv - j * cv);
            bool fast = false;
            if (NV > 0 && cnt == 256u * NV && consumers == 256u) {
                uint32_t c = 0;
                if (BIAS) {
                    c = a.hwv_div.div(v0 + j * cv);
                    fast = a.vec_uniform && c == a.hwv_div.div(v0 + j * cv + cnt - 1u);
                } else {
                    fast = true;
                }
                if (fast) {
                    float sh = shift;
                    if (BIAS) {
                        const float e = to_float<T>(erow[c]);
                        if (j == 0) shift += e;
                        sh = shift - e;
                    }
                    uint4 v[NV > 0 ? NV : 1];
#pragma unroll
                    for (int k = 0; k < NV; ++k) v[k] = sv[tid + k * 256];
#pragma unroll
                    for (int k = 0; k < NV; ++k) stats_vec<T>(v[k], sh, s, q);
                    nvec_mine += NV;
                }
            }
            if (fast) {
            } else if (!BIAS) {
#pragma unroll 2
                for (uint32_t i = tid; i < cnt; i += consumers) {
                    stats_vec<T>(sv[i], shift, s, q);
                    ++nvec_mine;
                }
            } else if (a.vec_uniform && hwv >= consumers) {
                // (x + e_c) - shift = x - (shift - e_c): walk channel by channel
                const uint32_t lo = j * cv, hi = lo + cnt;
                uint32_t i0 = lo;
                while (i0 < hi) {
                    const uint32_t c = a.hwv_div.div(v0 + i0);
                    const uint32_t seg_end = min(hi, (c + 1) * hwv - v0);
                    const float e = to_float<T>(erow[c]);
                    if (j == 0 && i0 == lo) shift += e;          // shift = first value of x + e
                    const float sh = shift - e;
#pragma unroll 2
                    for (uint32_t i = i0 + tid; i < seg_end; i += consumers) {
                        stats_vec<T>(sv[i - lo], sh, s, q);
                        ++nvec_mine;
                    }
                    i0 = seg_end;
                }
            } else {
                const uint32_t lo = j * cv;
                for (uint32_t i = tid; i < cnt; i += consumers) {
                    float f[VEC];
                    unpack<T>(sv[i], f);
                    const uint32_t e0 = (v0 + lo + i) * VEC;
                    float sl[2] = {0.f, 0.f}, ql[2] = {0.f, 0.f};
#pragma unroll
                    for (int l = 0; l < VEC; ++l) {
                        const float d = f[l] + to_float<T>(erow[a.hw_div.div(e0 + l)]) - shift;
                        sl[l & 1] += d;
                        ql[l & 1] = fmaf(d, d, ql[l & 1]);
                    }
                    s[0] += sl[0]; s[1] += sl[1]; q[0] += ql[0]; q[1] += ql[1];
                    ++nvec_mine;
                }
            }
            if (j + H < P) {       // not one of the chunks held for pass 2
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_addr(&empty[slot]));
            }
        }
        Moments m;
        {
            const float cnt = static_cast<float>(nvec_mine * VEC);
            const float ss = s[0] + s[1], qq = q[0] + q[1];
            m.n = cnt;
            m.mean = nvec_mine ? shift + ss / cnt : 0.f;
            m.m2 = nvec_mine ? fmaxf(qq - ss * ss / cnt, 0.f) : 0.f;
        }
        m = warp_merge(m);
        if (lane == 0) warp_m[warp] = m;
        consumer_sync(consumers);
        if (warp == 0) {
            // This CTA's moments -> slot [par][rank] of every CTA of the cluster (itself
            // included), one lane per destination, then one arrival on that CTA's barrier.
            Moments t = lane < cwarps ? warp_m[lane] : Moments{0.f, 0.f, 0.f};
            t = warp_merge(t);
            const float cta_mean = __shfl_sync(0xffffffffu, t.mean, 0);
            const float cta_m2 = __shfl_sync(0xffffffffu, t.m2, 0);
            if (lane < csize) {
                st_peer_f32x2(map_to_rank(smem_addr(&peer_stats[(par * 16u + rank) * 2u]), lane),
                              cta_mean, cta_m2);
                mbar_arrive_peer(map_to_rank(smem_addr(&stat_bar[par]), lane));
            }
        }
        // All csize CTAs have written their pair once the barrier's phase completes.  Every
        // warp folds the pairs itself (same order everywhere -> same bits everywhere).
        if (!mbar_wait_cluster_bounded(smem_addr(&stat_bar[par]), (it >> 1) & 1u,
                                       timed_out ? kWaitCyclesAfterTimeout : kWaitCycles))
            timed_out = true;
        float mean, rstd;
        {
            Moments t{0.f, 0.f, 0.f};
            if (lane < csize) {
                const uint32_t q0 = static_cast<uint32_t>((static_cast<uint64_t>(a.slab_vecs) * lane) / csize);
                const uint32_t q1 = static_cast<uint32_t>((static_cast<uint64_t>(a.slab_vecs) * (lane + 1)) / csize);
                t.n = static_cast<float>(q1 - q0) * VEC;
                t.mean = peer_stats[(par * 16u + lane) * 2u];
                t.m2 = peer_stats[(par * 16u + lane) * 2u + 1u];
            }
            t = warp_merge(t);
            const float var = __shfl_sync(0xffffffffu, t.m2, 0) / static_cast<float>(a.slab_elems);   // biased: group_norm.cl:53-55
            mean = __shfl_sync(0xffffffffu, t.mean, 0);
            rstd = 1.0f / sqrtf(var + a.eps);
        }

        // pass 2: normalise + affine (+ activation) from shared memory to global; each slot is
        // handed back to the producer as soon as this warp is done with it.  Held chunks
        // (P-H .. P-1, already in their slots) first, then chunks 0 .. P-H-1 as they come back.
        const uint32_t ch0 = (unit % a.groups) * a.cpg;
        uint4 *gv = reinterpret_cast<uint4 *>(static_cast<unsigned char *>(a.out) +
                                              (static_cast<size_t>(unit) * a.slab_vecs + v0) * 16u);
        for (uint32_t k = 0; k < P; ++k) {
            const bool held = k < H;
            const uint32_t j = held ? P - H + k : k - H;          // chunk of the share
            const uint32_t p = held ? p0 + j : p0 + P + j;        // its position in the ring
            const uint32_t slot = p % S, round = p / S;
            if (!held) {
                if (!mbar_wait_bounded(smem_addr(&full[slot]), round & 1u,
                                       timed_out ? kWaitCyclesAfterTimeout : kWaitCycles))
                    timed_out = true;
            }
            const uint4 *sv = reinterpret_cast<const uint4 *>(data + slot * chunk_bytes);
            const uint32_t lo = j * cv;                 // part-relative vector index of the chunk
            const uint32_t hi = min(nv, lo + cv);
            bool fast = false;
            if (NV > 0 && hi - lo == 256u * NV && consumers == 256u && a.vec_uniform) {
                const uint32_t c = a.hwv_div.div(v0 + lo);
                if (c == a.hwv_div.div(v0 + hi - 1u)) {
                    fast = true;
                    const float mc = BIAS ? mean - to_float<T>(erow[c]) : mean;
                    const Affine<T> af = make_affine<T, ACT>(mc, rstd, __ldg(a.w + ch0 + c),
                                                            __ldg(a.b + ch0 + c));
                    uint4 v[NV > 0 ? NV : 1];
#pragma unroll
                    for (int k = 0; k < NV; ++k) v[k] = sv[tid + k * 256];
#pragma unroll
                    for (int k = 0; k < NV; ++k)
                        st_stream(&gv[lo + tid + k * 256], norm_vec<T, ACT>(v[k], af));
                }
            }
            if (fast) {
            } else if (a.vec_uniform && hwv >= consumers) {
                // long channels: walk channel by channel, weights hoisted out of the vector loop
                uint32_t i0 = lo;
                while (i0 < hi) {
                    const uint32_t c = a.hwv_div.div(v0 + i0);
                    const uint32_t seg_end = min(hi, (c + 1) * hwv - v0);
                    const float mc = BIAS ? mean - to_float<T>(erow[c]) : mean;
                    const Affine<T> af = make_affine<T, ACT>(mc, rstd, __ldg(a.w + ch0 + c),
                                                            __ldg(a.b + ch0 + c));
#pragma unroll 2
                    for (uint32_t i = i0 + tid; i < seg_end; i += consumers)
                        st_stream(&gv[i], norm_vec<T, ACT>(sv[i - lo], af));
                    i0 = seg_end;
                }
            } else if (a.vec_uniform) {
                for (uint32_t i = lo + tid; i < hi; i += consumers) {
                    const uint32_t cl = a.hwv_div.div(v0 + i), c = ch0 + cl;
                    const float mc = BIAS ? mean - to_float<T>(erow[cl]) : mean;
                    const Affine<T> af = make_affine<T, ACT>(mc, rstd, __ldg(a.w + c), __ldg(a.b + c));
                    st_stream(&gv[i], norm_vec<T, ACT>(sv[i - lo], af));
                }
            } else {
                for (uint32_t i = lo + tid; i < hi; i += consumers) {
                    float f[VEC];
                    unpack<T>(sv[i - lo], f);
                    const uint32_t e = (v0 + i) * VEC;
#pragma unroll
                    for (int l = 0; l < VEC; ++l) {
                        const uint32_t cl = a.hw_div.div(e + l), c = ch0 + cl;
                        const float mc = BIAS ? mean - to_float<T>(erow[cl]) : mean;
                        f[l] = activate<ACT, HALF>(
                            fmaf((f[l] - mc) * rstd, __ldg(a.w + c), __ldg(a.b + c)));
                    }
                    st_stream(&gv[i], pack<T>(f));
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_addr(&empty[slot]));
        }
        pos = p0 + loads_per_slab;
    }
    if (timed_out && lane == 0) atomicOr(&g_gn_status, 1u);
    // No barrier at exit: nobody reads a peer's shared memory; a CTA's own slots are written
    // only by peers whose arrivals it has already waited for.
}

// ---------------------------------------------------------------------------------------------
// Register path: one CTA per slab, the whole slab in the CTA's registers
// ---------------------------------------------------------------------------------------------
// For the slabs of the UNet (5-240 KB) the cluster kernel's fixed costs (cluster start-up, barrier
// set-up, the exchange) are most of its time.  Here a CTA of 512 threads loads its slab with up to
// NVT 16-byte vectors per thread, all loads in flight at once, folds the moments through one
// __syncthreads and normalises from registers: one HBM read, one write, no shared-memory staging.
// Every load of a slab precedes every store to it, so out == in is safe.
constexpr int kRegThreads = 512;
constexpr int kRegMaxVecs = 24;      // per thread: slabs up to 512 * 24 * 16 B = 192 KB

struct RegArgs {
    const void *in;
    void *out;
    const float *w;
    const float *b;
    const void *bias;      // [batch, C] addend of the storage type, or nullptr
    uint32_t units, slab_vecs, slab_elems, cpg, groups, channels;
    uint32_t vec_uniform;  // hw % lanes-per-vector == 0
    float eps;
    FastDiv hw_div;        // element offset in the slab -> channel of the group
    FastDiv hwv_div;       // vector offset -> channel (when vec_uniform)
    // channels-last output (NHWC template flag)
    uint32_t hw, hw_vecs;
    uint32_t row_bytes;    // shared-memory stride of one channel's pixels: hw * sizeof(T) rounded up to 4, plus 4
    uint32_t pair;         // fp16 and an even number of channels per group: two channels per store
    FastDiv out_div;       // output index within the slab -> pixel (divides by cpg, or cpg / 2 when pair)
    // input as two tensors concatenated along the channels (see ResidentArgs); needs vec_uniform
    const void *in2;
    uint32_t c1;
};

// NHWC: the result is written channels-last, out[n][p][c] (the permute3D__0_2_1 that follows the
// norm of a SpatialTransformer block, SpatialTransformer.cpp:127-140, fused into the store).  The
// normalised slab [cpg][hw] goes through shared memory with a 4-byte skew per channel row and
// leaves as runs of cpg consecutive channels per pixel.
template <typename T, int ACT, bool BIAS, int NVT, bool NHWC>
__global__ void __launch_bounds__(kRegThreads, NVT <= 4 ? 2 : 1)
gn_register_kernel(const RegArgs a) {
    constexpr int VEC = VecOf<T>::N;
    constexpr bool HALF = sizeof(T) == 2;
    __shared__ Moments warp_m[kRegThreads / 32];
    extern __shared__ __align__(16) unsigned char tsm[];      // NHWC only: cpg rows of row_bytes
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    for (uint32_t unit = blockIdx.x; unit < a.units; unit += gridDim.x) {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.in) + static_cast<size_t>(unit) * a.slab_vecs;
        uint4 *dst = reinterpret_cast<uint4 *>(a.out) + static_cast<size_t>(unit) * a.slab_vecs;
        const T *erow = BIAS ? static_cast<const T *>(a.bias) +
                                   static_cast<size_t>(unit / a.groups) * a.channels + (unit % a.groups) * a.cpg
                             : nullptr;
        // two-source input: vectors [0, split) of the slab come from `in`, the rest from `in2`
        const uint4 *src2 = src;
        uint32_t split = 0xffffffffu;
        if (a.in2 != nullptr) {
            const uint32_t n = unit / a.groups, c_first = (unit % a.groups) * a.cpg;
            const uint32_t k1 = c_first >= a.c1 ? 0u : min(a.cpg, a.c1 - c_first);
            split = k1 * a.hw_vecs;
            src = reinterpret_cast<const uint4 *>(a.in) + (static_cast<size_t>(n) * a.c1 + c_first) * a.hw_vecs;
            src2 = reinterpret_cast<const uint4 *>(a.in2) +
                   (static_cast<size_t>(n) * (a.channels - a.c1) + (max(c_first, a.c1) - a.c1)) * a.hw_vecs - split;
        }
        uint4 v[NVT];
#pragma unroll
        for (int k = 0; k < NVT; ++k) {
            const uint32_t idx = tid + k * kRegThreads;
            if (idx < a.slab_vecs) v[k] = ld_stream((idx < split ? src : src2) + idx);
        }
        // this thread's moments, shifted by its first value
        float s[2] = {0.f, 0.f}, q[2] = {0.f, 0.f};
        float shift = 0.f;
        uint32_t mine = 0;
        if (tid < a.slab_vecs) {
            shift = HALF ? __half2float(__ushort_as_half(static_cast<unsigned short>(v[0].x & 0xffffu)))
                         : __uint_as_float(v[0].x);
            if (BIAS) shift += to_float<T>(erow[a.hw_div.div(tid * VEC)]);
        }
#pragma unroll
        for (int k = 0; k < NVT; ++k) {
            const uint32_t idx = tid + k * kRegThreads;
            if (idx < a.slab_vecs) {
                if (!BIAS) {
                    stats_vec<T>(v[k], shift, s, q);
                } else if (a.vec_uniform) {
                    stats_vec<T>(v[k], shift - to_float<T>(erow[a.hwv_div.div(idx)]), s, q);
                } else {
                    float f[VEC];
                    unpack<T>(v[k], f);
#pragma unroll
                    for (int l = 0; l < VEC; ++l) {
                        const float d = f[l] + to_float<T>(erow[a.hw_div.div(idx * VEC + l)]) - shift;
                        s[l & 1] += d;
                        q[l & 1] = fmaf(d, d, q[l & 1]);
                    }
                }
                ++mine;
            }
        }
        Moments m;
        {
            const float cnt = static_cast<float>(mine * VEC);
            const float ss = s[0] + s[1], qq = q[0] + q[1];
            m.n = cnt;
            m.mean = mine ? shift + ss / cnt : 0.f;
            m.m2 = mine ? fmaxf(qq - ss * ss / cnt, 0.f) : 0.f;
        }
        m = warp_merge(m);
        if (lane == 0) warp_m[warp] = m;
        __syncthreads();
        // every warp folds the 16 per-warp moments itself, in the same order
        Moments t = lane < kRegThreads / 32 ? warp_m[lane] : Moments{0.f, 0.f, 0.f};
        t = warp_merge(t);
        const float mean = __shfl_sync(0xffffffffu, t.mean, 0);
        const float var = __shfl_sync(0xffffffffu, t.m2, 0) / static_cast<float>(a.slab_elems);   // biased
        const float rstd = 1.0f / sqrtf(var + a.eps);
        const uint32_t ch0 = (unit % a.groups) * a.cpg;
#pragma unroll
        for (int k = 0; k < NVT; ++k) {
            const uint32_t idx = tid + k * kRegThreads;
            if (idx < a.slab_vecs) {
                if (a.vec_uniform) {
                    const uint32_t cl = a.hwv_div.div(idx), c = ch0 + cl;
                    const float mc = BIAS ? mean - to_float<T>(erow[cl]) : mean;
                    const Affine<T> af = make_affine<T, ACT>(mc, rstd, __ldg(a.w + c), __ldg(a.b + c));
                    const uint4 r = norm_vec<T, ACT>(v[k], af);
                    if (NHWC) {
                        const uint32_t p0 = (idx - cl * a.hw_vecs) * VEC;
                        uint32_t *d = reinterpret_cast<uint32_t *>(tsm + cl * a.row_bytes + p0 * sizeof(T));
                        d[0] = r.x; d[1] = r.y; d[2] = r.z; d[3] = r.w;
                    } else {
                        st_stream(dst + idx, r);
                    }
                } else {
                    float f[VEC];
                    unpack<T>(v[k], f);
#pragma unroll
                    for (int l = 0; l < VEC; ++l) {
                        const uint32_t cl = a.hw_div.div(idx * VEC + l), c = ch0 + cl;
                        const float mc = BIAS ? mean - to_float<T>(erow[cl]) : mean;
                        f[l] = activate<ACT, HALF>(fmaf((f[l] - mc) * rstd, __ldg(a.w + c), __ldg(a.b + c)));
                        if (NHWC) {
                            const uint32_t p = idx * VEC + l - cl * a.hw;
                            *reinterpret_cast<T *>(tsm + cl * a.row_bytes + p * sizeof(T)) = from_float<T>(f[l]);
                        }
                    }
                    if (!NHWC) st_stream(dst + idx, pack<T>(f));
                }
            }
        }
        __syncthreads();       // warp_m is reused by the next slab; NHWC: the slab is in shared memory
        if (NHWC) {
            // out[n][p][ch0 + c]: consecutive threads take consecutive channels of a pixel
            T *outp = static_cast<T *>(a.out) + static_cast<size_t>(unit / a.groups) * a.hw * a.channels + ch0;
            if (HALF && a.pair) {
                const uint32_t hp = a.cpg >> 1, total = a.hw * hp;
                for (uint32_t o = tid; o < total; o += kRegThreads) {
                    const uint32_t p = a.out_div.div(o), c = 2u * (o - p * hp);
                    const unsigned short lo = *reinterpret_cast<const unsigned short *>(tsm + c * a.row_bytes + p * 2u);
                    const unsigned short hi = *reinterpret_cast<const unsigned short *>(tsm + (c + 1u) * a.row_bytes + p * 2u);
                    *reinterpret_cast<uint32_t *>(outp + static_cast<size_t>(p) * a.channels + c) =
                        static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
                }
            } else {
                const uint32_t total = a.hw * a.cpg;
                for (uint32_t o = tid; o < total; o += kRegThreads) {
                    const uint32_t p = a.out_div.div(o), c = o - p * a.cpg;
                    outp[static_cast<size_t>(p) * a.channels + c] =
                        *reinterpret_cast<const T *>(tsm + c * a.row_bytes + p * sizeof(T));
                }
            }
            __syncthreads();   // the next slab overwrites the staging rows
        }
    }
}

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
    if (a.vec) {
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
    const T *erow = a.bias ? static_cast<const T *>(a.bias) +
                                 static_cast<size_t>(unit / a.groups) * a.channels + ch0
                           : nullptr;
    if (a.vec) {
        const uint4 *xv = reinterpret_cast<const uint4 *>(x);
        uint4 *yv = reinterpret_cast<uint4 *>(y);
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

// Per-device, per-kernel-instance one-time attribute set-up (maximum dynamic shared memory and
// the opt-in for 16-CTA clusters), so that launches themselves make no attribute calls.
constexpr int kMaxDevices = 64;

template <typename T, int ACT, bool BIAS, int NV>
cudaError_t ensure_resident_attrs() {
    static std::atomic<bool> done[kMaxDevices];
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < kMaxDevices && done[dev].load(std::memory_order_acquire)) return cudaSuccess;
    auto kernel = gn_resident_kernel<T, ACT, BIAS, NV>;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kHeaderBytes + kMaxPartBytes));
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < kMaxDevices) done[dev].store(true, std::memory_order_release);
    return cudaSuccess;
}

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

template <typename T, int ACT, bool BIAS, int NV>
cudaError_t launch_resident_nv(const ResidentArgs &a, const GnPlan &plan, cudaStream_t stream) {
    cudaError_t err = ensure_resident_attrs<T, ACT, BIAS, NV>();
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cluster_config(&cfg, attr, static_cast<unsigned>(plan.nclusters * plan.cluster), plan.cluster,
                   plan.threads, plan.smem, stream);
    err = cudaLaunchKernelEx(&cfg, gn_resident_kernel<T, ACT, BIAS, NV>, a);
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

// The unrolled variants need 256 consumer threads and chunks of 256 * NV vectors.
inline int plan_unroll(int threads, int chunk_vecs) {
    if (threads != 288) return 0;
    return chunk_vecs == 2048 ? 8 : chunk_vecs == 1024 ? 4 : 0;
}

template <typename T, int ACT, bool BIAS>
cudaError_t launch_resident_as(const ResidentArgs &a, const GnPlan &plan, cudaStream_t stream) {
    switch (plan_unroll(plan.threads, plan.chunk_vecs)) {
        case 8: return launch_resident_nv<T, ACT, BIAS, 8>(a, plan, stream);
        case 4: return launch_resident_nv<T, ACT, BIAS, 4>(a, plan, stream);
        default: return launch_resident_nv<T, ACT, BIAS, 0>(a, plan, stream);
    }
}

template <typename T, int ACT>
cudaError_t launch_resident(const ResidentArgs &a, const GnPlan &plan, cudaStream_t stream) {
    return a.bias ? launch_resident_as<T, ACT, true>(a, plan, stream)
                  : launch_resident_as<T, ACT, false>(a, plan, stream);
}

constexpr size_t kRegMaxStageBytes = 200 * 1024;   // shared-memory staging of the channels-last store

template <typename T, int ACT, int NVT>
cudaError_t launch_register_nhwc(const RegArgs &a, unsigned grid, size_t smem, cudaStream_t stream) {
    static std::atomic<bool> done[kMaxDevices];
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (!(dev >= 0 && dev < kMaxDevices && done[dev].load(std::memory_order_acquire))) {
        err = cudaFuncSetAttribute(gn_register_kernel<T, ACT, false, NVT, true>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kRegMaxStageBytes));
        if (err != cudaSuccess) return err;
        if (dev >= 0 && dev < kMaxDevices) done[dev].store(true, std::memory_order_release);
    }
    gn_register_kernel<T, ACT, false, NVT, true><<<grid, kRegThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

template <typename T, int ACT, bool BIAS>
cudaError_t launch_register_as(const RegArgs &a, bool nhwc, cudaStream_t stream) {
    const uint32_t per_thread = (a.slab_vecs + kRegThreads - 1) / kRegThreads;
    const unsigned grid = a.units < 148u * 64u ? a.units : 148u * 64u;
    cudaError_t err;
    if (nhwc) {
        if (BIAS) return cudaErrorInvalidValue;
        const size_t smem = static_cast<size_t>(a.cpg) * a.row_bytes;
        err = per_thread <= 4    ? launch_register_nhwc<T, ACT, 4>(a, grid, smem, stream)
              : per_thread <= 12 ? launch_register_nhwc<T, ACT, 12>(a, grid, smem, stream)
                                 : launch_register_nhwc<T, ACT, kRegMaxVecs>(a, grid, smem, stream);
    } else {
        if (per_thread <= 4)
            gn_register_kernel<T, ACT, BIAS, 4, false><<<grid, kRegThreads, 0, stream>>>(a);
        else if (per_thread <= 12)
            gn_register_kernel<T, ACT, BIAS, 12, false><<<grid, kRegThreads, 0, stream>>>(a);
        else
            gn_register_kernel<T, ACT, BIAS, kRegMaxVecs, false><<<grid, kRegThreads, 0, stream>>>(a);
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

template <typename T, int ACT>
cudaError_t launch_register(const RegArgs &a, bool nhwc, cudaStream_t stream) {
    return a.bias ? launch_register_as<T, ACT, true>(a, nhwc, stream)
                  : launch_register_as<T, ACT, false>(a, nhwc, stream);
}

// How many clusters of this size, block size and shared-memory footprint can be resident at
// once (a cluster must fit inside one GPC).  Asked of the driver once per (device, dtype,
// cluster, threads, shared-memory size in KiB) and remembered.
template <typename T, int NV>
cudaError_t active_clusters_nv(cudaLaunchConfig_t *cfg, int *n) {
    cudaError_t err = ensure_resident_attrs<T, kActSilu, false, NV>();
    if (err != cudaSuccess) return err;
    return cudaOccupancyMaxActiveClusters(n, gn_resident_kernel<T, kActSilu, false, NV>, cfg);
}

template <typename T>
cudaError_t resident_active_clusters(int cluster, int threads, size_t smem, int chunk_vecs, int *active) {
    static std::mutex mu;
    static std::map<uint64_t, int> cache;
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    const uint64_t kb = (smem + 1023) / 1024;
    const uint64_t key = (static_cast<uint64_t>(dev) << 48) | (static_cast<uint64_t>(sizeof(T)) << 40) |
                         (static_cast<uint64_t>(cluster) << 32) |
                         (static_cast<uint64_t>(threads) << 16) | kb |
                         (static_cast<uint64_t>(plan_unroll(threads, chunk_vecs)) << 56);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *active = it->second; return cudaSuccess; }
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cluster_config(&cfg, attr, static_cast<unsigned>(cluster), cluster, threads, smem, nullptr);
    int n = 0;
    switch (plan_unroll(threads, chunk_vecs)) {
        case 8: err = active_clusters_nv<T, 8>(&cfg, &n); break;
        case 4: err = active_clusters_nv<T, 4>(&cfg, &n); break;
        default: err = active_clusters_nv<T, 0>(&cfg, &n); break;
    }
    if (err != cudaSuccess) return err;
    *active = n;
    std::lock_guard<std::mutex> lock(mu);
    cache[key] = n;
    return cudaSuccess;
}

constexpr int kSmCount = 148;

// When the register path beats the cluster path (launches timed back to back on B200, fp16 and
// fp32, 32-256 slabs of 5-240 KB): always for slabs up to 48 KB (3.5-6 us against 5.5-7); for
// larger ones once there are at least 64 slabs, i.e. enough CTAs to pull on HBM from many SMs
// (with 32 slabs of 60-160 KB a cluster of 8 per slab is 0.3-1 us faster).
inline bool prefer_register(int64_t slab_bytes, int64_t units) {
    return slab_bytes <= 48 * 1024 || units >= 64;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Planning
// ---------------------------------------------------------------------------------------------
// Slabs up to this size take the one-kernel channels-last path (statistics, normalise and the
// transposing store by the one CTA that holds the slab); beyond it the CTA's scattered
// cpg-element runs cost more than a second kernel: statistics, then a tiled apply over all SMs.
constexpr int64_t kNhwcFusedMaxSlabBytes = 48 * 1024;

// Shared-memory row stride of the channels-last store: a channel's pixels, 4-byte aligned, plus a
// 4-byte skew so that consecutive channels start in consecutive banks.
int64_t gn_nhwc_row_bytes(const GnShape &s) {
    const int64_t esz = s.dtype == kF16 ? 2 : 4;
    return ((s.hw * esz + 3) / 4) * 4 + 4;
}

bool gn_nhwc_fused_ok(const GnShape &s, const void *in, const void *out) {
    const int64_t esz = s.dtype == kF16 ? 2 : 4;
    if (s.groups <= 0 || s.channels % s.groups != 0) return false;
    const int64_t cpg = s.channels / s.groups;
    const int64_t slab_bytes = cpg * s.hw * esz;
    return aligned16(in) && aligned16(out) && slab_bytes % 16 == 0 && slab_bytes >= 16 &&
           slab_bytes <= kNhwcFusedMaxSlabBytes &&
           cpg * gn_nhwc_row_bytes(s) <= static_cast<int64_t>(kRegMaxStageBytes) &&
           s.batch * s.groups < (1ll << 27) && s.hw * cpg < (1ll << 31);
}

cudaError_t gn_make_plan(const GnShape &s, const void *in, const void *out, int force_path,
                         int force_cluster, GnPlan *plan) {
    const int64_t esz = s.dtype == kF16 ? 2 : 4;
    const int64_t vec = 16 / esz;
    const int64_t cpg = s.channels / s.groups;
    const int64_t slab_elems = cpg * s.hw;
    const int64_t slab_bytes = slab_elems * esz;
    const int64_t units = s.batch * s.groups;
    *plan = GnPlan{};

    bool resident_ok = aligned16(in) && aligned16(out) && slab_bytes % 16 == 0 && slab_bytes >= 16 &&
                       units < (1ll << 27);
    if (force_path == kGnSplit) resident_ok = false;

    // One CTA per slab with the slab in registers: no start-up or exchange latency.
    const bool register_ok = resident_ok && slab_bytes <= static_cast<int64_t>(kRegThreads) * kRegMaxVecs * 16;
    if (force_path == kGnRegister && !register_ok) return cudaErrorInvalidConfiguration;
    if (register_ok && (force_path == kGnRegister || (force_path == kGnAuto && prefer_register(slab_bytes, units)))) {
        plan->path = kGnRegister;
        plan->cluster = 1;
        plan->threads = kRegThreads;
        plan->nclusters = static_cast<int>(units < 148 * 64 ? units : 148 * 64);
        plan->chunk_vecs = static_cast<int>((slab_bytes / 16 + kRegThreads - 1) / kRegThreads);
        return cudaSuccess;
    }

    if (resident_ok) {
        // Ring geometry and cluster size, from sweeps on B200 (fp16 and fp32 behave alike per
        // byte).  A small ring (3 slots of 16-32 KB, 8 consumer warps) with the second read
        // served by L2 beats full shared-memory residency at every size tried: it keeps 2-4 CTAs
        // on each SM, so one CTA's cluster exchange hides behind the others' traffic.  The
        // cluster grows with the slab so that a CTA's share is about 256 KB: the slabs in flight
        // (256 CTAs x share = 64 MB) stay well inside L2; with few slabs it grows further so that
        // every SM still gets a CTA.
        const int64_t slab_vecs = slab_bytes / 16;
        const int k_cluster = force_cluster & 0xff, k_slots = (force_cluster >> 8) & 0xff;
        const int k_chunk_kb = (force_cluster >> 16) & 0xff, k_cwarps = (force_cluster >> 24) & 0xf;
        int c = slab_bytes <= 640 * 1024 ? 2 : slab_bytes <= 1280 * 1024 ? 4 : 8;
        // Few slabs: grow the cluster while the grid stays within 256 CTAs (more CTAs than that
        // only add start-up cost); not beyond 8, only about half as many 16-CTA clusters can
        // be co-resident.
        while (c < 8 && units * c * 2 <= 256 && slab_bytes / (2 * c) >= 8 * 1024) c *= 2;
        while (c > 1 && slab_bytes / c < 8 * 1024) c /= 2;
        if (k_cluster > 0) c = k_cluster;
        if (c > 16) c = 16;
        if (c > slab_vecs) c = 1;
        for (; c >= 1; c = (k_cluster > 0 ? 0 : c / 2)) {
            const int64_t part_vecs = (slab_vecs + c - 1) / c;
            const int64_t part_bytes = part_vecs * 16;
            // One slab per cluster at most (a single wave, e.g. one image per GPU): the launch is
            // a fill / exchange / drain latency chain, where fewer, larger chunks and more
            // consumer warps won in the sweeps, and shares up to 96 KB stay resident.
            const bool single_wave = units * c <= 2 * 128 && part_bytes >= 64 * 1024;
            const bool large = part_bytes >= 256 * 1024 || single_wave;
            int64_t chunk_vecs = k_chunk_kb > 0 ? k_chunk_kb * 64 : (large ? 2048 : 1024);
            if (chunk_vecs > part_vecs) chunk_vecs = part_vecs;
            const int64_t chunks = (part_vecs + chunk_vecs - 1) / chunk_vecs;
            const int64_t chunk_bytes = chunk_vecs * 16;
            int64_t nslots = k_slots > 0 ? k_slots : 3;
            if (k_slots == 0 && chunks < nslots) nslots = chunks;      // tiny parts: fully resident
            if (nslots > kMaxSlots || nslots * chunk_bytes > kMaxPartBytes || nslots < 1) {
                if (k_cluster > 0) break;
                continue;
            }
            if (nslots < chunks && nslots < 2) { if (k_cluster > 0) break; continue; }
            const size_t smem = kHeaderBytes + static_cast<size_t>(nslots * chunk_bytes);
            // 256 consumer threads: full chunks are then 4 or 8 vectors per thread (the
            // unrolled kernel variants)
            int consumers = k_cwarps > 0 ? k_cwarps * 32 : part_bytes >= 8 * 1024 ? 256 : 96;
            if (consumers > 480) consumers = 480;
            const int threads = consumers + 32;
            int active = 0;
            cudaError_t err = s.dtype == kF16
                                  ? resident_active_clusters<__half>(c, threads, smem, static_cast<int>(chunk_vecs), &active)
                                  : resident_active_clusters<float>(c, threads, smem, static_cast<int>(chunk_vecs), &active);
            if (err != cudaSuccess) { (void)cudaGetLastError(); active = 0; }
            if (active <= 0) { if (k_cluster > 0) break; continue; }
            const int64_t waves = (units + active - 1) / active;
            plan->path = kGnResident;
            plan->cluster = c;
            plan->threads = threads;
            plan->smem = smem;
            plan->nclusters = static_cast<int>((units + waves - 1) / waves);
            plan->chunk_vecs = static_cast<int>(chunk_vecs);
            plan->nslots = static_cast<int>(nslots);
            plan->hold = (force_cluster >> 28) & 3 ? ((force_cluster >> 28) & 3) - 1 : static_cast<int>(nslots) - 1;
            return cudaSuccess;
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
    if (force_cluster > 0) splits = force_cluster & 0xffff;
    int64_t chunk = (slab_elems + splits - 1) / splits;
    chunk = ((chunk + vec - 1) / vec) * vec;
    splits = (slab_elems + chunk - 1) / chunk;
    plan->splits = static_cast<int>(splits);
    plan->workspace = static_cast<size_t>(units * splits * 2) * sizeof(float);
    return cudaSuccess;
}

bool gn_concat_fused_ok(const GnShape &s, const GnPlan &plan, const void *in1, const void *in2, int64_t c1) {
    const int64_t esz = s.dtype == kF16 ? 2 : 4;
    return (plan.path == kGnResident || plan.path == kGnRegister) && !plan.nhwc && aligned16(in1) &&
           aligned16(in2) && (s.hw * esz) % 16 == 0 && c1 > 0 && c1 < s.channels;
}

cudaError_t gn_launch(const GnShape &s, const GnPlan &plan, const void *in, void *out,
                      const float *w, const float *b, void *workspace, cudaStream_t stream,
                      const void *bias, const void *in2, int64_t c1) {
    const int64_t esz = s.dtype == kF16 ? 2 : 4;
    const int64_t vec = 16 / esz;
    const int64_t cpg = s.channels / s.groups;
    const int64_t slab_elems = cpg * s.hw;
    const int64_t units = s.batch * s.groups;
    if (units == 0 || slab_elems == 0) return cudaSuccess;

    if (plan.path == kGnRegister) {
        RegArgs a;
        a.in = in; a.out = out; a.w = w; a.b = b; a.bias = bias;
        a.units = static_cast<uint32_t>(units);
        a.slab_vecs = static_cast<uint32_t>(slab_elems * esz / 16);
        a.slab_elems = static_cast<uint32_t>(slab_elems);
        a.cpg = static_cast<uint32_t>(cpg);
        a.groups = static_cast<uint32_t>(s.groups);
        a.channels = static_cast<uint32_t>(s.channels);
        a.vec_uniform = s.hw % vec == 0;
        a.eps = s.eps;
        a.hw_div = FastDiv::make(static_cast<uint32_t>(s.hw));
        a.hwv_div = FastDiv::make(a.vec_uniform ? static_cast<uint32_t>(s.hw / vec) : 1u);
        a.hw = static_cast<uint32_t>(s.hw);
        a.hw_vecs = a.vec_uniform ? static_cast<uint32_t>(s.hw / vec) : 1u;
        a.row_bytes = static_cast<uint32_t>(gn_nhwc_row_bytes(s));
        a.pair = s.dtype == kF16 && cpg % 2 == 0;
        a.out_div = FastDiv::make(static_cast<uint32_t>(a.pair ? cpg / 2 : cpg));
        a.in2 = in2;
        a.c1 = static_cast<uint32_t>(c1);
        if (in2 != nullptr && !gn_concat_fused_ok(s, plan, in, in2, c1)) return cudaErrorInvalidValue;
        const bool nhwc = plan.nhwc != 0;
        if (s.dtype == kF16)
            return s.act == kActSilu ? launch_register<__half, kActSilu>(a, nhwc, stream)
                                     : launch_register<__half, kActNone>(a, nhwc, stream);
        return s.act == kActSilu ? launch_register<float, kActSilu>(a, nhwc, stream)
                                 : launch_register<float, kActNone>(a, nhwc, stream);
    }

    if (plan.path == kGnResident) {
        ResidentArgs a;
        a.in = in; a.out = out; a.w = w; a.b = b;
        a.units = static_cast<uint32_t>(units);
        a.slab_vecs = static_cast<uint32_t>(slab_elems * esz / 16);
        a.slab_elems = static_cast<uint32_t>(slab_elems);
        a.cpg = static_cast<uint32_t>(cpg);
        a.groups = static_cast<uint32_t>(s.groups);
        a.chunk_vecs = static_cast<uint32_t>(plan.chunk_vecs);
        a.nslots = static_cast<uint32_t>(plan.nslots);
        a.hold = static_cast<uint32_t>(plan.hold);
        a.channels = static_cast<uint32_t>(s.channels);
        a.bias = bias;
        a.in2 = in2;
        a.c1 = static_cast<uint32_t>(c1);
        if (in2 != nullptr && !gn_concat_fused_ok(s, plan, in, in2, c1)) return cudaErrorInvalidValue;
        a.vec_uniform = s.hw % vec == 0;
        a.hw_vecs = a.vec_uniform ? static_cast<uint32_t>(s.hw / vec) : 1u;
        a.eps = s.eps;
        a.hw_div = FastDiv::make(static_cast<uint32_t>(s.hw));
        a.hwv_div = FastDiv::make(a.hw_vecs);
        if (s.dtype == kF16)
            return s.act == kActSilu ? launch_resident<__half, kActSilu>(a, plan, stream)
                                     : launch_resident<__half, kActNone>(a, plan, stream);
        return s.act == kActSilu ? launch_resident<float, kActSilu>(a, plan, stream)
                                 : launch_resident<float, kActNone>(a, plan, stream);
    }

    if (workspace == nullptr || in2 != nullptr) return cudaErrorInvalidValue;
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
#define SDFL_NHWC_APPLY(T, ACT)                                                              \
        do {                                                                                 \
            if (pairs) gn_apply_nhwc_kernel<T, ACT, true><<<tgrid, tblock, 0, stream>>>(a, hw32);   \
            else gn_apply_nhwc_kernel<T, ACT, false><<<tgrid, tblock, 0, stream>>>(a, hw32);        \
        } while (0)
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
// One warp waits, with a short limit, on an mbarrier that nothing will ever complete; the wait
// must give up by itself and raise the status word, leaving the context usable.
__global__ void wait_selftest_kernel(long long limit_cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_addr(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool ok = mbar_wait_bounded(smem_addr(&bar), 0, limit_cycles);
    if (!ok && threadIdx.x == 0) atomicOr(&g_gn_status, 1u);
}
}  // namespace

cudaError_t gn_wait_selftest(long long limit_cycles, cudaStream_t stream) {
    if (limit_cycles < 1000) limit_cycles = 1000;
    if (limit_cycles > 2000000000LL) limit_cycles = 2000000000LL;
    wait_selftest_kernel<<<1, 32, 0, stream>>>(limit_cycles);
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) g_launches.fetch_add(1);
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
