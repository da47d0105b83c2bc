// GroupNorm (+SiLU), register path: one CTA per (image, group) slab, the slab in the CTA's
// registers (group_norm.cl:1-76 and util.cl:124-134 in one launch, one read and one write).
#include "gn_device.cuh"

namespace sdfl {

namespace {

// ---------------------------------------------------------------------------------------------
// Register path: one CTA per slab, the whole slab in the CTA's registers
// ---------------------------------------------------------------------------------------------
// For the slabs of the UNet (5-240 KB) the cluster kernel's fixed costs (cluster start-up, barrier
// set-up, the exchange) are most of its time.  Here a CTA of 512 threads loads its slab with up to
// NVT 16-byte vectors per thread, all loads in flight at once, folds the moments through one
// __syncthreads and normalises from registers: one HBM read, one write, no shared-memory staging.
// Every load of a slab precedes every store to it, so out == in is safe.
constexpr int kRegThreads = kGnRegThreads;
constexpr int kRegMaxVecs = kGnRegMaxVecs;
// A group's scale and shift are fetched together with the slab and parked in shared memory when the
// group has at most this many channels: fetched after the statistics instead, their DRAM round
// trip (cold weights: every layer has its own) was 10-20 % of a small launch.
constexpr uint32_t kRegStagedChannels = 256;
constexpr int kRegMaxCluster = kGnRegMaxCluster;

__device__ unsigned int g_reg_status;   // sticky; bit 0: a bounded wait for the cluster's moments ran out

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
    // CLU: a cluster of `cluster` CTAs per slab, each holding `share_vecs` consecutive vectors of it
    uint32_t cluster, share_vecs;
};

// NHWC: the result is written channels-last, out[n][p][c] (the permute3D__0_2_1 that follows the
// norm of a SpatialTransformer block, SpatialTransformer.cpp:127-140, fused into the store).  The
// normalised slab [cpg][hw] goes through shared memory with a 4-byte skew per channel row and
// leaves as runs of cpg consecutive channels per pixel.
//
// CLU: the slab is shared by a thread-block cluster, CTA r holding vectors [r * share, (r + 1) * share)
// of it, so that slabs of 64-240 KB are pulled by 2-8 SMs instead of one.  Each CTA pushes its
// (n, mean, M2) into every CTA of the cluster (distributed shared memory) and signals that CTA's
// mbarrier; everybody folds the same values in the same order, so all CTAs of a slab normalise with
// bit-identical statistics.
template <typename T, int ACT, bool BIAS, int NVT, bool NHWC, bool CLU>
__global__ void __launch_bounds__(kRegThreads, (NVT <= 4 || (CLU && NVT <= 8)) ? 2 : 1)
gn_register_kernel(const RegArgs a) {
    static_assert(!(NHWC && CLU), "the channels-last store needs the whole slab in one CTA");
    constexpr int VEC = VecOf<T>::N;
    constexpr bool HALF = sizeof(T) == 2;
    __shared__ Moments warp_m[kRegThreads / 32];
    __shared__ float s_w[kRegStagedChannels], s_b[kRegStagedChannels];
    __shared__ __align__(16) float4 cl_m[2][kRegMaxCluster];  // CLU: (n, mean, M2, -) of every CTA of the cluster
    __shared__ __align__(8) uint64_t cl_bar[2];               // CLU: one arrival per CTA of the cluster
    extern __shared__ __align__(16) unsigned char tsm[];      // NHWC only: cpg rows of row_bytes
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const bool staged = a.cpg <= kRegStagedChannels;
    uint32_t rank = 0;
    if (CLU) {
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
        if (tid == 0) {
            mbar_init(smem_addr(&cl_bar[0]), a.cluster);
            mbar_init(smem_addr(&cl_bar[1]), a.cluster);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        // Every CTA of the cluster has started and set up its barriers once this completes; it
        // is waited for only before the first push, behind the slab's loads.
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    }
    const uint32_t lo = CLU ? rank * a.share_vecs : 0u;
    const uint32_t hi = CLU ? min(lo + a.share_vecs, a.slab_vecs) : a.slab_vecs;
    const uint32_t first = CLU ? blockIdx.x / a.cluster : blockIdx.x;
    const uint32_t stride = CLU ? gridDim.x / a.cluster : gridDim.x;
    bool timed_out = false;
    uint32_t it = 0;
    for (uint32_t unit = first; unit < a.units; unit += stride, ++it) {
        const uint32_t ch0 = (unit % a.groups) * a.cpg;
        float w_mine = 0.f, b_mine = 0.f;
        if (staged && tid < a.cpg) {             // in flight together with the slab's loads
            w_mine = __ldg(a.w + ch0 + tid);
            b_mine = __ldg(a.b + ch0 + tid);
        }
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
            const uint32_t idx = lo + tid + k * kRegThreads;
            if (idx < hi) v[k] = ld_stream((idx < split ? src : src2) + idx);
        }
        if (staged && tid < a.cpg) {             // visible after the barrier that follows the moments
            s_w[tid] = w_mine;
            s_b[tid] = b_mine;
        }
        // this thread's moments, shifted by its first value
        float s[2] = {0.f, 0.f}, q[2] = {0.f, 0.f};
        float shift = 0.f;
        uint32_t mine = 0;
        if (lo + tid < hi) {
            shift = HALF ? __half2float(__ushort_as_half(static_cast<unsigned short>(v[0].x & 0xffffu)))
                         : __uint_as_float(v[0].x);
            if (BIAS) shift += to_float<T>(erow[a.hw_div.div((lo + tid) * VEC)]);
        }
#pragma unroll
        for (int k = 0; k < NVT; ++k) {
            const uint32_t idx = lo + tid + k * kRegThreads;
            if (idx < hi) {
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
        if (CLU) {
            const uint32_t par = it & 1u;
            if (it == 0) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            if (warp == 0) {
                const float bn = __shfl_sync(0xffffffffu, t.n, 0), bmean = __shfl_sync(0xffffffffu, t.mean, 0),
                            bm2 = __shfl_sync(0xffffffffu, t.m2, 0);
                if (lane < a.cluster) {
                    const uint32_t dst_m = map_to_rank(smem_addr(&cl_m[par][rank]), lane);
                    st_peer_f32x2(dst_m, bn, bmean);
                    st_peer_f32x2(dst_m + 8u, bm2, 0.f);
                    mbar_arrive_peer(map_to_rank(smem_addr(&cl_bar[par]), lane));
                }
            }
            if (!mbar_wait_cluster_bounded(smem_addr(&cl_bar[par]), (it >> 1) & 1u,
                                           timed_out ? kWaitCyclesAfterTimeout : kWaitCycles))
                timed_out = true;
            const float4 pm = lane < a.cluster ? cl_m[par][lane] : make_float4(0.f, 0.f, 0.f, 0.f);
            t = warp_merge(Moments{pm.x, pm.y, pm.z});
        }
        const float mean = __shfl_sync(0xffffffffu, t.mean, 0);
        const float var = __shfl_sync(0xffffffffu, t.m2, 0) / static_cast<float>(a.slab_elems);   // biased
        const float rstd = 1.0f / sqrtf(var + a.eps);
#pragma unroll
        for (int k = 0; k < NVT; ++k) {
            const uint32_t idx = lo + tid + k * kRegThreads;
            if (idx < hi) {
                if (a.vec_uniform) {
                    const uint32_t cl = a.hwv_div.div(idx), c = ch0 + cl;
                    const float mc = BIAS ? mean - to_float<T>(erow[cl]) : mean;
                    const Affine<T> af = make_affine<T, ACT>(mc, rstd, staged ? s_w[cl] : __ldg(a.w + c),
                                                            staged ? s_b[cl] : __ldg(a.b + c));
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
                        f[l] = activate<ACT, HALF>(fmaf((f[l] - mc) * rstd, staged ? s_w[cl] : __ldg(a.w + c),
                                                        staged ? s_b[cl] : __ldg(a.b + c)));
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
    if (CLU && timed_out && tid == 0) atomicOr(&g_reg_status, 1u);
}

constexpr size_t kRegMaxStageBytes = kGnRegMaxStageBytes;

template <typename T, int ACT, int NVT>
cudaError_t launch_register_nhwc(const RegArgs &a, unsigned grid, size_t smem, cudaStream_t stream) {
    static std::atomic<bool> done[kMaxDevices];
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (!(dev >= 0 && dev < kMaxDevices && done[dev].load(std::memory_order_acquire))) {
        err = cudaFuncSetAttribute(gn_register_kernel<T, ACT, false, NVT, true, false>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kRegMaxStageBytes));
        if (err != cudaSuccess) return err;
        if (dev >= 0 && dev < kMaxDevices) done[dev].store(true, std::memory_order_release);
    }
    gn_register_kernel<T, ACT, false, NVT, true, false><<<grid, kRegThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

template <typename T, int ACT, bool BIAS, int NVT>
cudaError_t launch_register_cluster(const RegArgs &a, unsigned grid, cudaStream_t stream) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cluster_config(&cfg, attr, grid, static_cast<int>(a.cluster), kRegThreads, 0, stream);
    return cudaLaunchKernelEx(&cfg, gn_register_kernel<T, ACT, BIAS, NVT, false, true>, a);
}

template <typename T, int ACT, bool BIAS>
cudaError_t launch_register_as(const RegArgs &a, bool nhwc, cudaStream_t stream) {
    if (a.cluster > 1) {
        if (nhwc) return cudaErrorInvalidValue;
        const uint32_t per_thread = (a.share_vecs + kRegThreads - 1) / kRegThreads;
        // whole clusters only; a persistent grid beyond what the device holds would only queue
        const unsigned max_clusters = static_cast<unsigned>(sm_count()) * 64u / a.cluster;
        const unsigned grid = (a.units < max_clusters ? a.units : max_clusters) * a.cluster;
        cudaError_t err = per_thread <= 4    ? launch_register_cluster<T, ACT, BIAS, 4>(a, grid, stream)
                          : per_thread <= 8  ? launch_register_cluster<T, ACT, BIAS, 8>(a, grid, stream)
                          : per_thread <= 12 ? launch_register_cluster<T, ACT, BIAS, 12>(a, grid, stream)
                                             : launch_register_cluster<T, ACT, BIAS, kRegMaxVecs>(a, grid, stream);
        if (err == cudaSuccess) g_launches.fetch_add(1);
        return err;
    }
    const uint32_t per_thread = (a.slab_vecs + kRegThreads - 1) / kRegThreads;
    const unsigned grid = a.units < static_cast<unsigned>(sm_count()) * 64u ? a.units : static_cast<unsigned>(sm_count()) * 64u;
    cudaError_t err;
    if (nhwc) {
        if (BIAS) return cudaErrorInvalidValue;
        const size_t smem = static_cast<size_t>(a.cpg) * a.row_bytes;
        err = per_thread <= 4    ? launch_register_nhwc<T, ACT, 4>(a, grid, smem, stream)
              : per_thread <= 12 ? launch_register_nhwc<T, ACT, 12>(a, grid, smem, stream)
                                 : launch_register_nhwc<T, ACT, kRegMaxVecs>(a, grid, smem, stream);
    } else {
        if (per_thread <= 4)
            gn_register_kernel<T, ACT, BIAS, 4, false, false><<<grid, kRegThreads, 0, stream>>>(a);
        else if (per_thread <= 12)
            gn_register_kernel<T, ACT, BIAS, 12, false, false><<<grid, kRegThreads, 0, stream>>>(a);
        else
            gn_register_kernel<T, ACT, BIAS, kRegMaxVecs, false, false><<<grid, kRegThreads, 0, stream>>>(a);
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

}  // namespace

cudaError_t gn_register_launch(const GnShape &s, const GnPlan &plan, const void *in, void *out,
                               const float *w, const float *b, cudaStream_t stream, const void *bias,
                               const void *in2, int64_t c1) {
    const int64_t esz = s.dtype == kF16 ? 2 : 4;
    const int64_t vec = 16 / esz;
    const int64_t cpg = s.channels / s.groups;
    const int64_t slab_elems = cpg * s.hw;
    const int64_t units = s.batch * s.groups;
    if (units == 0 || slab_elems == 0) return cudaSuccess;
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
    a.cluster = static_cast<uint32_t>(plan.cluster > 1 ? plan.cluster : 1);
    if (a.cluster > static_cast<uint32_t>(kRegMaxCluster)) return cudaErrorInvalidValue;
    a.share_vecs = (a.slab_vecs + a.cluster - 1) / a.cluster;
    if (in2 != nullptr && !gn_concat_fused_ok(s, plan, in, in2, c1)) return cudaErrorInvalidValue;
    const bool nhwc = plan.nhwc != 0;
    if (s.dtype == kF16)
        return s.act == kActSilu ? launch_register<__half, kActSilu>(a, nhwc, stream)
                                 : launch_register<__half, kActNone>(a, nhwc, stream);
    return s.act == kActSilu ? launch_register<float, kActSilu>(a, nhwc, stream)
                             : launch_register<float, kActNone>(a, nhwc, stream);
}

cudaError_t gn_register_read_status(unsigned int *value, bool clear, cudaStream_t stream) {
    cudaError_t err = cudaMemcpyFromSymbolAsync(value, g_reg_status, sizeof(unsigned int), 0,
                                                cudaMemcpyDeviceToHost, stream);
    if (err != cudaSuccess) return err;
    err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) return err;
    if (clear && *value != 0) {
        const unsigned int zero = 0;
        err = cudaMemcpyToSymbolAsync(g_reg_status, &zero, sizeof(unsigned int), 0,
                                      cudaMemcpyHostToDevice, stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    }
    return err;
}

}  // namespace sdfl
