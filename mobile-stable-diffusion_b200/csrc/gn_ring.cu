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
#include "gn_device.cuh"

namespace sdfl {

namespace {

__device__ unsigned int g_gn_status;   // sticky; bit 0: a bounded mbarrier wait ran out

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
        // Scale and shift of the first chunk of the normalise pass: fetched now, so that their L2
        // round trip runs beside the exchange instead of behind it.
        const uint32_t ch0 = (unit % a.groups) * a.cpg;
        const uint32_t c_first = a.vec_uniform ? a.hwv_div.div(v0 + (P - H) % P * cv) : 0u;
        const float w_first = __ldg(a.w + ch0 + c_first), b_first = __ldg(a.b + ch0 + c_first);
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
                    const bool first = k == 0 && c == c_first;
                    const Affine<T> af = make_affine<T, ACT>(mc, rstd, first ? w_first : __ldg(a.w + ch0 + c),
                                                            first ? b_first : __ldg(a.b + ch0 + c));
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

// Per-device, per-kernel-instance one-time attribute set-up (maximum dynamic shared memory and
// the opt-in for 16-CTA clusters), so that launches themselves make no attribute calls.
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

inline int plan_unroll(int threads, int chunk_vecs) { return gn_ring_unroll(threads, chunk_vecs); }

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

// How many clusters of this size, block size and shared-memory footprint can be resident at
// once (a cluster must fit inside one GPC).  Asked of the driver once per (device, kernel
// instance, cluster, threads, shared-memory size in KiB) and remembered; the instance asked about
// is the one that will be launched (activation and addend change its register count).
template <typename T, int ACT, bool BIAS, int NV>
cudaError_t active_clusters_of(cudaLaunchConfig_t *cfg, int *n) {
    cudaError_t err = ensure_resident_attrs<T, ACT, BIAS, NV>();
    if (err != cudaSuccess) return err;
    return cudaOccupancyMaxActiveClusters(n, gn_resident_kernel<T, ACT, BIAS, NV>, cfg);
}

template <typename T, int ACT, bool BIAS>
cudaError_t active_clusters_nv(int nv, cudaLaunchConfig_t *cfg, int *n) {
    switch (nv) {
        case 8: return active_clusters_of<T, ACT, BIAS, 8>(cfg, n);
        case 4: return active_clusters_of<T, ACT, BIAS, 4>(cfg, n);
        default: return active_clusters_of<T, ACT, BIAS, 0>(cfg, n);
    }
}

template <typename T>
cudaError_t resident_active_clusters(int act, bool bias, int cluster, int threads, size_t smem, int chunk_vecs,
                                     int *active) {
    static std::mutex mu;
    static std::map<uint64_t, int> cache;
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    const uint64_t kb = (smem + 1023) / 1024;
    const int nv = plan_unroll(threads, chunk_vecs);
    const uint64_t key = (static_cast<uint64_t>(dev) << 48) | (static_cast<uint64_t>(sizeof(T)) << 40) |
                         (static_cast<uint64_t>(cluster) << 32) |
                         (static_cast<uint64_t>(threads) << 16) | kb | (static_cast<uint64_t>(nv) << 56) |
                         (static_cast<uint64_t>(act == kActSilu) << 60) | (static_cast<uint64_t>(bias) << 61);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *active = it->second; return cudaSuccess; }
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    cluster_config(&cfg, attr, static_cast<unsigned>(cluster), cluster, threads, smem, nullptr);
    int n = 0;
    if (act == kActSilu)
        err = bias ? active_clusters_nv<T, kActSilu, true>(nv, &cfg, &n) : active_clusters_nv<T, kActSilu, false>(nv, &cfg, &n);
    else
        err = bias ? active_clusters_nv<T, kActNone, true>(nv, &cfg, &n) : active_clusters_nv<T, kActNone, false>(nv, &cfg, &n);
    if (err != cudaSuccess) return err;
    *active = n;
    std::lock_guard<std::mutex> lock(mu);
    cache[key] = n;
    return cudaSuccess;
}

}  // namespace

cudaError_t gn_ring_active_clusters(int dtype, int act, bool bias, int cluster, int threads, size_t smem,
                                    int chunk_vecs, int *active) {
    return dtype == kF16 ? resident_active_clusters<__half>(act, bias, cluster, threads, smem, chunk_vecs, active)
                         : resident_active_clusters<float>(act, bias, cluster, threads, smem, chunk_vecs, active);
}

cudaError_t gn_ring_launch(const GnShape &s, const GnPlan &plan, const void *in, void *out, const float *w,
                           const float *b, cudaStream_t stream, const void *bias, const void *in2, int64_t c1) {
    const int64_t esz = s.dtype == kF16 ? 2 : 4;
    const int64_t vec = 16 / esz;
    const int64_t cpg = s.channels / s.groups;
    const int64_t slab_elems = cpg * s.hw;
    const int64_t units = s.batch * s.groups;
    if (units == 0 || slab_elems == 0) return cudaSuccess;
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

}  // namespace sdfl
