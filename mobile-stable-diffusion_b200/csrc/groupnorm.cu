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
//
// This file: the choice of path and geometry (gn_make_plan) and the dispatch (gn_launch).  The
// kernels are in gn_ring.cu (cluster ring), gn_register.cu (one CTA per slab) and gn_split.cu.
#include "common.cuh"
#include "gn_internal.h"

namespace sdfl {

namespace {

constexpr int kMaxSlots = kGnMaxSlots;
constexpr uint32_t kHeaderBytes = kGnHeaderBytes;
constexpr uint32_t kMaxPartBytes = kGnMaxPartBytes;
constexpr int kRegThreads = kGnRegThreads;
constexpr int kRegMaxVecs = kGnRegMaxVecs;
constexpr size_t kRegMaxStageBytes = kGnRegMaxStageBytes;
constexpr int kSplitThreads = 512;

inline bool aligned16(const void *p) { return gn_aligned16(p); }

// When the register path beats the cluster path (launches timed back to back on B200, fp16 and
// fp32, 32-256 slabs of 5-240 KB): always for slabs up to 48 KB (3.5-6 us against 5.5-7); for
// larger ones once there are at least 64 slabs, i.e. enough CTAs to pull on HBM from many SMs
// (with 32 slabs a cluster of 8 per slab is 0.6-1.4 us faster from 120 KB on, and 0.3-0.6 us
// slower up to 80 KB).
inline bool prefer_register(int64_t slab_bytes, int64_t units) {
    return slab_bytes <= 48 * 1024 || units >= 64 || (units >= 32 && slab_bytes <= 96 * 1024);
}

// CTAs per slab on the register path (launches timed back to back on B200): four from 100 KB
// on when there are at most 64 slabs (10.4 against 11.6 us for 64 x 160 KB, 12.4 against 15.6 us
// for 64 x 240 KB, 7.7 against 9.2 us for 32 x 160 KB), eight for up to 32 slabs of 256-512 KB;
// below 100 KB, or with more slabs, a cluster only adds its start-up (0.4-1.3 us for clusters of
// 2-4, 5 us for 64 clusters of 8).
inline int register_cluster_for(int64_t slab_bytes, int64_t units) {
    if (units >= 24 && units <= 64 && slab_bytes >= 100 * 1024 && slab_bytes <= 256 * 1024) return 4;
    if (units >= 24 && units <= 32 && slab_bytes > 256 * 1024 && slab_bytes <= 512 * 1024) return 8;
    return 1;
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
    // A cluster of CTAs per slab, each with its share in registers: when a forced plan asks for it,
    // and for at most 64 slabs of 100-512 KB, where one CTA per slab leaves more than half of the
    // SMs without work and the ring kernel's start-up is most of such a short launch.
    int reg_cluster = 1;
    if (force_path == kGnRegister && (force_cluster & 0xff) > 1) {
        reg_cluster = force_cluster & 0xff;
        if (reg_cluster > kGnRegMaxCluster || (reg_cluster & (reg_cluster - 1)) != 0) return cudaErrorInvalidConfiguration;
    } else if (force_path == kGnAuto) {
        reg_cluster = register_cluster_for(slab_bytes, units);
    }
    const int64_t reg_share_vecs = (slab_bytes / 16 + reg_cluster - 1) / reg_cluster;
    const bool register_ok = resident_ok && reg_share_vecs <= static_cast<int64_t>(kRegThreads) * kRegMaxVecs;
    if (force_path == kGnRegister && !register_ok) return cudaErrorInvalidConfiguration;
    if (register_ok && (force_path == kGnRegister || reg_cluster > 1 ||
                        (force_path == kGnAuto && prefer_register(slab_bytes, units)))) {
        plan->path = kGnRegister;
        plan->cluster = reg_cluster;
        plan->threads = kRegThreads;
        const int64_t max_clusters = sm_count() * 64 / reg_cluster;
        plan->nclusters = static_cast<int>(units < max_clusters ? units : max_clusters);
        plan->chunk_vecs = static_cast<int>((reg_share_vecs + kRegThreads - 1) / kRegThreads);
        return cudaSuccess;
    }

    if (resident_ok) {
        // Ring geometry and cluster size (fp16 and fp32 behave alike per byte).  A small ring
        // (3 slots of 16-32 KB, 8 consumer warps) with the second read served by L2 rather than
        // full shared-memory residency: it keeps 2-4 CTAs on each SM, so one CTA's cluster
        // exchange hides behind the others' traffic.  The
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
            // a fill / exchange / drain latency chain: fewer, larger chunks, and shares up to
            // 96 KB stay resident.
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
            cudaError_t err = gn_ring_active_clusters(s.dtype, s.act, s.bias != 0, c, threads, smem, static_cast<int>(chunk_vecs), &active);
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
    int64_t splits = (sm_count() * 4 + units - 1) / units;
    const int64_t max_splits = (slab_elems + 16383) / 16384;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > 1024) splits = 1024;
    if (force_cluster > 0) splits = force_cluster & 0xffff;
    if (splits < 1) splits = 1;          // a forced count whose low 16 bits are zero
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
    if (plan.path == kGnRegister) return gn_register_launch(s, plan, in, out, w, b, stream, bias, in2, c1);
    if (plan.path == kGnResident) return gn_ring_launch(s, plan, in, out, w, b, stream, bias, in2, c1);
    if (in2 != nullptr) return cudaErrorInvalidValue;
    return gn_split_launch(s, plan, in, out, w, b, workspace, stream, bias);
}

}  // namespace sdfl
