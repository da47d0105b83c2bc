// GroupNorm (+SiLU) over a LIST of NCHW tensors in one persistent launch (group_norm.cl:1-76 and
// util.cl:124-134 for every tensor of the list; one HBM read and one HBM write of each).
//
// Why a list: the norms of independent tensors (the images of a batch shard, the two halves of a
// classifier-free-guidance pair, the layers of a benchmark step) each pay a start-up, a first-data
// latency, an exchange and a drain when they are launched one by one, and a launch whose slabs do
// not fill the machine leaves SMs idle.  Here all slabs of all tensors form one list of work items
// and one grid of resident CTAs walks it, so those costs are paid once and every CTA slot of
// every SM is used.
//
// Structure.  The grid is cut into GANGS of K consecutive CTAs (K = 8 for the VAE sizes).  The slabs
// ((image, group) pairs) of all tensors, largest first, form one list of work items.  A gang takes
// its first item by position and every further one from a counter in global memory (one atomicAdd
// per gang and item by the gang's first CTA, which publishes the answer to the others), so gangs
// that run faster simply take more items; with few items per gang the upper half of the gangs
// draws from the small end of the list, which keeps the gangs out of step with each other
// (reading, exchanging and writing at different times).  "static" order (gang g takes items g,
// g + G, ...) is kept as an option.
// A tensor with small slabs does not need all K CTAs on one slab: it gets a TEAM size k that divides
// K, the gang falls into K / k teams, and one item of that tensor is K / k consecutive slabs, one per
// team.  k is chosen so that a CTA's share of a slab is about 256 KB: a slab spread over more CTAs
// pays the exchange for little work each, a larger share leaves more slabs waiting in L2.  CTA r
// of a team owns the r-th k-th of its slab and moves it in chunks of 16 or 32 KB through a ring of
// shared-memory slots:
//   producer warp : cp.async.bulk global -> shared with one "full" mbarrier per slot, refilled as
//                   soon as the consumers release the slot ("empty" mbarrier), across item and
//                   tensor boundaries; the slot of an item's first chunk also carries its number;
//   consumer warps: F phase: shifted sums of the chunks as they land -> (n, mean, M2) by Chan merges;
//                   team-wide exchange of the partial results; S phase: normalise + affine
//                   (+ SiLU) from the ring to global memory.  The last chunks of F stay in the ring
//                   for S; the others are loaded a second time (first load with an L2 evict_last
//                   hint, so the second is served by L2: K / k slabs per gang wait there, which
//                   bounds the number of gangs).
// Exchange of the partial (n, mean, M2) results.  A gang is K plain CTAs of a grid that is
// resident as a whole (at most the number of CTAs the device can hold at once), not a thread-block
// cluster: clusters of 8 reach 264 of the 296 CTA slots of a B200 and cannot change their size from
// item to item.  A CTA publishes its result in a global scratch as two 64-bit words that
// carry the item's token beside the value, and polls its team's words until they show the token
// (relaxed accesses at GPU scope, bounded).  Tokens are launch-unique: all CTAs
// read a sequence word at start and the last CTA to leave (an arrival counter) advances it and
// clears the item counter, so the scratch needs no clearing between launches; it has to be zero
// before its first use only.  Launches that share a scratch must not overlap on the GPU.
// No CTA ever waits on another launch; every wait is bounded (see mbar_wait_bounded).
#include "gn_device.cuh"

#include <algorithm>
#include <vector>

namespace sdfl {

namespace {

__device__ unsigned int g_multi_status;   // sticky; bit 0: a bounded wait ran out

constexpr int kMultiMaxTeam = 32;                // CTAs per gang
constexpr int kMultiThreads = 288;               // 8 consumer warps + the producer warp
constexpr uint32_t kMultiMaxRingBytes = 96 * 1024;
constexpr uint32_t kNumBufs = 8;                 // exchange buffers in rotation (item ordinal mod 8)

// shared-memory header
constexpr uint32_t kOffFull = 0, kOffEmpty = 128, kOffStatBar = 256, kOffWarpM = 384, kOffMetaItem = 576,
                   kOffMetaTurn = 640, kOffPeer = 704;
constexpr uint32_t kMultiHeader = 4864;
static_assert(kOffPeer + kNumBufs * 32 * 16 <= kMultiHeader, "header layout");
constexpr uint32_t kEndMark = 0xffffffffu;       // in a slot's item word: no more items for this CTA
static_assert(kMultiHeader % 128 == 0, "header layout");

// A CTA's result for one item: two 64-bit words, each the launch-unique token of the item in its upper
// half and one value in its lower half.  A word is written and read whole, so a reader that finds the
// token has the value with it and needs no fence or second round trip.
struct ExchSlot { unsigned long long mean, m2; };
struct ExchScratch {
    uint32_t seq;        // tokens of a launch are seq + 1 + turn
    uint32_t done;       // CTAs of the running launch that have finished
    // dynamic order: items handed out from the front of the list (low word) and from its back (high word)
    unsigned long long next;
    unsigned long long turn[kGnMultiMaxGangs][kNumBufs];   // (token << 32) | item of a gang's n-th turn, published by its first CTA
    uint32_t progress[kGnMultiMaxCtas];            // seq + number of turns a CTA has read
    ExchSlot slot[kGnMultiMaxCtas][kNumBufs];
};
static_assert(sizeof(ExchScratch) == kGnMultiScratchBytes, "scratch layout");

// Scratch of the global exchange for callers that pass none: zero when the module is loaded and
// left consistent by every launch.  Launches that share it must not overlap on the GPU.
static __device__ __align__(256) ExchScratch g_multi_scratch;

struct MultiTensor {
    const void *in;
    void *out;
    const float *w;
    const float *b;
    uint32_t item0;        // index of this tensor's first item in the item list (an item = K / k slabs)
    uint32_t units;        // slabs = batch * groups
    uint32_t slab_vecs;    // 16-byte vectors per slab
    uint32_t slab_elems;
    uint32_t cpg;          // channels per group
    uint32_t groups;
    uint32_t hw_vecs;      // vectors per channel
    uint32_t team;         // k: CTAs per slab (divides the gang size)
    float eps;
    FastDiv hwv_div;       // vector offset in the slab -> channel of the group
};

struct MultiArgs {
    MultiTensor t[kGnMultiMaxTensors];
    uint32_t ntensors;
    uint32_t total_items;
    uint32_t chunk_vecs;   // vectors per ring chunk
    uint32_t nslots;
    uint32_t hold;         // chunks kept in their slots between F and S
    uint32_t gang;         // K
    uint32_t items_per_gang;   // of the busiest gang
    uint32_t reverse_from; // gangs from this index on walk the list from its end
    uint32_t dynamic;      // gangs draw their items from a counter instead of taking every G-th
    ExchScratch *x;
    unsigned long long *trace;   // TRACE only: [gridDim.x][16] globaltimer stamps and counters
};

// One item as seen by one CTA: its team's slab `unit` (valid: the tensor has that many slabs), of
// which the CTA owns vectors [v0, v0 + nv), P chunks; the last H stay in the ring between F and S.
struct Geom { uint32_t ti, unit, k, r, first_cta, v0, nv, P, H; bool valid; };

__device__ __forceinline__ Geom item_geom(const MultiArgs &a, uint32_t item, uint32_t rank, uint32_t gang) {
    Geom g;
    uint32_t ti = 0;
    while (ti + 1 < a.ntensors && item >= a.t[ti + 1].item0) ++ti;
    g.ti = ti;
    const uint32_t k = a.t[ti].team, teams = a.gang / k;
    const uint32_t team = rank / k;
    g.k = k;
    g.r = rank - team * k;
    g.first_cta = gang * a.gang + team * k;
    g.unit = (item - a.t[ti].item0) * teams + team;
    g.valid = g.unit < a.t[ti].units;
    const uint32_t sv = a.t[ti].slab_vecs;
    g.v0 = static_cast<uint32_t>((static_cast<uint64_t>(sv) * g.r) / k);
    const uint32_t v1 = static_cast<uint32_t>((static_cast<uint64_t>(sv) * (g.r + 1)) / k);
    g.nv = v1 - g.v0;
    g.P = (g.nv + a.chunk_vecs - 1) / a.chunk_vecs;
    g.H = g.P <= a.nslots ? g.P : min(a.hold, a.nslots - 1u);
    return g;
}

__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_gpu_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// blockDim.x = 288: 256 consumer threads + the producer warp.  Chunks are 256 * NV vectors, so a full
// chunk inside one channel is NV vectors per thread at compile-time offsets.
template <typename T, int ACT, int NV, bool TRACE>
__global__ void __launch_bounds__(kMultiThreads, NV == 4 ? 4 : 2)
gn_multi_kernel(const MultiArgs a) {
    constexpr int VEC = VecOf<T>::N;
    constexpr uint32_t kConsumers = kMultiThreads - 32;
    constexpr uint32_t kCWarps = kConsumers / 32;
    const uint32_t K = a.gang;
    const uint32_t gang = blockIdx.x / K;
    const uint32_t rank = blockIdx.x - gang * K;
    const uint32_t ngangs = gridDim.x / K;
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    unsigned long long *trace = TRACE ? a.trace + static_cast<size_t>(blockIdx.x) * 16 : nullptr;
    if (TRACE && tid == 0) trace[0] = global_timer();

    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kOffFull);          // [kMaxSlots]
    uint64_t *empty = reinterpret_cast<uint64_t *>(smem + kOffEmpty);        // [kMaxSlots]
    uint64_t *stat_bar = reinterpret_cast<uint64_t *>(smem + kOffStatBar);   // [kNumBufs]
    Moments *warp_m = reinterpret_cast<Moments *>(smem + kOffWarpM);         // [2][8]
    uint32_t *meta_item = reinterpret_cast<uint32_t *>(smem + kOffMetaItem); // [kMaxSlots] item whose first chunk is in the slot
    uint32_t *meta_turn = reinterpret_cast<uint32_t *>(smem + kOffMetaTurn); // [kMaxSlots] and the gang's turn number
    float4 *peer = reinterpret_cast<float4 *>(smem + kOffPeer);              // [kNumBufs][32] (-, n, mean, M2)
    unsigned char *data = smem + kMultiHeader;

    const uint32_t cv = a.chunk_vecs;
    const uint32_t S = a.nslots;
    const uint32_t chunk_bytes = cv * 16u;
    // this gang's items: list positions gang, gang + G, ... (walked backwards by the upper gangs)
    const uint32_t n_mine = gang < a.total_items ? (a.total_items - gang + ngangs - 1u) / ngangs : 0u;
    const bool reversed = gang >= a.reverse_from;
    auto item_at = [&](uint32_t it) { return gang + (reversed ? n_mine - 1u - it : it) * ngangs; };

    if (warp == kCWarps) {
        // ---------------- producer warp ----------------------------------------------------------
        if (lane == 0) {
            for (uint32_t k = 0; k < S; ++k) {
                mbar_init(smem_addr(&full[k]), 1);
                mbar_init(smem_addr(&empty[k]), kCWarps);
            }
            for (uint32_t k = 0; k < kNumBufs; ++k) mbar_init(smem_addr(&stat_bar[k]), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // inits before the copy engine's arrivals
        }
        __syncthreads();           // the consumers may use the barriers from here on
        if (lane != 0) return;
        bool timed_out = false;
        const uint64_t keep = policy_evict_last(), drop = policy_evict_first();
        const uint32_t base = ld_relaxed_gpu(&a.x->seq);
        uint32_t slot = 0, round = 0;
        bool first = true;
        auto claim = [&]() {       // the slot's previous occupant must have been released
            if (round > 0) {
                if (!mbar_wait_bounded(smem_addr(&empty[slot]), (round - 1) & 1u,
                                       timed_out ? kWaitCyclesAfterTimeout : kWaitCycles))
                    timed_out = true;
            }
        };
        auto spin_until = [&](auto &&ready) {
            if (ready()) return;
            const long long t0 = clock64();
            while (!ready()) {
                if (clock64() - t0 > (timed_out ? kWaitCyclesAfterTimeout : kWaitCycles)) { timed_out = true; return; }
                __nanosleep(32);
            }
        };
        for (uint32_t turn = 0;; ++turn) {
            // ---- which item is this gang's turn-th? ----
            uint32_t item = kEndMark;
            if (a.dynamic && turn == 0) {
                // The first turn needs no counter: the front gangs take the first items of the list,
                // the others its last ones (the counter's words start at zero and count from there).
                const uint32_t nfront = min(a.reverse_from, ngangs);
                if (ngangs <= a.total_items) item = reversed ? a.total_items - 1u - (gang - nfront) : gang;
                else if (gang < a.total_items) item = gang;
            } else if (a.dynamic) {
                unsigned long long *q = &a.x->turn[gang][turn % kNumBufs];
                const uint32_t token = base + turn + 1u;
                if (rank == 0) {
                    // The entry is reused every kNumBufs turns: every CTA of the gang must have read
                    // its previous content (teams of a gang do not wait for each other).
                    if (turn >= kNumBufs)
                        for (uint32_t m = 0; m < K; ++m)
                            spin_until([&] { return static_cast<int32_t>(ld_relaxed_gpu(&a.x->progress[gang * K + m]) -
                                                                         (base + turn - (kNumBufs - 1u))) >= 0; });
                    const unsigned long long old = atomicAdd(&a.x->next, reversed ? (1ull << 32) : 1ull);
                    // items already given out in the first turn: nfront from the front, the rest from the back
                    const uint32_t nfront = min(a.reverse_from, ngangs);
                    const unsigned long long front = static_cast<uint32_t>(old) + static_cast<unsigned long long>(nfront);
                    const unsigned long long back = static_cast<uint32_t>(old >> 32) + static_cast<unsigned long long>(ngangs - nfront);
                    uint32_t mine = kEndMark;
                    if (front + back < a.total_items)
                        mine = reversed ? a.total_items - 1u - static_cast<uint32_t>(back) : static_cast<uint32_t>(front);
                    st_relaxed_gpu_u64(q, (static_cast<unsigned long long>(token) << 32) | mine);
                }
                unsigned long long word = 0;
                spin_until([&] { word = ld_relaxed_gpu_u64(q); return static_cast<uint32_t>(word >> 32) == token; });
                item = timed_out ? kEndMark : static_cast<uint32_t>(word);
                asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(&a.x->progress[blockIdx.x]), "r"(token) : "memory");
            } else if (turn < n_mine) {
                item = item_at(turn);
            }
            if (item == kEndMark) {
                // end mark: a slot without data, completed by a plain arrival
                claim();
                meta_item[slot] = kEndMark;
                mbar_arrive(smem_addr(&full[slot]));
                break;
            }
            const Geom g = item_geom(a, item, rank, gang);
            if (!g.valid) continue;          // the tensor's last item may not fill every team
            const unsigned char *gsrc = static_cast<const unsigned char *>(a.t[g.ti].in) +
                                        (static_cast<size_t>(g.unit) * a.t[g.ti].slab_vecs + g.v0) * 16u;
            // F: the share's chunks, the last H stay in the ring.  S: the others again (from L2).
            for (uint32_t j = 0; j < 2u * g.P - g.H; ++j) {
                const uint32_t c = j < g.P ? j : j - g.P;
                const uint32_t lo = c * cv;
                const uint32_t bytes = (min(cv, g.nv - lo)) * 16u;
                claim();
                if (j == 0) { meta_item[slot] = item; meta_turn[slot] = turn; }
                const uint32_t bar = smem_addr(&full[slot]);
                mbar_expect_tx(bar, bytes);
                // a chunk that will be read a second time should stay in L2; a last read need not
                bulk_load_hint(smem_addr(data + slot * chunk_bytes), gsrc + static_cast<size_t>(lo) * 16u, bytes, bar,
                               (j < g.P && c + g.H < g.P) ? keep : drop);
                if (TRACE && first) { trace[7] = global_timer(); first = false; }
                if (++slot == S) { slot = 0; ++round; }
            }
        }
        if (timed_out) atomicOr(&g_multi_status, 1u);
        return;
    }

    // ---------------- consumer warps -------------------------------------------------------------
    uint32_t base = 0;
    if (warp == 0) base = ld_relaxed_gpu(&a.x->seq);
    __syncthreads();
    if (TRACE && tid == 0) trace[1] = global_timer();

    bool timed_out = false;
    uint32_t pos = 0;                        // ring position of the next slot to consume
    uint32_t bar_phase = 0;                  // bit b: parity of stat_bar[b]'s next completion
    uint32_t done_items = 0;
    unsigned long long wait_x = 0, wait_p1 = 0, wait_p2 = 0, stamp = 0;
    auto wait_full = [&](uint32_t p) {
        if (!mbar_wait_bounded(smem_addr(&full[p % S]), (p / S) & 1u,
                               timed_out ? kWaitCyclesAfterTimeout : kWaitCycles))
            timed_out = true;
    };
    auto release = [&](uint32_t p) {
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_addr(&empty[p % S]));
    };
    for (;;) {
        // the producer names the item in the slot of its first chunk
        if (TRACE && tid == 0) stamp = global_timer();
        wait_full(pos);
        if (TRACE && tid == 0) wait_p1 += global_timer() - stamp;
        const uint32_t item = meta_item[pos % S];
        if (item == kEndMark || timed_out) break;
        const uint32_t it = meta_turn[pos % S];      // the gang's turn: same number in all its CTAs
        const Geom g = item_geom(a, item, rank, gang);
        const MultiTensor &t = a.t[g.ti];
        const uint32_t buf = it % kNumBufs;
        const bool traced = TRACE && tid == 0 && done_items == 0;
        ++done_items;

        // ---- F: shifted sums, chunk by chunk as the copies land ----------------------------------
        const uint32_t p_first = pos;
        float s[2] = {0.f, 0.f}, sq[2] = {0.f, 0.f};
        float shift = 0.f;
        uint32_t nvec_mine = 0;
        for (uint32_t j = 0; j < g.P; ++j) {
            const uint32_t p = pos++;
            if (j > 0) {
                if (TRACE && tid == 0) stamp = global_timer();
                wait_full(p);
                if (TRACE && tid == 0) wait_p1 += global_timer() - stamp;
            }
            if (traced && j == 0) trace[2] = global_timer();
            const uint4 *sv = reinterpret_cast<const uint4 *>(data + (p % S) * chunk_bytes);
            if (j == 0) shift = to_float<T>(reinterpret_cast<const T *>(sv)[0]);
            const uint32_t cnt = min(cv, g.nv - j * cv);
            if (cnt == 256u * NV) {
                uint4 v[NV];
#pragma unroll
                for (int k = 0; k < NV; ++k) v[k] = sv[tid + k * 256];
#pragma unroll
                for (int k = 0; k < NV; ++k) stats_vec<T>(v[k], shift, s, sq);
                nvec_mine += NV;
            } else {
#pragma unroll 2
                for (uint32_t i = tid; i < cnt; i += kConsumers) {
                    stats_vec<T>(sv[i], shift, s, sq);
                    ++nvec_mine;
                }
            }
            if (j + g.H < g.P) release(p);      // the last H chunks are held for S
        }
        Moments m;
        {
            const float cnt = static_cast<float>(nvec_mine * VEC);
            const float ss = s[0] + s[1], qq = sq[0] + sq[1];
            m.n = cnt;
            m.mean = nvec_mine ? shift + ss / cnt : 0.f;
            m.m2 = nvec_mine ? fmaxf(qq - ss * ss / cnt, 0.f) : 0.f;
        }
        m = warp_merge(m);
        if (lane == 0) warp_m[(it & 1u) * kCWarps + warp] = m;
        consumer_sync(kConsumers);
        if (traced) trace[3] = global_timer();
        const uint32_t token = base + it + 1u;
        if (warp == 0) {
            // warp_m alternates between two sets: a warp can be at most one F phase ahead of warp 0
            Moments c = lane < kCWarps ? warp_m[(it & 1u) * kCWarps + lane] : Moments{0.f, 0.f, 0.f};
            c = warp_merge(c);
            if (g.k == 1) {
                // a team of one: the slab's moments are this CTA's, nothing to exchange
                peer[buf * 32u + lane] = lane == 0 ? make_float4(0.f, c.n, c.mean, c.m2) : make_float4(0.f, 0.f, 0.f, 0.f);
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_addr(&stat_bar[buf]));
            } else if (lane == 0) {
                ExchSlot *mine = &a.x->slot[blockIdx.x][buf];
                st_relaxed_gpu_u64(&mine->mean, (static_cast<unsigned long long>(token) << 32) | __float_as_uint(c.mean));
                st_relaxed_gpu_u64(&mine->m2, (static_cast<unsigned long long>(token) << 32) | __float_as_uint(c.m2));
            }
        }

        // ---- S: wait for the team's results, then normalise + affine (+ activation) ---------------
        const uint32_t hwv = t.hw_vecs;
        const FastDiv hwv_div = t.hwv_div;
        const uint32_t ch0 = (g.unit % t.groups) * t.cpg;
        const float *wp = t.w + ch0, *bp = t.b + ch0;
        // first chunk of S (a held one if any) and its channel: scale and shift are fetched now, so
        // that their L2 round trip runs beside the wait
        const uint32_t c_first = hwv_div.div(g.v0 + (g.P - g.H) % g.P * cv);
        const float w_first = __ldg(wp + c_first), b_first = __ldg(bp + c_first);
        if (TRACE && tid == 0) stamp = global_timer();
        if (warp == 0 && g.k > 1) {
            // collect the team's results from global memory into shared memory
            float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
            if (lane < g.k) {
                const ExchSlot *ps = &a.x->slot[g.first_cta + lane][buf];
                unsigned long long wm = ld_relaxed_gpu_u64(&ps->mean), w2 = ld_relaxed_gpu_u64(&ps->m2);
                auto both = [&] { return static_cast<uint32_t>(wm >> 32) == token && static_cast<uint32_t>(w2 >> 32) == token; };
                if (!both()) {
                    const long long t0 = clock64();
                    const long long limit = timed_out ? kWaitCyclesAfterTimeout : kWaitCycles;
                    do {
                        if (clock64() - t0 > limit) { timed_out = true; break; }
                        wm = ld_relaxed_gpu_u64(&ps->mean);
                        w2 = ld_relaxed_gpu_u64(&ps->m2);
                    } while (!both());
                }
                // peer `lane` owns vectors [q0, q1) of the slab
                const uint32_t q0 = static_cast<uint32_t>((static_cast<uint64_t>(t.slab_vecs) * lane) / g.k);
                const uint32_t q1 = static_cast<uint32_t>((static_cast<uint64_t>(t.slab_vecs) * (lane + 1)) / g.k);
                r.y = static_cast<float>(q1 - q0) * VEC;
                r.z = __uint_as_float(static_cast<uint32_t>(wm));
                r.w = __uint_as_float(static_cast<uint32_t>(w2));
            }
            peer[buf * 32u + lane] = r;
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_addr(&stat_bar[buf]));
        }
        if (!mbar_wait_bounded(smem_addr(&stat_bar[buf]), (bar_phase >> buf) & 1u,
                               timed_out ? kWaitCyclesAfterTimeout : kWaitCycles))
            timed_out = true;
        bar_phase ^= 1u << buf;
        if (TRACE && tid == 0) wait_x += global_timer() - stamp;
        float mean, rstd;
        {
            // every warp folds the results itself, in rank order (same bits in every CTA of the team)
            const float4 r = peer[buf * 32u + lane];
            Moments f{r.y, r.z, r.w};
            f = warp_merge(f);
            const float var = __shfl_sync(0xffffffffu, f.m2, 0) / static_cast<float>(t.slab_elems);   // biased: group_norm.cl:53-55
            mean = __shfl_sync(0xffffffffu, f.mean, 0);
            rstd = 1.0f / sqrtf(var + t.eps);
        }
        if (traced) trace[4] = global_timer();

        // Held chunks (P-H .. P-1, still in their slots since F) first, then chunks 0 .. P-H-1 as
        // they come back.
        uint4 *gv0 = reinterpret_cast<uint4 *>(static_cast<unsigned char *>(t.out) +
                                               (static_cast<size_t>(g.unit) * t.slab_vecs + g.v0) * 16u);
        for (uint32_t k = 0; k < g.P; ++k) {
            const bool held = k < g.H;
            const uint32_t c = held ? g.P - g.H + k : k - g.H;         // chunk of the share
            const uint32_t p = held ? p_first + c : pos++;             // its ring position
            if (!held) {
                if (TRACE && tid == 0) stamp = global_timer();
                wait_full(p);
                if (TRACE && tid == 0) wait_p2 += global_timer() - stamp;
            }
            const uint4 *sv = reinterpret_cast<const uint4 *>(data + (p % S) * chunk_bytes);
            const uint32_t lo = c * cv;                 // share-relative vector index of the chunk
            const uint32_t hi = min(g.nv, lo + cv);
            uint4 *gv = gv0 + lo;
            bool fast = false;
            if (hi - lo == 256u * NV) {
                const uint32_t ch = hwv_div.div(g.v0 + lo);
                if (ch == hwv_div.div(g.v0 + hi - 1u)) {
                    fast = true;
                    const bool first = k == 0 && ch == c_first;
                    const Affine<T> af = make_affine<T, ACT>(mean, rstd, first ? w_first : __ldg(wp + ch),
                                                            first ? b_first : __ldg(bp + ch));
                    uint4 v[NV];
#pragma unroll
                    for (int n = 0; n < NV; ++n) v[n] = sv[tid + n * 256];
#pragma unroll
                    for (int n = 0; n < NV; ++n)
                        st_stream(&gv[tid + n * 256], norm_vec<T, ACT>(v[n], af));
                }
            }
            if (fast) {
            } else if (hwv >= kConsumers) {
                // long channels: walk channel by channel, weights hoisted out of the vector loop
                uint32_t i0 = lo;
                while (i0 < hi) {
                    const uint32_t ch = hwv_div.div(g.v0 + i0);
                    const uint32_t seg_end = min(hi, (ch + 1) * hwv - g.v0);
                    const Affine<T> af = make_affine<T, ACT>(mean, rstd, __ldg(wp + ch), __ldg(bp + ch));
#pragma unroll 2
                    for (uint32_t i = i0 + tid; i < seg_end; i += kConsumers)
                        st_stream(&gv[i - lo], norm_vec<T, ACT>(sv[i - lo], af));
                    i0 = seg_end;
                }
            } else {
                for (uint32_t i = lo + tid; i < hi; i += kConsumers) {
                    const uint32_t ch = hwv_div.div(g.v0 + i);
                    const Affine<T> af = make_affine<T, ACT>(mean, rstd, __ldg(wp + ch), __ldg(bp + ch));
                    st_stream(&gv[i - lo], norm_vec<T, ACT>(sv[i - lo], af));
                }
            }
            release(p);
        }
        if (traced) trace[5] = global_timer();
    }
    if (TRACE && tid == 0) {
        trace[6] = global_timer();
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        trace[8] = smid;
        trace[9] = done_items;
        trace[10] = wait_x;      // ns this thread waited for its team's statistics, all items
        trace[11] = wait_p1;     // ... for chunks to land in F phases
        trace[12] = wait_p2;     // ... for chunks to come back in S phases
    }
    if (timed_out && lane == 0) atomicOr(&g_multi_status, 1u);
    // The last CTA to get here advances the token sequence for the next launch.
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&a.x->done, 1u) == gridDim.x - 1u) {
            a.x->done = 0u;
            a.x->next = 0ull;
            a.x->seq = base + a.items_per_gang + 1u;
            __threadfence();
        }
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <typename T, int ACT, int NV, bool TR>
cudaError_t ensure_attrs() {
    static std::atomic<bool> done[kMaxDevices];
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < kMaxDevices && done[dev].load(std::memory_order_acquire)) return cudaSuccess;
    err = cudaFuncSetAttribute(gn_multi_kernel<T, ACT, NV, TR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kMultiHeader + kMultiMaxRingBytes));
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < kMaxDevices) done[dev].store(true, std::memory_order_release);
    return cudaSuccess;
}

// How many CTAs of this kernel the device holds at once (the whole grid has to be resident:
// the CTAs of a gang wait for each other).
template <typename T, int ACT, int NV, bool TR>
cudaError_t capacity_of(size_t smem, int *ctas) {
    static std::mutex mu;
    static std::map<uint64_t, int> cache;
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    const uint64_t key = (static_cast<uint64_t>(dev) << 32) | (smem >> 8);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *ctas = it->second; return cudaSuccess; }
    }
    err = ensure_attrs<T, ACT, NV, TR>();
    if (err != cudaSuccess) return err;
    int per_sm = 0, sms = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gn_multi_kernel<T, ACT, NV, TR>,
                                                        kMultiThreads, smem);
    if (err != cudaSuccess) return err;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    std::lock_guard<std::mutex> lock(mu);
    cache[key] = per_sm * sms;
    *ctas = per_sm * sms;
    return cudaSuccess;
}

template <typename T, int ACT, int NV, bool TR>
cudaError_t launch_as(const MultiArgs &a, int grid, size_t smem, bool cooperative, cudaStream_t stream) {
    cudaError_t err = ensure_attrs<T, ACT, NV, TR>();
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(kMultiThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (cooperative) {
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.numAttrs = 1;
    }
    err = cudaLaunchKernelEx(&cfg, gn_multi_kernel<T, ACT, NV, TR>, a);
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

struct Flavour { int nv; bool trace; };

template <typename T, int ACT>
cudaError_t dispatch_capacity(const Flavour &f, size_t smem, int *ctas) {
    if (f.trace) return capacity_of<T, ACT, 8, true>(smem, ctas);
    return f.nv == 8 ? capacity_of<T, ACT, 8, false>(smem, ctas) : capacity_of<T, ACT, 4, false>(smem, ctas);
}

template <typename T, int ACT>
cudaError_t dispatch_launch(const Flavour &f, const MultiArgs &a, int grid, size_t smem, bool coop,
                            cudaStream_t stream) {
    if (f.trace) return launch_as<T, ACT, 8, true>(a, grid, smem, coop, stream);
    return f.nv == 8 ? launch_as<T, ACT, 8, false>(a, grid, smem, coop, stream)
                     : launch_as<T, ACT, 4, false>(a, grid, smem, coop, stream);
}

cudaError_t scratch_address(void **ptr) {
    static std::mutex mu;
    static void *address[kMaxDevices] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (address[dev] == nullptr) {
        err = cudaGetSymbolAddress(&address[dev], g_multi_scratch);
        if (err != cudaSuccess) { address[dev] = nullptr; return err; }
    }
    *ptr = address[dev];
    return cudaSuccess;
}

// One candidate plan: gang size K and a team size per tensor (a divisor of K).
struct Deal {
    int gang = 0, gangs = 0;
    std::vector<int> team;       // per tensor (sorted order)
    std::vector<int64_t> items;  // per tensor: ceil(slabs / teams per gang)
    double cost = 0;
};

// Cost of dealing the item list round-robin to the gangs: the bytes the busiest CTA moves, plus a
// per-item allowance for the exchange and the pipeline turn-around (expressed in bytes of traffic).
double deal_cost(const Deal &d, const std::vector<int64_t> &slab_bytes) {
    constexpr double kItemOverheadBytes = 64.0 * 1024;
    std::vector<double> load(static_cast<size_t>(d.gangs), 0.0);
    int64_t item0 = 0;
    for (size_t k = 0; k < slab_bytes.size(); ++k) {
        const double per = static_cast<double>(slab_bytes[k]) / d.team[k] + kItemOverheadBytes;
        for (int g = 0; g < d.gangs; ++g) {
            // items item0 .. item0 + n - 1 congruent to g modulo gangs
            const int64_t first = item0 + ((g - item0 % d.gangs) + d.gangs) % d.gangs;
            const int64_t n = first < item0 + d.items[k] ? (item0 + d.items[k] - 1 - first) / d.gangs + 1 : 0;
            load[static_cast<size_t>(g)] += per * static_cast<double>(n);
        }
        item0 += d.items[k];
    }
    double worst = 0;
    for (double v : load) worst = std::max(worst, v);
    return worst;
}

// The same for the dynamic order (a gang draws its next item when it is free): items go to the least
// loaded gang, largest first; equal items of one tensor are dealt in bulk.
double deal_cost_dynamic(const Deal &d, const std::vector<int64_t> &slab_bytes) {
    constexpr double kItemOverheadBytes = 64.0 * 1024;
    std::vector<double> load(static_cast<size_t>(d.gangs), 0.0);
    for (size_t k = 0; k < slab_bytes.size(); ++k) {
        const double per = static_cast<double>(slab_bytes[k]) / d.team[k] + kItemOverheadBytes;
        const int64_t each = d.items[k] / d.gangs, rest = d.items[k] % d.gangs;
        for (double &v : load) v += per * static_cast<double>(each);
        std::sort(load.begin(), load.end());
        for (int64_t g = 0; g < rest; ++g) load[static_cast<size_t>(g)] += per;
    }
    return *std::max_element(load.begin(), load.end());
}

// Fill in teams / items / gangs / cost for gang size K.  `sized`: a team per tensor such that a
// CTA's share of a slab is about `target` bytes; otherwise the whole gang on every slab.
// Returns false when the plan is not allowed (shares below 1 KB, or more slabs waiting in L2
// between their two reads than fit).
bool make_deal(Deal *d, int K, bool sized, int64_t target, bool dynamic, int ctas,
               const std::vector<GnMultiTensor> &ts, const std::vector<int64_t> &slab_bytes) {
    constexpr double kMaxInFlightBytes = 80.0 * 1024 * 1024;
    d->gang = K;
    d->team.clear();
    d->items.clear();
    int64_t total = 0;
    for (size_t k = 0; k < ts.size(); ++k) {
        int team = K;
        if (sized) {
            // the divisor of K whose share is closest to the target (in ratio)
            double best = 0;
            for (int c = 1; c <= K; ++c) {
                if (K % c) continue;
                const double share = static_cast<double>(slab_bytes[k]) / c;
                const double off = share > target ? share / target : target / share;
                if (c == 1 || off < best) { best = off; team = c; }
            }
        }
        if (slab_bytes[k] / 16 / team < 64 && team > 1) return false;
        const int64_t slabs = ts[k].batch * ts[k].groups;
        const int64_t teams = K / team;
        d->team.push_back(team);
        d->items.push_back((slabs + teams - 1) / teams);
        total += d->items.back();
    }
    d->gangs = ctas / K;
    if (d->gangs > total) d->gangs = static_cast<int>(total);
    if (d->gangs < 1) return false;
    {
        // Bytes between their two reads at once: every gang holds one item; the worst case is the
        // `gangs` largest items of the list (a tensor contributes no more items than it has).
        std::vector<std::pair<double, int64_t>> by_size;      // (bytes of one item, number of such items)
        for (size_t k = 0; k < ts.size(); ++k) {
            const int64_t slabs = ts[k].batch * ts[k].groups;
            const int64_t per_item = std::min<int64_t>(K / d->team[k], slabs);
            by_size.emplace_back(static_cast<double>(per_item) * static_cast<double>(slab_bytes[k]), d->items[k]);
        }
        std::sort(by_size.begin(), by_size.end(), [](const auto &x, const auto &y) { return x.first > y.first; });
        double in_flight = 0;
        int64_t left = d->gangs;
        for (const auto &e : by_size) {
            const int64_t n = std::min(left, e.second);
            in_flight += e.first * static_cast<double>(n);
            left -= n;
            if (left == 0) break;
        }
        if (in_flight > kMaxInFlightBytes) return false;
    }
    d->cost = dynamic ? deal_cost_dynamic(*d, slab_bytes) : deal_cost(*d, slab_bytes);
    return true;
}

}  // namespace

int gn_multi_check(const GnMultiTensor *ts, int n, int dtype) {
    if (n < 1 || n > kGnMultiMaxTensors) return 1;
    const int64_t esz = dtype == kF16 ? 2 : 4;
    int64_t total = 0;
    for (int k = 0; k < n; ++k) {
        const GnMultiTensor &t = ts[k];
        if (t.groups <= 0 || t.channels % t.groups != 0) return 2;
        const int64_t cpg = t.channels / t.groups;
        const int64_t slab_bytes = cpg * t.hw * esz;
        if (!gn_aligned16(t.in) || !gn_aligned16(t.out)) return 3;
        if ((t.hw * esz) % 16 != 0 || t.hw <= 0) return 4;
        if (slab_bytes / 16 < kMultiMaxTeam) return 5;             // every CTA of a gang needs a share
        if (slab_bytes >= (1ll << 31) || t.batch <= 0) return 6;
        total += t.batch * t.groups;
    }
    return total < (1ll << 27) ? 0 : 7;
}

cudaError_t gn_multi_launch(const GnMultiTensor *ts_in, int n, int dtype, int act, int knobs, void *scratch,
                            unsigned long long *trace, int *plan_out, cudaStream_t stream) {
    if (gn_multi_check(ts_in, n, dtype) != 0) return cudaErrorInvalidValue;
    const int64_t esz = dtype == kF16 ? 2 : 4;
    const int k_team = knobs & 0xff, k_sized = (knobs >> 8) & 0x3, k_coop = (knobs >> 10) & 1;
    const int k_reverse = ((knobs >> 11) & 1) | ((knobs >> 30) & 2), k_target = (knobs >> 12) & 0x3, k_order = (knobs >> 14) & 0x3;
    const int k_chunk_kb = (knobs >> 16) & 0xff, k_slots = (knobs >> 24) & 0xf, k_hold = (knobs >> 28) & 0x3;

    // largest slabs first
    std::vector<GnMultiTensor> ts(ts_in, ts_in + n);
    auto slab_of = [&](const GnMultiTensor &t) { return (t.channels / t.groups) * t.hw * esz; };
    std::stable_sort(ts.begin(), ts.end(), [&](const GnMultiTensor &x, const GnMultiTensor &y) {
        return slab_of(x) > slab_of(y);
    });
    std::vector<int64_t> slab_bytes;
    for (const auto &t : ts) slab_bytes.push_back(slab_of(t));
    int64_t total_items = 0;

    Flavour f;
    f.trace = trace != nullptr;
    const int chunk_kb = k_chunk_kb > 0 ? k_chunk_kb : 32;
    if (chunk_kb != 32 && chunk_kb != 16) return cudaErrorInvalidValue;
    f.nv = chunk_kb == 32 ? 8 : 4;
    if (f.trace && f.nv != 8) return cudaErrorInvalidValue;
    const int nslots = k_slots > 0 ? k_slots : 3;
    if (nslots < 2 || nslots > kMaxSlots) return cudaErrorInvalidValue;
    const size_t ring = static_cast<size_t>(nslots) * chunk_kb * 1024;
    if (ring > kMultiMaxRingBytes) return cudaErrorInvalidValue;
    const size_t smem = kMultiHeader + ring;

    int ctas = 0;
    {
        cudaError_t err;
        if (dtype == kF16)
            err = act == kActSilu ? dispatch_capacity<__half, kActSilu>(f, smem, &ctas)
                                  : dispatch_capacity<__half, kActNone>(f, smem, &ctas);
        else
            err = act == kActSilu ? dispatch_capacity<float, kActSilu>(f, smem, &ctas)
                                  : dispatch_capacity<float, kActNone>(f, smem, &ctas);
        if (err != cudaSuccess) return err;
    }
    if (ctas > kGnMultiMaxCtas) ctas = kGnMultiMaxCtas;
    if (ctas < 1) return cudaErrorInvalidConfiguration;

    // Gang size and teams: the plan that gives the busiest CTA the least to do.
    const bool dynamic = k_order != 1;
    Deal deal;
    bool have = false;
    for (int sized = 0; sized < 2; ++sized) {
        if ((k_sized == 1 && sized) || (k_sized == 2 && !sized)) continue;
        for (int tg = 1; tg <= 3; ++tg) {
            if ((k_target > 0 && tg != k_target) || (!sized && tg != 2)) continue;
            if (k_target == 0 && tg != 2) continue;      // 256 KB shares unless asked otherwise
            for (int k = 1; k <= kMultiMaxTeam && k <= ctas; k = (k_team > 0 ? k + 1 : k * 2)) {
                if (k_team > 0 && k != k_team) continue;
                Deal d;
                if (!make_deal(&d, k, sized != 0, tg * 128 * 1024, dynamic, ctas, ts, slab_bytes)) continue;
                if (!have || d.cost < deal.cost * 0.985) { deal = d; have = true; }
            }
        }
    }
    if (!have) return cudaErrorInvalidConfiguration;
    if (k_target == 0 && k_sized != 1) {
        // One or two items per gang: the launch is a couple of waves and its length is that of the
        // busiest gang; shares of 128 KB deal the work out more evenly than shares of 256 KB.
        int64_t items = 0;
        for (int64_t v : deal.items) items += v;
        Deal fine;
        if (items < 2 * static_cast<int64_t>(deal.gangs) &&
            make_deal(&fine, deal.gang, true, 128 * 1024, dynamic, ctas, ts, slab_bytes))
            deal = fine;
    }
    const int team = deal.gang, gangs = deal.gangs, grid = deal.gangs * deal.gang;
    total_items = 0;
    for (int64_t v : deal.items) total_items += v;
    if (gangs > kGnMultiMaxGangs || grid > kGnMultiMaxCtas) return cudaErrorInvalidConfiguration;

    MultiArgs a = {};
    int64_t item0 = 0;
    for (int k = 0; k < n; ++k) {
        const GnMultiTensor &t = ts[static_cast<size_t>(k)];
        MultiTensor &m = a.t[k];
        const int64_t cpg = t.channels / t.groups;
        m.in = t.in; m.out = t.out; m.w = t.w; m.b = t.b;
        m.item0 = static_cast<uint32_t>(item0);
        m.units = static_cast<uint32_t>(t.batch * t.groups);
        m.slab_vecs = static_cast<uint32_t>(cpg * t.hw * esz / 16);
        m.slab_elems = static_cast<uint32_t>(cpg * t.hw);
        m.cpg = static_cast<uint32_t>(cpg);
        m.groups = static_cast<uint32_t>(t.groups);
        m.hw_vecs = static_cast<uint32_t>(t.hw * esz / 16);
        m.team = static_cast<uint32_t>(deal.team[static_cast<size_t>(k)]);
        m.eps = t.eps;
        m.hwv_div = FastDiv::make(m.hw_vecs);
        item0 += deal.items[static_cast<size_t>(k)];
    }
    a.ntensors = static_cast<uint32_t>(n);
    a.total_items = static_cast<uint32_t>(total_items);
    a.chunk_vecs = static_cast<uint32_t>(chunk_kb * 64);
    a.nslots = static_cast<uint32_t>(nslots);
    a.hold = k_hold > 0 ? static_cast<uint32_t>(k_hold - 1) : static_cast<uint32_t>(nslots - 1);
    a.gang = static_cast<uint32_t>(team);
    a.items_per_gang = static_cast<uint32_t>(dynamic ? total_items + 1 : (total_items + gangs - 1) / gangs + 1);
    a.dynamic = dynamic ? 1u : 0u;
    a.trace = trace;
    // A launch of one or two waves: the upper half of the gangs starts at the small end of the list, so
    // that the gangs are not all in the same phase (reading, exchanging, writing) at the same time.
    const bool reverse = k_reverse == 1 || (k_reverse == 0 && total_items <= 2 * static_cast<int64_t>(gangs));
    a.reverse_from = reverse ? static_cast<uint32_t>((gangs + 1) / 2) : static_cast<uint32_t>(gangs);
    void *p = scratch;
    if (p == nullptr) {
        cudaError_t err = scratch_address(&p);
        if (err != cudaSuccess) return err;
    }
    a.x = static_cast<ExchScratch *>(p);
    if (plan_out != nullptr) {
        plan_out[0] = team; plan_out[1] = grid; plan_out[3] = static_cast<int>(smem);
        plan_out[2] = 0;                     // the tensors' team sizes, 8 bits each, in the caller's order
        for (int k = 0; k < n && k < 4; ++k)
            for (int q = 0; q < n; ++q)
                if (ts[static_cast<size_t>(q)].in == ts_in[k].in && ts[static_cast<size_t>(q)].out == ts_in[k].out) {
                    plan_out[2] |= deal.team[static_cast<size_t>(q)] << (8 * k);
                    break;
                }
    }
    if (dtype == kF16)
        return act == kActSilu ? dispatch_launch<__half, kActSilu>(f, a, grid, smem, k_coop != 0, stream)
                               : dispatch_launch<__half, kActNone>(f, a, grid, smem, k_coop != 0, stream);
    return act == kActSilu ? dispatch_launch<float, kActSilu>(f, a, grid, smem, k_coop != 0, stream)
                           : dispatch_launch<float, kActNone>(f, a, grid, smem, k_coop != 0, stream);
}

cudaError_t gn_multi_read_status(unsigned int *value, bool clear, cudaStream_t stream) {
    cudaError_t err = cudaMemcpyFromSymbolAsync(value, g_multi_status, sizeof(unsigned int), 0,
                                                cudaMemcpyDeviceToHost, stream);
    if (err != cudaSuccess) return err;
    err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) return err;
    if (clear && *value != 0) {
        const unsigned int zero = 0;
        err = cudaMemcpyToSymbolAsync(g_multi_status, &zero, sizeof(unsigned int), 0,
                                      cudaMemcpyHostToDevice, stream);
        // A launch that gave up a wait may have left the library's own scratch (sequence word, arrival
        // and item counters) half-way: start it afresh.  A caller's workspace is the caller's to clear.
        void *p = nullptr;
        if (err == cudaSuccess) err = scratch_address(&p);
        if (err == cudaSuccess) err = cudaMemsetAsync(p, 0, sizeof(ExchScratch), stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    }
    return err;
}

}  // namespace sdfl
