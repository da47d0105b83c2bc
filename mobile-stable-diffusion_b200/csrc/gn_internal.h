// Interfaces between the GroupNorm translation units (planner / dispatch in groupnorm.cu, the
// cluster ring kernel in gn_ring.cu, the register kernel in gn_register.cu, the split path and the
// stand-alone kernels in gn_split.cu).  Not part of the library's public surface.
#pragma once

#include "kernels.h"

namespace sdfl {

// ---- cluster ring kernel (gn_ring.cu) ----------------------------------------------------------
constexpr int kGnMaxSlots = 16;
constexpr uint32_t kGnHeaderBytes = 1024;            // mbarriers, merge scratch, published moments
constexpr uint32_t kGnMaxPartBytes = 226 * 1024;     // per-CTA ring (227 KB less the header)

// The unrolled kernel variants need 256 consumer threads and chunks of 256 * NV vectors.
inline int gn_ring_unroll(int threads, int chunk_vecs) {
    if (threads != 288) return 0;
    return chunk_vecs == 2048 ? 8 : chunk_vecs == 1024 ? 4 : 0;
}
// How many clusters of this size, block size and shared-memory footprint can be resident at once.
cudaError_t gn_ring_active_clusters(int dtype, int act, bool bias, int cluster, int threads, size_t smem,
                                    int chunk_vecs, int *active);
cudaError_t gn_ring_launch(const GnShape &s, const GnPlan &plan, const void *in, void *out, const float *w,
                           const float *b, cudaStream_t stream, const void *bias, const void *in2, int64_t c1);

// ---- register kernel (gn_register.cu) ----------------------------------------------------------
constexpr int kGnRegThreads = 512;
constexpr int kGnRegMaxVecs = 24;                    // per thread: slabs up to 512 * 24 * 16 B = 192 KB
constexpr size_t kGnRegMaxStageBytes = 200 * 1024;   // shared-memory staging of the channels-last store
constexpr int kGnRegMaxCluster = 8;                  // CTAs that may share one slab (portable cluster size)
cudaError_t gn_register_launch(const GnShape &s, const GnPlan &plan, const void *in, void *out,
                               const float *w, const float *b, cudaStream_t stream, const void *bias,
                               const void *in2, int64_t c1);

// ---- split path (gn_split.cu) ------------------------------------------------------------------
cudaError_t gn_split_launch(const GnShape &s, const GnPlan &plan, const void *in, void *out, const float *w,
                            const float *b, void *workspace, cudaStream_t stream, const void *bias);

inline bool gn_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace sdfl
