// Host-side launchers of the CUDA kernels; the C ABI (capi.cu) validates arguments and calls
// these.  Every launcher returns the cudaError_t of its launch and adds the number of kernels
// it enqueued to g_launches.
#pragma once

#include <atomic>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sdfl {

extern std::atomic<long long> g_launches;

// ---- GroupNorm (+SiLU) ------------------------------------------------------------------------
// Two device paths:
//   kGnResident  one thread-block cluster per (image, group) slab; the slab is staged in the
//                cluster's shared memory by bulk-copy engine transfers, so statistics, affine
//                and activation cost one HBM read and one HBM write.
//   kGnSplit     two kernels with a caller-provided scratch of per-chunk (mean, M2) partials;
//                any size, any alignment; one extra read of the tensor (mostly L2 for mid sizes).
//   kGnRegister  one CTA per slab, the slab in its registers (slabs up to 192 KB): lowest latency.
enum GnPath : int { kGnAuto = 0, kGnResident = 1, kGnSplit = 2, kGnRegister = 3 };

struct GnPlan {
    int path;          // kGnResident, kGnSplit or kGnRegister
    int cluster;       // CTAs per slab (resident): 1..16
    int threads;       // threads per CTA (resident: consumer warps + one producer warp)
    int nclusters;     // persistent clusters launched (resident)
    int chunk_vecs;    // 16-byte vectors per shared-memory ring chunk (resident)
    int nslots;        // chunk slots in the ring (resident); fewer than a part's chunks = re-read mode
    int hold;          // chunks kept in their slots between the two passes in re-read mode
    int splits;        // chunks per slab (split path)
    size_t smem;       // dynamic shared memory per CTA (resident)
    size_t workspace;  // scratch bytes the split path needs
    int nhwc;          // register path only: write the result channels-last ([batch, hw, channels])
};

struct GnShape {
    int64_t batch, channels, hw, groups;
    int dtype;         // kF32 / kF16
    float eps;
    int act;           // kActNone / kActSilu
    int bias;          // a per-(image, channel) addend will be passed to gn_launch
};

// Decide the path.  `force_path` / `force_cluster` (0 = automatic) are for tests and sweeps.
// in/out alignment matters for the resident path (16-byte bulk copies).
cudaError_t gn_make_plan(const GnShape &s, const void *in, const void *out, int force_path,
                         int force_cluster, GnPlan *plan);

// Whether GroupNorm with a channels-last store can run as one kernel (slab in one CTA's registers,
// transposed through shared memory); otherwise the caller normalises into a scratch tensor and
// transposes it with permute_021_launch.
bool gn_nhwc_fused_ok(const GnShape &s, const void *in, const void *out);
int64_t gn_nhwc_row_bytes(const GnShape &s);

// bias: optional [batch, channels] addend of the storage type, applied before the statistics.
// in2 / c1: the input is given as two tensors to be concatenated along the channels,
// in = [batch, c1, hw] and in2 = [batch, channels - c1, hw] (only where gn_concat_fused_ok).
cudaError_t gn_launch(const GnShape &s, const GnPlan &plan, const void *in, void *out,
                      const float *w, const float *b, void *workspace, cudaStream_t stream,
                      const void *bias = nullptr, const void *in2 = nullptr, int64_t c1 = 0);
bool gn_concat_fused_ok(const GnShape &s, const GnPlan &plan, const void *in1, const void *in2, int64_t c1);

// up_sample_nearest over `planes` images of H x W; concat of two [batch, n1] / [batch, n2] blocks.
cudaError_t upsample_nearest_launch(const void *in, void *out, int64_t planes, int64_t H, int64_t W,
                                    int64_t scale, int dtype, cudaStream_t stream);
cudaError_t concat_launch(const void *in1, const void *in2, void *out, int64_t batch, int64_t n1,
                          int64_t n2, int dtype, cudaStream_t stream);

// GroupNorm (+SiLU) over a list of tensors in one persistent launch (gn_multi.cu).  All tensors
// share dtype and activation; each needs 16-byte aligned buffers, hw * element size a multiple
// of 16 and slabs of at least 512 bytes (gn_multi_check returns 0).
constexpr int kGnMultiMaxTensors = 8;
constexpr int kGnMultiMaxCtas = 512;
constexpr int kGnMultiMaxGangs = 512;
constexpr size_t kGnMultiScratchBytes = 16 + static_cast<size_t>(kGnMultiMaxGangs) * 8 * 8 +
                                        static_cast<size_t>(kGnMultiMaxCtas) * (4 + 8 * 16);
struct GnMultiTensor {
    const void *in;
    void *out;
    const float *w;
    const float *b;
    int64_t batch, channels, hw, groups;
    float eps;
};
int gn_multi_check(const GnMultiTensor *ts, int n, int dtype);
// knobs (0 = automatic): bits 0-7 CTAs per gang; 8-9 teams (1: the whole gang on every slab, 2: a team
// size per tensor); 10 cooperative launch; 11 upper half of the gangs starts at the small end of the
// list (30: never); 12-13 share of a slab per CTA the team sizes aim at, in units of 128 KB; 14-15
// order of the items (1 static, 2 drawn from a counter); 16-23 ring chunk in KB (16 or 32); 24-27
// ring slots; 28-29 held chunks + 1.
// scratch: kGnMultiScratchBytes of device memory, zero before its first use, or nullptr for the
// library's own.  trace: nullptr, or [grid][16] device words for the time stamps of one launch.
// plan_out (optional): {CTAs per gang, grid, split, shared memory bytes}.
cudaError_t gn_multi_launch(const GnMultiTensor *ts, int n, int dtype, int act, int knobs, void *scratch,
                            unsigned long long *trace, int *plan_out, cudaStream_t stream);
cudaError_t gn_multi_read_status(unsigned int *value, bool clear, cudaStream_t stream);

// The split path with its scratch in a fixed array inside the library (64 KiB per device: up to
// 8192 (mean, M2) pairs, i.e. batch * groups * chunks-per-slab <= 8192).  Allocates nothing; the
// first call on a device resolves the array's device address.
constexpr size_t kGnStaticScratchBytes = 64 * 1024;
cudaError_t gn_launch_static_scratch(const GnShape &s, const GnPlan &plan, const void *in, void *out,
                                     const float *w, const float *b, cudaStream_t stream);

// Sticky device-side status word of the GroupNorm kernels (bit 0: a bounded wait on a bulk
// copy ran out).  Reads it, optionally clears it.
cudaError_t gn_read_status(unsigned int *value, bool clear, cudaStream_t stream);
// The same word of the register kernel's cluster variant (a wait for the cluster's moments).
cudaError_t gn_register_read_status(unsigned int *value, bool clear, cudaStream_t stream);

// Enqueues a one-warp kernel whose bounded wait is bound to run out (nothing completes its
// barrier): the wait ends after `limit_cycles` clock cycles and raises bit 0 of the status word.
cudaError_t gn_wait_selftest(long long limit_cycles, cudaStream_t stream);

// Stand-alone statistics / apply kernels that keep the reference's three-launch call sequence.
cudaError_t stats_mean_launch(const void *in, float *out, int64_t groups, int64_t n, int dtype,
                              cudaStream_t stream);
cudaError_t stats_var_launch(const void *in, const float *mean, float *out, int64_t groups,
                             int64_t n, int dtype, cudaStream_t stream);
cudaError_t gn_apply_launch(const void *in, const float *mean, const float *var, const float *w,
                            const float *b, int64_t group_size, int64_t channel_size, float eps,
                            void *out, int64_t n, int64_t channels, int dtype, cudaStream_t stream);
cudaError_t ln_apply_launch(const void *in, const float *mean, const float *var, const float *w,
                            const float *b, int64_t dim, float eps, void *out, int64_t n, int dtype,
                            cudaStream_t stream);

// ---- LayerNorm --------------------------------------------------------------------------------
cudaError_t ln_launch(const void *in, void *out, const float *w, const float *b, int64_t rows,
                      int64_t dim, float eps, int dtype, cudaStream_t stream);

// sum_out = a + b (rounded to the storage type), out = LayerNorm(sum_out); one launch when possible.
cudaError_t add_ln_launch(const void *a, const void *b2, void *sum_out, void *out, const float *w,
                          const float *b, int64_t rows, int64_t dim, float eps, int dtype,
                          cudaStream_t stream);

// ---- Elementwise ------------------------------------------------------------------------------
cudaError_t geglu_launch(const void *ab, void *dst, int64_t rows, int64_t d, int dtype,
                         cudaStream_t stream);
cudaError_t act_launch(int act, const void *src, void *dst, int64_t n, int dtype,
                       cudaStream_t stream);
cudaError_t add_launch(const void *a, const void *b, void *c, int64_t n, int dtype,
                       cudaStream_t stream);
// C[i] = A[i] + chunk[i / chunk_size]   (util.cl:136-148)
// Row softmax over the last dimension of [rows, dim]; out == in allowed.
cudaError_t softmax_launch(const void *in, void *out, int64_t rows, int64_t dim, int dtype,
                           cudaStream_t stream);

// dst[i][k][j] = src[i][j][k] (+ res[i][k][j] when res != nullptr): the reference's
// permute3D__0_2_1, optionally fused with the residual add that follows it.
cudaError_t permute_021_launch(const void *src, const void *res, void *dst, int64_t I, int64_t J,
                               int64_t K, int dtype, cudaStream_t stream);
cudaError_t chunkwise_add_launch(const void *a, const void *chunk, void *c, int64_t n,
                                 int64_t chunk_size, int dtype, cudaStream_t stream);

// ---- Embeddings -------------------------------------------------------------------------------
cudaError_t token_embedding_launch(const int64_t *ids, const void *table, const void *pos,
                                   void *out, int64_t batch, int64_t t, int64_t d, int64_t vocab,
                                   int dtype, int *d_status, cudaStream_t stream);
cudaError_t timestep_embedding_launch(const int64_t *t, void *out, int64_t batch, int64_t dim,
                                      float max_period, int dtype, cudaStream_t stream);

}  // namespace sdfl
