/* sdfl -- Stable-Diffusion fused layer kernels for NVIDIA B200 (sm_100a): C ABI.
 *
 * Drop-in boundary for the fused-layer path of the reference app (its OpenCL C kernels and the
 * C++ operator classes that enqueue them).  Each entry point names the reference interface it
 * replaces; paths are inside the reference project:
 *   K/  = app/src/main/assets/kernel/        NN/ = app/src/main/cpp/modules/nn/
 *   M/  = app/src/main/cpp/modules/
 *
 * Conventions
 *   - All tensor pointers are CUDA device pointers owned by the caller unless a name starts with
 *     h_.  `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  Calls
 *     only enqueue work; ordering is the stream's (the reference returned cl_events instead).
 *   - dtype: SDFL_F32 or SDFL_F16 storage; arithmetic is always fp32; weights (gamma, beta) are
 *     always fp32, as in the reference.
 *   - Return value: 0 on success, a negative SDFL_ERR_* otherwise.  Nothing throws, nothing
 *     aborts.  The reference returned cl_int (0 = CL_SUCCESS) and threw std::runtime_error on
 *     contract violations (NN/GroupNorm.cpp:83-93); those cases are SDFL_ERR_INVALID_VALUE here.
 *   - out == in is allowed wherever the reference allows it (GroupNorm, LayerNorm, activations:
 *     NN/ResBlock.cpp:222, NN/ResBlock.cpp:136-137); partial overlap is SDFL_ERR_OVERLAP.
 *   - The library keeps no mutable host state per call and may be driven from several host
 *     threads, one CUDA device each.
 */
#ifndef SDFL_H_
#define SDFL_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { SDFL_F32 = 0, SDFL_F16 = 1 };

enum {
    SDFL_OK = 0,
    SDFL_ERR_INVALID_VALUE = -1,   /* bad size / shape / enum */
    SDFL_ERR_INVALID_POINTER = -2, /* NULL where a buffer is required */
    SDFL_ERR_UNSUPPORTED = -3,     /* shape outside what any kernel path handles */
    SDFL_ERR_CUDA = -4,            /* a CUDA call failed; see sdfl_last_cuda_error() */
    SDFL_ERR_OVERLAP = -5,         /* input and output partially overlap */
    SDFL_ERR_WORKSPACE = -6,       /* scratch buffer missing or too small */
    SDFL_ERR_DEVICE_FLAG = -7      /* a kernel raised its device-side status word */
};

/* GroupNorm path selection for sdfl_groupnorm_forward_ex (tests and sweeps). */
enum { SDFL_GN_AUTO = 0, SDFL_GN_RESIDENT = 1, SDFL_GN_SPLIT = 2, SDFL_GN_REGISTER = 3 };

const char *sdfl_version(void);
const char *sdfl_status_string(int status);
/* cudaError_t of the most recent failing CUDA call on this host thread, and its text. */
int sdfl_last_cuda_error(void);
const char *sdfl_last_cuda_error_string(void);
/* Number of kernels this library has enqueued since load (all threads). */
long long sdfl_launch_count(void);

/* ------------------------------------------------------------------------------------------
 * Fused operators (one launch where the reference needs three or four)
 * ---------------------------------------------------------------------------------------- */

/* GroupNorm with optional fused SiLU on an NCHW tensor [batch, channels, hw].
 * Replaces GroupNorm::forward (NN/GroupNorm.cpp:68-170: local_reduction_mean +
 * local_reduction_variance + group_norm, K/group_norm.cl:1-76) and, with fuse_silu != 0, the
 * silu launch that follows it at every call site (K/util.cl:124-134; NN/ResBlock.cpp:125-142,
 * M/UNetModel.cpp:1797-1809, M/Decoder.cpp:523-536).
 * Same group semantics (group g of an image = channels [g*C/G, (g+1)*C/G), biased variance,
 * eps inside the square root).  Added: the batch dimension (the reference is batch-1 and would
 * index gamma out of range on a batched buffer, K/group_norm.cl:71).
 * The reference demands group size % 64 == 0 (NN/GroupNorm.cpp:89-93); this does not.
 * workspace: scratch of at least sdfl_groupnorm_workspace_bytes() bytes (may be NULL when that
 * is 0, i.e. when the shared-memory-resident path applies). */
int sdfl_groupnorm_forward(const void *in, void *out, const float *gamma, const float *beta,
                           int64_t batch, int64_t channels, int64_t hw, int64_t num_groups,
                           float eps, int fuse_silu, int dtype, void *workspace,
                           size_t workspace_bytes, void *stream);

size_t sdfl_groupnorm_workspace_bytes(int64_t batch, int64_t channels, int64_t hw,
                                      int64_t num_groups, int dtype);

/* Same, with the device path and cluster size (resident; register: 1, 2, 4 or 8 CTAs per
 * slab) / chunk count (split) forced; 0 = automatic.  A forced path that cannot run the shape
 * returns SDFL_ERR_UNSUPPORTED.
 * The workspace must then hold sdfl_groupnorm_workspace_bytes_ex() bytes. */
int sdfl_groupnorm_forward_ex(const void *in, void *out, const float *gamma, const float *beta,
                              int64_t batch, int64_t channels, int64_t hw, int64_t num_groups,
                              float eps, int fuse_silu, int dtype, void *workspace,
                              size_t workspace_bytes, int path, int cluster_or_splits, void *stream);

size_t sdfl_groupnorm_workspace_bytes_ex(int64_t batch, int64_t channels, int64_t hw,
                                         int64_t num_groups, int dtype, int path,
                                         int cluster_or_splits);

/* Which path sdfl_groupnorm_forward would take for 16-byte aligned buffers:
 * plan[0] = path, [1] = cluster size, [2] = threads per CTA, [3] = chunks per slab (split),
 * [4] = dynamic shared memory bytes per CTA, [5] = workspace bytes, [6] = persistent clusters
 * launched (resident), [7] = 16-byte vectors per shared-memory ring chunk (resident). */
int sdfl_groupnorm_plan(int64_t batch, int64_t channels, int64_t hw, int64_t num_groups, int dtype,
                        int path, int cluster_or_splits, int64_t plan[8]);

/* GroupNorm(+SiLU) of a list of independent tensors in ONE launch.  The reference normalises one
 * tensor per GroupNorm::forward call (NN/GroupNorm.cpp:68-170) and runs its call sites one after
 * another on one queue (NN/ResBlock.cpp:125-142, M/Decoder.cpp:523-536); tensors that do not depend
 * on each other -- the images of a batch shard held as separate buffers, the conditional and
 * unconditional halves of a guidance pair, the layers of a benchmark step -- can be handed over
 * together here.  Every (image, group) slab of every tensor becomes one item of a work list that a
 * single grid of resident CTAs walks (largest slabs first), so the launch, first-data and drain
 * latencies are paid once and small tensors fill the SMs that large ones leave idle.  Results per
 * tensor are those of sdfl_groupnorm_forward within the rounding of a different summation order.
 * All tensors share dtype and fuse_silu; each has its own shape, eps and weights.
 * Requirements per tensor: 16-byte aligned in/out, hw * element size a multiple of 16, slabs
 * (channels / num_groups * hw elements) of at least 512 bytes; at most SDFL_GN_MULTI_MAX non-empty
 * tensors.  Otherwise SDFL_ERR_UNSUPPORTED is returned and nothing is launched (call
 * sdfl_groupnorm_forward per tensor).  out == in is allowed per tensor; different tensors must not
 * overlap (SDFL_ERR_OVERLAP).
 * workspace: NULL, or sdfl_groupnorm_multi_workspace_bytes() bytes of device memory that were
 * zero-filled once before their first use (the kernel leaves them ready for the next launch).
 * The CTAs that share a slab exchange their partial moments through it and the work list's
 * counter lives there.  With NULL a buffer inside the library is used, shared by all such calls
 * on the device: pass an own workspace per stream when two of these launches could overlap on the
 * GPU.  The grid is sized to be resident as a whole (its CTAs wait for each other, every wait
 * bounded): run it on a device that is not oversubscribed by other long-running kernels.  If a wait
 * does run out, sdfl_device_status() reports bit 0 and the launch's output is not valid; clearing the
 * status also resets the library's own buffer, and a caller's workspace must be zero-filled again
 * before its next use. */
enum { SDFL_GN_MULTI_MAX = 8 };
typedef struct sdfl_gn_tensor {
    const void *in;
    void *out;
    const float *gamma;
    const float *beta;
    int64_t batch, channels, hw, num_groups;
    float eps;
} sdfl_gn_tensor;
size_t sdfl_groupnorm_multi_workspace_bytes(void);
int sdfl_groupnorm_forward_multi(const sdfl_gn_tensor *tensors, int count, int fuse_silu, int dtype,
                                 void *workspace, size_t workspace_bytes, void *stream);
/* The same with tuning knobs (tests, sweeps, profiling); knobs = 0 is the automatic plan.
 * knobs: bits 0-7 CTAs per gang (a gang works on one large slab, or on several small ones at once);
 * 8-9 team size per tensor (1 = the whole gang on every slab, 2 = by slab size); bit 10 cooperative
 * launch; bit 11 / bit 30 force / forbid that half of the gangs start at the small end of the list;
 * 12-13 the share of a slab per CTA that team sizes aim at, in units of 128 KB; 14-15 item order
 * (1 = static, 2 = drawn from a counter); 16-23 ring chunk in KB (16 or 32); 24-27 ring slots; 28-29
 * chunks held between the passes + 1.
 * d_trace: NULL, or device memory of grid * 16 64-bit words that receives, per CTA, nanosecond time
 * stamps (start, barriers set up, first chunk landed, first slab's moments done, its statistics
 * known, its stores issued, all slabs done, first copy issued), the SM number, the number of
 * slabs handled and the time one thread spent waiting for statistics / for chunks in either pass.
 * plan (optional, host): {CTAs per gang, grid size, team sizes of the first four tensors (8 bits
 * each), shared memory per CTA}. */
int sdfl_groupnorm_forward_multi_ex(const sdfl_gn_tensor *tensors, int count, int fuse_silu, int dtype,
                                    void *workspace, size_t workspace_bytes, int knobs,
                                    unsigned long long *d_trace, int plan[4], void *stream);

/* GroupNorm(+SiLU) for callers that may not allocate device memory and therefore cannot supply
 * the workspace sdfl_groupnorm_forward may ask for.  (No counterpart in the reference: it
 * creates and releases its mean/variance buffers inside every forward call,
 * NN/GroupNorm.cpp:95-103,164-165.)
 * Who needs it: a host application that hands all device memory to its own pools at start-up
 * and forbids later cudaMalloc calls, plugins running inside such a host, and latency-critical
 * threads that cannot take the device-wide synchronisation an allocator call may imply.
 * It always runs the two-kernel split path; the per-chunk (mean, M2) scratch lives in a fixed
 * 64 KiB array inside the library image (resident on every device that loads the library, for
 * the life of the process).  This call and everything under it makes no cudaMalloc / cudaFree /
 * allocating-library call.
 * Limit: batch * num_groups * chunks-per-slab * 8 bytes <= 65536 (e.g. batch 8 x 32 groups with
 * up to 32 chunks per slab); larger problems return SDFL_ERR_WORKSPACE and touch nothing.
 * The first call on a device looks up the array's device address (once per device, with that
 * device current); make that first call before starting any stream capture on the device.
 * The address is remembered per device ordinal for the life of the process: it belongs to the
 * device's primary context, so do not call cudaDeviceReset between calls and do not use this
 * entry point from another (driver-API) context on the same device.
 * All calls on a device share the one array and it keeps the previous call's values: nothing
 * in it needs clearing (each call overwrites every entry it later reads), but two calls whose
 * kernels can overlap on the GPU (different streams, no dependency) race on it -- order them.
 * Results equal sdfl_groupnorm_forward_ex(..., SDFL_GN_SPLIT, 0, ...) bit for bit. */
int sdfl_groupnorm_forward_noalloc(const void *in, void *out, const float *gamma, const float *beta,
                                   int64_t batch, int64_t channels, int64_t hw, int64_t num_groups,
                                   float eps, int fuse_silu, int dtype, void *stream);

/* GroupNorm(+SiLU) of x + e, where e[n, c] is a per-(image, channel) addend of the storage type
 * ([batch, channels]): the time-embedding broadcast add that precedes the out-norm of a ResBlock,
 * fused into the norm.  Replaces chunkwise_add (K/util.cl:136-148, launched at
 * NN/ResBlock.cpp:188-199) + GroupNorm::forward (NN/ResBlock.cpp:222) + silu (:225-231): six
 * more tensor passes saved on top of the plain fusion.  The sum is formed in fp32 and is not
 * written back.  Workspace as for sdfl_groupnorm_forward. */
int sdfl_groupnorm_bias_forward(const void *in, const void *channel_bias, void *out, const float *gamma,
                                const float *beta, int64_t batch, int64_t channels, int64_t hw,
                                int64_t num_groups, float eps, int fuse_silu, int dtype, void *workspace,
                                size_t workspace_bytes, void *stream);

/* The same with the path and tuning knob of sdfl_groupnorm_forward_ex (tests and sweeps). */
int sdfl_groupnorm_bias_forward_ex(const void *in, const void *channel_bias, void *out,
                                   const float *gamma, const float *beta, int64_t batch,
                                   int64_t channels, int64_t hw, int64_t num_groups, float eps,
                                   int fuse_silu, int dtype, void *workspace, size_t workspace_bytes,
                                   int path, int cluster_or_splits, void *stream);

/* GroupNorm(+SiLU) of an NCHW tensor written channels-last: out[n][p][c] ([batch, hw, channels]).
 * Replaces GroupNorm::forward followed by permute3D__0_2_1 with global size {1, channels, hw}
 * (NN/SpatialTransformer.cpp:127-140).  Slabs up to 48 KB in 16-byte aligned tensors: one kernel,
 * one read and one write of the tensor.  Otherwise two kernels: the statistics (one read), then a
 * tiled normalise-and-transpose over all SMs (a second read, from L2 for UNet sizes, and the
 * write) -- against three reads and two writes for the reference's sequence.  The workspace
 * (sdfl_groupnorm_nhwc_workspace_bytes, a few KB) holds the per-chunk moments.  in == out is an
 * error: a transpose cannot run in place. */
size_t sdfl_groupnorm_nhwc_workspace_bytes(int64_t batch, int64_t channels, int64_t hw,
                                           int64_t num_groups, int dtype);
int sdfl_groupnorm_nhwc_forward(const void *in, void *out, const float *gamma, const float *beta,
                                int64_t batch, int64_t channels, int64_t hw, int64_t num_groups,
                                float eps, int fuse_silu, int dtype, void *workspace,
                                size_t workspace_bytes, void *stream);

/* K/util.cl:47-64 permute3D__0_2_1(src, dst) with global size {I, J, K}: dst[i][k][j] = src[i][j][k]
 * (NN/SpatialTransformer.cpp:131-134 with {1, C, HW}; :154-157 with {1, HW, C}). */
int sdfl_permute3D__0_2_1(const void *src, void *dst, int64_t I, int64_t J, int64_t K, int dtype,
                          void *stream);

/* dst[i][k][j] = src[i][j][k] + residual[i][k][j]: the second permute of a SpatialTransformer
 * block fused with the elemwise_add that follows it (NN/SpatialTransformer.cpp:154-171).
 * residual may be dst (in-place accumulate); src may not overlap dst. */
int sdfl_permute_add(const void *src, const void *residual, void *dst, int64_t I, int64_t J, int64_t K,
                     int dtype, void *stream);

/* K/up_sample.cl:1-18 up_sample_nearest(input, output, scale) with global size {channels, height,
 * height} (NN/UpSample.cpp:93-102): output[c][i*scale+di][j*scale+dj] = input[c][i][j].  Width
 * is a separate argument here; a batch is folded into `channels`. */
int sdfl_up_sample_nearest(const void *input, void *output, int64_t channels, int64_t height, int64_t width,
                           int64_t scale, int dtype, void *stream);

/* M/UNetModel.cpp:1960-1990 concat_buffer(input1, input2, output): output = input1 followed by
 * input2.  With batch > 1 each image is [n1 | n2] elements (a concatenation along the channels of
 * NCHW tensors with n = channels * hw). */
int sdfl_concat_buffer(const void *input1, const void *input2, void *output, int64_t batch, int64_t n1,
                       int64_t n2, int dtype, void *stream);

/* GroupNorm(+SiLU) of the channel-wise concatenation of in1 [batch, channels1, hw] and in2
 * [batch, channels2, hw] without materialising it: concat_buffer (M/UNetModel.cpp:1960-1990) in
 * front of the first norm of an output-block ResBlock, fused into the norm's loads.  out is
 * [batch, channels1 + channels2, hw].  gamma/beta have channels1 + channels2 entries.  Falls back
 * to concat + in-place norm when the tensors are not 16-byte aligned or hw * element size is not
 * a multiple of 16.  Workspace as for sdfl_groupnorm_forward with the summed channel count. */
int sdfl_groupnorm_concat_forward(const void *in1, int64_t channels1, const void *in2, int64_t channels2,
                                  void *out, const float *gamma, const float *beta, int64_t batch,
                                  int64_t hw, int64_t num_groups, float eps, int fuse_silu, int dtype,
                                  void *workspace, size_t workspace_bytes, void *stream);

/* K/util.cl:150-187 softmax(input, output, __local sums, __local cache, chunkSize) launched with one
 * work-group per row (NN/CrossAttention.cpp:365-378, NN/AttnBlock.cpp:196-207):
 * output[r][i] = exp(input[r][i]) / sum_i exp(input[r][i]) over rows of chunk_size elements.
 * The row maximum is subtracted before exp (same quotient; the reference overflows above 88).
 * output == input allowed, as the reference's callers do. */
int sdfl_softmax(const void *input, void *output, int64_t rows, int64_t chunk_size, int dtype, void *stream);

/* K/multi_head_attention.cl:28-54 local_softmax(input, output, __local reductionSums) launched with one
 * work-group of CONTEXT_LENGTH = 77 work-items per row over numHeads * 77 rows, in place
 * (NN/MultiHeadAttention.cpp:213-225): the text encoder's attention softmax, after the causal mask
 * (-inf above the diagonal) has been added.  Same function as sdfl_softmax, kept under the
 * reference kernel's name; row_len is the work-group size of the reference launch.  Masked
 * entries come out as exact zeros. */
int sdfl_local_softmax(const void *input, void *output, int64_t rows, int64_t row_len, int dtype, void *stream);

/* K/util.cl:136-148  chunkwise_add(A, chunk, C, chunk_size) over n work-items:
 * C[i] = A[i] + chunk[i / chunk_size]; C may be A (NN/ResBlock.cpp:188-191). */
int sdfl_chunkwise_add(const void *A, const void *chunk, void *C, int64_t n, int64_t chunk_size,
                       int dtype, void *stream);

/* LayerNorm over the last dimension of [rows, dim].
 * Replaces LayerNorm::forward (NN/LayerNorm.cpp:66-162; K/layer_norm.cl:1-78).  eps is an
 * argument; the reference fixes it at 1e-5 (K/layer_norm.cl:58).  The reference demands
 * dim % 64 == 0 (NN/LayerNorm.cpp:61-63); this does not. */
int sdfl_layernorm_forward(const void *in, void *out, const float *gamma, const float *beta,
                           int64_t rows, int64_t dim, float eps, int dtype, void *stream);

/* Residual add fused into the LayerNorm that follows it: sum_out = a + b, out = LayerNorm(sum_out).
 * Replaces the elemwise_add launch + LayerNorm::forward pairs of the transformer block
 * (NN/BasicTransformerBlock.cpp:126-136 and :149-158: the sum is kept as the next residual, the
 * normalised tensor feeds the next attention / feed-forward).  Five tensor passes become four.
 * sum_out may be a or b (the reference adds in place); out must not overlap sum_out.  The sum is
 * rounded to the storage type before it is normalised, exactly as the two separate steps do. */
int sdfl_add_layernorm_forward(const void *a, const void *b, void *sum_out, void *out,
                               const float *gamma, const float *beta, int64_t rows, int64_t dim,
                               float eps, int dtype, void *stream);

/* Token + position embedding: out[b,t,:] = table[ids[b,t],:] + pos[t,:].
 * Replaces TextEncoder::createTokenEmbeddingBuffer (M/TextEncoder.cpp:105-125, a host loop
 * over a host-resident table) followed by elemwise_add with the positional table
 * (M/TextEncoder.cpp:141-151).  ids are int64 like the reference's std::vector<long>.
 * d_status (device int, may be NULL): bit 0 is raised if an id is outside [0, vocab); such rows
 * are written as zeros (the reference reads out of bounds instead). */
int sdfl_token_embedding(const int64_t *ids, const void *table, const void *pos, void *out,
                         int64_t batch, int64_t seq_len, int64_t dim, int64_t vocab, int dtype,
                         int *d_status, void *stream);

/* Sinusoidal timestep embedding: out[n, :] = [cos(t[n] * f_i) | sin(t[n] * f_i)],
 * f_i = exp(-log(max_period) * i / (dim/2)).
 * Replaces UNetModel::createTimestepEmbedding (M/UNetModel.cpp:1935-1958; host code, one
 * timestep); here t is a device array of `batch` int64 timesteps. */
int sdfl_timestep_embedding(const int64_t *t, void *out, int64_t batch, int64_t dim,
                            float max_period, int dtype, void *stream);

/* ------------------------------------------------------------------------------------------
 * Per-kernel entry points: one per reference __kernel, same pointer order; NDRange extents
 * become trailing integer arguments and the __local scratch argument is dropped.
 * ---------------------------------------------------------------------------------------- */

/* K/group_norm.cl:1-27 and K/layer_norm.cl:1-27  local_reduction_mean(input, output, scratch,
 * reductionSize) over `groups` work-groups: output[g] = mean of input[g*n, (g+1)*n) with
 * n = group_elems (= 64 * reductionSize in the reference). */
int sdfl_local_reduction_mean(const void *input, float *output, int64_t groups, int64_t group_elems,
                              int dtype, void *stream);

/* K/group_norm.cl:29-57  local_reduction_variance(input, mean, output, scratch, reductionSize):
 * biased variance around the given mean. */
int sdfl_local_reduction_variance(const void *input, const float *mean, float *output,
                                  int64_t groups, int64_t group_elems, int dtype, void *stream);

/* K/group_norm.cl:59-76  group_norm(input, mean, variance, weight, bias, groupSize,
 * channelSize, epsilon, output) over n work-items.  weight/bias index = (i / channelSize) %
 * num_channels, which equals the reference's i / channelSize for a single image. */
int sdfl_group_norm(const void *input, const float *mean, const float *variance,
                    const float *weight, const float *bias, int64_t groupSize, int64_t channelSize,
                    float epsilon, void *output, int64_t n, int64_t num_channels, int dtype,
                    void *stream);

/* K/layer_norm.cl:63-78  layer_norm(input, mean, variance, weight, bias, chunkSize, output)
 * over n work-items; epsilon is the kernel file's constant in the reference. */
int sdfl_layer_norm(const void *input, const float *mean, const float *variance,
                    const float *weight, const float *bias, int64_t chunkSize, void *output,
                    int64_t n, float epsilon, int dtype, void *stream);

/* K/geglu.cl:1-25  gelu_multiply(AB, dst) over the 2-D range {rows, D} (NN/GEGLU.cpp:71-77):
 * dst[r, j] = AB[r, j] * gelu_erf(AB[r, D + j]); AB is [rows, 2D], dst is [rows, D]. */
int sdfl_gelu_multiply(const void *AB, void *dst, int64_t rows, int64_t D, int dtype, void *stream);

/* K/util.cl:104-122  gelu(src, dst): x * 0.5 * (1 + erf(x / sqrt 2)) over n work-items. */
int sdfl_gelu(const void *src, void *dst, int64_t n, int dtype, void *stream);

/* K/util.cl:124-134  silu(src, dst): x / (1 + exp(-x)) over n work-items. */
int sdfl_silu(const void *src, void *dst, int64_t n, int dtype, void *stream);

/* x / (1 + exp(-1.702 x)).  The reference has no quick_gelu kernel; this follows silu's form. */
int sdfl_quick_gelu(const void *src, void *dst, int64_t n, int dtype, void *stream);

/* K/util.cl:1-12  elemwise_add(A, B, C): C = A + B over n work-items. */
int sdfl_elemwise_add(const void *A, const void *B, void *C, int64_t n, int dtype, void *stream);

/* ------------------------------------------------------------------------------------------
 * Operator objects: the reference's classes as opaque C handles, for binders that cannot use the
 * C++ wrapper of sdfl_operators.hpp (the reference side is JNI).
 *   GroupNorm(ctx, queue, num_groups, num_channels, eps, weight_name, bias_name, kernel); init();
 *   forward(in, out, n_wait, wait, event)                         NN/GroupNorm.h:15-29
 *   LayerNorm(ctx, queue, dim, weight_name, bias_name, kernel)    NN/LayerNorm.h:16-28
 *   GEGLU(ctx, queue, in_features, out_features, ...)             NN/GEGLU.h:18-36
 * create = constructor + init(); *_op_forward = forward(); destroy = the destructor.  The OpenCL
 * context / queue / kernel-holder arguments are gone and a stream replaces the event list.
 * Ownership follows the reference: the caller owns input and output; gamma and beta are DEVICE
 * arrays that the caller loads (the reference's .npy file names are app glue) and must keep alive
 * as long as the handle; the handle owns its metadata and a scratch buffer that is allocated at
 * create time for the stated maximum shape and never inside forward (the reference allocates and
 * frees its mean / variance buffers in every forward call, NN/GroupNorm.cpp:95-103,164-165).
 * A handle belongs to the device that was current at create time; forward with another device
 * current, or with a shape beyond the stated maximum that needs more scratch than was reserved,
 * returns SDFL_ERR_INVALID_VALUE / SDFL_ERR_WORKSPACE.  One handle may be used from one host thread
 * at a time (calls on different streams would share its scratch).
 * ---------------------------------------------------------------------------------------- */
typedef struct sdfl_groupnorm sdfl_groupnorm;
typedef struct sdfl_layernorm sdfl_layernorm;
typedef struct sdfl_geglu sdfl_geglu;

/* num_channels % num_groups != 0 -> SDFL_ERR_INVALID_VALUE (the reference throws at
 * NN/GroupNorm.cpp:83-87).  max_batch / max_hw / max_dtype: the largest [batch, channels, hw] tensor
 * of storage type max_dtype that forward will be given (sizes the scratch). */
int sdfl_groupnorm_create(sdfl_groupnorm **op, int64_t num_groups, int64_t num_channels, float eps,
                          const float *d_gamma, const float *d_beta, int fuse_silu, int64_t max_batch,
                          int64_t max_hw, int max_dtype);
/* in / out: [batch, num_channels, hw] device tensors; out may be in (NN/ResBlock.cpp:222). */
int sdfl_groupnorm_op_forward(sdfl_groupnorm *op, const void *in, void *out, int64_t batch, int64_t hw,
                              int dtype, void *stream);
int sdfl_groupnorm_destroy(sdfl_groupnorm *op);

int sdfl_layernorm_create(sdfl_layernorm **op, int64_t dim, float eps, const float *d_gamma,
                          const float *d_beta);
/* in / out: [rows, dim] device tensors; out may be in. */
int sdfl_layernorm_op_forward(sdfl_layernorm *op, const void *in, void *out, int64_t rows, int dtype,
                              void *stream);
int sdfl_layernorm_destroy(sdfl_layernorm *op);

/* The gelu_multiply stage of GEGLU::forward (NN/GEGLU.cpp:71-77); the Linear in front of it
 * (NN/GEGLU.cpp:32-34) is a dense layer and stays with the caller.  weight_shape receives the
 * reference's public weightShape member {2 * out_features, in_features} (NN/GEGLU.h:36). */
int sdfl_geglu_create(sdfl_geglu **op, int64_t in_features, int64_t out_features);
int sdfl_geglu_weight_shape(const sdfl_geglu *op, int64_t weight_shape[2]);
/* projected: [rows, 2 * out_features]; out: [rows, out_features]. */
int sdfl_geglu_op_forward(sdfl_geglu *op, const void *projected, void *out, int64_t rows, int dtype,
                          void *stream);
int sdfl_geglu_destroy(sdfl_geglu *op);

/* ------------------------------------------------------------------------------------------
 * Device status and host-buffer convenience path
 * ---------------------------------------------------------------------------------------- */

/* Reads (and, if clear != 0, clears) the sticky status word of the GroupNorm kernels on the
 * current device.  Bit 0: a bounded wait on a bulk copy ran out -- results of that launch are
 * not valid.  Synchronises `stream`. */
int sdfl_device_status(unsigned int *value, int clear, void *stream);

/* Failure-detection self-test.  Every wait inside the kernels (on a bulk copy, or on the
 * cluster peers' moments) is bounded; when one runs out the kernel raises the status word and
 * finishes instead of hanging.  This enqueues a one-warp kernel whose wait can never be
 * satisfied, with `limit_cycles` (clamped to [1e3, 2e9]) as its bound, so that a caller can
 * check the whole chain -- the wait ends, sdfl_device_status() reports bit 0, later launches
 * still work -- without faulting or hanging the device. */
int sdfl_selftest_bounded_wait(long long limit_cycles, void *stream);

/* Host-buffer GroupNorm(+SiLU): what a caller holding host tensors uses (the reference's
 * models take and return std::vector<float>, JNI boundary).  A pipeline object owns `depth`
 * device staging slots and streams, created once; forward_host copies image slabs in,
 * normalises, and copies out, overlapping the three, and returns when h_out is complete.
 * Host buffers should be page-locked (sdfl_host_alloc) for the copies to overlap.  gamma and
 * beta are DEVICE pointers, as everywhere else.  A pipeline belongs to the device that was
 * current when it was created (calls made with another device current are refused with
 * SDFL_ERR_INVALID_VALUE) and to one host thread at a time. */
typedef struct sdfl_host_pipeline sdfl_host_pipeline;

int sdfl_host_pipeline_create(sdfl_host_pipeline **pipe, size_t max_slot_bytes, int depth);
int sdfl_host_pipeline_destroy(sdfl_host_pipeline *pipe);
int sdfl_groupnorm_forward_host(sdfl_host_pipeline *pipe, const void *h_in, void *h_out,
                                const float *gamma, const float *beta, int64_t batch,
                                int64_t channels, int64_t hw, int64_t num_groups, float eps,
                                int fuse_silu, int dtype);
/* The same without the final wait: enqueues the copies and kernels of one tensor on the
 * pipeline's streams and returns; several tensors can be queued back to back and
 * sdfl_host_pipeline_sync() waits for all of them (h_out buffers are complete after it). */
int sdfl_groupnorm_forward_host_async(sdfl_host_pipeline *pipe, const void *h_in, void *h_out,
                                      const float *gamma, const float *beta, int64_t batch,
                                      int64_t channels, int64_t hw, int64_t num_groups, float eps,
                                      int fuse_silu, int dtype);
int sdfl_host_pipeline_sync(sdfl_host_pipeline *pipe);
int sdfl_host_alloc(void **h_ptr, size_t bytes);
int sdfl_host_free(void *h_ptr);

#ifdef __cplusplus
}
#endif

#endif /* SDFL_H_ */
