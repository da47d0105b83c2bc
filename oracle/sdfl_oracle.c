/* TEST INFRASTRUCTURE ONLY -- the CPU checker for the CUDA kernels, never part of the
 * product path.  Only tests/, __graft_entry__.smoke() and the cpu-baseline / reference legs of
 * bench.py may load this library.
 *
 * A plain-C restatement of the algorithm of the reference's fused-layer path: the OpenCL C
 * kernels of group_norm.cl, layer_norm.cl, geglu.cl and three kernels of util.cl, and the two
 * host functions that build the token and timestep embeddings.  Every function names the
 * reference file:line it follows (paths are inside the reference project).
 *
 * Arithmetic is fp32 with the reference's operation order.  A work-group of 64 work-items
 * that meets barriers is written as phase-ordered loops: the order of every floating-point
 * addition is fixed by the kernel source (strided per-item sums, then a 6-step tree), so the
 * loops give the same bits as any conforming execution of the kernel as long as the compiler
 * does not contract a*b+c (build with -ffp-contract=off).
 *
 * PINNING: the reference ships no golden vector for this path (its test tensors are not in
 * its repository).  This file is instead pinned against the reference's own kernel source
 * compiled as C++ (oracle/_ref, built by `make ref`): tests/test_oracle_pin.py demands
 * bit-equality between the two wherever the reference accepts the shape, and
 * tests/golden/ holds outputs of oracle/_ref for machines where the reference is absent.
 * Not pinned by the reference (it has no such code): quick_gelu, shapes whose group/row size
 * is not a multiple of 64, and batch > 1 for GroupNorm (defined as one reference run per image).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define WORK_GROUP_SIZE 64 /* nn/GroupNorm.cpp:13, nn/LayerNorm.cpp:11 */
#define SQRT1_2_F 0.70710678118654752440f /* OpenCL M_SQRT1_2_F */

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* One work-group of local_reduction_mean / local_reduction_variance.
 * group_norm.cl:1-27 and :29-57 (same text in layer_norm.cl:1-27, :29-56).
 * Item l adds x[l], x[l+64], x[l+128] ... in that order (group_norm.cl:11-14); the partials
 * are folded by offset 32,16,...,1 (:17-22); the root divides by the element count (:25).
 * `n` need not be a multiple of 64 here: items past the ragged tail simply add fewer terms
 * (the reference refuses such sizes at nn/GroupNorm.cpp:89-93, so that case is an extension). */
static float group_sum(const float *x, size_t n, int centered, float mean) {
    float partial[WORK_GROUP_SIZE];
    for (int l = 0; l < WORK_GROUP_SIZE; ++l) {
        float sum = 0.0f;
        for (size_t j = (size_t)l; j < n; j += WORK_GROUP_SIZE) {
            if (centered) {
                sum += (x[j] - mean) * (x[j] - mean); /* group_norm.cl:42 */
            } else {
                sum += x[j]; /* group_norm.cl:13 */
            }
        }
        partial[l] = sum;
    }
    for (int offset = WORK_GROUP_SIZE / 2; offset > 0; offset /= 2) {
        for (int l = 0; l < offset; ++l) partial[l] += partial[l + offset];
    }
    return partial[0];
}

/* group_norm.cl:1-27: out[w] = sum(in[w*n .. (w+1)*n)) / n with n = 64 * reductionSize. */
void oracle_local_reduction_mean(const float *in, float *out, size_t groups, size_t n) {
#pragma omp parallel for schedule(static)
    for (long w = 0; w < (long)groups; ++w) {
        out[w] = group_sum(in + (size_t)w * n, n, 0, 0.0f) / (float)n;
    }
}

/* group_norm.cl:29-57: biased variance, divisor n (comment at :54). */
void oracle_local_reduction_variance(const float *in, const float *mean, float *out, size_t groups,
                                     size_t n) {
#pragma omp parallel for schedule(static)
    for (long w = 0; w < (long)groups; ++w) {
        out[w] = group_sum(in + (size_t)w * n, n, 1, mean[w]) / (float)n;
    }
}

/* util.cl:124-134 */
static inline float silu_f(float x) {
    float temp = expf(-x);
    temp = 1.0f / (1.0f + temp);
    return x * temp;
}

/* util.cl:104-122 */
static inline float gelu_f(float x) {
    float temp = x * SQRT1_2_F;
    temp = 1.0f + erff(temp);
    return x * 0.5f * temp;
}

/* No reference kernel exists for quick_gelu; written in the form of silu (util.cl:124-134)
 * with the 1.702 slope: x * 1/(1 + exp(-1.702 x)).  Not pinned by the reference. */
static inline float quick_gelu_f(float x) {
    float temp = expf(-1.702f * x);
    temp = 1.0f / (1.0f + temp);
    return x * temp;
}

/* group_norm.cl:59-76 applied to one image of `n` elements:
 * g = i / groupSize, c = i / channelSize, y = fma((x - mean[g]) / sqrt(var[g] + eps), w[c], b[c]). */
static void group_norm_apply(const float *in, const float *mean, const float *var, const float *w,
                             const float *b, size_t groupSize, size_t channelSize, float eps,
                             float *out, size_t n, int apply_silu) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; ++i) {
        size_t g = (size_t)i / groupSize;
        size_t c = (size_t)i / channelSize;
        float temp = in[i] - mean[g];
        temp /= sqrtf(var[g] + eps);
        float y = fmaf(temp, w[c], b[c]);
        out[i] = apply_silu ? silu_f(y) : y; /* silu: separate launch at nn/ResBlock.cpp:136-142 */
    }
}

/* GroupNorm::forward (nn/GroupNorm.cpp:68-170) once per image; the reference is batch-1
 * (UNetModel.cpp:1073) and its kernel indexes weight[i / channelSize] with no "% C"
 * (group_norm.cl:71), so a batch is defined as B independent runs.  in/out: [batch, C, hw]
 * (NCHW with hw = H*W), w/b: [C].  mean_out/var_out: [batch*G] or NULL.
 * Returns -1 if C % G != 0 (the reference's input_size % weightSize check covers the rest). */
int oracle_group_norm(const float *in, float *out, const float *w, const float *b, size_t batch,
                      size_t C, size_t hw, size_t G, float eps, int apply_silu, float *mean_out,
                      float *var_out) {
    if (G == 0 || C == 0 || C % G != 0) return -1;
    const size_t per_image = C * hw;
    const size_t groupSize = per_image / G; /* nn/GroupNorm.cpp:80 */
    float *mean = (float *)malloc(sizeof(float) * G);
    float *var = (float *)malloc(sizeof(float) * G);
    if (!mean || !var) { free(mean); free(var); return -3; }
    for (size_t n = 0; n < batch; ++n) {
        const float *x = in + n * per_image;
        oracle_local_reduction_mean(x, mean, G, groupSize);
        oracle_local_reduction_variance(x, mean, var, G, groupSize);
        group_norm_apply(x, mean, var, w, b, groupSize, hw /* channelSize, :130 */, eps,
                         out + n * per_image, per_image, apply_silu);
        if (mean_out) memcpy(mean_out + n * G, mean, sizeof(float) * G);
        if (var_out) memcpy(var_out + n * G, var, sizeof(float) * G);
    }
    free(mean);
    free(var);
    return 0;
}

/* LayerNorm::forward (nn/LayerNorm.cpp:66-162) + layer_norm.cl:63-78.  The reference's eps is
 * the constant 1e-5 of layer_norm.cl:58; here it is an argument with that default upstream. */
int oracle_layer_norm(const float *in, float *out, const float *w, const float *b, size_t rows,
                      size_t D, float eps, float *mean_out, float *var_out) {
    if (D == 0) return -1;
    float *mean = (float *)malloc(sizeof(float) * (rows ? rows : 1));
    float *var = (float *)malloc(sizeof(float) * (rows ? rows : 1));
    if (!mean || !var) { free(mean); free(var); return -3; }
    oracle_local_reduction_mean(in, mean, rows, D);
    oracle_local_reduction_variance(in, mean, var, rows, D);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)(rows * D); ++i) {
        size_t k = (size_t)i % D; /* layer_norm.cl:72 */
        size_t r = (size_t)i / D; /* layer_norm.cl:73 */
        float temp = in[i] - mean[r];
        temp /= sqrtf(var[r] + eps);
        out[i] = fmaf(temp, w[k], b[k]);
    }
    if (mean_out) memcpy(mean_out, mean, sizeof(float) * rows);
    if (var_out) memcpy(var_out, var, sizeof(float) * rows);
    free(mean);
    free(var);
    return 0;
}

/* geglu.cl:1-25 over the 2-D range {rows, D} of nn/GEGLU.cpp:75:
 * a = AB[r*2D + j], b = AB[r*2D + D + j], dst[r*D + j] = a * (b * 0.5 * (1 + erf(b / sqrt 2))). */
void oracle_gelu_multiply(const float *AB, float *dst, size_t rows, size_t D) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) {
        for (size_t j = 0; j < D; ++j) {
            const float a = AB[(size_t)r * D * 2 + j];
            const float bb = AB[(size_t)r * D * 2 + j + D];
            float temp = bb * SQRT1_2_F;
            temp = 1.0f + erff(temp);
            temp = bb * 0.5f * temp;
            dst[(size_t)r * D + j] = a * temp;
        }
    }
}

void oracle_gelu(const float *src, float *dst, size_t n) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; ++i) dst[i] = gelu_f(src[i]);
}

void oracle_silu(const float *src, float *dst, size_t n) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; ++i) dst[i] = silu_f(src[i]);
}

void oracle_quick_gelu(const float *src, float *dst, size_t n) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; ++i) dst[i] = quick_gelu_f(src[i]);
}

/* util.cl:1-12 */
void oracle_elemwise_add(const float *A, const float *B, float *C, size_t n) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; ++i) C[i] = A[i] + B[i];
}

/* up_sample.cl:1-18 with global size {channels, H, H} (nn/UpSample.cpp:93-102), generalised to
 * H x W planes: out[c][i*scale + di][j*scale + dj] = in[c][i][j] for di, dj < scale. */
void oracle_up_sample_nearest(const float *in, float *out, size_t channels, size_t H, size_t W, size_t scale) {
#pragma omp parallel for schedule(static) collapse(2)
    for (long c = 0; c < (long)channels; ++c)
        for (long i = 0; i < (long)H; ++i)
            for (size_t j = 0; j < W; ++j) {
                const float v = in[((size_t)c * H + (size_t)i) * W + j];
                for (size_t di = 0; di < scale; ++di)
                    for (size_t dj = 0; dj < scale; ++dj)
                        out[((size_t)c * scale * H + ((size_t)i * scale + di)) * scale * W + (j * scale + dj)] = v;
            }
}

/* util.cl:150-187 softmax with one work-group of 64 items per row (nn/CrossAttention.cpp:360-378):
 * item l adds exp(x[l]), exp(x[l+64]), ... in that order and keeps each exp in `cache` (:163-169);
 * the partial sums are folded by the halving loop of :172-180 (for 64 items: offsets 32..1, the
 * odd-size bookkeeping never triggers); every element is cache[i] / sums[0] (:184-186).  No
 * maximum is subtracted, as in the reference.  out may be in. */
void oracle_softmax(const float *in, float *out, size_t rows, size_t chunk) {
#pragma omp parallel
    {
        float *cache = (float *)malloc(sizeof(float) * (chunk ? chunk : 1));
#pragma omp for schedule(static)
        for (long r = 0; r < (long)rows; ++r) {
            const float *x = in + (size_t)r * chunk;
            float sums[WORK_GROUP_SIZE];
            for (int l = 0; l < WORK_GROUP_SIZE; ++l) {
                float sum = 0.0f;
                for (size_t j = (size_t)l; j < chunk; j += WORK_GROUP_SIZE) {
                    const float e = expf(x[j]);
                    sum += e;
                    cache[j] = e;
                }
                sums[l] = sum;
            }
            int remainder = WORK_GROUP_SIZE % 2;
            for (int offset = WORK_GROUP_SIZE / 2; offset > 0; offset /= 2) {
                for (int l = 0; l < offset; ++l) sums[l + remainder] += sums[l + offset + remainder];
                offset += remainder;
                remainder = offset % 2;
            }
            float *y = out + (size_t)r * chunk;
            for (size_t j = 0; j < chunk; ++j) y[j] = cache[j] / sums[0];
        }
        free(cache);
    }
}

/* multi_head_attention.cl:28-54 local_softmax with one work-group of row_len work-items per row
 * (nn/MultiHeadAttention.cpp:213-225, row_len = 77): item l holds exp(x[l]); the partial sums are
 * folded by halving with a carry for odd sizes (offset = n/2; items below offset add the item
 * `offset` above them, shifted by the remainder; the odd element in front joins the next round);
 * every item then divides its own exponential by sums[0].  No maximum is subtracted. */
void oracle_local_softmax(const float *in, float *out, size_t rows, size_t row_len) {
#pragma omp parallel
    {
        float *sums = (float *)malloc(sizeof(float) * (row_len ? row_len : 1));
        float *e = (float *)malloc(sizeof(float) * (row_len ? row_len : 1));
#pragma omp for schedule(static)
        for (long r = 0; r < (long)rows; ++r) {
            const float *x = in + (size_t)r * row_len;
            for (size_t l = 0; l < row_len; ++l) sums[l] = e[l] = expf(x[l]);
            int remainder = (int)(row_len % 2);
            for (int offset = (int)(row_len / 2); offset > 0; offset /= 2) {
                for (int l = 0; l < offset; ++l) sums[l + remainder] += sums[l + offset + remainder];
                offset += remainder;
                remainder = offset % 2;
            }
            float *y = out + (size_t)r * row_len;
            for (size_t l = 0; l < row_len; ++l) y[l] = e[l] / sums[0];
        }
        free(sums);
        free(e);
    }
}

/* util.cl:47-64 permute3D__0_2_1 with global size {I, J, K}: dst[i][k][j] = src[i][j][k]
 * (src_idx = i*J*K + j*K + k, dst_idx = i*K*J + k*J + j).  nn/SpatialTransformer.cpp:131-134
 * runs it with {1, C, HW} after the block's GroupNorm and :154-157 with {1, HW, C} before the
 * residual elemwise_add. */
void oracle_permute3D__0_2_1(const float *src, float *dst, size_t I, size_t J, size_t K) {
#pragma omp parallel for schedule(static) collapse(2)
    for (long i = 0; i < (long)I; ++i)
        for (long j = 0; j < (long)J; ++j)
            for (size_t k = 0; k < K; ++k)
                dst[(size_t)i * K * J + k * J + (size_t)j] = src[(size_t)i * J * K + (size_t)j * K + k];
}

/* util.cl:136-148: C[i] = A[i] + chunk[i / chunk_size] (the time-embedding broadcast add of
 * nn/ResBlock.cpp:188-199, chunk_size = H*W). */
void oracle_chunkwise_add(const float *A, const float *chunk, float *C, size_t n, size_t chunk_size) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)n; ++i) C[i] = A[i] + chunk[(size_t)i / chunk_size];
}

/* TextEncoder::createTokenEmbeddingBuffer (TextEncoder.cpp:105-125): out[i,:] = table[token[i],:]
 * copied row by row (:117-120), then elemwise_add with the positional table in place
 * (TextEncoder.cpp:141-151).  Batch > 1 repeats the positional table per sequence.
 * ids: [batch*T] int64 (the reference holds std::vector<long>).  The reference does not check
 * ids; here an id outside [0, vocab) returns -1 without touching `out`. */
int oracle_token_embedding(const int64_t *ids, const float *table, const float *pos, float *out,
                           size_t batch, size_t T, size_t D, size_t vocab) {
    for (size_t i = 0; i < batch * T; ++i) {
        if (ids[i] < 0 || (uint64_t)ids[i] >= vocab) return -1;
    }
    for (size_t i = 0; i < batch * T; ++i) {
        memcpy(out + i * D, table + (size_t)ids[i] * D, sizeof(float) * D);
    }
    for (size_t i = 0; i < batch * T * D; ++i) {
        out[i] = out[i] + pos[i % (T * D)];
    }
    return 0;
}

/* UNetModel::createTimestepEmbedding (UNetModel.cpp:1935-1958), all arithmetic in float:
 * freq = exp((-log(max_period)) * i / half); arg = (float)t * freq;
 * out[i] = cos(arg); out[i + half] = sin(arg)   (layout [cos | sin], :1952-1953).
 * One row per timestep (the reference builds one row for its single `long timestep`). */
void oracle_timestep_embedding(const int64_t *t, float *out, size_t batch, size_t dim,
                               float max_period) {
    const int half = (int)(dim / 2);
    for (size_t n = 0; n < batch; ++n) {
        for (int i = 0; i < half; ++i) {
            float freq = expf((-logf(max_period)) * (float)i / (float)half);
            float arg = (float)t[n] * freq;
            out[n * dim + (size_t)i] = cosf(arg);
            out[n * dim + (size_t)(i + half)] = sinf(arg);
        }
    }
}
