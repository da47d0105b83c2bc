// The C ABI of include/sdfl.h: argument validation, status codes, and the host-buffer
// pipeline.  No kernel lives here.
#include "../../include/sdfl.h"

#include "common.cuh"
#include "kernels.h"

#include <new>
#include <vector>

namespace sdfl {
std::atomic<long long> g_launches{0};
}

namespace {

thread_local cudaError_t tl_last_cuda = cudaSuccess;

inline int cuda_fail(cudaError_t e) {
    tl_last_cuda = e;
    (void)cudaGetLastError();   // clear the sticky-free error so the next call starts clean
    return SDFL_ERR_CUDA;
}

inline int wrap(cudaError_t e) { return e == cudaSuccess ? SDFL_OK : cuda_fail(e); }

inline bool dtype_ok(int dtype) { return dtype == SDFL_F32 || dtype == SDFL_F16; }
inline int64_t esize(int dtype) { return dtype == SDFL_F16 ? 2 : 4; }
inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }

// 0: disjoint or identical; 1: partial overlap.
inline bool partial_overlap(const void *a, int64_t abytes, const void *b, int64_t bbytes) {
    if (a == b) return false;
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
    return a0 < b0 + static_cast<uintptr_t>(bbytes) && b0 < a0 + static_cast<uintptr_t>(abytes);
}

// Any overlap at all (for ops whose in and out have different shapes).
inline bool any_overlap(const void *a, int64_t abytes, const void *b, int64_t bbytes) {
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
    return a0 < b0 + static_cast<uintptr_t>(bbytes) && b0 < a0 + static_cast<uintptr_t>(abytes);
}

int gn_validate(const void *in, const void *out, const float *gamma, const float *beta,
                int64_t batch, int64_t channels, int64_t hw, int64_t groups, float eps, int dtype) {
    if (!dtype_ok(dtype)) return SDFL_ERR_INVALID_VALUE;
    if (batch < 0 || channels <= 0 || hw < 0 || groups <= 0) return SDFL_ERR_INVALID_VALUE;
    if (channels % groups != 0) return SDFL_ERR_INVALID_VALUE;   // NN/GroupNorm.cpp:83-87
    if (!(eps >= 0.f)) return SDFL_ERR_INVALID_VALUE;
    if (hw >= (1ll << 31) || channels >= (1ll << 31)) return SDFL_ERR_UNSUPPORTED;
    if ((channels / groups) * hw >= (1ll << 31)) return SDFL_ERR_UNSUPPORTED;
    if (batch * groups >= (1ll << 27)) return SDFL_ERR_UNSUPPORTED;
    if (batch == 0 || hw == 0) return SDFL_OK;
    if (!in || !out || !gamma || !beta) return SDFL_ERR_INVALID_POINTER;
    const int64_t bytes = batch * channels * hw * esize(dtype);
    if (partial_overlap(in, bytes, out, bytes)) return SDFL_ERR_OVERLAP;
    return SDFL_OK;
}

int gn_forward(const void *in, void *out, const float *gamma, const float *beta, int64_t batch,
               int64_t channels, int64_t hw, int64_t groups, float eps, int fuse_silu, int dtype,
               void *workspace, size_t workspace_bytes, int path, int cluster, cudaStream_t stream,
               const void *bias = nullptr) {
    int rc = gn_validate(in, out, gamma, beta, batch, channels, hw, groups, eps, dtype);
    if (rc != SDFL_OK) return rc;
    if (batch == 0 || hw == 0) return SDFL_OK;
    if (path < SDFL_GN_AUTO || path > SDFL_GN_REGISTER || cluster < 0) return SDFL_ERR_INVALID_VALUE;
    sdfl::GnShape s{batch, channels, hw, groups, dtype, eps,
                    fuse_silu ? sdfl::kActSilu : sdfl::kActNone, bias != nullptr};
    sdfl::GnPlan plan;
    cudaError_t e = sdfl::gn_make_plan(s, in, out, path, cluster, &plan);
    if (e == cudaErrorInvalidConfiguration || e == cudaErrorInvalidValue) return SDFL_ERR_UNSUPPORTED;
    if (e != cudaSuccess) return cuda_fail(e);
    if (plan.path == sdfl::kGnSplit && (workspace == nullptr || workspace_bytes < plan.workspace))
        return SDFL_ERR_WORKSPACE;
    return wrap(sdfl::gn_launch(s, plan, in, out, gamma, beta, workspace, stream, bias));
}

int unary(int act, const void *src, void *dst, int64_t n, int dtype, void *stream) {
    if (!dtype_ok(dtype) || n < 0) return SDFL_ERR_INVALID_VALUE;
    if (n == 0) return SDFL_OK;
    if (!src || !dst) return SDFL_ERR_INVALID_POINTER;
    if (partial_overlap(src, n * esize(dtype), dst, n * esize(dtype))) return SDFL_ERR_OVERLAP;
    return wrap(sdfl::act_launch(act, src, dst, n, dtype, as_stream(stream)));
}

}  // namespace

struct sdfl_groupnorm {
    int64_t num_groups, num_channels;
    float eps;
    const float *gamma, *beta;
    int fuse_silu;
    void *ws;
    size_t ws_bytes;
    int device;
};

struct sdfl_layernorm {
    int64_t dim;
    float eps;
    const float *gamma, *beta;
    int device;
};

struct sdfl_geglu {
    int64_t in_features, out_features;
};

struct sdfl_host_pipeline {
    struct Slot {
        void *d_in = nullptr;
        void *d_out = nullptr;
        void *d_ws = nullptr;
        cudaStream_t stream = nullptr;
    };
    std::vector<Slot> slots;
    size_t slot_bytes = 0;
    size_t ws_bytes = 0;
    size_t next = 0;      // round-robin slot cursor
    int device = 0;
};

extern "C" {

const char *sdfl_version(void) { return "sdfl 0.1 (sm_100a)"; }

const char *sdfl_status_string(int status) {
    switch (status) {
        case SDFL_OK: return "ok";
        case SDFL_ERR_INVALID_VALUE: return "invalid value";
        case SDFL_ERR_INVALID_POINTER: return "invalid (null) pointer";
        case SDFL_ERR_UNSUPPORTED: return "unsupported shape";
        case SDFL_ERR_CUDA: return "CUDA error";
        case SDFL_ERR_OVERLAP: return "input and output partially overlap";
        case SDFL_ERR_WORKSPACE: return "workspace missing or too small";
        case SDFL_ERR_DEVICE_FLAG: return "device status word raised";
        default: return "unknown status";
    }
}

int sdfl_last_cuda_error(void) { return static_cast<int>(tl_last_cuda); }
const char *sdfl_last_cuda_error_string(void) { return cudaGetErrorString(tl_last_cuda); }
long long sdfl_launch_count(void) { return sdfl::g_launches.load(); }

int sdfl_groupnorm_forward(const void *in, void *out, const float *gamma, const float *beta,
                           int64_t batch, int64_t channels, int64_t hw, int64_t num_groups,
                           float eps, int fuse_silu, int dtype, void *workspace,
                           size_t workspace_bytes, void *stream) {
    return gn_forward(in, out, gamma, beta, batch, channels, hw, num_groups, eps, fuse_silu, dtype,
                      workspace, workspace_bytes, SDFL_GN_AUTO, 0, as_stream(stream));
}

int sdfl_groupnorm_forward_ex(const void *in, void *out, const float *gamma, const float *beta,
                              int64_t batch, int64_t channels, int64_t hw, int64_t num_groups,
                              float eps, int fuse_silu, int dtype, void *workspace,
                              size_t workspace_bytes, int path, int cluster_or_splits, void *stream) {
    return gn_forward(in, out, gamma, beta, batch, channels, hw, num_groups, eps, fuse_silu, dtype,
                      workspace, workspace_bytes, path, cluster_or_splits, as_stream(stream));
}

size_t sdfl_groupnorm_multi_workspace_bytes(void) { return sdfl::kGnMultiScratchBytes; }

// GroupNorm(+SiLU) of up to SDFL_GN_MULTI_MAX tensors in one persistent launch; see sdfl.h.
int sdfl_groupnorm_forward_multi_ex(const sdfl_gn_tensor *tensors, int count, int fuse_silu, int dtype,
                                    void *workspace, size_t workspace_bytes, int knobs,
                                    unsigned long long *d_trace, int plan[4], void *stream) {
    if (plan) plan[0] = plan[1] = plan[2] = plan[3] = 0;
    if (count < 0 || !dtype_ok(dtype) || knobs < 0) return SDFL_ERR_INVALID_VALUE;
    if (count == 0) return SDFL_OK;
    if (!tensors) return SDFL_ERR_INVALID_POINTER;
    if (workspace != nullptr && workspace_bytes < sdfl::kGnMultiScratchBytes) return SDFL_ERR_WORKSPACE;
    sdfl::GnMultiTensor ts[SDFL_GN_MULTI_MAX];
    int n = 0;
    for (int k = 0; k < count; ++k) {
        const sdfl_gn_tensor &t = tensors[k];
        int rc = gn_validate(t.in, t.out, t.gamma, t.beta, t.batch, t.channels, t.hw, t.num_groups, t.eps, dtype);
        if (rc != SDFL_OK) return rc;
        if (t.batch == 0 || t.hw == 0) continue;            // an empty tensor is no work
        if (n == SDFL_GN_MULTI_MAX) return SDFL_ERR_UNSUPPORTED;
        ts[n++] = sdfl::GnMultiTensor{t.in, t.out, t.gamma, t.beta, t.batch, t.channels, t.hw, t.num_groups, t.eps};
    }
    // outputs must not overlap one another or another tensor's input
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < n; ++j) {
            if (i == j) continue;
            const int64_t bi = ts[i].batch * ts[i].channels * ts[i].hw * esize(dtype);
            const int64_t bj = ts[j].batch * ts[j].channels * ts[j].hw * esize(dtype);
            if (any_overlap(ts[i].out, bi, ts[j].out, bj) || any_overlap(ts[i].out, bi, ts[j].in, bj))
                return SDFL_ERR_OVERLAP;
        }
    if (n == 0) return SDFL_OK;
    if (sdfl::gn_multi_check(ts, n, dtype) != 0) return SDFL_ERR_UNSUPPORTED;
    cudaError_t e = sdfl::gn_multi_launch(ts, n, dtype, fuse_silu ? sdfl::kActSilu : sdfl::kActNone, knobs,
                                          workspace, d_trace, plan, as_stream(stream));
    if (e == cudaErrorInvalidConfiguration || e == cudaErrorInvalidValue) return SDFL_ERR_UNSUPPORTED;
    return wrap(e);
}

int sdfl_groupnorm_forward_multi(const sdfl_gn_tensor *tensors, int count, int fuse_silu, int dtype,
                                 void *workspace, size_t workspace_bytes, void *stream) {
    return sdfl_groupnorm_forward_multi_ex(tensors, count, fuse_silu, dtype, workspace, workspace_bytes, 0,
                                           nullptr, nullptr, stream);
}

// GroupNorm(+SiLU) through the split path with the scratch in the library's own fixed device
// array: for callers that are not allowed to allocate (see sdfl.h).  No allocation is made
// here or below; shapes whose scratch would exceed the array are refused before any launch.
int sdfl_groupnorm_forward_noalloc(const void *in, void *out, const float *gamma, const float *beta,
                                   int64_t batch, int64_t channels, int64_t hw, int64_t num_groups,
                                   float eps, int fuse_silu, int dtype, void *stream) {
    int rc = gn_validate(in, out, gamma, beta, batch, channels, hw, num_groups, eps, dtype);
    if (rc != SDFL_OK) return rc;
    if (batch == 0 || hw == 0) return SDFL_OK;
    sdfl::GnShape s{batch, channels, hw, num_groups, dtype, eps,
                    fuse_silu ? sdfl::kActSilu : sdfl::kActNone};
    sdfl::GnPlan plan;
    cudaError_t e = sdfl::gn_make_plan(s, in, out, sdfl::kGnSplit, 0, &plan);
    if (e == cudaErrorInvalidConfiguration || e == cudaErrorInvalidValue) return SDFL_ERR_UNSUPPORTED;
    if (e != cudaSuccess) return cuda_fail(e);
    if (plan.workspace > sdfl::kGnStaticScratchBytes) return SDFL_ERR_WORKSPACE;   // beyond the fixed array
    return wrap(sdfl::gn_launch_static_scratch(s, plan, in, out, gamma, beta, as_stream(stream)));
}

int sdfl_groupnorm_bias_forward(const void *in, const void *channel_bias, void *out, const float *gamma,
                                const float *beta, int64_t batch, int64_t channels, int64_t hw,
                                int64_t num_groups, float eps, int fuse_silu, int dtype, void *workspace,
                                size_t workspace_bytes, void *stream) {
    if (!channel_bias && batch > 0 && hw > 0) return SDFL_ERR_INVALID_POINTER;
    return gn_forward(in, out, gamma, beta, batch, channels, hw, num_groups, eps, fuse_silu, dtype,
                      workspace, workspace_bytes, SDFL_GN_AUTO, 0, as_stream(stream), channel_bias);
}

int sdfl_groupnorm_bias_forward_ex(const void *in, const void *channel_bias, void *out,
                                   const float *gamma, const float *beta, int64_t batch,
                                   int64_t channels, int64_t hw, int64_t num_groups, float eps,
                                   int fuse_silu, int dtype, void *workspace, size_t workspace_bytes,
                                   int path, int cluster_or_splits, void *stream) {
    if (!channel_bias && batch > 0 && hw > 0) return SDFL_ERR_INVALID_POINTER;
    return gn_forward(in, out, gamma, beta, batch, channels, hw, num_groups, eps, fuse_silu, dtype,
                      workspace, workspace_bytes, path, cluster_or_splits, as_stream(stream), channel_bias);
}

size_t sdfl_groupnorm_nhwc_workspace_bytes(int64_t batch, int64_t channels, int64_t hw,
                                           int64_t num_groups, int dtype) {
    if (!dtype_ok(dtype) || batch <= 0 || channels <= 0 || hw <= 0 || num_groups <= 0 ||
        channels % num_groups != 0)
        return 0;
    // the per-chunk moments of the statistics kernel (the two-kernel form; the one-kernel form
    // for small slabs needs none, but which one runs also depends on the pointers' alignment)
    return sdfl_groupnorm_workspace_bytes_ex(batch, channels, hw, num_groups, dtype, SDFL_GN_SPLIT, 0);
}

int sdfl_groupnorm_nhwc_forward(const void *in, void *out, const float *gamma, const float *beta,
                                int64_t batch, int64_t channels, int64_t hw, int64_t num_groups,
                                float eps, int fuse_silu, int dtype, void *workspace,
                                size_t workspace_bytes, void *stream) {
    int rc = gn_validate(in, out, gamma, beta, batch, channels, hw, num_groups, eps, dtype);
    if (rc != SDFL_OK) return rc;
    if (batch == 0 || hw == 0) return SDFL_OK;
    if (batch > 65535) return SDFL_ERR_UNSUPPORTED;
    const int64_t bytes = batch * channels * hw * esize(dtype);
    if (in == out || partial_overlap(in, bytes, out, bytes)) return SDFL_ERR_OVERLAP;   // a transpose cannot run in place
    sdfl::GnShape s{batch, channels, hw, num_groups, dtype, eps,
                    fuse_silu ? sdfl::kActSilu : sdfl::kActNone};
    sdfl::GnPlan plan;
    const bool fused = sdfl::gn_nhwc_fused_ok(s, in, out);
    cudaError_t e = sdfl::gn_make_plan(s, in, out, fused ? sdfl::kGnRegister : sdfl::kGnSplit, 0, &plan);
    if (e == cudaErrorInvalidConfiguration || e == cudaErrorInvalidValue) return SDFL_ERR_UNSUPPORTED;
    if (e != cudaSuccess) return cuda_fail(e);
    plan.nhwc = 1;
    if (!fused && (workspace == nullptr || workspace_bytes < plan.workspace)) return SDFL_ERR_WORKSPACE;
    return wrap(sdfl::gn_launch(s, plan, in, out, gamma, beta, workspace, as_stream(stream)));
}

static int permute_checked(const void *src, const void *res, void *dst, int64_t I, int64_t J, int64_t K,
                           int dtype, void *stream) {
    if (!dtype_ok(dtype) || I < 0 || J < 0 || K < 0) return SDFL_ERR_INVALID_VALUE;
    if (J >= (1ll << 31) || K >= (1ll << 31)) return SDFL_ERR_UNSUPPORTED;
    if (I == 0 || J == 0 || K == 0) return SDFL_OK;
    if (!src || !dst) return SDFL_ERR_INVALID_POINTER;
    const int64_t bytes = I * J * K * esize(dtype);
    if (src == dst || partial_overlap(src, bytes, dst, bytes)) return SDFL_ERR_OVERLAP;
    if (res && res != dst && partial_overlap(res, bytes, dst, bytes)) return SDFL_ERR_OVERLAP;
    return wrap(sdfl::permute_021_launch(src, res, dst, I, J, K, dtype, as_stream(stream)));
}

int sdfl_permute3D__0_2_1(const void *src, void *dst, int64_t I, int64_t J, int64_t K, int dtype,
                          void *stream) {
    return permute_checked(src, nullptr, dst, I, J, K, dtype, stream);
}

int sdfl_permute_add(const void *src, const void *residual, void *dst, int64_t I, int64_t J, int64_t K,
                     int dtype, void *stream) {
    if (!residual && I > 0 && J > 0 && K > 0) return SDFL_ERR_INVALID_POINTER;
    return permute_checked(src, residual, dst, I, J, K, dtype, stream);
}

int sdfl_up_sample_nearest(const void *input, void *output, int64_t channels, int64_t height, int64_t width,
                           int64_t scale, int dtype, void *stream) {
    if (!dtype_ok(dtype) || channels < 0 || height < 0 || width < 0 || scale < 1) return SDFL_ERR_INVALID_VALUE;
    if (height >= (1ll << 31) / scale || width >= (1ll << 31) / scale) return SDFL_ERR_UNSUPPORTED;
    if (channels == 0 || height == 0 || width == 0) return SDFL_OK;
    if (!input || !output) return SDFL_ERR_INVALID_POINTER;
    const int64_t ib = channels * height * width * esize(dtype);
    if (input == output || partial_overlap(input, ib, output, ib * scale * scale)) return SDFL_ERR_OVERLAP;
    return wrap(sdfl::upsample_nearest_launch(input, output, channels, height, width, scale, dtype, as_stream(stream)));
}

int sdfl_concat_buffer(const void *input1, const void *input2, void *output, int64_t batch, int64_t n1,
                       int64_t n2, int dtype, void *stream) {
    if (!dtype_ok(dtype) || batch < 0 || n1 < 0 || n2 < 0) return SDFL_ERR_INVALID_VALUE;
    if (batch == 0 || n1 + n2 == 0) return SDFL_OK;
    if ((n1 && !input1) || (n2 && !input2) || !output) return SDFL_ERR_INVALID_POINTER;
    const int64_t ob = batch * (n1 + n2) * esize(dtype);
    if ((n1 && partial_overlap(input1, batch * n1 * esize(dtype), output, ob)) || input1 == output ||
        (n2 && partial_overlap(input2, batch * n2 * esize(dtype), output, ob)) || input2 == output)
        return SDFL_ERR_OVERLAP;
    return wrap(sdfl::concat_launch(input1, input2, output, batch, n1, n2, dtype, as_stream(stream)));
}

int sdfl_groupnorm_concat_forward(const void *in1, int64_t channels1, const void *in2, int64_t channels2,
                                  void *out, const float *gamma, const float *beta, int64_t batch,
                                  int64_t hw, int64_t num_groups, float eps, int fuse_silu, int dtype,
                                  void *workspace, size_t workspace_bytes, void *stream) {
    if (channels1 <= 0 || channels2 <= 0) return SDFL_ERR_INVALID_VALUE;
    const int64_t channels = channels1 + channels2;
    // shape checks on the concatenated tensor (in1 is smaller than that: its own overlap test follows)
    int rc = gn_validate(out, out, gamma, beta, batch, channels, hw, num_groups, eps, dtype);
    if (rc != SDFL_OK) return rc;
    if (batch == 0 || hw == 0) return SDFL_OK;
    if (!in1 || !in2) return SDFL_ERR_INVALID_POINTER;
    const int64_t ob = batch * channels * hw * esize(dtype);
    if (in1 == out || in2 == out || partial_overlap(in1, batch * channels1 * hw * esize(dtype), out, ob) ||
        partial_overlap(in2, batch * channels2 * hw * esize(dtype), out, ob))
        return SDFL_ERR_OVERLAP;
    sdfl::GnShape s{batch, channels, hw, num_groups, dtype, eps,
                    fuse_silu ? sdfl::kActSilu : sdfl::kActNone};
    sdfl::GnPlan plan;
    cudaError_t e = sdfl::gn_make_plan(s, in1, out, SDFL_GN_AUTO, 0, &plan);
    if (e == cudaErrorInvalidConfiguration || e == cudaErrorInvalidValue) return SDFL_ERR_UNSUPPORTED;
    if (e != cudaSuccess) return cuda_fail(e);
    if (sdfl::gn_concat_fused_ok(s, plan, in1, in2, channels1))
        return wrap(sdfl::gn_launch(s, plan, in1, out, gamma, beta, workspace, as_stream(stream), nullptr, in2,
                                    channels1));
    // otherwise: the reference's two copies into `out`, then the norm in place
    rc = sdfl_concat_buffer(in1, in2, out, batch, channels1 * hw, channels2 * hw, dtype, stream);
    if (rc != SDFL_OK) return rc;
    return gn_forward(out, out, gamma, beta, batch, channels, hw, num_groups, eps, fuse_silu, dtype, workspace,
                      workspace_bytes, SDFL_GN_AUTO, 0, as_stream(stream));
}

int sdfl_softmax(const void *input, void *output, int64_t rows, int64_t chunk_size, int dtype, void *stream) {
    if (!dtype_ok(dtype) || rows < 0 || chunk_size < 0) return SDFL_ERR_INVALID_VALUE;
    if (chunk_size >= (1ll << 31)) return SDFL_ERR_UNSUPPORTED;
    if (rows == 0 || chunk_size == 0) return SDFL_OK;
    if (!input || !output) return SDFL_ERR_INVALID_POINTER;
    const int64_t bytes = rows * chunk_size * esize(dtype);
    if (partial_overlap(input, bytes, output, bytes)) return SDFL_ERR_OVERLAP;
    return wrap(sdfl::softmax_launch(input, output, rows, chunk_size, dtype, as_stream(stream)));
}

int sdfl_local_softmax(const void *input, void *output, int64_t rows, int64_t row_len, int dtype, void *stream) {
    return sdfl_softmax(input, output, rows, row_len, dtype, stream);
}

int sdfl_chunkwise_add(const void *A, const void *chunk, void *C, int64_t n, int64_t chunk_size,
                       int dtype, void *stream) {
    if (!dtype_ok(dtype) || n < 0 || chunk_size <= 0) return SDFL_ERR_INVALID_VALUE;
    if (n == 0) return SDFL_OK;
    if (!A || !chunk || !C) return SDFL_ERR_INVALID_POINTER;
    if (partial_overlap(A, n * esize(dtype), C, n * esize(dtype))) return SDFL_ERR_OVERLAP;
    return wrap(sdfl::chunkwise_add_launch(A, chunk, C, n, chunk_size, dtype, as_stream(stream)));
}

int sdfl_groupnorm_plan(int64_t batch, int64_t channels, int64_t hw, int64_t num_groups, int dtype,
                        int path, int cluster_or_splits, int64_t plan[8]) {
    if (!plan) return SDFL_ERR_INVALID_POINTER;
    for (int i = 0; i < 8; ++i) plan[i] = 0;
    if (!dtype_ok(dtype) || batch < 0 || channels <= 0 || hw < 0 || num_groups <= 0 ||
        channels % num_groups != 0 || path < SDFL_GN_AUTO || path > SDFL_GN_REGISTER ||
        cluster_or_splits < 0)
        return SDFL_ERR_INVALID_VALUE;
    if (hw >= (1ll << 31) || (channels / num_groups) * hw >= (1ll << 31) ||
        batch * num_groups >= (1ll << 27))
        return SDFL_ERR_UNSUPPORTED;
    if (batch == 0 || hw == 0) return SDFL_OK;
    sdfl::GnShape s{batch, channels, hw, num_groups, dtype, 0.f, sdfl::kActNone};
    sdfl::GnPlan p;
    // a 16-byte aligned stand-in address: only its alignment is looked at
    const void *aligned = reinterpret_cast<const void *>(static_cast<uintptr_t>(256));
    cudaError_t e = sdfl::gn_make_plan(s, aligned, aligned, path, cluster_or_splits, &p);
    if (e == cudaErrorInvalidConfiguration || e == cudaErrorInvalidValue) return SDFL_ERR_UNSUPPORTED;
    if (e != cudaSuccess) return cuda_fail(e);
    plan[0] = p.path; plan[1] = p.cluster; plan[2] = p.threads;
    plan[3] = p.path == sdfl::kGnSplit ? p.splits : p.nslots;
    plan[4] = static_cast<int64_t>(p.smem); plan[5] = static_cast<int64_t>(p.workspace);
    plan[6] = p.nclusters; plan[7] = p.chunk_vecs;
    return SDFL_OK;
}

size_t sdfl_groupnorm_workspace_bytes_ex(int64_t batch, int64_t channels, int64_t hw,
                                         int64_t num_groups, int dtype, int path,
                                         int cluster_or_splits) {
    // Sized for the split path whatever the automatic choice would be: the choice depends on
    // pointer alignment, which is only known at the call.
    if (!dtype_ok(dtype) || batch <= 0 || channels <= 0 || hw <= 0 || num_groups <= 0 ||
        channels % num_groups != 0 || (channels / num_groups) * hw >= (1ll << 31))
        return 0;
    sdfl::GnShape s{batch, channels, hw, num_groups, dtype, 0.f, sdfl::kActNone};
    sdfl::GnPlan p;
    const void *aligned = reinterpret_cast<const void *>(static_cast<uintptr_t>(256));
    const int splits = path == SDFL_GN_SPLIT ? cluster_or_splits : 0;
    if (sdfl::gn_make_plan(s, aligned, aligned, SDFL_GN_SPLIT, splits, &p) != cudaSuccess) return 0;
    return p.workspace;
}

size_t sdfl_groupnorm_workspace_bytes(int64_t batch, int64_t channels, int64_t hw,
                                      int64_t num_groups, int dtype) {
    return sdfl_groupnorm_workspace_bytes_ex(batch, channels, hw, num_groups, dtype, SDFL_GN_AUTO, 0);
}

int sdfl_layernorm_forward(const void *in, void *out, const float *gamma, const float *beta,
                           int64_t rows, int64_t dim, float eps, int dtype, void *stream) {
    if (!dtype_ok(dtype) || rows < 0 || dim <= 0 || !(eps >= 0.f)) return SDFL_ERR_INVALID_VALUE;
    if (dim >= (1ll << 31)) return SDFL_ERR_UNSUPPORTED;
    if (rows == 0) return SDFL_OK;
    if (!in || !out || !gamma || !beta) return SDFL_ERR_INVALID_POINTER;
    const int64_t bytes = rows * dim * esize(dtype);
    if (partial_overlap(in, bytes, out, bytes)) return SDFL_ERR_OVERLAP;
    return wrap(sdfl::ln_launch(in, out, gamma, beta, rows, dim, eps, dtype, as_stream(stream)));
}

int sdfl_add_layernorm_forward(const void *a, const void *b, void *sum_out, void *out,
                               const float *gamma, const float *beta, int64_t rows, int64_t dim,
                               float eps, int dtype, void *stream) {
    if (!dtype_ok(dtype) || rows < 0 || dim <= 0 || !(eps >= 0.f)) return SDFL_ERR_INVALID_VALUE;
    if (dim >= (1ll << 31)) return SDFL_ERR_UNSUPPORTED;
    if (rows == 0) return SDFL_OK;
    if (!a || !b || !sum_out || !out || !gamma || !beta) return SDFL_ERR_INVALID_POINTER;
    const int64_t bytes = rows * dim * esize(dtype);
    // sum_out may be a or b (the reference adds in place); out may be a or b but not sum_out
    if (partial_overlap(a, bytes, sum_out, bytes) || partial_overlap(b, bytes, sum_out, bytes) ||
        partial_overlap(a, bytes, out, bytes) || partial_overlap(b, bytes, out, bytes) ||
        any_overlap(sum_out, bytes, out, bytes))
        return SDFL_ERR_OVERLAP;
    return wrap(sdfl::add_ln_launch(a, b, sum_out, out, gamma, beta, rows, dim, eps, dtype, as_stream(stream)));
}

int sdfl_token_embedding(const int64_t *ids, const void *table, const void *pos, void *out,
                         int64_t batch, int64_t seq_len, int64_t dim, int64_t vocab, int dtype,
                         int *d_status, void *stream) {
    if (!dtype_ok(dtype) || batch < 0 || seq_len < 0 || dim < 0 || vocab <= 0)
        return SDFL_ERR_INVALID_VALUE;
    if (batch == 0 || seq_len == 0 || dim == 0) return SDFL_OK;
    if (!ids || !table || !pos || !out) return SDFL_ERR_INVALID_POINTER;
    return wrap(sdfl::token_embedding_launch(ids, table, pos, out, batch, seq_len, dim, vocab, dtype,
                                             d_status, as_stream(stream)));
}

int sdfl_timestep_embedding(const int64_t *t, void *out, int64_t batch, int64_t dim,
                            float max_period, int dtype, void *stream) {
    if (!dtype_ok(dtype) || batch < 0 || dim < 0 || !(max_period > 0.f)) return SDFL_ERR_INVALID_VALUE;
    if (batch * (dim / 2) >= (1ll << 31)) return SDFL_ERR_UNSUPPORTED;
    if (batch == 0 || dim == 0) return SDFL_OK;
    if (!t || !out) return SDFL_ERR_INVALID_POINTER;
    return wrap(sdfl::timestep_embedding_launch(t, out, batch, dim, max_period, dtype, as_stream(stream)));
}

int sdfl_local_reduction_mean(const void *input, float *output, int64_t groups, int64_t group_elems,
                              int dtype, void *stream) {
    if (!dtype_ok(dtype) || groups < 0 || group_elems <= 0) return SDFL_ERR_INVALID_VALUE;
    if (groups >= (1ll << 31)) return SDFL_ERR_UNSUPPORTED;
    if (groups == 0) return SDFL_OK;
    if (!input || !output) return SDFL_ERR_INVALID_POINTER;
    return wrap(sdfl::stats_mean_launch(input, output, groups, group_elems, dtype, as_stream(stream)));
}

int sdfl_local_reduction_variance(const void *input, const float *mean, float *output,
                                  int64_t groups, int64_t group_elems, int dtype, void *stream) {
    if (!dtype_ok(dtype) || groups < 0 || group_elems <= 0) return SDFL_ERR_INVALID_VALUE;
    if (groups >= (1ll << 31)) return SDFL_ERR_UNSUPPORTED;
    if (groups == 0) return SDFL_OK;
    if (!input || !mean || !output) return SDFL_ERR_INVALID_POINTER;
    return wrap(sdfl::stats_var_launch(input, mean, output, groups, group_elems, dtype, as_stream(stream)));
}

int sdfl_group_norm(const void *input, const float *mean, const float *variance,
                    const float *weight, const float *bias, int64_t groupSize, int64_t channelSize,
                    float epsilon, void *output, int64_t n, int64_t num_channels, int dtype,
                    void *stream) {
    if (!dtype_ok(dtype) || n < 0 || groupSize <= 0 || channelSize <= 0 || num_channels <= 0)
        return SDFL_ERR_INVALID_VALUE;
    if (n == 0) return SDFL_OK;
    if (!input || !mean || !variance || !weight || !bias || !output) return SDFL_ERR_INVALID_POINTER;
    if (partial_overlap(input, n * esize(dtype), output, n * esize(dtype))) return SDFL_ERR_OVERLAP;
    return wrap(sdfl::gn_apply_launch(input, mean, variance, weight, bias, groupSize, channelSize,
                                      epsilon, output, n, num_channels, dtype, as_stream(stream)));
}

int sdfl_layer_norm(const void *input, const float *mean, const float *variance,
                    const float *weight, const float *bias, int64_t chunkSize, void *output,
                    int64_t n, float epsilon, int dtype, void *stream) {
    if (!dtype_ok(dtype) || n < 0 || chunkSize <= 0) return SDFL_ERR_INVALID_VALUE;
    if (n == 0) return SDFL_OK;
    if (!input || !mean || !variance || !weight || !bias || !output) return SDFL_ERR_INVALID_POINTER;
    if (partial_overlap(input, n * esize(dtype), output, n * esize(dtype))) return SDFL_ERR_OVERLAP;
    return wrap(sdfl::ln_apply_launch(input, mean, variance, weight, bias, chunkSize, epsilon, output,
                                      n, dtype, as_stream(stream)));
}

int sdfl_gelu_multiply(const void *AB, void *dst, int64_t rows, int64_t D, int dtype, void *stream) {
    if (!dtype_ok(dtype) || rows < 0 || D < 0) return SDFL_ERR_INVALID_VALUE;
    if (rows == 0 || D == 0) return SDFL_OK;
    if (!AB || !dst) return SDFL_ERR_INVALID_POINTER;
    if (any_overlap(AB, rows * 2 * D * esize(dtype), dst, rows * D * esize(dtype)))
        return SDFL_ERR_OVERLAP;
    return wrap(sdfl::geglu_launch(AB, dst, rows, D, dtype, as_stream(stream)));
}

int sdfl_gelu(const void *src, void *dst, int64_t n, int dtype, void *stream) {
    return unary(sdfl::kActGelu, src, dst, n, dtype, stream);
}
int sdfl_silu(const void *src, void *dst, int64_t n, int dtype, void *stream) {
    return unary(sdfl::kActSilu, src, dst, n, dtype, stream);
}
int sdfl_quick_gelu(const void *src, void *dst, int64_t n, int dtype, void *stream) {
    return unary(sdfl::kActQuickGelu, src, dst, n, dtype, stream);
}

int sdfl_elemwise_add(const void *A, const void *B, void *C, int64_t n, int dtype, void *stream) {
    if (!dtype_ok(dtype) || n < 0) return SDFL_ERR_INVALID_VALUE;
    if (n == 0) return SDFL_OK;
    if (!A || !B || !C) return SDFL_ERR_INVALID_POINTER;
    const int64_t bytes = n * esize(dtype);
    if (partial_overlap(A, bytes, C, bytes) || partial_overlap(B, bytes, C, bytes))
        return SDFL_ERR_OVERLAP;
    return wrap(sdfl::add_launch(A, B, C, n, dtype, as_stream(stream)));
}

int sdfl_device_status(unsigned int *value, int clear, void *stream) {
    if (!value) return SDFL_ERR_INVALID_POINTER;
    unsigned int ring = 0, multi = 0, reg = 0;
    cudaError_t e = sdfl::gn_read_status(&ring, clear != 0, as_stream(stream));
    if (e == cudaSuccess) e = sdfl::gn_multi_read_status(&multi, clear != 0, as_stream(stream));
    if (e == cudaSuccess) e = sdfl::gn_register_read_status(&reg, clear != 0, as_stream(stream));
    *value = ring | multi | reg;
    return wrap(e);
}

int sdfl_selftest_bounded_wait(long long limit_cycles, void *stream) {
    return wrap(sdfl::gn_wait_selftest(limit_cycles, as_stream(stream)));
}

// ---- operator handles (NN/GroupNorm.h:15-29, NN/LayerNorm.h:16-28, NN/GEGLU.h:18-36) ------------------

int sdfl_groupnorm_create(sdfl_groupnorm **op, int64_t num_groups, int64_t num_channels, float eps,
                          const float *d_gamma, const float *d_beta, int fuse_silu, int64_t max_batch,
                          int64_t max_hw, int max_dtype) {
    if (!op) return SDFL_ERR_INVALID_POINTER;
    *op = nullptr;
    if (num_groups <= 0 || num_channels <= 0 || num_channels % num_groups != 0 || !(eps >= 0.f) ||
        max_batch < 0 || max_hw < 0 || !dtype_ok(max_dtype))
        return SDFL_ERR_INVALID_VALUE;
    if (!d_gamma || !d_beta) return SDFL_ERR_INVALID_POINTER;
    sdfl_groupnorm *p = new (std::nothrow) sdfl_groupnorm{num_groups, num_channels, eps, d_gamma, d_beta,
                                                          fuse_silu ? 1 : 0, nullptr, 0, 0};
    if (!p) return cuda_fail(cudaErrorMemoryAllocation);
    cudaError_t e = cudaGetDevice(&p->device);
    // scratch of the any-shape path for the largest tensor, in either storage type.  A smaller tensor
    // is cut into more chunks per slab, but never into more than about 600 chunks beyond its slabs.
    size_t need = static_cast<size_t>(600 + max_batch * num_groups) * 2 * sizeof(float);
    if (need < 64 * 1024) need = 64 * 1024;
    for (int dt = 0; dt <= max_dtype; ++dt) {
        const size_t n = sdfl_groupnorm_workspace_bytes_ex(max_batch, num_channels, max_hw, num_groups, dt,
                                                           SDFL_GN_SPLIT, 0);
        if (n > need) need = n;
    }
    if (e == cudaSuccess) e = cudaMalloc(&p->ws, need);
    if (e != cudaSuccess) { delete p; return cuda_fail(e); }
    p->ws_bytes = need;
    *op = p;
    return SDFL_OK;
}

int sdfl_groupnorm_op_forward(sdfl_groupnorm *op, const void *in, void *out, int64_t batch, int64_t hw,
                              int dtype, void *stream) {
    if (!op) return SDFL_ERR_INVALID_POINTER;
    int current = -1;
    cudaError_t e = cudaGetDevice(&current);
    if (e != cudaSuccess) return cuda_fail(e);
    if (current != op->device) return SDFL_ERR_INVALID_VALUE;
    return gn_forward(in, out, op->gamma, op->beta, batch, op->num_channels, hw, op->num_groups, op->eps,
                      op->fuse_silu, dtype, op->ws, op->ws_bytes, SDFL_GN_AUTO, 0, as_stream(stream));
}

int sdfl_groupnorm_destroy(sdfl_groupnorm *op) {
    if (!op) return SDFL_OK;
    cudaError_t e = op->ws ? cudaFree(op->ws) : cudaSuccess;
    delete op;
    return wrap(e);
}

int sdfl_layernorm_create(sdfl_layernorm **op, int64_t dim, float eps, const float *d_gamma,
                          const float *d_beta) {
    if (!op) return SDFL_ERR_INVALID_POINTER;
    *op = nullptr;
    if (dim <= 0 || !(eps >= 0.f)) return SDFL_ERR_INVALID_VALUE;
    if (!d_gamma || !d_beta) return SDFL_ERR_INVALID_POINTER;
    sdfl_layernorm *p = new (std::nothrow) sdfl_layernorm{dim, eps, d_gamma, d_beta, 0};
    if (!p) return cuda_fail(cudaErrorMemoryAllocation);
    cudaError_t e = cudaGetDevice(&p->device);
    if (e != cudaSuccess) { delete p; return cuda_fail(e); }
    *op = p;
    return SDFL_OK;
}

int sdfl_layernorm_op_forward(sdfl_layernorm *op, const void *in, void *out, int64_t rows, int dtype,
                              void *stream) {
    if (!op) return SDFL_ERR_INVALID_POINTER;
    int current = -1;
    cudaError_t e = cudaGetDevice(&current);
    if (e != cudaSuccess) return cuda_fail(e);
    if (current != op->device) return SDFL_ERR_INVALID_VALUE;
    return sdfl_layernorm_forward(in, out, op->gamma, op->beta, rows, op->dim, op->eps, dtype, stream);
}

int sdfl_layernorm_destroy(sdfl_layernorm *op) {
    delete op;
    return SDFL_OK;
}

int sdfl_geglu_create(sdfl_geglu **op, int64_t in_features, int64_t out_features) {
    if (!op) return SDFL_ERR_INVALID_POINTER;
    *op = nullptr;
    if (in_features <= 0 || out_features <= 0) return SDFL_ERR_INVALID_VALUE;
    sdfl_geglu *p = new (std::nothrow) sdfl_geglu{in_features, out_features};
    if (!p) return cuda_fail(cudaErrorMemoryAllocation);
    *op = p;
    return SDFL_OK;
}

int sdfl_geglu_weight_shape(const sdfl_geglu *op, int64_t weight_shape[2]) {
    if (!op || !weight_shape) return SDFL_ERR_INVALID_POINTER;
    weight_shape[0] = 2 * op->out_features;          // NN/GEGLU.cpp:36
    weight_shape[1] = op->in_features;
    return SDFL_OK;
}

int sdfl_geglu_op_forward(sdfl_geglu *op, const void *projected, void *out, int64_t rows, int dtype,
                          void *stream) {
    if (!op) return SDFL_ERR_INVALID_POINTER;
    return sdfl_gelu_multiply(projected, out, rows, op->out_features, dtype, stream);
}

int sdfl_geglu_destroy(sdfl_geglu *op) {
    delete op;
    return SDFL_OK;
}

// ---- host-buffer pipeline ---------------------------------------------------------------------

int sdfl_host_pipeline_create(sdfl_host_pipeline **pipe, size_t max_slot_bytes, int depth) {
    if (!pipe) return SDFL_ERR_INVALID_POINTER;
    *pipe = nullptr;
    if (max_slot_bytes == 0 || depth < 1 || depth > 16) return SDFL_ERR_INVALID_VALUE;
    sdfl_host_pipeline *p = nullptr;
    try {
        p = new sdfl_host_pipeline;
        p->slots.resize(static_cast<size_t>(depth));
    } catch (...) {              // no exception crosses the C boundary
        delete p;
        return cuda_fail(cudaErrorMemoryAllocation);
    }
    cudaError_t e = cudaGetDevice(&p->device);
    p->slot_bytes = (max_slot_bytes + 255) / 256 * 256;
    p->ws_bytes = 1 << 20;
    for (auto &s : p->slots) {
        if (e == cudaSuccess) e = cudaMalloc(&s.d_in, p->slot_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&s.d_out, p->slot_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&s.d_ws, p->ws_bytes);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking);
    }
    if (e != cudaSuccess) {
        sdfl_host_pipeline_destroy(p);
        return cuda_fail(e);
    }
    *pipe = p;
    return SDFL_OK;
}

int sdfl_host_pipeline_destroy(sdfl_host_pipeline *pipe) {
    if (!pipe) return SDFL_OK;
    for (auto &s : pipe->slots) {
        if (s.stream) { cudaStreamSynchronize(s.stream); cudaStreamDestroy(s.stream); }
        if (s.d_in) cudaFree(s.d_in);
        if (s.d_out) cudaFree(s.d_out);
        if (s.d_ws) cudaFree(s.d_ws);
    }
    delete pipe;
    return SDFL_OK;
}

int sdfl_groupnorm_forward_host_async(sdfl_host_pipeline *pipe, const void *h_in, void *h_out,
                                      const float *gamma, const float *beta, int64_t batch,
                                      int64_t channels, int64_t hw, int64_t num_groups, float eps,
                                      int fuse_silu, int dtype) {
    if (!pipe) return SDFL_ERR_INVALID_POINTER;
    int rc = gn_validate(h_in, h_out, gamma, beta, batch, channels, hw, num_groups, eps, dtype);
    if (rc != SDFL_OK) return rc;
    if (batch == 0 || hw == 0) return SDFL_OK;
    int current = -1;
    cudaError_t e = cudaGetDevice(&current);
    if (e != cudaSuccess) return cuda_fail(e);
    if (current != pipe->device) return SDFL_ERR_INVALID_VALUE;   // the slots live on another device
    // One pipeline step = a run of whole groups of one image, as many as fit a slot (and at
    // most ~32 MiB so that copy-in, kernel and copy-out of different steps overlap).
    const int64_t cpg = channels / num_groups;
    const int64_t group_bytes = cpg * hw * esize(dtype);
    int64_t limit = static_cast<int64_t>(pipe->slot_bytes);
    if (limit > (32ll << 20)) limit = 32ll << 20;
    int64_t gps = limit / group_bytes;            // groups per step
    if (gps < 1) {
        if (group_bytes > static_cast<int64_t>(pipe->slot_bytes)) return SDFL_ERR_WORKSPACE;
        gps = 1;
    }
    if (gps > num_groups) gps = num_groups;
    const char *src = static_cast<const char *>(h_in);
    char *dst = static_cast<char *>(h_out);
    for (int64_t n = 0; n < batch && rc == SDFL_OK && e == cudaSuccess; ++n) {
        for (int64_t g0 = 0; g0 < num_groups; g0 += gps) {
            const int64_t ng = g0 + gps <= num_groups ? gps : num_groups - g0;
            auto &s = pipe->slots[pipe->next++ % pipe->slots.size()];
            const size_t off = static_cast<size_t>((n * num_groups + g0) * group_bytes);
            const size_t bytes = static_cast<size_t>(ng * group_bytes);
            e = cudaMemcpyAsync(s.d_in, src + off, bytes, cudaMemcpyHostToDevice, s.stream);
            if (e != cudaSuccess) break;
            rc = gn_forward(s.d_in, s.d_out, gamma + g0 * cpg, beta + g0 * cpg, 1, ng * cpg, hw, ng,
                            eps, fuse_silu, dtype, s.d_ws, pipe->ws_bytes, SDFL_GN_AUTO, 0, s.stream);
            if (rc != SDFL_OK) break;
            e = cudaMemcpyAsync(dst + off, s.d_out, bytes, cudaMemcpyDeviceToHost, s.stream);
            if (e != cudaSuccess) break;
        }
    }
    if (rc != SDFL_OK) return rc;
    return wrap(e);
}

int sdfl_host_pipeline_sync(sdfl_host_pipeline *pipe) {
    if (!pipe) return SDFL_ERR_INVALID_POINTER;
    cudaError_t e = cudaSuccess;
    for (auto &s : pipe->slots) {
        cudaError_t se = cudaStreamSynchronize(s.stream);
        if (e == cudaSuccess) e = se;
    }
    return wrap(e);
}

int sdfl_groupnorm_forward_host(sdfl_host_pipeline *pipe, const void *h_in, void *h_out,
                                const float *gamma, const float *beta, int64_t batch,
                                int64_t channels, int64_t hw, int64_t num_groups, float eps,
                                int fuse_silu, int dtype) {
    const int rc = sdfl_groupnorm_forward_host_async(pipe, h_in, h_out, gamma, beta, batch, channels, hw,
                                                     num_groups, eps, fuse_silu, dtype);
    const int rs = sdfl_host_pipeline_sync(pipe);      // drain also after a failed enqueue
    return rc != SDFL_OK ? rc : rs;
}

int sdfl_host_alloc(void **h_ptr, size_t bytes) {
    if (!h_ptr) return SDFL_ERR_INVALID_POINTER;
    return wrap(cudaHostAlloc(h_ptr, bytes, cudaHostAllocDefault));
}

int sdfl_host_free(void *h_ptr) {
    if (!h_ptr) return SDFL_OK;
    return wrap(cudaFreeHost(h_ptr));
}

}  // extern "C"
