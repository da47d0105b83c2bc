// TEST INFRASTRUCTURE ONLY -- part of the CPU checker, never of the product path.
//
// Compiles the reference's OpenCL C kernel files, unchanged and from where they lie, as C++
// (through cl_shim.hpp) and launches them with the NDRange arithmetic of the reference's host
// operators.  The build recipe is oracle/Makefile (target `ref`); the only output is
// oracle/_ref/libsdfl_ref.so.  No reference source text is copied into this repository: the
// kernel files are pulled in by #include at build time via -I<reference>/app/src/main/assets/kernel.
//
// What is mine here: the work-item scheduler (fibers so that `barrier()` works), the launch
// helpers, and the C entry points.  What is the reference's: every line of arithmetic.
//
// Reference host code whose launch shapes are followed (paths inside the reference project):
//   app/src/main/cpp/modules/nn/GroupNorm.cpp:68-170      GroupNorm::forward
//   app/src/main/cpp/modules/nn/LayerNorm.cpp:66-162      LayerNorm::forward
//   app/src/main/cpp/modules/nn/GEGLU.cpp:48-84           GEGLU::forward (gelu_multiply stage)
//   app/src/main/cpp/modules/nn/ResBlock.cpp:136-142      silu launch
//   app/src/main/cpp/modules/nn/ResidualAttentionBlock.cpp:146-153  gelu launch
//   app/src/main/cpp/modules/TextEncoder.cpp:141-151      elemwise_add launch
//   app/src/main/cpp/modules/nn/MultiHeadAttention.cpp:213-225  local_softmax launch

#include "cl_shim.hpp"

#include <cstdio>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

// ----------------------------------------------------------------------------------------
// The reference kernels.  group_norm.cl and layer_norm.cl both define local_reduction_mean /
// local_reduction_variance, so each file gets its own namespace.
// ----------------------------------------------------------------------------------------
#pragma GCC diagnostic push
#pragma GCC diagnostic ignored "-Wsign-compare"
#pragma GCC diagnostic ignored "-Wunused-variable"
#pragma GCC diagnostic ignored "-Wunused-function"
namespace ref_gn {
#include "group_norm.cl"
}
namespace ref_ln {
#include "layer_norm.cl"
}
namespace ref_geglu {
#include "geglu.cl"
}
namespace ref_util {
#include "util.cl"
}
namespace ref_up {
#include "up_sample.cl"
}
namespace ref_mha {
#include "multi_head_attention.cl"
}
#pragma GCC diagnostic pop

// ----------------------------------------------------------------------------------------
// Fibers: one per work-item of a work-group, switched cooperatively at barrier().
// ----------------------------------------------------------------------------------------
#if defined(__x86_64__)
extern "C" void clshim_switch(void **save_sp, void *load_sp);
asm(R"(
.text
.globl clshim_switch
.type clshim_switch,@function
clshim_switch:
    pushq %rbp
    pushq %rbx
    pushq %r12
    pushq %r13
    pushq %r14
    pushq %r15
    movq %rsp, (%rdi)
    movq %rsi, %rsp
    popq %r15
    popq %r14
    popq %r13
    popq %r12
    popq %rbx
    popq %rbp
    ret
.size clshim_switch,.-clshim_switch
)");
#define CLSHIM_ASM_SWITCH 1
#else
#include <ucontext.h>
#define CLSHIM_ASM_SWITCH 0
#endif

namespace clshim {

thread_local ThreadState tls;

constexpr size_t kFiberStackBytes = 32 * 1024;

struct Fiber {
    WorkItem item;
    bool done;
    void (*entry)(void *);
    void *arg;
#if CLSHIM_ASM_SWITCH
    void *sp;
    void **sched_sp;
#else
    ucontext_t ctx;
    ucontext_t *sched_ctx;
#endif
    char *stack;
};

struct FiberPool {
    std::vector<Fiber> fibers;
    std::vector<char *> stacks;
    ~FiberPool() { for (char *s : stacks) std::free(s); }
    void reserve(size_t n) {
        while (stacks.size() < n) {
            void *p = nullptr;
            if (posix_memalign(&p, 64, kFiberStackBytes) != 0) std::abort();
            stacks.push_back(static_cast<char *>(p));
        }
        if (fibers.size() < n) fibers.resize(n);
    }
};

static thread_local FiberPool tl_pool;

static void fiber_main() {
    Fiber *f = tls.fiber;
    f->entry(f->arg);
    f->done = true;
#if CLSHIM_ASM_SWITCH
    void *dummy;
    clshim_switch(&dummy, *f->sched_sp);
#else
    swapcontext(&f->ctx, f->sched_ctx);
#endif
    std::abort();   // a finished fiber is never resumed
}

void fiber_barrier() {
    Fiber *f = tls.fiber;
    if (f == nullptr) {
        std::fprintf(stderr, "clshim: barrier() in a kernel launched without work-groups\n");
        std::abort();
    }
#if CLSHIM_ASM_SWITCH
    clshim_switch(&f->sp, *f->sched_sp);
#else
    swapcontext(&f->ctx, f->sched_ctx);
#endif
}

// Run the `local` work-items of work-group `group` (1-D range) to completion.  Work-items are
// resumed in id order; each runs until its next barrier() or its end, which is exactly the
// barrier contract as long as every item meets the same barriers (OpenCL requires that).
static void run_group_1d(void (*entry)(void *), void *arg, size_t group, size_t local) {
    FiberPool &pool = tl_pool;
    pool.reserve(local);
#if CLSHIM_ASM_SWITCH
    void *sched_sp = nullptr;
#else
    ucontext_t sched_ctx;
#endif
    for (size_t l = 0; l < local; ++l) {
        Fiber &f = pool.fibers[l];
        f.item = WorkItem{{group * local + l, 0, 0}, {l, 0, 0}, {group, 0, 0}};
        f.done = false;
        f.entry = entry;
        f.arg = arg;
        f.stack = pool.stacks[l];
#if CLSHIM_ASM_SWITCH
        uintptr_t top = (reinterpret_cast<uintptr_t>(f.stack) + kFiberStackBytes) & ~uintptr_t(15);
        void **s = reinterpret_cast<void **>(top);
        *--s = nullptr;                                   // fake return address of fiber_main
        *--s = reinterpret_cast<void *>(&fiber_main);     // popped by the first `ret`
        for (int r = 0; r < 6; ++r) *--s = nullptr;       // rbp rbx r12 r13 r14 r15
        f.sp = s;
        f.sched_sp = &sched_sp;
#else
        getcontext(&f.ctx);
        f.ctx.uc_stack.ss_sp = f.stack;
        f.ctx.uc_stack.ss_size = kFiberStackBytes;
        f.ctx.uc_link = nullptr;
        f.sched_ctx = &sched_ctx;
        makecontext(&f.ctx, fiber_main, 0);
#endif
    }
    size_t remaining = local;
    while (remaining) {
        for (size_t l = 0; l < local; ++l) {
            Fiber &f = pool.fibers[l];
            if (f.done) continue;
            tls.item = f.item;
            tls.fiber = &f;
#if CLSHIM_ASM_SWITCH
            clshim_switch(&sched_sp, f.sp);
#else
            swapcontext(&sched_ctx, &f.ctx);
#endif
            if (f.done) --remaining;
        }
    }
    tls.fiber = nullptr;
}

// clEnqueueNDRangeKernel(queue, k, 1, NULL, {global}, {local}, ...) for kernels with barriers.
template <class Args>
static void enqueue_1d_groups(size_t global, size_t local, void (*entry)(void *), Args *args) {
    const long groups = static_cast<long>(global / local);
#pragma omp parallel for schedule(static)
    for (long g = 0; g < groups; ++g) {
        tls.range = Range{{global, 1, 1}, {local, 1, 1}, {0, 0, 0}};
        run_group_1d(entry, args, static_cast<size_t>(g), local);
    }
}

// clEnqueueNDRangeKernel(queue, k, 3, NULL, {gx, gy, gz}, NULL, ...) for barrier-free kernels
// (local size 1 in every dimension, so group id == global id).
template <class F>
static void enqueue_3d_flat(size_t gx, size_t gy, size_t gz, F &&body) {
#pragma omp parallel
    {
        tls.range = Range{{gx, gy, gz}, {1, 1, 1}, {0, 0, 0}};
        tls.fiber = nullptr;
#pragma omp for schedule(static) collapse(2)
        for (long x = 0; x < static_cast<long>(gx); ++x)
            for (long y = 0; y < static_cast<long>(gy); ++y)
                for (size_t z = 0; z < gz; ++z) {
                    const size_t id[3] = {static_cast<size_t>(x), static_cast<size_t>(y), z};
                    for (int d = 0; d < 3; ++d) {
                        tls.item.global_id[d] = id[d];
                        tls.item.group_id[d] = id[d];
                        tls.item.local_id[d] = 0;
                    }
                    body();
                }
    }
}

// clEnqueueNDRangeKernel(queue, k, 1, NULL, {global}, NULL, ...) for barrier-free kernels.
template <class F>
static void enqueue_1d_flat(size_t global, F &&body) {
#pragma omp parallel
    {
        tls.range = Range{{global, 1, 1}, {1, 1, 1}, {0, 0, 0}};
        tls.fiber = nullptr;
#pragma omp for schedule(static)
        for (long i = 0; i < static_cast<long>(global); ++i) {
            tls.item.global_id[0] = static_cast<size_t>(i);
            tls.item.group_id[0] = static_cast<size_t>(i);
            tls.item.local_id[0] = 0;
            body();
        }
    }
}

// clEnqueueNDRangeKernel(queue, k, 2, NULL, {g0, g1}, NULL, ...) for barrier-free kernels.
template <class F>
static void enqueue_2d_flat(size_t g0, size_t g1, F &&body) {
#pragma omp parallel
    {
        tls.range = Range{{g0, g1, 1}, {1, 1, 1}, {0, 0, 0}};
        tls.fiber = nullptr;
#pragma omp for schedule(static)
        for (long i = 0; i < static_cast<long>(g0); ++i) {
            tls.item.global_id[0] = static_cast<size_t>(i);
            tls.item.group_id[0] = static_cast<size_t>(i);
            for (size_t j = 0; j < g1; ++j) {
                tls.item.global_id[1] = j;
                tls.item.group_id[1] = j;
                body();
            }
        }
    }
}

}  // namespace clshim

using clshim::enqueue_1d_flat;
using clshim::enqueue_1d_groups;
using clshim::enqueue_2d_flat;
using clshim::enqueue_3d_flat;

namespace {

constexpr size_t WORK_GROUP_SIZE = 64;   // nn/GroupNorm.cpp:13, nn/LayerNorm.cpp:11

struct MeanArgs { const float *in; float *out; size_t reductionSize; };
struct VarArgs { const float *in; const float *mean; float *out; size_t reductionSize; };

// The __local scratch is sized like the reference sets it (sizeof(float) * 64 per group).
void gn_mean_entry(void *p) {
    static thread_local float scratch[WORK_GROUP_SIZE];
    auto *a = static_cast<MeanArgs *>(p);
    ref_gn::local_reduction_mean(a->in, a->out, scratch, a->reductionSize);
}
void gn_var_entry(void *p) {
    static thread_local float scratch[WORK_GROUP_SIZE];
    auto *a = static_cast<VarArgs *>(p);
    ref_gn::local_reduction_variance(a->in, a->mean, a->out, scratch, a->reductionSize);
}
struct SoftmaxArgs { const float *in; float *out; size_t chunkSize; };
// __local reductionSums[workGroupSize] and cache[chunkSize], as nn/CrossAttention.cpp:367-368 sizes them.
void softmax_entry(void *p) {
    static thread_local float sums[WORK_GROUP_SIZE];
    static thread_local std::vector<float> cache;
    auto *a = static_cast<SoftmaxArgs *>(p);
    if (cache.size() < a->chunkSize) cache.resize(a->chunkSize);   // same for every fiber of the group
    ref_util::softmax(a->in, a->out, sums, cache.data(), a->chunkSize);
}
struct LocalSoftmaxArgs { const float *in; float *out; };
// __local reductionSums[CONTEXT_LENGTH], as nn/MultiHeadAttention.cpp:215 sizes it (one float per work-item).
void local_softmax_entry(void *p) {
    static thread_local std::vector<float> sums;
    auto *a = static_cast<LocalSoftmaxArgs *>(p);
    const size_t local = get_local_size(0);
    if (sums.size() < local) sums.resize(local);                   // same for every fiber of the group
    ref_mha::local_softmax(a->in, a->out, sums.data());
}
void ln_mean_entry(void *p) {
    static thread_local float scratch[WORK_GROUP_SIZE];
    auto *a = static_cast<MeanArgs *>(p);
    ref_ln::local_reduction_mean(a->in, a->out, scratch, a->reductionSize);
}
void ln_var_entry(void *p) {
    static thread_local float scratch[WORK_GROUP_SIZE];
    auto *a = static_cast<VarArgs *>(p);
    ref_ln::local_reduction_variance(a->in, a->mean, a->out, scratch, a->reductionSize);
}

}  // namespace

extern "C" {

int ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void ref_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// The three per-kernel launches of GroupNorm, individually callable (group_norm.cl).
// `groups` work-groups of 64 items, each item summing `reductionSize` strided elements.
void ref_gn_local_reduction_mean(const float *in, float *out, size_t groups, size_t reductionSize) {
    MeanArgs a{in, out, reductionSize};
    enqueue_1d_groups(groups * WORK_GROUP_SIZE, WORK_GROUP_SIZE, gn_mean_entry, &a);
}

void ref_gn_local_reduction_variance(const float *in, const float *mean, float *out, size_t groups,
                                     size_t reductionSize) {
    VarArgs a{in, mean, out, reductionSize};
    enqueue_1d_groups(groups * WORK_GROUP_SIZE, WORK_GROUP_SIZE, gn_var_entry, &a);
}

void ref_gn_group_norm(const float *in, const float *mean, const float *variance, const float *weight,
                       const float *bias, size_t groupSize, size_t channelSize, float epsilon,
                       float *out, size_t global) {
    enqueue_1d_flat(global, [=] {
        ref_gn::group_norm(in, mean, variance, weight, bias, groupSize, channelSize, epsilon, out);
    });
}

// GroupNorm::forward for ONE image (the reference has no batch): same size derivations, same
// two contract checks (returned as -1 / -2 where the reference throws), same three launches.
// `mean_out` / `var_out` (each [num_groups], may be NULL) expose the intermediate buffers the
// reference inspects at nn/LayerNorm.cpp:108-124.
int ref_group_norm_forward(const float *in, float *out, const float *weight, const float *bias,
                           size_t input_size, size_t num_groups, size_t num_channels, float eps,
                           float *mean_out, float *var_out) {
    const size_t weightSize = num_channels;
    const size_t groupSize = input_size / num_groups;
    const size_t reductionSize = groupSize / WORK_GROUP_SIZE;
    if (input_size % weightSize != 0) return -1;
    if (groupSize % WORK_GROUP_SIZE != 0) return -2;
    std::vector<float> mean(num_groups), var(num_groups);
    ref_gn_local_reduction_mean(in, mean.data(), num_groups, reductionSize);
    ref_gn_local_reduction_variance(in, mean.data(), var.data(), num_groups, reductionSize);
    const size_t channelSize = input_size / num_channels;
    ref_gn_group_norm(in, mean.data(), var.data(), weight, bias, groupSize, channelSize, eps, out,
                      input_size);
    if (mean_out) std::memcpy(mean_out, mean.data(), sizeof(float) * num_groups);
    if (var_out) std::memcpy(var_out, var.data(), sizeof(float) * num_groups);
    return 0;
}

void ref_silu(const float *src, float *dst, size_t n) {
    enqueue_1d_flat(n, [=] { ref_util::silu(const_cast<float *>(src), dst); });
}

void ref_gelu(const float *src, float *dst, size_t n) {
    enqueue_1d_flat(n, [=] { ref_util::gelu(const_cast<float *>(src), dst); });
}

// up_sample_nearest as launched at nn/UpSample.cpp:93-102: global size {channels, height, height}.
void ref_up_sample_nearest(const float *in, float *out, size_t channels, size_t height, size_t scale) {
    enqueue_3d_flat(channels, height, height,
                    [=] { ref_up::up_sample_nearest(const_cast<float *>(in), out, scale); });
}

// softmax as launched at nn/CrossAttention.cpp:365-378: one work-group of 64 per row of chunkSize.
void ref_softmax(const float *in, float *out, size_t rows, size_t chunkSize) {
    SoftmaxArgs a{in, out, chunkSize};
    enqueue_1d_groups(rows * WORK_GROUP_SIZE, WORK_GROUP_SIZE, softmax_entry, &a);
}

// local_softmax as launched at nn/MultiHeadAttention.cpp:213-225: global size rows * row_len, one
// work-group of row_len work-items per row (row_len = CONTEXT_LENGTH = 77 there, an odd size).
void ref_local_softmax(const float *in, float *out, size_t rows, size_t row_len) {
    LocalSoftmaxArgs a{in, out};
    enqueue_1d_groups(rows * row_len, row_len, local_softmax_entry, &a);
}

// permute3D__0_2_1 as launched at nn/SpatialTransformer.cpp:131-134 / :154-157: global size {I, J, K}.
void ref_permute3D__0_2_1(const float *src, float *dst, size_t I, size_t J, size_t K) {
    enqueue_3d_flat(I, J, K, [=] { ref_util::permute3D__0_2_1(const_cast<float *>(src), dst); });
}

void ref_chunkwise_add(const float *A, const float *chunk, float *C, size_t n, size_t chunk_size) {
    enqueue_1d_flat(n, [=] {
        ref_util::chunkwise_add(const_cast<float *>(A), const_cast<float *>(chunk), C, chunk_size);
    });
}

void ref_elemwise_add(const float *A, const float *B, float *C, size_t n) {
    enqueue_1d_flat(n, [=] {
        ref_util::elemwise_add(const_cast<float *>(A), const_cast<float *>(B), C);
    });
}

// What a caller of the reference does for "GroupNorm then SiLU" on a batch: the reference is
// batch-1, so each image slab goes through GroupNorm::forward on its own, then `silu` runs in
// place on the result (nn/ResBlock.cpp:125-142).
int ref_group_norm_silu_batched(const float *in, float *out, const float *weight, const float *bias,
                                size_t batch, size_t per_image, size_t num_groups,
                                size_t num_channels, float eps, int apply_silu) {
    for (size_t n = 0; n < batch; ++n) {
        int rc = ref_group_norm_forward(in + n * per_image, out + n * per_image, weight, bias,
                                        per_image, num_groups, num_channels, eps, nullptr, nullptr);
        if (rc != 0) return rc;
        if (apply_silu) ref_silu(out + n * per_image, out + n * per_image, per_image);
    }
    return 0;
}

void ref_ln_local_reduction_mean(const float *in, float *out, size_t rows, size_t reductionSize) {
    MeanArgs a{in, out, reductionSize};
    enqueue_1d_groups(rows * WORK_GROUP_SIZE, WORK_GROUP_SIZE, ln_mean_entry, &a);
}

void ref_ln_local_reduction_variance(const float *in, const float *mean, float *out, size_t rows,
                                     size_t reductionSize) {
    VarArgs a{in, mean, out, reductionSize};
    enqueue_1d_groups(rows * WORK_GROUP_SIZE, WORK_GROUP_SIZE, ln_var_entry, &a);
}

void ref_ln_layer_norm(const float *in, const float *mean, const float *variance, const float *weight,
                       const float *bias, size_t chunkSize, float *out, size_t global) {
    enqueue_1d_flat(global, [=] {
        ref_ln::layer_norm(in, mean, variance, weight, bias, chunkSize, out);
    });
}

// LayerNorm::forward: rows = input_size / dim, 64 items per row, eps is the kernel file's constant.
int ref_layer_norm_forward(const float *in, float *out, const float *weight, const float *bias,
                           size_t input_size, size_t dim, float *mean_out, float *var_out) {
    const size_t weightSize = dim;
    if (weightSize % WORK_GROUP_SIZE != 0) return -2;      // LayerNorm::init check
    if (input_size % weightSize != 0) return -1;
    const size_t rows = input_size / weightSize;
    const size_t reductionSize = weightSize / WORK_GROUP_SIZE;
    std::vector<float> mean(rows), var(rows);
    // global size = input_size / reductionSize = rows * 64
    ref_ln_local_reduction_mean(in, mean.data(), rows, reductionSize);
    ref_ln_local_reduction_variance(in, mean.data(), var.data(), rows, reductionSize);
    ref_ln_layer_norm(in, mean.data(), var.data(), weight, bias, weightSize, out, input_size);
    if (mean_out) std::memcpy(mean_out, mean.data(), sizeof(float) * rows);
    if (var_out) std::memcpy(var_out, var.data(), sizeof(float) * rows);
    return 0;
}

// gelu_multiply over a 2-D range {rows, D}; AB is [rows, 2*D], dst is [rows, D].
void ref_gelu_multiply(const float *AB, float *dst, size_t rows, size_t D) {
    enqueue_2d_flat(rows, D, [=] { ref_geglu::gelu_multiply(const_cast<float *>(AB), dst); });
}

}  // extern "C"
