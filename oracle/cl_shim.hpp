// TEST INFRASTRUCTURE ONLY -- part of the CPU checker, never of the product path.
//
// A minimal OpenCL C execution environment for a host CPU, so that the reference's `.cl`
// kernel files can be #included UNCHANGED into a C++ translation unit and run:
//   * address-space and kernel qualifiers become empty macros,
//   * work-item id functions read the state of the work-item that is currently running,
//   * `barrier()` is a cooperative yield between the work-items (fibers) of one work-group,
//   * the math built-ins resolve to the <cmath> float overloads (OpenCL C `exp(float)` is a
//     float function; so is `std::exp(float)`).
// The header knows nothing about the reference's files; `ref_harness.cpp` includes them.
#pragma once

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <algorithm>

#define __kernel
#define __global
#define __local
#define __constant static const
#define CLK_LOCAL_MEM_FENCE 1
#define CLK_GLOBAL_MEM_FENCE 2
#ifndef M_SQRT1_2_F
#define M_SQRT1_2_F 0.70710678118654752440f
#endif
#ifndef M_2_PI_F
#define M_2_PI_F 0.63661977236758134308f
#endif

namespace clshim {

// Identity of one work-item inside an NDRange of up to three dimensions.
struct WorkItem {
    size_t global_id[3];
    size_t local_id[3];
    size_t group_id[3];
};

// Geometry shared by all work-items of the running NDRange.
struct Range {
    size_t global_size[3];
    size_t local_size[3];
    size_t global_offset[3];
};

struct Fiber;

// Per host thread: the work-item now running, the range, and (inside a work-group that
// uses barriers) the fiber to yield from.
struct ThreadState {
    WorkItem item;
    Range range;
    Fiber *fiber;   // nullptr when the kernel runs as a plain loop (no barrier allowed)
};

extern thread_local ThreadState tls;

void fiber_barrier();   // defined in ref_harness.cpp

}  // namespace clshim

static inline size_t get_global_id(unsigned d) { return clshim::tls.item.global_id[d]; }
static inline size_t get_local_id(unsigned d) { return clshim::tls.item.local_id[d]; }
static inline size_t get_group_id(unsigned d) { return clshim::tls.item.group_id[d]; }
static inline size_t get_global_size(unsigned d) { return clshim::tls.range.global_size[d]; }
static inline size_t get_local_size(unsigned d) { return clshim::tls.range.local_size[d]; }
static inline size_t get_global_offset(unsigned d) { return clshim::tls.range.global_offset[d]; }
static inline void barrier(int) { clshim::fiber_barrier(); }

using std::exp;
using std::erf;
using std::sqrt;
using std::fma;
using std::tanh;
using std::max;
using std::min;
static inline float pown(float x, int n) { return std::pow(x, static_cast<float>(n)); }
