// Host-side helpers shared by the C-ABI entry points: TMA descriptor encoding through the
// driver entry point (no link-time dependency on libcuda), cached device properties, per-device
// one-time kernel configuration and the library's run-time options.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <atomic>

#include "../../include/msl.h"

namespace msl {

int sm_count();

// Current value of a run-time option (MSL_OPT_*).  The defaults come from the environment, read once
// when the first option is looked up; msl_set_option changes them afterwards.
int option(int which);

// One-time, per-device configuration of a kernel: the dynamic shared-memory limit is an attribute of
// (function, device), so a process that drives several GPUs must raise it on each of them.  One object
// per kernel instantiation (a function-local static at the launch site).
struct SmemConfig {
  std::atomic<uint64_t> done{0};          // bit d: configured on device d
  template <class Kernel>
  int ensure(Kernel* kernel, int bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MSL_ERR_CUDA;
    const uint64_t bit = 1ull << dev;
    if (done.load(std::memory_order_acquire) & bit) return MSL_OK;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
      return MSL_ERR_CUDA;
    done.fetch_or(bit, std::memory_order_release);
    return MSL_OK;
  }
};

// 2-D tensor map over a row-major matrix: `cols` elements per row (innermost), `rows` rows,
// `row_pitch_bytes` between rows; the box is box_cols x box_rows elements.
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t cols,
                 uint64_t rows, uint64_t row_pitch_bytes, uint32_t box_cols, uint32_t box_rows,
                 CUtensorMapSwizzle swizzle);

// 3-D tensor map (innermost first): dims d0 x d1 x d2 with byte pitches p1 (between d1 steps)
// and p2 (between d2 steps); box b0 x b1 x b2.
int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, uint64_t d0, uint64_t d1,
                 uint64_t d2, uint64_t p1, uint64_t p2, uint32_t b0, uint32_t b1, uint32_t b2,
                 CUtensorMapSwizzle swizzle);

}  // namespace msl
