// Host utilities: driver entry point lookup for cuTensorMapEncodeTiled, device property cache,
// run-time options, status strings.
#include <cudaTypedefs.h>

#include <cstdlib>
#include <mutex>

#include "msl_host.h"

namespace msl {

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Run-time options.  Their defaults are taken from the environment exactly once (the first look-up), so
// what a later launch does never depends on an environment change made in between; msl_set_option is the
// way to change one afterwards.
static std::atomic<int> g_options[MSL_OPT_COUNT];
static void init_options() {
  static std::once_flag once;
  std::call_once(once, [] {
    static const char* const names[MSL_OPT_COUNT] = {"MSL_GEMM_SPLITK", "MSL_GEMM_WIDE", "MSL_GROUPED_WIDE"};
    for (int i = 0; i < MSL_OPT_COUNT; ++i) {
      const char* env = getenv(names[i]);
      g_options[i].store(env && env[0] == '0' ? 0 : 1, std::memory_order_relaxed);
    }
  });
}
int option(int which) {
  if (which < 0 || which >= MSL_OPT_COUNT) return 0;
  init_options();
  return g_options[which].load(std::memory_order_relaxed);
}

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t cols,
                 uint64_t rows, uint64_t row_pitch_bytes, uint32_t box_cols, uint32_t box_rows,
                 CUtensorMapSwizzle swizzle) {
  auto fn = encode_fn();
  if (!fn) return MSL_ERR_CUDA;
  (void)elem_bytes;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MSL_OK : MSL_ERR_TENSORMAP;
}

int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, uint64_t d0, uint64_t d1,
                 uint64_t d2, uint64_t p1, uint64_t p2, uint32_t b0, uint32_t b1, uint32_t b2,
                 CUtensorMapSwizzle swizzle) {
  auto fn = encode_fn();
  if (!fn) return MSL_ERR_CUDA;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {p1, p2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dtype, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MSL_OK : MSL_ERR_TENSORMAP;
}

}  // namespace msl

extern "C" const char* msl_status_string(int code) {
  switch (code) {
    case MSL_OK: return "ok";
    case MSL_ERR_ARG: return "invalid argument";
    case MSL_ERR_ALIGN: return "pointer, pitch or size not aligned as required";
    case MSL_ERR_CUDA: return "CUDA runtime or driver call failed";
    case MSL_ERR_TENSORMAP: return "tensor map encoding failed";
    case MSL_ERR_DEVICE_TIMEOUT: return "a device-side wait ran out of time";
    case MSL_ERR_CAPACITY: return "a fixed-capacity buffer would overflow";
    case MSL_ERR_UNSUPPORTED: return "shape not supported by this build";
    default: return "unknown status";
  }
}

extern "C" int msl_abi_version(void) { return MSL_ABI_VERSION; }

extern "C" int msl_set_option(int option, int value) {
  if (option < 0 || option >= MSL_OPT_COUNT || (value != 0 && value != 1)) return MSL_ERR_ARG;
  msl::init_options();
  msl::g_options[option].store(value, std::memory_order_relaxed);
  return MSL_OK;
}

extern "C" int msl_get_option(int option) {
  if (option < 0 || option >= MSL_OPT_COUNT) return MSL_ERR_ARG;
  return msl::option(option);
}
