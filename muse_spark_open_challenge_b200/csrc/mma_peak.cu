// Measured tensor-core ceilings for the roofline denominators that the pool's peak file does not hold
// (FP8 and NVFP4): every SM issues the same tcgen05.mma back to back on operands that already sit in shared
// memory (no loads, no epilogue), so the rate is what the instruction shape itself can reach.  The shapes
// are the ones the kernels of this library issue: kind::f16 (bf16) M128 x N x K16, kind::f8f6f4 (e4m3)
// M128 x N x K32 as in the attention kernel, kind::mxf4nvf4 block-scaled M128 x N x K64 as in the opt-in
// expert mode.  The reference has no such probe; its roofline model uses the vendor's dense figures
// (muse_prefill_layer/reference.py:681-697).
#include "msl_common.cuh"
#include "msl_host.h"

namespace msl {

__device__ __forceinline__ void peak_cp_scales(uint32_t taddr, uint32_t saddr) {
  const uint64_t desc = make_sdesc(saddr, 16, 128, 0);
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void peak_mma_nvf4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa,
                                              uint32_t sfb, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}

// KIND: 0 = bf16, 1 = e4m3, 2 = nvfp4 (block scaled).  One CTA per SM, 128 threads.  Shared memory: an A
// tile of 128 rows x 128 B and a B tile of 256 rows x 128 B (128-byte swizzle, zero-filled), one scale atom.
template <int KIND>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int n, int iters, int* status) {
  extern __shared__ __align__(1024) uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sa = smem;
  uint8_t* sb = smem + 16384;
  uint8_t* sf = smem + 16384 + 32768;
  uint64_t* bar = reinterpret_cast<uint64_t*>(sf + 512);
  uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 1);
  for (int i = threadIdx.x; i < (16384 + 32768 + 512) / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) { mbar_init(bar, 1); mbar_fence_init(); }
  if (threadIdx.x < 32) tmem_alloc(slot, 512);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t base = *slot;
  if (threadIdx.x == 0) {
    // 128-byte rows hold 4 K steps (bf16: 4 x 16, e4m3: 4 x 32, e2m1: 4 x 64 elements)
    if constexpr (KIND == 2) {
      for (int c = 0; c < 8; ++c) peak_cp_scales(base + 448 + 4 * c, smem_u32(sf));     // SFA 4 + SFB up to 8 columns
      const uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | ((128u >> 4) << 24);
      for (int i = 0; i < iters; ++i)
        peak_mma_nvf4(base, make_sdesc(smem_u32(sa) + (i & 3) * 32, 16, 1024, 2),
                      make_sdesc(smem_u32(sb) + (i & 3) * 32, 16, 1024, 2), idesc, base + 448, base + 452, i != 0);
    } else {
      const uint32_t idesc = KIND == 0 ? make_idesc(1, 1, 128, n) : make_idesc(0, 0, 128, n);
      for (int i = 0; i < iters; ++i) {
        const uint64_t da = make_sdesc(smem_u32(sa) + (i & 3) * 32, 16, 1024, 2);
        const uint64_t db = make_sdesc(smem_u32(sb) + (i & 3) * 32, 16, 1024, 2);
        if constexpr (KIND == 0) tc_mma_f16(base, da, db, idesc, i != 0);
        else tc_mma_f8(base, da, db, idesc, i != 0);
      }
    }
    tc_commit(bar);
    if (!mbar_wait(bar, 0)) report_error(status, MSL_ERR_DEVICE_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(base, 512);
}

}  // namespace msl

using namespace msl;

extern "C" int msl_mma_peak(int kind, int n, int iters, int* status, void* stream) {
  if (kind < 0 || kind > 2 || iters <= 0 || iters > (1 << 22) || n < 16 || n > 256 || (n & 15)) return MSL_ERR_ARG;
  const int smem = 16384 + 32768 + 512 + 64 + 1024;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = sm_count();
  static SmemConfig c0, c1, c2;
  if (kind == 0) {
    if (int rc = c0.ensure(mma_peak_kernel<0>, smem)) return rc;
    mma_peak_kernel<0><<<grid, 128, smem, st>>>(n, iters, status);
  } else if (kind == 1) {
    if (int rc = c1.ensure(mma_peak_kernel<1>, smem)) return rc;
    mma_peak_kernel<1><<<grid, 128, smem, st>>>(n, iters, status);
  } else {
    if (int rc = c2.ensure(mma_peak_kernel<2>, smem)) return rc;
    mma_peak_kernel<2><<<grid, 128, smem, st>>>(n, iters, status);
  }
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}
