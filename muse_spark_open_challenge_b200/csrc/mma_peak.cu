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

// Issue rate of one scalar-pipe instruction, the other ceiling the attention kernel lives under: every warp of
// the one CTA per SM runs `iters` rounds of 16 independent instances; the longest CTA's clock64 span goes to
// max_cycles[0]; max_cycles[1] collects every warp's results.  OP 0: ex2.approx.ftz.f32 (x <- -ex2(x) stays within [-1, -0.5]); 1: cvt.rn.satfinite.e4m3x2.f32
// (one FP8 pair from two floats); 2: fma.rn.f32; 3: max.f32; 4: two ex2 and one conversion per instance.
template <int OP>
__global__ void __launch_bounds__(512, 1) unit_peak_kernel(int iters, unsigned long long* max_cycles) {
  constexpr int kChains = 16;
  uint32_t r[kChains];
#pragma unroll
  for (int i = 0; i < kChains; ++i) r[i] = 0xbf000000u + ((threadIdx.x * 7u + i) & 0xffffu);   // floats just below -0.5
  __syncthreads();
  const long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < kChains; ++i) {
      float a = __uint_as_float(r[i]);
      const float b = __uint_as_float(r[(i + 1) % kChains]);
      if constexpr (OP == 0) {
        asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(a));
        r[i] = __float_as_uint(-a);
      } else if constexpr (OP == 1) {
        uint16_t h;
        asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h) : "f"(a), "f"(b));
        r[i] = h;                       // fed back as it is: an OR to keep the value normal would cost the ALU pipe 2 cycles
      } else if constexpr (OP == 4) {
        // the softmax mix: two exponentials per converted pair.  The second takes its input from the first
        // (two instances with the same source register would be merged by the assembler)
        asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(a));
        float b2 = a - 1.0f;
        asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(b2));
        uint16_t h;
        asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h) : "f"(a), "f"(b2));
        r[i] = h;
      } else if constexpr (OP == 2) {
        asm volatile("fma.rn.f32 %0, %0, %1, %2;" : "+f"(a) : "f"(0.999f), "f"(-0.0005f));
        r[i] = __float_as_uint(a);
      } else {
        asm volatile("max.f32 %0, %0, %1;" : "+f"(a) : "f"(b));
        r[i] = __float_as_uint(a);
      }
    }
  }
  uint32_t acc = 0;
#pragma unroll
  for (int i = 0; i < kChains; ++i) acc ^= r[i];
  const long long t1 = clock64();
  // every thread's result is observable (word 1), so that no instance of the loop is dead code
  for (int o = 16; o > 0; o >>= 1) acc ^= __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) atomicXor(max_cycles + 1, static_cast<unsigned long long>(acc));
  if (threadIdx.x == 0) atomicMax(max_cycles, static_cast<unsigned long long>(t1 - t0));
}

}  // namespace msl

using namespace msl;

extern "C" int msl_unit_peak(int op, int warps, int iters, unsigned long long* max_cycles, void* stream) {
  if (op < 0 || op > 4 || warps < 1 || warps > 16 || iters <= 0 || iters > (1 << 20) || !max_cycles) return MSL_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = sm_count();
  switch (op) {
    case 0: unit_peak_kernel<0><<<grid, warps * 32, 0, st>>>(iters, max_cycles); break;
    case 1: unit_peak_kernel<1><<<grid, warps * 32, 0, st>>>(iters, max_cycles); break;
    case 2: unit_peak_kernel<2><<<grid, warps * 32, 0, st>>>(iters, max_cycles); break;
    case 4: unit_peak_kernel<4><<<grid, warps * 32, 0, st>>>(iters, max_cycles); break;
    default: unit_peak_kernel<3><<<grid, warps * 32, 0, st>>>(iters, max_cycles); break;
  }
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

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
