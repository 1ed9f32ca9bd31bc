// Dense BF16 GEMM on tcgen05: C[m, n] = sum over K segments of A[m, k] * B[n, k]^T, fp32
// accumulation in tensor memory.
//
// Replaces the cuBLAS calls the reference's layer makes through torch.mm for the QKV+gate, output,
// pooler, unpooler and router projections (muse_prefill_layer/submission.py:1082,1096,1113,1116,
// 1135); the fused SiLU(gate)*up epilogue also serves the BF16 shared expert.
//
// One persistent CTA per SM, 192 threads:
//   warp 0     TMA producer: A tile 128x64 and B tile BNx64 (bf16, 128-byte swizzle) per stage
//   warp 1     allocates tensor memory and issues tcgen05.mma (M=128, N=BN, K=16), 4 per stage
//   warps 2-5  epilogue: tcgen05.ld the fp32 accumulator (one row per thread), convert, store
// Two accumulator buffers (2 x BN columns of TMEM) let the epilogue of one tile overlap the main
// loop of the next.  (A cta_group::2 form of this kernel, two CTAs sharing one M=256 MMA, was built and
// measured at half this kernel's rate: its cross-CTA stage ring has twice the latency shared memory can
// cover.  It is not kept.)  Every mbarrier wait is bounded; a wait that runs out records
// MSL_ERR_DEVICE_TIMEOUT, and all roles fall through to the common teardown that frees the TMEM.
#include "msl_common.cuh"
#include "msl_host.h"

namespace msl {

constexpr int kBM = 128;
constexpr int kBK = 64;

// SUBS = 128-row MMAs per K step that share one B tile: 1 = 128 x BN tiles with two accumulator sets
// (the epilogue of one tile overlaps the main loop of the next); 2 = 256 x 256 tiles with one
// accumulator set (both sub-tiles fill the 512 TMEM columns), which stages and fetches a third fewer
// bytes per FLOP: the single-sub-tile kernel is limited by the L2 -> shared-memory traffic.
template <int BN, int STAGES, int SUBS = 1>
struct GemmSmem {
  static constexpr int kSubBytes = kBM * kBK * 2;
  static constexpr int kABytes = SUBS * kSubBytes;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem base, abort flag
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 4) * 8 + 16;
};

struct GemmArgs {
  void* c;
  int64_t ldc;
  int m, n, k;           // k = elements per segment
  int segs;              // number of K segments accumulated into one output
  int a_seg_stride;      // A column offset (elements) added per segment
  int b_seg_stride;      // B column offset (elements) added per segment
  float alpha;
  int* status;
  // Split-K (splits > 1, fp32 output only): K slice ks of every tile goes to c + ks * split_stride.
  int splits;
  int64_t split_stride;  // elements
};

// Tile order: groups of 16 M-tiles sweep N together so one wave of CTAs re-uses a band of A and
// a band of B out of L2.
__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int& mt, int& nt) {
  constexpr int GM = 16;
  const int per_group = GM * n_tiles;
  const int g = t / per_group;
  const int first = g * GM;
  const int gm = min(GM, m_tiles - first);
  const int r = t - g * per_group;
  mt = first + r % gm;
  nt = r / gm;
}

// SiLU(g) * u = g * u / (1 + exp(-g)) with the fast reciprocal: 2 ulp, far below the bf16 it is rounded to.
// For g < -88 the denominator is +inf and the quotient 0, the limit.
__device__ __forceinline__ float silu_mul(float g, float u) {
  return __fdividef(g * u, 1.0f + __expf(-g));
}

template <int BN, int OUT, int CH>
__device__ __forceinline__ void store_chunk(const GemmArgs& p, int row, int col0, const uint32_t (&acc)[CH],
                                            const uint32_t (&acc2)[CH], bool wide_ok) {
  // One thread owns CH consecutive output columns of one row; 32-byte stores where the output's base and
  // pitch allow them (every lane then writes whole sectors of its own row).
  if (row >= p.m) return;
  if constexpr (OUT == MSL_OUT_F32) {
    float* dst = reinterpret_cast<float*>(p.c) + static_cast<int64_t>(row) * p.ldc + col0;
    if (col0 + CH <= p.n && (p.ldc & 3) == 0) {
#pragma unroll
      for (int j = 0; j < CH; j += 8) {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = __float_as_uint(__uint_as_float(acc[j + i]) * p.alpha);
        if (wide_ok) {
          st_global_v8(dst + j, w);
        } else {
          *reinterpret_cast<uint4*>(dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(dst + j + 4) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
    } else {
      for (int j = 0; j < CH; ++j)
        if (col0 + j < p.n) dst[j] = __uint_as_float(acc[j]) * p.alpha;
    }
  } else {
    float v[CH];
    if constexpr (OUT == MSL_OUT_SWIGLU_BF16) {
#pragma unroll
      for (int j = 0; j < CH; ++j)
        v[j] = silu_mul(__uint_as_float(acc[j]) * p.alpha, __uint_as_float(acc2[j]) * p.alpha);
    } else {
#pragma unroll
      for (int j = 0; j < CH; ++j) v[j] = __uint_as_float(acc[j]) * p.alpha;
    }
    const int n_out = (OUT == MSL_OUT_SWIGLU_BF16) ? p.n / 2 : p.n;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + static_cast<int64_t>(row) * p.ldc + col0;
    if (col0 + CH <= n_out && (p.ldc & 7) == 0) {
#pragma unroll
      for (int j = 0; j < CH; j += 16) {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = pack_bf16x2(v[j + 2 * i], v[j + 2 * i + 1]);
        if (wide_ok) {
          st_global_v8(dst + j, w);
        } else {
          *reinterpret_cast<uint4*>(dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(dst + j + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
    } else {
      for (int j = 0; j < CH; ++j)
        if (col0 + j < n_out) dst[j] = __float2bfloat16(v[j]);
    }
  }
}

template <int BN, int STAGES, int OUT, int SUBS = 1>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, GemmArgs p) {
  using S = GemmSmem<BN, STAGES, SUBS>;
  constexpr int kTileM = kBM * SUBS;
  static_assert(SUBS == 1 || (SUBS == 2 && BN == 256), "two sub-tiles need all 512 TMEM columns");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // The swizzled tiles need 1024-byte alignment; the dynamic window is aligned by hand.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (p.m + kTileM - 1) / kTileM;
  const int n_tiles = (p.n + BN - 1) / BN;
  const int mn_tiles = m_tiles * n_tiles;
  const int total_tiles = mn_tiles * p.splits;             // work item t: K slice t / mn_tiles of tile t % mn_tiles
  const int kb_per_seg = (p.k + kBK - 1) / kBK;
  const int k_blocks = kb_per_seg * p.segs;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_base_slot, 2 * BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one elected lane)
    if (lane == 0) {
      tma_prefetch_desc(&tm_a);
      tma_prefetch_desc(&tm_b);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int mt, nt;
        tile_coords(t % mn_tiles, m_tiles, n_tiles, mt, nt);
        const int ks = t / mn_tiles;
        const int kb_lo = static_cast<int>(static_cast<int64_t>(ks) * k_blocks / p.splits);
        const int kb_hi = static_cast<int>(static_cast<int64_t>(ks + 1) * k_blocks / p.splits);
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (*abort_flag || !mbar_wait(&empty[s], ph ^ 1)) { ok = false; break; }
          const int seg = kb / kb_per_seg;
          const int kk = (kb - seg * kb_per_seg) * kBK;
          uint8_t* sa = smem + s * S::kStageBytes;
          mbar_expect_tx(&full[s], S::kStageBytes);
#pragma unroll
          for (int sub = 0; sub < SUBS; ++sub)
            tma_load_2d(sa + sub * S::kSubBytes, &tm_a, &full[s], seg * p.a_seg_stride + kk, mt * kTileM + sub * kBM);
          tma_load_2d(sa + S::kABytes, &tm_b, &full[s], seg * p.b_seg_stride + kk, nt * BN);
        }
      }
      if (!ok) {
        *abort_flag = 1;
        report_error(p.status, MSL_ERR_DEVICE_TIMEOUT);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // All 32 lanes run the control flow, so that addresses and descriptors are warp-uniform values; one
    // elected lane executes the MMAs and commits.
    {
      const uint32_t on = elect_one();
      constexpr uint32_t idesc = make_idesc(1, 1, kBM, BN);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_i) {
        // one accumulator set (SUBS == 2): index 0, the phase flips every tile; else two sets alternate
        const uint32_t acc = SUBS == 2 ? 0u : (tile_i & 1);
        const uint32_t acc_ph = SUBS == 2 ? (tile_i & 1) : ((tile_i >> 1) & 1);
        if (*abort_flag || !mbar_wait(&tmem_empty[acc], acc_ph ^ 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int ks = t / mn_tiles;
        const int kb_lo = static_cast<int>(static_cast<int64_t>(ks) * k_blocks / p.splits);
        const int kb_hi = static_cast<int>(static_cast<int64_t>(ks + 1) * k_blocks / p.splits);
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (*abort_flag || !mbar_wait(&full[s], ph)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
#pragma unroll
          for (int k16 = 0; k16 < kBK / 16; ++k16) {
            const uint64_t db = make_sdesc(sb + k16 * 32, 16, 1024, 2);
#pragma unroll
            for (int sub = 0; sub < SUBS; ++sub)
              tc_mma_f16_if(on, d_tmem + sub * BN, make_sdesc(sa + sub * S::kSubBytes + k16 * 32, 16, 1024, 2), db,
                            idesc, kb != kb_lo || k16 != 0);
          }
          tc_commit_if(on, &empty[s]);   // frees the stage once these MMAs have read it
        }
        if (ok) tc_commit_if(on, &tmem_full[acc]);
      }
      if (!ok && lane == 0) {
        *abort_flag = 1;
        report_error(p.status, MSL_ERR_DEVICE_TIMEOUT);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter + 32)
    uint32_t tile_i = 0;
    bool ok = true;
    const bool wide_ok = ((reinterpret_cast<uintptr_t>(p.c) | static_cast<uintptr_t>(p.ldc * (OUT == MSL_OUT_F32 ? 4 : 2)) |
                           (OUT == MSL_OUT_F32 ? static_cast<uintptr_t>(p.split_stride * 4) : 0)) & 31) == 0;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_i) {
      int mt, nt;
      tile_coords(t % mn_tiles, m_tiles, n_tiles, mt, nt);
      GemmArgs q = p;                                        // this K slice's output plane
      if constexpr (OUT == MSL_OUT_F32)
        q.c = reinterpret_cast<float*>(p.c) + static_cast<int64_t>(t / mn_tiles) * p.split_stride;
      const uint32_t acc = SUBS == 2 ? 0u : (tile_i & 1);
      const uint32_t acc_ph = SUBS == 2 ? (tile_i & 1) : ((tile_i >> 1) & 1);
      if (*abort_flag || !mbar_wait(&tmem_full[acc], acc_ph)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int sub = 0; sub < SUBS; ++sub) {
      const int row = mt * kTileM + sub * kBM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (acc + sub) * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (mt * kTileM + sub * kBM >= p.m) break;             // a whole sub-tile past the last row
      // The TMEM loads of a chunk are issued one chunk ahead of the arithmetic and the stores.
      if constexpr (OUT == MSL_OUT_SWIGLU_BF16) {
        // Columns [0, BN/2) of the tile are gate rows, [BN/2, BN) the matching up rows.
        uint32_t g[2][16], u[2][16];
        tmem_ld16(taddr, g[0]);
        tmem_ld16(taddr + BN / 2, u[0]);
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          tmem_ld_wait();
          tmem_ld16(taddr + c + 16, g[1]);
          tmem_ld16(taddr + BN / 2 + c + 16, u[1]);
          store_chunk<BN, OUT, 16>(p, row, nt * (BN / 2) + c, g[0], u[0], wide_ok);
          tmem_ld_wait();
          if (c + 32 < BN / 2) {
            tmem_ld16(taddr + c + 32, g[0]);
            tmem_ld16(taddr + BN / 2 + c + 32, u[0]);
          }
          store_chunk<BN, OUT, 16>(p, row, nt * (BN / 2) + c + 16, g[1], u[1], wide_ok);
        }
      } else if (OUT == MSL_OUT_BF16 && wide_ok && (nt + 1) * BN <= p.n) {
        // bf16 rows of a tile that lies inside the output: chunks of 64 columns, transposed within quads so
        // that four lanes write 128 contiguous bytes of one row per instruction (a lane writing 32 bytes of
        // its own row costs the memory pipe one request per lane and per instruction)
        const int q = lane & 3, row_base = row - q;
        __nv_bfloat16* obase = reinterpret_cast<__nv_bfloat16*>(p.c) + static_cast<int64_t>(row_base) * p.ldc + nt * BN + 16 * q;
        uint32_t a[32], b[32];
        tmem_ld32(taddr, a);
        tmem_ld32(taddr + 32, b);
#pragma unroll 1
        for (int c = 0; c < BN; c += 64) {
          tmem_ld_wait();
          uint32_t u[32], f[32];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            u[j / 2] = pack_bf16x2(__uint_as_float(a[j]) * p.alpha, __uint_as_float(a[j + 1]) * p.alpha);
            u[16 + j / 2] = pack_bf16x2(__uint_as_float(b[j]) * p.alpha, __uint_as_float(b[j + 1]) * p.alpha);
          }
          quad_transpose_units(u, f);
          if (c + 64 < BN) {
            tmem_ld32(taddr + c + 64, a);
            tmem_ld32(taddr + c + 96, b);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (row_base + j < p.m) st_global_v8(obase + static_cast<int64_t>(j) * p.ldc + c, &f[8 * j]);
        }
      } else {
        uint32_t v[2][32];
        tmem_ld32(taddr, v[0]);
#pragma unroll 1
        for (int c = 0; c < BN; c += 64) {
          tmem_ld_wait();
          tmem_ld32(taddr + c + 32, v[1]);
          store_chunk<BN, OUT, 32>(q, row, nt * BN + c, v[0], v[0], wide_ok);
          tmem_ld_wait();
          if (c + 64 < BN) tmem_ld32(taddr + c + 64, v[0]);
          store_chunk<BN, OUT, 32>(q, row, nt * BN + c + 32, v[1], v[1], wide_ok);
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      report_error(p.status, MSL_ERR_DEVICE_TIMEOUT);
    }
  }

  // ------------------------------------------------------------ teardown (all roles reach here)
  // Give loads already issued a bounded time to land before the CTA's shared memory goes away.
  if (warp == 0 && lane == 0 && *abort_flag) drain_pause();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int BN, int STAGES, int OUT, int SUBS = 1>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args, cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES, SUBS>;
  const int smem = S::kTotal + 1024;
  static SmemConfig config;         // one per template instance, tracked per device
  if (int rc = config.ensure(gemm_bf16_kernel<BN, STAGES, OUT, SUBS>, smem)) return rc;
  const int m_tiles = (args.m + kBM * SUBS - 1) / (kBM * SUBS);
  const int n_tiles = (args.n + BN - 1) / BN;
  const int grid = std::min(m_tiles * n_tiles * args.splits, sm_count());
  gemm_bf16_kernel<BN, STAGES, OUT, SUBS><<<grid, 192, smem, stream>>>(ta, tb, args);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}


// Sum of the K slices of a split-K product: out[m][n] = alpha * sum_s part[s][m][n], to bf16 or fp32.
// Fixed summation order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ part, int splits, int m, int n, float alpha, void* out, int64_t ldc,
                     int out_f32) {
  const int64_t quads = static_cast<int64_t>(m) * (n / 4);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < quads;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / (n / 4);
    const int col = static_cast<int>(i - row * (n / 4)) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(part + (static_cast<int64_t>(s) * m + row) * n + col);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= alpha; acc.y *= alpha; acc.z *= alpha; acc.w *= alpha;
    if (out_f32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + row * ldc + col) = acc;
    } else {
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + row * ldc + col) =
          make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
    }
  }
}

}  // namespace msl

using namespace msl;

// Choice of tile geometry and K slices from the sizes alone: a cost model in SM cycles.  A 128 x 256 tile takes
// about 880 cycles per 64-wide K step (its 48 KB per step arrive at the 55-60 bytes per clock one SM takes
// from L2; the four MMAs would need 512), a 256 x 256 tile about 1100 (64 KB, 1024 cycles of MMA), a 128 x
// 128 tile about 570; a work item costs a pipeline fill of about 1500 cycles; the epilogue (5000 cycles, 8000
// for 256 rows, 3000 for 128 columns) overlaps the next item's main loop only where there are two accumulator
// sets; the reduction over K slices reads its planes out of L2 at about 4 TB/s behind a launch of about 3 us.
// The step times hold where many row tiles share each weight tile.  Products of 753 rows on weights that come
// from HBM (three to six row tiles) move 7.5-10 TB/s from L2 to the SMs whatever the geometry, and a 256 x 256
// step then takes 1560-2300 cycles; the plans chosen here (QKV 5 slices of 256-row tiles, pooler 3, unpooler
// and output projection 256-row tiles unsliced) ran 41, 56, 52 and 19 us against 41, 58, 58 and 20 us under the
// rule they replace (256-row tiles only when they alone fill every SM, slices only below half a wave).
struct GemmPlan {
  int splits;
  bool wide;
  double cycles;
};

static double gemm_cost(int m, int n, int k_blocks, int bn, bool wide, int splits, int sms) {
  const int tile_m = wide ? 2 * kBM : kBM;
  const int64_t items = static_cast<int64_t>((m + tile_m - 1) / tile_m) * ((n + bn - 1) / bn) * splits;
  const double per_cta = static_cast<double>((items + sms - 1) / sms);
  const double stage = wide ? 1100.0 : (bn == 256 ? 880.0 : 570.0);
  const double epilogue = wide ? 8000.0 : (bn == 256 ? 5000.0 : 3000.0);
  const int kb = (k_blocks + splits - 1) / splits;
  double cycles = per_cta * (kb * stage + 1500.0) + (wide ? per_cta : 1.0) * epilogue;
  if (splits > 1) cycles += 1900.0 * (3.0 + static_cast<double>(splits) * m * n * 4.0 / 4.0e6);
  return cycles;
}

// Best geometry for a given number of K slices (`splits` > 0), or best of both (`splits` == 0, at most
// `max_splits` slices).  A slower-by-model plan with fewer slices wins unless slicing saves 5 %.
static GemmPlan gemm_plan(int m, int n, int k, int segs, int out_mode, int splits, int max_splits) {
  const bool narrow_n = (out_mode != MSL_OUT_SWIGLU_BF16) && (n <= 128 || (n % 256 != 0 && n % 128 == 0));
  const int bn = narrow_n ? 128 : 256;
  const int k_blocks = ((k + kBK - 1) / kBK) * segs;
  const int sms = sm_count();
  const bool may_wide = !narrow_n && m > kBM && option(MSL_OPT_GEMM_WIDE) != 0;
  GemmPlan best{1, false, 0.0};
  bool have = false;
  const int lo = splits > 0 ? splits : 1, hi = splits > 0 ? splits : std::max(1, max_splits);
  for (int s = lo; s <= hi; ++s) {
    for (int w = 0; w <= (may_wide ? 1 : 0); ++w) {
      const double c = gemm_cost(m, n, k_blocks, bn, w != 0, s, sms);
      if (!have || c < best.cycles * (s > best.splits ? 0.95 : 1.0)) {
        best = GemmPlan{s, w != 0, c};
        have = true;
      }
    }
  }
  return best;
}

static int gemm_entry(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int m, int n, int k,
                      int segs, int a_seg_stride, int b_seg_stride, int out_mode, float alpha, int splits,
                      void* workspace, int* status, void* stream) {
  if (!a || !b || !c || m < 0 || n <= 0 || k <= 0 || segs < 1) return MSL_ERR_ARG;
  if (splits < 1 || splits > 64) return MSL_ERR_ARG;
  if (splits > 1) {
    if (!workspace || out_mode == MSL_OUT_SWIGLU_BF16) return MSL_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15) || (n & 3) || (ldc & 3) ||
        (reinterpret_cast<uintptr_t>(c) & 15))
      return MSL_ERR_ALIGN;
    if (splits > ((k + kBK - 1) / kBK) * segs) return MSL_ERR_ARG;
  }
  if ((lda & 7) || (ldb & 7) || (k & 7) || (a_seg_stride & 7) || (b_seg_stride & 7)) return MSL_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return MSL_ERR_ALIGN;
  if (out_mode == MSL_OUT_SWIGLU_BF16 && (n % 256)) return MSL_ERR_ARG;
  if (segs > 1 && (k % kBK)) return MSL_ERR_ARG;   // a segment's K tail would read the next segment
  if (m == 0) return MSL_OK;
  const int a_cols = a_seg_stride * (segs - 1) + k;
  const int b_cols = b_seg_stride * (segs - 1) + k;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_cols, m, lda * 2, kBK, kBM,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  GemmArgs args{c, ldc, m, n, k, segs, a_seg_stride, b_seg_stride, alpha, status, 1, 0};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (splits > 1) {
    // K slices as fp32 planes [splits][m][n] in the workspace, then one reduction into c.
    GemmArgs part{workspace, n, m, n, k, segs, a_seg_stride, b_seg_stride, 1.0f, status, splits,
                  static_cast<int64_t>(m) * n};
    const bool narrow_n = n <= 128 || (n % 256 != 0 && n % 128 == 0);
    rc = make_tmap_2d(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_cols, n, ldb * 2, kBK, narrow_n ? 128 : 256,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    if (narrow_n) rc = launch_gemm<128, 6, MSL_OUT_F32>(ta, tb, part, st);
    else if (gemm_plan(m, n, k, segs, out_mode, splits, splits).wide) rc = launch_gemm<256, 3, MSL_OUT_F32, 2>(ta, tb, part, st);
    else rc = launch_gemm<256, 4, MSL_OUT_F32>(ta, tb, part, st);
    if (rc) return rc;
    const int64_t quads = static_cast<int64_t>(m) * (n / 4);
    const int blocks = static_cast<int>(std::min<int64_t>((quads + 255) / 256, 8 * static_cast<int64_t>(sm_count())));
    splitk_reduce_kernel<<<blocks, 256, 0, st>>>(static_cast<const float*>(workspace), splits, m, n, alpha, c, ldc,
                                                 out_mode == MSL_OUT_F32);
    return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
  }
  // Narrow outputs use a 128-column tile so more CTAs share the work.
  const bool narrow = (out_mode != MSL_OUT_SWIGLU_BF16) && (n <= 128 || (n % 256 != 0 && n % 128 == 0));
  const int bn = narrow ? 128 : 256;
  rc = make_tmap_2d(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b_cols, n, ldb * 2, kBK, bn,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  // 256 x 256 tiles where the cost model above prefers them.
  const bool wide = gemm_plan(m, n, k, segs, out_mode, 1, 1).wide;
  switch (out_mode) {
    case MSL_OUT_BF16:
      if (wide) return launch_gemm<256, 3, MSL_OUT_BF16, 2>(ta, tb, args, st);
      return narrow ? launch_gemm<128, 6, MSL_OUT_BF16>(ta, tb, args, st)
                    : launch_gemm<256, 4, MSL_OUT_BF16>(ta, tb, args, st);
    case MSL_OUT_F32:
      if (wide) return launch_gemm<256, 3, MSL_OUT_F32, 2>(ta, tb, args, st);
      return narrow ? launch_gemm<128, 6, MSL_OUT_F32>(ta, tb, args, st)
                    : launch_gemm<256, 4, MSL_OUT_F32>(ta, tb, args, st);
    case MSL_OUT_SWIGLU_BF16:
      // (with the earlier, longer SiLU epilogue the 128-row tiles, whose two accumulator sets overlap it, won:
      // 1413 against 1316 TFLOP/s; with the short one the 256-row tiles do: 1522 against 1437)
      if (wide) return launch_gemm<256, 3, MSL_OUT_SWIGLU_BF16, 2>(ta, tb, args, st);
      return launch_gemm<256, 4, MSL_OUT_SWIGLU_BF16>(ta, tb, args, st);
    default:
      return MSL_ERR_ARG;
  }
}

extern "C" int msl_gemm_bf16(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int m,
                             int n, int k, int segs, int a_seg_stride, int b_seg_stride, int out_mode, float alpha,
                             int* status, void* stream) {
  return gemm_entry(a, lda, b, ldb, c, ldc, m, n, k, segs, a_seg_stride, b_seg_stride, out_mode, alpha, 1, nullptr,
                    status, stream);
}

extern "C" int msl_gemm_splitk_plan(int m, int n, int k, int segs, int out_mode) {
  if (m <= 0 || n <= 0 || k <= 0 || segs < 1 || out_mode == MSL_OUT_SWIGLU_BF16 || (n & 3)) return 1;
  // Slicing K changes the order of the fp32 sums, so a product's low bits then depend on how many rows
  // it has; with the option off every product runs in one pass, for hosts that need batch-invariant bits.
  if (option(MSL_OPT_GEMM_SPLITK) == 0) return 1;
  const int k_blocks = ((k + kBK - 1) / kBK) * segs;
  if (k_blocks < 16) return 1;                               // too little K to slice
  return gemm_plan(m, n, k, segs, out_mode, 0, std::min(k_blocks / 8, 16)).splits;
}

extern "C" int msl_gemm_bf16_splitk(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc,
                                    int m, int n, int k, int segs, int a_seg_stride, int b_seg_stride, int out_mode,
                                    float alpha, int splits, void* workspace, int* status, void* stream) {
  return gemm_entry(a, lda, b, ldb, c, ldc, m, n, k, segs, a_seg_stride, b_seg_stride, out_mode, alpha, splits,
                    workspace, status, stream);
}
