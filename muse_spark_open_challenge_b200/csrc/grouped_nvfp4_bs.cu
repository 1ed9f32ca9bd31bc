// Grouped expert GEMM with NVFP4 weights AND NVFP4 activations on Blackwell's block-scaled tensor-core
// path (opt-in; the default expert path keeps BF16 activations, grouped_nvfp4.cu):
//   out[r, :] = gs_e * rs_r * (xq[r, :] (*) sx[r, :]) * (wq_e (*) sw_e)^T
// where xq / wq are e2m1 codes, sx / sw their UE4M3 scales of 16-element blocks, rs_r a per-row fp32
// scale of the activations and gs_e the per-expert fp32 scale of the weights.  tcgen05.mma
// kind::mxf4nvf4.block_scale multiplies codes and block scales inside the tensor core (K = 64 per
// instruction, four scales per row), so the weights are consumed in their stored 4-bit form (TMA from the
// reference's own [experts, rows, k/2] layout, no dequantisation warps) and the block scales travel
// shared memory -> tensor memory by tcgen05.cp.  Optional fused SiLU(gate) * up epilogue.
//
// The reference's shipped layer runs its experts W4A16 through a third-party kernel
// (muse_prefill_layer/submission.py:956-1002); quantising the activations to 4 bits is the experiment of
// tools/prefill/moe_kernel/ that this mode takes to the native instruction.  The format is nvfp4.py:66-97.
//
// One persistent CTA per SM, 192 threads:
//   warp 0     TMA producer per stage of K = 256: activation codes 128 rows x 128 B, weight codes 192 rows x
//              128 B (one box, or for a gate/up bank 96 gate rows + their 96 up rows), both 128-byte
//              swizzled, and the two scale blocks (2 KB + 4 KB, already in the layout tcgen05.cp expects)
//              by bulk copies
//   warp 1     TMEM allocation; per stage 12 tcgen05.cp (scales) and 4 tcgen05.mma (M=128, N=192, K=64)
//   warps 2-5  epilogue: accumulator row -> scales -> (SiLU * up) -> bf16; TMEM loads one chunk ahead, fast
//              reciprocal, 32-byte stores (at K = 1536 a tile's main loop is no longer than its epilogue)
// TMEM: accumulator 0 at columns [0, 192), scales at [192, 240), accumulator 1 at [256, 448): the epilogue
// of one tile overlaps the main loop of the next.  Every mbarrier wait is bounded.
//
// What bounds it (131072 rows x 3072 x 4096: 0.97 ms = 3390 TFLOP/s, 0.38 of the instruction's measured
// ceiling): a stage of K = 256 takes 1120 cycles against 400 of MMA time.  Two things meet there.  The tensor
// pipe runs the 12 scale copies and the 4 MMAs of a stage in order and no instruction on it takes less than
// about 57 cycles (12 x 57 + 4 x 100 = 1084).  And the loads are bound by latency, not by L2 bandwidth: with
// 4 x 46 KB in flight per SM and 1.8 us from issue to arrival the SMs together receive 11.5 TB/s (a probe that
// streams an L2-resident buffer by bulk copies with 128 KB in flight per SM reaches 9.6 TB/s; by plain 16-byte
// loads from 2048 threads per SM, 17 TB/s).  Leaving out 11 of the 12 copies (wrong results, timing only)
// changed nothing, tiles of 256 rows with three 64 KB stages and one accumulator set ran at 2135 TFLOP/s.
// Before the issuer ran warp-uniform (one elected lane instead of a one-lane branch) it was 2294 TFLOP/s.
//
// Scale layout ("atom", 512 bytes = 128 rows x 4 scales of one K = 64 step): byte (r % 32) * 16 +
// (r / 32) * 4 + j holds scale j of row r; tcgen05.cp 32x128b.warpx4 copies an atom into 4 TMEM columns
// of all four lane quarters.  Weight scales are re-tiled once at load time (msl_nvfp4_bs_sf_repack);
// activation scales are written in that layout by the quantiser (msl_nvfp4_bs_quantize), indexed by the
// scheduler's row tile so a tile's scales for one stage are one contiguous 2 KB block.
#include <cuda_fp4.h>

#include "grouped_sched.cuh"
#include "msl_host.h"

namespace msl {

constexpr int kBsM = 128;          // token rows per tile (TMEM lanes)
constexpr int kBsN = 192;          // weight rows per tile
constexpr int kBsK = 256;          // k per stage = 128 bytes of codes per row
constexpr int kBsStages = 4;
constexpr int kBsMaxGroups = 256;
constexpr int kAtom = 512;         // bytes of one scale atom

struct BsSmem {
  static constexpr int kABytes = kBsM * 128;
  static constexpr int kBBytes = kBsN * 128;
  static constexpr int kSfaBytes = 4 * kAtom;
  static constexpr int kSfbBytes = 4 * 2 * kAtom;
  static constexpr int kB = kABytes, kSfa = kB + kBBytes, kSfb = kSfa + kSfaBytes;
  static constexpr int kStageBytes = kSfb + kSfbBytes;               // 47104 = 46 * 1024
  static constexpr int kPrefix = kBsStages * kStageBytes;            // (kBsMaxGroups + 1) x int
  static constexpr int kBar = kPrefix + (kBsMaxGroups + 1) * 4 + 4;
  static constexpr int kTotal = kBar + (2 * kBsStages + 4) * 8 + 16;
  static_assert(kStageBytes % 1024 == 0 && kBar % 8 == 0, "tile and barrier alignment");
};

struct BsArgs {
  const uint8_t* x_sf;     // activation scales: [row tiles][k / 256][4][512]
  const float* x_rs;       // [slab rows] row scales
  const uint8_t* w_sf;     // weight scales: [banks][n tiles][k / 256][4][2][512]
  const float* gs;         // [banks]
  const int* offsets;      // [groups + 1]
  void* out;
  int64_t ld_out, slab_rows;
  int groups, wexperts, n_tiles, k, n_out, swiglu, inter;
  int* status;
};

__device__ __forceinline__ void bs_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// One scale atom shared memory -> 4 TMEM columns (all four lane quarters).
// `on`: predicate of the elected lane; the other lanes run the same control flow and skip the instruction.
__device__ __forceinline__ void tc_cp_scales(uint32_t on, uint32_t taddr, uint32_t saddr) {
  // no swizzle; rows of 16 bytes, 8-row groups 128 bytes apart
  const uint64_t desc = make_sdesc(saddr, 16, 128, 0);
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
               "@q tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n\t}" ::"r"(taddr), "l"(desc), "r"(on) : "memory");
}
// D[tmem] (+)= (A (*) SFA) * (B (*) SFB)^T, e2m1 operands packed two per byte, UE4M3 scales of 16-element
// blocks in TMEM, K = 64 per instruction.
__device__ __forceinline__ void tc_mma_nvf4(uint32_t on, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(on)
      : "memory");
}
// Instruction descriptor of the block-scaled kinds: [7,10) A format, [10,13) B format (1 = e2m1),
// [17,23) N >> 3, [23] scale format (0 = UE4M3), [24,29) M >> 4; scale ids and K size 0.
__host__ __device__ constexpr uint32_t make_idesc_nvf4(uint32_t m, uint32_t n) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__global__ void __launch_bounds__(192, 1)
grouped_nvfp4_bs_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, BsArgs p) {
  using S = BsSmem;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int* mt_prefix = reinterpret_cast<int*>(smem + S::kPrefix);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* empty = full + kBsStages;
  uint64_t* tmem_full = empty + kBsStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = p.k / kBsK;
  const int worker = static_cast<int>(blockIdx.x), n_workers = static_cast<int>(gridDim.x);

  if (warp == 0) row_tile_prefix(p.offsets, p.groups, kBsM, mt_prefix, lane);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kBsStages; ++s) {
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
  if (warp == 1) tmem_alloc(tmem_base_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const int total_tiles = mt_prefix[p.groups] * p.n_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      tma_prefetch_desc(&tm_w);
      uint32_t it = 0;
      bool ok = true;
      for (int g = worker; g < total_tiles && ok; g += n_workers) {
        const TileInfo ti = decode_tile(g, mt_prefix, p.offsets, p.groups, p.n_tiles, kBsM);
        const int bank = ti.expert % p.wexperts;
        const int row_tile = mt_prefix[ti.expert] + (ti.row0 - p.offsets[ti.expert]) / kBsM;
        const uint8_t* sfa = p.x_sf + static_cast<int64_t>(row_tile) * k_blocks * S::kSfaBytes;
        const uint8_t* sfb = p.w_sf + (static_cast<int64_t>(bank) * p.n_tiles + ti.nt) * k_blocks * S::kSfbBytes;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kBsStages;
          const uint32_t ph = (it / kBsStages) & 1;
          if (*abort_flag || !mbar_wait(&empty[s], ph ^ 1)) { ok = false; break; }
          uint8_t* st = smem + s * S::kStageBytes;
          mbar_expect_tx(&full[s], S::kStageBytes);
          tma_load_2d(st, &tm_x, &full[s], kb * 128, ti.row0);
          if (p.swiglu) {
            tma_load_3d(st + S::kB, &tm_w, &full[s], kb * 128, ti.nt * (kBsN / 2), bank);
            tma_load_3d(st + S::kB + (kBsN / 2) * 128, &tm_w, &full[s], kb * 128, p.inter + ti.nt * (kBsN / 2), bank);
          } else {
            tma_load_3d(st + S::kB, &tm_w, &full[s], kb * 128, ti.nt * kBsN, bank);
          }
          bs_bulk_load(st + S::kSfa, sfa + static_cast<int64_t>(kb) * S::kSfaBytes, S::kSfaBytes, &full[s]);
          bs_bulk_load(st + S::kSfb, sfb + static_cast<int64_t>(kb) * S::kSfbBytes, S::kSfbBytes, &full[s]);
        }
      }
      if (!ok) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // All 32 lanes run the control flow, so that addresses and descriptors are warp-uniform values; one
    // elected lane executes the copies, MMAs and commits.
    {
      const uint32_t on = elect_one();
      constexpr uint32_t idesc = make_idesc_nvf4(kBsM, kBsN);
      const uint32_t sfa_t = tmem_base + kBsN, sfb_t = tmem_base + kBsN + 16;
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int g = worker; g < total_tiles && ok; g += n_workers, ++tile_i) {
        const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
        if (*abort_flag || !mbar_wait(&tmem_empty[acc], acc_ph ^ 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * 256;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kBsStages;
          const uint32_t ph = (it / kBsStages) & 1;
          if (*abort_flag || !mbar_wait(&full[s], ph)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * S::kStageBytes);
          const uint32_t sb = sa + S::kB, ssfa = sa + S::kSfa, ssfb = sa + S::kSfb;
          // The scale copies and the MMAs run in issue order on the tensor pipe, so the copies of this
          // stage overwrite the TMEM scale columns only after the previous stage's MMAs have read them.
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            tc_cp_scales(on, sfa_t + 4 * ks, ssfa + ks * kAtom);
            tc_cp_scales(on, sfb_t + 8 * ks, ssfb + (2 * ks) * kAtom);
            tc_cp_scales(on, sfb_t + 8 * ks + 4, ssfb + (2 * ks + 1) * kAtom);
          }
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            tc_mma_nvf4(on, d_tmem, make_sdesc(sa + ks * 32, 16, 1024, 2), make_sdesc(sb + ks * 32, 16, 1024, 2), idesc,
                        sfa_t + 4 * ks, sfb_t + 8 * ks, (kb | ks) != 0);
          tc_commit_if(on, &empty[s]);
        }
        if (ok) tc_commit_if(on, &tmem_full[acc]);
      }
      if (!ok && lane == 0) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    uint32_t tile_i = 0;
    bool ok = true;
    for (int g = worker; g < total_tiles && ok; g += n_workers, ++tile_i) {
      const TileInfo ti = decode_tile(g, mt_prefix, p.offsets, p.groups, p.n_tiles, kBsM);
      const uint32_t acc = tile_i & 1, acc_ph = (tile_i >> 1) & 1;
      if (*abort_flag || !mbar_wait(&tmem_full[acc], acc_ph)) { ok = false; break; }
      tc_fence_after();
      const int r = quarter * 32 + lane;
      const int64_t row = static_cast<int64_t>(ti.row0) + r;
      const bool valid = r < ti.rows && row < p.slab_rows;
      const float alpha = valid ? p.gs[ti.expert % p.wexperts] * p.x_rs[row] : 0.f;
      const uint32_t taddr = tmem_base + acc * 256 + (static_cast<uint32_t>(quarter * 32) << 16);
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ld_out;
      const int out_cols = p.swiglu ? kBsN / 2 : kBsN;
      const bool wide_ok = ((reinterpret_cast<uintptr_t>(p.out) | static_cast<uintptr_t>(p.ld_out * 2)) & 31) == 0;
      // chunks of 32 output columns; the TMEM loads of a chunk are issued one chunk ahead of its arithmetic
      // and stores (with K = 1536 a tile's main loop is no longer than this epilogue)
      uint32_t a[2][32], b[2][32];
      auto load = [&](int c, uint32_t (&x)[32], uint32_t (&y)[32]) {
        tmem_ld32(taddr + c, x);
        if (p.swiglu) tmem_ld32(taddr + kBsN / 2 + c, y);
      };
      auto emit = [&](int c, const uint32_t (&x)[32], const uint32_t (&y)[32]) {
        const int col0 = ti.nt * out_cols + c;
        if (!(valid && col0 < p.n_out)) return;
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float v0 = __uint_as_float(x[j]) * alpha, v1 = __uint_as_float(x[j + 1]) * alpha;
          if (p.swiglu) {
            // SiLU(g) * u = g * u / (1 + exp(-g)) with the fast reciprocal (2 ulp; +inf denominator -> 0)
            v0 = __fdividef(v0 * (__uint_as_float(y[j]) * alpha), 1.0f + __expf(-v0));
            v1 = __fdividef(v1 * (__uint_as_float(y[j + 1]) * alpha), 1.0f + __expf(-v1));
          }
          packed[j / 2] = pack_bf16x2(v0, v1);
        }
        if (col0 + 32 <= p.n_out) {
          if (wide_ok) {
#pragma unroll
            for (int j = 0; j < 16; j += 8)
              asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(orow + col0 + 2 * j),
                           "r"(packed[j]), "r"(packed[j + 1]), "r"(packed[j + 2]), "r"(packed[j + 3]),
                           "r"(packed[j + 4]), "r"(packed[j + 5]), "r"(packed[j + 6]), "r"(packed[j + 7]) : "memory");
          } else {
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              *reinterpret_cast<uint4*>(orow + col0 + 2 * j) =
                  make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
          }
        } else {
          for (int j = 0; j < 32 && col0 + j < p.n_out; ++j)
            orow[col0 + j] = __ushort_as_bfloat16(
                static_cast<unsigned short>((j & 1) ? (packed[j / 2] >> 16) : (packed[j / 2] & 0xffffu)));
        }
      };
      if (!p.swiglu && wide_ok && (ti.nt + 1) * kBsN <= p.n_out) {
        // plain bf16 rows of a tile inside the output: 64-column chunks transposed within quads, so that four
        // lanes write 128 contiguous bytes of one row per instruction
        const int q = r & 3, r_base = r & ~3;
        __nv_bfloat16* obase = reinterpret_cast<__nv_bfloat16*>(p.out) +
                               (static_cast<int64_t>(ti.row0) + r_base) * p.ld_out + ti.nt * kBsN + 16 * q;
        tmem_ld32(taddr, a[0]);
        tmem_ld32(taddr + 32, b[0]);
#pragma unroll 1
        for (int c = 0; c < kBsN; c += 64) {
          tmem_ld_wait();
          uint32_t u[32], f[32];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            // every lane scales with ITS row's factor before the exchange
            u[j / 2] = pack_bf16x2(__uint_as_float(a[0][j]) * alpha, __uint_as_float(a[0][j + 1]) * alpha);
            u[16 + j / 2] = pack_bf16x2(__uint_as_float(b[0][j]) * alpha, __uint_as_float(b[0][j + 1]) * alpha);
          }
          quad_transpose_units(u, f);
          if (c + 64 < kBsN) {
            tmem_ld32(taddr + c + 64, a[0]);
            tmem_ld32(taddr + c + 96, b[0]);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int rj = r_base + j;
            if (rj < ti.rows && static_cast<int64_t>(ti.row0) + rj < p.slab_rows)
              st_global_v8(obase + static_cast<int64_t>(j) * p.ld_out + c, &f[8 * j]);
          }
        }
      } else {
      load(0, a[0], b[0]);
#pragma unroll 1
      for (int c = 0; c < out_cols; c += 64) {               // out_cols is 96 or 192
        tmem_ld_wait();
        const bool second = c + 32 < out_cols;
        if (second) load(c + 32, a[1], b[1]);
        emit(c, a[0], b[0]);
        if (second) {
          tmem_ld_wait();
          if (c + 64 < out_cols) load(c + 64, a[0], b[0]);
          emit(c + 32, a[1], b[1]);
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
    if (!ok && lane == 0) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
  }

  if (warp == 0 && lane == 0 && *abort_flag) drain_pause();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------- activation quantiser
// One warp per slab row: row scale rs = max|x| / (6 * 448) (so that every block scale fits UE4M3), per
// 16-element block the scale UE4M3(max|block| / (6 rs)) and the codes e2m1(x / (scale * rs)), round to
// nearest.  Codes go to xq[row][k / 2] (element 2i in the low nibble of byte i, the reference's packing,
// nvfp4.py:66-88); the scale of block b goes to the atom layout of the row's tile: row tile =
// (row tiles of the groups before the row's group) + (row - group start) / 128, exactly the tile index of
// the GEMM's scheduler.  Rows beyond the last group are skipped.
__global__ void __launch_bounds__(256)
nvfp4_bs_quantize_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int64_t slab_rows, int k,
                         const int* __restrict__ offsets, int groups, uint8_t* __restrict__ xq,
                         uint8_t* __restrict__ x_sf, float* __restrict__ x_rs) {
  __shared__ int mt_prefix[kBsMaxGroups + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) row_tile_prefix(offsets, groups, kBsM, mt_prefix, lane);
  __syncthreads();
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (row >= slab_rows || row >= offsets[groups]) return;
  int lo = 0, hi = groups - 1;                               // the group that holds this row
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (offsets[mid] <= row) lo = mid; else hi = mid - 1;
  }
  const int in_group = static_cast<int>(row - offsets[lo]);
  const int row_tile = mt_prefix[lo] + in_group / kBsM, rt = in_group % kBsM;
  const int blocks = k / 16, k_blocks = k / kBsK;
  const __nv_bfloat16* xr = x + row * ldx;
  // pass 1: row maximum (the row is read twice; the second read hits L1/L2)
  float amax = 0.f;
  for (int b = lane; b < blocks; b += 32) {
    const uint4 q0 = *reinterpret_cast<const uint4*>(xr + b * 16), q1 = *reinterpret_cast<const uint4*>(xr + b * 16 + 8);
    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i)
      amax = fmaxf(amax, fmaxf(fabsf(bf16_bits_to_f32(w[i] & 0xffffu)), fabsf(bf16_bits_to_f32(w[i] >> 16))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float rs = amax > 0.f ? amax / (6.0f * 448.0f) : 1.0f;
  if (lane == 0) x_rs[row] = rs;
  uint8_t* sf_tile = x_sf + static_cast<int64_t>(row_tile) * k_blocks * (4 * kAtom) + (rt % 32) * 16 + (rt / 32) * 4;
  for (int b0 = 0; b0 < blocks; b0 += 32) {
    const int b = b0 + lane;
    uint32_t sf_byte = 0;
    if (b < blocks) {
      const uint4 q0 = *reinterpret_cast<const uint4*>(xr + b * 16), q1 = *reinterpret_cast<const uint4*>(xr + b * 16 + 8);
      const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
      float v[16];
      float bmax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[2 * i] = bf16_bits_to_f32(w[i] & 0xffffu);
        v[2 * i + 1] = bf16_bits_to_f32(w[i] >> 16);
        bmax = fmaxf(bmax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
      }
      // the reference's order of operations (nvfp4.py:81-84): scale byte from amax / 6 / rs, then the
      // elements divided by the product scale * rs as fp32 rounds it
      const __nv_fp8_storage_t sf8 = __nv_cvt_float_to_fp8((bmax / 6.0f) / rs, __NV_SATFINITE, __NV_E4M3);
      sf_byte = sf8;
      const float scale = __half2float(__half(__nv_cvt_fp8_to_halfraw(sf8, __NV_E4M3))) * rs;
      const float inv = scale > 0.f ? 1.0f / scale : 0.f;
      uint32_t codes[2] = {0, 0};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t c = __nv_cvt_float2_to_fp4x2(make_float2(v[2 * i] * inv, v[2 * i + 1] * inv), __NV_E2M1,
                                                    cudaRoundNearest);
        codes[i >> 2] |= (c & 0xffu) << (8 * (i & 3));
      }
      *reinterpret_cast<uint2*>(xq + row * (k / 2) + b * 8) = make_uint2(codes[0], codes[1]);
    }
    // four consecutive blocks (one K = 64 step) form one 32-bit word of the atom: gathered in the first
    // lane of each group of four
    uint32_t word = sf_byte;
    word |= __shfl_down_sync(0xffffffffu, sf_byte, 1) << 8;
    word |= __shfl_down_sync(0xffffffffu, sf_byte, 2) << 16;
    word |= __shfl_down_sync(0xffffffffu, sf_byte, 3) << 24;
    if ((lane & 3) == 0 && b < blocks) {
      const int step = b / 4;                                // K = 64 step of the row: stage step / 4, atom step % 4
      *reinterpret_cast<uint32_t*>(sf_tile + (static_cast<int64_t>(step / 4) * 4 + (step % 4)) * kAtom) = word;
    }
  }
}

// ---------------------------------------------------------------------------- load-time scale re-tiling
// src: e4m3 scales [banks, rows, k / 16] of an expert bank as the reference stores it (baseline.py:74-79).
// dst: [banks][n tiles][k / 256][4][2][512]: for every tile of 192 weight rows (a gate/up bank: gate rows
// [96 t, 96 t + 96) then up rows inter + [96 t, 96 t + 96)) and every stage, the eight atoms the kernel
// copies to TMEM.  Rows beyond the bank get zero scales.
__global__ void nvfp4_bs_sf_repack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int banks,
                                          int rows, int k, int n_tiles, int swiglu) {
  const int k_blocks = k / kBsK, inter = rows / 2;
  const int64_t total = static_cast<int64_t>(banks) * n_tiles * k_blocks * 8 * kAtom;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int off = static_cast<int>(i % kAtom);
    int64_t q = i / kAtom;
    const int a = static_cast<int>(q % 2); q /= 2;
    const int ks = static_cast<int>(q % 4); q /= 4;
    const int kb = static_cast<int>(q % k_blocks); q /= k_blocks;
    const int nt = static_cast<int>(q % n_tiles);
    const int bank = static_cast<int>(q / n_tiles);
    const int rr = off / 16 + 32 * ((off % 16) / 4), j = off % 4;
    const int tr = 128 * a + rr;                             // row of the 192-row tile
    int src_row = -1;
    if (tr < kBsN) {
      if (swiglu) {
        const int half = kBsN / 2, idx = nt * half + (tr < half ? tr : tr - half);
        if (idx < inter) src_row = tr < half ? idx : inter + idx;
      } else {
        src_row = nt * kBsN + tr;
        if (src_row >= rows) src_row = -1;
      }
    }
    uint8_t v = 0;
    if (src_row >= 0) v = src[(static_cast<int64_t>(bank) * rows + src_row) * (k / 16) + kb * 16 + ks * 4 + j];
    dst[i] = v;
  }
}

}  // namespace msl

using namespace msl;

extern "C" int msl_nvfp4_bs_tiles(int rows, int swiglu) {
  if (rows <= 0) return 0;
  return swiglu ? (rows / 2 + kBsN / 2 - 1) / (kBsN / 2) : (rows + kBsN - 1) / kBsN;
}

extern "C" int64_t msl_nvfp4_bs_row_tiles(int64_t slab_rows, int groups) {
  if (slab_rows < 0 || groups < 0) return 0;
  return (slab_rows + kBsM - 1) / kBsM + groups;
}

extern "C" int msl_nvfp4_bs_sf_repack(const void* src_scales, void* dst_scales, int banks, int rows, int k, int swiglu,
                                      void* stream) {
  if (!src_scales || !dst_scales || banks <= 0 || rows <= 0 || k <= 0) return MSL_ERR_ARG;
  if (k % kBsK) return MSL_ERR_UNSUPPORTED;
  if (swiglu && (rows & 1)) return MSL_ERR_ARG;
  const int n_tiles = msl_nvfp4_bs_tiles(rows, swiglu);
  const int64_t total = static_cast<int64_t>(banks) * n_tiles * (k / kBsK) * 8 * kAtom;
  const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 16));
  nvfp4_bs_sf_repack_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src_scales), static_cast<uint8_t*>(dst_scales), banks, rows, k, n_tiles, swiglu);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

extern "C" int msl_nvfp4_bs_quantize(const void* x, int64_t ldx, int64_t slab_rows, int k, const int* offsets,
                                     int groups, void* codes, void* scales, float* row_scales, void* stream) {
  if (!x || !offsets || !codes || !scales || !row_scales || slab_rows < 0 || k <= 0 || groups <= 0 ||
      groups > kBsMaxGroups)
    return MSL_ERR_ARG;
  if (k % kBsK) return MSL_ERR_UNSUPPORTED;
  if ((ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(codes) & 15) ||
      (reinterpret_cast<uintptr_t>(scales) & 15))
    return MSL_ERR_ALIGN;
  if (slab_rows == 0) return MSL_OK;
  const int64_t blocks = (slab_rows + 7) / 8;
  nvfp4_bs_quantize_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, slab_rows, k, offsets, groups, static_cast<uint8_t*>(codes),
      static_cast<uint8_t*>(scales), row_scales);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

extern "C" int msl_grouped_gemm_nvfp4_bs(const void* x_codes, const void* x_scales, const float* x_row_scales,
                                         int64_t slab_rows, const void* w_codes, const void* w_scales_tiled,
                                         const float* global_scales, const int* offsets, void* out, int64_t ld_out,
                                         int groups, int weight_experts, int weight_rows, int k, int n_out, int swiglu,
                                         int* status, void* stream) {
  if (!x_codes || !x_scales || !x_row_scales || !w_codes || !w_scales_tiled || !global_scales || !offsets || !out)
    return MSL_ERR_ARG;
  if (groups <= 0 || groups > kBsMaxGroups || weight_experts <= 0 || weight_rows <= 0 || k <= 0 || n_out <= 0 ||
      slab_rows < 0 || (swiglu && (weight_rows & 1)))
    return MSL_ERR_ARG;
  if (k % kBsK) return MSL_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x_codes) & 15) || (reinterpret_cast<uintptr_t>(w_codes) & 15) ||
      (reinterpret_cast<uintptr_t>(x_scales) & 15) || (reinterpret_cast<uintptr_t>(w_scales_tiled) & 15) ||
      (ld_out & 7) || (reinterpret_cast<uintptr_t>(out) & 15))
    return MSL_ERR_ALIGN;
  if (slab_rows == 0) return MSL_OK;
  const int n_tiles = msl_nvfp4_bs_tiles(weight_rows, swiglu);
  CUtensorMap tx, tw;
  const uint64_t row_bytes = static_cast<uint64_t>(k) / 2;
  int rc = make_tmap_2d(&tx, x_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, row_bytes, slab_rows, row_bytes, 128, kBsM,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_tmap_3d(&tw, w_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, row_bytes, weight_rows, weight_experts, row_bytes,
                    row_bytes * weight_rows, 128, swiglu ? kBsN / 2 : kBsN, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  BsArgs a{static_cast<const uint8_t*>(x_scales), x_row_scales, static_cast<const uint8_t*>(w_scales_tiled),
           global_scales, offsets, out, ld_out, slab_rows, groups, weight_experts, n_tiles, k, n_out, swiglu,
           weight_rows / 2, status};
  const int smem = BsSmem::kTotal + 1024;
  static SmemConfig config;
  if (int rc2 = config.ensure(grouped_nvfp4_bs_kernel, smem)) return rc2;
  const int64_t max_tiles = ((slab_rows + kBsM - 1) / kBsM + groups) * n_tiles;
  const int grid = static_cast<int>(std::min<int64_t>(max_tiles, sm_count()));
  grouped_nvfp4_bs_kernel<<<grid, 192, smem, static_cast<cudaStream_t>(stream)>>>(tx, tw, a);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}
