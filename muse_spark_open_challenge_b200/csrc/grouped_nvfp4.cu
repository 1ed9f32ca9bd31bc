// Grouped expert GEMM with NVFP4 weights and BF16 activations on tcgen05 (W4A16):
//   out[r, :] = (x[r, :] * dq(W_e)^T) * gs_e      for the rows r of expert e's slab range,
// dq(W) = e2m1 code * e4m3 block scale (16-element blocks); the per-expert fp32 global scale is
// applied to the fp32 accumulator.  Optional fused SiLU(gate) * up epilogue.
//
// Replaces the third-party grouped GEMM launches and the separate SiLU kernel of the reference's
// layer (muse_prefill_layer/submission.py:956-1002, launches :1128-1130; _silu_mul_kernel
// :903-913) and restates the arithmetic of reference.py:433-442 / nvfp4.py:90-97.
//
// One persistent CTA per SM, 448 threads:
//   warp 0      TMA producer: activation tile 128 rows x 64 k (bf16, 128-byte swizzle)
//   warp 1      TMEM allocation + tcgen05.mma issue (M=128 tokens, N=256 weight rows, K=16)
//   warps 2-5   epilogue (TMEM -> registers -> global): TMEM loads issued one chunk ahead of the arithmetic,
//               SiLU with the fast reciprocal, 32-byte stores.  With 256-row tiles it does not overlap the
//               next tile's main loop (one accumulator set), so its length counts: it took 29.6 k cycles
//               per gate/up tile (main loop 74 k) before these three changes and takes 8.7 k now
//   warps 6-13  weight producers in two groups of 4 warps that take alternate stages: each thread
//               dequantises two weight rows of its stage (2 x (64 codes + 4 block scales) -> 128 bf16)
//               straight into the swizzled B tile in shared memory, while the codes of its next stage
//               are already in flight from L2
// N = 256 keeps the tensor core's operand fetch per FLOP low (a 128-column tile measured 25 % slower
// with the dequantisation switched off); producing a stage is a latency-bound chain, and two groups
// on different stages hide it (one group on every stage measured 30 % slower).  The weights were
// re-tiled once at load time (msl_nvfp4_repack) so a stage's codes are one contiguous 8 KiB block and
// its scales one contiguous 1 KiB block.
//
// Dequantisation without a table for the codes: a 4-bit code s|e1 e0|m placed at bf16 bits
// 15|8 7|6 is the bf16 number value * 2^-126 (also for the subnormal codes 0 and 0.5); the block
// scale is looked up as bf16(scale * 2^118); one bf16x2 multiply gives value * scale * 2^-8
// exactly (at most 6 significant bits), and the 2^8 is folded into the epilogue scale.  The idea of
// decoding e2m1 by bit placement plus one bf16 multiply with a biased block scale comes from the
// reference's experimental W4A16 kernel (tools/prefill/moe_kernel/moe_fp4.py:163-183); the bit layout
// (moved into the load-time repack so three of four pairs need one shift and one mask), the arithmetic
// scale decode and the table for special scale codes are this file's own.
#include "grouped_sched.cuh"
#include "msl_host.h"

namespace msl {

constexpr int kSubM = 128;     // rows of one CTA's MMA share (TMEM lanes)
constexpr int kGN = 256;       // weight rows per tile: N = 256 keeps the MMA operand fetch per FLOP low
constexpr int kGK = 64;        // k per stage
constexpr int kMaxLocal = 256; // row groups per call
constexpr int kProducers = 256;               // weight-producer threads per CTA
constexpr int kGroups = 2;                    // producer groups, each taking every kGroups-th stage
constexpr int kGroupThreads = kProducers / kGroups;

// Tile geometries (MODE):
//   kNarrow  128 token rows x 256 weight rows per tile, two accumulator sets (the epilogue of one tile
//            overlaps the main loop of the next).  For calls whose groups are small.
//   kWide    256 token rows (two 128-row MMAs per K step sharing one dequantised weight tile) x 256
//            weight rows, one accumulator set (both sub-tiles fill the 512 TMEM columns).
//            Halves the weight bytes staged, dequantised and fetched per FLOP.
// (A third geometry, two CTAs of a cluster sharing one M=256 MMA with cta_group::2, each dequantising
// half of the weight tile, was built and measured slower, 820 against 1012 TFLOP/s: not kept.)
constexpr int kNarrow = 0, kWide = 2;
template <int MODE>
struct GroupedCfg {
  static constexpr bool WIDE = MODE == kWide;
  static constexpr int kSubs = WIDE ? 2 : 1;                 // 128-row MMAs per K step in one CTA
  static constexpr int kTileM = WIDE ? 256 : 128;            // token rows per tile
  static constexpr int kBRows = 256;                         // weight rows dequantised per stage
  // The activation tiles (loaded by TMA) and the weight tiles (dequantised from registers that were
  // loaded two stages earlier) live in rings of their own, so that their depths can differ.  Measured
  // on 128 groups x 1024 rows (gate/up): 4 + 3 slots 1440 TFLOP/s, 3 + 4 the same, 5 + 2 about 10 % less
  // (each producer group needs a slot to fill while the one before it is being multiplied).  A timeline
  // of one SM (clock64 stamps of the issuer and of both producer groups) shows the K loop close to the
  // tensor pipe's pace: 1100-1180 cycles per stage against 1024 of MMA time, the weight tile of a stage
  // ready 200-1000 cycles before the issuer asks for it; hand-offs polled with mbarrier.test_wait instead
  // of try_wait, or one tcgen05.commit per stage instead of two, change nothing.  What is left per 256-row
  // gate/up tile: 64 stages x 1150 + an epilogue of 8.7 k cycles against 65.5 k of pure MMA time, at the
  // 1.5 GHz the power cap leaves this kernel.
  static constexpr int kAStages = WIDE ? 4 : 6;
  static constexpr int kBStages = 3;
  static constexpr int kRowsPerThread = kBRows / kGroupThreads;
  static constexpr int kSubBytes = kSubM * kGK * 2;
  static constexpr int kABytes = kSubs * kSubBytes;
  static constexpr int kBBytes = kBRows * kGK * 2;
  static constexpr int kBRing = kAStages * kABytes;                  // weight ring behind the activation ring
  static constexpr int kLutOffset = kBRing + kBStages * kBBytes;     // 256 x u32
  static constexpr int kPrefixOffset = kLutOffset + 1024;            // (kMaxLocal + 1) x int
  static constexpr int kBarOffset = kPrefixOffset + (kMaxLocal + 1) * 4 + 4;
  static constexpr int kTotal = kBarOffset + (2 * kAStages + 2 * kBStages + 4) * 8 + 16;
  static_assert(kBarOffset % 8 == 0, "barriers must be 8-byte aligned");
  static_assert(kTotal <= 232448, "shared memory of one CTA");
};

// Phase timing for development builds (-DMSL_GROUPED_PROF): cycles summed over all CTAs; read back with
// msl_debug_grouped_prof.
#ifdef MSL_GROUPED_PROF
__device__ unsigned long long g_grouped_prof[32];
#define GPROF_DECL long long prof_t = clock64(); long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define GPROF_MARK(i) do { const long long now_ = clock64(); prof_acc[i] += now_ - prof_t; prof_t = now_; } while (0)
#define GPROF_FLUSH(base, n) do { for (int i_ = 0; i_ < (n); ++i_) atomicAdd(&g_grouped_prof[(base) + i_], (unsigned long long)prof_acc[i_]); } while (0)
#else
#define GPROF_DECL do {} while (0)
#define GPROF_MARK(i) do {} while (0)
#define GPROF_FLUSH(base, n) do {} while (0)
#endif

struct GroupedArgs {
  const uint8_t* wq;       // [banks][n_tiles][k_blocks][256 rows][32 bytes]
  const uint8_t* sf;       // [banks][n_tiles][k_blocks][256 rows][4 bytes]
  const float* gs;         // [banks]
  const int* offsets;      // [groups + 1] slab row ranges
  void* out;
  int64_t ld_out;
  int64_t slab_rows;       // rows of x and of out: no row at or beyond it is stored
  int experts, n, k;       // experts = row groups; n = padded weight rows (multiple of 256), k multiple of 64
  int wexperts;            // weight banks: group g uses bank g % wexperts
  int n_out;               // valid output columns (after the SwiGLU halving when fused)
  int swiglu;
  int* status;
};

// Eight codes of one 32-bit word -> four bf16x2 words (elements 2j, 2j+1 in word j), times the
// block scale.  The repack put the even elements in the low half-word and the odd ones in the
// high half-word, element pair j at half-word bits: j=0: 15|8 7 6 (already in place), j=1: 12|5 4 3,
// j=2: 9|2 1 0, j=3: 14|13 11 10 (sign | e1 e0 m).  Pairs 0-2 need one shift and one mask.
// E4M3 block scale byte -> bf16(scale * 2^118) in both half-words.  A normal positive code s (exponent
// field e >= 1) is 2^(e-7) (1 + m/8): its bf16 pattern times 2^118 is ((e + 238) << 7) | (m << 4) =
// (s << 4) + 0x7700, so no table access (and none of its bank conflicts) is needed; zero, subnormal,
// negative and NaN codes (not produced by a quantiser, but legal) take the table.
__device__ __forceinline__ uint32_t scale_pair(const uint32_t* lut, uint32_t s) {
  if (__builtin_expect(s - 8u < 0x77u, 1)) {                // 0x08 <= s <= 0x7e
    const uint32_t b = (s << 4) + 0x7700u;
    return b * 0x10001u;
  }
  return lut[s];
}

__device__ __forceinline__ uint4 dequant8(uint32_t w, uint32_t scale2) {
  constexpr uint32_t kMask = 0x81C081C0u;
  uint32_t b[4];
  b[0] = w & kMask;
  b[1] = (w << 3) & kMask;
  b[2] = (w << 6) & kMask;
  b[3] = ((w >> 4) & 0x00C000C0u) | ((w >> 5) & 0x01000100u) | ((w << 1) & 0x80008000u);
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&b[j]),
                               *reinterpret_cast<const __nv_bfloat162*>(&scale2));
    o[j] = *reinterpret_cast<uint32_t*>(&v);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// SiLU(g) * u = g * u / (1 + exp(-g)) with the fast reciprocal: 2 ulp, far below the bf16 it is rounded to.
// For g < -88 the denominator is +inf and the quotient 0, the limit.
__device__ __forceinline__ float silu_mul(float g, float u) {
  return __fdividef(g * u, 1.0f + __expf(-g));
}

template <bool SWIGLU>
__device__ __forceinline__ void store_rows(const GroupedArgs& p, const TileInfo& ti, uint32_t taddr, int r,
                                           float alpha, uint64_t* release, long long* epi = nullptr) {
  // One thread owns row r of the tile: 256 accumulator columns -> 256 (or 128 fused) outputs, in chunks
  // whose TMEM loads are issued one chunk ahead of the arithmetic and the stores.  Offsets that run past
  // the slab (a routing that needs more rows than the buffers hold) store nothing.  `release` (the last
  // sub-tile of a tile): the accumulators are handed back as soon as the last chunk is in registers, before
  // its arithmetic and stores.
  const bool valid = r < ti.rows && static_cast<int64_t>(ti.row0) + r < p.slab_rows;
  __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(ti.row0 + r) * p.ld_out;
  const bool wide_ok = ((reinterpret_cast<uintptr_t>(p.out) | static_cast<uintptr_t>(p.ld_out * 2)) & 31) == 0;
  constexpr int kOutCols = SWIGLU ? kGN / 2 : kGN;
  constexpr int CH = SWIGLU ? 16 : 32;                       // output columns per chunk
  constexpr int NB = SWIGLU ? 2 : 1;                         // accumulator pieces per chunk (gate, up)
  uint32_t buf[2][NB][CH];
  auto load = [&](int c, uint32_t (&d)[NB][CH]) {
    if constexpr (SWIGLU) {
      tmem_ld16(taddr + c, d[0]);
      tmem_ld16(taddr + kGN / 2 + c, d[1]);
    } else {
      tmem_ld32(taddr + c, d[0]);
    }
  };
  auto emit = [&](int c, const uint32_t (&d)[NB][CH]) {
    const int col0 = ti.nt * kOutCols + c;
    if (!(valid && col0 < p.n_out)) return;
    uint32_t packed[CH / 2];
#pragma unroll
    for (int j = 0; j < CH; j += 2) {
      float v0 = __uint_as_float(d[0][j]) * alpha, v1 = __uint_as_float(d[0][j + 1]) * alpha;
      if constexpr (SWIGLU) {
        v0 = silu_mul(v0, __uint_as_float(d[NB - 1][j]) * alpha);
        v1 = silu_mul(v1, __uint_as_float(d[NB - 1][j + 1]) * alpha);
      }
      packed[j / 2] = pack_bf16x2(v0, v1);
    }
    if (col0 + CH <= p.n_out) {
      if (wide_ok) {
        // 32-byte stores: every lane writes whole sectors of its own row, half as many store instructions
#pragma unroll
        for (int j = 0; j < CH / 2; j += 8)
          asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(orow + col0 + 2 * j),
                       "r"(packed[j]), "r"(packed[j + 1]), "r"(packed[j + 2]), "r"(packed[j + 3]), "r"(packed[j + 4]),
                       "r"(packed[j + 5]), "r"(packed[j + 6]), "r"(packed[j + 7]) : "memory");
      } else {
#pragma unroll
        for (int j = 0; j < CH / 2; j += 4)
          *reinterpret_cast<uint4*>(orow + col0 + 2 * j) =
              make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
      }
    } else {
      for (int j = 0; j < CH && col0 + j < p.n_out; ++j)
        orow[col0 + j] = __ushort_as_bfloat16(
            static_cast<unsigned short>((j & 1) ? (packed[j / 2] >> 16) : (packed[j / 2] & 0xffffu)));
    }
  };
#ifdef MSL_GROUPED_PROF
  long long t_ = clock64();
#define EPI_MARK(i) do { const long long n_ = clock64(); if (epi) epi[i] += n_ - t_; t_ = n_; } while (0)
#else
#define EPI_MARK(i) do {} while (0)
#endif
  load(0, buf[0]);
#pragma unroll 1
  for (int c = 0; c < kOutCols; c += 2 * CH) {
    tmem_ld_wait();
    EPI_MARK(0);
    load(c + CH, buf[1]);                                    // kOutCols is a multiple of 2 CH
    emit(c, buf[0]);
    EPI_MARK(1);
    tmem_ld_wait();
    EPI_MARK(0);
    if (c + 2 * CH < kOutCols) {
      load(c + 2 * CH, buf[0]);
    } else if (release != nullptr) {
      tc_fence_before();
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(release);
    }
    emit(c + CH, buf[1]);
    EPI_MARK(1);
  }
}

// The plain bf16 output (down projection) when a whole 256-column tile lies inside the output and base and
// pitch allow 32-byte stores: chunks of 64 columns, transposed within quads so that four lanes write 128
// contiguous bytes of one row per instruction.  (With a lane writing 32 bytes of its own row, the 128 KB of a
// 256-row tile left the SM at 14 bytes per cycle and took 9.2 k cycles.)  Called by whole warps.
__device__ __forceinline__ void store_rows_quads(const GroupedArgs& p, const TileInfo& ti, uint32_t taddr, int r,
                                                 float alpha, uint64_t* release) {
  const int q = r & 3, r_base = r & ~3;
  __nv_bfloat16* obase = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(ti.row0 + r_base) * p.ld_out +
                         ti.nt * kGN + 16 * q;
  bool ok_row[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) ok_row[j] = r_base + j < ti.rows && static_cast<int64_t>(ti.row0) + r_base + j < p.slab_rows;
  uint32_t a[32], b[32];
  tmem_ld32(taddr, a);
  tmem_ld32(taddr + 32, b);
#pragma unroll 1
  for (int c = 0; c < kGN; c += 64) {
    tmem_ld_wait();
    uint32_t u[32], f[32];
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      u[j / 2] = pack_bf16x2(__uint_as_float(a[j]) * alpha, __uint_as_float(a[j + 1]) * alpha);
      u[16 + j / 2] = pack_bf16x2(__uint_as_float(b[j]) * alpha, __uint_as_float(b[j + 1]) * alpha);
    }
    quad_transpose_units(u, f);
    if (c + 64 < kGN) {
      tmem_ld32(taddr + c + 64, a);
      tmem_ld32(taddr + c + 96, b);
    } else if (release != nullptr) {
      tc_fence_before();
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(release);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (ok_row[j]) st_global_v8(obase + static_cast<int64_t>(j) * p.ld_out + c, &f[8 * j]);
  }
}

template <int MODE>
__global__ void __launch_bounds__(448, 1)
grouped_nvfp4_kernel(const __grid_constant__ CUtensorMap tm_x, GroupedArgs p) {
  using S = GroupedCfg<MODE>;
  constexpr bool WIDE = S::WIDE;
  constexpr int kAStages = S::kAStages, kBStages = S::kBStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  {
    // the launch asks for as much slack as fits below the limit of one CTA; the base is normally aligned already
    uint32_t dyn;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
    if (static_cast<uint32_t>(smem - smem_raw) + S::kTotal > dyn) {
      if (threadIdx.x == 0) report_error(p.status, MSL_ERR_CUDA);
      return;                                                // uniform for the CTA, before any barrier
    }
  }
  uint32_t* lut = reinterpret_cast<uint32_t*>(smem + S::kLutOffset);
  int* mt_prefix = reinterpret_cast<int*>(smem + S::kPrefixOffset);
  uint64_t* a_full = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* a_empty = a_full + kAStages;
  uint64_t* b_full = a_empty + kAStages;
  uint64_t* b_empty = b_full + kBStages;
  uint64_t* tmem_full = b_empty + kBStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = p.n / kGN;
  const int k_blocks = p.k / kGK;
  const int worker = static_cast<int>(blockIdx.x);
  const int n_workers = static_cast<int>(gridDim.x);

  // Scale table: e4m3 byte -> bf16(scale * 2^118) in both halves.  (0x7f / 0xff are NaN codes.)
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {
    const int e = (i >> 3) & 15, m = i & 7;
    float s = e ? ldexpf(1.0f + m * 0.125f, e - 7) : ldexpf(m * 0.125f, -6);
    if (i & 0x80) s = -s;
    if ((i & 0x7f) == 0x7f) s = __int_as_float(0x7fc00000);
    const uint32_t b = __float_as_uint(s * 3.32306998946228968e35f) >> 16;   // * 2^118: exact, top 16 bits
    lut[i] = b | (b << 16);
  }
  if (warp == 0) row_tile_prefix(p.offsets, p.experts, S::kTileM, mt_prefix, lane);
  if (threadIdx.x == 0) {
    // a_full: one expect_tx arrival of the TMA lane; b_full: the warps of one producer group; the empty
    // barriers: one tcgen05.commit; tmem_empty: the 4 epilogue warps.
    for (int s = 0; s < kAStages; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&a_empty[s], 1);
    }
    for (int s = 0; s < kBStages; ++s) {
      mbar_init(&b_full[s], kGroupThreads / 32);
      mbar_init(&b_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_base_slot, 2 * kGN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const int total_tiles = mt_prefix[p.experts] * n_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer: this CTA's 128 token rows
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      uint32_t it = 0;
      bool ok = true;
      for (int g = worker; g < total_tiles && ok; g += n_workers) {
        const TileInfo ti = decode_tile(g, mt_prefix, p.offsets, p.experts, n_tiles, S::kTileM);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kAStages;
          const uint32_t ph = (it / kAStages) & 1;
          if (*abort_flag || !mbar_wait(&a_empty[s], ph ^ 1)) { ok = false; break; }
          const int nsub = WIDE ? (ti.rows + kSubM - 1) / kSubM : 1;
          mbar_expect_tx(&a_full[s], nsub * S::kSubBytes);
          for (int sub = 0; sub < nsub; ++sub)
            tma_load_2d(smem + s * S::kABytes + sub * S::kSubBytes, &tm_x, &a_full[s], kb * kGK,
                        ti.row0 + sub * kSubM);
        }
      }
      if (!ok) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // All 32 lanes run the control flow, so that addresses and descriptors are warp-uniform values; one
    // elected lane executes the MMAs and commits.
    {
      const uint32_t on = elect_one();
      constexpr uint32_t idesc = make_idesc(1, 1, 128, kGN);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      GPROF_DECL;
      for (int g = worker; g < total_tiles && ok; g += n_workers, ++tile_i) {
        // kWide has one accumulator set (index 0, phase flips every tile); the others alternate two.
        const uint32_t acc = WIDE ? 0u : (tile_i & 1), acc_ph = WIDE ? (tile_i & 1) : ((tile_i >> 1) & 1);
        int nsub = 1;
        if constexpr (WIDE) {
          const TileInfo ti = decode_tile(g, mt_prefix, p.offsets, p.experts, n_tiles, S::kTileM);
          nsub = (ti.rows + kSubM - 1) / kSubM;
        }
        GPROF_MARK(0);
        if (*abort_flag || !mbar_wait(&tmem_empty[acc], acc_ph ^ 1)) { ok = false; break; }
        GPROF_MARK(1);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kGN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int as = it % kAStages, bs = it % kBStages;
          GPROF_MARK(0);
          if (*abort_flag || !mbar_wait(&b_full[bs], (it / kBStages) & 1)) { ok = false; break; }
          GPROF_MARK(2);
          if (!mbar_wait(&a_full[as], (it / kAStages) & 1)) { ok = false; break; }
          GPROF_MARK(3);
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + as * S::kABytes);
          const uint32_t sb = smem_u32(smem + S::kBRing + bs * S::kBBytes);
#pragma unroll
          for (int k16 = 0; k16 < kGK / 16; ++k16) {
            const uint64_t da = make_sdesc(sa + k16 * 32, 16, 1024, 2), db = make_sdesc(sb + k16 * 32, 16, 1024, 2);
            tc_mma_f16_if(on, d_tmem, da, db, idesc, (kb | k16) != 0);
            if (WIDE && nsub > 1)
              tc_mma_f16_if(on, d_tmem + kGN, make_sdesc(sa + S::kSubBytes + k16 * 32, 16, 1024, 2), db, idesc,
                            (kb | k16) != 0);
          }
          tc_commit_if(on, &a_empty[as]);
          tc_commit_if(on, &b_empty[bs]);
        }
        if (ok) tc_commit_if(on, &tmem_full[acc]);
      }
      GPROF_MARK(0);
#ifdef MSL_GROUPED_PROF
      prof_acc[7] = it;
      if (lane == 0) GPROF_FLUSH(0, 8);
#endif
      if (!ok && lane == 0) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    uint32_t tile_i = 0;
    bool ok = true;
#ifdef MSL_GROUPED_PROF
    long long epi_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#endif
    for (int g = worker; g < total_tiles && ok; g += n_workers, ++tile_i) {
      const TileInfo ti = decode_tile(g, mt_prefix, p.offsets, p.experts, n_tiles, S::kTileM);
      const uint32_t acc = WIDE ? 0u : (tile_i & 1), acc_ph = WIDE ? (tile_i & 1) : ((tile_i >> 1) & 1);
      if (*abort_flag || !mbar_wait(&tmem_full[acc], acc_ph)) { ok = false; break; }
      tc_fence_after();
      const float alpha = p.gs[ti.expert % p.wexperts] * 256.0f;
      const int nsub = WIDE ? (ti.rows + kSubM - 1) / kSubM : (ti.rows > 0 ? 1 : 0);   // uniform per CTA
      for (int sub = 0; sub < nsub; ++sub) {
        const uint32_t taddr = tmem_base + (acc + sub) * kGN + (static_cast<uint32_t>(quarter * 32) << 16);
        const int r = sub * kSubM + quarter * 32 + lane;
        uint64_t* release = sub == nsub - 1 ? &tmem_empty[acc] : nullptr;
        const bool quads = !p.swiglu && (ti.nt + 1) * kGN <= p.n_out &&
                           ((reinterpret_cast<uintptr_t>(p.out) | static_cast<uintptr_t>(p.ld_out * 2)) & 31) == 0;
#ifdef MSL_GROUPED_PROF
        if (p.swiglu) store_rows<true>(p, ti, taddr, r, alpha, release, epi_acc);
        else if (quads) store_rows_quads(p, ti, taddr, r, alpha, release);
        else store_rows<false>(p, ti, taddr, r, alpha, release, epi_acc);
#else
        if (p.swiglu) store_rows<true>(p, ti, taddr, r, alpha, release);
        else if (quads) store_rows_quads(p, ti, taddr, r, alpha, release);
        else store_rows<false>(p, ti, taddr, r, alpha, release);
#endif
      }
      if (nsub == 0) {                                       // an empty tile: nothing was read, hand the set back
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      }
    }
#ifdef MSL_GROUPED_PROF
    if (threadIdx.x == 64) { epi_acc[7] = tile_i; for (int i_ = 0; i_ < 8; ++i_) atomicAdd(&g_grouped_prof[24 + i_], (unsigned long long)epi_acc[i_]); }
#endif
    if (!ok && lane == 0) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
  } else {
    // ------------------------------------------------------------ weight producers (warps 6-13)
    // The 8 producer warps form kGroups groups; group q produces stages q, q + kGroups, ...  Each
    // stage's chain (wait for the free slot, table look-up, bit work, stores, proxy fence, arrive)
    // is latency-bound, so letting the groups work on different stages at the same time hides it.
    constexpr int kRows = S::kRowsPerThread;
    const int t = threadIdx.x - 6 * 32;        // 0..255
    const int gid = t / kGroupThreads, tg = t % kGroupThreads;
    // Packed codes and scales of the group's next stages are fetched into registers while the
    // current one is dequantised.
    struct Cursor {
      int g, kb;
      const uint8_t* wq;
      const uint8_t* sf;
    };
    auto seek = [&](Cursor& c) {               // pointers of tile c.g (if any)
      if (c.g < total_tiles) {
        const TileInfo ti = decode_tile(c.g, mt_prefix, p.offsets, p.experts, n_tiles, S::kTileM);
        const int64_t tile_id = (static_cast<int64_t>(ti.expert % p.wexperts) * n_tiles + ti.nt) * k_blocks;
        const int first_row = tg;
        c.wq = p.wq + tile_id * (kGN * 32) + first_row * 32;
        c.sf = p.sf + tile_id * (kGN * 4) + first_row * 4;
      }
    };
    auto advance = [&](Cursor& c, int n) {
      c.kb += n;
      bool moved = false;
      while (c.kb >= k_blocks && c.g < total_tiles) { c.kb -= k_blocks; c.g += n_workers; moved = true; }
      if (moved) seek(c);
    };
    constexpr int kBufs = 3;                   // register sets: the current stage and two in flight
    uint32_t wbuf[kBufs][kRows][8];
    uint32_t sbuf[kBufs][kRows];
    auto fetch = [&](const Cursor& c, uint32_t (&w)[kRows][8], uint32_t (&sc)[kRows]) {
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const uint8_t* wk = c.wq + static_cast<int64_t>(c.kb) * (kGN * 32) + r * (kGroupThreads * 32);
        const uint8_t* sk = c.sf + static_cast<int64_t>(c.kb) * (kGN * 4) + r * (kGroupThreads * 4);
        const uint4 c0 = __ldg(reinterpret_cast<const uint4*>(wk));
        const uint4 c1 = __ldg(reinterpret_cast<const uint4*>(wk + 16));
        w[r][0] = c0.x; w[r][1] = c0.y; w[r][2] = c0.z; w[r][3] = c0.w;
        w[r][4] = c1.x; w[r][5] = c1.y; w[r][6] = c1.z; w[r][7] = c1.w;
        sc[r] = __ldg(reinterpret_cast<const uint32_t*>(sk));
      }
    };
    Cursor cons{worker, 0, nullptr, nullptr};
    seek(cons);
    advance(cons, gid);
    Cursor pf = cons;
#pragma unroll
    for (int u = 0; u < kBufs - 1; ++u)
      if (pf.g < total_tiles) { fetch(pf, wbuf[u], sbuf[u]); advance(pf, kGroups); }
    uint32_t it = gid;
    bool ok = true;
    GPROF_DECL;
    while (cons.g < total_tiles && ok) {
#pragma unroll
      for (int u = 0; u < kBufs; ++u) {
        if (cons.g >= total_tiles) break;
        if (pf.g < total_tiles) {
          fetch(pf, wbuf[(u + kBufs - 1) % kBufs], sbuf[(u + kBufs - 1) % kBufs]);
          advance(pf, kGroups);
        }
        GPROF_MARK(0);
        const int s = it % kBStages;
        const uint32_t ph = (it / kBStages) & 1;
        if (*abort_flag || !mbar_wait(&b_empty[s], ph ^ 1)) { ok = false; break; }
        GPROF_MARK(1);
        uint8_t* sb = smem + S::kBRing + s * S::kBBytes;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const int row = tg + r * kGroupThreads;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint32_t scale2 = scale_pair(lut, (sbuf[u][r] >> (8 * (c >> 1))) & 0xffu);
            *reinterpret_cast<uint4*>(sb + swz128(row, c)) = dequant8(wbuf[u][r][c], scale2);
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&b_full[s]);
        GPROF_MARK(2);
        it += kGroups;
        advance(cons, kGroups);
        GPROF_MARK(3);
      }
    }
#ifdef MSL_GROUPED_PROF
    prof_acc[7] = it / kGroups;
    if (t == 0) GPROF_FLUSH(8, 8);
    if (t == kGroupThreads) GPROF_FLUSH(16, 8);
#endif
    if (!ok && lane == 0) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
  }

  if (warp == 0 && lane == 0 && *abort_flag) drain_pause();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 2 * kGN);
  }
}

// ---------------------------------------------------------------------------- load-time re-tiling
// src: codes [banks, rows, k/2] (element 2i in the low nibble of byte i), scales [banks, rows, k/16].
// dst tiles of 256 rows x 64 k; with `interleave` (gate/up bank, rows = 2 * inter) tile j holds gate
// rows [128 j, 128 j + 128) then up rows inter + [128 j, 128 j + 128).  Rows beyond the source are zero
// codes / zero scales.  Within each 32-bit word (8 consecutive k) the codes are re-placed bit by bit
// as dequant8 expects.  Lossless: a permutation of the input bits.
__device__ __forceinline__ uint32_t place_code(uint32_t code, int j) {
  const uint32_t mag = code & 7u, sgn = code >> 3;
  switch (j) {
    case 0: return (mag << 6) | (sgn << 15);
    case 1: return (mag << 3) | (sgn << 12);
    case 2: return mag | (sgn << 9);
    default: return ((code & 1u) << 10) | (((code >> 1) & 1u) << 11) | (((code >> 2) & 1u) << 13) | (sgn << 14);
  }
}

__global__ void nvfp4_repack_kernel(const uint8_t* __restrict__ src_q, const uint8_t* __restrict__ src_sf,
                                    uint8_t* __restrict__ dst_q, uint8_t* __restrict__ dst_sf, int experts, int rows,
                                    int k, int n_pad, int interleave) {
  const int k_blocks = k / kGK, n_tiles = n_pad / kGN;
  const int64_t total = static_cast<int64_t>(experts) * n_tiles * k_blocks * kGN;
  const int inter = rows / 2;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i % kGN);
    int64_t q = i / kGN;
    const int kb = static_cast<int>(q % k_blocks);
    q /= k_blocks;
    const int nt = static_cast<int>(q % n_tiles);
    const int e = static_cast<int>(q / n_tiles);
    int src_row;
    if (interleave) {
      const int gi = nt * (kGN / 2) + (r & (kGN / 2 - 1));
      src_row = gi < inter ? (r < kGN / 2 ? gi : inter + gi) : -1;
    } else {
      src_row = nt * kGN + r;
      if (src_row >= rows) src_row = -1;
    }
    uint32_t words[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint32_t sc = 0;
    if (src_row >= 0) {
      const uint8_t* sq = src_q + (static_cast<int64_t>(e) * rows + src_row) * (k / 2) + kb * 32;
      for (int w = 0; w < 8; ++w) {
        uint32_t out = 0;
        for (int b = 0; b < 4; ++b) {
          const uint32_t byte = sq[w * 4 + b];           // elements 2b (low nibble) and 2b+1 (high nibble)
          out |= place_code(byte & 0xfu, b) | (place_code(byte >> 4, b) << 16);
        }
        words[w] = out;
      }
      const uint8_t* ss = src_sf + (static_cast<int64_t>(e) * rows + src_row) * (k / 16) + kb * 4;
      sc = ss[0] | (ss[1] << 8) | (ss[2] << 16) | (static_cast<uint32_t>(ss[3]) << 24);
    }
    uint32_t* dq = reinterpret_cast<uint32_t*>(dst_q + i * 32);
    for (int w = 0; w < 8; ++w) dq[w] = words[w];
    *reinterpret_cast<uint32_t*>(dst_sf + i * 4) = sc;
  }
}

}  // namespace msl

using namespace msl;

extern "C" int64_t msl_nvfp4_padded_rows(int rows, int interleave) {
  if (interleave) {
    const int inter = rows / 2;
    return 2 * static_cast<int64_t>((inter + kGN / 2 - 1) / (kGN / 2)) * (kGN / 2);
  }
  return static_cast<int64_t>((rows + kGN - 1) / kGN) * kGN;
}

extern "C" int msl_nvfp4_repack(const void* src_codes, const void* src_scales, void* dst_codes, void* dst_scales,
                                int experts, int rows, int k, int interleave, void* stream) {
  if (!src_codes || !src_scales || !dst_codes || !dst_scales || experts <= 0 || rows <= 0 || k <= 0)
    return MSL_ERR_ARG;
  if (k % kGK) return MSL_ERR_UNSUPPORTED;
  if (interleave && (rows & 1)) return MSL_ERR_ARG;
  const int n_pad = static_cast<int>(msl_nvfp4_padded_rows(rows, interleave));
  const int64_t total = static_cast<int64_t>(experts) * n_pad * (k / kGK);
  const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 16));
  nvfp4_repack_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src_codes), static_cast<const uint8_t*>(src_scales),
      static_cast<uint8_t*>(dst_codes), static_cast<uint8_t*>(dst_scales), experts, rows, k, n_pad, interleave);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

template <int MODE>
static int launch_grouped(const CUtensorMap& tx, const GroupedArgs& a, int64_t slab_rows, int experts, int n_padded,
                          cudaStream_t st) {
  using S = GroupedCfg<MODE>;
  const int smem = std::min(S::kTotal + 1024, 232448);      // alignment slack as far as one CTA's limit allows
  static SmemConfig config;
  if (int rc = config.ensure(grouped_nvfp4_kernel<MODE>, smem)) return rc;
  // Upper bound on tiles without reading the device counts: every group may add one partial tile.
  const int64_t max_tiles = ((slab_rows + S::kTileM - 1) / S::kTileM + experts) * (n_padded / kGN);
  const int grid = static_cast<int>(std::min<int64_t>(max_tiles, sm_count()));
  grouped_nvfp4_kernel<MODE><<<grid, 448, smem, st>>>(tx, a);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

extern "C" int msl_grouped_gemm_nvfp4(const void* x, int64_t slab_rows, const void* codes, const void* scales,
                                      const float* global_scales, const int* offsets, void* out, int64_t ld_out,
                                      int experts, int weight_experts, int n_padded, int k, int n_out, int swiglu,
                                      int* status, void* stream) {
  if (!x || !codes || !scales || !global_scales || !offsets || !out) return MSL_ERR_ARG;
  if (experts <= 0 || experts > kMaxLocal || weight_experts <= 0 || n_padded <= 0 || k <= 0 || n_out <= 0 ||
      slab_rows < 0)
    return MSL_ERR_ARG;
  if ((n_padded % kGN) || (k % kGK)) return MSL_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (ld_out & 7) || (reinterpret_cast<uintptr_t>(out) & 15))
    return MSL_ERR_ALIGN;
  if (slab_rows == 0) return MSL_OK;
  CUtensorMap tx;
  int rc = make_tmap_2d(&tx, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, slab_rows, static_cast<uint64_t>(k) * 2, kGK,
                        kSubM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  GroupedArgs a{static_cast<const uint8_t*>(codes), static_cast<const uint8_t*>(scales), global_scales, offsets, out,
                ld_out, slab_rows, experts, n_padded, k, weight_experts, n_out, swiglu, status};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // 256-row tiles unless the groups are tiny on average.  Both geometries advance at the pace of the weight
  // producers when a tile has a single 128-row sub-tile (about 1150 cycles per K step), so a 256-row tile never
  // costs more per step than a 128-row one, and a skewed routing (the row counts live on the device, the host
  // sees the slab's size only) gives the busiest groups half as many tiles: 1367 rows on 14 of 32 groups, two
  // of them with a third of the rows each, take 4 instead of 5 rounds of tiles (203 + 107 against 222 + 133 us
  // for the two products).  What the 128-row geometry keeps is its second accumulator set (the epilogue, a
  // tenth of a tile at K = 4096, hides under the next tile), which pays when no group exceeds 128 rows.
  // (Letting single-sub-tile tiles of the 256-row geometry take the two halves of the accumulator columns in
  // turn recovers that overlap, 180 against 183 us on those 1367 rows, but measured 1 % slower wherever full
  // tiles dominate: not kept.  Three producer groups, 576 threads with 4 weight and 3 activation slots, were
  // slower on every shape tried: the 112 registers left per thread spill in the epilogue.  Asking L2 for a
  // step's packed weights eight steps ahead (cp.async.bulk.prefetch.L2 from the TMA lane) gave those 1367 rows
  // 566 against 574 us per layer, their weights coming from HBM with no other reader, and cost products whose
  // groups have many row tiles 1-3 %: not kept.)
  const bool use_wide = slab_rows >= 32LL * experts && option(MSL_OPT_GROUPED_WIDE) != 0;
  return use_wide ? launch_grouped<kWide>(tx, a, slab_rows, experts, n_padded, st)
                  : launch_grouped<kNarrow>(tx, a, slab_rows, experts, n_padded, st);
}

#ifdef MSL_GROUPED_PROF
extern "C" int msl_debug_grouped_prof(unsigned long long* out, int reset) {
  if (cudaMemcpyFromSymbol(out, msl::g_grouped_prof, sizeof(msl::g_grouped_prof)) != cudaSuccess) return MSL_ERR_CUDA;
  if (reset) {
    unsigned long long zero[32] = {};
    if (cudaMemcpyToSymbol(msl::g_grouped_prof, zero, sizeof(zero)) != cudaSuccess) return MSL_ERR_CUDA;
  }
  return MSL_OK;
}
#endif
