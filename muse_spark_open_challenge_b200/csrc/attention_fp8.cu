// Causal varlen attention over a paged FP8 (E4M3) K/V cache on tcgen05, GQA-packed.
//
// Replaces the reference layer's attention stage: the gather + sm_90a wgmma kernel + split-KV
// merge (muse_prefill_layer/submission.py:160-447,570-697), the library fallback for sliding
// windows (:712-721) and the per-head output norm and gate (:789-802); the arithmetic follows
// reference.py:376-409.
//
// One CTA per (request, KV head, block of 2 * 128/G query tokens), G = query heads per KV head.
// The CTA holds two 128-row query sub-tiles (rows are (token, head-in-group) pairs), so each K/V
// tile staged in shared memory serves 256 MMA rows.  384 threads:
//   warps 0-3, 4-7  softmax groups of sub-tile 0 / 1: one thread per row (TMEM lane = row).  The row of
//                   S (128 scores) is read from TMEM once and stays in registers; hidden keys of a tile
//                   on the causal diagonal or the window's edge are set to -inf by a separate mask pass,
//                   so the two hot passes exist once; row maximum (three-input max);
//                   P = 2^(8 - tau) exp2(s - m) as E4M3 written back to TMEM over the first 32 columns
//                   of the sub-tile's own S (four keys per 32-bit column: the layout of an 8-bit A
//                   operand in tensor memory), in two halves of 64 keys so that P V can start on the
//                   first half while the second is still being formed; running sum.  The running
//                   maximum moves only when some row of the warp exceeds it by more than tau; then all
//                   32 rows move to their newest maximum and O is rescaled in TMEM after the
//                   exponential pass, when the scores' registers are free to carry it in wide pieces.
//                   The two warps that share a scheduler (one of each group) TAKE TURNS at the
//                   exponential pass (a pair of mbarriers per scheduler): while one forms its
//                   exponentials the other waits for its next S, reads it and finds its maximum; the
//                   turn passes on after the first 64 keys of a tile.
//                   Epilogue (1/l, v_scale, optional per-head RMS norm * sigmoid(gate)) -> bf16
//   warp  8         TMEM allocation + tcgen05.mma issue.  All 32 lanes run the control flow (addresses
//                   and descriptors stay warp-uniform), one elected lane executes the MMAs and commits:
//                   S_s = Q_s K^T (both operands from shared memory) and O_s += P_s V with P as the A
//                   operand FROM TMEM and V consumed N-major straight from its [key][d] tile (FP8
//                   operands, fp32 accumulators in TMEM).  Per sub-tile the order is P V(j) then
//                   Q K^T(j+1): the tensor pipe runs them in that order, so S(j+1) may overwrite the
//                   columns P(j) was read from, and a finished Q K^T(j+1) implies a finished P V(j)
//                   (nobody waits for P V explicitly)
//   warp  9         TMA: the two Q sub-tiles, and whole 128-key K/V tiles as two 64-row boxes per
//                   tensor when the page size is a multiple of 64 and every key of the tile exists
//   warps 10-11     gather loaders for all other tiles (any page size, ragged tail), taking alternate
//                   tiles: four keys per lane, 16-byte copies into the swizzled tile, zeros for keys past
//                   the causal end
// K/V tiles move through a 4-stage ring.  TMEM: S0 | S1 | O0 | O1 (512 columns), P inside S.  Every
// wait is bounded.
//
// What bounds it (cycle counters of the development build below, 4 x 4096 tokens, head_dim 128, per
// 128-key tile and softmax warp): waiting for S 1200, reading it 115, maximum 450, waiting for the turn
// 400-600, exponentials + P 1450, rescale 220 (one tile in two has one), stores + arrivals 110: about
// 3900 cycles, of which the tensor pipe works about 1000.  The unit that sets the floor is the one that
// runs ex2: microbenchmarks on this GPU (msl_unit_peak) give 8 cycles per ex2.approx warp instruction and
// scheduler whatever the number of warps (ex2 on f16x2 pairs 16: no gain); the FP8 pair conversion takes 4
// alone and hides under the exponentials (two ex2 and one conversion: 16.0), so a tile costs each scheduler
// 2 warps x 128 x 8 = 2048 cycles there, twice its tensor time; the kernel runs at 53-55 % of that floor, the
// rest being the chain maximum -> exponentials -> P -> MMA of each sub-tile.  Other facts measured on the way: max
// with two or three inputs takes 2 cycles; a tcgen05.mma never takes less than about 57 cycles (M128 with
// N <= 64 runs as long as with N = 128), so smaller S tiles cost tensor time without saving any; a warp
// whose unrolled code outgrows the instruction cache loses half its speed, which is why two warps in
// lockstep on the same code did better than their instruction counts say.
// Variants that were built and measured slower on the same inputs (0.64 ms before the turns, 0.575 ms
// with them): two threads per row (16 softmax warps, 0.68 ms), one MMA issuer per sub-tile (0.72 ms),
// 64-key S halves as separate buffers so that the next S is formed under the softmax of the other half
// (0.64 ms in lockstep, 0.72 ms with turns: twice the Q K^T instructions and twice the per-pass ramps),
// part of the exponentials as a cubic on the FMA pipe (0.60 ms with turns, 0.60 ms without), S read
// from TMEM a second time for the exponential pass instead of being held in 128 registers (0.67 ms),
// mbarrier waits with a suspend-time hint (no change), tau = 6 (0.568 ms, not kept: less range below
// the reference maximum); at head_dim 64, where TMEM has room, P in columns of its own with Q K^T(j+1)
// issued as soon as S(j) is in registers (the wait for S shrinks from 800 to 470 cycles, the exponential
// pass grows by as much: 0.54 against 0.50 ms); no turns but a quarter of the exponentials as a cubic
// (0.582 ms, and 0.503 ms at head_dim 64: the same as the turns); an epilogue in which quads of lanes
// exchange 4 x 4 blocks by shuffles so that gate rows are read and output rows written 128 contiguous
// bytes at a time, as the GEMM epilogues do (0.581 against 0.573 ms at head_dim 128, 0.496 against
// 0.502 ms at 64: the 128 shuffles per 64 columns cost what the wider requests save).
#include "msl_common.cuh"
#include "msl_host.h"

namespace msl {

constexpr int kAM = 128;    // rows per query sub-tile
constexpr int kAN = 128;    // keys per tile
constexpr int kAStages = 4;
constexpr float kTau = 4.0f;   // log2 slack of the running softmax maximum before O is rescaled

// Phase timing for development builds (-DMSL_ATTN_PROF): cycles summed over all CTAs, per phase of two
// softmax warps and of the MMA issuer; read back with msl_debug_attn_prof.
#ifdef MSL_ATTN_PROF
__device__ unsigned long long g_attn_prof[32];
#define PROF_DECL long long prof_t = clock64(); long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define PROF_MARK(i) do { const long long now_ = clock64(); prof_acc[i] += now_ - prof_t; prof_t = now_; } while (0)
#define PROF_FLUSH(base, n) do { for (int i_ = 0; i_ < (n); ++i_) atomicAdd(&g_attn_prof[(base) + i_], (unsigned long long)prof_acc[i_]); } while (0)
#else
#define PROF_DECL do {} while (0)
#define PROF_MARK(i) do {} while (0)
#define PROF_FLUSH(base, n) do {} while (0)
#endif

struct AttnArgs {
  const uint8_t* k_cache;       // [cache rows][hkv][D] e4m3
  const uint8_t* v_cache;
  const int* page_table;        // [batch][max_pages]
  int max_pages;
  const int* seq_lens;          // [batch] cached tokens before the block
  const int* cu_seqlens_q;      // [batch + 1]
  const float* k_scale;         // device scalars
  const float* v_scale;
  float softmax_scale;          // sm_scale * qk_scale_factor (k_scale is applied in the kernel)
  int hq, hkv, page_size, window;
  int64_t cache_rows;
  void* out;                    // bf16 [tokens][hq * D]
  int64_t ld_out;
  const __nv_bfloat16* gate;    // bf16, row pitch ld_gate, column h * D + d; NULL = no norm/gate epilogue
  int64_t ld_gate;
  int* status;
  // Split-KV mode (kv_splits > 1): every CTA covers one slice of its query block's key tiles and
  // leaves an unnormalised partial result for merge_splits_kernel.
  int kv_splits;
  int tokens;
  float* part_o;                // [kv_splits][tokens][hq][D] fp32, relative to the slice's own maximum
  float* part_ml;               // [kv_splits][tokens][hq][2]: running maximum (log2 units), row sum
};

template <int D>
struct AttnSmem {
  static constexpr int kTile = kAN * D;                    // bytes of one K or V tile, and of one Q sub-tile
  static constexpr int kQ = 0;                             // 2 sub-tiles
  static constexpr int kKV = 2 * kTile;                    // stages of (K tile, V tile)
  static constexpr int kBar = kKV + kAStages * 2 * kTile;
  // q_full, kv_full[stages], kv_empty[stages], s_full[2], p_lo[2], p_hi[2], pv_done[2], turn[2][4]
  static constexpr int kNumBars = 1 + 2 * kAStages + 16;
  static constexpr int kTotal = kBar + kNumBars * 8 + 16;
};

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile with ROWB-byte rows (64 or 128) laid
// out with the matching swizzle: the chunk index is XORed with bits of the row index so that the
// pattern repeats every 1024 / 512 bytes (128-byte rows: row mod 8; 64-byte rows: (row / 2) mod 4).
template <int ROWB>
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk) {
  if constexpr (ROWB == 128) return row * 128u + ((chunk ^ (row & 7u)) << 4);
  else return row * 64u + ((chunk ^ ((row >> 1) & 3u)) << 4);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&o)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]),
      "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15]), "r"(o[16]),
      "r"(o[17]), "r"(o[18]), "r"(o[19]), "r"(o[20]), "r"(o[21]), "r"(o[22]), "r"(o[23]), "r"(o[24]), "r"(o[25]),
      "r"(o[26]), "r"(o[27]), "r"(o[28]), "r"(o[29]), "r"(o[30]), "r"(o[31])
      : "memory");
}

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3)) |
         (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3)) << 16);
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// One 64-column half of a row of S: exponentials (scaled by 2^(8 - tau)) summed into l and packed as
// E4M3, four keys per word in key order: the layout of an 8-bit A operand in TMEM.
__device__ __forceinline__ void softmax_half(const uint32_t (&s0)[32], const uint32_t (&s1)[32], float scale_log2,
                                             float neg_m, float& l, uint32_t (&packed)[16]) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t(&s)[32] = h ? s1 : s0;
    float e[32];
    float part[4] = {0.f, 0.f, 0.f, 0.f};                  // independent chains
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      e[i] = ex2_approx(fmaf(__uint_as_float(s[i]), scale_log2, neg_m));
      part[i & 3] += e[i];
    }
    l += (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
    for (int q = 0; q < 8; ++q)
      packed[8 * h + q] = e4m3x4(e[4 * q], e[4 * q + 1], e[4 * q + 2], e[4 * q + 3]);
  }
}

__device__ __forceinline__ float row_max_half(const uint32_t (&s0)[32], const uint32_t (&s1)[32], float m) {
  float acc[4] = {m, -INFINITY, -INFINITY, -INFINITY};     // independent chains
#pragma unroll
  for (int i = 0; i < 32; ++i) acc[i & 3] = max3(acc[i & 3], __uint_as_float(s0[i]), __uint_as_float(s1[i]));
  return fmaxf(fmaxf(acc[0], acc[1]), fmaxf(acc[2], acc[3]));
}

// Scores of hidden keys (column > lim_hi or <= lim_lo) become -inf: they then lose every maximum and
// their exponentials are exactly 0.  Only tiles that touch the causal diagonal or the window's edge
// come here, so the two passes above exist once, without the masks.
__device__ __forceinline__ void mask_quarter(uint32_t (&s)[32], int col0, int lim_hi, int lim_lo) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int col = col0 + i;
    if (!(col <= lim_hi && col > lim_lo)) s[i] = 0xff800000u;
  }
}

template <int D>
__global__ void __launch_bounds__(384, 1)
attention_fp8_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, AttnArgs p) {
  using S = AttnSmem<D>;
  constexpr uint32_t kSwz = (D == 128) ? 2u : 4u;          // descriptor swizzle code
  constexpr uint32_t kSbo = 8 * D;                         // bytes between 8-row groups
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + kAStages;
  uint64_t* s_full = kv_empty + kAStages;
  uint64_t* p_lo = s_full + 2;
  uint64_t* p_hi = p_lo + 2;
  uint64_t* pv_done = p_hi + 2;
  uint64_t* turn = pv_done + 2;                            // [group][warp in group]: the exponential unit's turn
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + S::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.hq / p.hkv;
  const int TQ = kAM / G;                                  // query tokens per sub-tile
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int q_begin = p.cu_seqlens_q[b], q_len = p.cu_seqlens_q[b + 1] - q_begin;
  // Longest key ranges first: later query blocks attend to more keys.
  const int n_qblk = (q_len + 2 * TQ - 1) / (2 * TQ);
  const int split = static_cast<int>(blockIdx.x) % p.kv_splits;
  const int qblk = n_qblk - 1 - static_cast<int>(blockIdx.x) / p.kv_splits;
  if (qblk < 0) return;                                    // uniform for the CTA, before any barrier
  const int q0 = qblk * 2 * TQ;
  const int seq = p.seq_lens[b];
  const int min_qpos = seq + q0;
  int kt_begin = p.window ? max(0, min_qpos - p.window + 1) / kAN : 0;
  // per sub-tile: valid rows, last query position, number of key tiles
  int rows_valid[2], max_qpos[2], n_sub[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const int first = q0 + s * TQ;
    const int cnt = max(0, min(TQ, q_len - first));
    rows_valid[s] = cnt * G;
    max_qpos[s] = seq + first + cnt - 1;
    n_sub[s] = cnt > 0 ? max_qpos[s] / kAN + 1 - kt_begin : 0;
  }
  if (p.kv_splits > 1) {
    // this CTA's slice of the key tiles; a slice may be empty for one or both sub-tiles
    const int n_full = max(n_sub[0], n_sub[1]);
    const int chunk = (n_full + p.kv_splits - 1) / p.kv_splits;
    const int lo = split * chunk, hi = min(n_full, lo + chunk);
#pragma unroll
    for (int s = 0; s < 2; ++s) n_sub[s] = max(0, min(n_sub[s], hi) - lo);
    kt_begin += lo;
    if (max(n_sub[0], n_sub[1]) == 0) {                    // uniform for the CTA, before any barrier
      for (int i = threadIdx.x; i < 2 * kAM; i += blockDim.x) {
        const int s = i / kAM, r = i % kAM;
        if (r < rows_valid[s]) {
          const int64_t idx = (static_cast<int64_t>(split) * p.tokens + q_begin + q0 + s * TQ + r / G) * p.hq +
                              kvh * G + r % G;
          p.part_ml[2 * idx] = -INFINITY;
          p.part_ml[2 * idx + 1] = 0.f;
        }
      }
      return;
    }
  }
  const int n_tiles = max(n_sub[0], n_sub[1]);
  const int last_qpos = max(max_qpos[0], max_qpos[1]);
  const bool tma_pages = (p.page_size % 64) == 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kAStages; ++i) { mbar_init(&kv_full[i], 3); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_lo[i], 4);
      mbar_init(&p_hi[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    for (int i = 0; i < 8; ++i) mbar_init(&turn[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 8) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // A tile goes by TMA when its pages can be addressed as two 64-row boxes and none of its keys
  // lies past the last query (rows the cache may never have initialised must not reach the MMA).
  auto tile_by_tma = [&](int j) { return tma_pages && (kt_begin + j) * kAN + kAN - 1 <= last_qpos; };

  if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    // All 32 lanes run the control flow, so that addresses and descriptors are warp-uniform values;
    // one elected lane executes the MMAs and commits.
    {
      const uint32_t on = elect_one();
      constexpr uint32_t idesc_qk = make_idesc(0, 0, kAM, kAN);
      constexpr uint32_t idesc_pv = make_idesc(0, 0, kAM, D, 0, 1);     // A = P from TMEM (K-major), B = V, N-major
      const uint32_t sq = smem_u32(smem + S::kQ);
      auto issue_qk = [&](int s, uint32_t sk) {
#pragma unroll
        for (int k = 0; k < D / 32; ++k)
          tc_mma_f8_if(on, tmem_base + s * kAN, make_sdesc(sq + s * S::kTile + k * 32, 16, kSbo, kSwz),
                       make_sdesc(sk + k * 32, 16, kSbo, kSwz), idesc_qk, k != 0);
        tc_commit_if(on, &s_full[s]);
      };
      // keys [64 half, 64 half + 64) of the tile: P columns [16 half, +16) of the sub-tile's S, 8 per MMA
      auto issue_pv_half = [&](int s, uint32_t sv, int half, bool first) {
#pragma unroll
        for (int k = 2 * half; k < 2 * half + 2; ++k)
          tc_mma_f8_ts_if(on, tmem_base + 2 * kAN + s * kAN, tmem_base + s * kAN + k * 8,
                          make_sdesc(sv + k * 32 * D, 16, kSbo, kSwz), idesc_pv, !(first && k == 0));
      };
      PROF_DECL;
      bool ok = mbar_wait(q_full, 0) && mbar_wait(&kv_full[0], 0);
      PROF_MARK(0);
      if (ok) {
        tc_fence_after();
        const uint32_t sk0 = smem_u32(smem + S::kKV);
        if (n_sub[0] > 0) issue_qk(0, sk0);
        if (n_sub[1] > 0) issue_qk(1, sk0);
      }
      // Per tile j and sub-tile s: P V(j) as soon as the group has published the halves of P(j), then
      // Q K^T(j+1) right behind it on the tensor pipe (it overwrites the S columns P(j) lived in).
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % kAStages;
        const uint32_t ph = j & 1;
        const uint32_t sv = smem_u32(smem + S::kKV + st * 2 * S::kTile + S::kTile);
        const int st1 = (j + 1) % kAStages;
        const uint32_t sk1 = smem_u32(smem + S::kKV + st1 * 2 * S::kTile);
        bool next_ready = false;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (j < n_sub[s]) {
            PROF_MARK(1);
            if (*abort_flag || !mbar_wait(&p_lo[s], ph)) { ok = false; break; }
            PROF_MARK(2);
            tc_fence_after();
            issue_pv_half(s, sv, 0, j == 0);
            PROF_MARK(1);
            if (*abort_flag || !mbar_wait(&p_hi[s], ph)) { ok = false; break; }
            PROF_MARK(3);
            tc_fence_after();
            issue_pv_half(s, sv, 1, false);
            if (j == n_sub[s] - 1) tc_commit_if(on, &pv_done[s]);
            if (j + 1 < n_sub[s]) {
              if (!next_ready) {
                PROF_MARK(1);
                if (*abort_flag || !mbar_wait(&kv_full[st1], ((j + 1) / kAStages) & 1)) { ok = false; break; }
                PROF_MARK(4);
                tc_fence_after();
                next_ready = true;
              }
              issue_qk(s, sk1);
            }
          }
        }
        if (!ok) break;
        tc_commit_if(on, &kv_empty[st]);
      }
      PROF_MARK(1);
      if (lane == 0) PROF_FLUSH(8, 5);
      if (!ok && lane == 0) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ TMA loader
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      const int nq = n_sub[1] > 0 ? 2 : 1;
      mbar_expect_tx(q_full, nq * S::kTile);
      for (int s = 0; s < nq; ++s)
        tma_load_3d(smem + S::kQ + s * S::kTile, &tm_q, q_full, 0, kvh * G, q_begin + q0 + s * TQ);
      const int* pt = p.page_table + static_cast<int64_t>(b) * p.max_pages;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % kAStages;
        if (*abort_flag || !mbar_wait(&kv_empty[st], ((j / kAStages) & 1) ^ 1, true)) { ok = false; break; }
        if (!tile_by_tma(j)) { mbar_arrive(&kv_full[st]); continue; }
        uint8_t* sk = smem + S::kKV + st * 2 * S::kTile;
        mbar_expect_tx(&kv_full[st], 2 * S::kTile);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int key0 = (kt_begin + j) * kAN + half * 64;
          const int pg = pt[key0 / p.page_size];
          const int row0 = pg * p.page_size + key0 % p.page_size;
          tma_load_3d(sk + half * 64 * D, &tm_k, &kv_full[st], 0, kvh, row0);
          tma_load_3d(sk + S::kTile + half * 64 * D, &tm_v, &kv_full[st], 0, kvh, row0);
        }
      }
      if (!ok) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
    }
  } else if (warp >= 10) {
    // ------------------------------------------------------------------ gather loaders
    // The two warps take alternate tiles, so that two tiles' chains (page table entry -> K/V rows -> shared
    // memory) are in flight at once: with one-token pages a chain takes longer than the softmax of a tile at
    // head_dim 64.  The warp that does not own a tile only passes the barrier on.  A lane carries kPass keys
    // at a time (rows lane, lane + 32, ... of the tile): all four at head_dim 64, two and two at 128.
    const int gw = warp - 10;
    constexpr int kPass = (D <= 64) ? 4 : 2;
    const int* pt = p.page_table + static_cast<int64_t>(b) * p.max_pages;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j % kAStages;
      const uint32_t e_ph = ((j / kAStages) & 1) ^ 1;
      if (tile_by_tma(j) || (j & 1) != gw) {
        if (*abort_flag || !mbar_wait(&kv_empty[st], e_ph, true)) { ok = false; break; }
        __syncwarp();
        if (lane == 0) mbar_arrive(&kv_full[st]);
        continue;
      }
      uint8_t* sk = smem + S::kKV + st * 2 * S::kTile;
      uint8_t* sv = sk + S::kTile;
#pragma unroll
      for (int h0 = 0; h0 < 4 && ok; h0 += kPass) {
        uint4 kq[kPass][D / 16], vq[kPass][D / 16];
#pragma unroll
        for (int h = 0; h < kPass; ++h) {
          const int key = (kt_begin + j) * kAN + lane + 32 * (h0 + h);
          int64_t row = -1;
          if (key <= last_qpos) {
            const int pg = pt[key / p.page_size];
            if (pg >= 0) row = static_cast<int64_t>(pg) * p.page_size + key % p.page_size;
            if (row >= p.cache_rows) row = -1;
          }
          if (row >= 0) {
            const uint4* ks = reinterpret_cast<const uint4*>(p.k_cache + (row * p.hkv + kvh) * D);
            const uint4* vs = reinterpret_cast<const uint4*>(p.v_cache + (row * p.hkv + kvh) * D);
#pragma unroll
            for (int c = 0; c < D / 16; ++c) { kq[h][c] = ks[c]; vq[h][c] = vs[c]; }
          } else {
#pragma unroll
            for (int c = 0; c < D / 16; ++c) { kq[h][c] = make_uint4(0, 0, 0, 0); vq[h][c] = make_uint4(0, 0, 0, 0); }
          }
        }
        if (h0 == 0) {                                       // the loads above are in flight while the slot frees
          if (*abort_flag || !mbar_wait(&kv_empty[st], e_ph, true)) { ok = false; break; }
        }
#pragma unroll
        for (int h = 0; h < kPass; ++h) {
#pragma unroll
          for (int c = 0; c < D / 16; ++c) {
            *reinterpret_cast<uint4*>(sk + swz<D>(lane + 32 * (h0 + h), c)) = kq[h][c];
            *reinterpret_cast<uint4*>(sv + swz<D>(lane + 32 * (h0 + h), c)) = vq[h][c];
          }
        }
      }
      if (!ok) break;
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&kv_full[st]);
    }
    if (!ok && lane == 0) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int sub = warp >> 2;                             // query sub-tile of this group
    const int r = (warp & 3) * 32 + lane;                  // row = TMEM lane
    const int n_mine = n_sub[sub], n_other = n_sub[sub ^ 1];
    const int tq = r / G, g = r - tq * G;
    const bool row_valid = r < rows_valid[sub];
    const int first_tok = q0 + sub * TQ;
    const int qpos = seq + min(first_tok + tq, max(q_len - 1, 0));
    const int sub_min_qpos = seq + first_tok;
    const float scale_log2 = p.softmax_scale * (*p.k_scale) * 1.4426950408889634f;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + sub * kAN + lane_sel;
    const uint32_t tmem_o = tmem_base + 2 * kAN + sub * kAN + lane_sel;
    float m_run = -INFINITY, l_run = 0.f;                  // l accumulates 2^(8 - kTau) * sum of exponentials
    bool ok = true;
    PROF_DECL;
    for (int j = 0; j < n_mine && ok; ++j) {
      const uint32_t ph = j & 1;
      const int key0 = (kt_begin + j) * kAN;
      if (*abort_flag || !mbar_wait(&s_full[sub], ph)) { ok = false; break; }
      PROF_MARK(0);
      tc_fence_after();
      const bool full_tile =
          (key0 + kAN - 1 <= sub_min_qpos) && (!p.window || key0 > max_qpos[sub] - p.window);
      const int lim_hi = qpos - key0;                       // visible columns: lim_lo < col <= lim_hi
      const int lim_lo = p.window ? qpos - p.window - key0 : -1;
      // The whole row of S (128 columns) is read from TMEM once and stays in registers for both passes.
      uint32_t sa[32], sb[32], sc[32], sd[32];
      tmem_ld32(tmem_s, sa);
      tmem_ld32(tmem_s + 32, sb);
      tmem_ld32(tmem_s + 64, sc);
      tmem_ld32(tmem_s + 96, sd);
      tmem_ld_wait();
      PROF_MARK(1);
      if (!full_tile) {
        mask_quarter(sa, 0, lim_hi, lim_lo);
        mask_quarter(sb, 32, lim_hi, lim_lo);
        mask_quarter(sc, 64, lim_hi, lim_lo);
        mask_quarter(sd, 96, lim_hi, lim_lo);
      }
      // pass 1: row maximum of the raw scores
      const float m_tile = row_max_half(sc, sd, row_max_half(sa, sb, -INFINITY));
      // The reference maximum m_run moves only when the tile's maximum exceeds it by more than kTau
      // (log2 units): the exponentials then stay below 2^kTau, P = 2^(8 - kTau) * exp2(.) stays within
      // E4M3's range (<= 256), and the rescale of O in TMEM below becomes rare instead of per tile.
      const float m_cand = m_tile * scale_log2;
      // When one row of the warp has to move, all 32 move to their newest maximum: the rescale below
      // costs the same for one row as for all, and rows brought up to date do not ask again soon.
      const bool event = __any_sync(0xffffffffu, m_cand > m_run + kTau || m_run == -INFINITY);
      float corr = 1.0f;
      if (event) {
        const float m_new = fmaxf(m_run, m_cand);
        corr = ex2_approx(m_run - ((m_new == -INFINITY) ? 0.f : m_new));   // 0 when m_run = -inf
        m_run = m_new;
      }
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      const bool resc = j > 0 && event;                     // warp-uniform
      PROF_MARK(2);
      // The two warps that share a scheduler (one of each group) take turns at the exponential pass:
      // alone, a warp keeps the ex2 unit busy; together they would run the pass in lockstep at half
      // speed each and then sit idle together while their next S tiles are formed.  Order: group 0
      // tile 0, group 1 tile 0, group 0 tile 1, ...; a turn is skipped where the partner has no such tile.
      if (sub == 0 ? (j >= 1 && j - 1 < n_other) : (j < n_other)) {
        if (*abort_flag || !mbar_wait(&turn[sub * 4 + (warp & 3)], (sub == 0 ? j - 1 : j) & 1)) { ok = false; break; }
      }
      PROF_MARK(3);
      // pass 2: P = 2^(8 - kTau) * exp2(s * scale - m) as E4M3 into TMEM, row sum in fp32.  On a tile
      // without a rescale the first 64 keys are published before the last 64 are formed.
      const float neg_m = (8.0f - kTau) - m_use;
      float l_tile = 0.f;
      uint32_t pk[16], pk2[16];
      softmax_half(sa, sb, scale_log2, neg_m, l_tile, pk);
      if (!resc) {
        tmem_st16(tmem_s, pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_lo[sub]);
      }
      // hand the turn to the partner warp (its tile j from group 0, its tile j + 1 from group 1) before the
      // second half: the partner's first exponentials fill the gaps of this warp's last ones (the same time at
      // head_dim 128, 0.493 against 0.501 ms at head_dim 64 on 4096 queries over 16384 cached keys)
      __syncwarp();
      if (lane == 0 && (sub == 0 ? (j < n_other) : (j + 1 < n_other))) mbar_arrive(&turn[(sub ^ 1) * 4 + (warp & 3)]);
      softmax_half(sc, sd, scale_log2, neg_m, l_tile, pk2);
      PROF_MARK(4);
      if (resc) {
        // O moves to the new maximum before any of this tile's P is used.  S(j) was ready only after
        // P V(j-1) had finished (the tensor pipe ran it first), so O is quiet; and the scores are no
        // longer needed, so their registers carry O through in wide pieces.
#pragma unroll
        for (int c = 0; c < D; c += 64) {
          uint32_t oa[32], ob[32];
          tmem_ld32(tmem_o + c, oa);
          tmem_ld32(tmem_o + c + 32, ob);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            oa[i] = __float_as_uint(__uint_as_float(oa[i]) * corr);
            ob[i] = __float_as_uint(__uint_as_float(ob[i]) * corr);
          }
          tmem_st32(tmem_o + c, oa);
          tmem_st32(tmem_o + c + 32, ob);
        }
        tmem_st16(tmem_s, pk);
      }
      PROF_MARK(5);
      tmem_st16(tmem_s + 16, pk2);
      tmem_st_wait();                                       // P and a rescaled O
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (resc) mbar_arrive(&p_lo[sub]);
        mbar_arrive(&p_hi[sub]);
      }
      PROF_MARK(6);
      l_run = l_run * corr + l_tile;
    }
#ifdef MSL_ATTN_PROF
    if (threadIdx.x == 0) { prof_acc[7] = n_mine; PROF_FLUSH(0, 8); }
    if (threadIdx.x == 128) { prof_acc[7] = n_mine; PROF_FLUSH(16, 8); }
#endif
    // ---------------------------------------------------------------- epilogue
    if (ok && n_mine > 0) {
      if (*abort_flag || !mbar_wait(&pv_done[sub], 0)) ok = false;     // committed once, behind the last P V
    }
    if (p.kv_splits > 1) {
      // partial result of this key slice: O as it stands in TMEM, with the maximum and sum it refers to
      const bool have = ok && n_mine > 0;
      if (have) tc_fence_after();
      const int64_t idx = (static_cast<int64_t>(split) * p.tokens + q_begin + first_tok + tq) * p.hq + kvh * G + g;
      if (row_valid) {
        p.part_ml[2 * idx] = have ? m_run : -INFINITY;
        p.part_ml[2 * idx + 1] = have ? l_run : 0.f;
      }
      if (have) {
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld32(tmem_o + c, o);
          tmem_ld_wait();
          if (row_valid) {
            float4* dst = reinterpret_cast<float4*>(p.part_o + idx * D + c);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[i] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]),
                                   __uint_as_float(o[4 * i + 2]), __uint_as_float(o[4 * i + 3]));
          }
        }
      }
    } else if (ok && n_mine > 0) {
      tc_fence_after();
      const float c_out = (*p.v_scale) / l_run;             // l_run carries the same power of two as P
      float r_norm = 1.0f;
      if (p.gate != nullptr) {
        float ss = 0.f;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld32(tmem_o + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) { const float v = __uint_as_float(o[i]) * c_out; ss += v * v; }
        }
        r_norm = 1.0f / sqrtf(ss / D + 1e-5f);
      }
      const int token = q_begin + first_tok + tq;
      const int head = kvh * G + g;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(token) * p.ld_out + head * D;
      const __nv_bfloat16* grow = p.gate ? p.gate + static_cast<int64_t>(token) * p.ld_gate + head * D : nullptr;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld32(tmem_o + c, o);
        tmem_ld_wait();
        if (row_valid) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i]) * c_out * r_norm;
          if (grow != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              const uint4 gq = *reinterpret_cast<const uint4*>(grow + c + i);
              const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float g0 = bf16_bits_to_f32(gw[e] & 0xffffu), g1 = bf16_bits_to_f32(gw[e] >> 16);
                v[i + 2 * e] *= 1.0f / (1.0f + __expf(-g0));
                v[i + 2 * e + 1] *= 1.0f / (1.0f + __expf(-g1));
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(orow + c + i) =
                make_uint4(pack_bf16x2(v[i], v[i + 1]), pack_bf16x2(v[i + 2], v[i + 3]),
                           pack_bf16x2(v[i + 4], v[i + 5]), pack_bf16x2(v[i + 6], v[i + 7]));
        }
      }
    }
    if (!ok && lane == 0) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
  }

  if (warp == 9 && lane == 0 && *abort_flag) drain_pause();
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// Merge of the key slices of split-KV attention: one warp per (token, head).  Slice s holds O_s and
// l_s relative to its own maximum m_s (log2 units); with M = max m_s the result is
// sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), then v_scale, the per-head RMS norm and the sigmoid
// gate exactly as in the single-pass epilogue.
template <int D>
__global__ void __launch_bounds__(256)
merge_splits_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int kv_splits, int tokens,
                    int hq, const float* __restrict__ v_scale, const __nv_bfloat16* __restrict__ gate,
                    int64_t ld_gate, __nv_bfloat16* __restrict__ out, int64_t ld_out) {
  constexpr int PER = D / 32;
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<int64_t>(tokens) * hq) return;
  const int64_t token = item / hq;
  const int head = static_cast<int>(item % hq);
  float m_all = -INFINITY;
  for (int s = 0; s < kv_splits; ++s) {
    const float* ml = part_ml + 2 * (static_cast<int64_t>(s) * tokens * hq + item);
    if (ml[1] > 0.f) m_all = fmaxf(m_all, ml[0]);
  }
  float acc[PER], l_all = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  for (int s = 0; s < kv_splits; ++s) {
    const int64_t at = static_cast<int64_t>(s) * tokens * hq + item;
    const float l_s = part_ml[2 * at + 1];
    if (l_s > 0.f) {
      const float w = ex2_approx(part_ml[2 * at] - m_all);
      l_all += l_s * w;
      const float* o = part_o + at * D + lane * PER;
#pragma unroll
      for (int i = 0; i < PER; ++i) acc[i] += o[i] * w;
    }
  }
  const float c_out = (*v_scale) / l_all;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) { acc[i] *= c_out; ss += acc[i] * acc[i]; }
  __nv_bfloat16* orow = out + token * ld_out + head * D + lane * PER;
  if (gate != nullptr) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float r_norm = 1.0f / sqrtf(ss / D + 1e-5f);
    const __nv_bfloat16* grow = gate + token * ld_gate + head * D + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] *= r_norm * (1.0f / (1.0f + __expf(-__bfloat162float(grow[i]))));
  }
#pragma unroll
  for (int i = 0; i < PER; i += 2)
    *reinterpret_cast<uint32_t*>(orow + i) = pack_bf16x2(acc[i], acc[i + 1]);
}

template <int D>
static int launch_attention(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnArgs& a,
                            int batch, int max_q_len, cudaStream_t st) {
  using S = AttnSmem<D>;
  const int smem = S::kTotal + 1024;
  static SmemConfig config;
  if (int rc = config.ensure(attention_fp8_kernel<D>, smem)) return rc;
  const int G = a.hq / a.hkv, TQ2 = 2 * (kAM / G);
  dim3 grid(((max_q_len + TQ2 - 1) / TQ2) * a.kv_splits, a.hkv, batch);
  attention_fp8_kernel<D><<<grid, 384, smem, st>>>(tq, tk, tv, a);
  if (a.kv_splits > 1) {
    const int64_t items = static_cast<int64_t>(a.tokens) * a.hq;
    merge_splits_kernel<D><<<static_cast<unsigned>((items + 7) / 8), 256, 0, st>>>(
        a.part_o, a.part_ml, a.kv_splits, a.tokens, a.hq, a.v_scale, a.gate, a.ld_gate,
        static_cast<__nv_bfloat16*>(a.out), a.ld_out);
  }
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

}  // namespace msl

using namespace msl;

static int attention_entry(const void* q8, const void* k_cache, const void* v_cache, const int* page_table,
                           int max_pages, const int* seq_lens, const int* cu_seqlens_q, const float* k_scale,
                           const float* v_scale, float softmax_scale, int batch, int max_q_len, int tokens, int hq,
                           int hkv, int head_dim, int page_size, int window, int64_t cache_rows, void* out,
                           int64_t ld_out, const void* gate, int64_t ld_gate, int kv_splits, void* workspace,
                           int* status, void* stream) {
  if (kv_splits < 1 || kv_splits > 64 || (kv_splits > 1 && !workspace)) return MSL_ERR_ARG;
  if (kv_splits > 1 && (reinterpret_cast<uintptr_t>(workspace) & 15)) return MSL_ERR_ALIGN;
  if (!q8 || !k_cache || !v_cache || !page_table || !seq_lens || !cu_seqlens_q || !k_scale || !v_scale || !out)
    return MSL_ERR_ARG;
  if (batch <= 0 || max_q_len <= 0 || tokens <= 0 || hq <= 0 || hkv <= 0 || hq % hkv || page_size <= 0 ||
      window < 0 || max_pages <= 0 || cache_rows <= 0)
    return MSL_ERR_ARG;
  const int G = hq / hkv;
  if (G > 128 || (G & (G - 1))) return MSL_ERR_UNSUPPORTED;
  if (head_dim != 64 && head_dim != 128) return MSL_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(q8) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (ld_out & 7) ||
      (gate && ((reinterpret_cast<uintptr_t>(gate) & 15) || (ld_gate & 7))))
    return MSL_ERR_ALIGN;
  AttnArgs a{static_cast<const uint8_t*>(k_cache), static_cast<const uint8_t*>(v_cache), page_table, max_pages,
             seq_lens, cu_seqlens_q, k_scale, v_scale, softmax_scale, hq, hkv, page_size, window, cache_rows, out,
             ld_out, static_cast<const __nv_bfloat16*>(gate), ld_gate, status, kv_splits, tokens, nullptr, nullptr};
  if (kv_splits > 1) {
    a.part_o = static_cast<float*>(workspace);
    a.part_ml = a.part_o + static_cast<int64_t>(kv_splits) * tokens * hq * head_dim;
  }
  CUtensorMap tq, tk, tv;
  const uint32_t box_t = static_cast<uint32_t>(kAM / G);
  const uint64_t d = static_cast<uint64_t>(head_dim);
  const CUtensorMapSwizzle swz_mode = head_dim == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  int rc = make_tmap_3d(&tq, q8, CU_TENSOR_MAP_DATA_TYPE_UINT8, d, hq, tokens, d, hq * d, head_dim, G, box_t, swz_mode);
  if (rc) return rc;
  // K/V caches as [rows][hkv][d]: one box = 64 consecutive cache rows of one KV head.
  rc = make_tmap_3d(&tk, k_cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, d, hkv, cache_rows, d, hkv * d, head_dim, 1, 64,
                    swz_mode);
  if (rc) return rc;
  rc = make_tmap_3d(&tv, v_cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, d, hkv, cache_rows, d, hkv * d, head_dim, 1, 64,
                    swz_mode);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return head_dim == 128 ? launch_attention<128>(tq, tk, tv, a, batch, max_q_len, st)
                         : launch_attention<64>(tq, tk, tv, a, batch, max_q_len, st);
}

extern "C" int msl_attention_fp8(const void* q8, const void* k_cache, const void* v_cache, const int* page_table,
                                 int max_pages, const int* seq_lens, const int* cu_seqlens_q, const float* k_scale,
                                 const float* v_scale, float softmax_scale, int batch, int max_q_len, int tokens,
                                 int hq, int hkv, int head_dim, int page_size, int window, int64_t cache_rows,
                                 void* out, int64_t ld_out, const void* gate, int64_t ld_gate, int* status,
                                 void* stream) {
  return attention_entry(q8, k_cache, v_cache, page_table, max_pages, seq_lens, cu_seqlens_q, k_scale, v_scale,
                         softmax_scale, batch, max_q_len, tokens, hq, hkv, head_dim, page_size, window, cache_rows,
                         out, ld_out, gate, ld_gate, 1, nullptr, status, stream);
}

extern "C" int msl_attention_split_plan(int batch, int max_q_len, int hq, int hkv, int max_pages, int page_size,
                                        int window) {
  if (batch <= 0 || max_q_len <= 0 || hq <= 0 || hkv <= 0 || hq % hkv || max_pages <= 0 || page_size <= 0) return 1;
  const int G = hq / hkv;
  if (G > 128) return 1;
  const int tq2 = 2 * (kAM / G);
  const int64_t ctas = static_cast<int64_t>((max_q_len + tq2 - 1) / tq2) * hkv * batch;
  // key tiles a CTA may have to walk, from the sizes alone (the lengths live on the device)
  int64_t keys = static_cast<int64_t>(max_pages) * page_size;
  if (window > 0) keys = std::min<int64_t>(keys, window + tq2);
  const int64_t tiles = (keys + kAN - 1) / kAN;
  const int sms = sm_count();
  if (ctas >= 2 * sms || tiles < 16) return 1;             // enough CTAs, or too little work to slice
  // One CTA runs per SM at a time, so the slices run in waves: take the number of slices (at most 16, at
  // least eight key tiles each) whose waves x tiles per slice is smallest; two tiles stand for a CTA's fixed
  // cost, and a slice more has to save 2 % to be taken (its partial results are merged afterwards).
  const int64_t most = std::max<int64_t>(1, std::min<int64_t>(tiles / 8, 16));
  int best = 1;
  double best_cost = 0.0;
  for (int64_t k = 1; k <= most; ++k) {
    const int64_t waves = (ctas * k + sms - 1) / sms;
    const double cost = static_cast<double>(waves) * static_cast<double>((tiles + k - 1) / k + 2);
    if (k == 1 || cost < 0.98 * best_cost) {
      best = static_cast<int>(k);
      best_cost = cost;
    }
  }
  return best;
}

extern "C" int64_t msl_attention_split_workspace(int kv_splits, int tokens, int hq, int head_dim) {
  if (kv_splits <= 1) return 0;
  return static_cast<int64_t>(kv_splits) * tokens * hq * (head_dim + 2) * 4;
}

extern "C" int msl_attention_fp8_split(const void* q8, const void* k_cache, const void* v_cache,
                                       const int* page_table, int max_pages, const int* seq_lens,
                                       const int* cu_seqlens_q, const float* k_scale, const float* v_scale,
                                       float softmax_scale, int batch, int max_q_len, int tokens, int hq, int hkv,
                                       int head_dim, int page_size, int window, int64_t cache_rows, void* out,
                                       int64_t ld_out, const void* gate, int64_t ld_gate, int kv_splits,
                                       void* workspace, int* status, void* stream) {
  return attention_entry(q8, k_cache, v_cache, page_table, max_pages, seq_lens, cu_seqlens_q, k_scale, v_scale,
                         softmax_scale, batch, max_q_len, tokens, hq, hkv, head_dim, page_size, window, cache_rows,
                         out, ld_out, gate, ld_gate, kv_splits, workspace, status, stream);
}

#ifdef MSL_ATTN_PROF
extern "C" int msl_debug_attn_prof(unsigned long long* out, int reset) {
  if (cudaMemcpyFromSymbol(out, msl::g_attn_prof, sizeof(msl::g_attn_prof)) != cudaSuccess) return MSL_ERR_CUDA;
  if (reset) {
    unsigned long long zero[32] = {};
    if (cudaMemcpyToSymbol(msl::g_attn_prof, zero, sizeof(zero)) != cudaSuccess) return MSL_ERR_CUDA;
  }
  return MSL_OK;
}
#endif
