// Causal varlen attention over a paged FP8 (E4M3) K/V cache on tcgen05, GQA-packed.
//
// Replaces the reference layer's attention stage: the gather + sm_90a wgmma kernel + split-KV
// merge (muse_prefill_layer/submission.py:160-447,570-697), the library fallback for sliding
// windows (:712-721) and the per-head output norm and gate (:789-802); the arithmetic follows
// reference.py:376-409.
//
// One CTA per (request, KV head, block of 128/G query tokens), G = query heads per KV head: the
// 128 MMA rows are (token, head-in-group) pairs, so one K/V tile serves all G heads.
//   warps 0-3  softmax + correction + epilogue, one thread per row (TMEM lane = row)
//   warp  4    TMEM allocation, tcgen05.mma issue (FP8 operands, fp32 accumulate)
//   warps 5-8  K/V loaders: one thread per key of the 128-key tile; the key's cache row is found
//              through the page table and copied, 16 bytes at a time, into the swizzled tile
// Per 128-key tile: S = Q K^T (TMEM, 128 columns) -> row softmax in the exp2 domain -> P as E4M3
// scaled by 2^8 into shared memory -> O += P V (TMEM, D columns, V consumed N-major straight from
// its [key][d] tile).  O is rescaled in TMEM only when a row's running maximum moved.  The Q tile
// arrives by one TMA load.  Two CTAs share an SM (TMEM 2 x (128 + D) columns), so one CTA's
// softmax overlaps the other's MMAs.  Every wait is bounded.
#include "msl_common.cuh"
#include "msl_host.h"

namespace msl {

constexpr int kAM = 128;    // rows per CTA
constexpr int kAN = 128;    // keys per tile

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
};

template <int D>
struct AttnSmem {
  static constexpr int kQ = 0;
  static constexpr int kTile = kAN * D;                    // bytes of one K or V tile
  static constexpr int kK = kAM * D;                       // after Q
  static constexpr int kV = kK + 2 * kTile;
  static constexpr int kP = kV + 2 * kTile;                // 128 x 128 bytes
  static constexpr int kBar = kP + kAM * kAN;
  // q_full, kv_full[2], kv_empty[2], s_full, p_full, pv_done
  static constexpr int kTotal = kBar + 8 * 8 + 16;
};

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile with ROWB-byte rows (64 or 128) laid
// out with the matching swizzle: the chunk index is XORed with bits of the row index so that the
// pattern repeats every 1024 bytes (128-byte rows: row mod 8; 64-byte rows: (row / 2) mod 4).
template <int ROWB>
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk) {
  if constexpr (ROWB == 128) return row * 128u + ((chunk ^ (row & 7u)) << 4);
  else return row * 64u + ((chunk ^ ((row >> 1) & 3u)) << 4);
}

template <int D>
__global__ void __launch_bounds__(288, 2)
attention_fp8_kernel(const __grid_constant__ CUtensorMap tm_q, AttnArgs p) {
  using S = AttnSmem<D>;
  constexpr uint32_t kSwz = (D == 128) ? 2u : 4u;          // descriptor swizzle code
  constexpr uint32_t kSbo = 8 * D;                         // bytes between 8-row groups
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBar);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 3;
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* pv_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.hq / p.hkv;
  const int TQ = kAM / G;                                  // query tokens per CTA
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int q_begin = p.cu_seqlens_q[b], q_len = p.cu_seqlens_q[b + 1] - q_begin;
  // Longest key ranges first: later query blocks attend to more keys.
  const int n_qblk = (q_len + TQ - 1) / TQ;
  const int qblk = n_qblk - 1 - static_cast<int>(blockIdx.x);
  if (qblk < 0) return;                                    // uniform for the CTA, before any barrier
  const int q0 = qblk * TQ;
  const int seq = p.seq_lens[b];
  const int rows_valid = min(TQ, q_len - q0) * G;
  const int max_qpos = seq + min(q0 + TQ, q_len) - 1;
  const int min_qpos = seq + q0;
  const int kt_end = max_qpos / kAN + 1;
  const int kt_begin = p.window ? max(0, min_qpos - p.window + 1) / kAN : 0;
  const int n_tiles = kt_end - kt_begin;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 4); mbar_init(&kv_empty[i], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) tmem_alloc(tmem_slot, 256);               // S: columns [0,128), O: [128, 128 + D)
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      mbar_expect_tx(q_full, kAM * D);
      tma_load_3d(smem + S::kQ, &tm_q, q_full, 0, kvh * G, q_begin + q0);
      constexpr uint32_t idesc_qk = make_idesc(0, 0, kAM, kAN);
      constexpr uint32_t idesc_pv = make_idesc(0, 0, kAM, D, 0, 1);     // B = V, N-major
      bool ok = mbar_wait(q_full, 0);
      const uint32_t sq = smem_u32(smem + S::kQ), sp = smem_u32(smem + S::kP);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int buf = j & 1;
        const uint32_t kv_ph = (j >> 1) & 1, ph = j & 1;
        if (*abort_flag || !mbar_wait(&kv_full[buf], kv_ph)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + S::kK + buf * S::kTile);
        const uint32_t sv = smem_u32(smem + S::kV + buf * S::kTile);
#pragma unroll
        for (int k = 0; k < D / 32; ++k)
          tc_mma_f8(tmem_s, make_sdesc(sq + k * 32, 16, kSbo, kSwz), make_sdesc(sk + k * 32, 16, kSbo, kSwz),
                    idesc_qk, k != 0);
        tc_commit(s_full);
        if (*abort_flag || !mbar_wait(p_full, ph)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kAN / 32; ++k)
          tc_mma_f8(tmem_o, make_sdesc(sp + k * 32, 16, 1024, 2), make_sdesc(sv + k * 32 * D, 16, kSbo, kSwz),
                    idesc_pv, (j | k) != 0);
        tc_commit(&kv_empty[buf]);
        tc_commit(pv_done);
      }
      if (!ok) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
    }
  } else if (warp >= 5) {
    // ------------------------------------------------------------------ K/V loaders
    const int r = threadIdx.x - 5 * 32;                    // key row of the tile
    const int* pt = p.page_table + static_cast<int64_t>(b) * p.max_pages;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int buf = j & 1;
      const uint32_t kv_ph = (j >> 1) & 1;
      const int key = (kt_begin + j) * kAN + r;
      int64_t row = -1;
      if (key <= max_qpos) {
        const int pg = pt[key / p.page_size];
        if (pg >= 0) row = static_cast<int64_t>(pg) * p.page_size + key % p.page_size;
        if (row >= p.cache_rows) row = -1;
      }
      uint4 kq[D / 16], vq[D / 16];
      if (row >= 0) {
        const uint4* ks = reinterpret_cast<const uint4*>(p.k_cache + (row * p.hkv + kvh) * D);
        const uint4* vs = reinterpret_cast<const uint4*>(p.v_cache + (row * p.hkv + kvh) * D);
#pragma unroll
        for (int c = 0; c < D / 16; ++c) { kq[c] = ks[c]; vq[c] = vs[c]; }
      } else {
#pragma unroll
        for (int c = 0; c < D / 16; ++c) { kq[c] = make_uint4(0, 0, 0, 0); vq[c] = make_uint4(0, 0, 0, 0); }
      }
      if (*abort_flag || !mbar_wait(&kv_empty[buf], kv_ph ^ 1)) { ok = false; break; }
      uint8_t* sk = smem + S::kK + buf * S::kTile;
      uint8_t* sv = smem + S::kV + buf * S::kTile;
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        *reinterpret_cast<uint4*>(sk + swz<D>(r, c)) = kq[c];
        *reinterpret_cast<uint4*>(sv + swz<D>(r, c)) = vq[c];
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&kv_full[buf]);
    }
    if (!ok && lane == 0) { *abort_flag = 1; report_error(p.status, MSL_ERR_DEVICE_TIMEOUT); }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int r = warp * 32 + lane;                        // row = TMEM lane
    const int tq = r / G, g = r - tq * G;
    const bool row_valid = r < rows_valid;
    const int qpos = seq + min(q0 + tq, q_len - 1);
    const float scale_log2 = p.softmax_scale * (*p.k_scale) * 1.4426950408889634f;
    const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    uint8_t* sp = smem + S::kP;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const uint32_t ph = j & 1;
      const int key0 = (kt_begin + j) * kAN;
      if (*abort_flag || !mbar_wait(s_full, ph)) { ok = false; break; }
      tc_fence_after();
      const bool full_tile = (key0 + kAN - 1 <= min_qpos) && (!p.window || key0 > max_qpos - p.window);
      const int lo_key = p.window ? qpos - p.window : -1;   // visible keys: lo_key < key <= qpos
      // pass 1: row maximum
      float m_tile = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kAN; c += 32) {
        uint32_t s[32];
        tmem_ld32(tmem_s + lane_sel + c, s);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = key0 + c + i;
          const bool vis = full_tile || (key <= qpos && key > lo_key);
          if (vis) m_tile = fmaxf(m_tile, __uint_as_float(s[i]));
        }
      }
      const float m_new = fmaxf(m_run, m_tile * scale_log2);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = exp2f(m_run - m_use);               // 0 when m_run = -inf
      m_run = m_new;
      // The previous tile's P V must have finished before O is rescaled or P overwritten.
      if (j > 0) {
        if (*abort_flag || !mbar_wait(pv_done, (j - 1) & 1)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t o[32];
            tmem_ld32(tmem_o + lane_sel + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                ::"r"(tmem_o + lane_sel + c), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]),
                "r"(o[6]), "r"(o[7]), "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]),
                "r"(o[14]), "r"(o[15]), "r"(o[16]), "r"(o[17]), "r"(o[18]), "r"(o[19]), "r"(o[20]), "r"(o[21]),
                "r"(o[22]), "r"(o[23]), "r"(o[24]), "r"(o[25]), "r"(o[26]), "r"(o[27]), "r"(o[28]), "r"(o[29]),
                "r"(o[30]), "r"(o[31])
                : "memory");
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      l_run *= corr;
      // pass 2: P = exp2(s - m) as E4M3 scaled by 2^8, row sum in fp32
      float l_tile = 0.f;
#pragma unroll 1
      for (int c = 0; c < kAN; c += 32) {
        uint32_t s[32];
        tmem_ld32(tmem_s + lane_sel + c, s);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = key0 + c + i;
          const bool vis = full_tile || (key <= qpos && key > lo_key);
          const float e = vis ? exp2f(__uint_as_float(s[i]) * scale_log2 - m_use) : 0.f;
          l_tile += e;
          pv[i] = e * 256.0f;
        }
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint4 packed = make_uint4(
              __nv_cvt_float2_to_fp8x2(make_float2(pv[16 * q + 0], pv[16 * q + 1]), __NV_SATFINITE, __NV_E4M3) |
                  (__nv_cvt_float2_to_fp8x2(make_float2(pv[16 * q + 2], pv[16 * q + 3]), __NV_SATFINITE, __NV_E4M3) << 16),
              __nv_cvt_float2_to_fp8x2(make_float2(pv[16 * q + 4], pv[16 * q + 5]), __NV_SATFINITE, __NV_E4M3) |
                  (__nv_cvt_float2_to_fp8x2(make_float2(pv[16 * q + 6], pv[16 * q + 7]), __NV_SATFINITE, __NV_E4M3) << 16),
              __nv_cvt_float2_to_fp8x2(make_float2(pv[16 * q + 8], pv[16 * q + 9]), __NV_SATFINITE, __NV_E4M3) |
                  (__nv_cvt_float2_to_fp8x2(make_float2(pv[16 * q + 10], pv[16 * q + 11]), __NV_SATFINITE, __NV_E4M3) << 16),
              __nv_cvt_float2_to_fp8x2(make_float2(pv[16 * q + 12], pv[16 * q + 13]), __NV_SATFINITE, __NV_E4M3) |
                  (__nv_cvt_float2_to_fp8x2(make_float2(pv[16 * q + 14], pv[16 * q + 15]), __NV_SATFINITE, __NV_E4M3) << 16));
          *reinterpret_cast<uint4*>(sp + swz<128>(r, c / 16 + q)) = packed;
        }
      }
      l_run += l_tile;
      tc_fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---------------------------------------------------------------- epilogue
    if (ok && n_tiles > 0) {
      if (*abort_flag || !mbar_wait(pv_done, (n_tiles - 1) & 1)) ok = false;
    }
    if (ok && n_tiles > 0) {
      tc_fence_after();
      const float c_out = (*p.v_scale) / (256.0f * l_run);
      float r_norm = 1.0f;
      if (p.gate != nullptr) {
        float ss = 0.f;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld32(tmem_o + lane_sel + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) { const float v = __uint_as_float(o[i]) * c_out; ss += v * v; }
        }
        r_norm = 1.0f / sqrtf(ss / D + 1e-5f);
      }
      const int token = q_begin + q0 + tq;
      const int head = kvh * G + g;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(token) * p.ld_out + head * D;
      const __nv_bfloat16* grow = p.gate ? p.gate + static_cast<int64_t>(token) * p.ld_gate + head * D : nullptr;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld32(tmem_o + lane_sel + c, o);
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

  if (warp == 4 && lane == 0 && *abort_flag) drain_pause();
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tmem_base, 256);
  }
}

template <int D>
static int launch_attention(const CUtensorMap& tq, const AttnArgs& a, int batch, int max_q_len, cudaStream_t st) {
  using S = AttnSmem<D>;
  const int smem = S::kTotal + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_fp8_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess)
      return MSL_ERR_CUDA;
    configured = true;
  }
  const int G = a.hq / a.hkv, TQ = kAM / G;
  dim3 grid((max_q_len + TQ - 1) / TQ, a.hkv, batch);
  attention_fp8_kernel<D><<<grid, 288, smem, st>>>(tq, a);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

}  // namespace msl

using namespace msl;

extern "C" int msl_attention_fp8(const void* q8, const void* k_cache, const void* v_cache, const int* page_table,
                                 int max_pages, const int* seq_lens, const int* cu_seqlens_q, const float* k_scale,
                                 const float* v_scale, float softmax_scale, int batch, int max_q_len, int tokens,
                                 int hq, int hkv, int head_dim, int page_size, int window, int64_t cache_rows,
                                 void* out, int64_t ld_out, const void* gate, int64_t ld_gate, int* status,
                                 void* stream) {
  if (!q8 || !k_cache || !v_cache || !page_table || !seq_lens || !cu_seqlens_q || !k_scale || !v_scale || !out)
    return MSL_ERR_ARG;
  if (batch <= 0 || max_q_len <= 0 || tokens <= 0 || hq <= 0 || hkv <= 0 || hq % hkv || page_size <= 0 ||
      window < 0 || max_pages <= 0)
    return MSL_ERR_ARG;
  const int G = hq / hkv;
  if (G > 128 || (G & (G - 1))) return MSL_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(q8) & 15) || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (ld_out & 7) ||
      (gate && ((reinterpret_cast<uintptr_t>(gate) & 15) || (ld_gate & 7))))
    return MSL_ERR_ALIGN;
  AttnArgs a{static_cast<const uint8_t*>(k_cache), static_cast<const uint8_t*>(v_cache), page_table, max_pages,
             seq_lens, cu_seqlens_q, k_scale, v_scale, softmax_scale, hq, hkv, page_size, window, cache_rows, out,
             ld_out, static_cast<const __nv_bfloat16*>(gate), ld_gate, status};
  CUtensorMap tq;
  const uint32_t box_t = static_cast<uint32_t>(kAM / G);
  int rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 128) {
    rc = make_tmap_3d(&tq, q8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 128, hq, tokens, 128, static_cast<uint64_t>(hq) * 128,
                      128, G, box_t, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    return launch_attention<128>(tq, a, batch, max_q_len, st);
  }
  if (head_dim == 64) {
    rc = make_tmap_3d(&tq, q8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 64, hq, tokens, 64, static_cast<uint64_t>(hq) * 64, 64,
                      G, box_t, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    return launch_attention<64>(tq, a, batch, max_q_len, st);
  }
  return MSL_ERR_UNSUPPORTED;
}
