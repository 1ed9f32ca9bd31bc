// The bandwidth-bound kernels of the layer: QK-norm + RoPE + FP8 quantise + paged cache store,
// the two residual boundaries, the router's top-k with slot assignment, token dispatch and the
// weighted combine.  All use 128-bit global accesses and keep a row in registers so each tensor
// crosses HBM once.
#include <atomic>
#include <mutex>

#include "msl_common.cuh"
#include "msl_host.h"

namespace msl {

__device__ __forceinline__ void unpack8(const uint4& q, float (&v)[8]) {
  v[0] = bf16_bits_to_f32(q.x & 0xffffu); v[1] = bf16_bits_to_f32(q.x >> 16);
  v[2] = bf16_bits_to_f32(q.y & 0xffffu); v[3] = bf16_bits_to_f32(q.y >> 16);
  v[4] = bf16_bits_to_f32(q.z & 0xffffu); v[5] = bf16_bits_to_f32(q.z >> 16);
  v[6] = bf16_bits_to_f32(q.w & 0xffffu); v[7] = bf16_bits_to_f32(q.w >> 16);
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  return make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                    pack_bf16x2(v[6], v[7]));
}
__device__ __forceinline__ uint32_t fp8x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// Sum over all threads of a block; `scratch` holds one float per warp (+1).  Every thread
// receives the total.  `n` values are reduced at once.
template <int N>
__device__ __forceinline__ void block_sum(float (&v)[N], float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = warp_sum(v[i]);
  __syncthreads();   // scratch may still be read from a previous use
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) scratch[warp * N + i] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float s = 0.f;
    for (int w = 0; w < nwarp; ++w) s += scratch[w * N + i];
    v[i] = s;
  }
}

// ============================================================================ QK-norm + RoPE + FP8 + cache store
// Block (x, y): tokens [kRopeTok x, +kRopeTok), lanes [256 y, +256) of the token's (HQ + 2 HKV) D / 8
// lanes; one group of D/8 lanes per head, each lane owning 8 consecutive channels of that head for every
// token of the block (one 16-byte load and one 8-byte store per token, the loads of all tokens issued
// before any arithmetic).  Heads 0..HQ-1 are queries, the next HKV keys, the next
// HKV values (the row layout of the QKV+gate projection; the gate columns after them are not read).
// A token's D/2 rotation angles are evaluated once per block (not once per head) while the loads are in
// flight, and shared through shared memory.
#ifndef MSL_ROPE_TOK
#define MSL_ROPE_TOK 2
#endif
constexpr int kRopeTok = MSL_ROPE_TOK;

template <int D>
__global__ void __launch_bounds__(256, 6)
qk_rope_store_kernel(const __nv_bfloat16* __restrict__ qkv, int64_t ld, const int64_t* __restrict__ positions,
                     const int64_t* __restrict__ cache_loc, const float* __restrict__ inv_freq,
                     const float* __restrict__ k_scale_p, const float* __restrict__ v_scale_p,
                     uint8_t* __restrict__ q8, uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache,
                     int tokens, int hq, int hkv, int64_t cache_rows, int* status) {
  constexpr int LPH = D / 8;   // lanes per head
  __shared__ float2 rot[kRopeTok][D / 2];                   // (cos, sin) of position * inv_freq[j]
  const int nh = hq + 2 * hkv;
  const int lanes = nh * LPH;
  const int t0 = blockIdx.x * kRopeTok;
  const int nt = min(kRopeTok, tokens - t0);
  uint4 raw[kRopeTok];
  auto fetch = [&](int idx) {
#pragma unroll
    for (int tt = 0; tt < kRopeTok; ++tt)
      raw[tt] = (idx < lanes && tt < nt)
                    ? *reinterpret_cast<const uint4*>(qkv + (t0 + tt) * ld + (idx / LPH) * D + (idx % LPH) * 8)
                    : make_uint4(0, 0, 0, 0);
  };
  const int idx = blockIdx.y * blockDim.x + threadIdx.x;
  fetch(idx);
  if (inv_freq != nullptr) {
    if (threadIdx.x < kRopeTok * (D / 2)) {
      const int tt = threadIdx.x / (D / 2), j = threadIdx.x % (D / 2);
      if (tt < nt) {
        const float ang = static_cast<float>(positions[t0 + tt]) * inv_freq[j];
        float sn, cs;
        sincosf(ang, &sn, &cs);
        rot[tt][j] = make_float2(cs, sn);
      }
    }
    __syncthreads();
  }
  const float k_scale = *k_scale_p, v_scale = *v_scale_p;
  {
    const bool live = idx < lanes;
    const int h = live ? idx / LPH : 0;
    const int sub = idx % LPH;
    const bool is_v = h >= hq + hkv;
#pragma unroll
    for (int tt = 0; tt < kRopeTok; ++tt) {
      float v[8];
      unpack8(raw[tt], v);
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
#pragma unroll
      for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (!live || tt >= nt) continue;
      const int t = t0 + tt;
      if (!is_v) {
        const float r = 1.0f / sqrtf(ss / D + 1e-5f);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= r;
        if (inv_freq != nullptr) {
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            const float2 cs = rot[tt][sub * 4 + i / 2];
            const float e = v[i], o = v[i + 1];
            v[i] = e * cs.x - o * cs.y;
            v[i + 1] = e * cs.y + o * cs.x;
          }
        }
      }
      uint8_t* dst;
      if (h < hq) {
        dst = q8 + (static_cast<int64_t>(t) * hq + h) * D + sub * 8;
      } else {
        const int64_t row = cache_loc[t];
        if (row < 0 || row >= cache_rows) {
          report_error(status, MSL_ERR_CAPACITY);
          continue;
        }
        const float scale = is_v ? v_scale : k_scale;
        // x / scale as the reference divides (reference.py:181-182); a reciprocal multiply would
        // round differently when the scale is not a power of two.
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = v[i] / scale;
        const int kvh = is_v ? h - hq - hkv : h - hq;
        dst = (is_v ? v_cache : k_cache) + (row * hkv + kvh) * D + sub * 8;
      }
      *reinterpret_cast<uint2*>(dst) = make_uint2(fp8x4(v[0], v[1], v[2], v[3]), fp8x4(v[4], v[5], v[6], v[7]));
    }
  }
}

// ============================================================================ residual boundary
// branch' = branch * branch_scale (optional); s_out = alpha * s_in + beta * rms(branch', eps_branch);
// h_out = rms(s_out, eps_out) * norm_w.  One block per token row; the row stays in registers.
template <int MAXC, int THREADS>
__global__ void __launch_bounds__(THREADS, (THREADS == 256 && MAXC <= 2) ? 5 : 1)
boundary_kernel(const __nv_bfloat16* __restrict__ branch, int64_t ld_branch, const float* __restrict__ branch_scale,
                const float* __restrict__ s_in, const float* __restrict__ alpha, const float* __restrict__ beta,
                const float* __restrict__ norm_w, float* __restrict__ s_out, __nv_bfloat16* __restrict__ h_out,
                int64_t ld_h, int hidden, float eps_branch, float eps_out) {
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;
  const int chunks = hidden / 8;
  float b[MAXC][8], s[MAXC][8];
  float ss[1] = {0.f};
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < chunks) {
      unpack8(*reinterpret_cast<const uint4*>(branch + row * ld_branch + ch * 8), b[c]);
      if (branch_scale != nullptr) {
        const float4 w0 = *reinterpret_cast<const float4*>(branch_scale + ch * 8);
        const float4 w1 = *reinterpret_cast<const float4*>(branch_scale + ch * 8 + 4);
        b[c][0] *= w0.x; b[c][1] *= w0.y; b[c][2] *= w0.z; b[c][3] *= w0.w;
        b[c][4] *= w1.x; b[c][5] *= w1.y; b[c][6] *= w1.z; b[c][7] *= w1.w;
      }
      const float4 s0 = *reinterpret_cast<const float4*>(s_in + row * hidden + ch * 8);
      const float4 s1 = *reinterpret_cast<const float4*>(s_in + row * hidden + ch * 8 + 4);
      s[c][0] = s0.x; s[c][1] = s0.y; s[c][2] = s0.z; s[c][3] = s0.w;
      s[c][4] = s1.x; s[c][5] = s1.y; s[c][6] = s1.z; s[c][7] = s1.w;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss[0] += b[c][i] * b[c][i];
    }
  }
  block_sum<1>(ss, scratch);
  const float rb = 1.0f / sqrtf(ss[0] / hidden + eps_branch);
  float s2[1] = {0.f};
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < chunks) {
      const float4 a0 = *reinterpret_cast<const float4*>(alpha + ch * 8);
      const float4 a1 = *reinterpret_cast<const float4*>(alpha + ch * 8 + 4);
      const float4 b0 = *reinterpret_cast<const float4*>(beta + ch * 8);
      const float4 b1 = *reinterpret_cast<const float4*>(beta + ch * 8 + 4);
      const float al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float be[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s[c][i] = al[i] * s[c][i] + be[i] * (b[c][i] * rb);
        s2[0] += s[c][i] * s[c][i];
      }
      float* dst = s_out + row * hidden + ch * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(s[c][0], s[c][1], s[c][2], s[c][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(s[c][4], s[c][5], s[c][6], s[c][7]);
    }
  }
  block_sum<1>(s2, scratch);
  const float rs = 1.0f / sqrtf(s2[0] / hidden + eps_out);
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < chunks) {
      const float4 w0 = *reinterpret_cast<const float4*>(norm_w + ch * 8);
      const float4 w1 = *reinterpret_cast<const float4*>(norm_w + ch * 8 + 4);
      const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = s[c][i] * rs * w[i];
      *reinterpret_cast<uint4*>(h_out + row * ld_h + ch * 8) = pack8(o);
    }
  }
}

// ============================================================================ router top-k + slots
// One warp per token.  score = sigmoid(multiplier * logit) in fp64 rounded to fp32 (the reference
// forms the logits and the sigmoid in fp64, reference.py:422-423); biased = score + bias chooses,
// lowest index winning exact ties; weights = score / (sum of picked + 1e-15).  Routes to experts
// [local_start, local_start + n_local) (modulo n_experts) get a slot from a per-expert counter:
// a shared-memory histogram per block, then one global atomic per (block, expert).
struct RouteArgs {
  const float* logits;
  int64_t ld;
  int hilo;
  const float* bias;
  float multiplier;
  const int* local_start;
  int tokens, n_experts, top_k, n_local;
  int* ids;
  float* weights;
  int* local_ids;
  int* slots;
  int* counts;
};

// Routes the tokens [group * warps, (group + 1) * warps) of one block (one warp per token).  hist:
// shared memory, [n_local] counts then [n_local] global bases.  Called by every thread of the block.
template <int MAXPL>   // experts per lane, n_experts <= 32 * MAXPL
__device__ __forceinline__ void route_group(const RouteArgs& a, int group, int* hist) {
  const float* __restrict__ logits = a.logits;
  const float* __restrict__ bias = a.bias;
  const int64_t ld = a.ld;
  const int hilo = a.hilo, tokens = a.tokens, n_experts = a.n_experts, top_k = a.top_k, n_local = a.n_local;
  const float multiplier = a.multiplier;
  const int* local_start_p = a.local_start;
  int* __restrict__ ids = a.ids;
  float* __restrict__ weights = a.weights;
  int* __restrict__ local_ids = a.local_ids;
  int* __restrict__ slots = a.slots;
  int* __restrict__ counts = a.counts;
  int* base = hist + n_local;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = group * (blockDim.x >> 5) + warp;
  __syncthreads();                       // the previous group's bases have been read
  for (int i = threadIdx.x; i < n_local; i += blockDim.x) hist[i] = 0;
  __syncthreads();

  float score[MAXPL], biased[MAXPL];
  int my_e = -1, my_rank = 0;           // lane j < top_k owns route j
  float my_w = 0.f;
  int my_id = 0;
  if (t < tokens) {
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      const int e = lane + 32 * i;
      if (e < n_experts) {
        float x = logits[t * ld + e];
        if (hilo) x += logits[t * ld + n_experts + e];
        const double z = static_cast<double>(x) * static_cast<double>(multiplier);
        score[i] = static_cast<float>(1.0 / (1.0 + exp(-z)));
        biased[i] = score[i] + bias[e];
      } else {
        score[i] = 0.f;
        biased[i] = -INFINITY;
      }
    }
    float sum = 0.f;
    const int ls = *local_start_p;
    for (int j = 0; j < top_k; ++j) {
      float best = -INFINITY;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < MAXPL; ++i) {
        const int e = lane + 32 * i;
        if (biased[i] > best) { best = biased[i]; best_e = e; }   // ascending e: first hit is the lowest index
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      // the owner removes the winner and broadcasts its unbiased score
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < MAXPL; ++i) {
        if (lane + 32 * i == best_e) { sc = score[i]; biased[i] = -INFINITY; }
      }
      sc = __shfl_sync(0xffffffffu, sc, best_e & 31);
      sum += sc;
      if (lane == j) { my_id = best_e; my_w = sc; }
    }
    if (lane < top_k) {
      my_w = my_w / (sum + 1e-15f);
      int le = (my_id - ls) % n_experts;
      if (le < 0) le += n_experts;
      my_e = le < n_local ? le : -1;
      if (my_e >= 0) my_rank = atomicAdd(&hist[my_e], 1);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_local; i += blockDim.x) base[i] = hist[i] ? atomicAdd(&counts[i], hist[i]) : 0;
  __syncthreads();
  if (t < tokens && lane < top_k) {
    const int64_t o = static_cast<int64_t>(t) * top_k + lane;
    ids[o] = my_id;
    weights[o] = my_w;
    local_ids[o] = my_e;
    slots[o] = my_e >= 0 ? base[my_e] + my_rank : -1;
  }
}

template <int MAXPL>
__global__ void __launch_bounds__(256) route_topk_kernel(RouteArgs a) {
  extern __shared__ int hist[];
  route_group<MAXPL>(a, blockIdx.x, hist);
}

// ============================================================================ dispatch
// Copies each token's row to one slab row per local route: row = offset[expert] + slot, offsets
// being the exclusive prefix sum of the per-expert counts (recomputed per block; block 0 also
// publishes it for the grouped GEMM).  With norm_w the row is RMS-normalised (eps 1e-5) and
// scaled first (the pooled layer's pre-expert norm, submission.py:890-899).
struct DispatchArgs {
  const __nv_bfloat16* x;
  int64_t ldx;
  const float* norm_w;
  const int* local_ids;
  const int* slots;
  const int* counts;
  int n_local, top_k, width;
  __nv_bfloat16* slab;
  int64_t slab_rows;
  int* rowmap;
  int* offsets_out;
  int* status;
};

// Exclusive prefix sum of counts[n_local] into offs[n_local + 1] (shared memory) by the block's first warp.
// The counters (and, in dispatch_token, the per-route expert/slot arrays) may have been written earlier in
// the same launch by other blocks: they are read with L2-only loads.
__device__ __forceinline__ void scan_counts(const int* counts, int n_local, int* offs) {
  if (threadIdx.x < 32) {
    // exclusive scan by one warp, n_local <= 1024
    int carry = 0;
    for (int b0 = 0; b0 < n_local; b0 += 32) {
      const int i = b0 + threadIdx.x;
      const int c = i < n_local ? __ldcg(counts + i) : 0;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (threadIdx.x >= o) inc += n;
      }
      if (i < n_local) offs[i] = carry + inc - c;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (threadIdx.x == 0) offs[n_local] = carry;
  }
  __syncthreads();
}

// Copies token t's row to the slab rows of its local routes.  Called by every thread of the block.
__device__ __forceinline__ void dispatch_token(const DispatchArgs& a, int t, const int* offs, float* scratch) {
  const __nv_bfloat16* __restrict__ x = a.x;
  const float* __restrict__ norm_w = a.norm_w;
  const int* local_ids = a.local_ids;
  const int* slots = a.slots;
  __nv_bfloat16* __restrict__ slab = a.slab;
  int* __restrict__ rowmap = a.rowmap;
  const int64_t ldx = a.ldx, slab_rows = a.slab_rows;
  const int top_k = a.top_k, width = a.width;
  int* status = a.status;
  const int chunks = width / 8;
  float ss[1] = {0.f};
  if (norm_w != nullptr) {
    for (int ch = threadIdx.x; ch < chunks; ch += blockDim.x) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(x + t * ldx + ch * 8), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss[0] += v[i] * v[i];
    }
    block_sum<1>(ss, scratch);
  }
  const float r = norm_w != nullptr ? 1.0f / sqrtf(ss[0] / width + 1e-5f) : 1.0f;
  int rows[16];
  int nr = 0;
  for (int j = 0; j < top_k && j < 16; ++j) {
    const int le = __ldcg(local_ids + t * top_k + j);
    int row = -1;
    if (le >= 0) {
      row = offs[le] + __ldcg(slots + t * top_k + j);
      if (row >= slab_rows) {
        if (threadIdx.x == 0) report_error(status, MSL_ERR_CAPACITY);
        row = -1;
      }
    }
    if (threadIdx.x == 0) rowmap[t * top_k + j] = row;
    if (row >= 0) rows[nr++] = row;
  }
  if (nr == 0) return;
  for (int ch = threadIdx.x; ch < chunks; ch += blockDim.x) {
    uint4 raw = *reinterpret_cast<const uint4*>(x + t * ldx + ch * 8);
    if (norm_w != nullptr) {
      float v[8];
      unpack8(raw, v);
      const float4 w0 = *reinterpret_cast<const float4*>(norm_w + ch * 8);
      const float4 w1 = *reinterpret_cast<const float4*>(norm_w + ch * 8 + 4);
      v[0] *= r * w0.x; v[1] *= r * w0.y; v[2] *= r * w0.z; v[3] *= r * w0.w;
      v[4] *= r * w1.x; v[5] *= r * w1.y; v[6] *= r * w1.z; v[7] *= r * w1.w;
      raw = pack8(v);
    }
    for (int j = 0; j < nr; ++j)
      *reinterpret_cast<uint4*>(slab + static_cast<int64_t>(rows[j]) * width + ch * 8) = raw;
  }
}

__global__ void __launch_bounds__(256) dispatch_kernel(DispatchArgs a) {
  extern __shared__ int offs[];          // [n_local + 1]
  __shared__ float scratch[32];
  scan_counts(a.counts, a.n_local, offs);
  if (blockIdx.x == 0 && a.offsets_out != nullptr)
    for (int i = threadIdx.x; i <= a.n_local; i += blockDim.x) a.offsets_out[i] = offs[i];
  dispatch_token(a, blockIdx.x, offs, scratch);
}

// Routing, slot assignment and dispatch as ONE launch (the reference runs two kernels,
// submission.py:859-886 and :890-899, after zeroing its counters).  Persistent blocks, launched
// cooperatively so that all of them are resident:
//   phase 1  groups of 8 tokens round-robin over the blocks: top-k, weights, slots (route_group);
//   barrier  over the grid (sync[0] counts arrivals; bounded wait);
//   phase 2  every block forms the offsets from the now final counts, then tokens round-robin over the
//            blocks: each row copied to its routes' slab rows (dispatch_token);
//   cleanup  the last block to finish (sync[1] counts them) zeroes the counters and both sync words, so
//            the next launch needs no memset: `counts` and `sync` are zeroed once by their owner and are
//            zero again whenever this kernel is not running.
template <int MAXPL>
__global__ void __launch_bounds__(256) route_dispatch_kernel(RouteArgs ra, DispatchArgs da, int* sync) {
  extern __shared__ int sh[];            // phase 1: hist + base [2 n_local]; phase 2: offs [n_local + 1]
  __shared__ float scratch[32];
  __shared__ int give_up;
  const int warps = blockDim.x >> 5;
  const int n_groups = (ra.tokens + warps - 1) / warps;
  for (int g = blockIdx.x; g < n_groups; g += gridDim.x) route_group<MAXPL>(ra, g, sh);
  __syncthreads();
  if (threadIdx.x == 0) {
    give_up = 0;
    __threadfence();
    atomicAdd(&sync[0], 1);
    const uint64_t t0 = global_ns();
    for (uint32_t i = 0;; ++i) {
      int seen;
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(sync) : "memory");
      if (seen >= static_cast<int>(gridDim.x)) break;
      if ((i & 255u) == 255u && global_ns() - t0 > kWaitLimitNs) {
        report_error(da.status, MSL_ERR_DEVICE_TIMEOUT);
        give_up = 1;
        break;
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
  if (!give_up) {
    scan_counts(da.counts, da.n_local, sh);
    if (blockIdx.x == 0 && da.offsets_out != nullptr)
      for (int i = threadIdx.x; i <= da.n_local; i += blockDim.x) da.offsets_out[i] = sh[i];
    for (int t = blockIdx.x; t < ra.tokens; t += gridDim.x) {
      dispatch_token(da, t, sh, scratch);
      __syncthreads();                   // scratch is reused by the next token's norm
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    give_up = atomicAdd(&sync[1], 1) == static_cast<int>(gridDim.x) - 1;   // reused: "this block is the last"
  }
  __syncthreads();
  if (give_up) {
    for (int i = threadIdx.x; i < ra.n_local; i += blockDim.x) ra.counts[i] = 0;
    if (threadIdx.x == 0) { sync[0] = 0; sync[1] = 0; }
  }
}

// ============================================================================ K/V row gather / scatter
// dst[dst_idx ? dst_idx[i] : i] = src[src_idx ? src_idx[i] : i] for rows of row_bytes (a multiple of
// 16).  Gathers a chunk's new cache rows into a contiguous send buffer and scatters rows received from
// the ranks that hold the earlier chunks of the same sequence into this rank's paged cache.
// A negative or out-of-range index skips the row (and is reported).
__global__ void __launch_bounds__(256)
kv_rows_copy_kernel(const uint8_t* __restrict__ src, const int64_t* __restrict__ src_idx, int64_t src_rows,
                    uint8_t* __restrict__ dst, const int64_t* __restrict__ dst_idx, int64_t dst_rows, int64_t n,
                    int row_bytes, int* status) {
  const int per_row = row_bytes / 16;
  const int64_t total = n * per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / per_row;
    const int part = static_cast<int>(i - row * per_row);
    const int64_t from = src_idx ? src_idx[row] : row;
    const int64_t to = dst_idx ? dst_idx[row] : row;
    if (from < 0 || from >= src_rows || to < 0 || to >= dst_rows) {
      if (part == 0) report_error(status, MSL_ERR_CAPACITY);
      continue;
    }
    reinterpret_cast<uint4*>(dst + to * row_bytes)[part] = reinterpret_cast<const uint4*>(src + from * row_bytes)[part];
  }
}

// ============================================================================ expert-parallel plan + dispatch
// counts_all[s][e]: routes of rank s to global expert e (all-gathered).  Rank d owns experts
// [d * el, (d + 1) * el); its slab holds row groups ordered (source rank, local expert).  For this
// rank `me`: dest_base[e] = first row, in the owner's slab, of the group (me, e); group_offsets =
// row ranges of this rank's own slab (consumed by the grouped GEMM), clamped to `cap`: a routing that
// would need more than `cap` rows is reported in *status, the groups past the end come out empty (the
// dispatch skips the same rows), and nothing downstream addresses a row at or beyond `cap`.
__global__ void ep_plan_kernel(const int* __restrict__ counts_all, int world, int el, int me, int cap,
                               int* __restrict__ dest_base, int* __restrict__ group_offsets, int* status) {
  const int n_experts = world * el;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    const int d = e / el;
    int base = 0;
    for (int s = 0; s < me; ++s)
      for (int x = d * el; x < (d + 1) * el; ++x) base += counts_all[s * n_experts + x];
    for (int x = d * el; x < e; ++x) base += counts_all[me * n_experts + x];
    dest_base[e] = base;
  }
  if (threadIdx.x == 0) {
    int run = 0;
    for (int s = 0; s < world; ++s)
      for (int le = 0; le < el; ++le) {
        group_offsets[s * el + le] = min(run, cap);
        run += counts_all[s * n_experts + me * el + le];
      }
    group_offsets[world * el] = min(run, cap);
    if (run > cap) report_error(status, MSL_ERR_CAPACITY);
  }
}

// Token dispatch straight into the expert-owning ranks' slabs (peer_bases[d], NVLink stores): the
// dispatch all-to-all of expert parallelism fused into the dispatch kernel.  rowmap receives
// d * cap + row.
__global__ void __launch_bounds__(256)
dispatch_peer_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const float* __restrict__ norm_w,
                     const int* __restrict__ ids, const int* __restrict__ slots, const int* __restrict__ dest_base,
                     __nv_bfloat16* const* __restrict__ peer_bases, int el, int cap, int top_k, int width,
                     int* __restrict__ rowmap) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int chunks = width / 8;
  float ss[1] = {0.f};
  if (norm_w != nullptr) {
    for (int ch = threadIdx.x; ch < chunks; ch += blockDim.x) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(x + t * ldx + ch * 8), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss[0] += v[i] * v[i];
    }
    block_sum<1>(ss, scratch);
  }
  const float r = norm_w != nullptr ? 1.0f / sqrtf(ss[0] / width + 1e-5f) : 1.0f;
  __nv_bfloat16* dst[16];
  int nr = 0;
  for (int j = 0; j < top_k && j < 16; ++j) {
    const int e = ids[t * top_k + j];
    const int d = e / el;
    const int row = dest_base[e] + slots[t * top_k + j];
    const bool ok = row < cap;                 // an overflowing slab was already reported by the plan
    if (threadIdx.x == 0) rowmap[t * top_k + j] = ok ? d * cap + row : -1;
    if (ok) dst[nr++] = peer_bases[d] + static_cast<int64_t>(row) * width;
  }
  for (int ch = threadIdx.x; ch < chunks; ch += blockDim.x) {
    uint4 raw = *reinterpret_cast<const uint4*>(x + t * ldx + ch * 8);
    if (norm_w != nullptr) {
      float v[8];
      unpack8(raw, v);
      const float4 w0 = *reinterpret_cast<const float4*>(norm_w + ch * 8);
      const float4 w1 = *reinterpret_cast<const float4*>(norm_w + ch * 8 + 4);
      v[0] *= r * w0.x; v[1] *= r * w0.y; v[2] *= r * w0.z; v[3] *= r * w0.w;
      v[4] *= r * w1.x; v[5] *= r * w1.y; v[6] *= r * w1.z; v[7] *= r * w1.w;
      raw = pack8(v);
    }
    for (int j = 0; j < nr; ++j) *reinterpret_cast<uint4*>(dst[j] + ch * 8) = raw;
  }
}

// Barrier over the ranks of one node.  flag_bases[r] -> rank r's i32 [world + 1] words in peer-mapped
// memory: word s = last barrier number rank s announced to r, word `world` = r's own barrier number.
// Every rank stores its next number into its word on every peer (release, system scope), then waits
// until every peer's number has reached it.  Each rank runs this on its own GPU.  A wait that
// exceeds `limit_ns` records MSL_ERR_DEVICE_TIMEOUT and returns.
__global__ void peer_barrier_kernel(int* const* __restrict__ flag_bases, int rank, int world, uint64_t limit_ns,
                                    int* status) {
  int* mine = flag_bases[rank];
  const int number = mine[world] + 1;            // only thread 0 rewrites it, after the barrier below
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag_bases[p] + rank), "r"(number) : "memory");
    const uint64_t t0 = global_ns();
    for (uint32_t i = 0;; ++i) {
      int seen;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine + p) : "memory");
      if (seen - number >= 0) break;
      if ((i & 255u) == 255u && global_ns() - t0 > limit_ns) {
        report_error(status, MSL_ERR_DEVICE_TIMEOUT);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) mine[world] = number;
}

// ============================================================================ weighted combine
// out[t] = sum_j w[t,j] * rms(y[rowmap[t,j]] * post_w, 1e-8) (+ addend[t]).  One block per token.  The
// routes that have a slab row (rowmap >= 0; under the reference's sharding only the local experts'
// routes do) are compacted in route order and ALL of them (up to kCombineRows per round; more only when
// top_k > 8) are requested at once: one elected thread moves whole rows global -> shared memory with
// cp.async.bulk (TMA, completion on an mbarrier) while every thread prefetches its part of the addend
// (and of the residual stream, when the boundary is fused) into registers.  Then one pass over shared
// memory forms the rows' sums of squares, ONE block-wide reduction turns them into the per-row factors
// r_j = w_j / sqrt(mean((y_j post_w)^2) + eps), and a second pass accumulates sum_j r_j y_j, which
// post_w multiplies once at the end (sum_j w_j rms(y_j post_w) = post_w sum_j r_j y_j).  Each row
// crosses HBM exactly once; a block holds 64 KB at width 4096 and top_k 8, three blocks per SM, so two
// blocks' loads are in flight while a third computes.  (An earlier form took the rows two at a time
// through two 16 KB buffers, five blocks per SM: four block-wide reductions and a dozen barriers per token
// left it at 0.64 of the copy bandwidth.  A persistent form, one block per SM walking over tokens with
// the next two tokens' rows already in flight and the per-column vectors held in registers, gave the same
// bits and ran slower, 0.75-0.89 against 0.53-0.59 ms fused with the boundary at 16384 tokens: a token
// costs a block about 1100 instructions per thread and three block-wide reductions, which three blocks
// per SM overlap and one block cannot.)
constexpr int kCombineThreads = 256;
constexpr int kCombineMaxChunks = 4;    // 8-element chunks per thread: width <= 8192 (MAXC = 2: <= 4096)
constexpr int kCombineRows = 8;         // rows staged per round

__device__ __forceinline__ void bulk_row_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Residual boundary applied to the combined row while it is still in registers (FUSED instantiation): the
// row f = bf16(sum) is what the unfused path would have written and re-read, so both paths give the same
// bits; then b = f * branch_scale, s_out = alpha * s_in + beta * rms(b, eps_branch),
// h_out = bf16(rms(s_out, eps_out) * norm_w), exactly as boundary_kernel.
struct BoundaryTail {
  const float* branch_scale;   // may be NULL
  const float* s_in;           // fp32 [tokens, width]
  const float* alpha;
  const float* beta;
  const float* norm_w;
  float* s_out;                // fp32 [tokens, width]
  __nv_bfloat16* h_out;        // bf16 [tokens, ld_h]
  int64_t ld_h;
  float eps_branch, eps_out;
};

template <int MAXC, bool FUSED>
__global__ void __launch_bounds__(kCombineThreads, MAXC <= 2 ? 3 : 1)
combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ rowmap, const float* __restrict__ w,
               const float* __restrict__ post_w, const __nv_bfloat16* __restrict__ addend, int64_t ld_add,
               __nv_bfloat16* __restrict__ out, int64_t ld_out, int top_k, int width, BoundaryTail bt, int* status) {
  constexpr int THREADS = kCombineThreads;
  constexpr int R = kCombineRows;
  extern __shared__ __align__(128) uint8_t rows_smem[];     // [R][width] bf16
  __shared__ __align__(8) uint64_t bar;
  __shared__ float scratch[32 * R];
  __shared__ int route_of[32], row_of[32];
  __shared__ int n_valid_s, failed_s;
  const int t = blockIdx.x;
  const int chunks = width / 8;
  const uint32_t row_bytes = static_cast<uint32_t>(width) * 2u;
  if (threadIdx.x < 32) {                                   // compact the routes that have a row, in route order
    const int j = threadIdx.x;
    const int row = j < top_k ? rowmap[t * top_k + j] : -1;
    const uint32_t have = __ballot_sync(0xffffffffu, row >= 0);
    if (row >= 0) {
      const int at = __popc(have & ((1u << j) - 1u));
      route_of[at] = j;
      row_of[at] = row;
    }
    __syncwarp();
    if (j == 0) {
      const int n = __popc(have);
      n_valid_s = n;
      failed_s = 0;
      mbar_init(&bar, 1);
      mbar_fence_init();
      if (n > 0) {                                          // round 0 goes out before anything else happens
        const int first = min(R, n);
        mbar_expect_tx(&bar, first * row_bytes);
        for (int q = 0; q < first; ++q)
          bulk_row_load(rows_smem + static_cast<size_t>(q) * row_bytes, y + static_cast<int64_t>(row_of[q]) * width,
                        row_bytes, &bar);
      }
    }
  }
  // what the tail needs from global memory, requested while the rows are in flight
  uint4 add_raw[MAXC];
  float s[FUSED ? MAXC : 1][8];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = threadIdx.x + c * THREADS;
    add_raw[c] = make_uint4(0, 0, 0, 0);
    if (ch < chunks) {
      if (addend != nullptr) add_raw[c] = *reinterpret_cast<const uint4*>(addend + t * ld_add + ch * 8);
      if constexpr (FUSED) {
        const float4 s0 = *reinterpret_cast<const float4*>(bt.s_in + static_cast<int64_t>(t) * width + ch * 8);
        const float4 s1 = *reinterpret_cast<const float4*>(bt.s_in + static_cast<int64_t>(t) * width + ch * 8 + 4);
        s[c][0] = s0.x; s[c][1] = s0.y; s[c][2] = s0.z; s[c][3] = s0.w;
        s[c][4] = s1.x; s[c][5] = s1.y; s[c][6] = s1.z; s[c][7] = s1.w;
      }
    }
  }
  __syncthreads();
  const int n_valid = n_valid_s;
  const int n_rounds = (n_valid + R - 1) / R;
  float acc[MAXC][8];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
  }
  for (int r = 0; r < n_rounds; ++r) {
    const int n_round = min(R, n_valid - r * R);
    // A bulk copy of mapped memory always lands; should the bounded wait run out all the same, the
    // block reports it and, after the next block-wide barrier, leaves without writing its token.
    if (!mbar_wait(&bar, r & 1)) {
      report_error(status, MSL_ERR_DEVICE_TIMEOUT);
      failed_s = 1;
    }
    float ss[R];
#pragma unroll
    for (int q = 0; q < R; ++q) ss[q] = 0.f;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * THREADS;
      if (ch < chunks) {
        const float4 w0 = *reinterpret_cast<const float4*>(post_w + ch * 8);
        const float4 w1 = *reinterpret_cast<const float4*>(post_w + ch * 8 + 4);
        const float pw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int q = 0; q < R; ++q) {
          if (q < n_round) {
            float v[8];
            unpack8(*reinterpret_cast<const uint4*>(rows_smem + static_cast<size_t>(q) * row_bytes + ch * 16), v);
#pragma unroll
            for (int i = 0; i < 8; ++i) { const float x = v[i] * pw[i]; ss[q] += x * x; }
          }
        }
      }
    }
    block_sum<R>(ss, scratch);
    if (failed_s) {                                         // uniform: written before the barriers inside block_sum
      if (threadIdx.x == 0) drain_pause();                  // copies still in flight target this block's memory
      __syncthreads();
      return;
    }
    float rr[R];
#pragma unroll
    for (int q = 0; q < R; ++q)
      rr[q] = q < n_round ? w[t * top_k + route_of[r * R + q]] / sqrtf(ss[q] / width + 1e-8f) : 0.f;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * THREADS;
      if (ch < chunks) {
#pragma unroll
        for (int q = 0; q < R; ++q) {
          if (q < n_round) {
            float v[8];
            unpack8(*reinterpret_cast<const uint4*>(rows_smem + static_cast<size_t>(q) * row_bytes + ch * 16), v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[c][i] += v[i] * rr[q];
          }
        }
      }
    }
    if (r + 1 < n_rounds) {                                 // top_k > 8 only: the next rows reuse the buffer
      fence_async_smem();                                   // generic reads of the buffer before its next bulk write
      __syncthreads();
      if (threadIdx.x == 0) {
        const int n = min(R, n_valid - (r + 1) * R);
        mbar_expect_tx(&bar, n * row_bytes);
        for (int q = 0; q < n; ++q)
          bulk_row_load(rows_smem + static_cast<size_t>(q) * row_bytes,
                        y + static_cast<int64_t>(row_of[(r + 1) * R + q]) * width, row_bytes, &bar);
      }
    }
  }
  // f = addend + post_w * sum, rounded to bf16
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = threadIdx.x + c * THREADS;
    if (ch < chunks) {
      const float4 w0 = *reinterpret_cast<const float4*>(post_w + ch * 8);
      const float4 w1 = *reinterpret_cast<const float4*>(post_w + ch * 8 + 4);
      const float pw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      float o[8];
      unpack8(add_raw[c], o);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += acc[c][i] * pw[i];
      const uint4 packed = pack8(o);
      if constexpr (FUSED) unpack8(packed, acc[c]);          // the bf16-rounded row, as the unfused path re-reads it
      else *reinterpret_cast<uint4*>(out + t * ld_out + ch * 8) = packed;
    }
  }
  if constexpr (FUSED) {
    const int64_t row = t;
    float ss[1] = {0.f};
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * THREADS;
      if (ch < chunks) {
        if (bt.branch_scale != nullptr) {
          const float4 w0 = *reinterpret_cast<const float4*>(bt.branch_scale + ch * 8);
          const float4 w1 = *reinterpret_cast<const float4*>(bt.branch_scale + ch * 8 + 4);
          acc[c][0] *= w0.x; acc[c][1] *= w0.y; acc[c][2] *= w0.z; acc[c][3] *= w0.w;
          acc[c][4] *= w1.x; acc[c][5] *= w1.y; acc[c][6] *= w1.z; acc[c][7] *= w1.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss[0] += acc[c][i] * acc[c][i];
      }
    }
    block_sum<1>(ss, scratch);
    const float rb = 1.0f / sqrtf(ss[0] / width + bt.eps_branch);
    float s2[1] = {0.f};
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * THREADS;
      if (ch < chunks) {
        const float4 a0 = *reinterpret_cast<const float4*>(bt.alpha + ch * 8);
        const float4 a1 = *reinterpret_cast<const float4*>(bt.alpha + ch * 8 + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(bt.beta + ch * 8);
        const float4 b1 = *reinterpret_cast<const float4*>(bt.beta + ch * 8 + 4);
        const float al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const float be[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          s[c][i] = al[i] * s[c][i] + be[i] * (acc[c][i] * rb);
          s2[0] += s[c][i] * s[c][i];
        }
        float* dst = bt.s_out + row * width + ch * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(s[c][0], s[c][1], s[c][2], s[c][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(s[c][4], s[c][5], s[c][6], s[c][7]);
      }
    }
    block_sum<1>(s2, scratch);
    const float rs = 1.0f / sqrtf(s2[0] / width + bt.eps_out);
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * THREADS;
      if (ch < chunks) {
        const float4 w0 = *reinterpret_cast<const float4*>(bt.norm_w + ch * 8);
        const float4 w1 = *reinterpret_cast<const float4*>(bt.norm_w + ch * 8 + 4);
        const float nw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = s[c][i] * rs * nw[i];
        *reinterpret_cast<uint4*>(bt.h_out + row * bt.ld_h + ch * 8) = pack8(o);
      }
    }
  }
}

// Peer form: the rows live in the expert-owning ranks' slabs (rowmap holds rank * peer_cap + row) and are
// read straight from that rank's memory (peer_bases[rank], NVLink): the combine all-to-all of expert
// parallelism fused into this kernel.  All of a token's rows are requested at once, 512 threads per
// block, every thread copying 16 bytes of each row with cp.async and pacing its requests by its own rowmap
// and pointer loads.  (A kernel that staged compacted rows in rounds, given peer pointers, measured 2.0 ms
// where this one takes 0.77 ms on two GPUs: a burst of requests from every block at once does not suit
// NVLink reads.)
template <int MAXK>
__global__ void __launch_bounds__(512)
combine_peer_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ rowmap, const float* __restrict__ w,
               const float* __restrict__ post_w, const __nv_bfloat16* __restrict__ addend, int64_t ld_add,
               __nv_bfloat16* __restrict__ out, int64_t ld_out, int top_k, int width,
               const __nv_bfloat16* const* __restrict__ peer_bases, int peer_cap) {
  extern __shared__ __align__(16) uint8_t peer_rows_smem[];      // [top_k][width] bf16
  __shared__ float scratch[32 * MAXK];
  const int t = blockIdx.x;
  const int chunks = width / 8;
  uint32_t valid = 0;                                       // bit j: route j has a slab row
  for (int j = 0; j < top_k; ++j) {
    const int row = rowmap[t * top_k + j];
    if (row >= 0) {
      valid |= 1u << j;
      const __nv_bfloat16* src = peer_bases[row / peer_cap] + static_cast<int64_t>(row % peer_cap) * width;
      for (int ch = threadIdx.x; ch < chunks; ch += blockDim.x) {
        const uint32_t dst = smem_u32(peer_rows_smem + (static_cast<size_t>(j) * width + ch * 8) * 2);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + ch * 8) : "memory");
      }
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  float ss[MAXK];
#pragma unroll
  for (int j = 0; j < MAXK; ++j) ss[j] = 0.f;
  for (int ch = threadIdx.x; ch < chunks; ch += blockDim.x) {
    const float4 w0 = *reinterpret_cast<const float4*>(post_w + ch * 8);
    const float4 w1 = *reinterpret_cast<const float4*>(post_w + ch * 8 + 4);
    const float pw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int j = 0; j < MAXK; ++j) {
      if (valid & (1u << j)) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(peer_rows_smem + (static_cast<size_t>(j) * width + ch * 8) * 2), v);
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float x = v[i] * pw[i]; ss[j] += x * x; }
      }
    }
  }
  block_sum<MAXK>(ss, scratch);
  float r[MAXK];
#pragma unroll
  for (int j = 0; j < MAXK; ++j)
    r[j] = (valid & (1u << j)) ? w[t * top_k + j] / sqrtf(ss[j] / width + 1e-8f) : 0.f;
  for (int ch = threadIdx.x; ch < chunks; ch += blockDim.x) {
    const float4 w0 = *reinterpret_cast<const float4*>(post_w + ch * 8);
    const float4 w1 = *reinterpret_cast<const float4*>(post_w + ch * 8 + 4);
    const float pw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (addend != nullptr) unpack8(*reinterpret_cast<const uint4*>(addend + t * ld_add + ch * 8), acc);
#pragma unroll
    for (int j = 0; j < MAXK; ++j) {
      if (valid & (1u << j)) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(peer_rows_smem + (static_cast<size_t>(j) * width + ch * 8) * 2), v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[i] * pw[i] * r[j];
      }
    }
    *reinterpret_cast<uint4*>(out + t * ld_out + ch * 8) = pack8(acc);
  }
}

}  // namespace msl

using namespace msl;

extern "C" int msl_qk_rope_store(const void* qkv, int64_t ld, const int64_t* positions, const int64_t* cache_loc,
                                 const float* inv_freq, const float* k_scale, const float* v_scale, void* q8,
                                 void* k_cache, void* v_cache, int tokens, int hq, int hkv, int head_dim,
                                 int64_t cache_rows, int* status, void* stream) {
  if (!qkv || !positions || !cache_loc || !k_scale || !v_scale || !q8 || !k_cache || !v_cache) return MSL_ERR_ARG;
  if (tokens < 0 || hq <= 0 || hkv <= 0) return MSL_ERR_ARG;
  if ((ld & 7) || (reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(q8) & 7) ||
      (reinterpret_cast<uintptr_t>(k_cache) & 7) || (reinterpret_cast<uintptr_t>(v_cache) & 7))
    return MSL_ERR_ALIGN;
  if (tokens == 0) return MSL_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int lanes = (hq + 2 * hkv) * (head_dim / 8);
  const int threads = std::max(kRopeTok * (head_dim / 2), std::min(256, ((lanes + 31) / 32) * 32));
  const dim3 blocks((tokens + kRopeTok - 1) / kRopeTok, (lanes + threads - 1) / threads);
  if (head_dim == 128) {
    qk_rope_store_kernel<128><<<blocks, threads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(qkv), ld, positions, cache_loc, inv_freq, k_scale, v_scale,
        static_cast<uint8_t*>(q8), static_cast<uint8_t*>(k_cache), static_cast<uint8_t*>(v_cache), tokens, hq, hkv,
        cache_rows, status);
  } else if (head_dim == 64) {
    qk_rope_store_kernel<64><<<blocks, threads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(qkv), ld, positions, cache_loc, inv_freq, k_scale, v_scale,
        static_cast<uint8_t*>(q8), static_cast<uint8_t*>(k_cache), static_cast<uint8_t*>(v_cache), tokens, hq, hkv,
        cache_rows, status);
  } else {
    return MSL_ERR_UNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

extern "C" int msl_boundary(const void* branch, int64_t ld_branch, const float* branch_scale, const float* stream_in,
                            const float* alpha, const float* beta, const float* norm_w, float* stream_out,
                            void* hidden_out, int64_t ld_hidden, int tokens, int hidden, float eps_branch,
                            float eps_out, void* stream) {
  if (!branch || !stream_in || !alpha || !beta || !norm_w || !stream_out || !hidden_out) return MSL_ERR_ARG;
  if (tokens < 0 || hidden <= 0 || (hidden & 7) || (ld_branch & 7) || (ld_hidden & 7)) return MSL_ERR_ALIGN;
  if (hidden > 8 * 1024 * 4) return MSL_ERR_UNSUPPORTED;
  if (tokens == 0) return MSL_OK;
  const int chunks = hidden / 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* b = static_cast<const __nv_bfloat16*>(branch);
  auto* h = static_cast<__nv_bfloat16*>(hidden_out);
  // Rows wider than 4096 spread over more threads rather than more registers per thread.
  const int want = chunks <= 512 ? 256 : (chunks <= 1024 ? 512 : 1024);
#define MSL_BOUNDARY(MAXC, THREADS)                                                                              \
  boundary_kernel<MAXC, THREADS><<<tokens, std::min(THREADS, ((chunks + 31) / 32) * 32), 0, st>>>(               \
      b, ld_branch, branch_scale, stream_in, alpha, beta, norm_w, stream_out, h, ld_hidden, hidden, eps_branch,  \
      eps_out)
  if (want >= 1024) {
    if (chunks <= 1024) MSL_BOUNDARY(1, 1024);
    else if (chunks <= 2048) MSL_BOUNDARY(2, 1024);
    else MSL_BOUNDARY(4, 1024);
  } else if (want >= 512) {
    if (chunks <= 512) MSL_BOUNDARY(1, 512);
    else if (chunks <= 1024) MSL_BOUNDARY(2, 512);
    else MSL_BOUNDARY(4, 512);
  } else {
    if (chunks <= 256) MSL_BOUNDARY(1, 256);
    else if (chunks <= 512) MSL_BOUNDARY(2, 256);
    else MSL_BOUNDARY(4, 256);
  }
#undef MSL_BOUNDARY
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

// Host-side argument checks shared by the routing / dispatch entry points (nothing is launched before
// every check of an entry point has passed).
static int check_route(const float* logits, const float* bias, const int* local_start, int tokens, int n_experts,
                       int top_k, int n_local, const int* ids, const float* weights) {
  if (!logits || !bias || !local_start || !ids || !weights) return MSL_ERR_ARG;
  if (tokens < 0 || n_experts <= 0 || top_k <= 0 || top_k > 32 || top_k > n_experts || n_local <= 0 ||
      n_local > n_experts)
    return MSL_ERR_ARG;
  if (n_experts > 512) return MSL_ERR_UNSUPPORTED;
  return MSL_OK;
}

static int check_dispatch(const void* x, int64_t ldx, int tokens, int n_local, int top_k, int width, const void* slab,
                          int64_t slab_rows, const int* rowmap) {
  if (!x || !slab || !rowmap) return MSL_ERR_ARG;
  if (tokens < 0 || n_local <= 0 || n_local > 1024 || top_k <= 0 || top_k > 16 || width <= 0 || slab_rows < 0)
    return MSL_ERR_ARG;
  if ((width & 7) || (ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(slab) & 15))
    return MSL_ERR_ALIGN;
  return MSL_OK;
}

static int launch_route(const RouteArgs& a, cudaStream_t st) {
  const int blocks = (a.tokens + 7) / 8;
  const size_t smem = 2 * static_cast<size_t>(a.n_local) * sizeof(int);
  if (a.n_experts <= 128) route_topk_kernel<4><<<blocks, 256, smem, st>>>(a);
  else if (a.n_experts <= 256) route_topk_kernel<8><<<blocks, 256, smem, st>>>(a);
  else route_topk_kernel<16><<<blocks, 256, smem, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

static int launch_dispatch(const DispatchArgs& a, int tokens, cudaStream_t st) {
  const int threads = std::min(256, ((a.width / 8 + 31) / 32) * 32);
  dispatch_kernel<<<tokens, threads, (a.n_local + 1) * sizeof(int), st>>>(a);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

extern "C" int msl_route_topk(const float* logits, int64_t ld, int hilo, const float* bias, float multiplier,
                              const int* local_start, int tokens, int n_experts, int top_k, int n_local, int* ids,
                              float* weights, int* local_ids, int* slots, int* counts, void* stream) {
  if (!local_ids || !slots || !counts) return MSL_ERR_ARG;
  if (int rc = check_route(logits, bias, local_start, tokens, n_experts, top_k, n_local, ids, weights)) return rc;
  if (tokens == 0) return MSL_OK;
  return launch_route(RouteArgs{logits, ld, hilo, bias, multiplier, local_start, tokens, n_experts, top_k, n_local, ids,
                                weights, local_ids, slots, counts},
                      static_cast<cudaStream_t>(stream));
}

extern "C" int msl_dispatch(const void* x, int64_t ldx, const float* norm_w, const int* local_ids, const int* slots,
                            const int* counts, int tokens, int n_local, int top_k, int width, void* slab,
                            int64_t slab_rows, int* rowmap, int* offsets_out, int* status, void* stream) {
  if (!local_ids || !slots || !counts) return MSL_ERR_ARG;
  if (int rc = check_dispatch(x, ldx, tokens, n_local, top_k, width, slab, slab_rows, rowmap)) return rc;
  if (tokens == 0) return MSL_OK;
  return launch_dispatch(DispatchArgs{static_cast<const __nv_bfloat16*>(x), ldx, norm_w, local_ids, slots, counts,
                                      n_local, top_k, width, static_cast<__nv_bfloat16*>(slab), slab_rows, rowmap,
                                      offsets_out, status},
                         tokens, static_cast<cudaStream_t>(stream));
}

// Resident blocks of the fused routing + dispatch kernel on the current device (cooperative launches
// may not exceed it), looked up once per device.
template <int MAXPL>
static int route_dispatch_max_blocks(size_t smem) {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  int v = cached[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, route_dispatch_kernel<MAXPL>, 256, smem) !=
            cudaSuccess || per_sm <= 0)
      return 0;
    v = per_sm * sm_count();
    cached[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

template <int MAXPL>
static int launch_route_dispatch(RouteArgs ra, DispatchArgs da, int* sync, cudaStream_t st) {
  // shared memory: the larger of phase 1's two histograms and phase 2's offsets (sized for the worst case
  // so that the occupancy look-up holds for every call)
  const size_t smem = 2 * 1024 * sizeof(int) + sizeof(int);
  const int most = route_dispatch_max_blocks<MAXPL>(smem);
  if (most <= 0) return MSL_ERR_CUDA;
  const int grid = std::max(1, std::min(most, ra.tokens));
  void* args[] = {&ra, &da, &sync};
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(route_dispatch_kernel<MAXPL>), dim3(grid),
                                     dim3(256), args, smem, st) == cudaSuccess
             ? MSL_OK
             : MSL_ERR_CUDA;
}

extern "C" int msl_route_dispatch(const float* logits, int64_t ld, int hilo, const float* bias, float multiplier,
                                  const int* local_start, const void* x, int64_t ldx, const float* norm_w,
                                  int tokens, int n_experts, int top_k, int n_local, int width, int* ids,
                                  float* weights, int* local_ids, int* slots, int* counts, int* sync, void* slab,
                                  int64_t slab_rows, int* rowmap, int* offsets_out, int* status, void* stream) {
  if (!local_ids || !slots || !counts || !sync || !offsets_out) return MSL_ERR_ARG;
  if (int rc = check_route(logits, bias, local_start, tokens, n_experts, top_k, n_local, ids, weights)) return rc;
  if (int rc = check_dispatch(x, ldx, tokens, n_local, top_k, width, slab, slab_rows, rowmap)) return rc;
  if (tokens == 0) return MSL_OK;
  const RouteArgs ra{logits, ld, hilo, bias, multiplier, local_start, tokens, n_experts, top_k, n_local, ids, weights,
                     local_ids, slots, counts};
  const DispatchArgs da{static_cast<const __nv_bfloat16*>(x), ldx, norm_w, local_ids, slots, counts, n_local, top_k,
                        width, static_cast<__nv_bfloat16*>(slab), slab_rows, rowmap, offsets_out, status};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_experts <= 128) return launch_route_dispatch<4>(ra, da, sync, st);
  if (n_experts <= 256) return launch_route_dispatch<8>(ra, da, sync, st);
  return launch_route_dispatch<16>(ra, da, sync, st);
}

static int combine_launch(const void* y, const int* rowmap, const float* weights, const float* post_w,
                          const void* addend, int64_t ld_addend, void* out, int64_t ld_out, int tokens, int top_k,
                          int width, const void* const* peer_bases, int peer_cap, const BoundaryTail* tail,
                          int* status, void* stream) {
  if ((!y && !peer_bases) || !rowmap || !weights || !post_w || (!out && !tail)) return MSL_ERR_ARG;
  if (tokens < 0 || top_k <= 0 || top_k > 32 || width <= 0) return MSL_ERR_ARG;
  if ((width & 7) || (ld_out & 7) || (ld_addend & 7)) return MSL_ERR_ALIGN;
  if (width > 8 * kCombineThreads * kCombineMaxChunks) return MSL_ERR_UNSUPPORTED;
  if (tokens == 0) return MSL_OK;
  constexpr int kPeerSmemMax = 200 * 1024;
  const int most = 200 * 1024;
  static SmemConfig c2, c4, c2f, c4f, p4, p8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* yy = static_cast<const __nv_bfloat16*>(y);
  auto* ad = static_cast<const __nv_bfloat16*>(addend);
  auto* oo = static_cast<__nv_bfloat16*>(out);
  auto* pb = reinterpret_cast<const __nv_bfloat16* const*>(peer_bases);
  if (pb != nullptr) {
    if (peer_cap <= 0 || tail != nullptr) return MSL_ERR_ARG;
    if (top_k > 8 || static_cast<int64_t>(top_k) * width * 2 > kPeerSmemMax) return MSL_ERR_UNSUPPORTED;
    const int threads = std::min(512, ((width / 8 + 31) / 32) * 32);
    const int smem = top_k * width * 2;                     // all of a token's rows
    if (top_k <= 4) {
      if (int rc = p4.ensure(combine_peer_kernel<4>, kPeerSmemMax)) return rc;
      combine_peer_kernel<4><<<tokens, threads, smem, st>>>(yy, rowmap, weights, post_w, ad, ld_addend, oo, ld_out,
                                                            top_k, width, pb, peer_cap);
    } else {
      if (int rc = p8.ensure(combine_peer_kernel<8>, kPeerSmemMax)) return rc;
      combine_peer_kernel<8><<<tokens, threads, smem, st>>>(yy, rowmap, weights, post_w, ad, ld_addend, oo, ld_out,
                                                            top_k, width, pb, peer_cap);
    }
    return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
  }
  if (reinterpret_cast<uintptr_t>(y) & 15) return MSL_ERR_ALIGN;
  const int smem = std::min(top_k, kCombineRows) * width * 2;     // all of a token's rows: 64 KB at width 4096, top_k 8
  if (smem > most) return MSL_ERR_UNSUPPORTED;
  const bool small = width <= 8 * kCombineThreads * 2;
  if (tail != nullptr) {
    if (small) {
      if (int rc = c2f.ensure(combine_kernel<2, true>, most)) return rc;
      combine_kernel<2, true><<<tokens, kCombineThreads, smem, st>>>(yy, rowmap, weights, post_w, ad, ld_addend, oo,
                                                                      ld_out, top_k, width, *tail, status);
    } else {
      if (int rc = c4f.ensure(combine_kernel<4, true>, most)) return rc;
      combine_kernel<4, true><<<tokens, kCombineThreads, smem, st>>>(yy, rowmap, weights, post_w, ad, ld_addend, oo,
                                                                      ld_out, top_k, width, *tail, status);
    }
  } else {
    const BoundaryTail none{};
    if (small) {
      if (int rc = c2.ensure(combine_kernel<2, false>, most)) return rc;
      combine_kernel<2, false><<<tokens, kCombineThreads, smem, st>>>(yy, rowmap, weights, post_w, ad, ld_addend, oo,
                                                                       ld_out, top_k, width, none, status);
    } else {
      if (int rc = c4.ensure(combine_kernel<4, false>, most)) return rc;
      combine_kernel<4, false><<<tokens, kCombineThreads, smem, st>>>(yy, rowmap, weights, post_w, ad, ld_addend, oo,
                                                                       ld_out, top_k, width, none, status);
    }
  }
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

extern "C" int msl_combine(const void* y, const int* rowmap, const float* weights, const float* post_w,
                           const void* addend, int64_t ld_addend, void* out, int64_t ld_out, int tokens, int top_k,
                           int width, int* status, void* stream) {
  if (!out) return MSL_ERR_ARG;
  return combine_launch(y, rowmap, weights, post_w, addend, ld_addend, out, ld_out, tokens, top_k, width, nullptr, 0,
                        nullptr, status, stream);
}

extern "C" int msl_combine_boundary(const void* y, const int* rowmap, const float* weights, const float* post_w,
                                    const void* addend, int64_t ld_addend, int tokens, int top_k, int width,
                                    const float* branch_scale, const float* stream_in, const float* alpha,
                                    const float* beta, const float* norm_w, float* stream_out, void* hidden_out,
                                    int64_t ld_hidden, float eps_branch, float eps_out, int* status, void* stream) {
  if (!stream_in || !alpha || !beta || !norm_w || !stream_out || !hidden_out) return MSL_ERR_ARG;
  if (ld_hidden & 7) return MSL_ERR_ALIGN;
  const BoundaryTail tail{branch_scale, stream_in, alpha, beta, norm_w, stream_out,
                          static_cast<__nv_bfloat16*>(hidden_out), ld_hidden, eps_branch, eps_out};
  return combine_launch(y, rowmap, weights, post_w, addend, ld_addend, nullptr, 0, tokens, top_k, width, nullptr, 0,
                        &tail, status, stream);
}

extern "C" int msl_combine_peer(const void* const* peer_bases, int peer_cap, const int* rowmap, const float* weights,
                                const float* post_w, const void* addend, int64_t ld_addend, void* out, int64_t ld_out,
                                int tokens, int top_k, int width, void* stream) {
  if (!peer_bases || !out) return MSL_ERR_ARG;
  return combine_launch(nullptr, rowmap, weights, post_w, addend, ld_addend, out, ld_out, tokens, top_k, width,
                        peer_bases, peer_cap, nullptr, nullptr, stream);
}


// ============================================================================ routing + dispatch without caller scratch
// For hosts that must not allocate device memory when they call in: an inference server that
// hands all of HBM to its own pool at start-up (a later cudaMalloc fails or fragments the pool), or
// a request path where the implicit device-wide synchronisation of cudaMalloc / cudaFree is not
// acceptable.  The per-expert counters and the per-route expert/slot arrays that msl_route_topk
// hands to msl_dispatch live in this file-scope array instead of caller memory.  Every GPU that
// loads the library holds the array (about 2 MiB) until the process exits.
constexpr int kStaticMaxLocal = 1024;            // experts per call
constexpr int kStaticMaxRoutes = 1 << 18;        // tokens * top_k per call
static __device__ __align__(256) int g_route_scratch[kStaticMaxLocal + 2 * kStaticMaxRoutes];

__global__ void zero_ints_kernel(int* p, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = 0;
}

// The array's name is only a host-side handle; kernels need the device address, looked up once per
// device (with that device current) by the first call made on it.
static int* route_scratch_ptr() {
  static int* ptrs[64] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_route_scratch) != cudaSuccess || p == nullptr) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

extern "C" int msl_route_dispatch_static(const float* logits, int64_t ld, int hilo, const float* bias,
                                         float multiplier, const int* local_start, const void* x, int64_t ldx,
                                         const float* norm_w, int tokens, int n_experts, int top_k, int n_local,
                                         int width, int* ids, float* weights, void* slab, int64_t slab_rows,
                                         int* rowmap, int* offsets_out, int* status, void* stream) {
  // Every argument is checked before the scratch is touched or anything is enqueued, so a rejected call
  // leaves the outputs and the shared array as they were.
  if (int rc = check_route(logits, bias, local_start, tokens, n_experts, top_k, n_local, ids, weights)) return rc;
  if (n_local > kStaticMaxLocal || static_cast<int64_t>(tokens) * top_k > kStaticMaxRoutes) return MSL_ERR_CAPACITY;
  if (int rc = check_dispatch(x, ldx, tokens, n_local, top_k, width, slab, slab_rows, rowmap)) return rc;
  if (tokens == 0) return MSL_OK;
  int* scratch = route_scratch_ptr();
  if (scratch == nullptr) return MSL_ERR_CUDA;
  int* counts = scratch;
  int* local_ids = scratch + kStaticMaxLocal;
  int* slots = local_ids + kStaticMaxRoutes;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The counters keep the previous call's totals: clear them on the stream before counting again.
  zero_ints_kernel<<<(n_local + 255) / 256, 256, 0, st>>>(counts, n_local);
  if (cudaGetLastError() != cudaSuccess) return MSL_ERR_CUDA;
  int rc = launch_route(RouteArgs{logits, ld, hilo, bias, multiplier, local_start, tokens, n_experts, top_k, n_local,
                                  ids, weights, local_ids, slots, counts},
                        st);
  if (rc != MSL_OK) return rc;
  return launch_dispatch(DispatchArgs{static_cast<const __nv_bfloat16*>(x), ldx, norm_w, local_ids, slots, counts,
                                      n_local, top_k, width, static_cast<__nv_bfloat16*>(slab), slab_rows, rowmap,
                                      offsets_out, status},
                         tokens, st);
}


extern "C" int msl_ep_plan(const int* counts_all, int world, int local_experts, int rank, int cap, int* dest_base,
                           int* group_offsets, int* status, void* stream) {
  if (!counts_all || !dest_base || !group_offsets || world <= 0 || local_experts <= 0 || rank < 0 || rank >= world ||
      cap <= 0)
    return MSL_ERR_ARG;
  ep_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts_all, world, local_experts, rank, cap,
                                                                    dest_base, group_offsets, status);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

extern "C" int msl_dispatch_peer(const void* x, int64_t ldx, const float* norm_w, const int* ids, const int* slots,
                                 const int* dest_base, void* const* peer_bases, int local_experts, int cap,
                                 int tokens, int top_k, int width, int* rowmap, void* stream) {
  if (!x || !ids || !slots || !dest_base || !peer_bases || !rowmap) return MSL_ERR_ARG;
  if (tokens < 0 || local_experts <= 0 || cap <= 0 || top_k <= 0 || top_k > 16 || width <= 0) return MSL_ERR_ARG;
  if ((width & 7) || (ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15)) return MSL_ERR_ALIGN;
  if (tokens == 0) return MSL_OK;
  const int threads = std::min(256, ((width / 8 + 31) / 32) * 32);
  dispatch_peer_kernel<<<tokens, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, norm_w, ids, slots, dest_base,
      reinterpret_cast<__nv_bfloat16* const*>(peer_bases), local_experts, cap, top_k, width, rowmap);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

extern "C" int msl_peer_barrier(int* const* flag_bases, int rank, int world, int timeout_ms, int* status,
                                void* stream) {
  if (!flag_bases || world <= 0 || world > 64 || rank < 0 || rank >= world || timeout_ms <= 0) return MSL_ERR_ARG;
  peer_barrier_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
      flag_bases, rank, world, static_cast<uint64_t>(timeout_ms) * 1000000ull, status);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}

extern "C" int msl_kv_rows_copy(const void* src, const int64_t* src_idx, int64_t src_rows, void* dst,
                                const int64_t* dst_idx, int64_t dst_rows, int64_t n, int row_bytes, int* status,
                                void* stream) {
  if (!src || !dst || n < 0 || src_rows <= 0 || dst_rows <= 0 || row_bytes <= 0) return MSL_ERR_ARG;
  if ((row_bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
    return MSL_ERR_ALIGN;
  if (n == 0) return MSL_OK;
  const int64_t total = n * (row_bytes / 16);
  const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 8 * static_cast<int64_t>(sm_count())));
  kv_rows_copy_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), src_idx, src_rows, static_cast<uint8_t*>(dst), dst_idx, dst_rows, n,
      row_bytes, status);
  return cudaGetLastError() == cudaSuccess ? MSL_OK : MSL_ERR_CUDA;
}
