// The whole decoder layer behind three C entry points, for hosts that do not run Python:
//   msl_layer_prepare         one-time weight preparation (the reference's prepare(), submission.py:1013-1070)
//   msl_layer_workspace_bytes scratch needed by one call, from the sizes alone
//   msl_layer_prefill         one layer call (the reference's kernel_fn(), submission.py:1073-1140)
// The launch order, the fork of the routing chain onto a side stream next to the dense GEMM that does not
// depend on it, and the carving of the caller-owned workspace are the same as in the Python host
// (layer.py); every kernel is one of this library's own entry points.  Nothing here allocates or
// synchronises; the fork and join are events the caller owns.
#include <cmath>

#include "msl_common.cuh"
#include "msl_host.h"

namespace msl {

constexpr float kRouterMultiplier = 0.1767766952966369f;     // reference.py:51
constexpr float kRmsEps = 1e-5f, kPostNormEps = 1e-8f;        // reference.py:38-39
constexpr int kSlicedMaxTokens = 8;                           // reference.py:58

__host__ __device__ inline int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

// ---------------------------------------------------------------------------- preparation kernels
// out[i] = 1 + w[i]  (the (1 + w) form of every RMS-norm weight, reference.py:189-191)
__global__ void one_plus_kernel(const __nv_bfloat16* __restrict__ w, float* __restrict__ out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = 1.0f + __bfloat162float(w[i]);
}
// Residual coefficients (reference.py:339-344): w = g / 0.3; beta = sigmoid(w);
// alpha = sqrt(max(sigmoid(-w) (1 + beta), 1e-3)).
__global__ void coeffs_kernel(const __nv_bfloat16* __restrict__ gate, float* __restrict__ alpha,
                              float* __restrict__ beta, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float w = __bfloat162float(gate[i]) / 0.3f;
  const float b = 1.0f / (1.0f + expf(-w));
  const float nb = 1.0f / (1.0f + expf(w));
  beta[i] = b;
  alpha[i] = sqrtf(fmaxf(nb * (1.0f + b), 1e-3f));
}
// fp32 router [e, h] -> bf16 [e, 2h]: hi | lo per row with lo = bf16(r - float(hi)) (TASK.md:88 allows
// the split; the two-segment GEMM adds the halves back in fp32).
__global__ void router_split_kernel(const float* __restrict__ r, __nv_bfloat16* __restrict__ out, int e, int h) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(e) * h) return;
  const int64_t row = i / h, col = i - row * h;
  const float v = r[i];
  const __nv_bfloat16 hi = __float2bfloat16(v);
  out[row * 2 * h + col] = hi;
  out[row * 2 * h + h + col] = __float2bfloat16(v - __bfloat162float(hi));
}
// Gate-then-up rows [2 inter, k] -> blocks of 128 gate rows followed by their 128 up rows (the row order
// of the fused SiLU * up epilogue).
__global__ void interleave_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int inter, int chunks) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(2) * inter * chunks) return;
  const int64_t row = i / chunks, c = i - row * chunks;
  const int64_t blk = row / 256, in_blk = row % 256;
  const int64_t from = in_blk < 128 ? blk * 128 + in_blk : inter + blk * 128 + (in_blk - 128);
  dst[i] = src[from * chunks + c];
}
__global__ void inv_freq_kernel(float* __restrict__ out, float theta, int head_dim) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (2 * i < head_dim) out[i] = 1.0f / powf(theta, static_cast<float>(2 * i) / head_dim);
}

// ---------------------------------------------------------------------------- layouts
struct Carver {
  int64_t at = 0;
  int64_t take(int64_t bytes) { const int64_t o = at; at += align256(bytes); return o; }
};

struct PreparedLayout {
  int64_t router_hilo, a1, b1, a2, b2, w_pre_ffn, w_post_exp, w_post_ffn, w_next, w_pre_exp, inv_freq, w13_q, w13_s,
      w2_q, w2_s, shared_w13, total;
  int64_t w13_rows, w2_rows;
};

static PreparedLayout prepared_layout(const MslLayerConfig& c) {
  PreparedLayout L{};
  Carver k;
  const int64_t h = c.hidden, w = c.moe_width;
  L.router_hilo = k.take(static_cast<int64_t>(c.n_experts) * 2 * h * 2);
  L.a1 = k.take(h * 4); L.b1 = k.take(h * 4); L.a2 = k.take(h * 4); L.b2 = k.take(h * 4);
  L.w_pre_ffn = k.take(h * 4); L.w_post_exp = k.take(w * 4); L.w_post_ffn = k.take(h * 4); L.w_next = k.take(h * 4);
  L.w_pre_exp = k.take(c.pooled ? w * 4 : 0);
  L.inv_freq = k.take(c.rope_theta != 0.f ? c.head_dim / 2 * 4 : 0);
  L.w13_rows = msl_nvfp4_padded_rows(2 * c.inter, 1);
  L.w2_rows = msl_nvfp4_padded_rows(c.moe_width, 0);
  // re-tiled banks: 32 code bytes + 4 scale bytes per (row, 64 k)
  L.w13_q = k.take(static_cast<int64_t>(c.n_local) * L.w13_rows * (w / 64) * 32);
  L.w13_s = k.take(static_cast<int64_t>(c.n_local) * L.w13_rows * (w / 64) * 4);
  L.w2_q = k.take(static_cast<int64_t>(c.n_local) * L.w2_rows * (c.inter / 64) * 32);
  L.w2_s = k.take(static_cast<int64_t>(c.n_local) * L.w2_rows * (c.inter / 64) * 4);
  L.shared_w13 = k.take(c.shared_inter ? static_cast<int64_t>(2) * c.shared_inter * w * 2 : 0);
  L.total = k.at;
  return L;
}

struct WorkLayout {
  int64_t qkv, q8, attn, a, s1, h, logits, tw, local_ids, slots, rowmap, counts, sync, offsets, slab_x, slab_i,
      s_inter, shared, pooled, moe, f, gemm_ws, gemm_half, attn_ws, total;
  int kv_splits;
};

static int qkv_size(const MslLayerConfig& c) { return 2 * c.hq * c.head_dim + 2 * c.hkv * c.head_dim; }

static int64_t splitk_bytes(int m, int n, int k, int segs, int out_mode) {
  const int s = msl_gemm_splitk_plan(m, n, k, segs, out_mode);
  return s > 1 ? static_cast<int64_t>(s) * m * n * 4 : 0;
}

static WorkLayout work_layout(const MslLayerConfig& c) {
  WorkLayout L{};
  Carver k;
  const int64_t t = c.tokens, h = c.hidden, w = c.moe_width, qd = static_cast<int64_t>(c.hq) * c.head_dim;
  const int64_t routes = t * c.top_k;
  L.qkv = k.take(t * qkv_size(c) * 2);
  L.q8 = k.take(t * qd);
  L.attn = k.take(t * qd * 2);
  L.a = k.take(t * h * 2);
  L.s1 = k.take(t * h * 4);
  L.h = k.take(t * h * 2);
  L.logits = k.take(t * c.n_experts * 4);
  L.tw = k.take(routes * 4);
  L.local_ids = k.take(routes * 4);
  L.slots = k.take(routes * 4);
  L.rowmap = k.take(routes * 4);
  L.counts = k.take(static_cast<int64_t>(c.n_local) * 4);
  L.sync = k.take(8);
  L.offsets = k.take((static_cast<int64_t>(c.n_local) + 1) * 4);
  L.slab_x = k.take(routes * w * 2);
  L.slab_i = k.take(routes * c.inter * 2);
  L.s_inter = k.take(c.shared_inter ? t * c.shared_inter * 2 : 0);
  L.shared = k.take(c.shared_inter ? t * w * 2 : 0);
  L.pooled = k.take(c.pooled ? t * w * 2 : 0);
  L.moe = k.take(c.pooled ? t * w * 2 : 0);
  L.f = k.take(c.pooled ? t * h * 2 : 0);
  int64_t ws = 0;
  ws = std::max(ws, splitk_bytes(c.tokens, qkv_size(c), c.hidden, 1, MSL_OUT_BF16));
  ws = std::max(ws, splitk_bytes(c.tokens, c.hidden, static_cast<int>(qd), 1, MSL_OUT_BF16));
  ws = std::max(ws, splitk_bytes(c.tokens, c.n_experts, c.hidden, 2, MSL_OUT_F32));
  if (c.pooled) {
    ws = std::max(ws, splitk_bytes(c.tokens, c.moe_width, c.hidden, 1, MSL_OUT_BF16));
    ws = std::max(ws, splitk_bytes(c.tokens, c.hidden, c.moe_width, 1, MSL_OUT_BF16));
  }
  if (c.pooled && c.tokens <= kSlicedMaxTokens)
    ws = std::max(ws, splitk_bytes(c.tokens, c.hidden / 8, c.moe_width, 1, MSL_OUT_BF16));
  if (c.shared_inter) ws = std::max(ws, splitk_bytes(c.tokens, c.moe_width, c.shared_inter, 1, MSL_OUT_BF16));
  L.gemm_half = align256(ws);          // two halves: the main and the side stream may both run a split-K product
  L.gemm_ws = k.take(2 * L.gemm_half);
  L.kv_splits = msl_attention_split_plan(c.batch, c.max_q_len, c.hq, c.hkv, c.max_pages, c.page_size, c.window);
  L.attn_ws = k.take(msl_attention_split_workspace(L.kv_splits, c.tokens, c.hq, c.head_dim));
  L.total = k.at;
  return L;
}

static int check_config(const MslLayerConfig* c) {
  if (!c) return MSL_ERR_ARG;
  if (c->tokens <= 0 || c->batch <= 0 || c->max_q_len <= 0 || c->hidden <= 0 || c->hq <= 0 || c->hkv <= 0 ||
      c->n_experts <= 0 || c->n_local <= 0 || c->n_local > c->n_experts || c->top_k <= 0 || c->moe_width <= 0 ||
      c->inter <= 0 || c->page_size <= 0 || c->max_pages <= 0 || c->cache_rows <= 0 || c->shared_inter < 0)
    return MSL_ERR_ARG;
  if (c->head_dim != 64 && c->head_dim != 128) return MSL_ERR_UNSUPPORTED;
  if ((c->hidden & 7) || (c->moe_width % 64) || (c->inter % 64) || (c->inter % 128) || (c->shared_inter % 128))
    return MSL_ERR_ALIGN;
  if (!c->pooled && c->moe_width != c->hidden) return MSL_ERR_ARG;
  if (c->pooled && c->shared_inter) return MSL_ERR_UNSUPPORTED;
  return MSL_OK;
}

// One GEMM, split over K when the plan says so (the slices' planes go to `ws`).
static int gemm(const void* a, int64_t lda, const void* b, int64_t ldb, void* out, int64_t ldc, int m, int n, int k,
                int segs, int b_seg_stride, int out_mode, void* ws, int* status, void* stream) {
  const int splits = msl_gemm_splitk_plan(m, n, k, segs, out_mode);
  if (splits > 1)
    return msl_gemm_bf16_splitk(a, lda, b, ldb, out, ldc, m, n, k, segs, 0, b_seg_stride, out_mode, 1.0f, splits, ws,
                                status, stream);
  return msl_gemm_bf16(a, lda, b, ldb, out, ldc, m, n, k, segs, 0, b_seg_stride, out_mode, 1.0f, status, stream);
}

}  // namespace msl

using namespace msl;

extern "C" int64_t msl_layer_prepared_bytes(const MslLayerConfig* cfg) {
  if (check_config(cfg)) return -1;
  return prepared_layout(*cfg).total;
}

extern "C" int msl_layer_prepare(const MslLayerConfig* cfg, const MslLayerRawWeights* raw, void* prepared,
                                 int64_t prepared_bytes, MslLayerWeights* out, void* stream) {
  if (int rc = check_config(cfg)) return rc;
  if (!raw || !prepared || !out) return MSL_ERR_ARG;
  const MslLayerConfig& c = *cfg;
  const PreparedLayout L = prepared_layout(c);
  if (prepared_bytes < L.total) return MSL_ERR_CAPACITY;
  if (reinterpret_cast<uintptr_t>(prepared) & 255) return MSL_ERR_ALIGN;
  if (!raw->qkv_gate || !raw->o || !raw->attn_residual_gate || !raw->ffn_residual_gate || !raw->pre_ffn_norm ||
      !raw->post_expert_norm || !raw->post_ffn_norm || !raw->next_pre_attn_norm || !raw->router || !raw->router_bias ||
      !raw->w13 || !raw->w13_sf || !raw->w13_gs || !raw->w2 || !raw->w2_sf || !raw->w2_gs)
    return MSL_ERR_ARG;
  if (c.pooled && (!raw->pooler || !raw->unpooler || !raw->pre_expert_norm)) return MSL_ERR_ARG;
  if (c.shared_inter && (!raw->shared_w13 || !raw->shared_w2)) return MSL_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(prepared);
  auto f32 = [&](int64_t off) { return reinterpret_cast<float*>(base + off); };
  auto bf = [](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
  const int h = c.hidden, w = c.moe_width;
  auto blocks = [](int64_t n) { return static_cast<unsigned>((n + 255) / 256); };
  router_split_kernel<<<blocks(static_cast<int64_t>(c.n_experts) * h), 256, 0, st>>>(
      raw->router, reinterpret_cast<__nv_bfloat16*>(base + L.router_hilo), c.n_experts, h);
  coeffs_kernel<<<blocks(h), 256, 0, st>>>(bf(raw->attn_residual_gate), f32(L.a1), f32(L.b1), h);
  coeffs_kernel<<<blocks(h), 256, 0, st>>>(bf(raw->ffn_residual_gate), f32(L.a2), f32(L.b2), h);
  one_plus_kernel<<<blocks(h), 256, 0, st>>>(bf(raw->pre_ffn_norm), f32(L.w_pre_ffn), h);
  one_plus_kernel<<<blocks(w), 256, 0, st>>>(bf(raw->post_expert_norm), f32(L.w_post_exp), w);
  one_plus_kernel<<<blocks(h), 256, 0, st>>>(bf(raw->post_ffn_norm), f32(L.w_post_ffn), h);
  one_plus_kernel<<<blocks(h), 256, 0, st>>>(bf(raw->next_pre_attn_norm), f32(L.w_next), h);
  if (c.pooled) one_plus_kernel<<<blocks(w), 256, 0, st>>>(bf(raw->pre_expert_norm), f32(L.w_pre_exp), w);
  if (c.rope_theta != 0.f)
    inv_freq_kernel<<<1, 64, 0, st>>>(f32(L.inv_freq), c.rope_theta, c.head_dim);
  if (cudaGetLastError() != cudaSuccess) return MSL_ERR_CUDA;
  int rc = msl_nvfp4_repack(raw->w13, raw->w13_sf, base + L.w13_q, base + L.w13_s, c.n_local, 2 * c.inter, w, 1, stream);
  if (rc) return rc;
  rc = msl_nvfp4_repack(raw->w2, raw->w2_sf, base + L.w2_q, base + L.w2_s, c.n_local, w, c.inter, 0, stream);
  if (rc) return rc;
  if (c.shared_inter) {
    const int chunks = w / 8;
    interleave_rows_kernel<<<blocks(static_cast<int64_t>(2) * c.shared_inter * chunks), 256, 0, st>>>(
        static_cast<const uint4*>(raw->shared_w13), reinterpret_cast<uint4*>(base + L.shared_w13), c.shared_inter, chunks);
    if (cudaGetLastError() != cudaSuccess) return MSL_ERR_CUDA;
  }
  MslLayerWeights o{};
  o.qkv_gate = raw->qkv_gate;
  o.o = raw->o;
  o.router_hilo = base + L.router_hilo;
  o.router_bias = raw->router_bias;
  o.a1 = f32(L.a1); o.b1 = f32(L.b1); o.a2 = f32(L.a2); o.b2 = f32(L.b2);
  o.w_pre_ffn = f32(L.w_pre_ffn); o.w_post_exp = f32(L.w_post_exp); o.w_post_ffn = f32(L.w_post_ffn);
  o.w_next = f32(L.w_next);
  o.w_pre_exp = c.pooled ? f32(L.w_pre_exp) : nullptr;
  o.inv_freq = c.rope_theta != 0.f ? f32(L.inv_freq) : nullptr;
  o.pooler = raw->pooler;
  o.unpooler = raw->unpooler;
  o.w13_q = base + L.w13_q; o.w13_s = base + L.w13_s; o.w13_gs = raw->w13_gs; o.w13_rows = static_cast<int>(L.w13_rows);
  o.w2_q = base + L.w2_q; o.w2_s = base + L.w2_s; o.w2_gs = raw->w2_gs; o.w2_rows = static_cast<int>(L.w2_rows);
  o.shared_w13 = c.shared_inter ? base + L.shared_w13 : nullptr;
  o.shared_w2 = raw->shared_w2;
  *out = o;
  return MSL_OK;
}

extern "C" int64_t msl_layer_workspace_bytes(const MslLayerConfig* cfg) {
  if (check_config(cfg)) return -1;
  return work_layout(*cfg).total;
}

extern "C" int msl_layer_prefill(const MslLayerConfig* cfg, const MslLayerWeights* wt, const MslLayerInputs* in,
                                 const MslLayerOutputs* out, void* workspace, int64_t workspace_bytes,
                                 const MslLayerStreams* streams, int* status) {
  if (int rc = check_config(cfg)) return rc;
  if (!wt || !in || !out || !workspace || !streams) return MSL_ERR_ARG;
  if (!in->stream || !in->attn_input || !in->k_cache || !in->v_cache || !in->positions || !in->cache_loc ||
      !in->seq_lens || !in->cu_seqlens_q || !in->page_table || !in->k_scale || !in->v_scale || !in->local_start ||
      !out->hidden || !out->stream || !out->ids)
    return MSL_ERR_ARG;
  const MslLayerConfig& c = *cfg;
  const WorkLayout L = work_layout(c);
  if (workspace_bytes < L.total) return MSL_ERR_CAPACITY;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return MSL_ERR_ALIGN;
  const bool fork = streams->side != nullptr;
  if (fork && (!streams->fork_event || !streams->join_event)) return MSL_ERR_ARG;
  void* main = streams->main;
  void* side = fork ? streams->side : main;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const int t = c.tokens, h = c.hidden, w = c.moe_width, d = c.head_dim;
  const int qd = c.hq * d, qkv_n = qkv_size(c);
  void* gemm_ws_main = ws + L.gemm_ws;
  void* gemm_ws_side = ws + L.gemm_ws + L.gemm_half;
  int rc;
#define MSL_TRY(call) do { rc = (call); if (rc != MSL_OK) return rc; } while (0)
  // ---- attention stage
  MSL_TRY(gemm(in->attn_input, h, wt->qkv_gate, h, ws + L.qkv, qkv_n, t, qkv_n, h, 1, 0, MSL_OUT_BF16, gemm_ws_main,
               status, main));
  MSL_TRY(msl_qk_rope_store(ws + L.qkv, qkv_n, in->positions, in->cache_loc, wt->inv_freq, in->k_scale, in->v_scale,
                            ws + L.q8, in->k_cache, in->v_cache, t, c.hq, c.hkv, d, c.cache_rows, status, main));
  const __nv_bfloat16* gate = reinterpret_cast<const __nv_bfloat16*>(ws + L.qkv) + (c.hq + 2 * c.hkv) * d;
  if (L.kv_splits > 1)
    MSL_TRY(msl_attention_fp8_split(ws + L.q8, in->k_cache, in->v_cache, in->page_table, c.max_pages, in->seq_lens,
                                    in->cu_seqlens_q, in->k_scale, in->v_scale, c.softmax_scale, c.batch, c.max_q_len,
                                    t, c.hq, c.hkv, d, c.page_size, c.window, c.cache_rows, ws + L.attn, qd, gate,
                                    qkv_n, L.kv_splits, ws + L.attn_ws, status, main));
  else
    MSL_TRY(msl_attention_fp8(ws + L.q8, in->k_cache, in->v_cache, in->page_table, c.max_pages, in->seq_lens,
                              in->cu_seqlens_q, in->k_scale, in->v_scale, c.softmax_scale, c.batch, c.max_q_len, t,
                              c.hq, c.hkv, d, c.page_size, c.window, c.cache_rows, ws + L.attn, qd, gate, qkv_n, status,
                              main));
  MSL_TRY(gemm(ws + L.attn, qd, wt->o, qd, ws + L.a, h, t, h, qd, 1, 0, MSL_OUT_BF16, gemm_ws_main, status, main));
  MSL_TRY(msl_boundary(ws + L.a, h, nullptr, in->stream, wt->a1, wt->b1, wt->w_pre_ffn,
                       reinterpret_cast<float*>(ws + L.s1), ws + L.h, h, t, h, kPostNormEps, kRmsEps, main));
  // ---- MoE stage: the router product runs on the side stream next to the dense GEMM that does not need it
  cudaStream_t m_st = static_cast<cudaStream_t>(main), s_st = static_cast<cudaStream_t>(side);
  if (fork) {
    if (cudaEventRecord(static_cast<cudaEvent_t>(streams->fork_event), m_st) != cudaSuccess ||
        cudaStreamWaitEvent(s_st, static_cast<cudaEvent_t>(streams->fork_event), 0) != cudaSuccess)
      return MSL_ERR_CUDA;
  }
  if (cudaMemsetAsync(ws + L.counts, 0, (L.offsets - L.counts), s_st) != cudaSuccess) return MSL_ERR_CUDA;   // counts + sync
  MSL_TRY(gemm(ws + L.h, h, wt->router_hilo, 2 * h, ws + L.logits, c.n_experts, t, c.n_experts, h, 2, h, MSL_OUT_F32,
               gemm_ws_side, status, side));
  auto route_dispatch = [&](const void* x, int64_t ldx, const float* norm_w, void* stream) {
    return msl_route_dispatch(reinterpret_cast<const float*>(ws + L.logits), c.n_experts, 0, wt->router_bias,
                              kRouterMultiplier, in->local_start, x, ldx, norm_w, t, c.n_experts, c.top_k, c.n_local, w,
                              out->ids, reinterpret_cast<float*>(ws + L.tw), reinterpret_cast<int*>(ws + L.local_ids),
                              reinterpret_cast<int*>(ws + L.slots), reinterpret_cast<int*>(ws + L.counts),
                              reinterpret_cast<int*>(ws + L.sync), ws + L.slab_x, static_cast<int64_t>(t) * c.top_k,
                              reinterpret_cast<int*>(ws + L.rowmap), reinterpret_cast<int*>(ws + L.offsets), status,
                              stream);
  };
  if (!c.pooled) MSL_TRY(route_dispatch(ws + L.h, h, nullptr, side));
  const void* shared = nullptr;
  if (c.pooled) {
    MSL_TRY(gemm(ws + L.h, h, wt->pooler, h, ws + L.pooled, w, t, w, h, 1, 0, MSL_OUT_BF16, gemm_ws_main, status, main));
  } else if (c.shared_inter) {
    MSL_TRY(gemm(ws + L.h, h, wt->shared_w13, w, ws + L.s_inter, c.shared_inter, t, 2 * c.shared_inter, w, 1, 0,
                 MSL_OUT_SWIGLU_BF16, gemm_ws_main, status, main));
    MSL_TRY(gemm(ws + L.s_inter, c.shared_inter, wt->shared_w2, c.shared_inter, ws + L.shared, w, t, w, c.shared_inter,
                 1, 0, MSL_OUT_BF16, gemm_ws_main, status, main));
    shared = ws + L.shared;
  }
  if (fork) {
    if (cudaEventRecord(static_cast<cudaEvent_t>(streams->join_event), s_st) != cudaSuccess ||
        cudaStreamWaitEvent(m_st, static_cast<cudaEvent_t>(streams->join_event), 0) != cudaSuccess)
      return MSL_ERR_CUDA;
  }
  if (c.pooled) MSL_TRY(route_dispatch(ws + L.pooled, w, wt->w_pre_exp, main));
  const int64_t routes = static_cast<int64_t>(t) * c.top_k;
  const int* offsets = reinterpret_cast<const int*>(ws + L.offsets);
  MSL_TRY(msl_grouped_gemm_nvfp4(ws + L.slab_x, routes, wt->w13_q, wt->w13_s, wt->w13_gs, offsets, ws + L.slab_i,
                                 c.inter, c.n_local, c.n_local, wt->w13_rows, w, c.inter, 1, status, main));
  MSL_TRY(msl_grouped_gemm_nvfp4(ws + L.slab_i, routes, wt->w2_q, wt->w2_s, wt->w2_gs, offsets, ws + L.slab_x, w,
                                 c.n_local, c.n_local, wt->w2_rows, c.inter, w, 0, status, main));
  const int* rowmap = reinterpret_cast<const int*>(ws + L.rowmap);
  const float* tw = reinterpret_cast<const float*>(ws + L.tw);
  if (!c.pooled) {
    // combine and FFN boundary as one kernel
    MSL_TRY(msl_combine_boundary(ws + L.slab_x, rowmap, tw, wt->w_post_exp, shared, w, t, c.top_k, w, wt->w_post_ffn,
                                 reinterpret_cast<const float*>(ws + L.s1), wt->a2, wt->b2, wt->w_next, out->stream,
                                 out->hidden, h, kPostNormEps, kRmsEps, status, main));
    return MSL_OK;
  }
  MSL_TRY(msl_combine(ws + L.slab_x, rowmap, tw, wt->w_post_exp, nullptr, 0, ws + L.moe, w, t, c.top_k, w, status, main));
  if (t > kSlicedMaxTokens) {
    MSL_TRY(gemm(ws + L.moe, w, wt->unpooler, w, ws + L.f, h, t, h, w, 1, 0, MSL_OUT_BF16, gemm_ws_main, status, main));
  } else {
    // decode steps and verify blocks: only the first hidden / 8 columns are formed, the rest is zero
    // (reference.py:56-58,468-470)
    const int cols = h / 8;
    if (cudaMemsetAsync(ws + L.f, 0, static_cast<size_t>(t) * h * 2, m_st) != cudaSuccess) return MSL_ERR_CUDA;
    MSL_TRY(gemm(ws + L.moe, w, wt->unpooler, w, ws + L.f, h, t, cols, w, 1, 0, MSL_OUT_BF16, gemm_ws_main, status, main));
  }
  MSL_TRY(msl_boundary(ws + L.f, h, wt->w_post_ffn, reinterpret_cast<const float*>(ws + L.s1), wt->a2, wt->b2,
                       wt->w_next, out->stream, out->hidden, h, t, h, kPostNormEps, kRmsEps, main));
#undef MSL_TRY
  return MSL_OK;
}
