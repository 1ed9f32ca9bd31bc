/* C ABI of libmsl: the B200 (sm_100a) kernels of one MoE decoder layer at prefill.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream (cudaStream_t passed as
 * void*), launches asynchronously on that stream, allocates nothing, never synchronises and
 * returns an int status (0 = launched; negative = rejected on the host before any launch).
 * Kernels that wait on hardware barriers bound every wait; a wait that runs out stores
 * MSL_ERR_DEVICE_TIMEOUT into the caller-provided `status` word (device memory, may be NULL),
 * which the caller reads after the stream has drained.
 *
 * The reference (nvbkdw/muse-spark-open-challenge) has no C interface for this path: its layer is
 * a Python `kernel_fn(data, state)` that launches Triton / NVRTC / library kernels.  Each entry
 * below names the launch site in muse_prefill_layer/submission.py that it replaces.
 */
#ifndef MSL_H_
#define MSL_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSL_ABI_VERSION 2

enum {
  MSL_OK = 0,
  MSL_ERR_ARG = -1,
  MSL_ERR_ALIGN = -2,
  MSL_ERR_CUDA = -3,
  MSL_ERR_TENSORMAP = -4,
  MSL_ERR_DEVICE_TIMEOUT = -5,
  MSL_ERR_CAPACITY = -6,
  MSL_ERR_UNSUPPORTED = -7
};

/* Output modes of the GEMMs. */
enum {
  MSL_OUT_BF16 = 0,        /* c: bf16 [m, n] */
  MSL_OUT_F32 = 1,         /* c: fp32 [m, n] */
  MSL_OUT_SWIGLU_BF16 = 2  /* b rows come in blocks of 256 = 128 gate rows then their 128 up rows;
                              c: bf16 [m, n/2] = silu(gate) * up */
};

int msl_abi_version(void);
const char* msl_status_string(int code);

/* Run-time options (process-wide, 0 or 1).  Their defaults are read from the environment once, at the
 * first use of any option (variable of the same name as the comment gives, "0" switches off), so a
 * later change of the environment never changes what a launch does; msl_set_option is the way to change
 * one afterwards.  A CUDA graph keeps the choice that was in force when it was captured.  The reference
 * has no such switches (its tile choices are compile-time constants of its Triton kernels). */
enum {
  MSL_OPT_GEMM_SPLITK = 0,  /* MSL_GEMM_SPLITK: msl_gemm_splitk_plan may recommend slicing K (default 1).  Off:
                               every product runs in one pass and its low bits do not depend on its row count */
  MSL_OPT_GEMM_WIDE = 1,    /* MSL_GEMM_WIDE: the dense GEMM may choose 256 x 256 tiles (1) */
  MSL_OPT_GROUPED_WIDE = 2, /* MSL_GROUPED_WIDE: 256-row tiles in the grouped GEMM unless the slab has under 32 rows per group (1) */
  MSL_OPT_COUNT = 3
};
int msl_set_option(int option, int value);
int msl_get_option(int option);

/* Dense BF16 GEMM, fp32 accumulate: c[m, n] = alpha * sum_{s < segs} A_s * B_s^T with
 * A_s = a[:, s*a_seg_stride : s*a_seg_stride + k] and B_s = b[:, s*b_seg_stride : ... + k];
 * a is bf16 [m, lda] row-major, b is bf16 [n, ldb] row-major (a weight matrix as stored).
 * Two segments with a_seg_stride = 0 give the router's "BF16 hi + lo" product.
 * Replaces torch.mm at submission.py:1082 (QKV+gate), :1096 (O), :1113 (router, fp32 out),
 * :1116 (pooler), :1135 (unpooler).  lda, ldb, k, strides: multiples of 8; a, b: 16-byte aligned. */
int msl_gemm_bf16(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int m, int n,
                  int k, int segs, int a_seg_stride, int b_seg_stride, int out_mode, float alpha, int* status,
                  void* stream);

/* Split-K form of msl_gemm_bf16 for products with few output tiles and a long K (decode steps, verify
 * blocks, short continuation chunks; the router's two-segment product): every tile's K range is cut into
 * `splits` slices that run as separate CTAs and leave fp32 planes [splits][m][n] in `workspace`
 * (splits * m * n * 4 bytes of caller-owned device memory, 16-byte aligned); a second kernel sums the
 * planes in a fixed order, applies alpha and writes c (MSL_OUT_BF16 or MSL_OUT_F32; n and ldc multiples
 * of 4).  msl_gemm_splitk_plan recommends the slice count from the sizes alone (1 = call
 * msl_gemm_bf16; always 1 while MSL_OPT_GEMM_SPLITK is off: slicing K changes the order of the fp32 sums,
 * so a product's low bits then depend on its number of rows).  The reference leaves these products to
 * cuBLAS (submission.py:1082,1096,1113). */
int msl_gemm_splitk_plan(int m, int n, int k, int segs, int out_mode);
int msl_gemm_bf16_splitk(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int m, int n,
                         int k, int segs, int a_seg_stride, int b_seg_stride, int out_mode, float alpha, int splits,
                         void* workspace, int* status, void* stream);

/* Per-head RMS norm (eps 1e-5, no weight) of q and k, interleaved RoPE when inv_freq != NULL
 * (pairs (2i, 2i+1) rotate by positions[t] * inv_freq[i]), q -> E4M3 [tokens, hq, head_dim],
 * k / *k_scale and v / *v_scale -> E4M3 written to row cache_loc[t] of the paged caches
 * ([cache_rows, hkv, head_dim]).  qkv is the bf16 projection output, q heads then k heads then v
 * heads in each row of pitch ld.  A cache_loc outside [0, cache_rows) is skipped and reported in
 * *status.  Replaces _qk_rope_store_kernel (submission.py:740-785, launch :1086-1089).
 * head_dim 64 or 128. */
int msl_qk_rope_store(const void* qkv, int64_t ld, const int64_t* positions, const int64_t* cache_loc,
                      const float* inv_freq, const float* k_scale, const float* v_scale, void* q8, void* k_cache,
                      void* v_cache, int tokens, int hq, int hkv, int head_dim, int64_t cache_rows, int* status,
                      void* stream);

/* Residual boundary: b = branch * branch_scale (branch_scale may be NULL);
 * stream_out = alpha * stream_in + beta * rms(b, eps_branch);
 * hidden_out = bf16(rms(stream_out, eps_out) * norm_w).  alpha, beta, norm_w, branch_scale: fp32
 * [hidden], prepared once from the gate / norm weights.  Replaces _attn_boundary_kernel and
 * _ffn_boundary_kernel (submission.py:806-855, launches :1101, :1138). */
int msl_boundary(const void* branch, int64_t ld_branch, const float* branch_scale, const float* stream_in,
                 const float* alpha, const float* beta, const float* norm_w, float* stream_out, void* hidden_out,
                 int64_t ld_hidden, int tokens, int hidden, float eps_branch, float eps_out, void* stream);

/* Router top-k with slot assignment.  logits fp32 [tokens, ld]: columns [0, n_experts) and, when
 * hilo != 0, a second half [n_experts, 2 n_experts) that is added (BF16 hi + lo router product).
 * score = sigmoid(multiplier * logit); top_k of score + bias, lowest index first among ties;
 * weights = score / (sum of the picked scores + 1e-15).  Experts [*local_start, *local_start +
 * n_local) modulo n_experts are local: local_ids holds id - local_start (or -1) and slots the
 * route's index among its expert's routes, drawn from counts[n_local] (zeroed by the caller).
 * Replaces _routing_kernel (submission.py:859-886, launch :1114). */
int msl_route_topk(const float* logits, int64_t ld, int hilo, const float* bias, float multiplier,
                   const int* local_start, int tokens, int n_experts, int top_k, int n_local, int* ids,
                   float* weights, int* local_ids, int* slots, int* counts, void* stream);

/* Token dispatch: copies row t of x (bf16 [tokens, ldx], `width` columns) to slab row
 * offsets[e] + slot for every local route, offsets being the exclusive prefix sum of counts
 * (written to offsets_out[n_local + 1] when not NULL); rowmap[tokens, top_k] receives the slab row
 * or -1.  With norm_w (fp32 [width]) the row is first RMS-normalised (eps 1e-5) and scaled.
 * Replaces _dispatch_kernel (submission.py:890-899, launch :1123) with a compact slab instead of
 * one token-count-sized slab per expert. */
int msl_dispatch(const void* x, int64_t ldx, const float* norm_w, const int* local_ids, const int* slots,
                 const int* counts, int tokens, int n_local, int top_k, int width, void* slab, int64_t slab_rows,
                 int* rowmap, int* offsets_out, int* status, void* stream);

/* msl_route_topk and msl_dispatch as ONE kernel launch (the reference launches _routing_kernel and
 * _dispatch_kernel separately after zeroing its counters, submission.py:859-899,1114-1123): persistent
 * blocks route all tokens, meet at a grid-wide barrier, form the offsets from the final counts and copy
 * the rows.  Same outputs as the two calls.  `counts` i32 [n_local] and `sync` i32 [2] are zeroed ONCE by
 * their owner; the kernel returns both to zero before it ends (the per-expert counts of a call are
 * offsets_out[e + 1] - offsets_out[e]), so calls on one stream need no memset between them.  offsets_out
 * is required.  The launch is cooperative (all blocks resident); its barrier wait is bounded and reports
 * MSL_ERR_DEVICE_TIMEOUT in *status.  Calls that share `counts` / `sync` must not overlap on the GPU. */
int msl_route_dispatch(const float* logits, int64_t ld, int hilo, const float* bias, float multiplier,
                       const int* local_start, const void* x, int64_t ldx, const float* norm_w, int tokens,
                       int n_experts, int top_k, int n_local, int width, int* ids, float* weights, int* local_ids,
                       int* slots, int* counts, int* sync, void* slab, int64_t slab_rows, int* rowmap,
                       int* offsets_out, int* status, void* stream);

/* Routing and dispatch in one call that needs no scratch memory from the caller: the same
 * results as msl_route_topk followed by msl_dispatch (ids, weights, rowmap, offsets_out, slab),
 * with the per-expert counters and per-route expert/slot arrays kept in a fixed array inside the
 * library.  No counterpart in the reference.  It exists for hosts that cannot allocate when they
 * call in: a server whose memory pool already owns all of HBM, or a request path that cannot take
 * the device-wide synchronisation cudaMalloc implies.  It calls no allocator of any kind.
 * Limits: tokens * top_k <= 262144, otherwise MSL_ERR_CAPACITY (the array also has room for 1024
 * local experts, more than msl_route_topk's own limit of 512 experts allows); the array (about
 * 2 MiB) stays resident on every GPU that loads the library.  The first call on a device
 * looks up the array's device address (cudaGetSymbolAddress); make that first call outside any
 * stream capture.  All calls share the one array, so two calls whose kernels overlap on the GPU
 * (different streams, or different host threads on one device) race: serialise them.  All arguments
 * are checked before anything is enqueued or the array is touched (same rules as msl_route_topk and
 * msl_dispatch: top_k <= 16, n_experts <= 512, 1 <= n_local <= n_experts, width and ldx multiples of 8,
 * x and slab 16-byte aligned); a rejected call changes nothing. */
int msl_route_dispatch_static(const float* logits, int64_t ld, int hilo, const float* bias, float multiplier,
                              const int* local_start, const void* x, int64_t ldx, const float* norm_w, int tokens,
                              int n_experts, int top_k, int n_local, int width, int* ids, float* weights, void* slab,
                              int64_t slab_rows, int* rowmap, int* offsets_out, int* status, void* stream);

/* Weighted combine: out[t] = sum_j weights[t, j] * rms(y[rowmap[t, j]] * post_w, eps 1e-8)
 * (+ addend[t] when not NULL); rowmap < 0 contributes nothing.  y: bf16 [slab rows, width].  The rows are
 * staged by bulk copies whose bounded wait reports MSL_ERR_DEVICE_TIMEOUT in *status (may be NULL); a
 * block whose wait ran out writes nothing.  Replaces _combine_kernel (submission.py:917-928, launch :1132). */
int msl_combine(const void* y, const int* rowmap, const float* weights, const float* post_w, const void* addend,
                int64_t ld_addend, void* out, int64_t ld_out, int tokens, int top_k, int width, int* status,
                void* stream);

/* msl_combine fused with the residual boundary that follows it in a layer without an unpooler (width =
 * hidden size): the combined row f, rounded to bf16 exactly as msl_combine would store it, goes straight
 * into msl_boundary's arithmetic (b = f * branch_scale; stream_out = alpha * stream_in + beta * rms(b,
 * eps_branch); hidden_out = bf16(rms(stream_out, eps_out) * norm_w)) without being written to memory.
 * Same bits as msl_combine followed by msl_boundary for width <= 4096.  Replaces _combine_kernel +
 * _ffn_boundary_kernel (submission.py:917-928, 832-855; launches :1132, :1138). */
int msl_combine_boundary(const void* y, const int* rowmap, const float* weights, const float* post_w,
                         const void* addend, int64_t ld_addend, int tokens, int top_k, int width,
                         const float* branch_scale, const float* stream_in, const float* alpha, const float* beta,
                         const float* norm_w, float* stream_out, void* hidden_out, int64_t ld_hidden,
                         float eps_branch, float eps_out, int* status, void* stream);

/* Expert parallelism over peer memory (one process per GPU, every rank's row slab mapped into every
 * other rank's address space).  These three calls stand where the reference leaves identities for
 * the cross-GPU steps (reference.py:438 all-gather, :451 reduce-scatter, :467 "LOCAL experts") and
 * have no kernel counterpart there.
 *
 * msl_ep_plan: counts_all i32 [world, world * local_experts] (row s = routes of rank s per global
 * expert, all-gathered).  Writes dest_base i32 [world * local_experts] (first row, in the owning
 * rank's slab, of this rank's rows for each expert) and group_offsets i32 [world * local_experts + 1]
 * (row ranges of this rank's own slab, groups ordered (source rank, local expert)), clamped to `cap`.
 * Sets *status to MSL_ERR_CAPACITY when this rank's slab would need more than `cap` rows: the groups
 * beyond the end then come out empty and msl_dispatch_peer skips the same rows, so no kernel that
 * consumes the plan addresses a row at or beyond `cap`. */
int msl_ep_plan(const int* counts_all, int world, int local_experts, int rank, int cap, int* dest_base,
                int* group_offsets, int* status, void* stream);

/* Barrier over the ranks of one node, on the stream: flag_bases is a DEVICE array of `world` pointers
 * to the ranks' i32 [world + 1] flag words (peer-mapped, zeroed once before the first barrier).
 * Orders every earlier peer store of every rank before every later peer load.  A rank that waits longer
 * than timeout_ms sets *status to MSL_ERR_DEVICE_TIMEOUT and carries on.  Each rank must run on its
 * own GPU. */
int msl_peer_barrier(int* const* flag_bases, int rank, int world, int timeout_ms, int* status, void* stream);

/* Dispatch into the owning ranks' slabs: peer_bases is a DEVICE array of `world` pointers to the
 * ranks' bf16 [cap, width] slabs; ids i32 [tokens, top_k] are global expert ids, slots the ranks
 * within (this rank, expert) from msl_route_topk.  The row of route (t, j) lands at
 * peer_bases[e / local_experts] + (dest_base[e] + slot) * width; rowmap receives
 * rank * cap + row (or -1 for a row beyond cap).  Optional RMS norm as in msl_dispatch. */
int msl_dispatch_peer(const void* x, int64_t ldx, const float* norm_w, const int* ids, const int* slots,
                      const int* dest_base, void* const* peer_bases, int local_experts, int cap, int tokens,
                      int top_k, int width, int* rowmap, void* stream);

/* msl_combine with the rows read from the owning ranks' slabs (rowmap from msl_dispatch_peer). */
int msl_combine_peer(const void* const* peer_bases, int peer_cap, const int* rowmap, const float* weights,
                     const float* post_w, const void* addend, int64_t ld_addend, void* out, int64_t ld_out,
                     int tokens, int top_k, int width, void* stream);

/* Row gather / scatter for the K/V hand-off of a sequence whose chunks are prefilled on different
 * ranks: dst[dst_idx ? dst_idx[i] : i] = src[src_idx ? src_idx[i] : i], i < n, rows of row_bytes
 * (multiple of 16; e.g. hkv * head_dim FP8 bytes).  Indices are device int64 arrays; an index outside
 * [0, src_rows) / [0, dst_rows) skips the row and sets *status to MSL_ERR_CAPACITY.  The reference runs
 * one GPU with synthetic cached context (reference.py:195-224) and has no such step. */
int msl_kv_rows_copy(const void* src, const int64_t* src_idx, int64_t src_rows, void* dst, const int64_t* dst_idx,
                     int64_t dst_rows, int64_t n, int row_bytes, int* status, void* stream);

/* Rows of a re-tiled NVFP4 bank: `rows` padded to whole 256-row tiles (for a gate/up bank,
 * interleave != 0, each half padded to whole 128-row blocks). */
int64_t msl_nvfp4_padded_rows(int rows, int interleave);

/* Load-time, lossless re-tiling of an NVFP4 expert bank (weights w13 / w2 of the reference,
 * baseline.py:74-79): codes uint8 [experts, rows, k/2], scales e4m3 [experts, rows, k/16] ->
 * tiles [experts, n_padded/256, k/64, 256, 32] and [.., 256, 4] consumed by
 * msl_grouped_gemm_nvfp4.  With interleave != 0 the bank is gate rows then up rows and tile j
 * holds gate rows [128 j, 128 j + 128) followed by their up rows.  A permutation of the input
 * bits; padding rows are zero.  Takes the place of the reference's load-time
 * weight repack (submission.py:934-950).  k: multiple of 64. */
int msl_nvfp4_repack(const void* src_codes, const void* src_scales, void* dst_codes, void* dst_scales, int experts,
                     int rows, int k, int interleave, void* stream);

/* Grouped expert GEMM, NVFP4 weights x BF16 activations, fp32 accumulate:
 * out[r, :] = global_scales[e] * x[r, :] * dq(W_e)^T for slab rows offsets[g] <= r < offsets[g+1],
 * e = g % weight_experts (row groups may outnumber the weight banks: under expert parallelism a
 * group is (source rank, expert), source-major); x bf16 [slab_rows, k]; out bf16 [slab_rows,
 * ld_out] with n_out valid columns; experts = number of row groups (<= 256); with swiglu != 0
 * the bank is an interleaved gate/up bank and out = silu(gate) * up (n_out = intermediate size).
 * offsets is device memory [experts + 1]; no host synchronisation; rows at or beyond slab_rows (offsets
 * that overrun the buffers) are neither read nor written.  Replaces the two grouped GEMM
 * launches and _silu_mul_kernel (submission.py:956-1002, 903-913; launches :1128-1130). */
int msl_grouped_gemm_nvfp4(const void* x, int64_t slab_rows, const void* codes, const void* scales,
                           const float* global_scales, const int* offsets, void* out, int64_t ld_out, int experts,
                           int weight_experts, int n_padded, int k, int n_out, int swiglu, int* status, void* stream);

/* ---- Opt-in expert mode: NVFP4 activations x NVFP4 weights on the block-scaled tensor-core path
 * (tcgen05.mma kind::mxf4nvf4, UE4M3 scales of 16-element blocks, K = 64 per instruction).  The default
 * expert path (msl_grouped_gemm_nvfp4) keeps BF16 activations, as the reference's contract states
 * (TASK.md:89); this mode quantises them to 4 bits and therefore has its own, larger error.  It follows
 * the format of muse_prefill_layer/nvfp4.py:66-97 and stands where the reference's experiment
 * tools/prefill/moe_kernel/moe_fp4.py:362-448 (tested by test_moe_fp4.py:124-169) runs its W4A16 kernel.
 * k must be a multiple of 256.
 *
 * msl_nvfp4_bs_tiles: weight-row tiles (192 rows; for a gate/up bank 96 gate rows + their 96 up rows) of
 * a bank with `rows` rows.  msl_nvfp4_bs_row_tiles: upper bound of the 128-row activation tiles of a slab
 * with `groups` row groups (sizes the activation scale buffer: row tiles * (k / 256) * 2048 bytes).
 *
 * msl_nvfp4_bs_sf_repack (load time, lossless): e4m3 block scales [banks, rows, k / 16] of a bank as the
 * reference stores it (baseline.py:74-79) -> [banks][tiles][k / 256][4][2][512 bytes], the per-stage
 * blocks the kernel copies to tensor memory.  The 4-bit codes themselves are consumed in place, in the
 * reference's own [banks, rows, k / 2] layout.
 *
 * msl_nvfp4_bs_quantize: rows [0, offsets[groups]) of x (bf16 [slab_rows, ldx], k columns) -> codes u8
 * [slab_rows, k / 2] (element 2i in the low nibble of byte i), block scales in the kernel's tile layout
 * (indexed by the same row tiles the GEMM's scheduler forms from `offsets`), and one fp32 scale per row
 * (max |x| / (6 * 448)), round to nearest throughout. */
int msl_nvfp4_bs_tiles(int rows, int swiglu);
int64_t msl_nvfp4_bs_row_tiles(int64_t slab_rows, int groups);
int msl_nvfp4_bs_sf_repack(const void* src_scales, void* dst_scales, int banks, int rows, int k, int swiglu,
                           void* stream);
int msl_nvfp4_bs_quantize(const void* x, int64_t ldx, int64_t slab_rows, int k, const int* offsets, int groups,
                          void* codes, void* scales, float* row_scales, void* stream);

/* out[r, :] = global_scales[e] * x_row_scales[r] * (xq (*) sx)[r, :] * (wq_e (*) sw_e)^T for the slab rows of
 * row group g (e = g % weight_experts), with the operands of msl_nvfp4_bs_quantize and
 * msl_nvfp4_bs_sf_repack; w_codes is the reference's u8 [weight_experts, weight_rows, k / 2].  With
 * swiglu != 0 the bank is gate rows then up rows and out = silu(gate) * up (n_out = weight_rows / 2).
 * Same scheduling, bounds and status conventions as msl_grouped_gemm_nvfp4. */
int msl_grouped_gemm_nvfp4_bs(const void* x_codes, const void* x_scales, const float* x_row_scales,
                              int64_t slab_rows, const void* w_codes, const void* w_scales_tiled,
                              const float* global_scales, const int* offsets, void* out, int64_t ld_out, int groups,
                              int weight_experts, int weight_rows, int k, int n_out, int swiglu, int* status,
                              void* stream);

/* Causal attention of the new tokens over the paged FP8 cache (which already holds the new
 * tokens' K/V rows): q8 e4m3 [tokens, hq, head_dim]; caches e4m3 [cache_rows, hkv, head_dim];
 * request b owns query rows cu_seqlens_q[b] .. cu_seqlens_q[b+1] at positions seq_lens[b] + i and
 * sees keys 0 .. position (the last `window` of them when window > 0) through
 * page_table[b, pos / page_size].  softmax_scale = sm_scale * qk_scale_factor; *k_scale and
 * *v_scale dequantise the cache.  out bf16 [tokens, ld_out], column h * head_dim + d.  With gate
 * != NULL (bf16, pitch ld_gate, same columns) the epilogue applies the per-head RMS norm (eps
 * 1e-5) and multiplies by sigmoid(gate).  Replaces submission.py:639-721 (gather, attn_fwd,
 * combine, library fallback) and _onorm_gate_kernel (:789-802).  head_dim 64 or 128; hq / hkv a
 * power of two <= 128. */
int msl_attention_fp8(const void* q8, const void* k_cache, const void* v_cache, const int* page_table,
                      int max_pages, const int* seq_lens, const int* cu_seqlens_q, const float* k_scale,
                      const float* v_scale, float softmax_scale, int batch, int max_q_len, int tokens, int hq,
                      int hkv, int head_dim, int page_size, int window, int64_t cache_rows, void* out,
                      int64_t ld_out, const void* gate, int64_t ld_gate, int* status, void* stream);

/* Split-KV form of msl_attention_fp8 for short query blocks over long cached contexts (continuation
 * chunks, verify blocks, decode steps), where the query blocks alone cannot fill the GPU: every query
 * block's key tiles are cut into kv_splits slices, each slice runs as its own CTA and leaves an
 * unnormalised partial result (O, running maximum, row sum) in `workspace`, and a second kernel merges
 * the slices and applies the same epilogue.  Stands where the reference cuts long contexts into splits
 * and merges them (submission.py:649-697: pick_splits, split attn_fwd launches; :610 _attn_combine_kernel).
 * msl_attention_split_plan recommends a slice count from the sizes alone (1 = use msl_attention_fp8);
 * msl_attention_split_workspace gives the workspace size in bytes (device memory, 16-byte aligned,
 * owned by the caller, no initialisation needed). */
int msl_attention_split_plan(int batch, int max_q_len, int hq, int hkv, int max_pages, int page_size, int window);
int64_t msl_attention_split_workspace(int kv_splits, int tokens, int hq, int head_dim);
int msl_attention_fp8_split(const void* q8, const void* k_cache, const void* v_cache, const int* page_table,
                            int max_pages, const int* seq_lens, const int* cu_seqlens_q, const float* k_scale,
                            const float* v_scale, float softmax_scale, int batch, int max_q_len, int tokens, int hq,
                            int hkv, int head_dim, int page_size, int window, int64_t cache_rows, void* out,
                            int64_t ld_out, const void* gate, int64_t ld_gate, int kv_splits, void* workspace,
                            int* status, void* stream);

/* Measured ceiling of one tensor-core instruction shape: every SM issues `iters` tcgen05.mma of
 * M = 128 x N = n back to back on operands resident in shared memory (kind 0: bf16, K = 16; 1: e4m3,
 * K = 32; 2: NVFP4 block scaled, K = 64), no loads and no epilogue.  The caller times the launch
 * (2 * 128 * n * K * iters flops per SM).  It supplies the FP8 and NVFP4 denominators of the roofline
 * fractions; the reference's own model takes the vendor's dense figures (reference.py:681-697). */
int msl_mma_peak(int kind, int n, int iters, int* status, void* stream);

/* Measured issue rate of one scalar-pipe instruction (op 0: ex2.approx.ftz.f32, 1: cvt.rn.satfinite.e4m3x2.f32,
 * 2: fma.rn.f32, 3: max.f32, 4: two ex2 and one such conversion per instance): one CTA of `warps` warps (1..16) per SM, each warp `iters` rounds of 16 independent
 * instances; the longest CTA's span in SM cycles is left in max_cycles[0] by an atomic maximum (two 64-bit device
 * words zeroed by the caller; the second collects the instances' results).  Cycles per warp instruction and scheduler = span / (iters * 16 * warps / 4).  The exponentials
 * and the FP8 conversion of the attention kernel's softmax share one such unit; the reference has no such probe. */
int msl_unit_peak(int op, int warps, int iters, unsigned long long* max_cycles, void* stream);

/* ---- The whole layer for hosts that do not run Python.  These three calls stand where the reference's
 * harness calls `state = prepare(weights)` once and `kernel_fn(data, state)` per step
 * (muse_prefill_layer/submission.py:1013-1070, 1073-1140; tools/prefill/judge.py:94,113,124): the same
 * launch order, side-stream fork of the routing chain (submission.py:1105-1117) and output contract
 * (hidden bf16 [T, H], stream fp32 [T, H], expert ids i32 [T, K], in-place K/V cache writes), with all
 * memory owned by the caller.  All pointers are device memory unless stated. */
typedef struct MslLayerConfig {
  int tokens, batch, max_q_len;   /* T; requests; longest request of the call */
  int hidden, hq, hkv, head_dim;
  int n_experts, n_local, top_k;
  int moe_width, inter;           /* experts' input/output width and intermediate size */
  int pooled;                     /* pooler / unpooler / pre-expert norm present (the reference's shard) */
  int shared_inter;               /* BF16 shared expert's intermediate size, 0 = none (not with `pooled`) */
  int page_size, max_pages, window;
  int64_t cache_rows;             /* rows of each K/V cache: pages * page_size */
  float softmax_scale;            /* sm_scale * qk_scale_factor (reference.py:36, baseline.py:304) */
  float rope_theta;               /* 0 = no RoPE */
} MslLayerConfig;

/* The reference's Weights dict (baseline.py:66-86) as stored: bf16 matrices and vectors, fp32 router and
 * router bias, NVFP4 banks (u8 codes, e4m3 block scales, fp32 per-expert scales). */
typedef struct MslLayerRawWeights {
  const void *qkv_gate, *o, *attn_residual_gate, *ffn_residual_gate, *pre_ffn_norm, *post_expert_norm, *post_ffn_norm,
      *next_pre_attn_norm, *pre_expert_norm, *pooler, *unpooler, *shared_w13, *shared_w2;
  const float *router, *router_bias;
  const void *w13, *w13_sf, *w2, *w2_sf;
  const float *w13_gs, *w2_gs;
} MslLayerRawWeights;

/* What msl_layer_prefill consumes (filled by msl_layer_prepare; points into `prepared` and into the raw
 * weights, which must stay alive). */
typedef struct MslLayerWeights {
  const void *qkv_gate, *o, *router_hilo, *pooler, *unpooler, *shared_w13, *shared_w2;
  const float *router_bias, *a1, *b1, *a2, *b2, *w_pre_ffn, *w_post_exp, *w_post_ffn, *w_next, *w_pre_exp, *inv_freq;
  const void *w13_q, *w13_s, *w2_q, *w2_s;
  const float *w13_gs, *w2_gs;
  int w13_rows, w2_rows;          /* padded rows of the re-tiled banks */
} MslLayerWeights;

typedef struct MslLayerInputs {   /* the reference's Inputs dict, baseline.py:88-105 */
  const float* stream;            /* fp32 [T, H] */
  const void* attn_input;         /* bf16 [T, H] */
  void *k_cache, *v_cache;        /* e4m3 [cache_rows, hkv, head_dim]; the new rows are written in place */
  const int64_t *positions, *cache_loc;
  const int *seq_lens, *cu_seqlens_q, *page_table;   /* page_table i32 [batch, max_pages] */
  const float *k_scale, *v_scale; /* device scalars */
  const int* local_start;         /* device scalar */
} MslLayerInputs;

typedef struct MslLayerOutputs {
  void* hidden;                   /* bf16 [T, H] */
  float* stream;                  /* fp32 [T, H] */
  int* ids;                       /* i32 [T, top_k] */
} MslLayerOutputs;

/* cudaStream_t / cudaEvent_t as void*.  With side == NULL everything runs on `main`; otherwise the router
 * product (and, without a pooler, routing + dispatch) is forked onto `side` and joined again through the
 * two events, which the caller creates once (cudaEventDisableTiming) and owns. */
typedef struct MslLayerStreams {
  void *main, *side, *fork_event, *join_event;
} MslLayerStreams;

/* Bytes of `prepared` / of the per-call workspace for this configuration (-1: configuration rejected). */
int64_t msl_layer_prepared_bytes(const MslLayerConfig* cfg);
int64_t msl_layer_workspace_bytes(const MslLayerConfig* cfg);
/* One-time preparation into caller-owned memory (256-byte aligned): router hi + lo split, residual
 * coefficients, (1 + w) norm vectors, RoPE frequencies, lossless re-tiling of the expert banks, gate/up
 * interleave of the shared expert.  Asynchronous on `stream`. */
int msl_layer_prepare(const MslLayerConfig* cfg, const MslLayerRawWeights* raw, void* prepared, int64_t prepared_bytes,
                      MslLayerWeights* out, void* stream);
/* One layer call.  `workspace` (256-byte aligned, msl_layer_workspace_bytes) needs no initialisation and
 * may be reused by the next call on the same stream; calls that overlap on the GPU need separate
 * workspaces.  Device-side failures (timed-out waits, out-of-range cache rows) are reported in *status. */
int msl_layer_prefill(const MslLayerConfig* cfg, const MslLayerWeights* weights, const MslLayerInputs* in,
                      const MslLayerOutputs* out, void* workspace, int64_t workspace_bytes,
                      const MslLayerStreams* streams, int* status);

#ifdef __cplusplus
}
#endif
#endif /* MSL_H_ */
