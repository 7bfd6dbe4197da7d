/*
 * lvar_b200 - C ABI of the B200 (sm_100a) sparse-attention kernels.
 *
 * Every entry point is asynchronous on the CUDA stream it is given, allocates nothing unless its
 * comment says otherwise, and returns LVAR_OK or a negative LVAR_ERR_* code; lvar_last_error()
 * gives the message of the calling thread's last failure.  All tensor pointers are DEVICE pointers.
 * Tensors are bf16 [B, H, L, D] views with a contiguous last dimension; strides are in ELEMENTS.
 *
 * Each declaration names the interface of the reference project (Weepingchestnut/Lvar, paths relative
 * to its root) that it stands in for.
 */
#ifndef LVAR_B200_H_
#define LVAR_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LVAR_OK 0
#define LVAR_ERR_ARG (-1)          /* bad pointer, shape, stride or flag */
#define LVAR_ERR_UNSUPPORTED (-2)  /* valid request outside what the kernels cover (e.g. head dim) */
#define LVAR_ERR_CUDA (-3)         /* a CUDA runtime or driver call failed */
#define LVAR_ERR_LIMIT (-4)        /* a size exceeds a documented maximum */

/* Device status word values (int32 in device memory, set by a kernel; 0 = fine). */
#define LVAR_DEV_OK 0
#define LVAR_DEV_TIMEOUT_PRODUCER 1
#define LVAR_DEV_TIMEOUT_MMA 2
#define LVAR_DEV_TIMEOUT_SOFTMAX 3
#define LVAR_DEV_TIMEOUT_DRAIN 4
#define LVAR_DEV_BAD_INDEX 5
#define LVAR_DEV_FORCED_TIMEOUT 6

/* Default per-wait limit of the kernels' bounded waits, in nanoseconds. */
#define LVAR_DEFAULT_WAIT_NS 2000000000ull

typedef void* lvar_stream_t; /* a cudaStream_t */

/* Argument block shared by the three attention entry points. Zero-initialise, then fill. */
typedef struct lvar_attn_args {
  /* problem */
  int32_t B, H, Lq, Lkv, D; /* D in {64, 128}; query heads == kv heads */
  float scale;              /* softmax scale (> 0), applied to q.k before the softmax */
  /* q [B,H,Lq,D], k/v [B,H,Lkv,D], o [B,H,Lq,D]: bf16, 16-byte aligned, strides multiples of 8
     (an o whose base and strides are multiples of 32 bytes is written with 256-bit stores) */
  const void* q;
  int64_t q_sb, q_sh, q_sl;
  const void* k;
  int64_t k_sb, k_sh, k_sl;
  const void* v;
  int64_t v_sb, v_sh, v_sl;
  void* o;
  int64_t o_sb, o_sh, o_sl;
  /* optional row statistics, fp32 [B,H,Lq] contiguous (dense / block-sparse only):
   *   M = max_j(s_ij * scale) * log2(e),  L = sum_j exp2(s_ij * scale * log2e - M)  */
  float* M;
  float* L;
  /* lvar_dense_colsum_attn only: column sums per 128-row query tile, fp32 [B,H,ceil(Lq/128),Lkv], strides in
   * elements (innermost 1) */
  float* cs;
  int64_t cs_sb, cs_sh, cs_st;
  /* 1 (also when 0): one row of cs per 128-row query tile.  2: one row per 256-row group,
   * fp32 [B,H,ceil(Lq/256),Lkv]; the caller zeroes cs first and the group's two tiles add into the row
   * (two addends onto zero: the same bits in either order). */
  int32_t cs_group_tiles;
  /* block-sparse only: uint8 mask [*, *, ceil(Lq/bs), ceil(Lkv/bs)], nonzero = attend, bs = block_size.
   * A stride of 0 broadcasts over batch / head. Innermost stride is 1. */
  const uint8_t* block_mask;
  int64_t bm_sb, bm_sh, bm_sq;
  int32_t block_size; /* 128 (also when 0) or 64 */
  /* column-sparse only */
  const int32_t* indices; /* [B,H,G,>=max count], G = ceil(Lq/group_rows); entries in [0,Lkv) */
  int64_t i_sb, i_sh, i_sg;
  const int32_t* counts; /* [B,H,G]: number of leading entries of each list that are used */
  int64_t c_sb, c_sh;
  int32_t group_rows; /* query rows that share one index list ("bm") */
  const void* o_in;   /* bf16 [B,H,Lq,D] accumulate input; may be the same buffer as o */
  int64_t oi_sb, oi_sh, oi_sl;
  int32_t o_scale; /* +1 or -1 */
  /* o_in_side > 0: o_in is instead a cache [B,H,o_in_side^2,D] over a square token grid, and the accumulate
   * input of query row y * o_side + x (o_side^2 == Lq) is its bilinear resize to the o_side grid
   * (align_corners = False, fp32 interpolation rounded to bf16 once), bit-identical to lvar_upsample_ocache
   * followed by a plain accumulate; o_in must then not be the output buffer.  0: o_in is [B,H,Lq,D]. */
  int32_t o_in_side, o_side;
  /* scheduling: the kernels are persistent (one CTA per SM) and draw work items from a counter in
   * device memory.  sched_scratch points to TWO int32 that are zero when the kernel starts; the kernel
   * leaves them zero, so one zeroed buffer serves every later launch on the same stream.  Launches
   * that may overlap on the GPU need separate buffers.
   * A work item is a PAIR of adjacent 128-row query tiles of one (batch, head): pair id =
   * (b * H + h) * ceil(Lq / 256) + pair index (column-sparse: groups of group_rows rows take the place of
   * Lq).  work_order (optional, device int32[B * H * pairs per head]) is a permutation of the pair ids: the
   * pair at position i is handed out i-th, e.g. heaviest first for a ragged block mask.  When the last wave
   * of pairs fills at most half of the SMs, the pairs at the END of the order are handed out as single
   * tiles; dense and block-sparse attention run such a tile on both halves of the CTA, each half taking
   * half of the tile's KV blocks, and merge the two partial results in the epilogue. */
  int32_t* sched_scratch;
  const int32_t* work_order;
  /* plumbing */
  int32_t* dev_status;    /* optional device int32, must be zeroed by the caller; see LVAR_DEV_* */
  uint64_t wait_limit_ns; /* per-wait limit of the kernel's bounded waits; 0 forces every pending wait to fail */
  /* scheduling switches (0 = default; for measurements and tests): LVAR_SCHED_* bits */
  int32_t sched_flags;
  /* lvar_dense_colsum_attn_given only: the row statistics to normalise with, fp32 [B,H,Lq] contiguous, in the
   * convention of M and L above (as lvar_dense_attn writes them) */
  const float* M_in;
  const float* L_in;
} lvar_attn_args;

#define LVAR_SCHED_PAIRS_ONLY 1     /* never hand the last wave out as single tiles */
#define LVAR_SCHED_SINGLE_ONE_SLOT 2 /* a single tile runs on one half of the CTA (no KV split, no merge) */
#define LVAR_SCHED_SERIALIZE_LAUNCH 4 /* launch without the programmatic-dependent-launch attribute */

/* Dense attention o = softmax(q k^T * scale) v with row statistics.
 * Replaces torch.ops.chipmunk.dense_attn (kernels/chipmunk/csrc/attn/dense_attn.cu:248-372) and
 * sattn_triton.dense_attn (kernels/sparse_attn/triton/attn_dense.py:186-231), called from
 * kernels/sparse_attn/sparse_attn_ops.py:21-59 and models/sparvar/basic_sparvar.py:384. */
int lvar_dense_attn(const lvar_attn_args* args, lvar_stream_t stream);

/* Dense attention and, in the same launch, the exact attention column sums of every 128-row query tile:
 * cs[b,h,t,j] = sum over the rows i of tile t of softmax(q k^T * scale)[i,j].  After a work item's attention
 * sweep the kernel holds the final row statistics, keeps the two Q tiles in shared memory, streams the K tiles
 * a second time and takes the TRANSPOSED product K Q^T, so that a thread owns a key column and sums its 128
 * probabilities in registers (fixed order, bit-reproducible).  Sums over larger query groups (multiples of
 * 128 rows) are sums of adjacent tiles.  Replaces dense_colsum_attn_q / _s (dense attention followed by a
 * separate column-sum kernel, kernels/sparse_attn/sparse_attn_ops.py:65-149,
 * kernels/sparse_attn/triton/attn_dense_colsum.py:101-296) when the group size is a multiple of 128. */
int lvar_dense_colsum_attn(const lvar_attn_args* args, lvar_stream_t stream);

/* Dense attention and its column sums in ONE sweep, for a caller that already holds the row statistics of this
 * attention (args->M_in, args->L_in): every probability is formed once, already normalised,
 *   p_ij = exp2(q_i.k_j * scale * log2e - M_in_i) / L_in_i,
 * feeds both o = P v and cs[b,h,t,j] = sum over the rows i of tile t of p_ij (cs, cs_group_tiles as in
 * lvar_dense_colsum_attn; fixed summation order, bit-reproducible).  o is divided by the measured row sums of p,
 * so it is this attention's exact output also when the statistics come from another pass over slightly
 * different data (they must be within a factor 2^100 of the true normaliser); the column sums are normalised by
 * the GIVEN statistics, as in the reference.  args->M / args->L, when non-null, receive M_in and L_in times the
 * row sum (the true statistics in the same convention).
 * Replaces torch.ops.chipmunk.dense_colsum_attn(q, k, v, p) (kernels/chipmunk/csrc/attn/dense_colsum_attn.cu:
 * 354-522; the column sums of the P tile it already holds for P V, :270-280), which the reference's
 * dense_colsum_attn_s calls after dense_attn (kernels/sparse_attn/sparse_attn_ops.py:65-113). */
int lvar_dense_colsum_attn_given(const lvar_attn_args* args, lvar_stream_t stream);

/* The attention column sums alone, per 128-row query tile (cs as in lvar_dense_colsum_attn); v, o and their
 * strides are not read and may be null / 0.  stats_given = 0: one launch takes the row statistics in a first
 * sweep that does everything but P and PV (M and L are written when non-null) and the sums in a second one.
 * stats_given != 0: args->M and args->L are inputs (as lvar_dense_attn writes them) and only the second sweep
 * runs.  This is the KV-importance score of a scale when no attention output is wanted
 * (the scores dense_colsum_attn_q / _s return next to o, kernels/sparse_attn/sparse_attn_ops.py:65-149; the
 * reference has no entry point without the output). */
int lvar_colsum_tiles(const lvar_attn_args* args, int32_t stats_given, lvar_stream_t stream);

/* Block-sparse attention under a 128x128 block mask; rows whose blocks are all masked give 0.
 * Replaces flex_attention(q, k, v, block_mask=...) in SparseFlexAttn.forward
 * (models/sparvar/basic_sparvar.py:187-194). */
int lvar_block_sparse_attn(const lvar_attn_args* args, lvar_stream_t stream);

/* Column-sparse ("csp") attention: for each group of `group_rows` queries, attention over the keys
 * listed in indices[b,h,g,:counts[b,h,g]] (a multiset), then o = o_in + o_scale * delta.
 * Replaces torch.ops.chipmunk.csp_attn (kernels/chipmunk/csrc/attn/csp_attn.cu:318-433) and
 * sattn_triton.csp_attn (kernels/sparse_attn/triton/attn_csp.py:215-265), called from
 * kernels/sparse_attn/sparse_attn_ops.py:273-292. Unlike the reference, counts need not be a
 * multiple of the KV tile.  With o_in_side > 0 the launch also takes over the O-cache resize that
 * precedes it in a sparse step (upsample_Ocache, models/sparvar/sparse_attn.py:324-362). */
int lvar_csp_attn(const lvar_attn_args* args, lvar_stream_t stream);

/* Attention column sums (KV-importance scores) given the row statistics of a previous attention pass:
 *   cs[b,h,g,j] = sum_{i in group g} exp2(q_i.k_j * scale * log2e - M_i) / L_i,   g = i / group_rows
 * q [B,H,Lq,D], k [B,H,Lkv,D] bf16; M, L fp32 [B,H,Lq] contiguous (as written by lvar_dense_attn);
 * cs fp32 [B,H,ceil(Lq/group_rows),Lkv] with the given strides (innermost 1); every element is
 * written, no zero-fill needed, and the summation order is fixed (bit-reproducible).
 * group_rows must be a multiple of 32.
 * Replaces the second sweep of _full_attn_fwd (kernels/sparse_attn/triton/attn_dense_colsum.py:198-234)
 * and the colsum of torch.ops.chipmunk.dense_colsum_attn(q,k,v,p)
 * (kernels/chipmunk/csrc/attn/dense_colsum_attn.cu:354-522), reached through dense_colsum_attn_q/_s
 * (kernels/sparse_attn/sparse_attn_ops.py:65-149). */
int lvar_colsum(const void* q, const void* k, const float* M, const float* L, float* cs, int32_t B, int32_t H,
                int32_t Lq, int32_t Lkv, int32_t D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb,
                int64_t k_sh, int64_t k_sl, int64_t cs_sb, int64_t cs_sh, int64_t cs_sg, int32_t group_rows,
                float scale, int32_t* dev_status, uint64_t wait_limit_ns, lvar_stream_t stream);

/* Per-KV-block scores: out[r, j] = sum of cs[r, j*block : (j+1)*block] (columns past Lkv count as 0),
 * r over `rows` = B*H*G rows of cs spaced cs_row_stride elements apart; out is [rows, ceil(Lkv/block)]
 * contiguous.  Fixed summation order.  Feeds the block top-k that the benchmark's mask recipe and a
 * block-level version of the decision step (models/sparvar/sparse_attn.py:1012-1016) need. */
int lvar_block_scores(const float* cs, float* out, int64_t rows, int32_t Lkv, int32_t block,
                      int64_t cs_row_stride, lvar_stream_t stream);

/* Block mask = always-kept blocks U the highest-scoring remaining blocks, so that every row has
 * max(k_total, |always|) active blocks.  scores fp32 [BH, nq, nk]; always uint8 [nq, nk] or NULL;
 * mask uint8 [BH, nq, nk] out; optional lists int32 [BH, nq, nk] (active block ids ascending, tail -1)
 * and counts int32 [BH, nq].  Descending score, lower block index wins a tie.
 * The block-level counterpart of the reference's sink + local-window + top-k policy
 * (models/sparvar/basic_sparvar.py:109-173, models/sparvar/sparse_attn.py:1012-1036). */
int lvar_build_block_mask(const float* scores, const uint8_t* always, uint8_t* mask, int32_t* lists,
                          int32_t* counts, int64_t BH, int32_t nq, int32_t nk, int32_t k_total,
                          lvar_stream_t stream);

/* lvar_block_scores + lvar_build_block_mask in one pass over the column sums: cs fp32 [BH*nq, Lkv] (rows
 * cs_row_stride elements apart) -> mask uint8 [BH, nq, nk], nk = ceil(Lkv / block), with the same selection rule
 * and the same bits in the block scores (scores_out, optional fp32 [BH, nq, nk]; lists / counts optional as in
 * lvar_build_block_mask).  The column sums are read once and no score tensor has to exist in between. */
int lvar_block_mask_from_colsums(const float* cs, int64_t cs_row_stride, const uint8_t* always, uint8_t* mask,
                                 float* scores_out, int32_t* lists, int32_t* counts, int64_t BH, int32_t nq,
                                 int32_t Lkv, int32_t block, int32_t k_total, lvar_stream_t stream);

/* Exact, deterministic top-k of each row of an fp32 matrix [rows, n] (row_stride elements apart).
 * out int32 [rows, out_cols] (out_stride apart): the first k entries are the selected column ids,
 * descending by value with equal values in ascending index order, or, if ascending_index != 0, the
 * same set sorted by index; entries k..out_cols-1 are set to 0.  counts (optional, int32 [rows]) is
 * set to count_value.  Shared memory bounds the row: 4*n + 8*nextpow2(k) <= 204800 bytes.
 * Replaces torch.topk(bs, k, dim=-1).indices + the padding that follows it
 * (models/sparvar/sparse_attn.py:1016-1036) and the approximate torch.ops.chipmunk.topk_indices
 * (kernels/chipmunk/csrc/indexed_io/topk_indices.cu:145-218). */
int lvar_topk_indices(const float* scores, int64_t rows, int32_t n, int64_t row_stride, int32_t k,
                      int32_t ascending_index, int32_t* out, int64_t out_stride, int32_t out_cols,
                      int32_t* counts, int32_t count_value, lvar_stream_t stream);

/* bool/uint8 mask [rows, n] -> index lists int32 [rows, pad_n] and counts int32 [rows]; same list
 * order and padding rule as torch.ops.chipmunk.mask_to_indices
 * (kernels/chipmunk/csrc/indexed_io/mask_to_indices.cu:21-142): grouped by (column mod 32), count
 * rounded up to multiple_of with the first unset columns.  Entries past the count are not written. */
int lvar_mask_to_indices(const uint8_t* mask, int32_t* indices, int32_t* counts, int64_t rows, int32_t n,
                         int32_t pad_n, int32_t multiple_of, lvar_stream_t stream);

/* Little-endian bit packing of n_bits bool bytes into ceil(n_bits/8) bytes, and its inverse
 * (kernels/sparse_attn/sparse_attn_ops.py:300-366). */
int lvar_bitpack(const uint8_t* mask, uint8_t* packed, int64_t n_bits, lvar_stream_t stream);
int lvar_bitunpack(const uint8_t* packed, uint8_t* mask, int64_t n_bits, lvar_stream_t stream);

/* Key lists of a sparse step from the decision-scale lists: for each target query group g the list of
 * source group remap[g] (first cnt entries, clamped to [0, k_len); a source list shorter than cnt is
 * stretched by repeating each entry), then the scale's static local band band[g, 0:band_count];
 * out int32 [BH, Gk, out_cols] (tail 0), counts int32 [BH, Gk] = count_value (the reference writes
 * the unrounded source count + band_count there, cnt being that source count rounded up to the list padding).
 * src int32 [BH, Gs, >= src_cols] with the given strides; remap int32 [Gk]; band int32 [Gk, band_count].
 * One pass on the device instead of the reference's index_select / repeat_interleave / clamp / two
 * torch.cat with a host read of the count (models/sparvar/sparse_attn.py:365-421 and 1056-1121). */
int lvar_sparse_step_lists(const int32_t* src, const int32_t* remap, const int32_t* band, int32_t* out,
                           int32_t* counts, int64_t BH, int32_t Gs, int32_t src_cols, int64_t src_g_stride,
                           int64_t src_bh_stride, int32_t Gk, int32_t cnt, int32_t band_count, int32_t k_len,
                           int32_t out_cols, int32_t count_value, lvar_stream_t stream);

/* ScaleKV cache compaction (models/scalekv/scale_kv.py:163-301, ScaleKVCluster.update_kv), device part.
 * window: int32 [w] distinct key indices of the current scale's window grid (same for every batch and head).
 *
 * lvar_scalekv_scores: scores fp32 [B*H, Lkv] = sum over the w window queries (query row
 * clamp(window[i] - offset, 0, Lq-1)) of bf16(bf16(q_i . k_j) / sqrt(D)), rounded to bf16, -inf on the
 * window's own columns: the reference's matmul / sqrt(head_dim), masked_fill(-inf) and sum(dim=2) on bf16
 * tensors (scale_kv.py:245-253).
 * lvar_scalekv_pool: pooled fp32 [rows, Lkv] = max_pool1d / avg_pool1d(scores, ksize, padding ksize/2,
 * stride 1) (scale_kv.py:255-258) with the window columns then set to +inf, so that
 * lvar_topk_indices(pooled, k = max_capacity, ascending_index = 1) yields the reference's
 * sort(cat(top-(max_capacity - w) of the non-window columns, window)) (scale_kv.py:260-276).
 * lvar_gather_rows: dst bf16 [B,H,n,D] contiguous = src[b,h,clamp(idx[b*H+h, i]),:] (scale_kv.py:288-294);
 * idx int32 rows of idx_row_stride entries.  q, k, src: bf16 with element strides, last dim contiguous. */
int lvar_scalekv_scores(const void* q, const void* k, const int32_t* window, float* scores, int32_t B, int32_t H,
                        int32_t Lq, int32_t Lkv, int32_t D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb,
                        int64_t k_sh, int64_t k_sl, int32_t w, int32_t offset, lvar_stream_t stream);
int lvar_scalekv_pool(const float* scores, const int32_t* window, int32_t w, float* pooled, int64_t rows, int32_t Lkv,
                      int32_t ksize, int32_t avg, lvar_stream_t stream);
int lvar_gather_rows(const void* src, const int32_t* idx, void* dst, int32_t B, int32_t H, int32_t L, int32_t n,
                     int32_t D, int64_t s_sb, int64_t s_sh, int64_t s_sl, int64_t idx_row_stride, lvar_stream_t stream);

/* QKV prologue of a self-attention layer during generation, fused: L2-normalise q and k over the head
 * dimension (eps 1e-12), scale q by scale_mul[h], rotate both with the 2-D RoPE table rows
 * rope_start .. rope_start+L-1 (cos/sin fp32 [*, c/2], pairs (2i, 2i+1)), write q as bf16 [B,H,L,c] and append
 * k and v at row cache_pos of bf16 caches [B,H,cap,c] (models/sparvar/basic_sparvar.py:321-350: F.normalize,
 * .mul(scale_mul), apply_rotary_emb, torch.cat onto cached_k / cached_v, and the q.to(v.dtype) / k.to(v.dtype)
 * at the attention call sites :371-384; models/infinity/basic_infinity.py:111-133).
 * qkv: bf16 projection output, element (b, l, which, h, e) at b*s_b + l*s_l + which*s_w + h*s_h + e.
 * scale_mul NULL: no normalisation and no scale (cos_attn off); rope_cos/rope_sin NULL: no rotation. */
int lvar_qkv_prologue(const void* qkv, int64_t s_b, int64_t s_l, int64_t s_w, int64_t s_h, const float* scale_mul,
                      const float* rope_cos, const float* rope_sin, int32_t rope_start, void* q_out, int64_t q_sb,
                      int64_t q_sh, int64_t q_sl, void* k_cache, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                      void* v_cache, int64_t v_sb, int64_t v_sh, int64_t v_sl, int32_t cache_pos, int32_t B, int32_t L,
                      int32_t H, int32_t c, lvar_stream_t stream);

/* Bilinear (align_corners = false) resize of an attention-output cache between two square token grids:
 * src bf16 [BH, src_side^2, D] -> dst bf16 [BH, dst_side^2, D] (strides in elements, D a multiple of 8).
 * Replaces upsample_Ocache(o, L_src, L_tgt, mode='2d', upsample_mode='bilinear')
 * (models/sparvar/sparse_attn.py:324-362), which reshapes and calls F.interpolate. */
int lvar_upsample_ocache(const void* src, void* dst, int64_t BH, int32_t src_side, int32_t dst_side, int32_t D,
                         int64_t src_bh_stride, int64_t src_row_stride, int64_t dst_bh_stride,
                         int64_t dst_row_stride, lvar_stream_t stream);

/* Largest B*H*Lq the allocation-free entry point below accepts. */
#define LVAR_STATIC_MAX_ROWS 262144

/* Dense attention plus attention column sums WITHOUT any caller- or library-side allocation:
 * o = softmax(q k^T * scale) v and cs[b,h,g,j] = sum over the rows of query group g of the softmax
 * column j (same definitions, layouts and bit patterns as lvar_dense_attn followed by lvar_colsum).
 * This entry point has no counterpart in the reference; it exists for hosts that cannot call
 * cudaMalloc on the attention path (all HBM owned by their own pool, or a no-allocation-after-warm-up
 * rule): the row statistics that connect the two kernels and the attention kernel's work counter
 * live in a device array that is part of the library image.
 *   - Limit: B*H*Lq <= LVAR_STATIC_MAX_ROWS, else LVAR_ERR_LIMIT and nothing is launched.  Every GPU
 *     that loads the library holds that array (2 MiB + 256 B) until the process exits.
 *   - All calls on a device share the array and it keeps the last call's contents; the call clears
 *     the one word that must start at zero on `stream`.  Calls that can overlap on the GPU race:
 *     order them (same stream, or events).
 *   - The first call on each device resolves the array's address and sets kernel attributes; make it
 *     before any stream capture.
 * Calls no cudaMalloc / cudaFree and no allocating library routine. */
int lvar_dense_colsum_attn_static(const void* q, const void* k, const void* v, void* o, float* cs, int32_t B,
                                  int32_t H, int32_t Lq, int32_t Lkv, int32_t D, int64_t q_sb, int64_t q_sh,
                                  int64_t q_sl, int64_t k_sb, int64_t k_sh, int64_t k_sl, int64_t v_sb,
                                  int64_t v_sh, int64_t v_sl, int64_t o_sb, int64_t o_sh, int64_t o_sl,
                                  int64_t cs_sb, int64_t cs_sh, int64_t cs_sg, int32_t group_rows, float scale,
                                  int32_t* dev_status, uint64_t wait_limit_ns, lvar_stream_t stream);

/* Message of the calling thread's most recent failing call ("" if none). Never NULL. */
const char* lvar_last_error(void);

/* Library version, e.g. "0.1.0". */
const char* lvar_version(void);

/* Tile geometry callers must respect, the counterpart of get_kernel_config_attn()
 * (kernels/sparse_attn/sparse_attn_config.py:82-98). */
void lvar_kernel_config_attn(int32_t* bm, int32_t* counts_multiple_of, int32_t* indices_pad_to);

#ifdef __cplusplus
}
#endif

#endif /* LVAR_B200_H_ */
