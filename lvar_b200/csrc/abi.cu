// extern "C" surface of the library (declared in include/lvar_b200.h) plus the host helpers the
// launchers share.  No torch types cross this boundary.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace lvar {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point: no link-time libcuda dependency.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

int encode_bhld_map(CUtensorMap* out, const void* base, int B, int H, int L, int D, int64_t sb, int64_t sh,
                    int64_t sl, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  LVAR_REQUIRE(fn != nullptr, LVAR_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available (no CUDA driver?)");
  // A stride of zero is not encodable; size-1 dimensions get a harmless dummy stride.
  const cuuint64_t row_bytes = (cuuint64_t)D * 2;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t st_l = (cuuint64_t)sl * 2, st_h = (cuuint64_t)sh * 2, st_b = (cuuint64_t)sb * 2;
  if (L == 1 && st_l == 0) st_l = row_bytes;
  if (H == 1 && st_h == 0) st_h = st_l * (cuuint64_t)L;
  if (B == 1 && st_b == 0) st_b = st_h * (cuuint64_t)H;
  LVAR_REQUIRE(st_l >= row_bytes && st_h > 0 && st_b > 0, LVAR_ERR_ARG,
               "tensor strides must be positive (got l=%lld h=%lld b=%lld elements)", (long long)sl, (long long)sh,
               (long long)sb);
  cuuint64_t strides[3] = {st_l, st_h, st_b};
  cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, 1u, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  LVAR_REQUIRE(r == CUDA_SUCCESS, LVAR_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return LVAR_OK;
}

int launch_attention(const lvar_attn_args* a, int mode, cudaStream_t stream);
int launch_colsum(const void* q, const void* k, const float* M, const float* L, float* cs, int B, int H, int Lq,
                  int Lkv, int D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                  int64_t cs_sb, int64_t cs_sh, int64_t cs_sg, int group_rows, float scale, int* dev_status,
                  uint64_t wait_limit_ns, cudaStream_t stream);

int launch_block_scores(const float* cs, float* out, int64_t rows, int Lkv, int block, int64_t cs_row_stride,
                        cudaStream_t stream);
int launch_build_block_mask(const float* scores, const uint8_t* always, uint8_t* mask, int32_t* lists,
                            int32_t* counts, int64_t BH, int nq, int nk, int k_total, cudaStream_t stream);
int launch_block_mask_from_colsums(const float* cs, int64_t cs_row_stride, const uint8_t* always, uint8_t* mask,
                                   float* scores_out, int32_t* lists, int32_t* counts, int64_t BH, int nq, int Lkv,
                                   int block, int k_total, cudaStream_t stream);
int launch_topk(const float* scores, int64_t rows, int n, int64_t row_stride, int k, int ascending_index,
                int32_t* out, int64_t out_stride, int out_cols, int32_t* counts, int count_value,
                cudaStream_t stream);
int launch_mask_to_indices(const uint8_t* mask, int32_t* indices, int32_t* counts, int64_t rows, int n, int pad_n,
                           int multiple_of, cudaStream_t stream);
int launch_bitpack(const uint8_t* mask, uint8_t* packed, int64_t n_bits, cudaStream_t stream);
int launch_bitunpack(const uint8_t* packed, uint8_t* mask, int64_t n_bits, cudaStream_t stream);

int launch_sparse_step_lists(const int32_t* src, const int32_t* remap, const int32_t* band, int32_t* out,
                             int32_t* counts, int64_t BH, int Gs, int src_cols, int64_t src_g_stride,
                             int64_t src_bh_stride, int Gk, int cnt, int band_count, int k_len, int out_cols,
                             int count_value, cudaStream_t stream);
int launch_scalekv_scores(const void* q, const void* k, const int32_t* window, float* scores, int B, int H, int Lq,
                          int Lkv, int D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb, int64_t k_sh,
                          int64_t k_sl, int w, int offset, cudaStream_t stream);
int launch_scalekv_pool(const float* scores, const int32_t* window, int w, float* pooled, int64_t rows, int Lkv,
                        int ksize, int avg, cudaStream_t stream);
int launch_gather_rows(const void* src, const int32_t* idx, void* dst, int B, int H, int L, int n, int D, int64_t s_sb,
                       int64_t s_sh, int64_t s_sl, int64_t idx_row_stride, cudaStream_t stream);
int launch_qkv_prologue(const void* qkv, int64_t s_b, int64_t s_l, int64_t s_w, int64_t s_h, const float* scale_mul,
                        const float* rope_cos, const float* rope_sin, int rope_start, void* q_out, int64_t q_sb,
                        int64_t q_sh, int64_t q_sl, void* k_cache, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                        void* v_cache, int64_t v_sb, int64_t v_sh, int64_t v_sl, int cache_pos, int B, int L, int H,
                        int c, cudaStream_t stream);
int launch_upsample_ocache(const void* src, void* dst, int64_t BH, int src_side, int dst_side, int D,
                           int64_t src_bh_stride, int64_t src_row_stride, int64_t dst_bh_stride,
                           int64_t dst_row_stride, cudaStream_t stream);

}  // namespace lvar

extern "C" {

int lvar_sparse_step_lists(const int32_t* src, const int32_t* remap, const int32_t* band, int32_t* out,
                           int32_t* counts, int64_t BH, int32_t Gs, int32_t src_cols, int64_t src_g_stride,
                           int64_t src_bh_stride, int32_t Gk, int32_t cnt, int32_t band_count, int32_t k_len,
                           int32_t out_cols, int32_t count_value, lvar_stream_t stream) {
  return lvar::launch_sparse_step_lists(src, remap, band, out, counts, BH, Gs, src_cols, src_g_stride, src_bh_stride,
                                        Gk, cnt, band_count, k_len, out_cols, count_value, static_cast<cudaStream_t>(stream));
}

int lvar_scalekv_scores(const void* q, const void* k, const int32_t* window, float* scores, int32_t B, int32_t H,
                        int32_t Lq, int32_t Lkv, int32_t D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb,
                        int64_t k_sh, int64_t k_sl, int32_t w, int32_t offset, lvar_stream_t stream) {
  return lvar::launch_scalekv_scores(q, k, window, scores, B, H, Lq, Lkv, D, q_sb, q_sh, q_sl, k_sb, k_sh, k_sl, w, offset,
                                     static_cast<cudaStream_t>(stream));
}

int lvar_scalekv_pool(const float* scores, const int32_t* window, int32_t w, float* pooled, int64_t rows, int32_t Lkv,
                      int32_t ksize, int32_t avg, lvar_stream_t stream) {
  return lvar::launch_scalekv_pool(scores, window, w, pooled, rows, Lkv, ksize, avg, static_cast<cudaStream_t>(stream));
}

int lvar_gather_rows(const void* src, const int32_t* idx, void* dst, int32_t B, int32_t H, int32_t L, int32_t n,
                     int32_t D, int64_t s_sb, int64_t s_sh, int64_t s_sl, int64_t idx_row_stride, lvar_stream_t stream) {
  return lvar::launch_gather_rows(src, idx, dst, B, H, L, n, D, s_sb, s_sh, s_sl, idx_row_stride,
                                  static_cast<cudaStream_t>(stream));
}

int lvar_qkv_prologue(const void* qkv, int64_t s_b, int64_t s_l, int64_t s_w, int64_t s_h, const float* scale_mul,
                      const float* rope_cos, const float* rope_sin, int32_t rope_start, void* q_out, int64_t q_sb,
                      int64_t q_sh, int64_t q_sl, void* k_cache, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                      void* v_cache, int64_t v_sb, int64_t v_sh, int64_t v_sl, int32_t cache_pos, int32_t B, int32_t L,
                      int32_t H, int32_t c, lvar_stream_t stream) {
  return lvar::launch_qkv_prologue(qkv, s_b, s_l, s_w, s_h, scale_mul, rope_cos, rope_sin, rope_start, q_out, q_sb, q_sh,
                                   q_sl, k_cache, k_sb, k_sh, k_sl, v_cache, v_sb, v_sh, v_sl, cache_pos, B, L, H, c,
                                   static_cast<cudaStream_t>(stream));
}

int lvar_upsample_ocache(const void* src, void* dst, int64_t BH, int32_t src_side, int32_t dst_side, int32_t D,
                         int64_t src_bh_stride, int64_t src_row_stride, int64_t dst_bh_stride,
                         int64_t dst_row_stride, lvar_stream_t stream) {
  return lvar::launch_upsample_ocache(src, dst, BH, src_side, dst_side, D, src_bh_stride, src_row_stride,
                                      dst_bh_stride, dst_row_stride, static_cast<cudaStream_t>(stream));
}

int lvar_dense_attn(const lvar_attn_args* args, lvar_stream_t stream) {
  return lvar::launch_attention(args, 0, static_cast<cudaStream_t>(stream));
}

int lvar_dense_colsum_attn(const lvar_attn_args* args, lvar_stream_t stream) {
  return lvar::launch_attention(args, 3, static_cast<cudaStream_t>(stream));
}

int lvar_dense_colsum_attn_given(const lvar_attn_args* args, lvar_stream_t stream) {
  return lvar::launch_attention(args, 6, static_cast<cudaStream_t>(stream));
}

int lvar_colsum_tiles(const lvar_attn_args* args, int32_t stats_given, lvar_stream_t stream) {
  return lvar::launch_attention(args, stats_given ? 5 : 4, static_cast<cudaStream_t>(stream));
}

int lvar_block_sparse_attn(const lvar_attn_args* args, lvar_stream_t stream) {
  return lvar::launch_attention(args, 1, static_cast<cudaStream_t>(stream));
}

int lvar_csp_attn(const lvar_attn_args* args, lvar_stream_t stream) {
  return lvar::launch_attention(args, 2, static_cast<cudaStream_t>(stream));
}

int lvar_colsum(const void* q, const void* k, const float* M, const float* L, float* cs, int32_t B, int32_t H,
                int32_t Lq, int32_t Lkv, int32_t D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb,
                int64_t k_sh, int64_t k_sl, int64_t cs_sb, int64_t cs_sh, int64_t cs_sg, int32_t group_rows,
                float scale, int32_t* dev_status, uint64_t wait_limit_ns, lvar_stream_t stream) {
  return lvar::launch_colsum(q, k, M, L, cs, B, H, Lq, Lkv, D, q_sb, q_sh, q_sl, k_sb, k_sh, k_sl, cs_sb, cs_sh,
                             cs_sg, group_rows, scale, dev_status, wait_limit_ns, static_cast<cudaStream_t>(stream));
}

int lvar_block_scores(const float* cs, float* out, int64_t rows, int32_t Lkv, int32_t block,
                      int64_t cs_row_stride, lvar_stream_t stream) {
  return lvar::launch_block_scores(cs, out, rows, Lkv, block, cs_row_stride, static_cast<cudaStream_t>(stream));
}

int lvar_build_block_mask(const float* scores, const uint8_t* always, uint8_t* mask, int32_t* lists,
                          int32_t* counts, int64_t BH, int32_t nq, int32_t nk, int32_t k_total,
                          lvar_stream_t stream) {
  return lvar::launch_build_block_mask(scores, always, mask, lists, counts, BH, nq, nk, k_total,
                                       static_cast<cudaStream_t>(stream));
}

int lvar_block_mask_from_colsums(const float* cs, int64_t cs_row_stride, const uint8_t* always, uint8_t* mask,
                                 float* scores_out, int32_t* lists, int32_t* counts, int64_t BH, int32_t nq,
                                 int32_t Lkv, int32_t block, int32_t k_total, lvar_stream_t stream) {
  return lvar::launch_block_mask_from_colsums(cs, cs_row_stride, always, mask, scores_out, lists, counts, BH, nq, Lkv,
                                              block, k_total, static_cast<cudaStream_t>(stream));
}

int lvar_topk_indices(const float* scores, int64_t rows, int32_t n, int64_t row_stride, int32_t k,
                      int32_t ascending_index, int32_t* out, int64_t out_stride, int32_t out_cols,
                      int32_t* counts, int32_t count_value, lvar_stream_t stream) {
  return lvar::launch_topk(scores, rows, n, row_stride, k, ascending_index, out, out_stride, out_cols, counts,
                           count_value, static_cast<cudaStream_t>(stream));
}

int lvar_mask_to_indices(const uint8_t* mask, int32_t* indices, int32_t* counts, int64_t rows, int32_t n,
                         int32_t pad_n, int32_t multiple_of, lvar_stream_t stream) {
  return lvar::launch_mask_to_indices(mask, indices, counts, rows, n, pad_n, multiple_of,
                                      static_cast<cudaStream_t>(stream));
}

int lvar_bitpack(const uint8_t* mask, uint8_t* packed, int64_t n_bits, lvar_stream_t stream) {
  return lvar::launch_bitpack(mask, packed, n_bits, static_cast<cudaStream_t>(stream));
}

int lvar_bitunpack(const uint8_t* packed, uint8_t* mask, int64_t n_bits, lvar_stream_t stream) {
  return lvar::launch_bitunpack(packed, mask, n_bits, static_cast<cudaStream_t>(stream));
}

const char* lvar_last_error(void) { return lvar::g_err; }

const char* lvar_version(void) { return "0.1.0"; }

void lvar_kernel_config_attn(int32_t* bm, int32_t* counts_multiple_of, int32_t* indices_pad_to) {
  if (bm) *bm = 256;
  if (counts_multiple_of) *counts_multiple_of = 128;
  if (indices_pad_to) *indices_pad_to = 4;
}

}  // extern "C"
