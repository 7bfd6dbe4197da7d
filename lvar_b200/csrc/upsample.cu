// Bilinear resize of an attention-output cache between two square token grids, bf16 in / bf16 out:
// the O-cache upsample of the column-sparse policy (upsample_Ocache, mode '2d', 'bilinear',
// align_corners=False, models/sparvar/sparse_attn.py:324-362).  [B,H,s*s,D] -> [B,H,t*t,D].
// HBM-bound: every output row is written once; the four source rows of a pixel come from a cache
// that is t^2/s^2 times smaller and stays in L2.  One thread produces 8 channels (16 bytes) of one
// output token; interpolation in fp32, one rounding to bf16 at the end (as PyTorch does for bf16 input).
#include "common.cuh"

namespace lvar {

namespace {

__global__ void upsample_ocache_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                       int64_t BH, int s, int t, int D, int64_t src_bh_stride, int64_t src_row_stride,
                                       int64_t dst_bh_stride, int64_t dst_row_stride, float ratio) {
  const int chunks = D / 8;
  const int64_t total = BH * t * t * chunks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % chunks);
    const int64_t pix = i / chunks;
    const int x = (int)(pix % t);
    const int y = (int)((pix / t) % t);
    const int64_t bh = pix / ((int64_t)t * t);
    const BilinearTaps tp = bilinear_taps(y, x, s, ratio);
    const __nv_bfloat16* base = src + bh * src_bh_stride + c * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(base + (int64_t)tp.r00 * src_row_stride);
    const uint4 b = *reinterpret_cast<const uint4*>(base + (int64_t)tp.r01 * src_row_stride);
    const uint4 cc = *reinterpret_cast<const uint4*>(base + (int64_t)tp.r10 * src_row_stride);
    const uint4 d = *reinterpret_cast<const uint4*>(base + (int64_t)tp.r11 * src_row_stride);
    *reinterpret_cast<uint4*>(dst + bh * dst_bh_stride + (int64_t)(y * t + x) * dst_row_stride + c * 8) =
        bilinear_mix8(tp, a, b, cc, d);
  }
}

}  // namespace

int launch_upsample_ocache(const void* src, void* dst, int64_t BH, int src_side, int dst_side, int D,
                           int64_t src_bh_stride, int64_t src_row_stride, int64_t dst_bh_stride,
                           int64_t dst_row_stride, cudaStream_t stream) {
  LVAR_REQUIRE(src && dst, LVAR_ERR_ARG, "src and dst must be non-null");
  LVAR_REQUIRE(BH >= 1 && src_side >= 1 && dst_side >= 1, LVAR_ERR_ARG, "BH and the grid sides must be >= 1");
  LVAR_REQUIRE(D >= 8 && D % 8 == 0, LVAR_ERR_ARG, "D must be a positive multiple of 8");
  LVAR_REQUIRE(aligned16(src) && aligned16(dst), LVAR_ERR_ARG, "src and dst must be 16-byte aligned");
  const int64_t strides[] = {src_bh_stride, src_row_stride, dst_bh_stride, dst_row_stride};
  for (int64_t s : strides) LVAR_REQUIRE(s % 8 == 0 && s >= 0, LVAR_ERR_ARG, "strides must be multiples of 8 elements");
  const int64_t total = BH * dst_side * dst_side * (D / 8);
  int dev = 0, sms = 0;
  LVAR_CUDA_OK(cudaGetDevice(&dev));
  LVAR_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  int64_t blocks = (total + 255) / 256;
  if (blocks > (int64_t)sms * 16) blocks = (int64_t)sms * 16;
  upsample_ocache_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), BH, src_side, dst_side, D,
      src_bh_stride, src_row_stride, dst_bh_stride, dst_row_stride, (float)src_side / (float)dst_side);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

}  // namespace lvar
