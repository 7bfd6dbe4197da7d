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
    // source index: ratio * (dst + 0.5) - 0.5, clamped at 0
    const float fy = fmaxf(ratio * (y + 0.5f) - 0.5f, 0.f);
    const float fx = fmaxf(ratio * (x + 0.5f) - 0.5f, 0.f);
    const int y0 = min((int)fy, s - 1), x0 = min((int)fx, s - 1);
    const int y1 = min(y0 + 1, s - 1), x1 = min(x0 + 1, s - 1);
    const float ly = fy - (float)y0, lx = fx - (float)x0;
    const float hy = 1.f - ly, hx = 1.f - lx;
    const __nv_bfloat16* base = src + bh * src_bh_stride + c * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(base + (int64_t)(y0 * s + x0) * src_row_stride);
    const uint4 b = *reinterpret_cast<const uint4*>(base + (int64_t)(y0 * s + x1) * src_row_stride);
    const uint4 cc = *reinterpret_cast<const uint4*>(base + (int64_t)(y1 * s + x0) * src_row_stride);
    const uint4 d = *reinterpret_cast<const uint4*>(base + (int64_t)(y1 * s + x1) * src_row_stride);
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
    const uint32_t cv[4] = {cc.x, cc.y, cc.z, cc.w}, dv[4] = {d.x, d.y, d.z, d.w};
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float r[2];
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        const float va = __uint_as_float(hlf ? (av[j] & 0xffff0000u) : (av[j] << 16));
        const float vb = __uint_as_float(hlf ? (bv[j] & 0xffff0000u) : (bv[j] << 16));
        const float vc = __uint_as_float(hlf ? (cv[j] & 0xffff0000u) : (cv[j] << 16));
        const float vd = __uint_as_float(hlf ? (dv[j] & 0xffff0000u) : (dv[j] << 16));
        r[hlf] = hy * (hx * va + lx * vb) + ly * (hx * vc + lx * vd);
      }
      const __nv_bfloat162 pk = __floats2bfloat162_rn(r[0], r[1]);
      out[j] = *reinterpret_cast<const uint32_t*>(&pk);
    }
    *reinterpret_cast<uint4*>(dst + bh * dst_bh_stride + (int64_t)(y * t + x) * dst_row_stride + c * 8) =
        make_uint4(out[0], out[1], out[2], out[3]);
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
