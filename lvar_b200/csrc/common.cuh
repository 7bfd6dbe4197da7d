// Host-side helpers shared by the launchers: error codes of the C ABI, TMA descriptor encoding
// through the driver entry point (no link-time dependency on libcuda), and small checks.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lvar_b200.h"

namespace lvar {

// Sets the thread-local message returned by lvar_last_error() and hands back `code`.
int fail(int code, const char* fmt, ...);

#define LVAR_REQUIRE(cond, code, ...) \
  do {                                \
    if (!(cond)) return ::lvar::fail((code), __VA_ARGS__); \
  } while (0)

#define LVAR_CUDA_OK(expr)                                                               \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess)                                                               \
      return ::lvar::fail(LVAR_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

// Encodes a 4-D bf16 tensor map over a [B, H, L, D] view (D contiguous) with a
// [1, 1, box_rows, 64] box and 128-byte swizzle; out-of-range rows read as zeros.
// Strides are in elements.  Returns an LVAR_* code.
int encode_bhld_map(CUtensorMap* out, const void* base, int B, int H, int L, int D, int64_t sb, int64_t sh,
                    int64_t sl, int box_rows);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Bilinear resize between two square token grids (align_corners = False): the four source tokens and the
// weights of output pixel (y, x) of a side-t grid read from a side-s grid, ratio = s / t.  The stand-alone
// resize kernel and the column-sparse attention epilogue share these two functions, so that both give the
// same bits.
struct BilinearTaps {
  int r00, r01, r10, r11;  // source token indices (row-major in the side-s grid)
  float hy, ly, hx, lx;    // weights of the upper / lower row and of the left / right column
};

__device__ __forceinline__ BilinearTaps bilinear_taps(int y, int x, int s, float ratio) {
  // source coordinate: ratio * (dst + 0.5) - 0.5, clamped at 0
  const float fy = fmaxf(ratio * (y + 0.5f) - 0.5f, 0.f);
  const float fx = fmaxf(ratio * (x + 0.5f) - 0.5f, 0.f);
  const int y0 = min((int)fy, s - 1), x0 = min((int)fx, s - 1);
  const int y1 = min(y0 + 1, s - 1), x1 = min(x0 + 1, s - 1);
  BilinearTaps t;
  t.r00 = y0 * s + x0;
  t.r01 = y0 * s + x1;
  t.r10 = y1 * s + x0;
  t.r11 = y1 * s + x1;
  t.ly = fy - (float)y0;
  t.lx = fx - (float)x0;
  t.hy = 1.f - t.ly;
  t.hx = 1.f - t.lx;
  return t;
}

// hy * (hx * a + lx * b) + ly * (hx * c + lx * d) with the roundings written out
__device__ __forceinline__ float bilinear_mix(const BilinearTaps& t, float a, float b, float c, float d) {
  const float top = fmaf(t.lx, b, __fmul_rn(t.hx, a));
  const float bot = fmaf(t.lx, d, __fmul_rn(t.hx, c));
  return fmaf(t.ly, bot, __fmul_rn(t.hy, top));
}

// The same for 8 bf16 channels held in a uint4 per source token; the result is rounded to bf16 once.
__device__ __forceinline__ uint4 bilinear_mix8(const BilinearTaps& t, const uint4& a, const uint4& b, const uint4& c,
                                               const uint4& d) {
  const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
  const uint32_t cv[4] = {c.x, c.y, c.z, c.w}, dv[4] = {d.x, d.y, d.z, d.w};
  uint32_t out[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float lo = bilinear_mix(t, __uint_as_float(av[j] << 16), __uint_as_float(bv[j] << 16),
                                  __uint_as_float(cv[j] << 16), __uint_as_float(dv[j] << 16));
    const float hi = bilinear_mix(t, __uint_as_float(av[j] & 0xffff0000u), __uint_as_float(bv[j] & 0xffff0000u),
                                  __uint_as_float(cv[j] & 0xffff0000u), __uint_as_float(dv[j] & 0xffff0000u));
    const __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
    out[j] = *reinterpret_cast<const uint32_t*>(&pk);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

}  // namespace lvar
