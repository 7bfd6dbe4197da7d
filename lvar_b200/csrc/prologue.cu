// QKV prologue of a self-attention layer during generation (models/sparvar/basic_sparvar.py:321-350,
// models/infinity/basic_infinity.py:111-133), one HBM-bound pass instead of normalize, mul, stack, RoPE,
// two torch.cat of the whole KV cache and a cast of the cache at every attention call:
//   q_out[b,h,l,:]            = bf16( rope( q / max(|q|, 1e-12) * scale_mul[h] ) )
//   k_cache[b,h,pos + l,:]    = bf16( rope( k / max(|k|, 1e-12) ) )
//   v_cache[b,h,pos + l,:]    = v
// from the projection output qkv bf16 [B, L, 3, H, c].  All arithmetic in fp32 on the widened bf16 inputs,
// in the reference's order (division by the clamped norm, then the per-head scale, then the rotation with
// separate multiplies and add/subtract), one rounding to bf16 at the end: the reference keeps q and k in
// fp32 and casts them to v's dtype at every call site.
// rope(x)[2i] = cos[p,i] x[2i] - sin[p,i] x[2i+1],  rope(x)[2i+1] = sin[p,i] x[2i] + cos[p,i] x[2i+1],
// p = rope_start + l.  One warp per (b, l, h) row, two rows per iteration; a lane holds c/32 consecutive elements
// (whole pairs).
#include <math.h>

#include <type_traits>

#include "common.cuh"

namespace lvar {

namespace {

struct PrologueParams {
  const __nv_bfloat16* qkv;
  int64_t s_b, s_l, s_w, s_h;
  const float* scale_mul;  // [H] or nullptr (no normalisation at all: plain copy + optional RoPE)
  const float* cos_t;      // [*, c/2] or nullptr (no RoPE)
  const float* sin_t;
  int rope_start;
  __nv_bfloat16* q_out;
  int64_t q_sb, q_sh, q_sl;
  __nv_bfloat16* k_cache;
  int64_t k_sb, k_sh, k_sl;
  __nv_bfloat16* v_cache;
  int64_t v_sb, v_sh, v_sl;
  int cache_pos;
  int B, L, H;
};

template <int EPL>  // elements per lane: 2 (c = 64) or 4 (c = 128)
__global__ void __launch_bounds__(256) qkv_prologue_kernel(const PrologueParams p) {
  constexpr int C = EPL * 32;
  constexpr int ROWS = 2;  // (b, l, h) rows per warp and iteration: their nine loads are issued before any arithmetic
  using Vec = typename std::conditional<EPL == 4, uint2, uint32_t>::type;
  const int lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)p.B * p.L * p.H;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t row0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row0 < rows; row0 += warps * ROWS) {
    Vec raw[ROWS][3];
    int hh[ROWS], ll[ROWS], bb_[ROWS];
    float cs[ROWS][EPL / 2], sn[ROWS][EPL / 2];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int64_t row = row0 + r * warps;
      if (row >= rows) continue;
      hh[r] = (int)(row % p.H);
      ll[r] = (int)((row / p.H) % p.L);
      bb_[r] = (int)(row / ((int64_t)p.H * p.L));
      const __nv_bfloat16* src = p.qkv + bb_[r] * p.s_b + ll[r] * p.s_l + hh[r] * p.s_h + lane * EPL;
#pragma unroll
      for (int which = 0; which < 3; ++which) raw[r][which] = *reinterpret_cast<const Vec*>(src + which * p.s_w);
      if (p.cos_t != nullptr) {
        const int64_t base = (int64_t)(p.rope_start + ll[r]) * (C / 2) + (lane * EPL >> 1);
#pragma unroll
        for (int e = 0; e < EPL / 2; ++e) {
          cs[r][e] = p.cos_t[base + e];
          sn[r][e] = p.sin_t[base + e];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int64_t row = row0 + r * warps;
      if (row >= rows) continue;  // warp-uniform
      const int h = hh[r], l = ll[r], b = bb_[r];
#pragma unroll
      for (int which = 0; which < 3; ++which) {
        __nv_bfloat16 el[EPL];
        *reinterpret_cast<Vec*>(el) = raw[r][which];
        __nv_bfloat16* dst;
        if (which == 0) {
          dst = p.q_out + b * p.q_sb + h * p.q_sh + (int64_t)l * p.q_sl;
        } else if (which == 1) {
          dst = p.k_cache + b * p.k_sb + h * p.k_sh + (int64_t)(p.cache_pos + l) * p.k_sl;
        } else {
          dst = p.v_cache + b * p.v_sb + h * p.v_sh + (int64_t)(p.cache_pos + l) * p.v_sl;
        }
        dst += lane * EPL;
        if (which < 2) {
          float x[EPL];
#pragma unroll
          for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(el[e]);
          if (p.scale_mul != nullptr) {
            float ssq = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) ssq = fmaf(x[e], x[e], ssq);
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, d);
            const float denom = fmaxf(sqrtf(ssq), 1e-12f);
            const float mul = which == 0 ? p.scale_mul[h] : 1.0f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
              x[e] = __fdiv_rn(x[e], denom);
              if (which == 0) x[e] = __fmul_rn(x[e], mul);
            }
          }
          if (p.cos_t != nullptr) {
#pragma unroll
            for (int e = 0; e < EPL; e += 2) {
              const float c1 = cs[r][e >> 1], s1 = sn[r][e >> 1];
              const float a = x[e], b2 = x[e + 1];
              x[e] = __fsub_rn(__fmul_rn(c1, a), __fmul_rn(s1, b2));
              x[e + 1] = __fadd_rn(__fmul_rn(s1, a), __fmul_rn(c1, b2));
            }
          }
#pragma unroll
          for (int e = 0; e < EPL; ++e) el[e] = __float2bfloat16_rn(x[e]);
        }
        *reinterpret_cast<Vec*>(dst) = *reinterpret_cast<const Vec*>(el);
      }
    }
  }
}

}  // namespace

int launch_qkv_prologue(const void* qkv, int64_t s_b, int64_t s_l, int64_t s_w, int64_t s_h, const float* scale_mul,
                        const float* rope_cos, const float* rope_sin, int rope_start, void* q_out, int64_t q_sb,
                        int64_t q_sh, int64_t q_sl, void* k_cache, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                        void* v_cache, int64_t v_sb, int64_t v_sh, int64_t v_sl, int cache_pos, int B, int L, int H,
                        int c, cudaStream_t stream) {
  LVAR_REQUIRE(qkv && q_out && k_cache && v_cache, LVAR_ERR_ARG, "qkv, q_out, k_cache and v_cache must be non-null");
  LVAR_REQUIRE(c == 64 || c == 128, LVAR_ERR_UNSUPPORTED, "Head dimension must be 64 or 128 (got %d)", c);
  LVAR_REQUIRE(B >= 1 && L >= 1 && H >= 1 && cache_pos >= 0 && rope_start >= 0, LVAR_ERR_ARG, "bad sizes");
  LVAR_REQUIRE((rope_cos == nullptr) == (rope_sin == nullptr), LVAR_ERR_ARG, "rope_cos and rope_sin go together");
  const int64_t strides[] = {s_b, s_l, s_w, s_h, q_sb, q_sh, q_sl, k_sb, k_sh, k_sl, v_sb, v_sh, v_sl};
  for (int64_t s : strides) LVAR_REQUIRE(s % 4 == 0 && s >= 0, LVAR_ERR_ARG, "strides must be non-negative multiples of 4 elements");
  const uintptr_t ptrs[] = {(uintptr_t)qkv, (uintptr_t)q_out, (uintptr_t)k_cache, (uintptr_t)v_cache};
  for (uintptr_t a : ptrs) LVAR_REQUIRE(a % 8 == 0, LVAR_ERR_ARG, "tensors must be 8-byte aligned");
  PrologueParams p{};
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.s_b = s_b; p.s_l = s_l; p.s_w = s_w; p.s_h = s_h;
  p.scale_mul = scale_mul;
  p.cos_t = rope_cos; p.sin_t = rope_sin; p.rope_start = rope_start;
  p.q_out = static_cast<__nv_bfloat16*>(q_out); p.q_sb = q_sb; p.q_sh = q_sh; p.q_sl = q_sl;
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache); p.k_sb = k_sb; p.k_sh = k_sh; p.k_sl = k_sl;
  p.v_cache = static_cast<__nv_bfloat16*>(v_cache); p.v_sb = v_sb; p.v_sh = v_sh; p.v_sl = v_sl;
  p.cache_pos = cache_pos;
  p.B = B; p.L = L; p.H = H;
  const int64_t rows = (int64_t)B * L * H;
  int64_t blocks = (rows + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (c == 128) qkv_prologue_kernel<4><<<(unsigned)blocks, 256, 0, stream>>>(p);
  else qkv_prologue_kernel<2><<<(unsigned)blocks, 256, 0, stream>>>(p);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

}  // namespace lvar
