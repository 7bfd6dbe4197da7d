// Device helpers shared by the attention kernels: swizzled tile addressing, the cp.async row
// gather, and the register-level softmax pieces (3-input max, packed exp2 + bf16 packing).
#pragma once

#include "ptx.cuh"

namespace lvar {

// Swizzled byte offset of 16-byte chunk `c16` (0..D/8-1) of row `r` inside a [128][D] tile made of
// [128][64] sub-tiles with the 128-byte TMA swizzle.
__device__ __forceinline__ uint32_t sw128_offset(int r, int c16) {
  return (uint32_t)((c16 >> 3) * 16384 + r * 128 + (((c16 & 7) ^ (r & 7)) << 4));
}

// One warp gathers the 128 rows of KV tile `j` of an index list into a swizzled [128][D] tile with
// 16-byte cp.async copies.  List positions past `cnt` read row 0 (their P columns are zero).
template <int D>
__device__ __forceinline__ void gather_tile(uint32_t dst, const __nv_bfloat16* base, int64_t row_stride,
                                            const int32_t* idx, int cnt, int j, int Lkv, int lane, int* status) {
  constexpr int CH = D / 8;        // 16-byte chunks per row
  constexpr int RPP = 32 / CH;     // rows per warp pass
  const int c16 = lane % CH;
#pragma unroll 4
  for (int rr = 0; rr < 128; rr += RPP) {
    const int r = rr + lane / CH;
    const int pos = j * 128 + r;
    int kv = (pos < cnt) ? __ldg(idx + pos) : 0;
    if ((unsigned)kv >= (unsigned)Lkv) {
      if (status) atomicCAS(status, 0, (int)DEV_BAD_INDEX);
      kv = 0;
    }
    cp_async_16(dst + sw128_offset(r, c16), base + (int64_t)kv * row_stride + c16 * 8);
  }
}

// max of a 32-element chunk of raw fp32 bits with 3-input max instructions
__device__ __forceinline__ float chunk_max(const uint32_t (&r)[32]) {
  float m0 = fmax3(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]));
  float m1 = fmax3(__uint_as_float(r[3]), __uint_as_float(r[4]), __uint_as_float(r[5]));
#pragma unroll
  for (int i = 6; i < 30; i += 4) {
    m0 = fmax3(m0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
    m1 = fmax3(m1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
  }
  return fmax3(m0, m1, fmaxf(__uint_as_float(r[30]), __uint_as_float(r[31])));
}

// p = exp2(s * scale - m) for one 32-column chunk: packed FMA, row-sum accumulation in two packed
// accumulators, bf16x2 packing of the 32 probabilities into pk[off .. off+15].
__device__ __forceinline__ void exp_pack_chunk(const uint32_t (&r)[32], uint64_t sc2, uint64_t nm2, uint64_t& sum_a,
                                               uint64_t& sum_b, uint32_t (&pk)[32], int off) {
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const uint64_t t0 = ffma2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), sc2, nm2);
    const uint64_t t1 = ffma2(pack_f32x2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])), sc2, nm2);
    float a0, a1, b0, b1;
    unpack_f32x2(t0, a0, a1);
    unpack_f32x2(t1, b0, b1);
    a0 = fast_exp2(a0);
    a1 = fast_exp2(a1);
    b0 = fast_exp2(b0);
    b1 = fast_exp2(b1);
    sum_a = fadd2(sum_a, pack_f32x2(a0, a1));
    sum_b = fadd2(sum_b, pack_f32x2(b0, b1));
    pk[off + i / 2] = pack_bf16x2(a0, a1);
    pk[off + i / 2 + 1] = pack_bf16x2(b0, b1);
  }
}


// exp2 of two values on the FMA pipe (no MUFU): x = j + f with j = round(x), |f| <= 0.5; 2^f by a
// degree-4 minimax polynomial (relative error 2.7e-6), 2^j by adding j to the exponent field.
// Valid for -126 <= x <= 100; the caller guarantees the range (no masked, i.e. -inf, inputs).
__device__ __forceinline__ void exp2_poly_x2(uint64_t x2, float& o0, float& o1) {
  const uint64_t magic = pack_f32x2(12582912.f, 12582912.f);  // 1.5 * 2^23: low mantissa bits = round(x)
  const uint64_t neg_magic = pack_f32x2(-12582912.f, -12582912.f);
  const uint64_t t2 = fadd2(x2, magic);
  const uint64_t j2 = fadd2(t2, neg_magic);
  const uint64_t f2 = ffma2(j2, pack_f32x2(-1.f, -1.f), x2);
  uint64_t p2 = pack_f32x2(0.00957401655614376f, 0.00957401655614376f);
  p2 = ffma2(p2, f2, pack_f32x2(0.055918190628290176f, 0.055918190628290176f));
  p2 = ffma2(p2, f2, pack_f32x2(0.2402464896440506f, 0.2402464896440506f));
  p2 = ffma2(p2, f2, pack_f32x2(0.6931217312812805f, 0.6931217312812805f));
  p2 = ffma2(p2, f2, pack_f32x2(0.9999992847442627f, 0.9999992847442627f));
  float p0, p1, t0, t1;
  unpack_f32x2(p2, p0, p1);
  unpack_f32x2(t2, t0, t1);
  o0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  o1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

// Same as exp_pack_chunk with the exponentials evaluated on the FMA pipe; only for tiles without
// masked columns.  Inputs below 2^-126 are clamped (they contribute ~1e-38 instead of 0).
__device__ __forceinline__ void exp_pack_chunk_poly(const uint32_t (&r)[32], uint64_t sc2, uint64_t nm2,
                                                    uint64_t& sum_a, uint64_t& sum_b, uint32_t (&pk)[32], int off) {
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const uint64_t t0 = ffma2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), sc2, nm2);
    const uint64_t t1 = ffma2(pack_f32x2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])), sc2, nm2);
    float a0, a1, b0, b1;
    unpack_f32x2(t0, a0, a1);
    unpack_f32x2(t1, b0, b1);
    exp2_poly_x2(pack_f32x2(fmaxf(a0, -126.f), fmaxf(a1, -126.f)), a0, a1);
    exp2_poly_x2(pack_f32x2(fmaxf(b0, -126.f), fmaxf(b1, -126.f)), b0, b1);
    sum_a = fadd2(sum_a, pack_f32x2(a0, a1));
    sum_b = fadd2(sum_b, pack_f32x2(b0, b1));
    pk[off + i / 2] = pack_bf16x2(a0, a1);
    pk[off + i / 2 + 1] = pack_bf16x2(b0, b1);
  }
}

}  // namespace lvar
