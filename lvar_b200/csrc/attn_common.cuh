// Device helpers shared by the attention kernels: the cp.async row gather into a swizzled tile and the
// register-level softmax pieces (3-input max, packed exp2 + bf16 packing).
#pragma once

#include "ptx.cuh"

namespace lvar {

// Column-sparse attention gathers the 128 rows of KV tile `j` of an index list into a swizzled [128][D]
// tile with 16-byte cp.async copies, one warp per tile.  The tile's 128 indices are read first, coalesced
// (lane l holds those of rows l, l+32, l+64, l+96; gather_rows_of_tile, which the loaders call one tile ahead
// so that the index latency is off the critical path).  gather_tile then copies 8 rows per instruction:
// four lanes share a row (its index comes by shuffle, one row pointer per pass) and copy adjacent chunks
// of it, which keeps both the number of cache lines per instruction (8) and the address arithmetic per
// copy low.  List positions past `cnt` read row 0 (their P columns are zero).
__device__ __forceinline__ void gather_rows_of_tile(int (&kv)[4], const int32_t* idx, int cnt, int j, int Lkv,
                                                    int lane, int* status) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int pos = j * 128 + i * 32 + lane;
    int v = (pos < cnt) ? __ldg(idx + pos) : 0;
    if ((unsigned)v >= (unsigned)Lkv) {
      if (status) atomicCAS(status, 0, (int)DEV_BAD_INDEX);
      v = 0;
    }
    kv[i] = v;
  }
}
// True (on every lane) when the tile's 128 list entries are all inside the list and name 128 consecutive
// keys kv[0] of lane 0, +1, ...: such a tile can be fetched with one TMA tile copy.
__device__ __forceinline__ bool tile_is_run(const int (&kv)[4], int cnt, int j, int Lkv, int lane) {
  const int first = __shfl_sync(0xffffffffu, kv[0], 0);
  bool run = (j + 1) * 128 <= cnt && first + 128 <= Lkv;
#pragma unroll
  for (int i = 0; i < 4; ++i) run = run && kv[i] == first + i * 32 + lane;
  return __all_sync(0xffffffffu, run);
}
template <int D>
__device__ __forceinline__ void gather_tile(uint32_t dst, const __nv_bfloat16* base, int64_t row_stride,
                                            const int (&kv)[4], int lane) {
  constexpr int CH = D / 8;      // 16-byte chunks per row
  constexpr int RPI = 8;         // rows per instruction (measured: 8 beats 2, 4, 16 and 32)
  constexpr int LPR = 32 / RPI;  // lanes that share a row
  constexpr int CPL = CH / LPR;  // chunks per lane and row
  const int g = lane / LPR, cq = lane % LPR;
#pragma unroll
  for (int pass = 0; pass < 128 / RPI; ++pass) {
    const int r = pass * RPI + g;
    const int row = __shfl_sync(0xffffffffu, kv[(pass * RPI) >> 5], r & 31);
    const __nv_bfloat16* src = base + (int64_t)row * row_stride;
    const uint32_t drow = dst + (uint32_t)r * 128u;
    const uint32_t x = (uint32_t)(r & 7);
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      const int c = i * LPR + cq;
      cp_async_16_l1(drow + (uint32_t)(c >> 3) * 16384u + ((((uint32_t)c & 7u) ^ x) << 4), src + c * 8);
    }
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

// p = exp2(s * scale - m) for one 32-column chunk: packed FMA, row-sum accumulation in two packed
// accumulators, bf16x2 packing of the 32 probabilities into pk[off .. off+15].
// Groups of four whose bit is set in POLY take their exponentials from exp2_poly_x2 (inputs clamped at -126,
// so the caller must not pass masked, i.e. -inf, scores with POLY != 0: they would come out as 2^-126, not 0).
template <uint32_t POLY = 0>
__device__ __forceinline__ void exp_pack_chunk(const uint32_t (&r)[32], uint64_t sc2, uint64_t nm2, uint64_t& sum_a,
                                               uint64_t& sum_b, uint32_t (&pk)[32], int off) {
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const uint64_t t0 = ffma2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), sc2, nm2);
    const uint64_t t1 = ffma2(pack_f32x2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])), sc2, nm2);
    float a0, a1, b0, b1;
    unpack_f32x2(t0, a0, a1);
    unpack_f32x2(t1, b0, b1);
    if ((POLY >> (i / 4)) & 1u) {
      exp2_poly_x2(pack_f32x2(fmaxf(a0, -126.f), fmaxf(a1, -126.f)), a0, a1);
      exp2_poly_x2(pack_f32x2(fmaxf(b0, -126.f), fmaxf(b1, -126.f)), b0, b1);
    } else {
      a0 = fast_exp2(a0);
      a1 = fast_exp2(a1);
      b0 = fast_exp2(b0);
      b1 = fast_exp2(b1);
    }
    sum_a = fadd2(sum_a, pack_f32x2(a0, a1));
    sum_b = fadd2(sum_b, pack_f32x2(b0, b1));
    pk[off + i / 2] = pack_bf16x2(a0, a1);
    pk[off + i / 2 + 1] = pack_bf16x2(b0, b1);
  }
}

// exp_pack_chunk without the packing: only the row sum of the 32 exponentials is kept.
__device__ __forceinline__ void exp_sum_chunk(const uint32_t (&r)[32], uint64_t sc2, uint64_t nm2, uint64_t& sum_a,
                                              uint64_t& sum_b) {
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const uint64_t t0 = ffma2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), sc2, nm2);
    const uint64_t t1 = ffma2(pack_f32x2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])), sc2, nm2);
    float a0, a1, b0, b1;
    unpack_f32x2(t0, a0, a1);
    unpack_f32x2(t1, b0, b1);
    sum_a = fadd2(sum_a, pack_f32x2(fast_exp2(a0), fast_exp2(a1)));
    sum_b = fadd2(sum_b, pack_f32x2(fast_exp2(b0), fast_exp2(b1)));
  }
}

// Sum over 32 queries of exp2(s_i * scale + c_i): one 32-column chunk of a key's S^T row (raw fp32 bits in r),
// the per-query constants c_i = -(M_i + log2 L_i) read as float4 from shared memory (the same address for the
// whole warp: a broadcast).
// Groups of four whose bit is set in POLY take their exponentials from exp2_poly_x2 (inputs clamped at -126).
template <uint32_t POLY>
__device__ __forceinline__ float colsum_chunk(const uint32_t (&r)[32], const float4* nc4, uint64_t sc2) {
  uint64_t a = 0ull, b = 0ull;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 nc = nc4[i];
    const uint64_t t0 = ffma2(pack_f32x2(__uint_as_float(r[4 * i + 0]), __uint_as_float(r[4 * i + 1])), sc2,
                              pack_f32x2(nc.x, nc.y));
    const uint64_t t1 = ffma2(pack_f32x2(__uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])), sc2,
                              pack_f32x2(nc.z, nc.w));
    float x0, x1, y0, y1;
    unpack_f32x2(t0, x0, x1);
    unpack_f32x2(t1, y0, y1);
    if ((POLY >> i) & 1u) {
      exp2_poly_x2(pack_f32x2(fmaxf(x0, -126.f), fmaxf(x1, -126.f)), x0, x1);
      exp2_poly_x2(pack_f32x2(fmaxf(y0, -126.f), fmaxf(y1, -126.f)), y0, y1);
      a = fadd2(a, pack_f32x2(x0, x1));
      b = fadd2(b, pack_f32x2(y0, y1));
    } else {
      a = fadd2(a, pack_f32x2(fast_exp2(x0), fast_exp2(x1)));
      b = fadd2(b, pack_f32x2(fast_exp2(y0), fast_exp2(y1)));
    }
  }
  float a0, a1, b0, b1;
  unpack_f32x2(a, a0, a1);
  unpack_f32x2(b, b0, b1);
  return (a0 + a1) + (b0 + b1);
}

}  // namespace lvar
