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


}  // namespace lvar
