// Attention forward for sm_100a: dense, block-sparse (128x128 block mask) and column-sparse
// (token-index gather, "csp") variants of one warp-specialised tcgen05 kernel.
//
// One CTA owns two 128-row query tiles ("slots") of one (batch, head) and walks one list of
// 128-key KV tiles; each list entry says which of the two slots uses the tile.
//   warps 0-3   softmax warpgroup of slot 0 (thread = one query row = one TMEM lane)
//   warps 4-7   softmax warpgroup of slot 1
//   warp  8     K loader (+ the two Q tiles): TMA, or 16-byte cp.async row gathers for csp
//   warp  9     V loader
//   warp  10    allocates TMEM and issues every tcgen05.mma from one thread
//   warp  11    idle; completes the fourth warpgroup so registers can be re-balanced (setmaxnreg)
// TMEM (512 columns x 128 lanes, fp32): S0 | S1 | O0 | O1.  S_s = Q_s K^T lands in S_s; the softmax
// warpgroup overwrites the first 64 columns of S_s with bf16 P_s, which is then the TMEM A operand of
// O_s += P_s V.  Shared memory: Q0,Q1 + 2 K stages + 2 V stages, all 128-byte-swizzled [128][64]
// bf16 sub-tiles (exactly what a [64 x 128] TMA box writes), K-major for Q/K and MN-major for V.
//
// Softmax keeps a per-row reference maximum that is only moved when the running maximum exceeds it
// by more than 2^8 (the exponent offset is arbitrary as long as numerator and denominator share it),
// so the O accumulator in TMEM is rescaled rarely.  Row statistics are written in the layout of the
// reference's Triton kernels: M = rowmax(s*scale)*log2(e), L = sum_j exp2(s_j*scale*log2e - M)
// (kernels/sparse_attn/triton/attn_dense.py:209-227).
//
// Every wait is bounded (ptx.cuh: mbar_wait); a wait that runs out records a status code, raises a
// CTA-wide abort flag, lets the loaders drain their copies, frees TMEM and returns.
#include <math.h>

#include "common.cuh"
#include "ptx.cuh"

namespace lvar {

namespace {

constexpr int kThreads = 384;  // 8 softmax warps + K loader + V loader + MMA issuer + 1 idle warp
constexpr int kRegsSoftmax = 208, kRegsOther = 72;
constexpr int kMaxSteps = 2048;  // list capacity per CTA (KV tiles)
constexpr int kStages = 2;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

enum AttnMode : int { MODE_DENSE = 0, MODE_BLOCK = 1, MODE_CSP = 2 };

struct AttnParams {
  int B, H, Lq, Lkv, mode;
  float scale_log2;
  // output
  __nv_bfloat16* o;
  int64_t o_sb, o_sh, o_sl;
  float* M;  // [B,H,Lq] or nullptr
  float* L;  // [B,H,Lq] or nullptr
  // block mask (MODE_BLOCK): uint8 [*,*,nqb,nkb], broadcast over batch/head when the stride is 0
  const uint8_t* mask;
  int64_t m_sb, m_sh, m_sq;
  int nkb;
  // csp (MODE_CSP)
  const int32_t* indices;  // [B,H,G,idx_cols]
  int64_t i_sb, i_sh, i_sg;
  const int32_t* counts;  // [B,H,G]
  int64_t c_sb, c_sh;
  int bm;                 // query rows per index group
  int chunks_per_group;   // ceil(bm / 256)
  const __nv_bfloat16* k;  // raw pointers for the gather
  const __nv_bfloat16* v;
  int64_t k_sb, k_sh, k_sl, v_sb, v_sh, v_sl;
  const __nv_bfloat16* o_in;  // accumulate input (may alias o)
  int64_t oi_sb, oi_sh, oi_sl;
  float o_scale;
  // plumbing
  int* status;
  unsigned long long wait_limit_ns;
};

template <int D>
struct Smem {
  static constexpr int kTile = 128 * D * 2;  // bytes of one Q/K/V tile
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + 2 * kTile;
  static constexpr int kV = kK + kStages * kTile;
  static constexpr int kAux = kV + kStages * kTile;
  // aux: barriers then scalars then the step list
  static constexpr int kBarBytes = 256;
  static constexpr int kList = kAux + kBarBytes;
  static constexpr int kTotal = kList + kMaxSteps * 2;
  static constexpr int kDynamic = kTotal + 1024;  // slack for manual 1024-byte alignment
};

struct Bars {
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages];
  uint64_t v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], o_full[2];
  uint64_t mma_done;
  uint32_t tmem_base;
  int abort_flag;
  int n_steps;
  int n_act[2];
};
static_assert(sizeof(Bars) <= 256, "barrier block too large");

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

}  // namespace

template <int D, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using SM = Smem<D>;
  constexpr int NSUB = D / 64;
  constexpr int KSTEPS_QK = D / 16;
  constexpr uint32_t IDESC_QK = make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t IDESC_PV = make_idesc_bf16(128, D, 0, 1);
  constexpr uint32_t TM_O = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + SM::kAux);
  uint16_t* list = reinterpret_cast<uint16_t*>(smem + SM::kList);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int bh = blockIdx.y;
  const int b = bh / p.H;
  const int h = bh % p.H;

  // Row ranges of the two slots.
  int row0[2], row_end[2];
  int group = 0;
  if (MODE == MODE_CSP) {
    group = blockIdx.x / p.chunks_per_group;
    const int chunk = blockIdx.x % p.chunks_per_group;
    const int gend = min(p.Lq, (group + 1) * p.bm);
    row0[0] = group * p.bm + chunk * 256;
    row0[1] = row0[0] + 128;
    row_end[0] = gend;
    row_end[1] = gend;
  } else {
    row0[0] = blockIdx.x * 256;
    row0[1] = row0[0] + 128;
    row_end[0] = p.Lq;
    row_end[1] = p.Lq;
  }
  const bool slot_live[2] = {row0[0] < row_end[0], row0[1] < row_end[1]};

  // ---------------------------------------------------------------- setup
  if (tid == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bars->k_full[i], MODE == MODE_CSP ? 32 : 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], MODE == MODE_CSP ? 32 : 1);
      mbar_init(&bars->v_empty[i], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_full[s], 128);
      mbar_init(&bars->o_full[s], 1);
    }
    mbar_init(&bars->mma_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 10) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    if (MODE != MODE_CSP) {
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
    }
  }
  // Step list: entry = kv tile index | (slot bits << 14).
  if (warp == 0) {
    int n = 0, a0 = 0, a1 = 0;
    if (MODE == MODE_BLOCK) {
      const int qb0 = blockIdx.x * 2;
      const uint8_t* m0 = p.mask + b * p.m_sb + h * p.m_sh + (int64_t)qb0 * p.m_sq;
      const uint8_t* m1 = m0 + p.m_sq;
      for (int base = 0; base < p.nkb; base += 32) {
        const int j = base + lane;
        uint32_t bits = 0;
        if (j < p.nkb) {
          if (slot_live[0] && m0[j]) bits |= 1u;
          if (slot_live[1] && m1[j]) bits |= 2u;
        }
        const uint32_t vote = __ballot_sync(0xffffffffu, bits != 0);
        const int pos = n + __popc(vote & ((1u << lane) - 1u));
        if (bits && pos < kMaxSteps) list[pos] = (uint16_t)(j | (bits << 14));
        n += __popc(vote);
        a0 += __popc(__ballot_sync(0xffffffffu, bits & 1u));
        a1 += __popc(__ballot_sync(0xffffffffu, bits & 2u));
      }
    } else if (MODE == MODE_DENSE) {
      n = p.nkb;
      a0 = slot_live[0] ? n : 0;
      a1 = slot_live[1] ? n : 0;
    } else {
      const int cnt = p.counts[b * p.c_sb + h * p.c_sh + group];
      n = (cnt + 127) / 128;
      a0 = slot_live[0] ? n : 0;
      a1 = slot_live[1] ? n : 0;
    }
    if (!slot_live[0] && !slot_live[1]) n = 0;  // chunk past the end of its query group: nothing to do
    if (lane == 0) {
      bars->n_steps = (MODE == MODE_BLOCK) ? min(n, kMaxSteps) : n;
      bars->n_act[0] = a0;
      bars->n_act[1] = a1;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = bars->tmem_base;
  const int n_steps = bars->n_steps;
  const uint32_t dense_bits = (slot_live[0] ? 1u : 0u) | (slot_live[1] ? 2u : 0u);
  WaitCtx wc{p.status, &bars->abort_flag, p.wait_limit_ns};

  auto get_step = [&](int j, int& kvb, uint32_t& bits) {
    if (MODE == MODE_BLOCK) {
      const uint16_t e = list[j];
      kvb = e & 0x3FFF;
      bits = e >> 14;
    } else {
      kvb = j;
      bits = dense_bits;
    }
  };

  uint8_t* sQ = smem + SM::kQ;
  uint8_t* sK = smem + SM::kK;
  uint8_t* sV = smem + SM::kV;

  if (warp < 8) {
    // ============================================================ softmax warpgroups
    setmaxnreg_inc<kRegsSoftmax>();
    const int s = warp >> 2;
    const int quad = warp & 3;
    const int r_in_tile = quad * 32 + lane;
    const int row = row0[s] + r_in_tile;
    const bool row_ok = row < row_end[s];
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const uint32_t tS = tmem_base + lane_off + (uint32_t)s * 128u;
    const uint32_t tO = tmem_base + lane_off + TM_O + (uint32_t)s * D;
    const int cnt_total = (MODE == MODE_CSP) ? p.counts[b * p.c_sb + h * p.c_sh + group] : 0;

    float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
    int it = 0;
    bool ok = true;
    for (int j = 0; j < n_steps; ++j) {
      int kvb;
      uint32_t bits;
      get_step(j, kvb, bits);
      if (!((bits >> s) & 1u)) continue;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[s], it & 1, wc, DEV_TIMEOUT_SOFTMAX));
      if (!ok) break;  // warp-uniform: the TMEM accesses below are warp-collective
      tc_fence_after();

      // raw fp32 bits of the S row, four 32-column chunks kept in registers
      uint32_t s0[32], s1[32], s2[32], s3[32];
      tmem_ld_x32(tS + 0, s0);
      tmem_ld_x32(tS + 32, s1);
      tmem_ld_x32(tS + 64, s2);
      tmem_ld_x32(tS + 96, s3);
      tmem_wait_ld();

      const int valid = (MODE == MODE_CSP) ? (cnt_total - j * 128) : (p.Lkv - kvb * 128);
      if (valid < 128) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i >= valid) s0[i] = 0xff800000u;  // -inf
          if (i + 32 >= valid) s1[i] = 0xff800000u;
          if (i + 64 >= valid) s2[i] = 0xff800000u;
          if (i + 96 >= valid) s3[i] = 0xff800000u;
        }
      }
      const float mx = fmax3(fmaxf(chunk_max(s0), chunk_max(s1)), chunk_max(s2), chunk_max(s3));
      const float mx_s = mx * p.scale_log2;
      m_true = fmaxf(m_true, mx_s);
      const bool need = mx_s > m_ref + kRescaleThreshold;
      if (__any_sync(0xffffffffu, need)) {
        float alpha = 1.0f;
        if (need) {
          alpha = fast_exp2(m_ref - mx_s);
          m_ref = mx_s;
        }
        l *= alpha;
        if (it > 0) {
          const uint64_t a2 = pack_f32x2(alpha, alpha);
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_x32(tO + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const uint64_t t = fmul2(pack_f32x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), a2);
              float x0, x1;
              unpack_f32x2(t, x0, x1);
              r[2 * i] = __float_as_uint(x0);
              r[2 * i + 1] = __float_as_uint(x1);
            }
            tmem_st_x32(tO + c * 32, r);
          }
          tmem_wait_st();
        }
      }
      const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2);
      const uint64_t nm2 = pack_f32x2(-m_ref, -m_ref);
      uint64_t sum_a = 0ull, sum_b = 0ull;  // two packed accumulators = four partial row sums
      {
        uint32_t pk[32];
        exp_pack_chunk(s0, sc2, nm2, sum_a, sum_b, pk, 0);
        exp_pack_chunk(s1, sc2, nm2, sum_a, sum_b, pk, 16);
        tmem_st_x32(tS, pk);
      }
      {
        uint32_t pk[32];
        exp_pack_chunk(s2, sc2, nm2, sum_a, sum_b, pk, 0);
        exp_pack_chunk(s3, sc2, nm2, sum_a, sum_b, pk, 16);
        tmem_st_x32(tS + 32, pk);
      }
      {
        float a0, a1, b0, b1;
        unpack_f32x2(sum_a, a0, a1);
        unpack_f32x2(sum_b, b0, b1);
        l += (a0 + a1) + (b0 + b1);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&bars->p_full[s]);
      ++it;
    }

    // ---- epilogue: O / l -> bf16 -> global; row statistics
    if (ok && it > 0) ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full[s], 0, wc, DEV_TIMEOUT_SOFTMAX));
    if (ok) {
      tc_fence_after();
      const float inv_l = (it > 0) ? (1.0f / l) : 0.f;
      __nv_bfloat16* orow = p.o + b * p.o_sb + h * p.o_sh + (int64_t)row * p.o_sl;
      const __nv_bfloat16* irow =
          (MODE == MODE_CSP) ? (p.o_in + b * p.oi_sb + h * p.oi_sh + (int64_t)row * p.oi_sl) : nullptr;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        if (it > 0) {
          tmem_ld_x32(tO + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float x0 = __uint_as_float(r[q4 * 8 + 2 * i]) * inv_l;
              const float x1 = __uint_as_float(r[q4 * 8 + 2 * i + 1]) * inv_l;
              w[i] = pack_bf16x2(x0, x1);
            }
            if (MODE == MODE_CSP) {
              // out = bf16(o_in + o_scale * bf16(delta)): same rounding points as the reference's
              // `o + o_delta * o_scale` on bf16 tensors (kernels/sparse_attn/sparse_attn_ops.py:288).
              const uint4 prev = *reinterpret_cast<const uint4*>(irow + c * 32 + q4 * 8);
              const uint32_t pv[4] = {prev.x, prev.y, prev.z, prev.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float d0 = __uint_as_float(w[i] << 16), d1 = __uint_as_float(w[i] & 0xffff0000u);
                const float a0 = __uint_as_float(pv[i] << 16), a1 = __uint_as_float(pv[i] & 0xffff0000u);
                w[i] = pack_bf16x2(fmaf(p.o_scale, d0, a0), fmaf(p.o_scale, d1, a1));
              }
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (row_ok && MODE != MODE_CSP) {
        const int64_t si = (int64_t)bh * p.Lq + row;
        if (p.M) p.M[si] = m_true;
        if (p.L) p.L[si] = (it > 0) ? l * fast_exp2(m_ref - m_true) : 0.f;
      }
    }
  } else if (warp == 8) {
    // ============================================================ K (and Q) loader
    setmaxnreg_dec<kRegsOther>();
    int issued = 0;
    bool ok = true;
    if (MODE != MODE_CSP) {
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars->q_full, 2 * SM::kTile);
        for (int s = 0; s < 2; ++s)
          for (int sub = 0; sub < NSUB; ++sub)
            tma_load_4d(sQ + s * SM::kTile + sub * 16384, &tmQ, &bars->q_full, sub * 64, row0[s], h, b);
        for (int j = 0; j < n_steps; ++j) {
          int kvb;
          uint32_t bits;
          get_step(j, kvb, bits);
          const int st = j % kStages;
          ok = mbar_wait(&bars->k_empty[st], ((j / kStages) & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars->k_full[st], SM::kTile);
          for (int sub = 0; sub < NSUB; ++sub)
            tma_load_4d(sK + st * SM::kTile + sub * 16384, &tmK, &bars->k_full[st], sub * 64, kvb * 128, h, b);
          issued = j + 1;
        }
        // Drain on abort: copies in flight must land before the CTA's shared memory is released.
        if (bars->abort_flag) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&bars->q_full, 0) && globaltimer_ns() - t0 < 2000000000ull) {
          }
          for (int j = max(0, issued - kStages); j < issued; ++j) {
            const int st = j % kStages;
            const uint64_t t1 = globaltimer_ns();
            while (!mbar_try_wait(&bars->k_full[st], (j / kStages) & 1) && globaltimer_ns() - t1 < 2000000000ull) {
            }
          }
        }
      }
    } else {
      // csp: Q by TMA (lane 0), K rows gathered by the whole warp with 16-byte cp.async.
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars->q_full, 2 * SM::kTile);
        for (int s = 0; s < 2; ++s)
          for (int sub = 0; sub < NSUB; ++sub)
            tma_load_4d(sQ + s * SM::kTile + sub * 16384, &tmQ, &bars->q_full, sub * 64, row0[s], h, b);
      }
      const int32_t* idx = p.indices + b * p.i_sb + h * p.i_sh + (int64_t)group * p.i_sg;
      const int cnt = p.counts[b * p.c_sb + h * p.c_sh + group];
      const __nv_bfloat16* kbase = p.k + b * p.k_sb + h * p.k_sh;
      for (int j = 0; j < n_steps; ++j) {
        const int st = j % kStages;
        ok = mbar_wait(&bars->k_empty[st], ((j / kStages) & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        gather_tile<D>(smem_u32(sK + st * SM::kTile), kbase, p.k_sl, idx, cnt, j, p.Lkv, lane, p.status);
        cp_async_commit();
        issued = j + 1;
        if (j > 0) {  // tile j-1 has landed once at most one group is still pending
          cp_async_wait<1>();
          fence_proxy_async_smem();
          mbar_arrive(&bars->k_full[(j - 1) % kStages]);
        }
      }
      cp_async_wait<0>();  // also drains on abort
      if (issued > 0 && ok) {
        fence_proxy_async_smem();
        mbar_arrive(&bars->k_full[(issued - 1) % kStages]);
      }
      if (lane == 0 && bars->abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&bars->q_full, 0) && globaltimer_ns() - t0 < 2000000000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ============================================================ V loader
    setmaxnreg_dec<kRegsOther>();
    bool ok = true;
    if (MODE != MODE_CSP) {
      if (lane == 0) {
        int issued = 0;
        for (int j = 0; j < n_steps; ++j) {
          int kvb;
          uint32_t bits;
          get_step(j, kvb, bits);
          const int st = j % kStages;
          ok = mbar_wait(&bars->v_empty[st], ((j / kStages) & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars->v_full[st], SM::kTile);
          for (int sub = 0; sub < NSUB; ++sub)
            tma_load_4d(sV + st * SM::kTile + sub * 16384, &tmV, &bars->v_full[st], sub * 64, kvb * 128, h, b);
          issued = j + 1;
        }
        if (bars->abort_flag) {
          for (int j = max(0, issued - kStages); j < issued; ++j) {
            const int st = j % kStages;
            const uint64_t t1 = globaltimer_ns();
            while (!mbar_try_wait(&bars->v_full[st], (j / kStages) & 1) && globaltimer_ns() - t1 < 2000000000ull) {
            }
          }
        }
      }
    } else {
      const int32_t* idx = p.indices + b * p.i_sb + h * p.i_sh + (int64_t)group * p.i_sg;
      const int cnt = p.counts[b * p.c_sb + h * p.c_sh + group];
      const __nv_bfloat16* vbase = p.v + b * p.v_sb + h * p.v_sh;
      int issued = 0;
      for (int j = 0; j < n_steps; ++j) {
        const int st = j % kStages;
        ok = mbar_wait(&bars->v_empty[st], ((j / kStages) & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        gather_tile<D>(smem_u32(sV + st * SM::kTile), vbase, p.v_sl, idx, cnt, j, p.Lkv, lane, nullptr);
        cp_async_commit();
        issued = j + 1;
        if (j > 0) {  // tile j-1 has landed once at most one group is still pending
          cp_async_wait<1>();
          fence_proxy_async_smem();
          mbar_arrive(&bars->v_full[(j - 1) % kStages]);
        }
      }
      cp_async_wait<0>();  // also drains on abort
      if (issued > 0 && ok) {
        fence_proxy_async_smem();
        mbar_arrive(&bars->v_full[(issued - 1) % kStages]);
      }
    }
    __syncwarp();
  } else if (warp == 10) {
    // ============================================================ MMA issuer (one thread)
    setmaxnreg_dec<kRegsOther>();
    if (lane == 0) {
      bool ok = mbar_wait(&bars->q_full, 0, wc, DEV_TIMEOUT_MMA);
      const uint32_t qaddr = smem_u32(sQ), kaddr = smem_u32(sK), vaddr = smem_u32(sV);
      uint32_t prev_bits = 0;
      int prev_st = 0, prev_j = 0;
      int npv[2] = {0, 0};
      for (int j = 0; j <= n_steps && ok; ++j) {
        int kvb = 0;
        uint32_t bits = 0;
        if (j < n_steps) get_step(j, kvb, bits);
        const int st = j % kStages;
        if (bits) {
          ok = mbar_wait(&bars->k_full[st], (j / kStages) & 1, wc, DEV_TIMEOUT_MMA);
          if (!ok) break;
        }
        if (prev_bits) {
          ok = mbar_wait(&bars->v_full[prev_st], (prev_j / kStages) & 1, wc, DEV_TIMEOUT_MMA);
          if (!ok) break;
        }
        tc_fence_after();
        for (int s = 0; s < 2 && ok; ++s) {
          if ((prev_bits >> s) & 1u) {
            ok = mbar_wait(&bars->p_full[s], npv[s] & 1, wc, DEV_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tP = tmem_base + (uint32_t)s * 128u;
            const uint32_t tOs = tmem_base + TM_O + (uint32_t)s * D;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t bd = make_sw128_desc(vaddr + prev_st * SM::kTile + ks * 2048, 16384, 1024);
              umma_ts(tOs, tP + ks * 8, bd, IDESC_PV, (npv[s] > 0 || ks > 0) ? 1u : 0u);
            }
            ++npv[s];
          }
          if ((bits >> s) & 1u) {
            const uint32_t tSs = tmem_base + (uint32_t)s * 128u;
#pragma unroll
            for (int ks = 0; ks < KSTEPS_QK; ++ks) {
              const uint32_t koff = (ks >> 2) * 16384 + (ks & 3) * 32;
              const uint64_t ad = make_sw128_desc(qaddr + s * SM::kTile + koff, 16, 1024);
              const uint64_t bd = make_sw128_desc(kaddr + st * SM::kTile + koff, 16, 1024);
              umma_ss(tSs, ad, bd, IDESC_QK, ks > 0 ? 1u : 0u);
            }
            umma_commit(&bars->s_full[s]);
          }
        }
        if (!ok) break;
        if (prev_bits) umma_commit(&bars->v_empty[prev_st]);
        if (bits) umma_commit(&bars->k_empty[st]);
        prev_bits = bits;
        prev_st = st;
        prev_j = j;
      }
      if (ok) {
        if (npv[0] > 0) umma_commit(&bars->o_full[0]);
        if (npv[1] > 0) umma_commit(&bars->o_full[1]);
      }
      // TMEM must not be freed (nor the CTA retire) while an MMA is still in flight, also on abort.
      umma_commit(&bars->mma_done);
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(&bars->mma_done, 0)) {
        if (globaltimer_ns() - t0 > 2000000000ull) {
          if (p.status) atomicCAS(p.status, 0, (int)DEV_TIMEOUT_DRAIN);
          break;
        }
      }
    }
    __syncwarp();
  } else {
    setmaxnreg_dec<kRegsOther>();  // idle warp: only takes part in the register re-balancing
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 10) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// -------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------
namespace {

template <int D, int MODE>
int launch_mode(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, dim3 grid,
                cudaStream_t stream) {
  auto kern = attn_fwd_kernel<D, MODE>;
  static bool attr_set[16] = {false};
  int dev = 0;
  LVAR_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 16 && !attr_set[dev]) {
    LVAR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<D>::kDynamic));
    attr_set[dev] = true;
  } else if (dev >= 16) {
    LVAR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<D>::kDynamic));
  }
  kern<<<grid, kThreads, Smem<D>::kDynamic, stream>>>(tq, tk, tv, p);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

template <int D>
int launch_d(int mode, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
             dim3 grid, cudaStream_t stream) {
  switch (mode) {
    case MODE_DENSE: return launch_mode<D, MODE_DENSE>(tq, tk, tv, p, grid, stream);
    case MODE_BLOCK: return launch_mode<D, MODE_BLOCK>(tq, tk, tv, p, grid, stream);
    default: return launch_mode<D, MODE_CSP>(tq, tk, tv, p, grid, stream);
  }
}

}  // namespace

int launch_attention(const lvar_attn_args* a, int mode, cudaStream_t stream) {
  LVAR_REQUIRE(a != nullptr, LVAR_ERR_ARG, "null argument block");
  LVAR_REQUIRE(a->D == 64 || a->D == 128, LVAR_ERR_UNSUPPORTED, "Head dimension must be 64 or 128 (got %d)", a->D);
  LVAR_REQUIRE(a->B >= 1 && a->H >= 1 && a->Lq >= 1 && a->Lkv >= 1, LVAR_ERR_ARG,
               "B, H, Lq, Lkv must be >= 1 (got %d %d %d %d)", a->B, a->H, a->Lq, a->Lkv);
  LVAR_REQUIRE(a->q && a->k && a->v && a->o, LVAR_ERR_ARG, "q, k, v, o must be non-null device pointers");
  LVAR_REQUIRE(aligned16(a->q) && aligned16(a->k) && aligned16(a->v) && aligned16(a->o), LVAR_ERR_ARG,
               "q, k, v, o must be 16-byte aligned");
  LVAR_REQUIRE(a->scale > 0.f && isfinite(a->scale), LVAR_ERR_ARG, "softmax scale must be positive and finite");
  const int64_t strides[] = {a->q_sb, a->q_sh, a->q_sl, a->k_sb, a->k_sh, a->k_sl,
                             a->v_sb, a->v_sh, a->v_sl, a->o_sb, a->o_sh, a->o_sl};
  for (int64_t s : strides)
    LVAR_REQUIRE(s % 8 == 0 && s >= 0, LVAR_ERR_ARG, "tensor strides must be non-negative multiples of 8 elements");
  LVAR_REQUIRE((int64_t)a->B * a->H <= 65535, LVAR_ERR_UNSUPPORTED, "B*H must be <= 65535");

  AttnParams p{};
  p.B = a->B;
  p.H = a->H;
  p.Lq = a->Lq;
  p.Lkv = a->Lkv;
  p.mode = mode;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.o = static_cast<__nv_bfloat16*>(a->o);
  p.o_sb = a->o_sb;
  p.o_sh = a->o_sh;
  p.o_sl = a->o_sl;
  p.M = a->M;
  p.L = a->L;
  p.nkb = (a->Lkv + 127) / 128;
  p.status = a->dev_status;
  p.wait_limit_ns = a->wait_limit_ns;

  dim3 grid;
  if (mode == MODE_BLOCK) {
    LVAR_REQUIRE(a->block_mask != nullptr, LVAR_ERR_ARG, "block mask is null");
    LVAR_REQUIRE(p.nkb <= kMaxSteps, LVAR_ERR_UNSUPPORTED, "Lkv too long for the block list (max %d keys)",
                 kMaxSteps * 128);
    p.mask = a->block_mask;
    p.m_sb = a->bm_sb;
    p.m_sh = a->bm_sh;
    p.m_sq = a->bm_sq;
  }
  if (mode == MODE_DENSE) {
    LVAR_REQUIRE(p.nkb <= 16383, LVAR_ERR_UNSUPPORTED, "Lkv too long (max %d keys)", 16383 * 128);
  }
  if (mode == MODE_CSP) {
    LVAR_REQUIRE(a->indices && a->counts && a->o_in, LVAR_ERR_ARG, "indices, counts and o_in must be non-null");
    LVAR_REQUIRE(a->group_rows >= 1, LVAR_ERR_ARG, "group_rows must be >= 1");
    LVAR_REQUIRE(a->o_scale == 1 || a->o_scale == -1, LVAR_ERR_ARG, "o_scale must be 1 or -1");
    LVAR_REQUIRE(aligned16(a->o_in) && a->oi_sb % 8 == 0 && a->oi_sh % 8 == 0 && a->oi_sl % 8 == 0, LVAR_ERR_ARG,
                 "o_in must be 16-byte aligned with strides that are multiples of 8 elements");
    p.indices = a->indices;
    p.i_sb = a->i_sb;
    p.i_sh = a->i_sh;
    p.i_sg = a->i_sg;
    p.counts = a->counts;
    p.c_sb = a->c_sb;
    p.c_sh = a->c_sh;
    p.bm = a->group_rows;
    p.chunks_per_group = (a->group_rows + 255) / 256;
    p.k = static_cast<const __nv_bfloat16*>(a->k);
    p.v = static_cast<const __nv_bfloat16*>(a->v);
    p.k_sb = a->k_sb;
    p.k_sh = a->k_sh;
    p.k_sl = a->k_sl;
    p.v_sb = a->v_sb;
    p.v_sh = a->v_sh;
    p.v_sl = a->v_sl;
    p.o_in = static_cast<const __nv_bfloat16*>(a->o_in);
    p.oi_sb = a->oi_sb;
    p.oi_sh = a->oi_sh;
    p.oi_sl = a->oi_sl;
    p.o_scale = (float)a->o_scale;
    const int groups = (a->Lq + a->group_rows - 1) / a->group_rows;
    grid = dim3(groups * p.chunks_per_group, a->B * a->H, 1);
  } else {
    grid = dim3((a->Lq + 255) / 256, a->B * a->H, 1);
  }

  CUtensorMap tq, tk, tv;
  int rc = encode_bhld_map(&tq, a->q, a->B, a->H, a->Lq, a->D, a->q_sb, a->q_sh, a->q_sl, 128);
  if (rc != LVAR_OK) return rc;
  rc = encode_bhld_map(&tk, a->k, a->B, a->H, a->Lkv, a->D, a->k_sb, a->k_sh, a->k_sl, 128);
  if (rc != LVAR_OK) return rc;
  rc = encode_bhld_map(&tv, a->v, a->B, a->H, a->Lkv, a->D, a->v_sb, a->v_sh, a->v_sl, 128);
  if (rc != LVAR_OK) return rc;

  if (a->D == 128) return launch_d<128>(mode, tq, tk, tv, p, grid, stream);
  return launch_d<64>(mode, tq, tk, tv, p, grid, stream);
}

}  // namespace lvar
