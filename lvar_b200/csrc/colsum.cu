// Attention column sums ("colsum", the KV-importance score) for sm_100a:
//   cs[b,h,g,j] = sum over query rows i of group g of softmax(q k^T * scale)[i,j]
// given the per-row softmax statistics (M, L) of a previous attention pass.  The L x L probability
// matrix is never materialised.  This is the second sweep of the reference's _full_attn_fwd
// (kernels/sparse_attn/triton/attn_dense_colsum.py:198-234) and the column-sum half of
// chipmunk::dense_colsum_attn (kernels/chipmunk/csrc/attn/dense_colsum_attn.cu:270-280).
//
// The product is taken TRANSPOSED: S^T = K_tile Q_tile^T, so one TMEM lane (= one thread) is one
// key column and the 128 queries of a tile sit in that thread's registers.  The column sum is then an
// in-thread sum: no shuffles, no atomics, and a fixed summation order (bit-reproducible output).
//   p_ij = exp2(s_ij * scale * log2e - c_i),   c_i = M_i + log2(L_i)
// One CTA owns one 128-key tile (the resident A operand) and streams every 128-query tile of the
// (batch, head) through a 3-stage TMA ring; S^T is 4-deep in TMEM.
//   warps 0-3  consumer warpgroup A: even query tiles
//   warps 4-7  consumer warpgroup B: odd query tiles; partial sums handed to A through shared memory
//   warp  8    loader: K tile, Q tiles (TMA) and the c_i vector of each query tile
//   warp  9    TMEM allocation and tcgen05.mma issue
// Query rows past Lq get c_i = +inf (p = 0); key columns past Lkv are not stored.
#include <math.h>

#include "common.cuh"
#include "ptx.cuh"

namespace lvar {

namespace {

constexpr int kCsThreads = 320;
constexpr int kQStages = 2;
constexpr int kSBufs = 2;
constexpr uint32_t kCsTmemCols = 256;  // two CTAs per SM: 2 x 256 TMEM columns, 2 x ~100 KB shared memory

struct ColsumParams {
  int B, H, Lq, Lkv, bm, G;
  float scale_log2;
  const float* M;
  const float* L;
  float* cs;  // [B,H,G,Lkv]
  int64_t cs_sb, cs_sh, cs_sg;
  int* status;
  unsigned long long wait_limit_ns;
};

template <int D>
struct CsSmem {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kK = 0;
  static constexpr int kQ = kTile;
  static constexpr int kC = kQ + kQStages * kTile;        // negc[kQStages][128] fp32
  static constexpr int kPart = kC + kQStages * 128 * 4;   // part[2][128] fp32
  static constexpr int kBars = kPart + 2 * 128 * 4;
  static constexpr int kTotal = kBars + 256;
  static constexpr int kDynamic = kTotal + 1024;
};

struct CsBars {
  uint64_t k_full;
  uint64_t q_full[kQStages], q_empty[kQStages];
  uint64_t s_full[kSBufs], s_empty[kSBufs];
  uint64_t part_full[2], part_empty[2];
  uint64_t mma_done;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(CsBars) <= 256, "barrier block too large");

}  // namespace

template <int D>
__global__ void __launch_bounds__(kCsThreads, 2)
colsum_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const ColsumParams p) {
  using SM = CsSmem<D>;
  constexpr int NSUB = D / 64;
  constexpr int KSTEPS = D / 16;
  constexpr uint32_t IDESC = make_idesc_bf16(128, 128, 0, 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  CsBars* bars = reinterpret_cast<CsBars*>(smem + SM::kBars);
  float* negc = reinterpret_cast<float*>(smem + SM::kC);
  float* part = reinterpret_cast<float*>(smem + SM::kPart);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kv0 = blockIdx.x * 128;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int n_tiles = (p.Lq + 127) / 128;

  if (tid == 0) {
    mbar_init(&bars->k_full, 1);
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(&bars->q_full[i], 1 + 32);  // TMA transaction + the 32 lanes that write c_i
      mbar_init(&bars->q_empty[i], 1 + 128);  // MMA commit + the consumer warpgroup that read c_i
    }
    for (int i = 0; i < kSBufs; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_empty[i], 128);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->part_full[i], 128);
      mbar_init(&bars->part_empty[i], 128);
    }
    mbar_init(&bars->mma_done, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(&bars->tmem_base, kCsTmemCols);
    tmem_relinquish();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = bars->tmem_base;
  WaitCtx wc{p.status, &bars->abort_flag, p.wait_limit_ns};
  uint8_t* sK = smem + SM::kK;
  uint8_t* sQ = smem + SM::kQ;

  if (warp < 8) {
    // ============================================================ consumers
    const int wg = warp >> 2;
    const int quad = warp & 3;
    const int col = kv0 + quad * 32 + lane;  // key column owned by this thread
    const bool col_ok = col < p.Lkv;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    float* out = p.cs + b * p.cs_sb + h * p.cs_sh + col;

    float acc = 0.f;
    int cur_group = 0;
    int n_flush = 0;
    bool ok = true;

    // Hands the finished group to global memory: warpgroup B parks its partial sum in shared memory,
    // warpgroup A adds it (fixed order: A + B) and stores.
    auto flush = [&](int g) -> bool {
      const int pb = n_flush & 1;
      const int ph = (n_flush >> 1) & 1;
      bool fine = true;
      if (wg == 1) {
        fine = __all_sync(0xffffffffu, mbar_wait(&bars->part_empty[pb], ph ^ 1, wc, DEV_TIMEOUT_SOFTMAX));
        if (fine) {
          part[pb * 128 + quad * 32 + lane] = acc;
          mbar_arrive(&bars->part_full[pb]);
        }
      } else {
        fine = __all_sync(0xffffffffu, mbar_wait(&bars->part_full[pb], ph, wc, DEV_TIMEOUT_SOFTMAX));
        if (fine) {
          const float total = acc + part[pb * 128 + quad * 32 + lane];
          mbar_arrive(&bars->part_empty[pb]);
          if (col_ok) out[(int64_t)g * p.cs_sg] = total;
        }
      }
      acc = 0.f;
      ++n_flush;
      return fine;
    };

    for (int t = 0; t < n_tiles && ok; ++t) {
      // chunks of 32 query rows; a chunk never straddles a group because bm % 32 == 0
      const bool mine = (t & 1) == wg;
      const int st = t % kQStages;
      const int buf = t % kSBufs;
      if (mine) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[buf], (t / kSBufs) & 1, wc, DEV_TIMEOUT_SOFTMAX));
        if (!ok) break;
        tc_fence_after();
      }
      const uint32_t tS = tmem_base + lane_off + (uint32_t)buf * 128u;
      const float4* nc4 = reinterpret_cast<const float4*>(negc + st * 128);
      const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2);
      auto chunk = [&](int c) {
        const int q0 = t * 128 + c * 32;
        if (q0 >= p.Lq || !ok) return;
        const int g = q0 / p.bm;
        if (g != cur_group) {
          ok = flush(cur_group);
          cur_group = g;
          if (!ok) return;
        }
        if (mine) {
          uint32_t r[32];
          tmem_ld_x32(tS + c * 32, r);
          tmem_wait_ld();
          uint64_t a = 0ull, bsum = 0ull;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 nc = nc4[c * 8 + i];
            const uint64_t t0 = ffma2(pack_f32x2(__uint_as_float(r[4 * i + 0]), __uint_as_float(r[4 * i + 1])), sc2,
                                      pack_f32x2(nc.x, nc.y));
            const uint64_t t1 = ffma2(pack_f32x2(__uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])), sc2,
                                      pack_f32x2(nc.z, nc.w));
            float x0, x1, y0, y1;
            unpack_f32x2(t0, x0, x1);
            unpack_f32x2(t1, y0, y1);
            a = fadd2(a, pack_f32x2(fast_exp2(x0), fast_exp2(x1)));
            bsum = fadd2(bsum, pack_f32x2(fast_exp2(y0), fast_exp2(y1)));
          }
          float a0, a1, b0, b1;
          unpack_f32x2(a, a0, a1);
          unpack_f32x2(bsum, b0, b1);
          acc += (a0 + a1) + (b0 + b1);
        }
      };
      chunk(0);
      chunk(1);
      chunk(2);
      chunk(3);
      if (!ok) break;
      if (mine) {
        tc_fence_before();
        mbar_arrive(&bars->s_empty[buf]);
        mbar_arrive(&bars->q_empty[st]);  // the c_i vector of this tile has been read
      }
    }
    if (ok) flush(cur_group);
  } else if (warp == 8) {
    // ============================================================ loader
    bool ok = true;
    int issued = 0;
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars->k_full, SM::kTile);
      for (int sub = 0; sub < NSUB; ++sub) tma_load_4d(sK + sub * 16384, &tmK, &bars->k_full, sub * 64, kv0, h, b);
    }
    const float* Mrow = p.M + (int64_t)bh * p.Lq;
    const float* Lrow = p.L + (int64_t)bh * p.Lq;
    for (int t = 0; t < n_tiles; ++t) {
      const int st = t % kQStages;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->q_empty[st], ((t / kQStages) & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER));
      if (!ok) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars->q_full[st], SM::kTile);
        for (int sub = 0; sub < NSUB; ++sub)
          tma_load_4d(sQ + st * SM::kTile + sub * 16384, &tmQ, &bars->q_full[st], sub * 64, t * 128, h, b);
      }
      issued = t + 1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = t * 128 + i * 32 + lane;
        float nc = -INFINITY;
        if (r < p.Lq) nc = -(Mrow[r] + log2f(Lrow[r]));
        negc[st * 128 + i * 32 + lane] = nc;
      }
      mbar_arrive(&bars->q_full[st]);
    }
    if (lane == 0 && bars->abort_flag) {
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(&bars->k_full, 0) && globaltimer_ns() - t0 < 2000000000ull) {
      }
      for (int t = max(0, issued - kQStages); t < issued; ++t) {
        const uint64_t t1 = globaltimer_ns();
        while (!mbar_try_wait(&bars->q_full[t % kQStages], (t / kQStages) & 1) &&
               globaltimer_ns() - t1 < 2000000000ull) {
        }
      }
    }
    __syncwarp();
  } else {
    // ============================================================ MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(&bars->k_full, 0, wc, DEV_TIMEOUT_MMA);
      const uint32_t kaddr = smem_u32(sK), qaddr = smem_u32(sQ);
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int st = t % kQStages;
        const int buf = t % kSBufs;
        ok = mbar_wait(&bars->q_full[st], (t / kQStages) & 1, wc, DEV_TIMEOUT_MMA);
        if (!ok) break;
        ok = mbar_wait(&bars->s_empty[buf], ((t / kSBufs) & 1) ^ 1, wc, DEV_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tS = tmem_base + (uint32_t)buf * 128u;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          const uint32_t koff = (ks >> 2) * 16384 + (ks & 3) * 32;
          const uint64_t ad = make_sw128_desc(kaddr + koff, 16, 1024);
          const uint64_t bd = make_sw128_desc(qaddr + st * SM::kTile + koff, 16, 1024);
          umma_ss(tS, ad, bd, IDESC, ks > 0 ? 1u : 0u);
        }
        umma_commit(&bars->s_full[buf]);
        umma_commit(&bars->q_empty[st]);
      }
      // TMEM must not be freed while an MMA is still in flight, also on abort.
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
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kCsTmemCols);
  }
}

template <int D>
static int launch_colsum_d(const CUtensorMap& tq, const CUtensorMap& tk, const ColsumParams& p, dim3 grid,
                           cudaStream_t stream) {
  auto kern = colsum_kernel<D>;
  LVAR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CsSmem<D>::kDynamic));
  LVAR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
  kern<<<grid, kCsThreads, CsSmem<D>::kDynamic, stream>>>(tq, tk, p);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

int launch_colsum(const void* q, const void* k, const float* M, const float* L, float* cs, int B, int H, int Lq,
                  int Lkv, int D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                  int64_t cs_sb, int64_t cs_sh, int64_t cs_sg, int group_rows, float scale, int* dev_status,
                  uint64_t wait_limit_ns, cudaStream_t stream) {
  LVAR_REQUIRE(D == 64 || D == 128, LVAR_ERR_UNSUPPORTED, "Head dimension must be 64 or 128 (got %d)", D);
  LVAR_REQUIRE(B >= 1 && H >= 1 && Lq >= 1 && Lkv >= 1, LVAR_ERR_ARG, "B, H, Lq, Lkv must be >= 1");
  LVAR_REQUIRE(q && k && M && L && cs, LVAR_ERR_ARG, "q, k, M, L, cs must be non-null device pointers");
  LVAR_REQUIRE(aligned16(q) && aligned16(k), LVAR_ERR_ARG, "q and k must be 16-byte aligned");
  LVAR_REQUIRE(group_rows >= 32 && group_rows % 32 == 0, LVAR_ERR_ARG,
               "group_rows must be a positive multiple of 32 (got %d)", group_rows);
  LVAR_REQUIRE(scale > 0.f && isfinite(scale), LVAR_ERR_ARG, "softmax scale must be positive and finite");
  LVAR_REQUIRE((int64_t)B * H <= 65535, LVAR_ERR_UNSUPPORTED, "B*H must be <= 65535");
  const int64_t strides[] = {q_sb, q_sh, q_sl, k_sb, k_sh, k_sl};
  for (int64_t s : strides)
    LVAR_REQUIRE(s % 8 == 0 && s >= 0, LVAR_ERR_ARG, "tensor strides must be non-negative multiples of 8 elements");

  ColsumParams p{};
  p.B = B;
  p.H = H;
  p.Lq = Lq;
  p.Lkv = Lkv;
  p.bm = group_rows;
  p.G = (Lq + group_rows - 1) / group_rows;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.M = M;
  p.L = L;
  p.cs = cs;
  p.cs_sb = cs_sb;
  p.cs_sh = cs_sh;
  p.cs_sg = cs_sg;
  p.status = dev_status;
  p.wait_limit_ns = wait_limit_ns;

  CUtensorMap tq, tk;
  int rc = encode_bhld_map(&tq, q, B, H, Lq, D, q_sb, q_sh, q_sl, 128);
  if (rc != LVAR_OK) return rc;
  rc = encode_bhld_map(&tk, k, B, H, Lkv, D, k_sb, k_sh, k_sl, 128);
  if (rc != LVAR_OK) return rc;
  dim3 grid((Lkv + 127) / 128, B * H, 1);
  if (D == 128) return launch_colsum_d<128>(tq, tk, p, grid, stream);
  return launch_colsum_d<64>(tq, tk, p, grid, stream);
}

}  // namespace lvar
