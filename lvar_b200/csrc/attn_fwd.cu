// Attention forward for sm_100a: dense, block-sparse (128x128 block mask) and column-sparse
// (token-index gather, "csp") variants of one warp-specialised tcgen05 kernel.
//
// The kernel is persistent (one CTA per SM, work items drawn from a global counter).  A work item is
// two 128-row query tiles ("slots") of one (batch, head); each slot walks its own ascending list of
// 128-key KV tiles, the two lists advance in lock step ("rounds") and a tile both slots need in the
// same round is loaded once (always the case for dense and column-sparse attention).
//   warps 0-3   softmax warpgroup of slot 0 (thread = one query row = one TMEM lane)
//   warps 4-7   softmax warpgroup of slot 1
//   warp  8     K loader (+ the two Q tiles): TMA, or 16-byte cp.async row gathers for csp (four lanes share
//               a row; the tile's barrier takes one arrival per lane as its copies land)
//   warp  9     V loader
//   warp  10    allocates TMEM; lane 0 issues every tcgen05.mma (descriptor words precomputed, all lanes
//               run the bookkeeping so that it stays out of a divergent branch)
//   warp  11    scheduler: takes work items from the global counter and builds their KV-tile lists
// TMEM (512 columns x 128 lanes, fp32): S0 | S1 | O0 | O1.  S_s = Q_s K^T lands in S_s; the softmax
// warpgroup overwrites the first 64 columns of S_s with bf16 P_s, which is then the TMEM A operand of
// O_s += P_s V.  Shared memory: Q0,Q1 + 2 K stages + 2 V stages, all 128-byte-swizzled [128][64]
// bf16 sub-tiles (exactly what a [64 x 128] TMA box writes), K-major for Q/K and MN-major for V.
//
// Softmax keeps a per-row reference maximum that is only moved when the running maximum exceeds it
// by more than 2^32 (the exponent offset is arbitrary as long as numerator and denominator share it),
// so the O accumulator in TMEM is rescaled rarely.  Row statistics are written in the layout of the
// reference's Triton kernels: M = rowmax(s*scale)*log2(e), L = sum_j exp2(s_j*scale*log2e - M)
// (kernels/sparse_attn/triton/attn_dense.py:209-227).
//
// Every wait is bounded (ptx.cuh: mbar_wait); a wait that runs out records a status code, raises a
// CTA-wide abort flag, lets the loaders drain their copies, frees TMEM and returns.
#include <math.h>

#include <type_traits>

#include "attn_common.cuh"
#include "common.cuh"
#include "ptx.cuh"

namespace lvar {

namespace {

constexpr int kThreads = 384;  // 8 softmax warps + K loader + V loader + MMA issuer + scheduler
constexpr int kRegsSoftmax = 208, kRegsOther = 72;
constexpr int kMaxSteps = 1024;  // per-slot KV tile list capacity (block-sparse: Lkv <= 131072)
constexpr int kStages = 2;
constexpr int kSchedStages = 2;
// TMEM buffers per slot for S^T in the column-sum sweep: 1 (S_s) or 2 (S_s and the O region).  Two buffers let
// the MMA of the next tile run under the softmax warps' reads and measured 6 % slower, like every other
// change that keeps the tensor pipe busy while TMEM is being read.
constexpr int kCsBufs = 1;
// Column-sum sweep: which of the 8 groups of four exponentials per 32-column chunk are evaluated on the FMA
// pipe (polynomial) instead of the exp2 unit, the sweep's bottleneck.  A quarter of them measured best
// (0.47 -> 0.42 ms for the sweep at 4096 x 10521 x 32 heads; three eighths or a half: 0.43-0.45 ms); the same
// mix in the statistics sweep of MODE_CS_ONLY gained nothing and is not used.
constexpr uint32_t kCsPolyMask = 0x88;
// Log2 units by which a row maximum may exceed the row's reference maximum before the reference moves
// (and O is rescaled).  bf16 has the exponent range of fp32, so P = exp2(s - reference) <= 2^32 is safe.
constexpr float kRescaleThreshold = 32.0f;

// MODE_DENSE_CS: dense attention followed, per work item, by a second sweep over the K tiles that takes
// the attention column sums of the item's two query tiles (see the softmax warps).
// MODE_CS_ONLY: the column sums alone.  The first sweep only takes the row statistics (no P, no PV, no V
// loads, no output), or is left out when the caller supplies them; the second sweep is MODE_DENSE_CS's.
// MODE_DENSE_CS1: dense attention and the column sums in ONE sweep, for callers that supply the row statistics
// (the form of the reference's CUDA operator, kernels/chipmunk/csrc/attn/dense_colsum_attn.cu:270-280): the
// probabilities that feed P V are normalised with the given constants as they are formed, and their column
// sums are taken from the same registers.  (5 is launch_attention's code for MODE_CS_ONLY on given statistics.)
enum AttnMode : int {
  MODE_DENSE = 0, MODE_BLOCK = 1, MODE_CSP = 2, MODE_DENSE_CS = 3, MODE_CS_ONLY = 4, MODE_DENSE_CS1 = 6
};

struct AttnParams {
  int B, H, Lq, Lkv, mode;
  float scale_log2;
  // output
  __nv_bfloat16* o;
  int64_t o_sb, o_sh, o_sl;
  float* M;  // [B,H,Lq] or nullptr
  float* L;  // [B,H,Lq] or nullptr
  int o_align32;  // rows of o start on 32-byte boundaries: the epilogue may use 256-bit stores
  float* cs;  // MODE_DENSE_CS / MODE_CS_ONLY: column sums per 128-row query tile [B,H,ceil(Lq/128),Lkv]
  int64_t cs_sb, cs_sh, cs_st;
  int cs_pair;  // 1: the two 128-row tiles of a 256-row group add into ONE zero-initialised row of cs
  const float* M_in;  // MODE_CS_ONLY: row statistics supplied by the caller (both or neither); the
  const float* L_in;  // statistics sweep is then skipped
  // block mask (MODE_BLOCK): uint8 [*,*,nqb,nkb], broadcast over batch/head when the stride is 0
  const uint8_t* mask;
  int64_t m_sb, m_sh, m_sq;
  int nkb;
  int mask_block;  // 128, or 64: four mask entries per 128x128 tile (sub-tile bits travel with the list)
  int nq_mask, nk_mask;  // mask extents in blocks
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
  int oi_side;      // > 0: o_in is a cache over an oi_side x oi_side token grid, resized on the fly
  int o_side;       // side of the query grid (o_side^2 == Lq) when oi_side > 0
  float oi_ratio;   // oi_side / o_side
  // persistent scheduling
  int n_x;            // query-tile pairs per (batch, head)
  int n_pair_items;   // items [0, n_pair_items) are pairs, [n_pair_items, total_items) single tiles
  int total_items;
  int split_singles;  // 1: a single-tile item runs on BOTH slots, each taking half of the tile's KV list
  int* sched_counter;  // device int32[2], zero on entry and left zero on exit
  const int32_t* work_order;  // optional permutation of the pair items: schedule position -> pair (heaviest first)
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
  static constexpr int kBarBytes = 512;
  static constexpr int kList = kAux + kBarBytes;
  static constexpr int kNegC = kList + kSchedStages * 2 * kMaxSteps * 2;    // [slot][128] fp32: -(M_i + log2 L_i)
  static constexpr int kXchg = kNegC + 2 * 128 * 4;  // [item parity][m_ref, l, m_true][128] fp32: slot 1 -> slot 0 of a split tile
  // MODE_DENSE_CS1: per-warp column sums of a tile [slot][buffer][warp][128] fp32, and the rows' sums [slot][128]
  static constexpr int kPart = kXchg + 2 * 3 * 128 * 4;
  static constexpr int kRowL = kPart + 2 * 2 * 4 * 128 * 4;
  static constexpr int kTotal = kRowL + 2 * 128 * 4;
  static constexpr int kDynamic = kTotal + 1024;  // slack for manual 1024-byte alignment
};

struct SchedEntry {
  int item;  // pair id, < 0: no more work
  int half;  // < 0: the whole pair; 0 / 1: only that 128-row tile of the pair
  int n0;    // KV tiles of slot 0
  int n1;    // KV tiles of slot 1
  int aux;   // csp: length of the item's index list
  int off1;  // dense, split tile: slot 1 starts at this KV tile (slot 0 takes the tiles before it)
};

// One round of the two slots' tile streams: slot s works on KV tile kvb[s] if has[s]; when both want
// the same tile it is loaded once and shared.
struct Round {
  bool has[2];
  bool shared;
  int kvb[2];
};

struct Bars {
  uint64_t q_full, q_empty;
  uint64_t k_full[kStages], k_empty[kStages];
  uint64_t v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], o_full[2], o_empty[2];
  uint64_t sched_full[kSchedStages], sched_empty[kSchedStages];
  uint64_t mma_done;
  uint64_t xchg_full[2];  // split tile: slot 1's partial result is complete (128 arrivals), by item parity
  uint64_t part_full[2][2];  // MODE_DENSE_CS1: the four warps' column sums of a tile are in shared memory [slot][buffer]
  uint64_t rowl_full[2];     // MODE_DENSE_CS1: the rows' probability sums of an item are in shared memory [slot]
  // column-sum sweep (MODE_DENSE_CS): S^T of a slot is double-buffered, [slot][buffer]
  uint64_t cs_full[2][2], cs_empty[2][2];
  SchedEntry sched[kSchedStages];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Bars) <= 512, "barrier block too large");

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
  constexpr bool kHasCs = MODE == MODE_DENSE_CS || MODE == MODE_CS_ONLY;  // column-sum sweep after the first one
  // Epilogue form: O_s read out in one go and stored with 256-bit stores, or 32 columns at a time with 128-bit
  // stores.  Chosen per mode by measurement (block-sparse +2.4 % with the first form, dense attention at 83 KV
  // tiles per item -1.6 %: the kernel is sensitive to the size and placement of code it runs once per item).
  constexpr bool kRegisterEpilogue = MODE == MODE_BLOCK || MODE == MODE_DENSE_CS || MODE == MODE_DENSE_CS1;
  // MODE_CS_ONLY with the caller's row statistics: no first sweep at all
  const bool stats_given = MODE == MODE_CS_ONLY && p.M_in != nullptr;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + SM::kAux);
  uint16_t* lists = reinterpret_cast<uint16_t*>(smem + SM::kList);  // [kSchedStages][kMaxSteps]
  float* negc = reinterpret_cast<float*>(smem + SM::kNegC);
  float* xchg = reinterpret_cast<float*>(smem + SM::kXchg);
  float* part = reinterpret_cast<float*>(smem + SM::kPart);
  float* rowl = reinterpret_cast<float*>(smem + SM::kRowL);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---------------------------------------------------------------- setup
  if (tid == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_empty, 1);
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
      mbar_init(&bars->o_empty[s], 128);
      for (int b = 0; b < 2; ++b) {
        mbar_init(&bars->cs_full[s][b], 1);
        mbar_init(&bars->cs_empty[s][b], 128);
      }
    }
    for (int i = 0; i < kSchedStages; ++i) {
      mbar_init(&bars->sched_full[i], 1);
      mbar_init(&bars->sched_empty[i], 11);  // 8 softmax warps + K loader + V loader + MMA issuer
    }
    mbar_init(&bars->mma_done, 1);
    mbar_init(&bars->xchg_full[0], 128);
    mbar_init(&bars->xchg_full[1], 128);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->part_full[s][0], 128);
      mbar_init(&bars->part_full[s][1], 128);
      mbar_init(&bars->rowl_full[s], 128);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 10) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == 8 && lane == 0) {
    griddep_launch_dependents();  // the next grid in the stream may take an SM as soon as this CTA has left it
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = bars->tmem_base;
  WaitCtx wc{p.status, &bars->abort_flag, p.wait_limit_ns};

  // A work item is one (batch, head) x (pair of 128-row query tiles), or one tile of such a pair.  Decoded by
  // every role itself.
  struct Item {
    int b, h, bh, group;
    int row0[2], row_end[2];
    uint32_t live;  // bit s: slot s has at least one query row
    bool split;     // both slots work on the SAME query tile, each on its own part of the tile's KV list
  };
  // The pairs of the last, partial wave are handed out as single tiles (see launch_attention).  A single tile
  // either runs on slot 0 with slot 1 idle, or (p.split_singles) on both slots: the slots then hold the same
  // query rows, walk disjoint halves of the KV list and slot 0's softmax warps merge the two partial results,
  // which halves the length of the tile's dependent QK -> softmax -> PV chain.
  auto decode = [&](int item, int half) {
    Item it;
    it.bh = item / p.n_x;
    const int x = item % p.n_x;
    it.b = it.bh / p.H;
    it.h = it.bh % p.H;
    it.group = 0;
    it.split = false;
    int gend = p.Lq;
    if (MODE == MODE_CSP) {
      it.group = x / p.chunks_per_group;
      const int chunk = x % p.chunks_per_group;
      gend = min(p.Lq, (it.group + 1) * p.bm);
      it.row0[0] = it.group * p.bm + chunk * 256;
    } else {
      it.row0[0] = x * 256;
    }
    it.row0[1] = it.row0[0] + 128;
    it.row_end[0] = it.row_end[1] = gend;
    if (half >= 0) {
      it.row0[0] += half * 128;
      it.split = p.split_singles != 0;
      it.row0[1] = it.split ? it.row0[0] : gend;  // not split: slot 0 takes the tile, slot 1 stays empty
    }
    it.live = (it.row0[0] < gend ? 1u : 0u) | (it.row0[1] < gend ? 2u : 0u);
    return it;
  };
  auto round_info = [&](const uint16_t* l0, const uint16_t* l1, const SchedEntry& e, int r) {
    Round rd;
    rd.has[0] = r < e.n0;
    rd.has[1] = r < e.n1;
    if (MODE == MODE_BLOCK) {
      rd.kvb[0] = rd.has[0] ? (l0[r] & 0xFFF) : 0;
      rd.kvb[1] = rd.has[1] ? (l1[r] & 0xFFF) : 0;
    } else {
      rd.kvb[0] = r;
      rd.kvb[1] = r + e.off1;
    }
    rd.shared = rd.has[0] && rd.has[1] && rd.kvb[0] == rd.kvb[1];
    return rd;
  };
  // Waits for the n-th schedule entry of this CTA; false on abort.
  auto acquire_item = [&](int n, SchedEntry& e, int code) {
    const int slot = n % kSchedStages;
    if (!mbar_wait(&bars->sched_full[slot], (n / kSchedStages) & 1, wc, code)) return false;
    e = bars->sched[slot];
    return true;
  };

  // the 128 threads of softmax warpgroup s meet at named barrier 1 + s
  auto wg_sync = [](int s) {
    if (s == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
    else asm volatile("bar.sync 2, 128;" ::: "memory");
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
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const uint32_t tS = tmem_base + lane_off + (uint32_t)s * 128u;
    const uint32_t tO = tmem_base + lane_off + TM_O + (uint32_t)s * D;
    int n_s = 0;  // S tiles consumed by this slot so far (parity of s_full)
    int n_o = 0;  // items in which this slot produced an output (parity of o_full)
    int n_cs[2] = {0, 0};  // column-sum sweep: S^T tiles read per buffer (parity of cs_full)
    int n_xc[2] = {0, 0};  // split tiles merged so far, by item parity (parity of xchg_full)
    int n_part[2] = {0, 0};  // MODE_DENSE_CS1: tiles reduced per buffer (parity of part_full)
    int n_rowl = 0;          // MODE_DENSE_CS1: items with tiles (parity of rowl_full)
    bool ok = true;

    for (int n = 0; ok; ++n) {
      SchedEntry e;
      ok = __all_sync(0xffffffffu, acquire_item(n, e, DEV_TIMEOUT_SOFTMAX));
      if (!ok || e.item < 0) break;
      const Item im = decode(e.item, e.half);
      const uint16_t* mylist = lists + ((n % kSchedStages) * 2 + s) * kMaxSteps;
      const int row = im.row0[s] + r_in_tile;
      const bool row_ok = row < im.row_end[s];
      const int cnt_total = (MODE == MODE_CSP) ? e.aux : 0;
      const int n_mine = s == 0 ? e.n0 : e.n1;

      float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
      int it = 0;
      if (MODE == MODE_DENSE_CS1 && n_mine > 0) {
        // ---- one sweep with the caller's row statistics.  S is read in the 16x256b shape: a thread holds FOUR
        // query rows (lanes tq, tq + 8, tq + 16, tq + 24 of the warp's window, tq = lane / 4) x 32 columns
        // (8k + 2 tc, + 1; tc = lane % 4), so the column sums start as in-thread adds over the four rows and
        // finish with a 28-shuffle transposing butterfly over the eight threads that share tc.  P goes back to
        // TMEM in the matching 16x128b shape.  p = exp2(s * scale - (M_i + log2 L_i)) is already normalised:
        // no running maximum, no rescale of O; the rows' sums of p are kept so that O and the statistics stay
        // exact for constants that are only approximately this attention's own.
        const int tq = lane >> 2, tc = lane & 3;
        float ncst[4];  // constants of rows tq + 8 i
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int rr = im.row0[s] + quad * 32 + tq + 8 * i;
          float c = -INFINITY;
          if (rr < im.row_end[s]) {
            const int64_t si = (int64_t)im.bh * p.Lq + rr;
            const float Lr = p.L_in[si];
            if (Lr > 0.f) c = -(p.M_in[si] + log2f(Lr));
          }
          ncst[i] = c;
        }
        uint64_t rs2[4] = {0ull, 0ull, 0ull, 0ull};  // packed partial sums of p over this thread's columns, per row
        const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2);
        const int tile = im.row0[s] >> 7;
        float* cs_row = p.cs + im.b * p.cs_sb + im.h * p.cs_sh + (int64_t)(p.cs_pair ? tile >> 1 : tile) * p.cs_st;
        const uint32_t b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
        const int col0 = 8 * ((b4 ? 8 : 0) + (b3 ? 4 : 0) + (b2 ? 2 : 0)) + 2 * tc;  // this thread's first result column
        for (int j = 0; j < n_mine; ++j) {
          ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[s], n_s & 1, wc, DEV_TIMEOUT_SOFTMAX));
          if (!ok) break;
          ++n_s;
          tc_fence_after();
          uint32_t ra[64], rb[64];
          tmem_ld_16x256b_x16(tS, ra);
          tmem_ld_16x256b_x16(tS + (16u << 16), rb);
          tmem_wait_ld();
          const int valid = p.Lkv - j * 128;
          uint64_t acc2[16];
          auto half_tile = [&](const uint32_t (&r)[64], int h, auto masked_tag) {
            constexpr bool MASKED = decltype(masked_tag)::value;
            const uint64_t nA = pack_f32x2(ncst[2 * h], ncst[2 * h]), nB = pack_f32x2(ncst[2 * h + 1], ncst[2 * h + 1]);
            uint32_t pk[32];
#pragma unroll
            for (int kk = 0; kk < 16; ++kk) {
              const uint64_t X = ffma2(pack_f32x2(__uint_as_float(r[4 * kk]), __uint_as_float(r[4 * kk + 1])), sc2, nA);
              const uint64_t Y = ffma2(pack_f32x2(__uint_as_float(r[4 * kk + 2]), __uint_as_float(r[4 * kk + 3])), sc2, nB);
              float x0, x1, y0, y1;
              unpack_f32x2(X, x0, x1);
              unpack_f32x2(Y, y0, y1);
              x0 = fast_exp2(x0); x1 = fast_exp2(x1); y0 = fast_exp2(y0); y1 = fast_exp2(y1);
              if (MASKED) {  // columns past the end of K
                const int c = 8 * kk + 2 * tc;
                if (c >= valid) x0 = y0 = 0.f;
                if (c + 1 >= valid) x1 = y1 = 0.f;
              }
              const uint64_t PX = pack_f32x2(x0, x1), PY = pack_f32x2(y0, y1);
              rs2[2 * h] = fadd2(rs2[2 * h], PX);
              rs2[2 * h + 1] = fadd2(rs2[2 * h + 1], PY);
              acc2[kk] = h == 0 ? fadd2(PX, PY) : fadd2(acc2[kk], fadd2(PX, PY));
              pk[2 * kk] = pack_bf16x2(x0, x1);
              pk[2 * kk + 1] = pack_bf16x2(y0, y1);
            }
            tmem_st_16x128b_x16(tS + ((uint32_t)(16 * h) << 16), pk);
          };
          if (valid < 128) {
            half_tile(ra, 0, std::true_type{});
            half_tile(rb, 1, std::true_type{});
          } else {
            half_tile(ra, 0, std::false_type{});
            half_tile(rb, 1, std::false_type{});
          }
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&bars->p_full[s]);
          // ---- column sums of the warp's 32 rows: transposing butterfly over lane bits 4, 3, 2 (fixed order)
          float a[32];
#pragma unroll
          for (int kk = 0; kk < 16; ++kk) unpack_f32x2(acc2[kk], a[2 * kk], a[2 * kk + 1]);
          float c16[16], d8[8], e4[4];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            c16[i] = (b4 ? a[i + 16] : a[i]) + __shfl_xor_sync(0xffffffffu, b4 ? a[i] : a[i + 16], 16);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            d8[i] = (b3 ? c16[i + 8] : c16[i]) + __shfl_xor_sync(0xffffffffu, b3 ? c16[i] : c16[i + 8], 8);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            e4[i] = (b2 ? d8[i + 4] : d8[i]) + __shfl_xor_sync(0xffffffffu, b2 ? d8[i] : d8[i + 4], 4);
          // e4[0..1]: columns col0, col0 + 1; e4[2..3]: columns col0 + 8, col0 + 9
          const int buf = j & 1;
          float* pw = part + ((s * 2 + buf) * 4 + quad) * 128;
          *reinterpret_cast<float2*>(pw + col0) = make_float2(e4[0], e4[1]);
          *reinterpret_cast<float2*>(pw + col0 + 8) = make_float2(e4[2], e4[3]);
          mbar_arrive(&bars->part_full[s][buf]);
          ok = __all_sync(0xffffffffu, mbar_wait(&bars->part_full[s][buf], n_part[buf] & 1, wc, DEV_TIMEOUT_SOFTMAX));
          if (!ok) break;
          ++n_part[buf];
          const float* pr = part + (s * 2 + buf) * 4 * 128 + r_in_tile;
          const float colsum = ((pr[0] + pr[128]) + pr[256]) + pr[384];
          const int key = j * 128 + r_in_tile;
          if (key < p.Lkv) {
            if (p.cs_pair) atomicAdd(cs_row + key, colsum);  // two addends onto zero: the same bits in either order
            else cs_row[key] = colsum;
          }
          ++it;
        }
        if (!ok) break;
        // the rows' sums of p: over this thread's columns, then over the four threads that share the rows
        float rs[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float x0, x1;
          unpack_f32x2(rs2[i], x0, x1);
          float v = x0 + x1;
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          rs[i] = v;
        }
        if (tc == 0) {
#pragma unroll
          for (int i = 0; i < 4; ++i) rowl[s * 128 + quad * 32 + tq + 8 * i] = rs[i];
        }
        mbar_arrive(&bars->rowl_full[s]);
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->rowl_full[s], n_rowl & 1, wc, DEV_TIMEOUT_SOFTMAX));
        if (!ok) break;
        ++n_rowl;
        l = rowl[s * 128 + r_in_tile];  // this thread's own row from here on (epilogue: thread = row)
        m_ref = m_true = 0.f;
      }
      const int n_first = (stats_given || MODE == MODE_DENSE_CS1) ? 0 : n_mine;
      for (int j = 0; j < n_first; ++j) {
        const int kvb = (MODE == MODE_BLOCK) ? (mylist[j] & 0xFFF) : j + (s == 1 ? e.off1 : 0);
        const uint32_t sub = (MODE == MODE_BLOCK) ? ((uint32_t)mylist[j] >> 12 >> (2 * (r_in_tile >> 6))) & 3u : 3u;
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[s], n_s & 1, wc, DEV_TIMEOUT_SOFTMAX));
        if (!ok) break;  // warp-uniform: the TMEM accesses below are warp-collective
        ++n_s;
        tc_fence_after();

        // raw fp32 bits of the S row, four 32-column chunks kept in registers
        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld_x32(tS + 0, s0);
        tmem_ld_x32(tS + 32, s1);
        tmem_ld_x32(tS + 64, s2);
        tmem_ld_x32(tS + 96, s3);
        tmem_wait_ld();
        if (MODE == MODE_CS_ONLY) {
          // nothing goes back into S_s: the next tile's product may land while this one is exponentiated
          tc_fence_before();
          mbar_arrive(&bars->p_full[s]);
        }

        const int valid = (MODE == MODE_CSP) ? (cnt_total - j * 128) : (p.Lkv - kvb * 128);
        if (valid < 128 || sub != 3u) {
          // columns past the end of K, and (64-wide masks) the column half this row's half does not attend
          const int lo = (sub & 1u) ? 0 : 64;
          const int hi = (sub & 2u) ? valid : min(valid, 64);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i < lo || i >= hi) s0[i] = 0xff800000u;  // -inf
            if (i + 32 < lo || i + 32 >= hi) s1[i] = 0xff800000u;
            if (i + 64 < lo || i + 64 >= hi) s2[i] = 0xff800000u;
            if (i + 96 < lo || i + 96 >= hi) s3[i] = 0xff800000u;
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
          if (MODE != MODE_CS_ONLY && it > 0) {
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
        const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;  // row with nothing to attend yet: all p = 0
        const uint64_t nm2 = pack_f32x2(neg_m, neg_m);
        uint64_t sum_a = 0ull, sum_b = 0ull;  // two packed accumulators = four partial row sums
        if (MODE == MODE_CS_ONLY) {
          exp_sum_chunk(s0, sc2, nm2, sum_a, sum_b);
          exp_sum_chunk(s1, sc2, nm2, sum_a, sum_b);
          exp_sum_chunk(s2, sc2, nm2, sum_a, sum_b);
          exp_sum_chunk(s3, sc2, nm2, sum_a, sum_b);
        } else {
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
        }
        {
          float a0, a1, b0, b1;
          unpack_f32x2(sum_a, a0, a1);
          unpack_f32x2(sum_b, b0, b1);
          l += (a0 + a1) + (b0 + b1);
        }
        if (MODE != MODE_CS_ONLY) {
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&bars->p_full[s]);
        }
        ++it;
      }
      if (!ok) break;

      // ---- epilogue: O / l -> bf16 -> global; row statistics
      const bool split = (MODE == MODE_DENSE || MODE == MODE_BLOCK) && im.split;
      float m_stat = m_true, l_stat = (it > 0 && l > 0.f) ? l * fast_exp2(m_ref - m_true) : 0.f;
      if (MODE == MODE_CSP && row_ok) {
        // Column-sparse: the epilogue adds this row of the accumulate input (or the four rows of the coarser grid
        // it is resized from).  Its 16-byte loads sit between stores they may not pass (o_in may alias o), one
        // exposed memory latency each; bring the lines close while the last P V is still running.
        const __nv_bfloat16* ib = p.o_in + im.b * p.oi_sb + im.h * p.oi_sh;
        if (p.oi_side > 0) {
          const BilinearTaps tp = bilinear_taps(row / p.o_side, row % p.o_side, p.oi_side, p.oi_ratio);
          const int rows4[4] = {tp.r00, tp.r01, tp.r10, tp.r11};
#pragma unroll
          for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int b128 = 0; b128 < D * 2; b128 += 128)
              prefetch_l1(reinterpret_cast<const char*>(ib + (int64_t)rows4[t] * p.oi_sl) + b128);
        } else {
#pragma unroll
          for (int b128 = 0; b128 < D * 2; b128 += 128)
            prefetch_l1(reinterpret_cast<const char*>(ib + (int64_t)row * p.oi_sl) + b128);
        }
      }
      if (MODE != MODE_CS_ONLY) {
        if (it > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full[s], n_o & 1, wc, DEV_TIMEOUT_SOFTMAX));
          if (!ok) break;
          ++n_o;
          tc_fence_after();
        }
        if (split && s == 1) {
          // Second half of a split tile: hand this row's reference maximum, denominator and true maximum to
          // slot 0's warpgroup, which reads both accumulators out of TMEM and merges them.
          float* x = xchg + (n & 1) * 3 * 128;
          x[r_in_tile] = (it > 0) ? m_ref : -INFINITY;
          x[128 + r_in_tile] = (it > 0) ? l : 0.f;
          x[256 + r_in_tile] = m_true;
          tc_fence_before();
          mbar_arrive(&bars->xchg_full[n & 1]);
        } else {
          float w0 = (it > 0 && l > 0.f) ? (1.0f / l) : 0.f, w1 = 0.f;  // out = O_0 * w0 + O_1 * w1
          bool other = false;  // slot 1 holds a partial result of this tile
          if (split) {
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->xchg_full[n & 1], n_xc[n & 1] & 1, wc, DEV_TIMEOUT_SOFTMAX));
            if (!ok) break;
            ++n_xc[n & 1];
            tc_fence_after();
            const float* x = xchg + (n & 1) * 3 * 128;
            const float m1 = x[r_in_tile], l1 = x[128 + r_in_tile], mt1 = x[256 + r_in_tile];
            other = e.n1 > 0;
            const float m0 = (it > 0) ? m_ref : -INFINITY;
            const float mm = fmaxf(m0, m1);
            const float a0 = (m0 == -INFINITY) ? 0.f : fast_exp2(m0 - mm);
            const float a1 = (m1 == -INFINITY) ? 0.f : fast_exp2(m1 - mm);
            const float lt = a0 * l + a1 * l1;
            const float inv = lt > 0.f ? 1.0f / lt : 0.f;
            w0 = a0 * inv;
            w1 = a1 * inv;
            m_stat = fmaxf(m_true, mt1);
            l_stat = lt > 0.f ? lt * fast_exp2(mm - m_stat) : 0.f;
          }
          const uint32_t tO1 = tmem_base + lane_off + TM_O + (uint32_t)D;  // slot 1's accumulator (split tiles)
          __nv_bfloat16* orow = p.o + im.b * p.o_sb + im.h * p.o_sh + (int64_t)row * p.o_sl;
          const __nv_bfloat16* irow =
              (MODE == MODE_CSP) ? (p.o_in + im.b * p.oi_sb + im.h * p.oi_sh + (int64_t)row * p.oi_sl) : nullptr;
          // accumulate input taken from a coarser token grid: this row's four source tokens and weights
          const bool resize = (MODE == MODE_CSP) && p.oi_side > 0;
          BilinearTaps tp = {};
          const __nv_bfloat16* ibase = nullptr;
          if (resize && row_ok) {
            tp = bilinear_taps(row / p.o_side, row % p.o_side, p.oi_side, p.oi_ratio);
            ibase = p.o_in + im.b * p.oi_sb + im.h * p.oi_sh;
          }
          if (kRegisterEpilogue) {
            // All of O_s goes to registers at once (the tile's S registers are dead here): one exposed TMEM
            // latency instead of one per 32 columns, the accumulator is released before any arithmetic, and a row
            // leaves in 32-byte stores.
            uint32_t ra[D / 32][32];
            if (it > 0) {
#pragma unroll
              for (int c = 0; c < D / 32; ++c) tmem_ld_x32(tO + c * 32, ra[c]);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int c = 0; c < D / 32; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) ra[c][i] = 0u;
            }
            float wf = w0;
            if (split && other) {
#pragma unroll
              for (int c = 0; c < D / 32; ++c) {
                uint32_t r1[32];
                tmem_ld_x32(tO1 + c * 32, r1);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  ra[c][i] = __float_as_uint(fmaf(__uint_as_float(r1[i]), w1, __uint_as_float(ra[c][i]) * w0));
              }
              wf = 1.0f;
            }
            // O has been read out of TMEM: the MMA warp may overwrite it for the next item.  For a split tile
            // this warpgroup read slot 1's accumulator too and releases it in its owner's stead.
            tc_fence_before();
            if (it > 0) mbar_arrive(&bars->o_empty[s]);
            if (split && other) mbar_arrive(&bars->o_empty[1]);
            if (row_ok) {
#pragma unroll
              for (int c = 0; c < D / 32; ++c) {
#pragma unroll
                for (int h8 = 0; h8 < 2; ++h8) {
                  uint32_t w[8];
#pragma unroll
                  for (int i = 0; i < 8; ++i)
                    w[i] = pack_bf16x2(__uint_as_float(ra[c][h8 * 16 + 2 * i]) * wf,
                                       __uint_as_float(ra[c][h8 * 16 + 2 * i + 1]) * wf);
                  if (p.o_align32) {
                    st_global_v8(orow + c * 32 + h8 * 16, w);
                  } else {
                    *reinterpret_cast<uint4*>(orow + c * 32 + h8 * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(orow + c * 32 + h8 * 16 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                  }
                }
              }
            }
          } else {
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
            if (split && other) {
              uint32_t r1[32];
              tmem_ld_x32(tO1 + c * 32, r1);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i)
                r[i] = __float_as_uint(fmaf(__uint_as_float(r1[i]), w1, __uint_as_float(r[i]) * w0));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * w0);
            }
            if (c == D / 32 - 1) {
              // O has been read out of TMEM: the MMA warp may overwrite it for the next item.  For a split tile
              // this warpgroup read slot 1's accumulator too and releases it in its owner's stead.
              tc_fence_before();
              if (it > 0) mbar_arrive(&bars->o_empty[s]);
              if (split && other) mbar_arrive(&bars->o_empty[1]);
            }
            if (row_ok) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  w[i] = pack_bf16x2(__uint_as_float(r[q4 * 8 + 2 * i]), __uint_as_float(r[q4 * 8 + 2 * i + 1]));
                if (MODE == MODE_CSP) {
                  // out = bf16(o_in + o_scale * bf16(delta)): same rounding points as the reference's
                  // `o + o_delta * o_scale` on bf16 tensors (kernels/sparse_attn/sparse_attn_ops.py:288).
                  uint4 prev;
                  if (resize) {
                    const __nv_bfloat16* ib = ibase + c * 32 + q4 * 8;
                    prev = bilinear_mix8(tp, *reinterpret_cast<const uint4*>(ib + (int64_t)tp.r00 * p.oi_sl),
                                         *reinterpret_cast<const uint4*>(ib + (int64_t)tp.r01 * p.oi_sl),
                                         *reinterpret_cast<const uint4*>(ib + (int64_t)tp.r10 * p.oi_sl),
                                         *reinterpret_cast<const uint4*>(ib + (int64_t)tp.r11 * p.oi_sl));
                  } else {
                    prev = *reinterpret_cast<const uint4*>(irow + c * 32 + q4 * 8);
                  }
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
          }
        }
      }
      if (stats_given) {
        // M = row maximum, L = row sum relative to it (both in log2 units of the scaled scores)
        const int64_t si = (int64_t)im.bh * p.Lq + row;
        m_ref = row_ok ? p.M_in[si] : -INFINITY;
        l = row_ok ? p.L_in[si] : 0.f;
      } else if (MODE == MODE_DENSE_CS1) {
        // statistics out: the given pair with L corrected by the measured row sum, so that 2^M * L is this
        // attention's true normaliser even when the given constants were another pass's
        if (row_ok && p.L) {
          const int64_t si = (int64_t)im.bh * p.Lq + row;
          if (p.M) p.M[si] = p.M_in[si];
          p.L[si] = p.L_in[si] * l;
        }
      } else if (row_ok && MODE != MODE_CSP && !(split && s == 1)) {
        const int64_t si = (int64_t)im.bh * p.Lq + row;
        if (p.M) p.M[si] = m_stat;
        if (p.L) p.L[si] = l_stat;
      }
      if (kHasCs && n_mine > 0) {
        // ---- second sweep: column sums of this slot's query tile.  S^T = K Q^T lands in S_s with one KEY per
        // TMEM lane, so this thread owns key column j*128 + r_in_tile and sums the 128 probabilities
        // p_i = exp2(s_i * scale - (M_i + log2 L_i)) of the tile's queries in registers.
        negc[s * 128 + r_in_tile] = (row_ok && l > 0.f) ? -(m_ref + log2f(l)) : -INFINITY;
        wg_sync(s);  // the warpgroup's 128 constants are in place
        const float4* nc4 = reinterpret_cast<const float4*>(negc + s * 128);
        // a tile with fewer than 128 queries carries -inf constants, which the polynomial cannot take
        const bool full_tile = im.row_end[s] - im.row0[s] >= 128;
        const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2);
        const int tile = im.row0[s] >> 7;
        float* cs_row = p.cs + im.b * p.cs_sb + im.h * p.cs_sh + (int64_t)(p.cs_pair ? tile >> 1 : tile) * p.cs_st;
        // the sweep over the KV tiles, compiled twice: the exponential mix is a compile-time choice (a run-time
        // choice per chunk measured 20 % slower)
        auto cs_sweep = [&](auto poly_tag) -> bool {
          constexpr uint32_t POLY = decltype(poly_tag)::value;
          for (int j = 0; j < n_mine; ++j) {
            // tile j of the sweep sits in buffer j % kCsBufs: S_s, or the (by now written out) O region
            const int buf = j % kCsBufs;
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->cs_full[s][buf], n_cs[buf] & 1, wc, DEV_TIMEOUT_SOFTMAX));
            if (!ok) return false;
            ++n_cs[buf];
            tc_fence_after();
            const uint32_t tT = buf == 0 ? tS : tmem_base + lane_off + TM_O + (uint32_t)s * 128u;
            float acc = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t r[32];
              tmem_ld_x32(tT + c * 32, r);
              tmem_wait_ld();
              acc += colsum_chunk<POLY>(r, nc4 + c * 8, sc2);
            }
            // S^T has been read: the MMA warp may overwrite the buffer with the tile after the next
            tc_fence_before();
            mbar_arrive(&bars->cs_empty[s][buf]);
            const int key = j * 128 + r_in_tile;
            if (key < p.Lkv) {
              // two addends onto zero give the same bits in either order
              if (p.cs_pair) atomicAdd(cs_row + key, acc);
              else cs_row[key] = acc;
            }
          }
          return true;
        };
        ok = full_tile ? cs_sweep(std::integral_constant<uint32_t, kCsPolyMask>{})
                       : cs_sweep(std::integral_constant<uint32_t, 0u>{});
        if (!ok) break;
        wg_sync(s);  // nobody still reads the constants
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->sched_empty[n % kSchedStages]);
    }
  } else if (warp == 8) {
    // ============================================================ K (and Q) loader
    setmaxnreg_dec<kRegsOther>();
    bool ok = true;
    int kc = 0;       // K tiles issued so far (stage = kc % kStages)
    int nq_items = 0; // items with at least one step (parity of q_full / q_empty)
    const bool issuer = (MODE == MODE_CSP) || lane == 0;
    if (issuer) {
      for (int n = 0; ok; ++n) {
        SchedEntry e;
        ok = acquire_item(n, e, DEV_TIMEOUT_PRODUCER);
        if (MODE == MODE_CSP) ok = __all_sync(0xffffffffu, ok);
        if (!ok || e.item < 0) break;
        const Item im = decode(e.item, e.half);
        const uint16_t* l0 = lists + ((n % kSchedStages) * 2) * kMaxSteps;
        const uint16_t* l1 = l0 + kMaxSteps;
        const int rounds = max(e.n0, e.n1);
        if (rounds > 0) {
          if (lane == 0) {
            ok = mbar_wait(&bars->q_empty, (nq_items & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER);
            if (ok) {
              mbar_arrive_expect_tx(&bars->q_full, 2 * SM::kTile);
              for (int s = 0; s < 2; ++s)
                for (int sub = 0; sub < NSUB; ++sub)
                  tma_load_4d(sQ + s * SM::kTile + sub * 16384, &tmQ, &bars->q_full, sub * 64, im.row0[s], im.h, im.b);
            }
          }
          if (MODE == MODE_CSP) ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ++nq_items;
        }
        if (MODE != MODE_CSP) {
          // MODE_DENSE_CS streams the K tiles a second time for the column-sum sweep
          const int sweeps = (kHasCs && !stats_given) ? 2 : 1;
          for (int rr = 0; rr < sweeps * rounds && ok; ++rr) {
            const int r = rr < rounds ? rr : rr - rounds;
            const Round rd = round_info(l0, l1, e, r);
            for (int s = 0; s < 2; ++s) {
              if (!rd.has[s] || (s == 1 && rd.shared)) continue;
              const int st = kc % kStages;
              ok = mbar_wait(&bars->k_empty[st], ((kc / kStages) & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER);
              if (!ok) break;
              mbar_arrive_expect_tx(&bars->k_full[st], SM::kTile);
              for (int sub = 0; sub < NSUB; ++sub)
                tma_load_4d(sK + st * SM::kTile + sub * 16384, &tmK, &bars->k_full[st], sub * 64, rd.kvb[s] * 128, im.h,
                            im.b);
              ++kc;
            }
          }
        } else {
          const int32_t* idx = p.indices + im.b * p.i_sb + im.h * p.i_sh + (int64_t)im.group * p.i_sg;
          const __nv_bfloat16* kbase = p.k + im.b * p.k_sb + im.h * p.k_sh;
          int kv[4];
          if (rounds > 0) gather_rows_of_tile(kv, idx, e.aux, 0, p.Lkv, lane, p.status);
          for (int j = 0; j < rounds; ++j) {
            const int st = kc % kStages;
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->k_empty[st], ((kc / kStages) & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER));
            if (!ok) break;
            if (tile_is_run(kv, e.aux, j, p.Lkv, lane)) {
              // 128 consecutive keys (the local band of a list): one tile copy instead of 2048 row pieces
              if (lane == 0) {
                mbar_arrive_expect_tx(&bars->k_full[st], SM::kTile);
                for (int sub = 0; sub < NSUB; ++sub)
                  tma_load_4d(sK + st * SM::kTile + sub * 16384, &tmK, &bars->k_full[st], sub * 64, kv[0], im.h, im.b);
              } else {
                mbar_arrive(&bars->k_full[st]);
              }
            } else {
              gather_tile<D>(smem_u32(sK + st * SM::kTile), kbase, p.k_sl, kv, lane);
              // each lane's arrival follows its own copies; nobody waits here (the MMA warp fences the proxies)
              cp_async_mbar_arrive(&bars->k_full[st]);
            }
            if (j + 1 < rounds) gather_rows_of_tile(kv, idx, e.aux, j + 1, p.Lkv, lane, p.status);
            ++kc;
          }
        }
        if (!ok) break;
        if (lane == 0) mbar_arrive(&bars->sched_empty[n % kSchedStages]);
      }
      if (MODE == MODE_CSP) cp_async_wait<0>();  // drains on abort too
      // Drain on abort: copies in flight must land before the CTA's shared memory is released.
      if (lane == 0 && bars->abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        if (nq_items > 0)
          while (!mbar_try_wait(&bars->q_full, (nq_items - 1) & 1) && globaltimer_ns() - t0 < 2000000000ull) {
          }
        if (MODE != MODE_CSP) {
          for (int c = max(0, kc - kStages); c < kc; ++c) {
            const uint64_t t1 = globaltimer_ns();
            while (!mbar_try_wait(&bars->k_full[c % kStages], (c / kStages) & 1) &&
                   globaltimer_ns() - t1 < 2000000000ull) {
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ============================================================ V loader
    setmaxnreg_dec<kRegsOther>();
    bool ok = true;
    int vc = 0;
    const bool issuer = (MODE == MODE_CSP) || lane == 0;
    if (issuer) {
      for (int n = 0; ok; ++n) {
        SchedEntry e;
        ok = acquire_item(n, e, DEV_TIMEOUT_PRODUCER);
        if (MODE == MODE_CSP) ok = __all_sync(0xffffffffu, ok);
        if (!ok || e.item < 0) break;
        const Item im = decode(e.item, e.half);
        const uint16_t* l0 = lists + ((n % kSchedStages) * 2) * kMaxSteps;
        const uint16_t* l1 = l0 + kMaxSteps;
        const int rounds = max(e.n0, e.n1);
        if (MODE == MODE_CS_ONLY) {
          // no V in this mode: the warp only follows the schedule
        } else if (MODE != MODE_CSP) {
          for (int r = 0; r < rounds && ok; ++r) {
            const Round rd = round_info(l0, l1, e, r);
            for (int s = 0; s < 2; ++s) {
              if (!rd.has[s] || (s == 1 && rd.shared)) continue;
              const int st = vc % kStages;
              ok = mbar_wait(&bars->v_empty[st], ((vc / kStages) & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER);
              if (!ok) break;
              mbar_arrive_expect_tx(&bars->v_full[st], SM::kTile);
              for (int sub = 0; sub < NSUB; ++sub)
                tma_load_4d(sV + st * SM::kTile + sub * 16384, &tmV, &bars->v_full[st], sub * 64, rd.kvb[s] * 128, im.h,
                            im.b);
              ++vc;
            }
          }
        } else {
          const int32_t* idx = p.indices + im.b * p.i_sb + im.h * p.i_sh + (int64_t)im.group * p.i_sg;
          const __nv_bfloat16* vbase = p.v + im.b * p.v_sb + im.h * p.v_sh;
          int kv[4];
          if (rounds > 0) gather_rows_of_tile(kv, idx, e.aux, 0, p.Lkv, lane, nullptr);
          for (int j = 0; j < rounds; ++j) {
            const int st = vc % kStages;
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->v_empty[st], ((vc / kStages) & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER));
            if (!ok) break;
            if (tile_is_run(kv, e.aux, j, p.Lkv, lane)) {
              if (lane == 0) {
                mbar_arrive_expect_tx(&bars->v_full[st], SM::kTile);
                for (int sub = 0; sub < NSUB; ++sub)
                  tma_load_4d(sV + st * SM::kTile + sub * 16384, &tmV, &bars->v_full[st], sub * 64, kv[0], im.h, im.b);
              } else {
                mbar_arrive(&bars->v_full[st]);
              }
            } else {
              gather_tile<D>(smem_u32(sV + st * SM::kTile), vbase, p.v_sl, kv, lane);
              cp_async_mbar_arrive(&bars->v_full[st]);
            }
            if (j + 1 < rounds) gather_rows_of_tile(kv, idx, e.aux, j + 1, p.Lkv, lane, nullptr);
            ++vc;
          }
        }
        if (!ok) break;
        if (lane == 0) mbar_arrive(&bars->sched_empty[n % kSchedStages]);
      }
      if (MODE == MODE_CSP) cp_async_wait<0>();
      if (MODE != MODE_CSP && lane == 0 && bars->abort_flag) {
        for (int c = max(0, vc - kStages); c < vc; ++c) {
          const uint64_t t1 = globaltimer_ns();
          while (!mbar_try_wait(&bars->v_full[c % kStages], (c / kStages) & 1) &&
                 globaltimer_ns() - t1 < 2000000000ull) {
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 10) {
    // ============================================================ MMA issuer (one thread)
    setmaxnreg_dec<kRegsOther>();
    // Every lane runs the (warp-uniform) bookkeeping; lane 0 alone issues the MMAs, commits and arrivals.
    const uint32_t leader = lane == 0 ? 1u : 0u;
    {
      bool ok = true;
      // Descriptor words: the high word is the same for every operand tile, the low word is the tile's
      // base plus (byte offset >> 4) of the stage and of the 16-element K step.
      constexpr uint32_t DESC_HI = sw128_desc_hi(1024);
      constexpr uint32_t TILE16 = SM::kTile >> 4;
      const uint32_t q_lo = sw128_desc_lo(smem_u32(sQ), 16);
      const uint32_t k_lo = sw128_desc_lo(smem_u32(sK), 16);
      const uint32_t v_lo = sw128_desc_lo(smem_u32(sV), 16384);
      int kc = 0, vc = 0;        // K / V tiles consumed so far
      int nq_items = 0;          // items with steps (parity of q_full)
      int n_p[2] = {0, 0};       // P tiles consumed per slot (parity of p_full)
      int n_o[2] = {0, 0};       // items in which the slot produced an output (parity of o_empty)
      int n_cst[2][2] = {{0, 0}, {0, 0}};  // column-sum sweep: S^T tiles issued per [slot][buffer]
      for (int n = 0; ok; ++n) {
        SchedEntry e;
        ok = acquire_item(n, e, DEV_TIMEOUT_MMA);
        if (!ok || e.item < 0) break;
        const Item im = decode(e.item, e.half);
        const uint16_t* l0 = lists + ((n % kSchedStages) * 2) * kMaxSteps;
        const uint16_t* l1 = l0 + kMaxSteps;
        const int rounds = max(e.n0, e.n1);
        if (rounds > 0) {
          ok = mbar_wait(&bars->q_full, nq_items & 1, wc, DEV_TIMEOUT_MMA);
          if (!ok) break;
          ++nq_items;
        }
        Round prev;
        prev.has[0] = prev.has[1] = prev.shared = false;
        prev.kvb[0] = prev.kvb[1] = 0;
        int pvs[2] = {0, 0}, pvp[2] = {0, 0};  // V stage / parity of the previous round, per slot
        int npv[2] = {0, 0};
        const int rounds_first = stats_given ? 0 : rounds;
        for (int r = 0; r <= rounds_first && ok; ++r) {
          Round cur;
          cur.has[0] = cur.has[1] = cur.shared = false;
          cur.kvb[0] = cur.kvb[1] = 0;
          if (r < rounds_first) cur = round_info(l0, l1, e, r);
          // stages of this round's tiles (same order as the loaders issue them)
          int ks[2] = {0, 0}, kp[2] = {0, 0}, vs[2] = {0, 0}, vp[2] = {0, 0};
          for (int s = 0; s < 2; ++s) {
            if (!cur.has[s]) continue;
            if (s == 1 && cur.shared) {
              ks[1] = ks[0]; kp[1] = kp[0]; vs[1] = vs[0]; vp[1] = vp[0];
              continue;
            }
            ks[s] = kc % kStages; kp[s] = (kc / kStages) & 1; ++kc;
            vs[s] = vc % kStages; vp[s] = (vc / kStages) & 1; ++vc;
          }
          for (int s = 0; s < 2 && ok; ++s) {
            if (prev.has[s] && MODE == MODE_CS_ONLY) {
              // statistics sweep: no PV; S_s is free again once the softmax warps have read the last product
              ok = mbar_wait(&bars->p_full[s], n_p[s] & 1, wc, DEV_TIMEOUT_MMA);
              if (!ok) break;
              ++n_p[s];
            } else if (prev.has[s]) {
              if (!(s == 1 && prev.shared)) {
                ok = mbar_wait(&bars->v_full[pvs[s]], pvp[s], wc, DEV_TIMEOUT_MMA);
                if (!ok) break;
              }
              if (npv[s] == 0) {
                // first PV of the item overwrites O_s: the previous item's epilogue must have read it
                ok = mbar_wait(&bars->o_empty[s], (n_o[s] & 1) ^ 1, wc, DEV_TIMEOUT_MMA);
                if (!ok) break;
              }
              ok = mbar_wait(&bars->p_full[s], n_p[s] & 1, wc, DEV_TIMEOUT_MMA);
              if (!ok) break;
              ++n_p[s];
              // column-sparse: V came by cp.async (generic proxy), the MMA reads it through the async proxy
              if (MODE == MODE_CSP) fence_proxy_async_smem();
              tc_fence_after();
              const uint32_t tP = tmem_base + (uint32_t)s * 128u;
              const uint32_t tOs = tmem_base + TM_O + (uint32_t)s * D;
              const uint32_t vb = v_lo + (uint32_t)pvs[s] * TILE16;
              umma_ts_if(leader, tOs, tP, vb, DESC_HI, IDESC_PV, npv[s] > 0 ? 1u : 0u);
#pragma unroll
              for (int ks8 = 1; ks8 < 8; ++ks8)
                umma_ts_if(leader, tOs, tP + ks8 * 8, vb + ks8 * 128, DESC_HI, IDESC_PV, 1u);
              ++npv[s];
              // release the V stage after its last user
              if (!(s == 0 && prev.shared)) umma_commit_if(leader, &bars->v_empty[pvs[s]]);
            }
            if (cur.has[s]) {
              if (!(s == 1 && cur.shared)) {
                ok = mbar_wait(&bars->k_full[ks[s]], kp[s], wc, DEV_TIMEOUT_MMA);
                if (!ok) break;
                if (MODE == MODE_CSP) fence_proxy_async_smem();
                tc_fence_after();
              }
              const uint32_t tSs = tmem_base + (uint32_t)s * 128u;
              const uint32_t qa = q_lo + (uint32_t)s * TILE16, kb = k_lo + (uint32_t)ks[s] * TILE16;
#pragma unroll
              for (int kq = 0; kq < KSTEPS_QK; ++kq) {
                const uint32_t koff = (kq >> 2) * 1024 + (kq & 3) * 2;  // (byte offset of the K step) >> 4
                umma_ss_if(leader, tSs, qa + koff, DESC_HI, kb + koff, DESC_HI, IDESC_QK, kq > 0 ? 1u : 0u);
              }
              umma_commit_if(leader, &bars->s_full[s]);
              if (!(s == 0 && cur.shared)) umma_commit_if(leader, &bars->k_empty[ks[s]]);
            }
          }
          if (!ok) break;
          prev = cur;
          pvs[0] = vs[0]; pvs[1] = vs[1]; pvp[0] = vp[0]; pvp[1] = vp[1];
        }
        if (!ok) break;
        for (int s = 0; s < 2; ++s) {
          if (npv[s] > 0) {
            umma_commit_if(leader, &bars->o_full[s]);
            ++n_o[s];
          }
        }
        if (kHasCs) {
          // ---- column-sum sweep: S_s^T = K Q_s^T per KV tile (the operands swap roles, the tiles stay where
          // they are); a slot's next product waits until its softmax warps have read the previous one.
          for (int r = 0; r < rounds && ok; ++r) {
            const Round cur = round_info(l0, l1, e, r);
            int ks = 0, kp = 0;
            if (cur.has[0] || cur.has[1]) {
              ks = kc % kStages;
              kp = (kc / kStages) & 1;
              ++kc;
            }
            const int buf = r % kCsBufs;
            bool waited = false;
            for (int s = 0; s < 2 && ok; ++s) {
              if (!cur.has[s]) continue;
              // the buffer is free once the softmax warps have read the tile before the previous one out of it
              if (n_cst[s][buf] > 0) {
                ok = mbar_wait(&bars->cs_empty[s][buf], (n_cst[s][buf] - 1) & 1, wc, DEV_TIMEOUT_MMA);
                if (!ok) break;
              }
              if (kCsBufs == 2 && r == 1) {
                // first use of the second buffer, which lies over the O accumulators (over both slots' when the
                // head dimension is 64): this item's epilogues must have read them
                for (int t = 0; t < 2 && ok; ++t)
                  if (t == s || D == 64) ok = mbar_wait(&bars->o_empty[t], (n_o[t] & 1) ^ 1, wc, DEV_TIMEOUT_MMA);
                if (!ok) break;
              }
              if (!waited) {
                ok = mbar_wait(&bars->k_full[ks], kp, wc, DEV_TIMEOUT_MMA);
                if (!ok) break;
                waited = true;
              }
              tc_fence_after();
              const uint32_t tT = tmem_base + (buf == 0 ? (uint32_t)s * 128u : TM_O + (uint32_t)s * 128u);
              const uint32_t qb = q_lo + (uint32_t)s * TILE16, ka = k_lo + (uint32_t)ks * TILE16;
#pragma unroll
              for (int kq = 0; kq < KSTEPS_QK; ++kq) {
                const uint32_t koff = (kq >> 2) * 1024 + (kq & 3) * 2;
                umma_ss_if(leader, tT, ka + koff, DESC_HI, qb + koff, DESC_HI, IDESC_QK, kq > 0 ? 1u : 0u);
              }
              umma_commit_if(leader, &bars->cs_full[s][buf]);
              ++n_cst[s][buf];
              if (s == 1 || !cur.has[1]) umma_commit_if(leader, &bars->k_empty[ks]);  // last reader of the K stage
            }
          }
          // the next item's attention sweep writes S_s and O_s again: the softmax warps' last reads first
          for (int s = 0; s < 2 && ok; ++s)
            for (int b = 0; b < 2 && ok; ++b)
              if (n_cst[s][b] > 0) ok = mbar_wait(&bars->cs_empty[s][b], (n_cst[s][b] - 1) & 1, wc, DEV_TIMEOUT_MMA);
          if (!ok) break;
        }
        if (rounds > 0) umma_commit_if(leader, &bars->q_empty);
        if (lane == 0) mbar_arrive(&bars->sched_empty[n % kSchedStages]);
      }
      // TMEM must not be freed (nor the CTA retire) while an MMA is still in flight, also on abort.
      if (lane == 0) {
        umma_commit(&bars->mma_done);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&bars->mma_done, 0)) {
          if (globaltimer_ns() - t0 > 2000000000ull) {
            if (p.status) atomicCAS(p.status, 0, (int)DEV_TIMEOUT_DRAIN);
            break;
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ============================================================ scheduler (warp 11)
    // Hands out work items from a global counter and builds each item's KV-tile list, one item ahead
    // of the slowest role.  The counter pair resets itself when the last CTA leaves.
    setmaxnreg_dec<kRegsOther>();
    // Everything before this point (barriers, TMEM, descriptors) touched no global memory and may have run
    // under the tail of the grid before this one in the stream; the work counter, the inputs and the output
    // are only touched after that grid has completed.  Every other role starts from an item this warp publishes.
    griddep_wait();
    bool ok = true;
    for (int n = 0; ok; ++n) {
      const int slot = n % kSchedStages;
      ok = __all_sync(0xffffffffu,
                      mbar_wait(&bars->sched_empty[slot], ((n / kSchedStages) & 1) ^ 1, wc, DEV_TIMEOUT_PRODUCER));
      if (!ok) break;
      int item = -1, half = -1;
      if (lane == 0) {
        const int idx = atomicAdd(p.sched_counter, 1);
        if (idx < p.total_items) {
          // schedule positions [0, n_pair_items) are whole pairs; the rest are the two tiles of each later pair
          int pos = idx;
          if (idx >= p.n_pair_items) {
            const int tile = 2 * p.n_pair_items + (idx - p.n_pair_items);
            pos = tile >> 1;
            half = tile & 1;
          }
          item = p.work_order ? p.work_order[pos] : pos;
        }
      }
      item = __shfl_sync(0xffffffffu, item, 0);
      half = __shfl_sync(0xffffffffu, half, 0);
      int n0 = 0, n1 = 0, aux = 0, off1 = 0;
      if (item >= 0) {
        const Item im = decode(item, half);
        // The item's Q tiles are read once in the whole launch, so they come from HBM, and their load sits
        // between two items with nothing to overlap it: start them towards L2 now, one item ahead.
        if (lane < 2 * NSUB && ((im.live >> (lane / NSUB)) & 1u) && !(im.split && lane >= NSUB))
          tma_prefetch_l2_4d(&tmQ, (lane % NSUB) * 64, lane < NSUB ? im.row0[0] : im.row0[1], im.h, im.b);
        uint16_t* l0 = lists + (slot * 2) * kMaxSteps;
        uint16_t* l1 = l0 + kMaxSteps;
        if (MODE == MODE_BLOCK) {
          // list entry: KV tile (12 bits) | sub-tile bits << 12.  Sub-tile bit (2*rh + ch) is set when the
          // 64-row half rh of the query tile attends the 64-column half ch of the KV tile; a 128-wide
          // mask sets all four.
          const uint8_t* mb = p.mask + im.b * p.m_sb + im.h * p.m_sh;
          const uint32_t lt = (1u << lane) - 1u;
          auto sub_bits = [&](int qtile, int j) -> uint32_t {
            if (p.mask_block == 128) return mb[(int64_t)qtile * p.m_sq + j] ? 0xFu : 0u;
            uint32_t bits = 0;
#pragma unroll
            for (int rh = 0; rh < 2; ++rh) {
              const int qr = 2 * qtile + rh;
              if (qr >= p.nq_mask) continue;
              const uint8_t* row = mb + (int64_t)qr * p.m_sq;
              if (row[2 * j]) bits |= 1u << (2 * rh);
              if (2 * j + 1 < p.nk_mask && row[2 * j + 1]) bits |= 1u << (2 * rh + 1);
            }
            return bits;
          };
          const int qt0 = im.row0[0] >> 7, qt1 = im.row0[1] >> 7;
          // Tiles that both slots want come first, in the same positions of both lists, so that they are
          // loaded once (a round shares a tile when both lists name it at the same position); the tiles
          // only one slot wants follow.  Ascending within each class.  A split tile has one list (slot 0's).
          for (int pass = 0; pass < 2; ++pass) {
            for (int base = 0; base < p.nkb; base += 32) {
              const int j = base + lane;
              uint32_t b0 = (j < p.nkb && (im.live & 1u)) ? sub_bits(qt0, j) : 0u;
              uint32_t b1 = (j < p.nkb && (im.live & 2u) && !im.split) ? sub_bits(qt1, j) : 0u;
              const bool both = b0 != 0 && b1 != 0;
              if (both != (pass == 0)) b0 = b1 = 0u;
              const uint32_t v0 = __ballot_sync(0xffffffffu, b0 != 0), v1 = __ballot_sync(0xffffffffu, b1 != 0);
              const int p0 = n0 + __popc(v0 & lt), p1 = n1 + __popc(v1 & lt);
              if (b0 && p0 < kMaxSteps) l0[p0] = (uint16_t)(j | (b0 << 12));
              if (b1 && p1 < kMaxSteps) l1[p1] = (uint16_t)(j | (b1 << 12));
              n0 += __popc(v0);
              n1 += __popc(v1);
            }
          }
          n0 = min(n0, kMaxSteps);
          n1 = min(n1, kMaxSteps);
          if (im.split) {
            // slot 0 keeps the first half of the tile's list, slot 1 gets the rest
            const int all = n0;
            n0 = (all + 1) / 2;
            n1 = all - n0;
            __syncwarp();
            for (int i = lane; i < n1; i += 32) l1[i] = l0[n0 + i];
          }
        } else {
          int n = p.nkb;
          if (MODE == MODE_CSP) {
            aux = p.counts[im.b * p.c_sb + im.h * p.c_sh + im.group];
            n = (aux + 127) / 128;
          }
          n0 = (im.live & 1u) ? n : 0;
          n1 = (im.live & 2u) ? n : 0;
          if (im.split && n0 > 0) {
            n0 = (n + 1) / 2;
            n1 = n - n0;
            off1 = n0;
          }
        }
      }
      __syncwarp();
      if (lane == 0) {
        bars->sched[slot].item = item;
        bars->sched[slot].half = half;
        bars->sched[slot].off1 = off1;
        bars->sched[slot].n0 = n0;
        bars->sched[slot].n1 = n1;
        bars->sched[slot].aux = aux;
        mbar_arrive(&bars->sched_full[slot]);
      }
      if (item < 0) break;
    }
    if (lane == 0) {
      __threadfence();
      if (atomicAdd(p.sched_counter + 1, 1) == (int)gridDim.x - 1) {
        p.sched_counter[0] = 0;
        p.sched_counter[1] = 0;
        __threadfence();
      }
    }
    __syncwarp();
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
                cudaStream_t stream, bool serialize_launch) {
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
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Smem<D>::kDynamic;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = serialize_launch ? 0 : 1;
  LVAR_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tq, tk, tv, p));
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

template <int D>
int launch_d(int mode, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
             dim3 grid, cudaStream_t stream, bool serialize_launch) {
  switch (mode) {
    case MODE_DENSE: return launch_mode<D, MODE_DENSE>(tq, tk, tv, p, grid, stream, serialize_launch);
    case MODE_BLOCK: return launch_mode<D, MODE_BLOCK>(tq, tk, tv, p, grid, stream, serialize_launch);
    case MODE_DENSE_CS: return launch_mode<D, MODE_DENSE_CS>(tq, tk, tv, p, grid, stream, serialize_launch);
    case MODE_CS_ONLY: return launch_mode<D, MODE_CS_ONLY>(tq, tk, tv, p, grid, stream, serialize_launch);
    case MODE_DENSE_CS1: return launch_mode<D, MODE_DENSE_CS1>(tq, tk, tv, p, grid, stream, serialize_launch);
    default: return launch_mode<D, MODE_CSP>(tq, tk, tv, p, grid, stream, serialize_launch);
  }
}

}  // namespace

// mode: an AttnMode, or MODE_CS_ONLY + 1 for the column sums from row statistics the caller supplies in
// a->M / a->L.  MODE_DENSE_CS1 reads its row statistics from a->M_in / a->L_in.
int launch_attention(const lvar_attn_args* a, int mode, cudaStream_t stream) {
  LVAR_REQUIRE(a != nullptr, LVAR_ERR_ARG, "null argument block");
  const bool stats_given = mode == MODE_CS_ONLY + 1;
  if (stats_given) mode = MODE_CS_ONLY;
  LVAR_REQUIRE(a->D == 64 || a->D == 128, LVAR_ERR_UNSUPPORTED, "Head dimension must be 64 or 128 (got %d)", a->D);
  LVAR_REQUIRE(a->B >= 1 && a->H >= 1 && a->Lq >= 1 && a->Lkv >= 1, LVAR_ERR_ARG,
               "B, H, Lq, Lkv must be >= 1 (got %d %d %d %d)", a->B, a->H, a->Lq, a->Lkv);
  // the column sums alone read neither v nor o
  const bool qk_only = mode == MODE_CS_ONLY;
  LVAR_REQUIRE(a->q && a->k && (qk_only || (a->v && a->o)), LVAR_ERR_ARG,
               "q, k, v, o must be non-null device pointers");
  LVAR_REQUIRE(aligned16(a->q) && aligned16(a->k) && (qk_only || (aligned16(a->v) && aligned16(a->o))), LVAR_ERR_ARG,
               "q, k, v, o must be 16-byte aligned");
  LVAR_REQUIRE(a->scale > 0.f && isfinite(a->scale), LVAR_ERR_ARG, "softmax scale must be positive and finite");
  const int64_t strides[] = {a->q_sb, a->q_sh, a->q_sl, a->k_sb, a->k_sh, a->k_sl,
                             a->v_sb, a->v_sh, a->v_sl, a->o_sb, a->o_sh, a->o_sl};
  for (int i = 0; i < (qk_only ? 6 : 12); ++i)
    LVAR_REQUIRE(strides[i] % 8 == 0 && strides[i] >= 0, LVAR_ERR_ARG,
                 "tensor strides must be non-negative multiples of 8 elements");

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
  p.o_align32 = (reinterpret_cast<uintptr_t>(a->o) % 32 == 0 && (a->o_sb * 2) % 32 == 0 && (a->o_sh * 2) % 32 == 0 &&
                 (a->o_sl * 2) % 32 == 0)
                     ? 1
                     : 0;
  p.M = a->M;
  p.L = a->L;
  if (stats_given) {
    LVAR_REQUIRE(a->M && a->L, LVAR_ERR_ARG, "M and L (row statistics, fp32 [B,H,Lq]) must be non-null");
    p.M_in = a->M;
    p.L_in = a->L;
    p.M = p.L = nullptr;
  }
  if (mode == MODE_DENSE_CS1) {
    LVAR_REQUIRE(a->M_in && a->L_in, LVAR_ERR_ARG,
                 "M_in and L_in (row statistics of this attention, fp32 [B,H,Lq]) must be non-null");
    LVAR_REQUIRE((a->M == nullptr) == (a->L == nullptr), LVAR_ERR_ARG, "M and L (statistics out) go together");
    p.M_in = a->M_in;
    p.L_in = a->L_in;
  }
  if (mode == MODE_DENSE_CS || mode == MODE_CS_ONLY || mode == MODE_DENSE_CS1) {
    LVAR_REQUIRE(a->cs != nullptr, LVAR_ERR_ARG, "cs (column sums per 128-row query tile) is null");
    p.cs = a->cs;
    p.cs_sb = a->cs_sb;
    p.cs_sh = a->cs_sh;
    p.cs_st = a->cs_st;
    LVAR_REQUIRE(a->cs_group_tiles == 0 || a->cs_group_tiles == 1 || a->cs_group_tiles == 2, LVAR_ERR_ARG,
                 "cs_group_tiles must be 1 (a row per 128-row tile) or 2 (a row per 256-row group)");
    p.cs_pair = a->cs_group_tiles == 2 ? 1 : 0;
  }
  p.nkb = (a->Lkv + 127) / 128;
  p.status = a->dev_status;
  p.wait_limit_ns = a->wait_limit_ns;

  LVAR_REQUIRE(a->sched_scratch != nullptr, LVAR_ERR_ARG,
               "sched_scratch must point to two zeroed device int32 (work counter of the persistent kernel)");
  p.sched_counter = a->sched_scratch;
  p.work_order = a->work_order;
  if (mode == MODE_BLOCK) {
    LVAR_REQUIRE(a->block_mask != nullptr, LVAR_ERR_ARG, "block mask is null");
    LVAR_REQUIRE(p.nkb <= kMaxSteps && p.nkb <= 4096, LVAR_ERR_UNSUPPORTED, "Lkv too long for the block list (max %d keys)",
                 kMaxSteps * 128);
    LVAR_REQUIRE(a->block_size == 0 || a->block_size == 128 || a->block_size == 64, LVAR_ERR_ARG,
                 "block_size must be 128 or 64");
    p.mask_block = a->block_size == 64 ? 64 : 128;
    p.nq_mask = (a->Lq + p.mask_block - 1) / p.mask_block;
    p.nk_mask = (a->Lkv + p.mask_block - 1) / p.mask_block;
    p.mask = a->block_mask;
    p.m_sb = a->bm_sb;
    p.m_sh = a->bm_sh;
    p.m_sq = a->bm_sq;
  }
  if (mode == MODE_DENSE || mode == MODE_DENSE_CS || mode == MODE_CS_ONLY || mode == MODE_DENSE_CS1) {
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
    p.oi_side = 0;
    if (a->o_in_side > 0) {
      LVAR_REQUIRE(a->o_side >= 1 && (int64_t)a->o_side * a->o_side == a->Lq, LVAR_ERR_ARG,
                   "o_in_side > 0 needs a square query grid: o_side * o_side must equal Lq");
      LVAR_REQUIRE(a->o_in != a->o, LVAR_ERR_ARG, "a resized o_in cannot be the output buffer");
      p.oi_side = a->o_in_side;
      p.o_side = a->o_side;
      p.oi_ratio = (float)a->o_in_side / (float)a->o_side;
    }
    const int groups = (a->Lq + a->group_rows - 1) / a->group_rows;
    p.n_x = groups * p.chunks_per_group;
  } else {
    p.n_x = (a->Lq + 255) / 256;
  }
  const int64_t total = (int64_t)p.n_x * a->B * a->H;
  LVAR_REQUIRE(total < (1ll << 30), LVAR_ERR_LIMIT, "too many work items");
  int dev = 0, sms = 0;
  LVAR_CUDA_OK(cudaGetDevice(&dev));
  LVAR_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  p.n_pair_items = (int)total;
  p.total_items = (int)total;
  // A single tile of the attention modes runs on both slots, each taking half of the tile's KV list
  // (see the kernel's decode); the column-sum modes keep one slot idle instead.
  p.split_singles = ((mode == MODE_DENSE || mode == MODE_BLOCK) && !(a->sched_flags & LVAR_SCHED_SINGLE_ONE_SLOT)) ? 1 : 0;
  if (mode != MODE_CSP && (total > sms || p.split_singles) && !(a->sched_flags & LVAR_SCHED_PAIRS_ONLY)) {
    // Wave quantisation: the pairs left over after the last full wave of CTAs are handed out as single
    // query tiles when those fit in one wave, so that the tail costs one short item per CTA instead of
    // one full pair on a few CTAs.  With work_order the tail is the end of the caller's order.
    const int64_t rem = total % sms;
    if (rem > 0 && 2 * rem <= sms) {
      p.n_pair_items = (int)(total - rem);
      p.total_items = (int)(total + rem);
    }
  }
  dim3 grid((unsigned)(p.total_items < sms ? p.total_items : sms), 1, 1);

  CUtensorMap tq, tk, tv;
  int rc = encode_bhld_map(&tq, a->q, a->B, a->H, a->Lq, a->D, a->q_sb, a->q_sh, a->q_sl, 128);
  if (rc != LVAR_OK) return rc;
  rc = encode_bhld_map(&tk, a->k, a->B, a->H, a->Lkv, a->D, a->k_sb, a->k_sh, a->k_sl, 128);
  if (rc != LVAR_OK) return rc;
  if (qk_only) {
    tv = tk;  // never used by the kernel in this mode
  } else {
    rc = encode_bhld_map(&tv, a->v, a->B, a->H, a->Lkv, a->D, a->v_sb, a->v_sh, a->v_sl, 128);
    if (rc != LVAR_OK) return rc;
  }

  const bool serialize_launch = (a->sched_flags & LVAR_SCHED_SERIALIZE_LAUNCH) != 0;
  if (a->D == 128) return launch_d<128>(mode, tq, tk, tv, p, grid, stream, serialize_launch);
  return launch_d<64>(mode, tq, tk, tv, p, grid, stream, serialize_launch);
}

}  // namespace lvar
