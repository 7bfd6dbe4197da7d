// Mask / index construction kernels (integer and byte work, HBM-bound):
//   block_scores      column sums -> per-KV-block scores (fixed summation order)
//   build_block_mask  always-kept blocks U top-k remaining blocks by score -> uint8 mask (+ lists)
//   topk              exact, deterministic top-k of fp32 rows -> int32 index lists (+ counts)
//   mask_to_indices   bool mask rows -> padded index lists in the reference kernel's order
//   bitpack/bitunpack little-endian bit packing of bool tensors
// Ordering rule used everywhere a selection is made: descending by value, equal values in
// ascending index order; -0.0 equals +0.0; NaNs with the sign bit clear sort above +inf.
#include <math.h>

#include "common.cuh"

namespace lvar {

namespace {

// Monotone map float -> uint32: a > b  <=>  key(a) > key(b)  (for non-NaN; -0 folded onto +0).
__device__ __forceinline__ uint32_t ordered_key(float x) {
  const uint32_t u = __float_as_uint(x + 0.0f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += t;
  }
  return v;
}

// ------------------------------------------------------------------------------------------------
// block scores
// ------------------------------------------------------------------------------------------------
// One warp per (row, kv block).  Lane partials are summed sequentially, then a fixed xor tree.
__global__ void block_scores_kernel(const float* __restrict__ cs, float* __restrict__ out, int64_t rows, int Lkv,
                                    int nk, int block, int64_t cs_row_stride) {
  const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= rows * nk) return;
  const int64_t row = w / nk;
  const int kb = (int)(w % nk);
  const float* src = cs + row * cs_row_stride + (int64_t)kb * block;
  const int valid = min(block, Lkv - kb * block);
  float acc = 0.f;
  for (int c = lane; c < block; c += 32) acc += (c < valid) ? src[c] : 0.f;
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) out[row * nk + kb] = acc;
}

// ------------------------------------------------------------------------------------------------
// block mask: always U top-(k_total - |always|) of the rest
// ------------------------------------------------------------------------------------------------
// One CTA (128 threads) per (b, h, q-block row).  Rank counting over the row held in shared memory.
__global__ void build_block_mask_kernel(const float* __restrict__ scores, const uint8_t* __restrict__ always,
                                        uint8_t* __restrict__ mask, int32_t* __restrict__ lists,
                                        int32_t* __restrict__ counts, int nq, int nk, int k_total) {
  extern __shared__ uint32_t sh[];
  uint32_t* keys = sh;                                      // [nk]
  uint8_t* flag = reinterpret_cast<uint8_t*>(keys + nk);    // [nk] 1 = always, then final selection
  __shared__ int n_always;
  const int64_t row = blockIdx.x;  // over B*H*nq
  const int qi = (int)(row % nq);
  const float* s = scores + row * nk;
  if (threadIdx.x == 0) n_always = 0;
  __syncthreads();
  int local = 0;
  for (int j = threadIdx.x; j < nk; j += blockDim.x) {
    keys[j] = ordered_key(s[j]);
    const uint8_t a = always ? (always[(int64_t)qi * nk + j] != 0) : 0;
    flag[j] = a;
    local += a;
  }
  if (local) atomicAdd(&n_always, local);
  __syncthreads();
  const int need = max(0, k_total - n_always);
  uint8_t* mrow = mask + row * nk;
  for (int j = threadIdx.x; j < nk; j += blockDim.x) {
    uint8_t sel = flag[j];
    if (!sel && need > 0) {
      const uint32_t kj = keys[j];
      int rank = 0;
      for (int i = 0; i < nk; ++i) {
        if (flag[i]) continue;
        const uint32_t ki = keys[i];
        rank += (ki > kj) || (ki == kj && i < j);
      }
      sel = rank < need;
    }
    mrow[j] = sel;
  }
  if (lists != nullptr) {
    __syncthreads();  // mrow visible to the CTA (global writes by this CTA; read back below)
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      int n = 0;
      for (int base = 0; base < nk; base += 32) {
        const int j = base + lane;
        const bool on = (j < nk) && mrow[j];
        const uint32_t vote = __ballot_sync(0xffffffffu, on);
        if (on) lists[row * nk + n + __popc(vote & ((1u << lane) - 1u))] = j;
        n += __popc(vote);
      }
      for (int j = n + lane; j < nk; j += 32) lists[row * nk + j] = -1;
      if (lane == 0 && counts) counts[row] = n;
    }
  }
}

// Column sums -> block mask in one pass: one CTA (256 threads) per (b, h, q-block row) reads its row of column
// sums once, forms the per-KV-block scores with block_scores_kernel's summation order (one warp per block: the
// same bits) and selects as build_block_mask_kernel does.  Scores, lists and counts are optional outputs.
__global__ void __launch_bounds__(256)
block_mask_from_colsums_kernel(const float* __restrict__ cs, int64_t cs_row_stride, const uint8_t* __restrict__ always,
                               uint8_t* __restrict__ mask, float* __restrict__ scores_out, int32_t* __restrict__ lists,
                               int32_t* __restrict__ counts, int nq, int nk, int Lkv, int block, int k_total) {
  extern __shared__ uint32_t sh[];
  uint32_t* keys = sh;                                      // [nk]
  uint8_t* flag = reinterpret_cast<uint8_t*>(keys + nk);    // [nk]
  __shared__ int n_always;
  const int64_t row = blockIdx.x;
  const int qi = (int)(row % nq);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  if (threadIdx.x == 0) n_always = 0;
  const float* src_row = cs + row * cs_row_stride;
  for (int kb = warp; kb < nk; kb += n_warps) {
    const float* src = src_row + (int64_t)kb * block;
    const int valid = min(block, Lkv - kb * block);
    float acc = 0.f;
    for (int c = lane; c < block; c += 32) acc += (c < valid) ? src[c] : 0.f;
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (lane == 0) {
      keys[kb] = ordered_key(acc);
      if (scores_out) scores_out[row * nk + kb] = acc;
    }
  }
  __syncthreads();
  int local = 0;
  for (int j = threadIdx.x; j < nk; j += blockDim.x) {
    const uint8_t a = always ? (always[(int64_t)qi * nk + j] != 0) : 0;
    flag[j] = a;
    local += a;
  }
  if (local) atomicAdd(&n_always, local);
  __syncthreads();
  const int need = max(0, k_total - n_always);
  uint8_t* mrow = mask + row * nk;
  for (int j = threadIdx.x; j < nk; j += blockDim.x) {
    uint8_t sel = flag[j];
    if (!sel && need > 0) {
      const uint32_t kj = keys[j];
      int rank = 0;
      for (int i = 0; i < nk; ++i) {
        if (flag[i]) continue;
        const uint32_t ki = keys[i];
        rank += (ki > kj) || (ki == kj && i < j);
      }
      sel = rank < need;
    }
    mrow[j] = sel;
  }
  if (lists != nullptr) {
    __syncthreads();
    if (threadIdx.x < 32) {
      int n = 0;
      for (int base = 0; base < nk; base += 32) {
        const int j = base + lane;
        const bool on = (j < nk) && mrow[j];
        const uint32_t vote = __ballot_sync(0xffffffffu, on);
        if (on) lists[row * nk + n + __popc(vote & ((1u << lane) - 1u))] = j;
        n += __popc(vote);
      }
      for (int j = n + lane; j < nk; j += 32) lists[row * nk + j] = -1;
      if (lane == 0 && counts) counts[row] = n;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// exact top-k
// ------------------------------------------------------------------------------------------------
constexpr int kTopkThreads = 1024;
constexpr int kHistCopies = 8, kHistStride = 257;

// One CTA per row.  Shared: keys[n] | pairs[K2] (descending-value order only) | hist[8][257] | scan[64].
__global__ void __launch_bounds__(kTopkThreads)
topk_kernel(const float* __restrict__ scores, int64_t row_stride, int n, int k, int ascending_index,
            int32_t* __restrict__ out, int64_t out_stride, int out_cols, int32_t* __restrict__ counts,
            int count_value, int K2) {
  extern __shared__ __align__(16) uint8_t sh_raw[];
  uint32_t* keys = reinterpret_cast<uint32_t*>(sh_raw);
  unsigned long long* pairs = reinterpret_cast<unsigned long long*>(sh_raw + (((size_t)n * 4 + 15) & ~(size_t)15));
  __shared__ int hist[kHistCopies * kHistStride];
  __shared__ int wsum_gt[32], wsum_eq[32];
  __shared__ uint32_t sh_prefix;
  __shared__ int sh_remaining;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row = blockIdx.x;
  const float* src = scores + row * row_stride;
  int32_t* dst = out + row * out_stride;

  for (int i = tid; i < n; i += kTopkThreads) keys[i] = ordered_key(src[i]);
  if (tid == 0) {
    sh_prefix = 0;
    sh_remaining = k;
  }
  __syncthreads();

  if (k > 0) {
    // radix select, most significant byte first: after 4 passes sh_prefix is the k-th largest key and
    // sh_remaining the number of elements equal to it that belong to the selection.
    // Scores of one row share most of their leading bits (attention column sums span a few binades), so most
    // keys of a pass fall into a handful of histogram bins: the histogram is kept in eight copies (one per lane
    // modulo 8, 257 words apart so that equal bins of different copies sit in different banks), which cuts the
    // serialisation of same-address atomics eightfold; the copies are added up when the bins are scanned.
    uint32_t maskbits = 0;
    for (int pass = 3; pass >= 0; --pass) {
      for (int i = tid; i < kHistCopies * kHistStride; i += kTopkThreads) hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = sh_prefix;
      const int shift = pass * 8;
      int* myhist = hist + (lane & (kHistCopies - 1)) * kHistStride;
      for (int i = tid; i < n; i += kTopkThreads) {
        const uint32_t key = keys[i];
        if ((key & maskbits) == prefix) atomicAdd(&myhist[(key >> shift) & 255u], 1);
      }
      __syncthreads();
      if (warp == 0) {
        // bins from the top: the bin that holds the rem-th largest candidate.  Lane l owns bins 8l .. 8l+7.
        const int rem = sh_remaining;
        int binc[8];  // this lane's eight bins, summed over the copies
        int own = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          int c = 0;
#pragma unroll
          for (int k2 = 0; k2 < kHistCopies; ++k2) c += hist[k2 * kHistStride + 8 * lane + j];
          binc[j] = c;
          own += c;
        }
        int suffix = own;  // candidates in this lane's bins and all higher ones
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int t = __shfl_down_sync(0xffffffffu, suffix, d);
          if (lane + d < 32) suffix += t;
        }
        const uint32_t reach = __ballot_sync(0xffffffffu, suffix >= rem);  // never empty: all candidates >= rem
        const int L = 31 - __clz(reach);
        if (lane == L) {
          int r = rem - (suffix - own);  // still to find inside this lane's bins
          int j = 7;
#pragma unroll
          for (int t = 7; t > 0; --t) {
            if (j == t && binc[t] < r) {
              r -= binc[t];
              j = t - 1;
            }
          }
          const int d = 8 * lane + j;
          sh_prefix = prefix | ((uint32_t)d << shift);
          sh_remaining = r;
        }
      }
      maskbits |= 0xFFu << shift;
      __syncthreads();
    }
  }
  const uint32_t T = sh_prefix;
  const int need_eq = (k > 0) ? sh_remaining : 0;

  // ordered compaction: thread t owns the contiguous range [t*per, (t+1)*per)
  const int per = (n + kTopkThreads - 1) / kTopkThreads;
  const int lo = min(n, tid * per), hi = min(n, lo + per);
  int gt = 0, eq = 0;
  if (k > 0) {
    for (int i = lo; i < hi; ++i) {
      const uint32_t key = keys[i];
      gt += key > T;
      eq += key == T;
    }
  }
  int gt_inc = warp_incl_scan(gt, lane), eq_inc = warp_incl_scan(eq, lane);
  if (lane == 31) {
    wsum_gt[warp] = gt_inc;
    wsum_eq[warp] = eq_inc;
  }
  __syncthreads();
  if (warp == 0) {
    int a = wsum_gt[lane], b = wsum_eq[lane];
    const int ai = warp_incl_scan(a, lane), bi = warp_incl_scan(b, lane);
    wsum_gt[lane] = ai - a;
    wsum_eq[lane] = bi - b;
  }
  __syncthreads();
  int gt_b = wsum_gt[warp] + gt_inc - gt;  // selected-by-value elements before this thread's range
  int eq_b = wsum_eq[warp] + eq_inc - eq;  // elements equal to T before this thread's range
  if (k > 0) {
    for (int i = lo; i < hi; ++i) {
      const uint32_t key = keys[i];
      int pos = -1;
      if (key > T) {
        pos = gt_b + min(eq_b, need_eq);
        ++gt_b;
      } else if (key == T) {
        if (eq_b < need_eq) pos = gt_b + eq_b;
        ++eq_b;
      }
      if (pos >= 0) {
        if (ascending_index) {
          dst[pos] = i;
        } else {
          pairs[pos] = ((unsigned long long)key << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
        }
      }
    }
  }
  if (!ascending_index && k > 0) {
    for (int i = k + tid; i < K2; i += kTopkThreads) pairs[i] = 0ull;  // sorts last
    __syncthreads();
    // bitonic sort, descending on (key, ~index): equal keys come out in ascending index order
    for (int size = 2; size <= K2; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int t = tid; t < (K2 >> 1); t += kTopkThreads) {
          const int i = 2 * t - (t & (stride - 1));
          const int j = i + stride;
          const bool desc = ((i & size) == 0);
          const unsigned long long a = pairs[i], b = pairs[j];
          if ((a < b) == desc) {
            pairs[i] = b;
            pairs[j] = a;
          }
        }
        __syncthreads();
      }
    }
    for (int i = tid; i < k; i += kTopkThreads) dst[i] = (int32_t)(0xFFFFFFFFu - (uint32_t)(pairs[i] & 0xFFFFFFFFull));
  }
  for (int i = k + tid; i < out_cols; i += kTopkThreads) dst[i] = 0;
  if (counts != nullptr && tid == 0) counts[row] = count_value;
}

// ------------------------------------------------------------------------------------------------
// mask_to_indices
// ------------------------------------------------------------------------------------------------
// One warp per row, row staged in shared memory with coalesced loads.  Output order: lane t owns
// columns t, t+32, ...; lanes write their set columns at the exclusive prefix of the lane counts.
// The count is rounded up to multiple_of using the first unset columns.
__global__ void mask_to_indices_kernel(const uint8_t* __restrict__ mask, int32_t* __restrict__ indices,
                                       int32_t* __restrict__ counts, int n, int pad_n, int multiple_of) {
  extern __shared__ uint8_t row_s[];
  const int64_t row = blockIdx.x;
  const int lane = threadIdx.x;
  const uint8_t* src = mask + row * n;
  for (int c = lane; c < n; c += 32) row_s[c] = src[c];
  __syncwarp();
  int local = 0;
  for (int c = lane; c < n; c += 32) local += row_s[c] != 0;
  const int incl = warp_incl_scan(local, lane);
  int offset = incl - local;
  const int total = __shfl_sync(0xffffffffu, incl, 31);
  const int padded = (total + multiple_of - 1) / multiple_of * multiple_of;
  int32_t* dst = indices + row * pad_n;
  for (int c = lane; c < n; c += 32)
    if (row_s[c]) dst[offset++] = c;
  int filled = total;
  for (int base = 0; base < n && filled < padded; base += 32) {
    const int c = base + lane;
    const bool off = (c < n) && (row_s[c] == 0);
    const uint32_t vote = __ballot_sync(0xffffffffu, off);
    const int pos = filled + __popc(vote & ((1u << lane) - 1u));
    if (off && pos < padded && pos < pad_n) dst[pos] = c;
    filled += __popc(vote);
  }
  if (lane == 0) counts[row] = padded;
}

// ------------------------------------------------------------------------------------------------
// bitpack / bitunpack
// ------------------------------------------------------------------------------------------------
__global__ void bitpack_kernel(const uint8_t* __restrict__ mask, uint8_t* __restrict__ packed, int64_t n_bits,
                               int64_t n_bytes) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_bytes) return;
  const int64_t base = i * 8;
  uint32_t v = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (base + j < n_bits && mask[base + j]) v |= 1u << j;
  packed[i] = (uint8_t)v;
}

__global__ void bitunpack_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ mask, int64_t n_bits) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_bits) return;
  mask[i] = (packed[i >> 3] >> (i & 7)) & 1u;
}

// ------------------------------------------------------------------------------------------------
// index lists of a sparse step: remapped decision-scale lists followed by the scale's local band
// ------------------------------------------------------------------------------------------------
// out[bh, g, c] = clamp(src[bh, remap[g], c / rep], 0, k_len - 1)   for c <  cnt
//               = band[g, c - cnt]                                  for cnt <= c < cnt + band_count
//               = 0                                                 beyond;   counts[bh, g] = count_value
__global__ void sparse_step_lists_kernel(const int32_t* __restrict__ src, const int32_t* __restrict__ remap,
                                         const int32_t* __restrict__ band, int32_t* __restrict__ out,
                                         int32_t* __restrict__ counts, int64_t BH, int Gs, int64_t src_g_stride,
                                         int64_t src_bh_stride, int Gk, int cnt, int rep, int band_count, int k_len,
                                         int out_cols, int count_value) {
  const int64_t total = BH * Gk * out_cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % out_cols);
    const int g = (int)((i / out_cols) % Gk);
    const int64_t bh = i / ((int64_t)out_cols * Gk);
    int32_t v = 0;
    if (c < cnt) {
      v = src[bh * src_bh_stride + (int64_t)remap[g] * src_g_stride + c / rep];
      v = max(0, min(v, k_len - 1));
    } else if (c < cnt + band_count) {
      v = band[(int64_t)g * band_count + (c - cnt)];
    }
    out[i] = v;
    if (c == 0) counts[bh * Gk + g] = count_value;
  }
}

}  // namespace

int launch_sparse_step_lists(const int32_t* src, const int32_t* remap, const int32_t* band, int32_t* out,
                             int32_t* counts, int64_t BH, int Gs, int src_cols, int64_t src_g_stride,
                             int64_t src_bh_stride, int Gk, int cnt, int band_count, int k_len, int out_cols,
                             int count_value, cudaStream_t stream) {
  LVAR_REQUIRE(src && remap && out && counts, LVAR_ERR_ARG, "src, remap, out and counts must be non-null");
  LVAR_REQUIRE(band != nullptr || band_count == 0, LVAR_ERR_ARG, "band is null but band_count > 0");
  LVAR_REQUIRE(BH >= 1 && Gs >= 1 && Gk >= 1 && src_cols >= 1 && k_len >= 1, LVAR_ERR_ARG, "bad sizes");
  LVAR_REQUIRE(cnt >= 0 && band_count >= 0 && cnt + band_count <= out_cols, LVAR_ERR_ARG,
               "cnt + band_count = %d does not fit in %d output columns", cnt + band_count, out_cols);
  // lists shorter than cnt are stretched by repeating every entry `rep` times (repeat_interleave)
  const int rep = src_cols >= cnt ? 1 : (cnt + src_cols - 1) / src_cols;
  const int64_t total = BH * Gk * out_cols;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  sparse_step_lists_kernel<<<(unsigned)blocks, 256, 0, stream>>>(src, remap, band, out, counts, BH, Gs, src_g_stride,
                                                                 src_bh_stride, Gk, cnt, rep, band_count, k_len,
                                                                 out_cols, count_value);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

int launch_block_scores(const float* cs, float* out, int64_t rows, int Lkv, int block, int64_t cs_row_stride,
                        cudaStream_t stream) {
  LVAR_REQUIRE(cs && out, LVAR_ERR_ARG, "cs and out must be non-null");
  LVAR_REQUIRE(rows >= 1 && Lkv >= 1, LVAR_ERR_ARG, "rows and Lkv must be >= 1");
  LVAR_REQUIRE(block >= 32 && block % 32 == 0, LVAR_ERR_ARG, "block must be a multiple of 32");
  const int nk = (Lkv + block - 1) / block;
  const int64_t warps = rows * nk;
  const int wpb = 8;
  const int64_t blocks = (warps + wpb - 1) / wpb;
  LVAR_REQUIRE(blocks < (1ll << 31), LVAR_ERR_LIMIT, "too many rows");
  block_scores_kernel<<<(unsigned)blocks, wpb * 32, 0, stream>>>(cs, out, rows, Lkv, nk, block, cs_row_stride);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

int launch_build_block_mask(const float* scores, const uint8_t* always, uint8_t* mask, int32_t* lists,
                            int32_t* counts, int64_t BH, int nq, int nk, int k_total, cudaStream_t stream) {
  LVAR_REQUIRE(scores && mask, LVAR_ERR_ARG, "scores and mask must be non-null");
  LVAR_REQUIRE(BH >= 1 && nq >= 1 && nk >= 1, LVAR_ERR_ARG, "BH, nq, nk must be >= 1");
  LVAR_REQUIRE(nk <= 8192, LVAR_ERR_LIMIT, "at most 8192 KV blocks per row (got %d)", nk);
  LVAR_REQUIRE(BH * nq < (1ll << 31), LVAR_ERR_LIMIT, "too many rows");
  const size_t smem = (size_t)nk * 5;
  build_block_mask_kernel<<<(unsigned)(BH * nq), 128, smem, stream>>>(scores, always, mask, lists, counts, nq, nk,
                                                                      k_total);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

int launch_block_mask_from_colsums(const float* cs, int64_t cs_row_stride, const uint8_t* always, uint8_t* mask,
                                   float* scores_out, int32_t* lists, int32_t* counts, int64_t BH, int nq, int Lkv,
                                   int block, int k_total, cudaStream_t stream) {
  LVAR_REQUIRE(cs && mask, LVAR_ERR_ARG, "cs and mask must be non-null");
  LVAR_REQUIRE(BH >= 1 && nq >= 1 && Lkv >= 1 && block >= 1, LVAR_ERR_ARG, "BH, nq, Lkv, block must be >= 1");
  const int nk = (Lkv + block - 1) / block;
  LVAR_REQUIRE(nk <= 8192, LVAR_ERR_LIMIT, "at most 8192 KV blocks per row (got %d)", nk);
  LVAR_REQUIRE(BH * nq < (1ll << 31), LVAR_ERR_LIMIT, "too many rows");
  const size_t smem = (size_t)nk * 5;
  block_mask_from_colsums_kernel<<<(unsigned)(BH * nq), 256, smem, stream>>>(cs, cs_row_stride, always, mask, scores_out,
                                                                             lists, counts, nq, nk, Lkv, block, k_total);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

int launch_topk(const float* scores, int64_t rows, int n, int64_t row_stride, int k, int ascending_index,
                int32_t* out, int64_t out_stride, int out_cols, int32_t* counts, int count_value,
                cudaStream_t stream) {
  LVAR_REQUIRE(scores && out, LVAR_ERR_ARG, "scores and out must be non-null");
  LVAR_REQUIRE(rows >= 1 && n >= 1, LVAR_ERR_ARG, "rows and n must be >= 1");
  LVAR_REQUIRE(k >= 0 && k <= n, LVAR_ERR_ARG, "k must be in [0, n] (k=%d, n=%d)", k, n);
  LVAR_REQUIRE(out_cols >= k && out_stride >= out_cols, LVAR_ERR_ARG, "output row too short for k entries");
  LVAR_REQUIRE(rows < (1ll << 31), LVAR_ERR_LIMIT, "too many rows");
  int K2 = 0;
  if (!ascending_index && k > 0) {
    K2 = 2;
    while (K2 < k) K2 <<= 1;
  }
  const size_t smem = (((size_t)n * 4 + 15) & ~(size_t)15) + (size_t)K2 * 8;
  LVAR_REQUIRE(smem <= 200 * 1024, LVAR_ERR_LIMIT,
               "row of %d scores with k=%d needs %zu bytes of shared memory (limit 204800)", n, k, smem);
  LVAR_CUDA_OK(cudaFuncSetAttribute(topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  topk_kernel<<<(unsigned)rows, kTopkThreads, smem, stream>>>(scores, row_stride, n, k, ascending_index, out,
                                                              out_stride, out_cols, counts, count_value, K2);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

int launch_mask_to_indices(const uint8_t* mask, int32_t* indices, int32_t* counts, int64_t rows, int n, int pad_n,
                           int multiple_of, cudaStream_t stream) {
  LVAR_REQUIRE(mask && indices && counts, LVAR_ERR_ARG, "mask, indices and counts must be non-null");
  LVAR_REQUIRE(rows >= 1 && n >= 1 && pad_n >= n && multiple_of >= 1, LVAR_ERR_ARG, "bad sizes");
  LVAR_REQUIRE(n <= 200 * 1024, LVAR_ERR_LIMIT, "rows longer than 204800 columns are not supported");
  LVAR_REQUIRE(rows < (1ll << 31), LVAR_ERR_LIMIT, "too many rows");
  if (n > 48 * 1024)
    LVAR_CUDA_OK(cudaFuncSetAttribute(mask_to_indices_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, n));
  mask_to_indices_kernel<<<(unsigned)rows, 32, n, stream>>>(mask, indices, counts, n, pad_n, multiple_of);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

int launch_bitpack(const uint8_t* mask, uint8_t* packed, int64_t n_bits, cudaStream_t stream) {
  LVAR_REQUIRE(mask && packed && n_bits >= 1, LVAR_ERR_ARG, "bad arguments");
  const int64_t n_bytes = (n_bits + 7) / 8;
  bitpack_kernel<<<(unsigned)((n_bytes + 255) / 256), 256, 0, stream>>>(mask, packed, n_bits, n_bytes);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

int launch_bitunpack(const uint8_t* packed, uint8_t* mask, int64_t n_bits, cudaStream_t stream) {
  LVAR_REQUIRE(mask && packed && n_bits >= 1, LVAR_ERR_ARG, "bad arguments");
  bitunpack_kernel<<<(unsigned)((n_bits + 255) / 256), 256, 0, stream>>>(packed, mask, n_bits);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

}  // namespace lvar
