// KV-cache compaction scores of ScaleKV (models/scalekv/scale_kv.py:232-301) and the row gather that
// builds the compacted cache.  All three kernels are HBM-bound byte movers:
//   scalekv_scores  score[b,h,j] = sum over the window queries i of bf16(bf16(q_i . k_j) / sqrt(D)), -inf on
//                   the window's own columns (the reference's matmul, division, masked_fill and sum on bf16
//                   tensors, rounding where torch rounds); K is read once
//   scalekv_pool    max- or average-pool over `ksize` neighbours (stride 1, padding ksize/2 as torch pads),
//                   then the window columns are raised to +inf so that one exact top-k of max_capacity
//                   entries in ascending index order returns sort(window U top-(max_capacity - w) of the rest),
//                   which is the reference's cat + sort
//   gather_rows     dst[b,h,i,:] = src[b,h,idx[b,h,i],:]
#include <math.h>

#include "common.cuh"

namespace lvar {

namespace {

constexpr int kMaxWindow = 64;

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// One warp per pass handles 32 / (D/8) keys: D/8 lanes read one 16-byte piece of a key row each.
template <int D>
__global__ void __launch_bounds__(256)
scalekv_scores_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                      const int32_t* __restrict__ window, float* __restrict__ scores, int H, int Lq, int Lkv,
                      int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb, int64_t k_sh, int64_t k_sl, int w,
                      int offset, float sqrt_d) {
  constexpr int LPK = D / 8;        // lanes per key
  constexpr int KPP = 32 / LPK;     // keys per warp pass
  __shared__ __align__(16) __nv_bfloat16 wq[kMaxWindow * D];
  __shared__ int wcol[kMaxWindow];
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const __nv_bfloat16* qb = q + b * q_sb + h * q_sh;
  const __nv_bfloat16* kb = k + b * k_sb + h * k_sh;
  // the window queries: query row clamp(window[i] - offset, 0, Lq - 1)
  for (int t = threadIdx.x; t < w * (D / 8); t += blockDim.x) {
    const int i = t / (D / 8), c = t % (D / 8);
    const int row = min(max(window[i] - offset, 0), Lq - 1);
    reinterpret_cast<uint4*>(wq)[i * (D / 8) + c] = *reinterpret_cast<const uint4*>(qb + (int64_t)row * q_sl + c * 8);
  }
  if (threadIdx.x < w) wcol[threadIdx.x] = window[threadIdx.x];
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int sub = lane / LPK, piece = lane % LPK;
  const int keys_per_block = nwarps * KPP;
  for (int j0 = blockIdx.x * keys_per_block; j0 < Lkv; j0 += gridDim.x * keys_per_block) {
    const int j = j0 + warp * KPP + sub;
    float kf[8];
    if (j < Lkv) {
      const uint4 raw = *reinterpret_cast<const uint4*>(kb + (int64_t)j * k_sl + piece * 8);
      const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        kf[2 * e] = __uint_as_float(u[e] << 16);
        kf[2 * e + 1] = __uint_as_float(u[e] & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) kf[e] = 0.f;
    }
    float total = 0.f;
    for (int i = 0; i < w; ++i) {
      const uint4 raw = reinterpret_cast<const uint4*>(wq)[i * (D / 8) + piece];
      const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        dot = fmaf(__uint_as_float(u[e] << 16), kf[2 * e], dot);
        dot = fmaf(__uint_as_float(u[e] & 0xffff0000u), kf[2 * e + 1], dot);
      }
#pragma unroll
      for (int d = LPK / 2; d >= 1; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
      // logit rounded to bf16 (matmul output), divided by sqrt(D) in fp32 and rounded again (bf16 / scalar)
      total += bf16_round(bf16_round(dot) / sqrt_d);
    }
    if (piece == 0 && j < Lkv) {
      bool in_window = false;
      for (int i = 0; i < w; ++i) in_window |= (wcol[i] == j);
      scores[(int64_t)bh * Lkv + j] = in_window ? -INFINITY : bf16_round(total);
    }
  }
}

// pooled[j] over neighbours j - r .. j + r (r = ksize / 2); max: torch pads with -inf; average: torch pads
// with zeros and divides by ksize, result rounded to bf16 like the input dtype.  Window columns -> +inf.
__global__ void scalekv_pool_kernel(const float* __restrict__ scores, const int32_t* __restrict__ window, int w,
                                    float* __restrict__ pooled, int Lkv, int ksize, int avg) {
  __shared__ int wcol[kMaxWindow];
  if (threadIdx.x < w) wcol[threadIdx.x] = window[threadIdx.x];
  __syncthreads();
  const int64_t row = blockIdx.y;
  const float* s = scores + row * Lkv;
  const int r = ksize / 2;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < Lkv; j += gridDim.x * blockDim.x) {
    float acc = avg ? 0.f : -INFINITY;
    for (int d = -r; d <= r; ++d) {
      const int t = j + d;
      if (t < 0 || t >= Lkv) continue;
      acc = avg ? acc + s[t] : fmaxf(acc, s[t]);
    }
    if (avg) acc = bf16_round(acc / (float)ksize);
    bool in_window = false;
    for (int i = 0; i < w; ++i) in_window |= (wcol[i] == j);
    pooled[row * Lkv + j] = in_window ? INFINITY : acc;
  }
}

// One 16-byte piece per thread.
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ idx,
                                   __nv_bfloat16* __restrict__ dst, int H, int L, int n, int D, int64_t s_sb,
                                   int64_t s_sh, int64_t s_sl, int64_t idx_row_stride, int64_t total_pieces) {
  const int ppr = D / 8;  // pieces per row
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total_pieces;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(t % ppr);
    const int64_t ri = t / ppr;      // (bh, i)
    const int i = (int)(ri % n);
    const int64_t bh = ri / n;
    const int b = (int)(bh / H), h = (int)(bh % H);
    const int row = min(max(idx[bh * idx_row_stride + i], 0), L - 1);
    const uint4 v = *reinterpret_cast<const uint4*>(src + b * s_sb + h * s_sh + (int64_t)row * s_sl + c * 8);
    reinterpret_cast<uint4*>(dst)[t] = v;
  }
}

}  // namespace

int launch_scalekv_scores(const void* q, const void* k, const int32_t* window, float* scores, int B, int H, int Lq,
                          int Lkv, int D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb, int64_t k_sh,
                          int64_t k_sl, int w, int offset, cudaStream_t stream) {
  LVAR_REQUIRE(q && k && window && scores, LVAR_ERR_ARG, "q, k, window and scores must be non-null");
  LVAR_REQUIRE(D == 64 || D == 128, LVAR_ERR_UNSUPPORTED, "Head dimension must be 64 or 128 (got %d)", D);
  LVAR_REQUIRE(B >= 1 && H >= 1 && Lq >= 1 && Lkv >= 1, LVAR_ERR_ARG, "B, H, Lq, Lkv must be >= 1");
  LVAR_REQUIRE(w >= 1 && w <= kMaxWindow, LVAR_ERR_UNSUPPORTED, "window of %d queries (supported: 1..%d)", w, kMaxWindow);
  LVAR_REQUIRE(aligned16(q) && aligned16(k), LVAR_ERR_ARG, "q and k must be 16-byte aligned");
  const int64_t strides[] = {q_sb, q_sh, q_sl, k_sb, k_sh, k_sl};
  for (int64_t s : strides)
    LVAR_REQUIRE(s % 8 == 0 && s >= 0, LVAR_ERR_ARG, "tensor strides must be non-negative multiples of 8 elements");
  LVAR_REQUIRE((int64_t)B * H <= 65535, LVAR_ERR_UNSUPPORTED, "B*H must be <= 65535");
  const int keys_per_block = 8 * (32 / (D / 8));
  int bx = (Lkv + keys_per_block - 1) / keys_per_block;
  if (bx > 148 * 4) bx = 148 * 4;
  dim3 grid((unsigned)bx, (unsigned)(B * H));
  const float sqrt_d = sqrtf((float)D);
  const auto* qp = static_cast<const __nv_bfloat16*>(q);
  const auto* kp = static_cast<const __nv_bfloat16*>(k);
  if (D == 128)
    scalekv_scores_kernel<128><<<grid, 256, 0, stream>>>(qp, kp, window, scores, H, Lq, Lkv, q_sb, q_sh, q_sl, k_sb, k_sh,
                                                         k_sl, w, offset, sqrt_d);
  else
    scalekv_scores_kernel<64><<<grid, 256, 0, stream>>>(qp, kp, window, scores, H, Lq, Lkv, q_sb, q_sh, q_sl, k_sb, k_sh,
                                                        k_sl, w, offset, sqrt_d);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

int launch_scalekv_pool(const float* scores, const int32_t* window, int w, float* pooled, int64_t rows, int Lkv,
                        int ksize, int avg, cudaStream_t stream) {
  LVAR_REQUIRE(scores && window && pooled, LVAR_ERR_ARG, "scores, window and pooled must be non-null");
  LVAR_REQUIRE(rows >= 1 && rows <= 65535 && Lkv >= 1, LVAR_ERR_ARG, "bad sizes");
  LVAR_REQUIRE(w >= 1 && w <= kMaxWindow, LVAR_ERR_UNSUPPORTED, "window of %d queries (supported: 1..%d)", w, kMaxWindow);
  LVAR_REQUIRE(ksize >= 1 && (ksize & 1), LVAR_ERR_ARG, "pooling kernel size must be odd and >= 1 (got %d)", ksize);
  int bx = (Lkv + 255) / 256;
  if (bx > 64) bx = 64;
  scalekv_pool_kernel<<<dim3((unsigned)bx, (unsigned)rows), 256, 0, stream>>>(scores, window, w, pooled, Lkv, ksize, avg);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

int launch_gather_rows(const void* src, const int32_t* idx, void* dst, int B, int H, int L, int n, int D, int64_t s_sb,
                       int64_t s_sh, int64_t s_sl, int64_t idx_row_stride, cudaStream_t stream) {
  LVAR_REQUIRE(src && idx && dst, LVAR_ERR_ARG, "src, idx and dst must be non-null");
  LVAR_REQUIRE(B >= 1 && H >= 1 && L >= 1 && n >= 1, LVAR_ERR_ARG, "B, H, L, n must be >= 1");
  LVAR_REQUIRE(D >= 8 && D % 8 == 0, LVAR_ERR_ARG, "row length must be a positive multiple of 8 elements (got %d)", D);
  LVAR_REQUIRE(aligned16(src) && aligned16(dst), LVAR_ERR_ARG, "src and dst must be 16-byte aligned");
  LVAR_REQUIRE(s_sb % 8 == 0 && s_sh % 8 == 0 && s_sl % 8 == 0, LVAR_ERR_ARG,
               "tensor strides must be multiples of 8 elements");
  LVAR_REQUIRE(idx_row_stride >= n, LVAR_ERR_ARG, "index rows shorter than n");
  const int64_t total = (int64_t)B * H * n * (D / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  gather_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), idx,
                                                           static_cast<__nv_bfloat16*>(dst), H, L, n, D, s_sb, s_sh,
                                                           s_sl, idx_row_stride, total);
  LVAR_CUDA_OK(cudaGetLastError());
  return LVAR_OK;
}

}  // namespace lvar
