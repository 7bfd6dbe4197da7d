// lvar_dense_colsum_attn_static: dense attention + attention column sums for callers that must not
// allocate device memory.  The intermediate data of the pair of kernels - the per-row softmax
// statistics (M, L) that the attention pass writes and the column-sum pass reads back, and the work
// counter of the persistent attention kernel - live in ONE file-scope device array instead of buffers
// the caller (or torch's allocator) would have to provide.
//
// Who needs this: hosts that have handed the whole HBM to their own pool (a KV-cache manager, a
// serving runtime with a frozen arena) or that run under a "no allocation after warm-up" rule, where
// a cudaMalloc inside the per-layer call is either forbidden or would synchronise the device.
//
// Limits and rules, also stated in include/lvar_b200.h:
//   * B * H * Lq <= LVAR_STATIC_MAX_ROWS (262144 rows: 2 MiB of statistics); larger calls are
//     rejected with LVAR_ERR_LIMIT before anything is launched.
//   * The array belongs to the library: every GPU that loads the library holds its 2 MiB + 256 B
//     until the process exits.
//   * All calls on a device share the array.  It keeps the previous call's contents; the one word
//     that must start at zero (the work counter) is cleared on the caller's stream by every call.
//     Two calls that may overlap on the GPU (different streams, no ordering) race on it: do not.
//   * The first call on each device looks the array's device address up (cudaGetSymbolAddress) and
//     sets kernel attributes; make that first call outside any stream capture.
#include <atomic>

#include "common.cuh"

namespace lvar {

int launch_attention(const lvar_attn_args* a, int mode, cudaStream_t stream);
int launch_colsum(const void* q, const void* k, const float* M, const float* L, float* cs, int B, int H, int Lq,
                  int Lkv, int D, int64_t q_sb, int64_t q_sh, int64_t q_sl, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                  int64_t cs_sb, int64_t cs_sh, int64_t cs_sg, int group_rows, float scale, int* dev_status,
                  uint64_t wait_limit_ns, cudaStream_t stream);

namespace {

constexpr size_t kCounterBytes = 256;  // work counter pair, padded to keep the statistics 256-byte aligned
constexpr size_t kStatBytes = (size_t)LVAR_STATIC_MAX_ROWS * sizeof(float);
constexpr size_t kScratchBytes = kCounterBytes + 2 * kStatBytes;

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress; it is not a
// device address and must never be passed to a kernel as one.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
// Per device: the looked-up address, published with release/acquire so that two host threads making their
// first call at the same time agree (both look the same address up; either store wins).  The address stays
// valid for the life of the device's primary context: a cudaDeviceReset unloads the library's module, and a
// host that resets a device must not call this entry point on it again in the same process.
std::atomic<unsigned char*> g_scratch_addr[kMaxDevices];

// Device address of the scratch on the current device; looked up once per device.
int scratch_base(unsigned char** out) {
  int dev = 0;
  LVAR_CUDA_OK(cudaGetDevice(&dev));
  LVAR_REQUIRE(dev >= 0 && dev < kMaxDevices, LVAR_ERR_LIMIT, "device ordinal %d not supported (max %d)", dev,
               kMaxDevices - 1);
  unsigned char* addr = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (addr == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(LVAR_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", dev,
                  cudaGetErrorString(e));
    addr = static_cast<unsigned char*>(ptr);
    g_scratch_addr[dev].store(addr, std::memory_order_release);
  }
  *out = addr;
  return LVAR_OK;
}

}  // namespace
}  // namespace lvar

extern "C" int lvar_dense_colsum_attn_static(const void* q, const void* k, const void* v, void* o, float* cs,
                                             int32_t B, int32_t H, int32_t Lq, int32_t Lkv, int32_t D, int64_t q_sb,
                                             int64_t q_sh, int64_t q_sl, int64_t k_sb, int64_t k_sh, int64_t k_sl,
                                             int64_t v_sb, int64_t v_sh, int64_t v_sl, int64_t o_sb, int64_t o_sh,
                                             int64_t o_sl, int64_t cs_sb, int64_t cs_sh, int64_t cs_sg,
                                             int32_t group_rows, float scale, int32_t* dev_status,
                                             uint64_t wait_limit_ns, lvar_stream_t stream_) {
  using namespace lvar;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  LVAR_REQUIRE(B >= 1 && H >= 1 && Lq >= 1, LVAR_ERR_ARG, "B, H, Lq must be >= 1");
  const int64_t rows = (int64_t)B * H * Lq;
  LVAR_REQUIRE(rows <= (int64_t)LVAR_STATIC_MAX_ROWS, LVAR_ERR_LIMIT,
               "B*H*Lq = %lld query rows exceed the static scratch of lvar_dense_colsum_attn_static (%d rows); "
               "use lvar_dense_attn + lvar_colsum with caller-provided buffers",
               (long long)rows, (int)LVAR_STATIC_MAX_ROWS);
  LVAR_REQUIRE(cs != nullptr, LVAR_ERR_ARG, "cs must be a non-null device pointer");

  unsigned char* base = nullptr;
  int rc = scratch_base(&base);
  if (rc != LVAR_OK) return rc;
  int32_t* counter = reinterpret_cast<int32_t*>(base);
  float* M = reinterpret_cast<float*>(base + kCounterBytes);
  float* L = reinterpret_cast<float*>(base + kCounterBytes + kStatBytes);

  // The counter must read zero when the attention kernel starts, whatever an earlier call left behind.
  LVAR_CUDA_OK(cudaMemsetAsync(counter, 0, 2 * sizeof(int32_t), stream));

  lvar_attn_args a{};
  a.B = B; a.H = H; a.Lq = Lq; a.Lkv = Lkv; a.D = D;
  a.scale = scale;
  a.q = q; a.q_sb = q_sb; a.q_sh = q_sh; a.q_sl = q_sl;
  a.k = k; a.k_sb = k_sb; a.k_sh = k_sh; a.k_sl = k_sl;
  a.v = v; a.v_sb = v_sb; a.v_sh = v_sh; a.v_sl = v_sl;
  a.o = o; a.o_sb = o_sb; a.o_sh = o_sh; a.o_sl = o_sl;
  a.M = M;
  a.L = L;
  a.sched_scratch = counter;
  a.dev_status = dev_status;
  a.wait_limit_ns = wait_limit_ns;
  rc = launch_attention(&a, /*dense*/ 0, stream);
  if (rc != LVAR_OK) return rc;
  return launch_colsum(q, k, M, L, cs, B, H, Lq, Lkv, D, q_sb, q_sh, q_sl, k_sb, k_sh, k_sl, cs_sb, cs_sh, cs_sg,
                       group_rows, scale, dev_status, wait_limit_ns, stream);
}
