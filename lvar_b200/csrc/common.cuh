// Host-side helpers shared by the launchers: error codes of the C ABI, TMA descriptor encoding
// through the driver entry point (no link-time dependency on libcuda), and small checks.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lvar_b200.h"

namespace lvar {

// Sets the thread-local message returned by lvar_last_error() and hands back `code`.
int fail(int code, const char* fmt, ...);

#define LVAR_REQUIRE(cond, code, ...) \
  do {                                \
    if (!(cond)) return ::lvar::fail((code), __VA_ARGS__); \
  } while (0)

#define LVAR_CUDA_OK(expr)                                                               \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess)                                                               \
      return ::lvar::fail(LVAR_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

// Encodes a 4-D bf16 tensor map over a [B, H, L, D] view (D contiguous) with a
// [1, 1, box_rows, 64] box and 128-byte swizzle; out-of-range rows read as zeros.
// Strides are in elements.  Returns an LVAR_* code.
int encode_bhld_map(CUtensorMap* out, const void* base, int B, int H, int L, int D, int64_t sb, int64_t sh,
                    int64_t sl, int box_rows);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace lvar
