// Pieces shared by the int4-weight GEMM kernels (gemm_w4a8.cu, gemm_w4a16.cu).
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {
namespace w4 {

constexpr int kMaxGroups = 1024;
constexpr uint32_t kTmemCols = 512;

struct RowMaps { CUtensorMap m[4]; };      // activation boxes of 16 / 32 / 64 / 128 rows x 128 bytes

// Bookkeeping of the copies a producer thread has in flight, so that it can wait for them (bounded) before the
// CTA leaves after a timeout elsewhere.
struct Armed {
  uint32_t mask = 0, parity = 0;
  __device__ __forceinline__ void arm(int s, uint32_t ph) { mask |= 1u << s; parity = (parity & ~(1u << s)) | (ph << s); }
  __device__ __forceinline__ void drain(uint64_t* bars, int n) {
    for (int s = 0; s < n; ++s) {
      if (!((mask >> s) & 1u)) continue;
      const uint64_t t0 = ptx::global_timer_ns();
      while (!ptx::mbar_try_wait(&bars[s], (parity >> s) & 1u) && ptx::global_timer_ns() - t0 < 20000000ull) {}
    }
  }
};

}  // namespace w4
}  // namespace b200moe
