// Permutation metadata: run_moe_ep_preproess of moe/group_gemm_kernel.py:48-78
// as a deterministic, stable counting sort (the reference uses torch.sort plus
// two Triton kernels, :19-45).
//
// The flat id array is cut into chunks of kChunk slots, one warp per chunk.
//   1. hist : per-chunk expert histogram            -> scratch[chunk][e]
//   2. scan : per expert, exclusive prefix over chunks (in place) and the
//             exclusive prefix over experts          -> seg_indptr
//   3. rank : each warp walks its chunk in order; a slot's row is
//             seg_indptr[e] + (same-expert slots in earlier chunks)
//                           + (same-expert slots earlier in this chunk)
// No step depends on the order in which atomics land, so the result is the
// stable sort bit for bit.  Ids outside [0, E) are ignored (src2dst = -1).
#include <mutex>

#include "common.cuh"

namespace b200moe {

constexpr int kChunk = 1024;        // slots per warp
constexpr int kWarpsPerBlock = 4;
constexpr int kMaxExperts = 1024;

__global__ void __launch_bounds__(kWarpsPerBlock * 32) route_hist_kernel(
    const int64_t* __restrict__ ids, int64_t n, int E, int32_t* __restrict__ scratch) {
  extern __shared__ int32_t s_cnt[];            // [kWarpsPerBlock][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  int32_t* cnt = s_cnt + warp * E;
  for (int e = lane; e < E; e += 32) cnt[e] = 0;
  __syncwarp();
  const int64_t base = chunk * kChunk;
  if (base < n) {
    const int64_t end = min(base + kChunk, n);
    for (int64_t i = base + lane; i < end; i += 32) {
      const int64_t e = ids[i];
      if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) scratch[chunk * E + e] = cnt[e];
  }
}

__global__ void __launch_bounds__(1024) route_scan_kernel(int32_t* __restrict__ scratch,
                                                          int64_t num_chunks, int E,
                                                          int64_t* __restrict__ seg_indptr) {
  __shared__ int64_t s_warp[32];
  const int e = threadIdx.x;
  int64_t run = 0;
  if (e < E) {
    for (int64_t c = 0; c < num_chunks; ++c) {
      const int32_t v = scratch[c * E + e];
      scratch[c * E + e] = static_cast<int32_t>(run);
      run += v;
    }
  }
  // inclusive scan of `run` over experts
  int64_t v = run;
  const int lane = e & 31, warp = e >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int64_t u = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += u;
  }
  if (lane == 31) s_warp[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int64_t w = s_warp[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int64_t u = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += u;
    }
    s_warp[lane] = w;
  }
  __syncthreads();
  const int64_t incl = v + (warp > 0 ? s_warp[warp - 1] : 0);
  if (e < E) seg_indptr[e + 1] = incl;
  if (e == 0) seg_indptr[0] = 0;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32) route_rank_kernel(
    const int64_t* __restrict__ ids, int64_t n, int E, const int32_t* __restrict__ scratch,
    const int64_t* __restrict__ seg_indptr, int64_t* __restrict__ reorder_ids,
    int32_t* __restrict__ src2dst) {
  extern __shared__ int32_t s_cnt[];            // [kWarpsPerBlock][E] next free row per expert
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t chunk = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  const int64_t base = chunk * kChunk;
  if (base >= n) return;
  int32_t* cnt = s_cnt + warp * E;
  for (int e = lane; e < E; e += 32)
    cnt[e] = static_cast<int32_t>(seg_indptr[e]) + scratch[chunk * E + e];
  __syncwarp();
  const int64_t end = min(base + kChunk, n);
  const uint32_t lt = (1u << lane) - 1u;
  for (int64_t i0 = base; i0 < end; i0 += 32) {
    const int64_t i = i0 + lane;
    const bool in = i < end;
    const int64_t e64 = in ? ids[i] : -1;
    const bool ok = in && e64 >= 0 && e64 < E;
    const int e = ok ? static_cast<int>(e64) : -1 - lane;   // distinct keys for idle lanes
    const uint32_t peers = __match_any_sync(0xffffffffu, e);
    int32_t dst = -1;
    if (ok) dst = cnt[e] + __popc(peers & lt);
    __syncwarp();
    if (ok && (peers & lt) == 0) cnt[e] += __popc(peers);   // first lane of the peer set
    __syncwarp();
    if (in) src2dst[i] = dst;
    if (ok) reorder_ids[dst] = e64;
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" size_t b200moe_route_metadata_workspace_bytes(int64_t num_slots, int num_experts) {
  if (num_slots <= 0 || num_experts <= 0) return 16;
  const int64_t chunks = (num_slots + kChunk - 1) / kChunk;
  return static_cast<size_t>(chunks) * num_experts * sizeof(int32_t);
}

extern "C" int b200moe_route_metadata(const int64_t* topk_ids, int64_t num_slots,
                                      int num_experts, int64_t* reorder_topk_ids,
                                      int32_t* src2dst, int64_t* seg_indptr, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  B200MOE_REQUIRE(seg_indptr, B200MOE_BAD_ARG, "route_metadata: null seg_indptr");
  B200MOE_REQUIRE(num_experts >= 1 && num_experts <= kMaxExperts, B200MOE_BAD_SHAPE,
                  "route_metadata: num_experts=%d not in [1,%d]", num_experts, kMaxExperts);
  B200MOE_REQUIRE(num_slots >= 0 && num_slots < (int64_t(1) << 31), B200MOE_BAD_SHAPE,
                  "route_metadata: num_slots=%lld does not fit int32 rows", (long long)num_slots);
  cudaStream_t st = as_stream(stream);
  if (num_slots == 0) {
    cudaMemsetAsync(seg_indptr, 0, sizeof(int64_t) * (num_experts + 1), st);
    return check_launch("route_metadata(memset)");
  }
  B200MOE_REQUIRE(topk_ids && reorder_topk_ids && src2dst && workspace, B200MOE_BAD_ARG,
                  "route_metadata: null pointer");
  B200MOE_REQUIRE(workspace_bytes >= b200moe_route_metadata_workspace_bytes(num_slots, num_experts),
                  B200MOE_WORKSPACE_TOO_SMALL, "route_metadata: workspace %zu < %zu bytes",
                  workspace_bytes, b200moe_route_metadata_workspace_bytes(num_slots, num_experts));
  B200MOE_REQUIRE(aligned(workspace, 4), B200MOE_BAD_ALIGN, "route_metadata: workspace alignment");
  const int64_t chunks = (num_slots + kChunk - 1) / kChunk;
  const unsigned grid = static_cast<unsigned>((chunks + kWarpsPerBlock - 1) / kWarpsPerBlock);
  const size_t smem = sizeof(int32_t) * kWarpsPerBlock * num_experts;
  int32_t* scratch = static_cast<int32_t*>(workspace);
  route_hist_kernel<<<grid, kWarpsPerBlock * 32, smem, st>>>(topk_ids, num_slots, num_experts, scratch);
  route_scan_kernel<<<1, 1024, 0, st>>>(scratch, chunks, num_experts, seg_indptr);
  route_rank_kernel<<<grid, kWarpsPerBlock * 32, smem, st>>>(topk_ids, num_slots, num_experts, scratch,
                                                             seg_indptr, reorder_topk_ids, src2dst);
  return check_launch("route_metadata");
}

// ---- variant that needs no caller-provided scratch ------------------------------------------
//
// Some callers have no way to hand this library a scratch buffer: a serving process whose
// framework reserved all of device memory for its own pool at start-up, a plug-in that is only
// given its input and output tensors, or a latency-critical loop in which cudaMalloc (which
// synchronises the whole device) must never run.  For them the counting sort's chunk-histogram
// table lives in a fixed array inside the library image.  Every GPU that loads the library
// carries this 1 MiB until the process exits, whether the entry point is used or not.
namespace b200moe {

constexpr int64_t kStaticScratchInts = 262144;  // 1 MiB: chunks (1024 slots each) x experts
static __device__ __align__(256) int32_t g_route_scratch[kStaticScratchInts];

constexpr int kMaxDevices = 64;
static std::mutex g_scratch_mutex;
static int32_t* g_scratch_ptr[kMaxDevices] = {};  // device address of g_route_scratch, per GPU

// In host code `g_route_scratch` is only a handle for the runtime, not a device address; the
// address on the current device has to be asked for.  Done once per device, on first use.
static int static_scratch_for_current_device(int32_t** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(B200MOE_UNSUPPORTED_DEVICE, "route_metadata_noalloc: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(B200MOE_UNSUPPORTED_DEVICE, "route_metadata_noalloc: device ordinal %d not in [0,%d)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    int32_t* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_route_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(B200MOE_LAUNCH_FAILED, "route_metadata_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return B200MOE_OK;
}

}  // namespace b200moe

extern "C" int b200moe_route_metadata_noalloc(const int64_t* topk_ids, int64_t num_slots,
                                              int num_experts, int64_t* reorder_topk_ids,
                                              int32_t* src2dst, int64_t* seg_indptr, void* stream) {
  B200MOE_REQUIRE(seg_indptr, B200MOE_BAD_ARG, "route_metadata_noalloc: null seg_indptr");
  B200MOE_REQUIRE(num_experts >= 1 && num_experts <= kMaxExperts, B200MOE_BAD_SHAPE,
                  "route_metadata_noalloc: num_experts=%d not in [1,%d]", num_experts, kMaxExperts);
  B200MOE_REQUIRE(num_slots >= 0 && num_slots < (int64_t(1) << 31), B200MOE_BAD_SHAPE,
                  "route_metadata_noalloc: num_slots=%lld does not fit int32 rows", (long long)num_slots);
  const int64_t chunks = (num_slots + kChunk - 1) / kChunk;
  B200MOE_REQUIRE(chunks * num_experts <= kStaticScratchInts, B200MOE_BAD_SHAPE,
                  "route_metadata_noalloc: ceil(num_slots/%d) * num_experts = %lld exceeds the built-in scratch of "
                  "%lld entries; use b200moe_route_metadata with a caller-provided workspace",
                  kChunk, (long long)(chunks * num_experts), (long long)kStaticScratchInts);
  cudaStream_t st = as_stream(stream);
  if (num_slots == 0) {
    cudaMemsetAsync(seg_indptr, 0, sizeof(int64_t) * (num_experts + 1), st);
    return check_launch("route_metadata_noalloc(memset)");
  }
  B200MOE_REQUIRE(topk_ids && reorder_topk_ids && src2dst, B200MOE_BAD_ARG, "route_metadata_noalloc: null pointer");
  int32_t* scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) return rc;
  // The table keeps whatever the previous call left in it.  Nothing has to be cleared: the
  // histogram pass stores (not adds) every one of the chunks x num_experts entries that the
  // later passes read.
  const unsigned grid = static_cast<unsigned>((chunks + kWarpsPerBlock - 1) / kWarpsPerBlock);
  const size_t smem = sizeof(int32_t) * kWarpsPerBlock * num_experts;
  route_hist_kernel<<<grid, kWarpsPerBlock * 32, smem, st>>>(topk_ids, num_slots, num_experts, scratch);
  route_scan_kernel<<<1, 1024, 0, st>>>(scratch, chunks, num_experts, seg_indptr);
  route_rank_kernel<<<grid, kWarpsPerBlock * 32, smem, st>>>(topk_ids, num_slots, num_experts, scratch,
                                                             seg_indptr, reorder_topk_ids, src2dst);
  return check_launch("route_metadata_noalloc");
}
