// Expert-parallel exchange folded into the kernels on either side of it, over peer-mapped memory.
//
// The reference's layer (moe/all2all_moe.py:131-262) sorts its slots by destination rank, runs
// all_to_all_single with host-side split sizes, computes, and runs the all-to-all back.  Here
// every rank maps every peer's receive and return buffers (NVLink peer mappings) and
//   1. all-gathers the per-expert slot counts (the only collective; E integers per rank),
//   2. ep_plan:   from the counts, on the device, where each of my expert blocks starts in its
//                 owner's receive buffer, my own group table, and for every row I will receive
//                 the address in its source rank's return buffer,
//   3. permute_quant_fp8_push: quantizes my tokens and stores each record straight into the
//                 owner's receive buffer, already grouped by (expert, source rank),
//   4. the grouped GEMMs run on the receive buffer; the down projection's epilogue stores every
//                 output row at its return address (grouped_gemm_fp8, c_row_addr).
// Nothing is read back by the host, so the whole layer is stream-ordered.  The two points where a
// rank must know that its peers' stores have landed (before the first GEMM, before the
// un-permute) are stream-ordered barriers issued by the caller.
#include "common.cuh"

namespace b200moe {

constexpr int kPlanThreads = 1024;

// One block.  counts[s * E + e]: slots rank s routes to global expert e (owner e / El).
//   dst_base[e]        byte address, in owner(e)'s receive buffer, of my first record for expert e
//                      (0 when that block does not fit: its records are dropped and info[1] is set)
//   local_seg[El + 1]  my group table: rows of local expert el are [local_seg[el], local_seg[el+1])
//   blk_start[El*ep+1] first receive row of block (el, s);  blk_dst[El*ep] return address of that row
//   info[0] rows received, info[1] overflow flag
// Capacity rule, the same on both sides: the block (expert e, source s) is accepted iff it fits whole,
// start + count <= cap_rows.  Block starts grow with (e, s), so the accepted blocks are a prefix of the
// owner's buffer: the owner computes only rows below the first rejected block's start, the source writes no
// record of a rejected block (and zero-fills the return rows of those slots, permute_quant_fp8_push).
__global__ void __launch_bounds__(kPlanThreads) ep_plan_kernel(
    const int64_t* __restrict__ counts, int rank, int ep, int E, int64_t cap_rows,
    const int64_t* __restrict__ recv_base, int64_t rec_bytes, const int64_t* __restrict__ back_base,
    int64_t back_row_bytes, int64_t* __restrict__ dst_base, int64_t* __restrict__ local_seg,
    int32_t* __restrict__ blk_start, int64_t* __restrict__ blk_dst, int32_t* __restrict__ info) {
  extern __shared__ int32_t sm[];
  int32_t* c = sm;                 // [ep][E] counts
  int32_t* pre = c + ep * E;       // [ep][E] exclusive prefix over e (rank s's own sorted order)
  int32_t* tot = pre + ep * E;     // [E]     rows expert e receives from all ranks
  int32_t* totpre = tot + E;       // [E + 1] exclusive prefix of tot
  const int El = E / ep;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  __shared__ int valid_rows;       // start of the first rejected block of MY buffer (all rows if none)
  for (int i = tid; i < ep * E; i += blockDim.x) c[i] = static_cast<int32_t>(counts[i]);
  if (tid == 0) { info[0] = 0; info[1] = 0; valid_rows = 0x7fffffff; }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < ep; ++s) t += c[s * E + e];
    tot[e] = t;
  }
  __syncthreads();
  // exclusive scans: rows 0..ep-1 are the per-rank counts, row ep is tot
  for (int r = warp; r <= ep; r += nwarps) {
    const int32_t* src = r < ep ? c + r * E : tot;
    int32_t* dst = r < ep ? pre + r * E : totpre;
    int run = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int v = e < E ? src[e] : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
      if (e < E) dst[e] = run + incl - v;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (r == ep && lane == 0) totpre[E] = run;
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    const int d = e / El;
    int64_t row = totpre[e] - totpre[d * El];
    for (int s = 0; s < rank; ++s) row += c[s * E + e];
    const bool fits = row + c[rank * E + e] <= cap_rows;
    dst_base[e] = fits ? recv_base[d] + row * rec_bytes : 0;
    if (!fits && c[rank * E + e] > 0) info[1] = 1;
  }
  for (int el = tid; el < El; el += blockDim.x) {          // first rejected block of my own buffer
    const int e = rank * El + el;
    int64_t run = totpre[e] - totpre[rank * El];
    for (int s = 0; s < ep; ++s) {
      const int cnt = c[s * E + e];
      if (cnt > 0 && run + cnt > cap_rows) { atomicMin(&valid_rows, static_cast<int>(min(run, cap_rows))); break; }
      run += cnt;
    }
  }
  __syncthreads();
  const int64_t all_rows = totpre[rank * El + El] - totpre[rank * El];
  const int64_t valid = min(static_cast<int64_t>(valid_rows), all_rows);
  for (int el = tid; el < El; el += blockDim.x) {
    const int e = rank * El + el;
    const int64_t ls = totpre[e] - totpre[rank * El];
    local_seg[el] = min(ls, valid);
    int64_t run = ls;
    for (int s = 0; s < ep; ++s) {
      blk_start[el * ep + s] = static_cast<int32_t>(min(run, valid));
      blk_dst[el * ep + s] = back_base[s] + static_cast<int64_t>(pre[s * E + e]) * back_row_bytes;
      run += c[s * E + e];
    }
    if (el == El - 1) {
      local_seg[El] = valid;
      blk_start[El * ep] = static_cast<int32_t>(valid);
      info[0] = static_cast<int32_t>(valid);
      if (valid < all_rows) info[1] = 1;
    }
  }
}

// back_addr[r] for every received row r: the block holding r by binary search.
__global__ void __launch_bounds__(256) ep_back_addr_kernel(const int32_t* __restrict__ blk_start,
                                                           const int64_t* __restrict__ blk_dst, int nblk,
                                                           int64_t back_row_bytes, int64_t cap_rows,
                                                           int64_t* __restrict__ back_addr) {
  const int total = blk_start[nblk];
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; r < cap_rows;
       r += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    if (r >= total) { back_addr[r] = 0; continue; }
    int lo = 0, hi = nblk;                      // last b with blk_start[b] <= r
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (blk_start[mid] <= r) lo = mid; else hi = mid;
    }
    back_addr[r] = blk_dst[lo] + (r - blk_start[lo]) * back_row_bytes;
  }
}

constexpr int kMaxTopK = 32;

// One CTA per token (as permute_quant_fp8).  The token's record (payload, then the f32 scales at
// byte H) is built ONCE in shared memory and then copied to each of its destinations,
// dst_base[e] + (src2dst[slot] - seg[e]) * rec_bytes, by one bulk asynchronous copy per destination:
// a record crosses NVLink as a few large writes issued by the copy hardware instead of hundreds of
// 8-byte stores from the SM.
template <typename TI>
__global__ void __launch_bounds__(256) permute_quant_fp8_push_kernel(
    const TI* __restrict__ x, const int32_t* __restrict__ src2dst, const int64_t* __restrict__ topk_ids,
    const int64_t* __restrict__ seg, const int64_t* __restrict__ dst_base, int num_experts, int topk,
    int64_t H, int64_t rec_bytes, uint8_t* __restrict__ back_local, int64_t back_row_bytes) {
  extern __shared__ __align__(128) uint8_t s_rec[];
  __shared__ int64_t s_addr[kMaxTopK];
  __shared__ int32_t s_drop[kMaxTopK];
  __shared__ int s_n, s_nd;
  const int64_t t = blockIdx.x;
  if (threadIdx.x == 0) {
    int n = 0, nd = 0;
    for (int j = 0; j < topk; ++j) {
      const int64_t e = topk_ids[t * topk + j];
      const int32_t d = src2dst[t * topk + j];
      if (e < 0 || e >= num_experts || d < 0) continue;
      const int64_t base = dst_base[e];
      if (base == 0) { s_drop[nd++] = d; continue; }   // the owner's buffer is full: dropped, flagged by ep_plan
      s_addr[n++] = base + (static_cast<int64_t>(d) - seg[e]) * rec_bytes;
    }
    s_n = n; s_nd = nd;
  }
  __syncthreads();
  const int n = s_n;
  // a dropped slot gets no result back: its row of my return buffer is cleared, so the un-permute adds zeros
  // instead of what an earlier step left there
  if (back_local)
    for (int j = 0; j < s_nd; ++j)
      for (int64_t b = threadIdx.x * 16; b < back_row_bytes; b += blockDim.x * 16)
        *reinterpret_cast<uint4*>(back_local + static_cast<int64_t>(s_drop[j]) * back_row_bytes + b) = make_uint4(0, 0, 0, 0);
  if (n == 0) return;
  const int64_t chunks = H / 8;
  const int64_t padded = (chunks + 31) & ~int64_t(31);
  for (int64_t i = threadIdx.x; i < padded; i += blockDim.x) {
    const bool live = i < chunks;
    float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (live) load8(x + t * H + i * 8, v);
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!live) continue;
    const float scale = __fdiv_rn(amax, 448.f);
    float q[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) q[k] = __fdiv_rn(v[k], scale);
    *reinterpret_cast<uint2*>(s_rec + i * 8) = pack8_e4m3(q);
    if ((threadIdx.x & 15) == 0) *reinterpret_cast<float*>(s_rec + H + (i / 16) * 4) = scale;
  }
  for (int64_t b = H + (H / 128) * 4 + threadIdx.x; b < rec_bytes; b += blockDim.x) s_rec[b] = 0;   // padding
  // make the generic-proxy writes visible to the bulk-copy engine, then one copy per destination
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < n) {
    const uint32_t src = static_cast<uint32_t>(__cvta_generic_to_shared(s_rec));
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(s_addr[threadIdx.x]), "r"(src), "r"(static_cast<uint32_t>(rec_bytes)) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the copy has been performed, not only read
    __threadfence_system();     // the records are read by another GPU after a stream-ordered barrier
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int64_t b200moe_ep_plan_workspace_bytes(int ep_size, int num_experts) {
  if (ep_size < 1 || num_experts < 1 || num_experts % ep_size) return -1;
  const int64_t nblk = num_experts;     // (E / ep) local experts x ep sources
  return (nblk + 1) * 4 + 12 /* pad to 8 */ + nblk * 8;
}

extern "C" int b200moe_ep_plan(const int64_t* counts_all, int rank, int ep_size, int num_experts, int64_t cap_rows,
                               const int64_t* recv_base, int64_t rec_bytes, const int64_t* back_base,
                               int64_t back_row_bytes, int64_t* dst_base, int64_t* local_seg,
                               int64_t* back_addr, int32_t* info, void* workspace, int64_t workspace_bytes,
                               void* stream) {
  B200MOE_REQUIRE(counts_all && recv_base && back_base && dst_base && local_seg && back_addr && info && workspace,
                  B200MOE_BAD_ARG, "ep_plan: null pointer");
  B200MOE_REQUIRE(ep_size >= 1 && ep_size <= 64 && rank >= 0 && rank < ep_size && num_experts >= ep_size &&
                  num_experts % ep_size == 0, B200MOE_BAD_SHAPE,
                  "ep_plan: rank %d of %d, %d experts", rank, ep_size, num_experts);
  const int64_t smem = (int64_t(2) * ep_size * num_experts + 2 * num_experts + 1) * 4;
  B200MOE_REQUIRE(smem <= 200 * 1024, B200MOE_BAD_SHAPE, "ep_plan: ep_size * num_experts = %d too large",
                  ep_size * num_experts);
  B200MOE_REQUIRE(cap_rows > 0 && cap_rows < (int64_t(1) << 31) && rec_bytes > 0 && rec_bytes % 16 == 0 &&
                  back_row_bytes > 0 && back_row_bytes % 16 == 0, B200MOE_BAD_ARG,
                  "ep_plan: capacity %lld, record %lld B, return row %lld B", (long long)cap_rows,
                  (long long)rec_bytes, (long long)back_row_bytes);
  B200MOE_REQUIRE(workspace_bytes >= b200moe_ep_plan_workspace_bytes(ep_size, num_experts) && aligned(workspace, 8),
                  B200MOE_WORKSPACE_TOO_SMALL, "ep_plan: workspace");
  const int nblk = num_experts;
  int32_t* blk_start = static_cast<int32_t*>(workspace);
  int64_t* blk_dst = reinterpret_cast<int64_t*>(static_cast<uint8_t*>(workspace) + ((nblk + 1) * 4 + 7) / 8 * 8);
  cudaStream_t st = as_stream(stream);
  cudaFuncSetAttribute(ep_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  ep_plan_kernel<<<1, kPlanThreads, smem, st>>>(counts_all, rank, ep_size, num_experts, cap_rows, recv_base, rec_bytes,
                                                back_base, back_row_bytes, dst_base, local_seg, blk_start, blk_dst, info);
  if (int rc = check_launch("ep_plan")) return rc;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((cap_rows + 255) / 256, 148 * 8));
  ep_back_addr_kernel<<<grid, 256, 0, st>>>(blk_start, blk_dst, nblk, back_row_bytes, cap_rows, back_addr);
  return check_launch("ep_back_addr");
}

extern "C" int b200moe_permute_quant_fp8_push(const void* x, int x_dtype, const int32_t* src2dst,
                                              const int64_t* topk_ids, const int64_t* seg_indptr,
                                              const int64_t* dst_base, int num_experts, int64_t T, int topk,
                                              int64_t H, int64_t rec_bytes, void* back_local,
                                              int64_t back_row_bytes, void* stream) {
  if (T == 0) return B200MOE_OK;      // an empty batch has no buffers to check
  B200MOE_REQUIRE(x && src2dst && topk_ids && seg_indptr && dst_base, B200MOE_BAD_ARG, "permute_quant_fp8_push: null pointer");
  B200MOE_REQUIRE(T >= 0 && H > 0 && H % 128 == 0, B200MOE_BAD_SHAPE,
                  "permute_quant_fp8_push: hidden_size=%lld must be divisible by block_size (block_size=128)", (long long)H);
  B200MOE_REQUIRE(topk >= 1 && topk <= kMaxTopK, B200MOE_BAD_SHAPE, "permute_quant_fp8_push: topk=%d", topk);
  B200MOE_REQUIRE(rec_bytes >= H + (H / 128) * 4 && rec_bytes % 16 == 0 && aligned(x, 16), B200MOE_BAD_ARG,
                  "permute_quant_fp8_push: record of %lld bytes for hidden_size %lld", (long long)rec_bytes, (long long)H);
  B200MOE_REQUIRE(back_local == nullptr || (aligned(back_local, 16) && back_row_bytes > 0 && back_row_bytes % 16 == 0),
                  B200MOE_BAD_ALIGN, "permute_quant_fp8_push: return buffer rows must be 16-byte multiples");
  if (T == 0) return B200MOE_OK;
  cudaStream_t st = as_stream(stream);
  const int64_t chunks = H / 8;
  const int th = chunks >= 256 ? 256 : static_cast<int>((chunks + 31) / 32 * 32);
  const unsigned grid = static_cast<unsigned>(T);
  const size_t smem = static_cast<size_t>(rec_bytes);
  uint8_t* bl = static_cast<uint8_t*>(back_local);
  B200MOE_REQUIRE(rec_bytes <= 40 * 1024, B200MOE_BAD_SHAPE, "permute_quant_fp8_push: record of %lld bytes (max 40960)",
                  (long long)rec_bytes);
  switch (x_dtype) {
    case B200MOE_BF16:
      permute_quant_fp8_push_kernel<__nv_bfloat16><<<grid, th, smem, st>>>(static_cast<const __nv_bfloat16*>(x), src2dst, topk_ids,
                                                                        seg_indptr, dst_base, num_experts, topk, H, rec_bytes, bl, back_row_bytes);
      break;
    case B200MOE_F16:
      permute_quant_fp8_push_kernel<__half><<<grid, th, smem, st>>>(static_cast<const __half*>(x), src2dst, topk_ids,
                                                                 seg_indptr, dst_base, num_experts, topk, H, rec_bytes, bl, back_row_bytes);
      break;
    case B200MOE_F32:
      permute_quant_fp8_push_kernel<float><<<grid, th, smem, st>>>(static_cast<const float*>(x), src2dst, topk_ids,
                                                                seg_indptr, dst_base, num_experts, topk, H, rec_bytes, bl, back_row_bytes);
      break;
    default:
      return fail(B200MOE_BAD_DTYPE, "permute_quant_fp8_push: x dtype %d", x_dtype);
  }
  return check_launch("permute_quant_fp8_push");
}
