// Grouped w4a16 GEMM (asymmetric group-128 int4 weights, bf16 activations) with the dequantization fused into the
// operand path (no expanded copy of the weights).
//
// One persistent CTA per SM, 512 threads:
//   warp 0       TMA producer of the PACKED weights (+ the K group's (scale, zero) pairs as bulk copies), 6-slot ring
//   warp 2       TMA producer of the bf16 activation tile (box of 16/32/64/128 rows x 128 B), 3-slot ring
//   warps 12-15  converters: one packed word (8 consecutive k of one output channel, quantization/bitpack.py:38-67)
//                becomes one 16-byte chunk of a bf16 operand row, w = bf16((q - zero) * scale) as
//                b200moe_w4a16_expand_bf16 (the zero-point extension of
//                fast_dequant/simple_marlin/marlin_w4a16_gemm.cu:44-64), written in the 128-byte-swizzled layout the
//                tensor core reads (2 slots); fence.proxy.async, arrive
//   warp 1       owns TMEM; 4 x tcgen05.mma.kind::f16 (M128 N256 K16) per K block; there are no block scales, so the
//                whole K loop accumulates in TMEM (one stage per tile, the epilogue of tile i overlaps tile i + 1)
//   warps 4-11   tile epilogue (plain, or act(gate) * up); warps whose 32 rows lie beyond the group's rows skip it
// Each weight tile is converted once per (m-tile, n-tile): the kernel is for groups of about one m-tile (decode);
// callers with many rows per expert expand once instead.
//
// Every wait is a bounded mbarrier wait; on expiry the kernel drains its copies, frees TMEM, writes
// B200MOE_DEVICE_TIMEOUT to the status word and returns.
#include <cuda.h>

#include "common.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"
#include "w4_common.cuh"

namespace b200moe {
namespace w4 {

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int kAStages = 3, kBStages = 2, kAccStages = 2;
constexpr uint32_t kABytes = BM * BK, kBBytes = BN * BK;
constexpr int kThreads = 512;
constexpr int kFirstEpiWarp = 4, kEpiWarps = 8, kFirstConvWarp = 12, kConvWarps = 4;

struct Tile { int m0, m_end, expert, nt; };

constexpr int kQStages = 6;                              // packed ring: 256 rows x 8 words = 8 KB per K block
constexpr uint32_t kQBytes = 256 * 8 * 4;
constexpr uint32_t kQPair = 128 * 4;                     // (scale, zero) of the 128 channels of one half
constexpr uint32_t kQSlot = kQBytes + 2 * kQPair;
struct Tail16 {
  uint64_t a_full[kAStages], a_empty[kAStages];
  uint64_t p_full[kQStages], p_empty[kQStages];
  uint64_t b_full[kBStages], b_empty[kBStages];
  uint64_t tmem_full[kAccStages], tmem_empty[kAccStages];
  uint32_t tmem_base;
  int abort_flag;
  int32_t seg[kMaxGroups + 1];
  int32_t pref[kMaxGroups + 1];
};
constexpr size_t kRing16 = size_t(kAStages) * kABytes + size_t(kBStages) * kBBytes + size_t(kQStages) * kQSlot;
constexpr size_t kSmem16 = 1024 + kRing16 + sizeof(Tail16);

struct Params16 {
  const uint32_t* sz_t;           // [W, K/128, N]: (scale, zero) bf16 pairs (scale in the low half), one group's pairs contiguous
  void* c; int64_t c_stride;      // bytes
  const int64_t* seg; const int64_t* widx;
  int64_t M_total;
  int N, K, num_groups, c_dtype, fused, act;    // K in elements; fused: 0 plain, 1 act(gate)*up -> bf16
  int32_t* status;
};

// One packed word (nibble i = k 8c + i) -> eight bf16 values (q - zero) * scale as four bf16x2 registers in k order.
// 0x4300 | q is the bf16 number 128 + q; the two subtractions are exact and the product is rounded once, which is
// the f32 evaluation of (q - zero) * scale rounded to bf16.
__device__ __forceinline__ uint4 dequant_word_bf16(uint32_t w, uint32_t scale_zero) {
  const __nv_bfloat162 sc = __bfloat162bfloat162(__ushort_as_bfloat16(static_cast<unsigned short>(scale_zero & 0xFFFFu)));
  const __nv_bfloat162 zp = __bfloat162bfloat162(__ushort_as_bfloat16(static_cast<unsigned short>(scale_zero >> 16)));
  const __nv_bfloat162 c128 = __bfloat162bfloat162(__ushort_as_bfloat16(0x4300));
  uint32_t pr[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) pr[j] = ((w >> (4 * j)) & 0x000F000Fu) | 0x43004300u;     // (nibble j, nibble j + 4)
  const uint32_t o[4] = {__byte_perm(pr[0], pr[1], 0x5410), __byte_perm(pr[2], pr[3], 0x5410),
                         __byte_perm(pr[0], pr[1], 0x7632), __byte_perm(pr[2], pr[3], 0x7632)};
  uint32_t r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&o[j]);
    v = __hmul2(__hsub2(__hsub2(v, c128), zp), sc);
    r[j] = *reinterpret_cast<const uint32_t*>(&v);
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}

__device__ __forceinline__ Tile decode_tile16(const Tail16* sh, const Params16& p, int t, int num_n_tiles) {
  const int mt = t / num_n_tiles;
  int lo = 0, hi = p.num_groups;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sh->pref[mid] <= mt) lo = mid; else hi = mid;
  }
  Tile tl;
  tl.m0 = sh->seg[lo] + (mt - sh->pref[lo]) * BM;
  tl.m_end = sh->seg[lo + 1];
  tl.expert = p.widx ? static_cast<int>(p.widx[lo]) : lo;
  tl.nt = t - mt * num_n_tiles;
  return tl;
}


__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a16_kernel(const __grid_constant__ RowMaps tmap_a, const __grid_constant__ CUtensorMap tmap_p, const Params16 p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem_a + size_t(kAStages) * kABytes;
  uint8_t* smem_p = smem_b + size_t(kBStages) * kBBytes;         // kQStages x ([256 rows][8 words] + pairs)
  Tail16* sh = reinterpret_cast<Tail16*>(smem_p + size_t(kQStages) * kQSlot);
  volatile int* abort_flag = &sh->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = p.K / 64;                                        // 64 bf16 = 128 bytes per K block
  const int KG = p.K / 128;                                       // scale groups along K
  const int num_n_tiles = p.fused ? (p.N / 2) / 128 : (p.N + BN - 1) / BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kAStages; ++s) { ptx::mbar_init(&sh->a_full[s], 1); ptx::mbar_init(&sh->a_empty[s], 1); }
    for (int s = 0; s < kQStages; ++s) { ptx::mbar_init(&sh->p_full[s], 1); ptx::mbar_init(&sh->p_empty[s], kConvWarps); }
    for (int s = 0; s < kBStages; ++s) { ptx::mbar_init(&sh->b_full[s], kConvWarps); ptx::mbar_init(&sh->b_empty[s], 1); }
    for (int s = 0; s < kAccStages; ++s) { ptx::mbar_init(&sh->tmem_full[s], 1); ptx::mbar_init(&sh->tmem_empty[s], kEpiWarps); }
    sh->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
#pragma unroll
    for (int i = 0; i < 4; ++i) ptx::prefetch_tensormap(&tmap_a.m[i]);
    ptx::prefetch_tensormap(&tmap_p);
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(&sh->tmem_base, kTmemCols);
    ptx::tmem_relinquish<1>();
  }
  for (int g = threadIdx.x; g <= p.num_groups; g += kThreads) sh->seg[g] = static_cast<int32_t>(p.seg[g]);
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (warp == 3) {
    int run = 0;
    for (int g0 = 0; g0 < p.num_groups; g0 += 32) {
      const int g = g0 + lane;
      int v = 0;
      if (g < p.num_groups) { const int m = sh->seg[g + 1] - sh->seg[g]; v = m > 0 ? (m + BM - 1) / BM : 0; }
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
      if (g < p.num_groups) sh->pref[g] = run + incl - v;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) sh->pref[p.num_groups] = run;
  }
  __syncthreads();
  const uint32_t tmem_base = sh->tmem_base;
  const int total_tiles = sh->pref[p.num_groups] * num_n_tiles;
  const int first = static_cast<int>(blockIdx.x), step = static_cast<int>(gridDim.x);
  auto half_rows = [&](const Tile& tl, int& row0, int& row1) {   // first weight row of the tile's two 128-row halves
    row0 = tl.expert * p.N + (p.fused ? tl.nt * 128 : tl.nt * BN);
    row1 = p.fused ? tl.expert * p.N + p.N / 2 + tl.nt * 128 : row0 + 128;
  };

  if (warp < kFirstEpiWarp) {
    ptx::setmaxnreg_dec<48>();
    if (warp == 0 && lane == 0) {
      // packed weights: two boxes of 128 rows x 8 words per K block
      int stage = 0; uint32_t phase = 0;
      Armed armed;
      bool ok = true;
      for (int t = first; ok && t < total_tiles; t += step) {
        const Tile tl = decode_tile16(sh, p, t, num_n_tiles);
        int row0, row1;
        half_rows(tl, row0, row1);
        const int n0 = row0 - tl.expert * p.N, n1 = row1 - tl.expert * p.N;
        const bool second = n1 < p.N;
        for (int kb = 0; kb < KB; ++kb) {
          if (!ptx::mbar_wait(&sh->p_empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sp = smem_p + size_t(stage) * kQSlot;
          const uint32_t* sz = p.sz_t + (static_cast<int64_t>(tl.expert) * KG + (kb >> 1)) * p.N;   // a group spans 2 K blocks
          ptx::mbar_arrive_expect_tx(&sh->p_full[stage], kQBytes + kQPair + (second ? kQPair : 0u));
          armed.arm(stage, phase);
          ptx::tma_load_2d(sp, &tmap_p, &sh->p_full[stage], kb * 8, row0);
          ptx::tma_load_2d(sp + kQBytes / 2, &tmap_p, &sh->p_full[stage], kb * 8, row1);
          ptx::bulk_load(sp + kQBytes, sz + n0, kQPair, &sh->p_full[stage]);
          if (second) ptx::bulk_load(sp + kQBytes + kQPair, sz + n1, kQPair, &sh->p_full[stage]);
          if (++stage == kQStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) armed.drain(sh->p_full, kQStages);
    } else if (warp == 2 && lane == 0) {
      int stage = 0; uint32_t phase = 0;
      Armed armed;
      bool ok = true;
      auto box_sel = [](int rows) { return rows <= 16 ? 0 : (rows <= 32 ? 1 : (rows <= 64 ? 2 : 3)); };
      for (int t = first; ok && t < total_tiles; t += step) {
        const Tile tl = decode_tile16(sh, p, t, num_n_tiles);
        const int sel = box_sel(min(BM, tl.m_end - tl.m0));
        const uint32_t bytes = (16u << sel) * BK;
        for (int kb = 0; kb < KB; ++kb) {
          if (!ptx::mbar_wait(&sh->a_empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(&sh->a_full[stage], bytes);
          armed.arm(stage, phase);
          ptx::tma_load_2d(smem_a + size_t(stage) * kABytes, &tmap_a.m[sel], &sh->a_full[stage], kb * BK, tl.m0);
          if (++stage == kAStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) armed.drain(sh->a_full, kAStages);
    } else if (warp == 1 && lane == 0) {
      constexpr uint32_t idesc = ptx::umma_idesc(1, 1, 1, BM, BN);     // D f32, A and B bf16
      int sa = 0, sb = 0, as = 0;
      uint32_t pa = 0, pb = 0, pacc = 0;
      bool ok = true;
      for (int t = first; ok && t < total_tiles; t += step) {
        if (!ptx::mbar_wait(&sh->tmem_empty[as], pacc ^ 1u, abort_flag)) break;     // the stage's previous tile has been read
        const uint32_t d = tmem_base + static_cast<uint32_t>(as) * BN;
        for (int kb = 0; kb < KB; ++kb) {
          if (!ptx::mbar_wait(&sh->a_full[sa], pa, abort_flag) || !ptx::mbar_wait(&sh->b_full[sb], pb, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint64_t adesc = ptx::umma_desc_sw128(ptx::smem_u32(smem_a + size_t(sa) * kABytes));
          const uint64_t bdesc = ptx::umma_desc_sw128(ptx::smem_u32(smem_b + size_t(sb) * kBBytes));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) ptx::umma_f16<1>(d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          ptx::umma_commit(&sh->a_empty[sa]);
          ptx::umma_commit(&sh->b_empty[sb]);
          if (++sa == kAStages) { sa = 0; pa ^= 1u; }
          if (++sb == kBStages) { sb = 0; pb ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit(&sh->tmem_full[as]);        // the tile's accumulators are complete
        if (++as == kAccStages) { as = 0; pacc ^= 1u; }
      }
    }
  } else if (warp >= kFirstConvWarp) {
    // converters: thread t owns operand rows t and t + 128 of the tile (all 8 words = 64 k of each)
    ptx::setmaxnreg_dec<96>();
    const int ct = threadIdx.x - kFirstConvWarp * 32;       // 0..127
    int sp = 0, sb = 0;
    uint32_t pp = 0, pb = 0;
    bool ok = true;
    for (int t = first; ok && t < total_tiles; t += step) {
      const Tile tl = decode_tile16(sh, p, t, num_n_tiles);
      const bool second = (p.fused ? p.N / 2 + tl.nt * 128 : tl.nt * BN + 128) < p.N;
      for (int kb = 0; kb < KB; ++kb) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&sh->p_full[sp], pp, abort_flag)) ||
            !__all_sync(0xffffffffu, ptx::mbar_wait(&sh->b_empty[sb], pb ^ 1u, abort_flag))) { ok = false; break; }
        const uint4* src = reinterpret_cast<const uint4*>(smem_p + size_t(sp) * kQSlot);
        const uint32_t* pz = reinterpret_cast<const uint32_t*>(smem_p + size_t(sp) * kQSlot + kQBytes);
        const uint32_t sz0 = pz[ct], sz1 = second ? pz[128 + ct] : 0u;
        uint8_t* dst = smem_b + size_t(sb) * kBBytes;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int n = ct + h * 128;                        // operand row
          const uint4 w0 = src[n * 2], w1 = src[n * 2 + 1];
          const uint32_t wd[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          const uint32_t sz = h ? sz1 : sz0;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(dst + static_cast<uint32_t>(n) * 128u + ((static_cast<uint32_t>(c) ^ (n & 7u)) << 4)) =
                dequant_word_bf16(wd[c], sz);
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) { ptx::mbar_arrive(&sh->b_full[sb]); ptx::mbar_arrive(&sh->p_empty[sp]); }
        if (++sp == kQStages) { sp = 0; pp ^= 1u; }
        if (++sb == kBStages) { sb = 0; pb ^= 1u; }
      }
    }
  } else {
    // epilogue warps: one TMEM read-back per tile
    ptx::setmaxnreg_inc<184>();
    const int e = warp - kFirstEpiWarp, q = warp & 3, hsel = e >> 2;
    const int r_in_tile = q * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    int as = 0; uint32_t pacc = 0;
    bool ok = true;
    for (int t = first; ok && t < total_tiles; t += step) {
      const Tile tl = decode_tile16(sh, p, t, num_n_tiles);
      const bool live = q * 32 < min(BM, tl.m_end - tl.m0);
      const int row = tl.m0 + r_in_tile;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&sh->tmem_full[as], pacc, abort_flag))) { ok = false; break; }
      ptx::tc_fence_after_sync();
      float acc[128];
      if (live) {
        const uint32_t tcol = tmem_base + lane_base + static_cast<uint32_t>(as) * BN + static_cast<uint32_t>(hsel) * 64;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          ptx::tmem_ld32(tcol + (c >> 1) * 128 + (c & 1) * 32, r);
          ptx::tmem_ld_wait32(r);
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = __uint_as_float(r[j]);
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&sh->tmem_empty[as]);
      if (++as == kAccStages) { as = 0; pacc ^= 1u; }
      if (!live || row >= tl.m_end) continue;
      uint8_t* dst = static_cast<uint8_t*>(p.c) + static_cast<int64_t>(row) * p.c_stride;
      if (!p.fused) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int col0 = tl.nt * BN + half * 128 + hsel * 64;
          if (col0 >= p.N) continue;
          if (p.c_dtype == B200MOE_F32) store_row64(reinterpret_cast<float*>(dst) + col0, acc + half * 64);
          else if (p.c_dtype == B200MOE_BF16) store_row64(reinterpret_cast<__nv_bfloat16*>(dst) + col0, acc + half * 64);
          else store_row64(reinterpret_cast<__half*>(dst) + col0, acc + half * 64);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float g = bf16r(acc[j]);
          const float u = bf16r(acc[64 + j]);
          acc[j] = bf16r(gate_act(g, p.act)) * u;
        }
        store_row64(reinterpret_cast<__nv_bfloat16*>(dst) + tl.nt * 128 + hsel * 64, acc);
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc<1>(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && sh->abort_flag && p.status) *p.status = B200MOE_DEVICE_TIMEOUT;
}

}  // namespace w4
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_grouped_gemm_w4a16(const void* a, int64_t a_row_stride_bytes, const void* b_packed,
                                          const void* scale_zero_t, void* c, int c_dtype, int64_t c_row_stride_bytes,
                                          int64_t M_total, int64_t N, int64_t K, int num_groups, int num_weights,
                                          const int64_t* seg_indptr, const int64_t* weight_indices, int epilogue,
                                          int32_t* status_word, void* stream) {
  B200MOE_REQUIRE(a && b_packed && scale_zero_t && c && seg_indptr, B200MOE_BAD_ARG, "grouped_gemm_w4a16: null pointer");
  B200MOE_REQUIRE(epilogue == 0 || epilogue == 2 || epilogue == 5, B200MOE_BAD_ARG,
                  "grouped_gemm_w4a16: epilogue %d (0 plain, 2 SiLU*up, 5 GELU*up)", epilogue);
  B200MOE_REQUIRE(M_total >= 0 && M_total < (int64_t(1) << 31) && N > 0 && K > 0 && K % 128 == 0 && N % 128 == 0,
                  B200MOE_BAD_SHAPE, "grouped_gemm_w4a16: M=%lld N=%lld K=%lld (N and K must be multiples of 128)",
                  (long long)M_total, (long long)N, (long long)K);
  B200MOE_REQUIRE(num_groups >= 1 && num_groups <= w4::kMaxGroups && num_weights >= 1 &&
                  static_cast<int64_t>(num_weights) * N < (int64_t(1) << 31), B200MOE_BAD_SHAPE,
                  "grouped_gemm_w4a16: num_groups=%d (max %d) num_weights=%d", num_groups, w4::kMaxGroups, num_weights);
  B200MOE_REQUIRE(aligned(a, 16) && aligned(b_packed, 16) && aligned(scale_zero_t, 4) && aligned(c, 16) &&
                  a_row_stride_bytes % 16 == 0 && a_row_stride_bytes >= 2 * K && c_row_stride_bytes % 16 == 0,
                  B200MOE_BAD_ALIGN, "grouped_gemm_w4a16: pointers and row strides must be 16-byte aligned");
  if (epilogue != 0) {
    B200MOE_REQUIRE(N % 256 == 0 && c_dtype == B200MOE_BF16 && c_row_stride_bytes >= N, B200MOE_BAD_ARG,
                    "grouped_gemm_w4a16: the fused epilogue needs N %% 256 == 0 and a bf16 [M, N/2] output");
  } else {
    B200MOE_REQUIRE(c_dtype == B200MOE_F32 || c_dtype == B200MOE_F16 || c_dtype == B200MOE_BF16, B200MOE_BAD_DTYPE,
                    "grouped_gemm_w4a16: c dtype %d", c_dtype);
    B200MOE_REQUIRE(c_row_stride_bytes >= N * (c_dtype == B200MOE_F32 ? 4 : 2), B200MOE_BAD_ARG, "grouped_gemm_w4a16: c row stride too small");
  }
  if (M_total == 0) return B200MOE_OK;
  int sms = 0;
  if (int rc = require_sm100(&sms)) return rc;
  w4::RowMaps ma;
  CUtensorMap mp;
  for (int i = 0; i < 4; ++i)
    if (int rc = cached_tensor_map_u8(&ma.m[i], a, static_cast<uint64_t>(M_total), static_cast<uint64_t>(2 * K),
                                      static_cast<uint64_t>(a_row_stride_bytes), 16u << i)) return rc;
  if (int rc = make_tensor_map_i32_plain(&mp, b_packed, static_cast<uint64_t>(num_weights) * N, static_cast<uint64_t>(K / 8),
                                         static_cast<uint64_t>(K / 8) * 4, 8, 128)) return rc;
  w4::Params16 p{static_cast<const uint32_t*>(scale_zero_t), c, c_row_stride_bytes, seg_indptr, weight_indices, M_total,
                 static_cast<int>(N), static_cast<int>(K), num_groups, c_dtype, epilogue != 0 ? 1 : 0,
                 epilogue == 5 ? 1 : 0, status_word};
  cudaFuncSetAttribute(w4::gemm_w4a16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(w4::kSmem16));
  w4::gemm_w4a16_kernel<<<sms, w4::kThreads, w4::kSmem16, as_stream(stream)>>>(ma, mp, p);
  return check_launch("gemm_w4a16_kernel");
}
