// fp8 (e4m3) blockwise-scaled GEMMs on the 5th-generation tensor cores.
//
//   dense    fp8_gemm             quantization/fp8_kernel.py:108-190
//   grouped  grouped_gemm_triton  moe/group_gemm_kernel.py:291-513 (block_shape=[128,128])
//
// Semantics (both): for every 128-wide K block kb
//     acc[m,n] += dot_kb(a[m,:], b[n,:]) * a_s[m,kb] * b_s[n/128,kb]
// The f32 scales are not a hardware block-scale format, so the promotion is done
// by CUDA cores: the tensor core produces the unscaled dot of one K block into a
// TMEM stage, epilogue warps read it back (tcgen05.ld) and FMA it into register
// accumulators while the tensor core fills the other TMEM stage.
//
// One persistent CTA per SM, 384 threads = 3 warpgroups:
//   warp 0      TMA producer: A tile 128x128 B, B tile 256x128 B per K block
//               (two 128-row boxes: gate rows + up rows for the SwiGLU epilogue,
//               or two consecutive N blocks otherwise), 4-stage ring
//   warp 1      owns TMEM (512 columns = 2 stages x 256 f32 columns), issues
//               4 x tcgen05.mma.kind::f8f6f4 (M128 N256 K32) per K block
//   warps 2-3   idle (they complete the first warpgroup, which gives its registers away)
//   warps 4-11  promotion + epilogue; warp w reads TMEM lanes 32*(w%4)..+31 and
//               64 gate + 64 up (or 64 + 64 plain) columns -> 128 accumulators plus
//               64 staging registers, so that two 32-column TMEM loads are always in
//               flight (setmaxnreg: 56 registers for warpgroup 0, 224 for the other two)
// Tiles are (group, m-tile, n-tile) with n fastest, so CTAs running together
// share an A tile and walk one expert's weights once through L2.
//
// Every wait is a bounded mbarrier wait; on expiry the kernel drains, frees TMEM,
// writes B200MOE_DEVICE_TIMEOUT to the status word and returns.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace b200moe {

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int kStages = 4;          // single-CTA tiles: 4 x (16 KB A + 32 KB B)
constexpr int kPairStages = 6;      // CTA pairs:        6 x (16 KB A + 16 KB B) per CTA
constexpr int kMaxStages = 6;
constexpr int kAccStages = 2;
constexpr int kEpiWarps = 8;
constexpr int kFirstEpiWarp = 4;
constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;
constexpr uint32_t kABytes = BM * BK;
constexpr uint32_t kBBytes = BN * BK;
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr int kMaxGroups = 1024;
constexpr uint32_t kTmemCols = 512;

struct SharedTail {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[kAccStages];
  uint64_t tmem_empty[kAccStages];
  uint64_t amax_bar[2];
  uint32_t tmem_base;
  int abort_flag;
  float amax[2][2][BM];          // [buffer][column half][row]
  alignas(16) uint8_t out_stage[kEpiWarps][2048];   // per warp: 16 rows x 128 B, 16-byte chunks XOR-swizzled
  int32_t seg[kMaxGroups + 1];   // row offsets of the groups
  int32_t pref[kMaxGroups + 1];  // exclusive prefix of m-tiles per group
};
constexpr uint32_t kPairStageBytes = kABytes + kBBytes / 2;
static_assert(kPairStages * kPairStageBytes == kStages * kStageBytes, "both layouts use the same ring size");
constexpr size_t kSmemBytes = 1024 + size_t(kStages) * kStageBytes + sizeof(SharedTail);

struct GemmParams {
  const float* a_s; int64_t a_s_stride;
  const float* b_s;
  void* c; int64_t c_stride;          // bytes
  float* c_s; int64_t c_s_stride;     // floats
  const int64_t* seg; const int64_t* widx;
  int64_t M_total;
  int N, K, num_groups, num_weights, c_dtype, swiglu;
  int32_t* status;
  // kBf16 only: split the K loop over `ksplits` tiles that write partial products `split_stride`
  // bytes apart (the caller sums them in a fixed order), and let the activation's K coordinate
  // wrap every `a_wrap` bytes (K = repeats of the same activation columns against different
  // weight columns, e.g. a weight split into bf16 hi/mid/lo parts).
  int ksplits; int64_t split_stride; int a_wrap;
  // plain epilogue: output row r is stored at row c_row_map[r] (null = identity)
  const int32_t* c_row_map;
  // plain epilogue: output row r is stored at the byte address c_row_addr[r] (null = unused).
  // The addresses may lie in another GPU's memory (peer mapping): the rows then cross NVLink as
  // plain stores straight from the epilogue, and the kernel ends with a system-scope fence.
  const int64_t* c_row_addr;
  // plain epilogue with a 16-bit output: c = round(c + round(product)), the sum a module computes
  // when it adds this GEMM's output to a tensor of the same dtype (shared experts added to the
  // routed output, moe/all2all_moe.py:182-183)
  int accumulate;
  // fused gate/up epilogues (swiglu != 0): 0 = SiLU, 1 = tanh-GELU
  int act;
};

struct Tile { int m0, m_end, expert, nt, ks; };

// The activation tile is fetched with the smallest of four boxes (16/32/64/128 rows) that covers
// the rows the group still has: a ragged group then moves only its own rows through L2 and the
// crossbar.  The tensor core still reads 128 rows; the stale ones only feed output rows that are
// never stored.
struct RowMaps { CUtensorMap m[4]; };

// bmt: rows per tile (128, or 256 for a CTA pair); m_off: row offset of this CTA inside the tile.
__device__ __forceinline__ Tile decode_tile(const SharedTail* sh, const GemmParams& p, int t,
                                            int num_n_tiles, int bmt = BM, int m_off = 0) {
  const int per = num_n_tiles * p.ksplits;
  const int mt = t / per;
  int lo = 0, hi = p.num_groups;           // last g with pref[g] <= mt
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sh->pref[mid] <= mt) lo = mid; else hi = mid;
  }
  Tile tl;
  tl.m0 = sh->seg[lo] + (mt - sh->pref[lo]) * bmt + m_off;
  tl.m_end = sh->seg[lo + 1];
  tl.expert = p.widx ? static_cast<int>(p.widx[lo]) : lo;
  const int rem = t - mt * per;
  tl.nt = rem / p.ksplits;
  tl.ks = rem - tl.nt * p.ksplits;
  return tl;
}

// Operand kinds.  All three share the pipeline; K is counted in bytes (128 per K block).
//   kFp8  e4m3 x e4m3 -> f32, per-K-block promotion with f32 scales
//   kI8   s8 x s8 -> s32,     per-K-block promotion with f32 scales (w4a8 path: weights arrive
//                             as int8 after the int4 -> int8 step of quantization/w4a8_kernel.py:44-101)
//   kBf16 bf16 x bf16 -> f32, no scales: the whole K loop accumulates in TMEM and the epilogue
//                             warps read each tile once (w4a16 path after dequantization)
enum : int { kFp8 = 0, kI8 = 1, kBf16 = 2, kF16 = 3 };   // kF16: as kBf16 with f16 operands

template <int KIND, int CG>
__device__ __forceinline__ void umma_kind(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  if constexpr (KIND == kFp8) ptx::umma_f8f6f4<CG>(d, a, b, idesc, acc);
  else if constexpr (KIND == kI8) ptx::umma_i8<CG>(d, a, b, idesc, acc);
  else ptx::umma_f16<CG>(d, a, b, idesc, acc);
}

template <int KIND>
__device__ __forceinline__ float tmem_value(uint32_t r) {
  if constexpr (KIND == kI8) return __int2float_rn(static_cast<int>(r));
  else return __uint_as_float(r);
}

// acc[0..32) += value(r[0..32)) * s.  The promotion is bound by FMA issue slots (8 warps x 128
// accumulators per K block), so f32 products go through the packed two-wide FMA.
template <int KIND>
__device__ __forceinline__ void promote32(float* acc, const uint32_t (&r)[32], float s) {
  if constexpr (KIND == kI8) {
#pragma unroll
    for (int j = 0; j < 32; ++j) acc[j] = fmaf(tmem_value<KIND>(r[j]), s, acc[j]);
  } else {
    const uint64_t s2 = ptx::pack_f32x2(s, s);
#pragma unroll
    for (int j = 0; j < 32; j += 2) ptx::ffma2(acc[j], acc[j + 1], r[j], r[j + 1], s2);
  }
}

// PAIR: the kernel is launched in clusters of two CTAs that share one 256 x 256 tile
// (tcgen05 cta_group::2).  CTA r of the pair loads rows [128 r, 128 r + 128) of the activation tile
// and the r-th 128-row box of the weight tile, so each SM moves 32 KB per K block through the
// crossbar instead of 48 KB; the even CTA (the leader) issues the MMAs for both, and each CTA
// promotes and stores the 128 x 256 half that lands in its own tensor memory.  All barriers that
// order the pair live in the leader: both CTAs' loads count their bytes on the leader's `full`
// barrier, the leader's commits arrive on `empty` and `tmem_full` of both CTAs, and both CTAs'
// promotion warps arrive on the leader's `tmem_empty`.
template <int KIND, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
gemm_block_kernel(const __grid_constant__ RowMaps tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedTail* sh = reinterpret_cast<SharedTail*>(smem + size_t(kStages) * kStageBytes);
  volatile int* abort_flag = &sh->abort_flag;
  constexpr int CG = PAIR ? 2 : 1;
  constexpr int NS = PAIR ? kPairStages : kStages;                  // ring depth
  constexpr uint32_t SB = PAIR ? kPairStageBytes : kStageBytes;     // bytes per ring slot in this CTA
  constexpr int BMT = PAIR ? 2 * BM : BM;                           // rows per tile
  const uint32_t cta_r = PAIR ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_r == 0;
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int nworkers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int m_off = static_cast<int>(cta_r) * BM;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = p.K / BK;                         // p.K is the K extent in BYTES
  constexpr bool kPromote = KIND == kFp8 || KIND == kI8;
  const int NB = p.N / 128;
  const int num_n_tiles = p.swiglu ? (p.N / 2) / 128 : (p.N + BN - 1) / BN;   // swiglu: 0 plain, 1 -> e4m3 + scales, 2 -> bf16

  // ---- setup: barriers, TMEM, group table -----------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) { ptx::mbar_init(&sh->full[s], 1); ptx::mbar_init(&sh->empty[s], 1); }
    for (int s = 0; s < kAccStages; ++s) { ptx::mbar_init(&sh->tmem_full[s], 1); ptx::mbar_init(&sh->tmem_empty[s], CG * kEpiWarps); }
    ptx::mbar_init(&sh->amax_bar[0], kEpiWarps);
    ptx::mbar_init(&sh->amax_bar[1], kEpiWarps);
    sh->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
#pragma unroll
    for (int i = 0; i < 4; ++i) ptx::prefetch_tensormap(&tmap_a.m[i]);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc<CG>(&sh->tmem_base, kTmemCols);
    ptx::tmem_relinquish<CG>();
  }
  // group row offsets
  for (int g = threadIdx.x; g <= p.num_groups; g += kThreads)
    sh->seg[g] = p.seg ? static_cast<int32_t>(p.seg[g]) : (g == 0 ? 0 : static_cast<int32_t>(p.M_total));
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (warp == 2) {  // exclusive prefix of m-tiles per group, 32 groups per step
    int run = 0;
    for (int g0 = 0; g0 < p.num_groups; g0 += 32) {
      const int g = g0 + lane;
      int v = 0;
      if (g < p.num_groups) { const int m = sh->seg[g + 1] - sh->seg[g]; v = m > 0 ? (m + BMT - 1) / BMT : 0; }
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
      if (g < p.num_groups) sh->pref[g] = run + incl - v;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) sh->pref[p.num_groups] = run;
  }
  __syncthreads();
  if constexpr (PAIR) ptx::cluster_sync();   // the peer's barriers exist before anything is sent to them
  const uint32_t tmem_base = sh->tmem_base;
  const int total_tiles = sh->pref[p.num_groups] * num_n_tiles * p.ksplits;
  const int KBs = (KB + p.ksplits - 1) / p.ksplits;   // K blocks per split

  // Register hand-over: the producer/MMA warpgroup keeps 56 registers per thread, the two
  // promotion warpgroups grow to 224 (384 x 168 = 128 x 56 + 256 x 224).
  if (warp < kFirstEpiWarp) {
    ptx::setmaxnreg_dec<56>();
  if (warp == 0) {
    // ================================ TMA producer ================================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      uint32_t armed = 0, armed_parity = 0;
      bool ok = true;
      auto box_sel = [](int rows) { return rows <= 16 ? 0 : (rows <= 32 ? 1 : (rows <= 64 ? 2 : 3)); };
      for (int t = worker; ok && t < total_tiles; t += nworkers) {
        const Tile tl = decode_tile(sh, p, t, num_n_tiles, BMT, m_off);
        const int brow0 = tl.expert * p.N + (p.swiglu ? tl.nt * 128 : tl.nt * BN);
        const int brow1 = p.swiglu ? tl.expert * p.N + p.N / 2 + tl.nt * 128 : brow0 + 128;
        // a half with no rows left (second CTA of a pair on a group's last tile) still fetches the
        // smallest box, at or past the group's end: the rows are never stored
        const int sel = box_sel(min(BM, tl.m_end - tl.m0));
        const CUtensorMap* ma = &tmap_a.m[sel];
        uint32_t bytes = kBBytes + (16u << sel) * BK;
        if constexpr (PAIR) bytes += (16u << box_sel(min(BM, tl.m_end - (tl.m0 + BM)))) * BK;   // the peer's box (leader only)
        for (int kb = tl.ks * KBs, kb1 = min(KB, kb + KBs); kb < kb1; ++kb) {
          if (!ptx::mbar_wait(&sh->empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + size_t(stage) * SB;
          uint8_t* sb = sa + kABytes;
          const int kx = p.a_wrap ? (kb * BK) % p.a_wrap : kb * BK;
          if constexpr (PAIR) {
            if (leader) {
              ptx::mbar_arrive_expect_tx(&sh->full[stage], bytes);
              armed |= 1u << stage;
              armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
            }
            const uint32_t bar = ptx::map_to_cta(ptx::smem_u32(&sh->full[stage]), 0);
            ptx::tma_load_2d_pair(sa, ma, bar, kx, tl.m0);
            ptx::tma_load_2d_pair(sb, &tmap_b, bar, kb * BK, leader ? brow0 : brow1);
          } else {
            ptx::mbar_arrive_expect_tx(&sh->full[stage], bytes);
            armed |= 1u << stage;
            armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
            ptx::tma_load_2d(sa, ma, &sh->full[stage], kx, tl.m0);
            ptx::tma_load_2d(sb, &tmap_b, &sh->full[stage], kb * BK, brow0);
            ptx::tma_load_2d(sb + kBBytes / 2, &tmap_b, &sh->full[stage], kb * BK, brow1);
          }
          if (++stage == NS) { stage = 0; phase ^= 1u; }
        }
      }
      if constexpr (PAIR) {
        // Neither CTA of a pair may leave while the other still reads its shared memory or signals
        // its barriers: wait until every slot this CTA filled has been released by the MMAs.
        for (int s = 0; ok && s < NS; ++s) {
          if (!ptx::mbar_wait(&sh->empty[stage], phase ^ 1u, abort_flag)) ok = false;
          if (++stage == NS) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // leave no bulk copy in flight behind us: wait (bounded) for every armed stage
        for (int s = 0; s < NS; ++s) {
          if (!((armed >> s) & 1u)) continue;
          const uint64_t t0 = ptx::global_timer_ns();
          while (!ptx::mbar_try_wait(&sh->full[s], (armed_parity >> s) & 1u) &&
                 ptx::global_timer_ns() - t0 < 20000000ull) {}
        }
        if (PAIR && !leader) {
          // this CTA's copies are counted on the leader's barriers; they take microseconds
          const uint64_t t0 = ptx::global_timer_ns();
          while (ptx::global_timer_ns() - t0 < 1000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer ==================================
    if (lane == 0 && leader) {
      // D f32 (1) / s32 (2); operand formats: e4m3 = 0, signed int8 = 1, bf16 = 1
      constexpr uint32_t idesc = KIND == kFp8 ? ptx::umma_idesc(1, 0, 0, BMT, BN)
                                 : (KIND == kI8 ? ptx::umma_idesc(2, 1, 1, BMT, BN)
                                 : (KIND == kBf16 ? ptx::umma_idesc(1, 1, 1, BMT, BN) : ptx::umma_idesc(1, 0, 0, BMT, BN)));
      // one arrive per CTA of the pair, on the barrier at the same offset
      auto commit = [&](uint64_t* bar) {
        if constexpr (PAIR) {
          const uint32_t a = ptx::smem_u32(bar);
          ptx::umma_commit_pair(ptx::map_to_cta(a, 0));
          ptx::umma_commit_pair(ptx::map_to_cta(a, 1));
        } else {
          ptx::umma_commit(bar);
        }
      };
      int stage = 0; uint32_t phase = 0;
      int as = 0; uint32_t aphase = 0;
      bool ok = true;
      for (int t = worker; ok && t < total_tiles; t += nworkers) {
        const int ks = (t % (num_n_tiles * p.ksplits)) % p.ksplits;
        const int kb0 = ks * KBs, kb1 = min(KB, kb0 + KBs);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(&sh->full[stage], phase, abort_flag)) { ok = false; break; }
          if (kPromote || kb == kb0)
            if (!ptx::mbar_wait(&sh->tmem_empty[as], aphase ^ 1u, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t sa = ptx::smem_u32(smem + size_t(stage) * SB);
          const uint64_t adesc = ptx::umma_desc_sw128(sa);
          const uint64_t bdesc = ptx::umma_desc_sw128(sa + kABytes);
          const uint32_t d = tmem_base + static_cast<uint32_t>(as) * BN;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)   // +32 bytes along K = +2 in the >>4 address field
            umma_kind<KIND, CG>(d, adesc + 2 * k, bdesc + 2 * k, idesc, (k > 0 || (!kPromote && kb > kb0)) ? 1u : 0u);
          commit(&sh->empty[stage]);                // smem slot reusable once the MMAs retire
          if (++stage == NS) { stage = 0; phase ^= 1u; }
          if (kPromote || kb == kb1 - 1) {
            commit(&sh->tmem_full[as]);             // K-block product (kBf16: whole tile) ready
            if (++as == kAccStages) { as = 0; aphase ^= 1u; }
          }
        }
      }
    }
  }
  } else {
    // ========================= promotion + epilogue warps ==========================
    ptx::setmaxnreg_inc<224>();
    const int e = warp - kFirstEpiWarp;
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int hsel = e >> 2;             // which 64-column half of each 128-column block
    const int r_in_tile = q * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    int as = 0; uint32_t aphase = 0;
    int it = 0;
    bool ok = true;
    // Per-tile scale pointers and the first K block's scales; fetched one tile ahead so that the
    // global-load latency hides behind the previous tile's epilogue.
    struct ScaleCursor { const float* as_ptr; const float* bs0_ptr; const float* bs1_ptr; float sa, b0, b1; };
    auto open_tile = [&](const Tile& tl) {
      ScaleCursor c = {nullptr, nullptr, nullptr, 1.f, 1.f, 1.f};
      if constexpr (kPromote) {
        const int64_t row_ld = min(static_cast<int64_t>(tl.m0 + r_in_tile), p.M_total - 1);
        const int nb0 = p.swiglu ? tl.nt : min(tl.nt * 2, NB - 1);
        const int nb1 = p.swiglu ? NB / 2 + tl.nt : min(tl.nt * 2 + 1, NB - 1);
        c.as_ptr = p.a_s + row_ld * p.a_s_stride;
        c.bs0_ptr = p.b_s + (static_cast<int64_t>(tl.expert) * NB + nb0) * KB;
        c.bs1_ptr = p.b_s + (static_cast<int64_t>(tl.expert) * NB + nb1) * KB;
        const int kb0 = tl.ks * KBs;               // first K block of this tile's K split
        c.sa = __ldg(c.as_ptr + kb0); c.b0 = __ldg(c.bs0_ptr + kb0); c.b1 = __ldg(c.bs1_ptr + kb0);
      }
      return c;
    };
    Tile tl_next = {};
    ScaleCursor cur_next = {};
    if (worker < total_tiles) {
      tl_next = decode_tile(sh, p, worker, num_n_tiles, BMT, m_off);
      cur_next = open_tile(tl_next);
    }
    for (int t = worker; ok && t < total_tiles; t += nworkers, ++it) {
      const Tile tl = tl_next;
      const int row = tl.m0 + r_in_tile;
      const float* as_ptr = cur_next.as_ptr;
      const float* bs0_ptr = cur_next.bs0_ptr;
      const float* bs1_ptr = cur_next.bs1_ptr;
      float sa_n = cur_next.sa, b0_n = cur_next.b0, b1_n = cur_next.b1;
      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;
      // TMEM read-backs of this tile: promoted kinds one per K block of the tile's K split, the others one
      const int kb0p = kPromote ? tl.ks * KBs : 0;
      const int kb1p = kPromote ? min(KB, kb0p + KBs) : 1;
      // Per K block: two batches of two 32-column loads.  The second batch is in flight during the
      // FMAs of the first; the first batch of the NEXT K block is issued before the last 64 FMAs of
      // this one whenever its product is already there, so those FMAs hide its latency too.
      uint32_t ra[32], rb[32];
      bool issued = false;                            // first batch of this K block already in flight
      for (int kb = kb0p; kb < kb1p; ++kb) {
        const float s0 = sa_n * b0_n, s1 = sa_n * b1_n;
        if (kPromote && kb + 1 < kb1p) { sa_n = __ldg(as_ptr + kb + 1); b0_n = __ldg(bs0_ptr + kb + 1); b1_n = __ldg(bs1_ptr + kb + 1); }
        const uint32_t tcol = tmem_base + lane_base + static_cast<uint32_t>(as) * BN + static_cast<uint32_t>(hsel) * 64;
        if (!issued) {
          // warp-uniform outcome: the TMEM loads below need the whole warp converged
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(&sh->tmem_full[as], aphase, abort_flag))) { ok = false; break; }
          ptx::tc_fence_after_sync();
          ptx::tmem_ld32(tcol, ra);
          ptx::tmem_ld32(tcol + 32, rb);
        }
        ptx::tmem_ld_wait32(ra); ptx::tmem_ld_wait32(rb);
        promote32<KIND>(acc, ra, s0);
        ptx::tmem_ld32(tcol + 128, ra);
        promote32<KIND>(acc + 32, rb, s0);
        ptx::tmem_ld32(tcol + 160, rb);
        ptx::tmem_ld_wait32(ra); ptx::tmem_ld_wait32(rb);
        // the stage goes back to the MMA warp as soon as its last load has landed
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (PAIR && !leader) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&sh->tmem_empty[as]), 0));
          else ptx::mbar_arrive(&sh->tmem_empty[as]);
        }
        if (++as == kAccStages) { as = 0; aphase ^= 1u; }
        issued = false;
        if (kb + 1 < kb1p && __all_sync(0xffffffffu, ptx::mbar_try_wait(&sh->tmem_full[as], aphase))) {
          const uint32_t ncol = tmem_base + lane_base + static_cast<uint32_t>(as) * BN + static_cast<uint32_t>(hsel) * 64;
          ptx::tc_fence_after_sync();
          promote32<KIND>(acc + 64, ra, s1);
          ptx::tmem_ld32(ncol, ra);
          promote32<KIND>(acc + 96, rb, s1);
          ptx::tmem_ld32(ncol + 32, rb);
          issued = true;
        } else {
          promote32<KIND>(acc + 64, ra, s1);
          promote32<KIND>(acc + 96, rb, s1);
        }
      }
      if (!ok) break;
      if (t + nworkers < total_tiles) {
        tl_next = decode_tile(sh, p, t + nworkers, num_n_tiles, BMT, m_off);
        cur_next = open_tile(tl_next);
      }
      const bool row_ok = row < tl.m_end;
      if (!p.swiglu) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int col0 = tl.nt * BN + half * 128 + hsel * 64;
          if (col0 >= p.N) continue;                       // warp-uniform
          if (p.c_dtype == B200MOE_F32) {
            if (row_ok) {
              const int64_t orow = p.c_row_map ? p.c_row_map[row] : row;
              uint8_t* dst = p.c_row_addr ? reinterpret_cast<uint8_t*>(p.c_row_addr[row])
                                          : static_cast<uint8_t*>(p.c) + tl.ks * p.split_stride + orow * p.c_stride;
              store_row64(reinterpret_cast<float*>(dst) + col0, acc + half * 64);
            }
            continue;
          }
          // 16-bit outputs: a thread owns 128 contiguous bytes of ITS row, so a direct store touches
          // 32 cache lines per instruction.  Transpose through shared memory (16 rows at a time,
          // 16-byte chunks XOR-swizzled by the row) so that 8 lanes write one full 128-byte row.
          uint4 v[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float lo = acc[half * 64 + c * 8 + 2 * i], hi = acc[half * 64 + c * 8 + 2 * i + 1];
              if (p.c_dtype == B200MOE_BF16) { __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi); w[i] = *reinterpret_cast<uint32_t*>(&t); }
              else { __half2 t = __floats2half2_rn(lo, hi); w[i] = *reinterpret_cast<uint32_t*>(&t); }
            }
            v[c] = make_uint4(w[0], w[1], w[2], w[3]);
          }
          uint8_t* stg = sh->out_stage[e];
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            if ((lane >> 4) == part) {
              const int r = lane & 15;
#pragma unroll
              for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(stg + r * 128 + ((c ^ (r & 7)) << 4)) = v[c];
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int r = (lane >> 3) + 4 * i;               // row inside this 16-row part
              const int cc = lane & 7;
              uint4 val = *reinterpret_cast<const uint4*>(stg + r * 128 + ((cc ^ (r & 7)) << 4));
              const int orow_in = tl.m0 + q * 32 + part * 16 + r;
              if (orow_in < tl.m_end) {
                const int64_t orow = p.c_row_map ? p.c_row_map[orow_in] : orow_in;
                uint8_t* dst = p.c_row_addr ? reinterpret_cast<uint8_t*>(p.c_row_addr[orow_in])
                                            : static_cast<uint8_t*>(p.c) + tl.ks * p.split_stride + orow * p.c_stride;
                uint4* out = reinterpret_cast<uint4*>(dst + static_cast<int64_t>(col0) * 2 + cc * 16);
                if (p.accumulate) {
                  const uint4 old = *out;
                  const uint32_t* o = &old.x;
                  uint32_t* n = &val.x;
#pragma unroll
                  for (int i2 = 0; i2 < 4; ++i2) {
                    if (p.c_dtype == B200MOE_BF16) {
                      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o[i2]));
                      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&n[i2]));
                      const __nv_bfloat162 t2 = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
                      n[i2] = *reinterpret_cast<const uint32_t*>(&t2);
                    } else {
                      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&o[i2]));
                      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&n[i2]));
                      const __half2 t2 = __floats2half2_rn(a.x + b.x, a.y + b.y);
                      n[i2] = *reinterpret_cast<const uint32_t*>(&t2);
                    }
                  }
                }
                *out = val;
              }
            }
            __syncwarp();
          }
        }
      } else if (p.swiglu == 2) {
        // SwiGLU with the reference's roundings, written as bf16 (no re-quantization)
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float g = bf16r(acc[j]);
          const float u = bf16r(acc[64 + j]);
          const float a = bf16r(gate_act(g, p.act));
          acc[j] = a * u;
        }
        if (row_ok) {
          uint8_t* dst = static_cast<uint8_t*>(p.c) + static_cast<int64_t>(row) * p.c_stride;
          store_row64(reinterpret_cast<__nv_bfloat16*>(dst) + tl.nt * 128 + hsel * 64, acc);
        }
      } else {
        // SwiGLU with the reference's roundings (gate/up GEMM output, silu and the
        // product each rounded to bf16), then 1x128 e4m3 quantization of the row block.
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float g = bf16r(acc[j]);
          const float u = bf16r(acc[64 + j]);
          const float a = bf16r(gate_act(g, p.act));
          const float h = bf16r(a * u);
          acc[j] = h;
          amax = fmaxf(amax, fabsf(h));
        }
        const int buf = it & 1;
        sh->amax[buf][hsel][r_in_tile] = amax;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sh->amax_bar[buf]);
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&sh->amax_bar[buf], (it >> 1) & 1u, abort_flag))) { ok = false; break; }
        amax = fmaxf(amax, sh->amax[buf][hsel ^ 1][r_in_tile]);
        if (row_ok) {
          const float scale = __fdiv_rn(amax, 448.f);
          // h / scale as h * (1/scale) plus one residual correction: equal to the correctly rounded
          // quotient except in rare last-bit cases, which the e4m3 rounding (3 mantissa bits) absorbs.
          const float inv = __frcp_rn(scale);
          uint8_t* dst = static_cast<uint8_t*>(p.c) + static_cast<int64_t>(row) * p.c_stride + tl.nt * 128 + hsel * 64;
#pragma unroll
          for (int j = 0; j < 64; j += 16) {
            float q0[8], q1[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float a0 = acc[j + i], a1 = acc[j + 8 + i];
              const float y0 = a0 * inv, y1 = a1 * inv;
              q0[i] = fmaf(fmaf(-y0, scale, a0), inv, y0);
              q1[i] = fmaf(fmaf(-y1, scale, a1), inv, y1);
            }
            const uint2 lo = pack8_e4m3(q0), hi = pack8_e4m3(q1);
            *reinterpret_cast<uint4*>(dst + j) = make_uint4(lo.x, lo.y, hi.x, hi.y);
          }
          if (hsel == 0) p.c_s[static_cast<int64_t>(row) * p.c_s_stride + tl.nt] = scale;
        }
      }
    }
  }

  // ---- teardown ----------------------------------------------------------------------
  if (p.c_row_addr) __threadfence_system();
  ptx::tc_fence_before_sync();
  __syncthreads();
  if constexpr (PAIR) ptx::cluster_sync();   // both CTAs are done with each other's memory and barriers
  if (warp == 1) ptx::tmem_dealloc<CG>(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && sh->abort_flag && p.status) *p.status = B200MOE_DEVICE_TIMEOUT;
}

// ---- host side ---------------------------------------------------------------------------
template <int KIND, bool PAIR>
static int launch_gemm_as(const RowMaps& ma, const CUtensorMap& mb, const GemmParams& p, int grid, cudaStream_t st) {
  cudaFuncSetAttribute(gemm_block_kernel<KIND, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       static_cast<int>(kSmemBytes));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_block_kernel<KIND, PAIR>, ma, mb, p);
  if (e != cudaSuccess) return fail(B200MOE_LAUNCH_FAILED, "gemm_block_kernel launch: %s", cudaGetErrorString(e));
  return check_launch("gemm_block_kernel");
}

// opts (may be null): per-call launch options of the grouped GEMMs (b200moe_gemm_opts).
template <int KIND>
static int launch_gemm(const void* a, int64_t a_stride, const void* b, GemmParams p, int64_t tiles_hint,
                       cudaStream_t st, const b200moe_gemm_opts* opts = nullptr) {
  const int max_ctas = opts ? opts->max_ctas : 0;
  const int pair_mode = opts ? opts->pair_mode : 0;
  B200MOE_REQUIRE(max_ctas >= 0 && (pair_mode == 0 || pair_mode == 1), B200MOE_BAD_ARG,
                  "gemm options: max_ctas %d, pair_mode %d", max_ctas, pair_mode);
  int sms = 0;
  if (int rc = require_sm100(&sms)) return rc;
  RowMaps ma;
  CUtensorMap mb;
  for (int i = 0; i < 4; ++i)
    if (int rc = cached_tensor_map_u8(&ma.m[i], a, static_cast<uint64_t>(p.M_total),
                                    static_cast<uint64_t>(p.a_wrap ? p.a_wrap : p.K),
                                    static_cast<uint64_t>(a_stride), 16u << i)) return rc;
  if (int rc = cached_tensor_map_u8(&mb, b, static_cast<uint64_t>(p.num_weights) * p.N, static_cast<uint64_t>(p.K),
                                  static_cast<uint64_t>(p.K), 128)) return rc;
  int grid = sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles_hint > 0 && tiles_hint < grid) grid = static_cast<int>(tiles_hint);
  // N must cover both halves of a pair's tile; split-K launches stay single.
  bool pair = pair_mode == 1;
  if (p.ksplits > 1 || grid < 2 || (!p.swiglu && p.N % BN != 0)) pair = false;
  if (pair) return launch_gemm_as<KIND, true>(ma, mb, p, grid & ~1, st);
  return launch_gemm_as<KIND, false>(ma, mb, p, grid, st);
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_gemm_fp8_block(const void* a, const float* a_s, const void* b,
                                      const float* b_s, void* c, int c_dtype, int64_t M,
                                      int64_t N, int64_t K, void* stream) {
  B200MOE_REQUIRE(a && a_s && b && b_s && c, B200MOE_BAD_ARG, "gemm_fp8_block: null pointer");
  B200MOE_REQUIRE(M >= 0 && M < (int64_t(1) << 31) && N > 0 && K > 0 && K % 128 == 0 && N % 128 == 0 && N * K < (int64_t(1) << 40),
                  B200MOE_BAD_SHAPE, "gemm_fp8_block: M=%lld N=%lld K=%lld (N and K must be multiples of 128)",
                  (long long)M, (long long)N, (long long)K);
  B200MOE_REQUIRE(c_dtype == B200MOE_F32 || c_dtype == B200MOE_F16 || c_dtype == B200MOE_BF16, B200MOE_BAD_DTYPE,
                  "gemm_fp8_block: c dtype %d", c_dtype);
  B200MOE_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(c, 16), B200MOE_BAD_ALIGN,
                  "gemm_fp8_block: Input tensors must be 16-byte aligned");
  if (M == 0) return B200MOE_OK;
  const int esz = c_dtype == B200MOE_F32 ? 4 : 2;
  GemmParams p{a_s, K / 128, b_s, c, N * esz, nullptr, 0, nullptr, nullptr, M,
               static_cast<int>(N), static_cast<int>(K), 1, 1, c_dtype, 0, nullptr, 1, 0, 0, nullptr, nullptr, 0, 0};
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  return launch_gemm<kFp8>(a, K, b, p, tiles, as_stream(stream));
}

namespace b200moe {
// out[i] = T(partials[0][i] + partials[1][i] + ...) in split order (deterministic), 4 values per thread
template <typename T>
__global__ void __launch_bounds__(256) sum_splits_kernel(const float* __restrict__ partials, int ksplits,
                                                         int64_t n, T* __restrict__ out) {
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x * 4) {
    float4 acc = *reinterpret_cast<const float4*>(partials + i);
    for (int s = 1; s < ksplits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partials + s * n + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(out + i) = acc;
    } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(out + i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else {
      __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(out + i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}
}  // namespace b200moe

extern "C" int b200moe_gemm_fp8_block_splitk(const void* a, const float* a_s, const void* b, const float* b_s,
                                             void* c, int c_dtype, int64_t M, int64_t N, int64_t K, int ksplits,
                                             float* partials, int64_t partials_bytes, void* stream) {
  B200MOE_REQUIRE(a && a_s && b && b_s && c && partials, B200MOE_BAD_ARG, "gemm_fp8_block_splitk: null pointer");
  B200MOE_REQUIRE(M >= 0 && M < (int64_t(1) << 31) && N > 0 && K > 0 && K % 128 == 0 && N % 128 == 0 && N * K < (int64_t(1) << 40),
                  B200MOE_BAD_SHAPE, "gemm_fp8_block_splitk: M=%lld N=%lld K=%lld (N and K must be multiples of 128)",
                  (long long)M, (long long)N, (long long)K);
  const int64_t KB = K / 128;
  const int64_t per = ksplits > 0 ? (KB + ksplits - 1) / ksplits : 0;
  B200MOE_REQUIRE(ksplits >= 1 && ksplits <= 16 && per * (ksplits - 1) < KB, B200MOE_BAD_ARG,
                  "gemm_fp8_block_splitk: %d splits of %lld K blocks (every split needs at least one)", ksplits, (long long)KB);
  B200MOE_REQUIRE(c_dtype == B200MOE_F32 || c_dtype == B200MOE_F16 || c_dtype == B200MOE_BF16, B200MOE_BAD_DTYPE,
                  "gemm_fp8_block_splitk: c dtype %d", c_dtype);
  B200MOE_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(c, 16) && aligned(partials, 16), B200MOE_BAD_ALIGN,
                  "gemm_fp8_block_splitk: Input tensors must be 16-byte aligned");
  B200MOE_REQUIRE(partials_bytes >= static_cast<int64_t>(ksplits) * M * N * 4, B200MOE_WORKSPACE_TOO_SMALL,
                  "gemm_fp8_block_splitk: partials need %lld bytes", (long long)(static_cast<int64_t>(ksplits) * M * N * 4));
  if (M == 0) return B200MOE_OK;
  GemmParams p{a_s, K / 128, b_s, partials, N * 4, nullptr, 0, nullptr, nullptr, M,
               static_cast<int>(N), static_cast<int>(K), 1, 1, B200MOE_F32, 0, nullptr, ksplits, M * N * 4, 0,
               nullptr, nullptr, 0, 0};
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * ksplits;
  if (int rc = launch_gemm<kFp8>(a, K, b, p, tiles, as_stream(stream))) return rc;
  const int64_t n = M * N;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((n / 4 + 255) / 256, 148 * 8));
  cudaStream_t st = as_stream(stream);
  if (c_dtype == B200MOE_F32) sum_splits_kernel<float><<<grid, 256, 0, st>>>(partials, ksplits, n, static_cast<float*>(c));
  else if (c_dtype == B200MOE_BF16) sum_splits_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(partials, ksplits, n, static_cast<__nv_bfloat16*>(c));
  else sum_splits_kernel<__half><<<grid, 256, 0, st>>>(partials, ksplits, n, static_cast<__half*>(c));
  return check_launch("sum_splits");
}

extern "C" int b200moe_grouped_gemm_fp8(const void* a, int64_t a_row_stride_bytes, const float* a_s,
                                        int64_t a_s_row_stride, const void* b, const float* b_s,
                                        void* c, int c_dtype, int64_t c_row_stride_bytes, float* c_s,
                                        int64_t c_s_row_stride, int64_t M_total, int64_t N, int64_t K,
                                        int num_groups, int num_weights, const int64_t* seg_indptr,
                                        const int64_t* weight_indices, int epilogue,
                                        const int32_t* c_row_map, const int64_t* c_row_addr,
                                        int32_t* status_word, const b200moe_gemm_opts* opts, void* stream) {
  B200MOE_REQUIRE(a && a_s && b && b_s && c && seg_indptr, B200MOE_BAD_ARG, "grouped_gemm_fp8: null pointer");
  B200MOE_REQUIRE((c_row_map == nullptr && c_row_addr == nullptr) || epilogue == 0, B200MOE_BAD_ARG,
                  "grouped_gemm_fp8: c_row_map / c_row_addr need epilogue 0");
  B200MOE_REQUIRE(c_row_map == nullptr || c_row_addr == nullptr, B200MOE_BAD_ARG,
                  "grouped_gemm_fp8: c_row_map and c_row_addr are exclusive");
  B200MOE_REQUIRE(epilogue == 0 || epilogue == 1 || epilogue == 4, B200MOE_BAD_ARG, "grouped_gemm_fp8: epilogue %d", epilogue);
  B200MOE_REQUIRE(M_total >= 0 && M_total < (int64_t(1) << 31) && N > 0 && K > 0 && K % 128 == 0 && N % 128 == 0,
                  B200MOE_BAD_SHAPE, "grouped_gemm_fp8: M=%lld N=%lld K=%lld (N and K must be multiples of 128)",
                  (long long)M_total, (long long)N, (long long)K);
  B200MOE_REQUIRE(num_groups >= 1 && num_groups <= kMaxGroups && num_weights >= 1 &&
                  static_cast<int64_t>(num_weights) * N < (int64_t(1) << 31),
                  B200MOE_BAD_SHAPE, "grouped_gemm_fp8: num_groups=%d (max %d) num_weights=%d", num_groups, kMaxGroups, num_weights);
  B200MOE_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(c, 16) && a_row_stride_bytes % 16 == 0 &&
                  a_row_stride_bytes >= K && c_row_stride_bytes % 16 == 0,
                  B200MOE_BAD_ALIGN, "grouped_gemm_fp8: pointers and row strides must be 16-byte aligned");
  B200MOE_REQUIRE(a_s_row_stride >= K / 128, B200MOE_BAD_ARG, "grouped_gemm_fp8: a_s row stride too small");
  if (epilogue != 0) {
    B200MOE_REQUIRE(N % 256 == 0, B200MOE_BAD_SHAPE, "grouped_gemm_fp8: the SwiGLU epilogue needs N %% 256 == 0, got %lld", (long long)N);
    B200MOE_REQUIRE(c_dtype == B200MOE_FP8_E4M3 && c_s && c_row_stride_bytes >= N / 2 && c_s_row_stride >= N / 256,
                    B200MOE_BAD_ARG, "grouped_gemm_fp8: the SwiGLU epilogue writes e4m3 rows and f32 scales");
  } else {
    B200MOE_REQUIRE(c_dtype == B200MOE_F32 || c_dtype == B200MOE_F16 || c_dtype == B200MOE_BF16, B200MOE_BAD_DTYPE,
                    "grouped_gemm_fp8: c dtype %d", c_dtype);
    B200MOE_REQUIRE(c_row_stride_bytes >= N * (c_dtype == B200MOE_F32 ? 4 : 2), B200MOE_BAD_ARG, "grouped_gemm_fp8: c row stride too small");
  }
  if (M_total == 0) return B200MOE_OK;
  GemmParams p{a_s, a_s_row_stride, b_s, c, c_row_stride_bytes, c_s, c_s_row_stride, seg_indptr,
               weight_indices, M_total, static_cast<int>(N), static_cast<int>(K), num_groups,
               num_weights, c_dtype, epilogue == 4 ? 1 : epilogue, status_word, 1, 0, 0, c_row_map, c_row_addr, 0,
               epilogue == 4 ? 1 : 0};
  return launch_gemm<kFp8>(a, a_row_stride_bytes, b, p, 0, as_stream(stream), opts);
}

// ---- int8 x int8 (w4a8 after the int4 -> int8 step) and bf16 x bf16 (w4a16 after dequantization) ----
static int check_grouped_common(const char* who, const void* a, const void* b, const void* c,
                                const int64_t* seg, int64_t a_stride, int64_t kbytes, int64_t M_total,
                                int64_t N, int num_groups, int num_weights) {
  B200MOE_REQUIRE(a && b && c && seg, B200MOE_BAD_ARG, "%s: null pointer", who);
  B200MOE_REQUIRE(M_total >= 0 && M_total < (int64_t(1) << 31) && N > 0 && N % 128 == 0 && kbytes > 0 && kbytes % 128 == 0,
                  B200MOE_BAD_SHAPE, "%s: M=%lld N=%lld (N must be a multiple of 128, K of 128 bytes)", who,
                  (long long)M_total, (long long)N);
  B200MOE_REQUIRE(num_groups >= 1 && num_groups <= kMaxGroups && num_weights >= 1 &&
                  static_cast<int64_t>(num_weights) * N < (int64_t(1) << 31), B200MOE_BAD_SHAPE,
                  "%s: num_groups=%d (max %d) num_weights=%d", who, num_groups, kMaxGroups, num_weights);
  B200MOE_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(c, 16) && a_stride % 16 == 0 && a_stride >= kbytes,
                  B200MOE_BAD_ALIGN, "%s: pointers and row strides must be 16-byte aligned", who);
  return B200MOE_OK;
}

extern "C" int b200moe_grouped_gemm_i8(const void* a, int64_t a_row_stride_bytes, const float* a_s,
                                       int64_t a_s_row_stride, const void* b, const float* b_s, void* c,
                                       int c_dtype, int64_t c_row_stride_bytes, int64_t M_total, int64_t N,
                                       int64_t K, int num_groups, int num_weights,
                                       const int64_t* seg_indptr, const int64_t* weight_indices,
                                       int32_t* status_word, const b200moe_gemm_opts* opts, void* stream) {
  if (int rc = check_grouped_common("grouped_gemm_i8", a, b, c, seg_indptr, a_row_stride_bytes, K, M_total, N,
                                    num_groups, num_weights)) return rc;
  B200MOE_REQUIRE(a_s && b_s && a_s_row_stride >= K / 128, B200MOE_BAD_ARG, "grouped_gemm_i8: scales");
  B200MOE_REQUIRE(c_dtype == B200MOE_F32 || c_dtype == B200MOE_F16 || c_dtype == B200MOE_BF16, B200MOE_BAD_DTYPE,
                  "grouped_gemm_i8: c dtype %d", c_dtype);
  B200MOE_REQUIRE(c_row_stride_bytes % 16 == 0 && c_row_stride_bytes >= N * (c_dtype == B200MOE_F32 ? 4 : 2),
                  B200MOE_BAD_ARG, "grouped_gemm_i8: c row stride");
  if (M_total == 0) return B200MOE_OK;
  GemmParams p{a_s, a_s_row_stride, b_s, c, c_row_stride_bytes, nullptr, 0, seg_indptr, weight_indices, M_total,
               static_cast<int>(N), static_cast<int>(K), num_groups, num_weights, c_dtype, 0, status_word, 1, 0, 0, nullptr, nullptr, 0, 0};
  return launch_gemm<kI8>(a, a_row_stride_bytes, b, p, 0, as_stream(stream), opts);
}

static int grouped_gemm_16bit(bool f16, const void* a, int64_t a_row_stride_bytes, const void* b, void* c,
                              int c_dtype, int64_t c_row_stride_bytes, int64_t M_total, int64_t N,
                              int64_t K, int num_groups, int num_weights,
                              const int64_t* seg_indptr, const int64_t* weight_indices,
                              int epilogue, int32_t* status_word, const b200moe_gemm_opts* opts, void* stream) {
  if (int rc = check_grouped_common("grouped_gemm_bf16", a, b, c, seg_indptr, a_row_stride_bytes, 2 * K, M_total, N,
                                    num_groups, num_weights)) return rc;
  B200MOE_REQUIRE(epilogue == 0 || epilogue == 3 || ((epilogue == 2 || epilogue == 5) && !f16), B200MOE_BAD_ARG,
                  "grouped_gemm_bf16: epilogue %d (0 plain, 2 SiLU*up / 5 GELU*up with bf16 operands, 3 plain added to c)", epilogue);
  B200MOE_REQUIRE(epilogue != 3 || c_dtype == B200MOE_BF16 || c_dtype == B200MOE_F16, B200MOE_BAD_DTYPE,
                  "grouped_gemm_bf16: epilogue 3 adds into a 16-bit c");
  if (epilogue == 2 || epilogue == 5) {
    B200MOE_REQUIRE(N % 256 == 0 && c_dtype == B200MOE_BF16 && c_row_stride_bytes >= N, B200MOE_BAD_ARG,
                    "grouped_gemm_bf16: the SwiGLU epilogue needs N %% 256 == 0 and a bf16 [M, N/2] output");
  } else {
    B200MOE_REQUIRE(c_dtype == B200MOE_F32 || c_dtype == B200MOE_F16 || c_dtype == B200MOE_BF16, B200MOE_BAD_DTYPE,
                    "grouped_gemm_bf16: c dtype %d", c_dtype);
    B200MOE_REQUIRE(c_row_stride_bytes >= N * (c_dtype == B200MOE_F32 ? 4 : 2), B200MOE_BAD_ARG, "grouped_gemm_bf16: c row stride");
  }
  B200MOE_REQUIRE(c_row_stride_bytes % 16 == 0, B200MOE_BAD_ALIGN, "grouped_gemm_bf16: c row stride alignment");
  if (M_total == 0) return B200MOE_OK;
  GemmParams p{nullptr, 0, nullptr, c, c_row_stride_bytes, nullptr, 0, seg_indptr, weight_indices, M_total,
               static_cast<int>(N), static_cast<int>(2 * K), num_groups, num_weights, c_dtype,
               epilogue == 3 ? 0 : (epilogue == 5 ? 2 : epilogue), status_word, 1, 0, 0, nullptr, nullptr,
               epilogue == 3 ? 1 : 0, epilogue == 5 ? 1 : 0};
  return f16 ? launch_gemm<kF16>(a, a_row_stride_bytes, b, p, 0, as_stream(stream), opts)
             : launch_gemm<kBf16>(a, a_row_stride_bytes, b, p, 0, as_stream(stream), opts);
}

extern "C" int b200moe_grouped_gemm_bf16(const void* a, int64_t a_row_stride_bytes, const void* b, void* c,
                                         int c_dtype, int64_t c_row_stride_bytes, int64_t M_total, int64_t N,
                                         int64_t K, int num_groups, int num_weights,
                                         const int64_t* seg_indptr, const int64_t* weight_indices,
                                         int epilogue, int32_t* status_word, const b200moe_gemm_opts* opts,
                                         void* stream) {
  return grouped_gemm_16bit(false, a, a_row_stride_bytes, b, c, c_dtype, c_row_stride_bytes, M_total, N, K,
                            num_groups, num_weights, seg_indptr, weight_indices, epilogue, status_word, opts, stream);
}

extern "C" int b200moe_grouped_gemm_f16(const void* a, int64_t a_row_stride_bytes, const void* b, void* c,
                                        int c_dtype, int64_t c_row_stride_bytes, int64_t M_total, int64_t N,
                                        int64_t K, int num_groups, int num_weights,
                                        const int64_t* seg_indptr, const int64_t* weight_indices,
                                        int32_t* status_word, const b200moe_gemm_opts* opts, void* stream) {
  return grouped_gemm_16bit(true, a, a_row_stride_bytes, b, c, c_dtype, c_row_stride_bytes, M_total, N, K,
                            num_groups, num_weights, seg_indptr, weight_indices, 0, status_word, opts, stream);
}

// ---- router logits on the tensor cores ------------------------------------------------------
// logits = x . W^T in f32-equivalent precision from bf16 MMAs: x is bf16 already, W (f32) is
// split offline into three bf16 parts hi + mid + lo (24 mantissa bits), stored side by side as
// w3 [E, 3H].  The products x*part are exact in f32, the three partial dot products accumulate
// in the same TMEM accumulator.  The K loop (3H) is split over `ksplits` CTAs per tile whose
// partial sums land in partials[ks] and are added in index order by b200moe_router_select.
extern "C" int b200moe_router_logits_bf16x3(const void* x_bf16, const void* w3_bf16, float* partials,
                                            int64_t T, int64_t H, int E, int ksplits, void* stream) {
  B200MOE_REQUIRE(x_bf16 && w3_bf16 && partials, B200MOE_BAD_ARG, "router_logits_bf16x3: null pointer");
  B200MOE_REQUIRE(T >= 0 && T < (int64_t(1) << 31) && H > 0 && H % 64 == 0 && E >= 1 && E % 128 == 0 && E <= 1024,
                  B200MOE_BAD_SHAPE, "router_logits_bf16x3: H=%lld must be a multiple of 64 and E=%d of 128", (long long)H, E);
  const int64_t KB = 3 * H * 2 / 128;
  B200MOE_REQUIRE(ksplits >= 1 && ksplits <= 16 && (KB + ksplits - 1) / ksplits * (ksplits - 1) < KB, B200MOE_BAD_ARG,
                  "router_logits_bf16x3: ksplits=%d leaves an empty split for %lld K blocks", ksplits, (long long)KB);
  B200MOE_REQUIRE(aligned(x_bf16, 16) && aligned(w3_bf16, 16) && aligned(partials, 16), B200MOE_BAD_ALIGN,
                  "router_logits_bf16x3: alignment");
  if (T == 0) return B200MOE_OK;
  GemmParams p{nullptr, 0, nullptr, partials, static_cast<int64_t>(E) * 4, nullptr, 0, nullptr, nullptr, T, E,
               static_cast<int>(3 * H * 2), 1, 1, B200MOE_F32, 0, nullptr, ksplits, T * static_cast<int64_t>(E) * 4,
               static_cast<int>(H * 2), nullptr, nullptr, 0, 0};
  const int64_t tiles = ((T + BM - 1) / BM) * ((E + BN - 1) / BN) * ksplits;
  return launch_gemm<kBf16>(x_bf16, H * 2, w3_bf16, p, tiles, as_stream(stream));
}
