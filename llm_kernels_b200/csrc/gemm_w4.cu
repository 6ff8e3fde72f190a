// Grouped w4a8 GEMM with the int4 -> int8 step fused into the operand path (no expanded copy of the weights).
//
//   reference: w4a8_gemm_kernel (quantization/w4a8_kernel.py:317-404) unpacks the nibbles, applies
//   (q - z4) * s4 and feeds the int8 dot product inside its K loop (:362-380); per K block
//   acc += float(dot in s32) * a_s[m,kb] * b_s[n/128,kb].  The grouped form follows grouped_gemm_triton
//   (moe/group_gemm_kernel.py:291-513).
//
// One persistent CTA per SM, 512 threads:
//   warp 0       TMA producer of the PACKED weights: per K block two boxes of 16 packed rows x 128 k (int32 words,
//                8 output channels per word, quantization/bitpack.py:9-36), 16 KB, 5-slot ring
//   warp 2       TMA producer of the int8 activation tile (box of 16/32/64/128 rows x 128 B), 3-slot ring
//   warps 12-15  converters: read a packed slot, split every word into its 8 nibbles with byte permutes,
//                w8 = int8((q - z4) * s4) four values at a time, and write the 256 x 128 B int8 operand tile in the
//                128-byte-swizzled layout the tensor core reads (2 slots); fence.proxy.async, arrive
//   warp 1       owns TMEM (2 stages x 256 s32 columns), 4 x tcgen05.mma.kind::i8 (M128 N256 K32) per K block
//   warps 4-11   per-K-block promotion (s32 -> f32, times a_s * b_s) and the tile epilogue; warps whose 32 rows
//                lie beyond the group's rows only keep the hand-over going
// HBM moves the packed weights once (0.5 byte per weight) plus the tiny scale tables; that is the roofline of the
// decode regime this kernel is for.  Each weight tile is converted once per (m-tile, n-tile), so the kernel is the
// right choice while groups have about one m-tile (callers with many rows per expert expand once instead).
//
// Every wait is a bounded mbarrier wait; on expiry the kernel drains its copies, frees TMEM, writes
// B200MOE_DEVICE_TIMEOUT to the status word and returns.
#include <cuda.h>

#include "common.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace b200moe {
namespace w4 {

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int kAStages = 3, kPStages = 5, kBStages = 2, kAccStages = 2;
constexpr uint32_t kABytes = BM * BK, kBBytes = BN * BK, kPBytes = 32 * BK * 4;   // 16 KB, 32 KB, 16 KB
constexpr int kThreads = 512;
constexpr int kFirstEpiWarp = 4, kEpiWarps = 8, kFirstConvWarp = 12, kConvWarps = 4;
constexpr int kMaxGroups = 1024;
constexpr uint32_t kTmemCols = 512;

struct Tail {
  uint64_t a_full[kAStages], a_empty[kAStages];
  uint64_t p_full[kPStages], p_empty[kPStages];
  uint64_t b_full[kBStages], b_empty[kBStages];
  uint64_t tmem_full[kAccStages], tmem_empty[kAccStages];
  uint32_t tmem_base;
  int abort_flag;
  uint64_t amax_bar[2][4];        // [buffer][lane quarter]: the two warps that share 32 rows exchange their amax
  float amax[2][2][BM];           // [buffer][column half][row]
  int32_t seg[kMaxGroups + 1];    // row offsets of the groups
  int32_t pref[kMaxGroups + 1];   // exclusive prefix of m-tiles per group
};
constexpr size_t kRingBytes = size_t(kAStages) * kABytes + size_t(kBStages) * kBBytes + size_t(kPStages) * kPBytes;
constexpr size_t kSmemBytes = 1024 + kRingBytes + sizeof(Tail);

struct Params {
  const float* a_s; int64_t a_s_stride;
  const float* b_s;               // [W, N/128, K/128]
  const uint8_t* sz_t;            // [W, K/128, N, 2]: (s4, z4) pairs, transposed so that a K block's pairs are contiguous
  void* c; int64_t c_stride;      // bytes
  float* c_s; int64_t c_s_stride; // floats
  const int64_t* seg; const int64_t* widx;
  int64_t M_total;
  int N, K, num_groups, c_dtype, fused;   // fused: 0 plain, 1 act(gate)*up + int8 re-quantization
  int act;                                 // 0 SiLU, 1 tanh-GELU
  int32_t* status;
};

struct Tile { int m0, m_end, expert, nt; };
struct RowMaps { CUtensorMap m[4]; };

__device__ __forceinline__ Tile decode_tile(const Tail* sh, const Params& p, int t, int num_n_tiles) {
  const int mt = t / num_n_tiles;
  int lo = 0, hi = p.num_groups;           // last g with pref[g] <= mt
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

// First weight row (of the [W*N, K] matrix) of the tile's two 128-row halves: gate rows and up rows of the same
// columns for the fused epilogue, two consecutive N blocks otherwise.
__device__ __forceinline__ void tile_rows(const Params& p, const Tile& tl, int& row0, int& row1) {
  row0 = tl.expert * p.N + (p.fused ? tl.nt * 128 : tl.nt * BN);
  row1 = p.fused ? tl.expert * p.N + p.N / 2 + tl.nt * 128 : row0 + 128;
}

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

// ---- int4 -> int8 in registers ---------------------------------------------------------------------------
// Four packed words (k .. k+3 of one packed row; nibble i of a word belongs to output channel 8r + i) -> eight
// registers, one per channel, each holding that channel's four values as bytes.  Even and odd nibbles are
// separated with two masks; a 4 x 4 byte transpose (eight byte permutes per half) gathers the channels.
__device__ __forceinline__ void unpack_quad(const uint4 w, uint32_t (&q)[8]) {
  const uint32_t src[2][4] = {{w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, w.z & 0x0F0F0F0Fu, w.w & 0x0F0F0F0Fu},
                              {(w.x >> 4) & 0x0F0F0F0Fu, (w.y >> 4) & 0x0F0F0F0Fu, (w.z >> 4) & 0x0F0F0F0Fu,
                               (w.w >> 4) & 0x0F0F0F0Fu}};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t t0 = __byte_perm(src[h][0], src[h][1], 0x5140), t1 = __byte_perm(src[h][2], src[h][3], 0x5140);
    const uint32_t t2 = __byte_perm(src[h][0], src[h][1], 0x7362), t3 = __byte_perm(src[h][2], src[h][3], 0x7362);
    q[h + 0] = __byte_perm(t0, t1, 0x5410);
    q[h + 2] = __byte_perm(t0, t1, 0x7632);
    q[h + 4] = __byte_perm(t2, t3, 0x5410);
    q[h + 6] = __byte_perm(t2, t3, 0x7632);
  }
}

// Four values at once: int8((q - z) * s) per byte with int8 wrap-around, as the reference's int8 product
// (quantization/w4a8_kernel.py:84-92).  For 0 <= s <= 17 the four products q * s (q <= 15) stay inside their bytes,
// so one 32-bit multiply and a carry-free byte-wise subtraction of (z * s) mod 256 do it; any other s (the
// reference's quantizer never produces one) goes byte by byte.
__device__ __forceinline__ uint32_t dequant4(uint32_t q, int s, int z) {
  if (s >= 0 && s <= 17) {
    const uint32_t H = 0x80808080u;
    const uint32_t p = q * static_cast<uint32_t>(s);
    const uint32_t zs = (static_cast<uint32_t>(z * s) & 0xFFu) * 0x01010101u;
    return ((p | H) - (zs & ~H)) ^ ((p ^ ~zs) & H);
  }
  uint32_t r = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    r |= (static_cast<uint32_t>((static_cast<int>((q >> (8 * j)) & 0xFu) - z) * s) & 0xFFu) << (8 * j);
  return r;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a8_kernel(const __grid_constant__ RowMaps tmap_a, const __grid_constant__ CUtensorMap tmap_p, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;                                        // kAStages x 16 KB, swizzled int8 rows
  uint8_t* smem_b = smem_a + size_t(kAStages) * kABytes;         // kBStages x 32 KB, swizzled int8 rows (converted)
  uint8_t* smem_p = smem_b + size_t(kBStages) * kBBytes;         // kPStages x 16 KB, [32 packed rows][128 words]
  Tail* sh = reinterpret_cast<Tail*>(smem_p + size_t(kPStages) * kPBytes);
  volatile int* abort_flag = &sh->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = p.K / BK;
  const int NB = p.N / 128;
  const int num_n_tiles = p.fused ? (p.N / 2) / 128 : (p.N + BN - 1) / BN;

  // ---- setup: barriers, TMEM, group table ---------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < kAStages; ++s) { ptx::mbar_init(&sh->a_full[s], 1); ptx::mbar_init(&sh->a_empty[s], 1); }
    for (int s = 0; s < kPStages; ++s) { ptx::mbar_init(&sh->p_full[s], 1); ptx::mbar_init(&sh->p_empty[s], kConvWarps); }
    for (int s = 0; s < kBStages; ++s) { ptx::mbar_init(&sh->b_full[s], kConvWarps); ptx::mbar_init(&sh->b_empty[s], 1); }
    for (int s = 0; s < kAccStages; ++s) { ptx::mbar_init(&sh->tmem_full[s], 1); ptx::mbar_init(&sh->tmem_empty[s], kEpiWarps); }
    for (int s = 0; s < 8; ++s) ptx::mbar_init(&sh->amax_bar[s >> 2][s & 3], 2);
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
  if (warp == 3) {  // exclusive prefix of m-tiles per group, 32 groups per step
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

  // Register hand-over: producers / MMA 48, converters 96, promotion + epilogue warps 184
  // (128 x 48 + 128 x 96 + 256 x 184 = 65536; released 128 x 80 + 128 x 32 = 14336 = taken 256 x 56).
  if (warp < kFirstEpiWarp) {
    ptx::setmaxnreg_dec<48>();
    if (warp == 0 && lane == 0) {
      // ============================ TMA producer: packed weights ============================
      int stage = 0; uint32_t phase = 0;
      Armed armed;
      bool ok = true;
      for (int t = first; ok && t < total_tiles; t += step) {
        const Tile tl = decode_tile(sh, p, t, num_n_tiles);
        int row0, row1;
        tile_rows(p, tl, row0, row1);
        for (int kb = 0; kb < KB; ++kb) {
          if (!ptx::mbar_wait(&sh->p_empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sp = smem_p + size_t(stage) * kPBytes;
          ptx::mbar_arrive_expect_tx(&sh->p_full[stage], kPBytes);
          armed.arm(stage, phase);
          ptx::tma_load_2d(sp, &tmap_p, &sh->p_full[stage], kb * BK, row0 / 8);
          ptx::tma_load_2d(sp + kPBytes / 2, &tmap_p, &sh->p_full[stage], kb * BK, row1 / 8);
          if (++stage == kPStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) armed.drain(sh->p_full, kPStages);
    } else if (warp == 2 && lane == 0) {
      // ============================ TMA producer: activation rows ===========================
      int stage = 0; uint32_t phase = 0;
      Armed armed;
      bool ok = true;
      auto box_sel = [](int rows) { return rows <= 16 ? 0 : (rows <= 32 ? 1 : (rows <= 64 ? 2 : 3)); };
      for (int t = first; ok && t < total_tiles; t += step) {
        const Tile tl = decode_tile(sh, p, t, num_n_tiles);
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
      // ================================== MMA issuer ========================================
      constexpr uint32_t idesc = ptx::umma_idesc(2, 1, 1, BM, BN);     // D s32, A and B signed int8
      int sa = 0, sb = 0, as = 0;
      uint32_t pa = 0, pb = 0, pacc = 0;
      bool ok = true;
      for (int t = first; ok && t < total_tiles; t += step) {
        for (int kb = 0; kb < KB; ++kb) {
          if (!ptx::mbar_wait(&sh->a_full[sa], pa, abort_flag) || !ptx::mbar_wait(&sh->b_full[sb], pb, abort_flag) ||
              !ptx::mbar_wait(&sh->tmem_empty[as], pacc ^ 1u, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint64_t adesc = ptx::umma_desc_sw128(ptx::smem_u32(smem_a + size_t(sa) * kABytes));
          const uint64_t bdesc = ptx::umma_desc_sw128(ptx::smem_u32(smem_b + size_t(sb) * kBBytes));
          const uint32_t d = tmem_base + static_cast<uint32_t>(as) * BN;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) ptx::umma_i8<1>(d, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
          ptx::umma_commit(&sh->a_empty[sa]);        // both operand slots are reusable once the MMAs retire
          ptx::umma_commit(&sh->b_empty[sb]);
          ptx::umma_commit(&sh->tmem_full[as]);      // this K block's s32 product is ready
          if (++sa == kAStages) { sa = 0; pa ^= 1u; }
          if (++sb == kBStages) { sb = 0; pb ^= 1u; }
          if (++as == kAccStages) { as = 0; pacc ^= 1u; }
        }
      }
    }
  } else if (warp >= kFirstConvWarp) {
    // ==================================== converters =========================================
    ptx::setmaxnreg_dec<96>();
    const int cw = warp - kFirstConvWarp;
    int sp = 0, sb = 0;
    uint32_t pp = 0, pb = 0;
    bool ok = true;
    for (int t = first; ok && t < total_tiles; t += step) {
      const Tile tl = decode_tile(sh, p, t, num_n_tiles);
      // channel (row of the expert's [N, K] weight) of the tile's two halves
      const int n0 = p.fused ? tl.nt * 128 : tl.nt * BN;
      const int n1 = p.fused ? p.N / 2 + tl.nt * 128 : n0 + 128;
      for (int kb = 0; kb < KB; ++kb) {
        const uint8_t* sz = p.sz_t + ((static_cast<int64_t>(tl.expert) * KB + kb) * p.N) * 2;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&sh->p_full[sp], pp, abort_flag)) ||
            !__all_sync(0xffffffffu, ptx::mbar_wait(&sh->b_empty[sb], pb ^ 1u, abort_flag))) { ok = false; break; }
        const uint4* src = reinterpret_cast<const uint4*>(smem_p + size_t(sp) * kPBytes);
        uint8_t* dst = smem_b + size_t(sb) * kBBytes;
        // warp cw converts packed rows cw, cw + 4, ... (8 of the 32); a lane owns k = 4 lane .. 4 lane + 3
#pragma unroll 2
        for (int j = 0; j < 8; ++j) {
          const int r = j * kConvWarps + cw;                  // packed row in the slot: 0..15 first half, 16..31 second
          const int ch = (r < 16 ? n0 : n1 - 128) + r * 8;   // first of its 8 channels (n1 - 128 + 8 r for r >= 16)
          // 8 x (s4, z4); a second half that lies beyond N (plain epilogue, N not a multiple of 256) converts to zeros
          const uint4 pairs = ch < p.N ? __ldg(reinterpret_cast<const uint4*>(sz + static_cast<int64_t>(ch) * 2))
                                       : make_uint4(0, 0, 0, 0);
          const uint4 w = src[r * 32 + lane];
          uint32_t q[8];
          unpack_quad(w, q);
          const uint32_t pr[4] = {pairs.x, pairs.y, pairs.z, pairs.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t sz16 = (pr[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
            const int s = static_cast<int8_t>(sz16 & 0xFFu), z = static_cast<int8_t>(sz16 >> 8);
            const int n = r * 8 + i;                          // operand row 0..255
            // 128-byte-swizzled K-major rows: 16-byte chunk c of row n sits at chunk c ^ (n & 7)
            const uint32_t off = static_cast<uint32_t>(n) * 128u + ((static_cast<uint32_t>(lane >> 2) ^ (n & 7u)) << 4) + ((lane & 3u) << 2);
            *reinterpret_cast<uint32_t*>(dst + off) = dequant4(q[i], s, z);
          }
        }
        ptx::fence_proxy_async();          // the tensor core reads the tile through the async proxy
        __syncwarp();
        if (lane == 0) { ptx::mbar_arrive(&sh->b_full[sb]); ptx::mbar_arrive(&sh->p_empty[sp]); }
        if (++sp == kPStages) { sp = 0; pp ^= 1u; }
        if (++sb == kBStages) { sb = 0; pb ^= 1u; }
      }
    }
  } else {
    // ============================ promotion + epilogue warps ================================
    ptx::setmaxnreg_inc<184>();
    const int e = warp - kFirstEpiWarp;
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int hsel = e >> 2;             // which 64-column half of each 128-column block
    const int r_in_tile = q * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    int as = 0; uint32_t pacc = 0;
    int epi_n = 0;                        // fused epilogues this warp has run (same count in its partner warp)
    bool ok = true;
    for (int t = first; ok && t < total_tiles; t += step) {
      const Tile tl = decode_tile(sh, p, t, num_n_tiles);
      const bool live = q * 32 < min(BM, tl.m_end - tl.m0);     // warp-uniform: do my 32 rows hold any row of the group
      const int row = tl.m0 + r_in_tile;
      const int64_t row_ld = min(static_cast<int64_t>(row), p.M_total - 1);
      const int nb0 = p.fused ? tl.nt : min(tl.nt * 2, NB - 1);
      const int nb1 = p.fused ? NB / 2 + tl.nt : min(tl.nt * 2 + 1, NB - 1);
      const float* as_ptr = p.a_s + row_ld * p.a_s_stride;
      const float* bs0_ptr = p.b_s + (static_cast<int64_t>(tl.expert) * NB + nb0) * KB;
      const float* bs1_ptr = p.b_s + (static_cast<int64_t>(tl.expert) * NB + nb1) * KB;
      float sa_n = __ldg(as_ptr), b0_n = __ldg(bs0_ptr), b1_n = __ldg(bs1_ptr);
      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;
      for (int kb = 0; kb < KB; ++kb) {
        const float s0 = sa_n * b0_n, s1 = sa_n * b1_n;
        if (kb + 1 < KB) { sa_n = __ldg(as_ptr + kb + 1); b0_n = __ldg(bs0_ptr + kb + 1); b1_n = __ldg(bs1_ptr + kb + 1); }
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&sh->tmem_full[as], pacc, abort_flag))) { ok = false; break; }
        ptx::tc_fence_after_sync();
        if (live) {
          const uint32_t tcol = tmem_base + lane_base + static_cast<uint32_t>(as) * BN + static_cast<uint32_t>(hsel) * 64;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            ptx::tmem_ld32(tcol + (c >> 1) * 128 + (c & 1) * 32, r);
            ptx::tmem_ld_wait32(r);
            const float s = c < 2 ? s0 : s1;
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(__int2float_rn(static_cast<int>(r[j])), s, acc[c * 32 + j]);
          }
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sh->tmem_empty[as]);
        if (++as == kAccStages) { as = 0; pacc ^= 1u; }
      }
      if (!ok) break;
      if (!live) continue;                                       // both warps of a lane quarter skip together
      const bool row_ok = row < tl.m_end;
      if (!p.fused) {
        if (row_ok) {
          uint8_t* dst = static_cast<uint8_t*>(p.c) + static_cast<int64_t>(row) * p.c_stride;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int col0 = tl.nt * BN + half * 128 + hsel * 64;
            if (col0 >= p.N) continue;
            if (p.c_dtype == B200MOE_F32) store_row64(reinterpret_cast<float*>(dst) + col0, acc + half * 64);
            else if (p.c_dtype == B200MOE_BF16) store_row64(reinterpret_cast<__nv_bfloat16*>(dst) + col0, acc + half * 64);
            else store_row64(reinterpret_cast<__half*>(dst) + col0, acc + half * 64);
          }
        }
      } else {
        // act(gate) * up with the roundings of the unfused chain (GEMM output, activation and product each rounded
        // to bf16; moe/group_gemm_kernel.py:120-235), then the int8 1x128 quantizer of
        // quantization/w4a8_kernel.py:145-168: s = amax / 127, y = floor(h / s + 0.5), s stored after an f16 rounding.
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
        const int buf = epi_n & 1;
        sh->amax[buf][hsel][r_in_tile] = amax;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sh->amax_bar[buf][q]);       // the two warps that share these 32 rows
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&sh->amax_bar[buf][q], (epi_n >> 1) & 1u, abort_flag))) { ok = false; break; }
        ++epi_n;
        amax = fmaxf(amax, sh->amax[buf][hsel ^ 1][r_in_tile]);
        if (row_ok) {
          const float scale = __fdiv_rn(amax, 127.f);
          uint8_t* dst = static_cast<uint8_t*>(p.c) + static_cast<int64_t>(row) * p.c_stride + tl.nt * 128 + hsel * 64;
#pragma unroll
          for (int j = 0; j < 64; j += 16) {
            uint32_t wd[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              uint32_t v = 0;
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const float rq = floorf(__fdiv_rn(acc[j + 4 * w + b], scale) + 0.5f);
                v |= (static_cast<uint32_t>(__float2int_rz(fminf(fmaxf(rq, -128.f), 127.f))) & 0xFFu) << (8 * b);
              }
              wd[w] = v;
            }
            *reinterpret_cast<uint4*>(dst + j) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
          }
          if (hsel == 0) p.c_s[static_cast<int64_t>(row) * p.c_s_stride + tl.nt] = __half2float(__float2half_rn(scale));
        }
      }
    }
  }

  // ---- teardown ------------------------------------------------------------------------------------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc<1>(tmem_base, kTmemCols);
  if (threadIdx.x == 0 && sh->abort_flag && p.status) *p.status = B200MOE_DEVICE_TIMEOUT;
}


// =========================================================================================================
// Grouped w4a16 GEMM (asymmetric group-128 int4 weights, bf16 activations) with the dequantization fused into
// the operand path; same roles as gemm_w4a8_kernel.  Differences: the packed words hold 8 consecutive k of one
// output channel (quantization/bitpack.py:38-67), so one word becomes one 16-byte chunk of a bf16 operand row;
// w = bf16((q - zero) * scale) as b200moe_w4a16_expand_bf16 (the zero-point extension of
// fast_dequant/simple_marlin/marlin_w4a16_gemm.cu:44-64); there are no block scales, so the whole K loop accumulates
// in TMEM (one stage per tile, the epilogue of tile i overlaps the MMAs of tile i + 1).
// =========================================================================================================
constexpr int kQStages = 6;                              // packed ring: 256 rows x 8 words = 8 KB per K block
constexpr uint32_t kQBytes = 256 * 8 * 4;
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
constexpr size_t kRing16 = size_t(kAStages) * kABytes + size_t(kBStages) * kBBytes + size_t(kQStages) * kQBytes;
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
  uint8_t* smem_p = smem_b + size_t(kBStages) * kBBytes;         // kQStages x [256 rows][8 words]
  Tail16* sh = reinterpret_cast<Tail16*>(smem_p + size_t(kQStages) * kQBytes);
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
        for (int kb = 0; kb < KB; ++kb) {
          if (!ptx::mbar_wait(&sh->p_empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sp = smem_p + size_t(stage) * kQBytes;
          ptx::mbar_arrive_expect_tx(&sh->p_full[stage], kQBytes);
          armed.arm(stage, phase);
          ptx::tma_load_2d(sp, &tmap_p, &sh->p_full[stage], kb * 8, row0);
          ptx::tma_load_2d(sp + kQBytes / 2, &tmap_p, &sh->p_full[stage], kb * 8, row1);
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
      const int n0 = (p.fused ? tl.nt * 128 : tl.nt * BN) + ct;             // channels of my two rows
      const int n1 = (p.fused ? p.N / 2 + tl.nt * 128 : tl.nt * BN + 128) + ct;
      const uint32_t* szb = p.sz_t + static_cast<int64_t>(tl.expert) * KG * p.N;
      uint32_t sz0 = 0, sz1 = 0;
      for (int kb = 0; kb < KB; ++kb) {
        if ((kb & 1) == 0) {                                 // a scale group spans two K blocks
          sz0 = n0 < p.N ? __ldg(szb + static_cast<int64_t>(kb >> 1) * p.N + n0) : 0u;
          sz1 = n1 < p.N ? __ldg(szb + static_cast<int64_t>(kb >> 1) * p.N + n1) : 0u;
        }
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&sh->p_full[sp], pp, abort_flag)) ||
            !__all_sync(0xffffffffu, ptx::mbar_wait(&sh->b_empty[sb], pb ^ 1u, abort_flag))) { ok = false; break; }
        const uint4* src = reinterpret_cast<const uint4*>(smem_p + size_t(sp) * kQBytes);
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

extern "C" int b200moe_grouped_gemm_w4a8(const void* a, int64_t a_row_stride_bytes, const float* a_s,
                                         int64_t a_s_row_stride, const void* b_packed, const void* s4z4_t,
                                         const float* b_s, void* c, int c_dtype, int64_t c_row_stride_bytes,
                                         float* c_s, int64_t c_s_row_stride, int64_t M_total, int64_t N, int64_t K,
                                         int num_groups, int num_weights, const int64_t* seg_indptr,
                                         const int64_t* weight_indices, int epilogue, int32_t* status_word,
                                         void* stream) {
  B200MOE_REQUIRE(a && a_s && b_packed && s4z4_t && b_s && c && seg_indptr, B200MOE_BAD_ARG, "grouped_gemm_w4a8: null pointer");
  B200MOE_REQUIRE(epilogue == 0 || epilogue == 1 || epilogue == 4, B200MOE_BAD_ARG, "grouped_gemm_w4a8: epilogue %d", epilogue);
  B200MOE_REQUIRE(M_total >= 0 && M_total < (int64_t(1) << 31) && N > 0 && K > 0 && K % 128 == 0 && N % 128 == 0,
                  B200MOE_BAD_SHAPE, "grouped_gemm_w4a8: M=%lld N=%lld K=%lld (N and K must be multiples of 128)",
                  (long long)M_total, (long long)N, (long long)K);
  B200MOE_REQUIRE(num_groups >= 1 && num_groups <= w4::kMaxGroups && num_weights >= 1 &&
                  static_cast<int64_t>(num_weights) * N < (int64_t(1) << 31), B200MOE_BAD_SHAPE,
                  "grouped_gemm_w4a8: num_groups=%d (max %d) num_weights=%d", num_groups, w4::kMaxGroups, num_weights);
  B200MOE_REQUIRE(aligned(a, 16) && aligned(b_packed, 16) && aligned(s4z4_t, 16) && aligned(c, 16) &&
                  a_row_stride_bytes % 16 == 0 && a_row_stride_bytes >= K && c_row_stride_bytes % 16 == 0,
                  B200MOE_BAD_ALIGN, "grouped_gemm_w4a8: pointers and row strides must be 16-byte aligned");
  B200MOE_REQUIRE(a_s_row_stride >= K / 128, B200MOE_BAD_ARG, "grouped_gemm_w4a8: a_s row stride too small");
  if (epilogue != 0) {
    B200MOE_REQUIRE(N % 256 == 0, B200MOE_BAD_SHAPE, "grouped_gemm_w4a8: the fused epilogue needs N %% 256 == 0, got %lld", (long long)N);
    B200MOE_REQUIRE(c_dtype == B200MOE_I8 && c_s && c_row_stride_bytes >= N / 2 && c_s_row_stride >= N / 256,
                    B200MOE_BAD_ARG, "grouped_gemm_w4a8: the fused epilogue writes int8 rows and f32 scales");
  } else {
    B200MOE_REQUIRE(c_dtype == B200MOE_F32 || c_dtype == B200MOE_F16 || c_dtype == B200MOE_BF16, B200MOE_BAD_DTYPE,
                    "grouped_gemm_w4a8: c dtype %d", c_dtype);
    B200MOE_REQUIRE(c_row_stride_bytes >= N * (c_dtype == B200MOE_F32 ? 4 : 2), B200MOE_BAD_ARG, "grouped_gemm_w4a8: c row stride too small");
  }
  if (M_total == 0) return B200MOE_OK;
  int sms = 0;
  if (int rc = require_sm100(&sms)) return rc;
  w4::RowMaps ma;
  CUtensorMap mp;
  for (int i = 0; i < 4; ++i)
    if (int rc = cached_tensor_map_u8(&ma.m[i], a, static_cast<uint64_t>(M_total), static_cast<uint64_t>(K),
                                      static_cast<uint64_t>(a_row_stride_bytes), 16u << i)) return rc;
  if (int rc = make_tensor_map_i32_plain(&mp, b_packed, static_cast<uint64_t>(num_weights) * (N / 8), static_cast<uint64_t>(K),
                                         static_cast<uint64_t>(K) * 4, 128, 16)) return rc;
  w4::Params p{a_s, a_s_row_stride, b_s, static_cast<const uint8_t*>(s4z4_t), c, c_row_stride_bytes, c_s, c_s_row_stride,
               seg_indptr, weight_indices, M_total, static_cast<int>(N), static_cast<int>(K), num_groups, c_dtype,
               epilogue != 0 ? 1 : 0, epilogue == 4 ? 1 : 0, status_word};
  cudaFuncSetAttribute(w4::gemm_w4a8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(w4::kSmemBytes));
  w4::gemm_w4a8_kernel<<<sms, w4::kThreads, w4::kSmemBytes, as_stream(stream)>>>(ma, mp, p);
  return check_launch("gemm_w4a8_kernel");
}

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
