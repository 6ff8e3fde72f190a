// Grouped w4a8 GEMM for few rows per expert (decode), with the int4 weights unpacked inside the kernel and the
// weights, not the tokens, on the 128-row side of the tensor-core tile.
//
//   reference: w4a8_gemm_kernel (quantization/w4a8_kernel.py:317-404) unpacks the nibbles, applies
//   (q - z4) * s4 and feeds the int8 dot product inside its K loop (:362-380); per K block
//   acc += float(dot in s32) * a_s[m,kb] * b_s[n/128,kb].  The grouped form follows grouped_gemm_triton
//   (moe/group_gemm_kernel.py:291-513).
//
// Three moves keep the per-weight work of the CUDA cores small in the decode regime:
//   * The dot product of a token row a with w8 = (q - z) * s over one 128-wide K block (one (s, z) per output channel
//     and K block) is  s * (a . q  -  z * sum_k a_k).  So the tensor core multiplies the int8 tokens with the RAW
//     nibbles q (0..15 as int8) and the promotion restores the exact integer with two integer multiply-adds per value.
//     This equals the reference's int8 product whenever (q - z) * s fits int8 for every nibble q the weight holds,
//     which its quantizer guarantees (quantization/w4a8_kernel.py:228-262); the Python layer checks it once per
//     weight (smallest and largest nibble of every scale group) and otherwise expands the weight to int8.
//   * Output channels are the M = 128 rows of the MMA and the tokens its N = 16..64 columns: a thread of the promotion
//     warps owns one channel, keeps that channel's (s, z) in registers and touches only as many accumulators as there
//     are tokens, so the per-K-block work of the CUDA cores shrinks with the batch instead of staying at 128 x 256.
//   * The weight operand is channel-major in shared memory (the MMA's "MN-major" A operand): for one k its 128 channels
//     are 128 consecutive bytes.  A packed word holds 8 channels at one k, so "word & 0x0F0F0F0F" and
//     "(word >> 4) & 0x0F0F0F0F" ARE eight operand bytes (channels 8r + 0,2,4,6 and 8r + 1,3,5,7), stored with one
//     8-byte store: three integer instructions per eight weights and no transposition.  The order of the channels inside
//     the tile is permuted by that; only the promotion threads need to know (TMEM lane -> channel).
//
// One persistent CTA per SM, 512 threads:
//   warp 0       TMA producer of the packed weights: per K block and half four boxes of 16 packed rows x 32 k (int32
//                words, 8 output channels per word, quantization/bitpack.py:9-36; 128-byte swizzle so that the
//                converters read without bank conflicts), 16 KB per K block, 5-slot ring
//   warp 2       TMA producer of the int8 token rows (box of 16/32/64 rows x 128 B) and of the tile's 2 x 128 (s4, z4)
//                pairs (two 256-byte bulk copies), 6-slot ring
//   warp 3       per K block and token: sum of the 128 int8 values (dp4a) and the token's scale times the two
//                block scales, written beside the token stage
//   warps 8-15   converters: mask the nibbles of every packed word and write the two [128 k][128 channels] int8 operand
//                tiles in the 128-byte-swizzled layout the tensor core reads (2 slots)
//   warp 1       owns TMEM (4 stages x 128 s32 columns); per K block 2 x 4 tcgen05.mma.kind::i8 (M128, N = tokens, K32)
//   warps 4-7    promotion (one channel of each half per thread) and the tile epilogue
//
// Every wait is a bounded mbarrier wait; on expiry the kernel drains its copies, frees TMEM, writes
// B200MOE_DEVICE_TIMEOUT to the status word and returns.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"
#include "w4_common.cuh"

namespace b200moe {
namespace w4 {

constexpr int kChunk = 64;                       // tokens per tile at most
constexpr int kPStages = 5, kWStages = 2, kTStages = 6, kAccStages = 4;
constexpr uint32_t kPBytes = 32 * 128 * 4;       // 32 packed rows x 128 words
constexpr uint32_t kWBytes = 2 * 128 * 128;      // two halves of 128 channels x 128 B
constexpr uint32_t kTBytes = kChunk * 128;       // 64 token rows x 128 B
constexpr int kThreads8 = 512;
constexpr int kPromoWarp0 = 4, kPromoWarps = 4, kConvWarp0 = 8, kConvWarps8 = 8;
// Register hand-over: the kernel starts with 128 registers per thread; the promotion warps may only grow by what the
// other warps of the same CTA have released (an increase beyond that would wait forever).
constexpr int kRegsLaunch = 128, kRegsLow = 96, kRegsConv = 80, kRegsPromo = 240;
static_assert((kRegsLaunch - kRegsLow) * kPromoWarp0 + (kRegsLaunch - kRegsConv) * kConvWarps8 >=
              (kRegsPromo - kRegsLaunch) * kPromoWarps, "setmaxnreg budget");

struct Tail8 {
  uint64_t p_full[kPStages], p_empty[kPStages];
  uint64_t w_full[kWStages], w_empty[kWStages];
  uint64_t t_full[kTStages], t_empty[kTStages];
  uint64_t x_full[kTStages];                     // the token stage's sums and scales have been written
  uint64_t tmem_full[kAccStages], tmem_empty[kAccStages];
  uint64_t stage_full, stage_free;               // fused epilogue: the bf16 stage has been written / read
  uint32_t tmem_base;
  int abort_flag;
  // travelling with a token stage (one K block):
  alignas(16) int32_t rsum[kTStages][kChunk];    // sum of the token's 128 int8 values
  alignas(16) float2 tscale[kTStages][kChunk];   // the token's scale times the block scale of each half
  alignas(16) uint16_t sz[kTStages][256];        // (s4, z4) of the tile's 2 x 128 channels (bulk copies)
  alignas(16) __nv_bfloat16 hstage[kChunk][128]; // fused epilogue: act(gate) * up of one tile, [token][channel]
  int32_t seg[kMaxGroups + 1];
  int32_t pref[kMaxGroups + 1];                  // exclusive prefix of token chunks per group
};
constexpr size_t kRing8 = size_t(kWStages) * kWBytes + size_t(kTStages) * kTBytes + size_t(kPStages) * kPBytes;
constexpr size_t kSmem8 = 1024 + kRing8 + sizeof(Tail8);
static_assert(kSmem8 <= 232448, "shared memory of one CTA");

struct Params8 {
  const float* a_s; int64_t a_s_stride;
  const float* b_s;               // [W, N/128, K/128]
  const uint16_t* sz_t;           // [W, K/128, N]: (s4, z4) int8 pairs, s4 in the low byte
  void* c; int64_t c_stride;      // bytes
  float* c_s; int64_t c_s_stride; // floats
  const int64_t* seg; const int64_t* widx;
  int64_t M_total;
  int N, K, num_groups, c_dtype, fused, act;
  int32_t* status;
};

struct Tile8 { int m0, rows, tn, expert, ct; };

__device__ __forceinline__ Tile8 decode_tile8(const Tail8* sh, const Params8& p, int t, int num_ct) {
  const int mc = t / num_ct;
  int lo = 0, hi = p.num_groups;           // last g with pref[g] <= mc
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sh->pref[mid] <= mc) lo = mid; else hi = mid;
  }
  Tile8 tl;
  tl.m0 = sh->seg[lo] + (mc - sh->pref[lo]) * kChunk;
  tl.rows = min(kChunk, sh->seg[lo + 1] - tl.m0);
  tl.tn = (tl.rows + 15) & ~15;
  tl.expert = p.widx ? static_cast<int>(p.widx[lo]) : lo;
  tl.ct = t - mc * num_ct;
  return tl;
}

// A whole warp waits for a barrier phase (every lane queries it: measured faster than one lane and a shuffle).
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag));
}

__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&a)[16], uint32_t (&b)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]),
                 "+r"(a[8]), "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15]),
                 "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]),
                 "+r"(b[8]), "+r"(b[9]), "+r"(b[10]), "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15])
               :: "memory");
}

__global__ void __launch_bounds__(kThreads8, 1)
gemm_w4a8_kernel(const __grid_constant__ RowMaps tmap_a, const __grid_constant__ CUtensorMap tmap_p, const Params8 p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_w = smem;                                          // int8 weight operand tiles (converter output)
  uint8_t* smem_t = smem_w + size_t(kWStages) * kWBytes;           // int8 token tiles (TMA)
  uint8_t* smem_p = smem_t + size_t(kTStages) * kTBytes;           // packed words (TMA)
  Tail8* sh = reinterpret_cast<Tail8*>(smem_p + size_t(kPStages) * kPBytes);
  volatile int* abort_flag = &sh->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = p.K / 128, NB = p.N / 128;
  const int num_ct = p.fused ? (p.N / 2) / 128 : (p.N + 255) / 256;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) { ptx::mbar_init(&sh->p_full[s], 1); ptx::mbar_init(&sh->p_empty[s], kConvWarps8); }
    for (int s = 0; s < kWStages; ++s) { ptx::mbar_init(&sh->w_full[s], kConvWarps8); ptx::mbar_init(&sh->w_empty[s], 1); }
    for (int s = 0; s < kTStages; ++s) {
      ptx::mbar_init(&sh->t_full[s], 1); ptx::mbar_init(&sh->t_empty[s], 1 + kPromoWarps); ptx::mbar_init(&sh->x_full[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) { ptx::mbar_init(&sh->tmem_full[s], 1); ptx::mbar_init(&sh->tmem_empty[s], kPromoWarps); }
    ptx::mbar_init(&sh->stage_full, kPromoWarps); ptx::mbar_init(&sh->stage_free, kPromoWarps);
    sh->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
#pragma unroll
    for (int i = 0; i < 3; ++i) ptx::prefetch_tensormap(&tmap_a.m[i]);
    ptx::prefetch_tensormap(&tmap_p);
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(&sh->tmem_base, kTmemCols);
    ptx::tmem_relinquish<1>();
  }
  for (int g = threadIdx.x; g <= p.num_groups; g += kThreads8) sh->seg[g] = static_cast<int32_t>(p.seg[g]);
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (warp == 3) {
    int run = 0;
    for (int g0 = 0; g0 < p.num_groups; g0 += 32) {
      const int g = g0 + lane;
      int v = 0;
      if (g < p.num_groups) { const int m = sh->seg[g + 1] - sh->seg[g]; v = m > 0 ? (m + kChunk - 1) / kChunk : 0; }
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
  const int total_tiles = sh->pref[p.num_groups] * num_ct;
  const int first = static_cast<int>(blockIdx.x), step = static_cast<int>(gridDim.x);
  // first output channel of the tile's two 128-channel halves (within the expert's N channels)
  auto half_ch = [&](const Tile8& tl, int& n0, int& n1) {
    n0 = p.fused ? tl.ct * 128 : tl.ct * 256;
    n1 = p.fused ? p.N / 2 + tl.ct * 128 : n0 + 128;
  };

  if (warp < kPromoWarp0) {
    ptx::setmaxnreg_dec<kRegsLow>();
    if (warp == 0 && lane == 0) {
      // ---- packed weights: per K block and half four boxes of 16 packed rows (128 channels) x 32 k -----------------
      int stage = 0; uint32_t phase = 0;
      Armed armed;
      bool ok = true;
      for (int t = first; ok && t < total_tiles; t += step) {
        const Tile8 tl = decode_tile8(sh, p, t, num_ct);
        int n0, n1;
        half_ch(tl, n0, n1);
        const int prow0 = (tl.expert * p.N + n0) >> 3, prow1 = (tl.expert * p.N + n1) >> 3;
        for (int kb = 0; kb < KB; ++kb) {
          if (!ptx::mbar_wait(&sh->p_empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sp = smem_p + size_t(stage) * kPBytes;
          ptx::mbar_arrive_expect_tx(&sh->p_full[stage], kPBytes);
          armed.arm(stage, phase);
#pragma unroll
          for (int g = 0; g < 4; ++g) {            // boxes of 16 packed rows x 32 k, 128-byte swizzle
            ptx::tma_load_2d(sp + g * 2048, &tmap_p, &sh->p_full[stage], kb * 128 + g * 32, prow0);
            ptx::tma_load_2d(sp + kPBytes / 2 + g * 2048, &tmap_p, &sh->p_full[stage], kb * 128 + g * 32, prow1);   // past the tensor: zero fill
          }
          if (++stage == kPStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) armed.drain(sh->p_full, kPStages);
    } else if (warp == 2 && lane == 0) {
      // ---- token rows and the channels' (s4, z4) pairs -------------------------------------------------------------
      int stage = 0; uint32_t phase = 0;
      Armed armed;
      bool ok = true;
      for (int t = first; ok && t < total_tiles; t += step) {
        const Tile8 tl = decode_tile8(sh, p, t, num_ct);
        const int sel = tl.tn <= 16 ? 0 : (tl.tn <= 32 ? 1 : 2);
        const uint32_t bytes = (16u << sel) * 128u + 512u;
        int n0, n1;
        half_ch(tl, n0, n1);
        if (n1 >= p.N) n1 = n0;
        const uint16_t* szp = p.sz_t + static_cast<int64_t>(tl.expert) * KB * p.N;
        for (int kb = 0; kb < KB; ++kb) {
          if (!ptx::mbar_wait(&sh->t_empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(&sh->t_full[stage], bytes);
          armed.arm(stage, phase);
          ptx::tma_load_2d(smem_t + size_t(stage) * kTBytes, &tmap_a.m[sel], &sh->t_full[stage], kb * 128, tl.m0);
          ptx::bulk_load(&sh->sz[stage][0], szp + static_cast<int64_t>(kb) * p.N + n0, 256u, &sh->t_full[stage]);
          ptx::bulk_load(&sh->sz[stage][128], szp + static_cast<int64_t>(kb) * p.N + n1, 256u, &sh->t_full[stage]);
          if (++stage == kTStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) armed.drain(sh->t_full, kTStages);
    } else if (warp == 1 && lane == 0) {
      // ---- MMA issuer: channels are the M = 128 rows, tokens the N columns ---------------------------------------
      int sw = 0, st = 0, as = 0;
      uint32_t pw = 0, pt = 0, pacc = 0;
      bool ok = true;
      for (int t = first; ok && t < total_tiles; t += step) {
        const Tile8 tl = decode_tile8(sh, p, t, num_ct);
        // D s32, A and B signed int8; bit 15: the A operand (weights) is channel-major in shared memory
        const uint32_t idesc = ptx::umma_idesc(2, 1, 1, 128, static_cast<uint32_t>(tl.tn)) | (1u << 15);
        for (int kb = 0; kb < KB; ++kb) {
          // x_full (sums written) follows t_full (tokens and pairs landed): the warp that arrives on it waited for
          // t_full.  Waiting for it here lets the promotion warps wait for tmem_full alone.
          if (!ptx::mbar_wait(&sh->w_full[sw], pw, abort_flag) || !ptx::mbar_wait(&sh->x_full[st], pt, abort_flag) ||
              !ptx::mbar_wait(&sh->tmem_empty[as], pacc ^ 1u, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t d = tmem_base + static_cast<uint32_t>(as) * 128u;
          const uint64_t wdesc = ptx::umma_desc_sw128(ptx::smem_u32(smem_w + size_t(sw) * kWBytes));
          const uint64_t tdesc = ptx::umma_desc_sw128(ptx::smem_u32(smem_t + size_t(st) * kTBytes));
          // Weights: 32 k of one half are four 1 KB groups of 8 k x 128 channels (4 KB per instruction).  The two
          // halves alternate, so that an instruction does not wait for the one that feeds its accumulator.
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            ptx::umma_i8<1>(d, wdesc + (4096u >> 4) * k, tdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
            ptx::umma_i8<1>(d + 64u, wdesc + (kWBytes / 2 >> 4) + (4096u >> 4) * k, tdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
          }
          ptx::umma_commit(&sh->w_empty[sw]);
          ptx::umma_commit(&sh->t_empty[st]);
          ptx::umma_commit(&sh->tmem_full[as]);
          if (++sw == kWStages) { sw = 0; pw ^= 1u; }
          if (++st == kTStages) { st = 0; pt ^= 1u; }
          if (++as == kAccStages) { as = 0; pacc ^= 1u; }
        }
      }
    } else if (warp == 3) {
      // ---- per K block: each token's sum of its 128 int8 values and its scale times the two block scales, written
      //      beside the token stage for the promotion warps ----------------------------------------------------------
      int st = 0;
      uint32_t pt = 0;
      bool ok = true;
      // four K blocks of scales per 16-byte load when the rows allow it
      const bool vec = (KB & 3) == 0 && (p.a_s_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(p.a_s) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(p.b_s) & 15) == 0;
      for (int t = first; ok && t < total_tiles; t += step) {
        const Tile8 tl = decode_tile8(sh, p, t, num_ct);
        const bool two = tl.tn > 32;
        const int64_t last = p.M_total - 1;
        int n0, n1;
        half_ch(tl, n0, n1);
        if (n1 >= p.N) n1 = n0;
        const float* src[4] = {p.a_s + min(static_cast<int64_t>(tl.m0 + lane), last) * p.a_s_stride,
                               p.a_s + min(static_cast<int64_t>(tl.m0 + lane + 32), last) * p.a_s_stride,
                               p.b_s + (static_cast<int64_t>(tl.expert) * NB + (n0 >> 7)) * KB,
                               p.b_s + (static_cast<int64_t>(tl.expert) * NB + (n1 >> 7)) * KB};
        // The scales of K blocks kb + 4 .. kb + 7 are requested while kb .. kb + 3 are worked on: a load issued and
        // consumed in the same iteration would put an L2 round trip into every K block.
        float cur[4][4], nxt[4][4];
        auto fetch = [&](float (&dst)[4][4], int kb0) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (v == 1 && !two) { dst[1][0] = dst[1][1] = dst[1][2] = dst[1][3] = 0.f; continue; }
            if (vec) {
              const float4 f = __ldg(reinterpret_cast<const float4*>(src[v] + kb0));
              dst[v][0] = f.x; dst[v][1] = f.y; dst[v][2] = f.z; dst[v][3] = f.w;
            } else {
#pragma unroll
              for (int u = 0; u < 4; ++u) dst[v][u] = kb0 + u < KB ? __ldg(src[v] + kb0 + u) : 0.f;
            }
          }
        };
        fetch(nxt, 0);
        for (int kb0 = 0; ok && kb0 < KB; kb0 += 4) {
#pragma unroll
          for (int v = 0; v < 4; ++v)
#pragma unroll
            for (int u = 0; u < 4; ++u) cur[v][u] = nxt[v][u];
          if (kb0 + 4 < KB) fetch(nxt, kb0 + 4);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (kb0 + u >= KB) break;
            if (!warp_wait(&sh->t_full[st], pt, abort_flag)) { ok = false; break; }
            // A row's 16-byte chunks are permuted by the swizzle, which a sum does not see; lanes start at different
            // chunks so that the 32 rows (128 bytes apart) do not meet in the same banks.
            const uint8_t* slot = smem_t + size_t(st) * kTBytes;
            int ra[4] = {0, 0, 0, 0}, rb[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint4 v = *reinterpret_cast<const uint4*>(slot + lane * 128 + (((j + lane) & 7) << 4));
              ra[0] = __dp4a(static_cast<int>(v.x), 0x01010101, ra[0]); ra[1] = __dp4a(static_cast<int>(v.y), 0x01010101, ra[1]);
              ra[2] = __dp4a(static_cast<int>(v.z), 0x01010101, ra[2]); ra[3] = __dp4a(static_cast<int>(v.w), 0x01010101, ra[3]);
            }
            if (two) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint4 v = *reinterpret_cast<const uint4*>(slot + (lane + 32) * 128 + (((j + lane) & 7) << 4));
                rb[0] = __dp4a(static_cast<int>(v.x), 0x01010101, rb[0]); rb[1] = __dp4a(static_cast<int>(v.y), 0x01010101, rb[1]);
                rb[2] = __dp4a(static_cast<int>(v.z), 0x01010101, rb[2]); rb[3] = __dp4a(static_cast<int>(v.w), 0x01010101, rb[3]);
              }
            }
            sh->rsum[st][lane] = (ra[0] + ra[1]) + (ra[2] + ra[3]);
            sh->rsum[st][lane + 32] = (rb[0] + rb[1]) + (rb[2] + rb[3]);
            sh->tscale[st][lane] = make_float2(cur[0][u] * cur[2][u], cur[0][u] * cur[3][u]);
            sh->tscale[st][lane + 32] = make_float2(cur[1][u] * cur[2][u], cur[1][u] * cur[3][u]);
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&sh->x_full[st]);
            if (++st == kTStages) { st = 0; pt ^= 1u; }
          }
        }
      }
    }
  } else if (warp >= kConvWarp0) {
    // ---- converters: packed word -> eight int8 nibbles, written where the tensor core expects them -------------------
    ptx::setmaxnreg_dec<kRegsConv>();
    const int cw = warp - kConvWarp0;
    const int r16 = lane & 15, kk = lane >> 4;
    // source: box (k group) cw / 4, row r16, chunk ((cw % 4) * 2 + kk) ^ (r16 % 8) of the 128-byte-swizzled box
    const uint32_t ld_off = (cw >> 2) * 2048 + r16 * 128 + (((((cw & 3) << 1) + kk) ^ (r16 & 7)) << 4);
    // destination of word 0: k = 32 (cw / 4) + 8 (cw % 4) + 4 kk; 1 KB per 8 k, 128 bytes per k, chunk (r16 / 2) ^ (k % 8)
    const uint32_t st_off = cw * 1024 + kk * 512 + (((r16 >> 1) ^ (kk << 2)) << 4) + (r16 & 1) * 8;
    int sp = 0, sw = 0;
    uint32_t pp = 0, pw = 0;
    bool ok = true;
    for (int t = first; ok && t < total_tiles; t += step) {
      for (int kb = 0; kb < KB; ++kb) {
        if (!warp_wait(&sh->p_full[sp], pp, abort_flag) ||
            !warp_wait(&sh->w_empty[sw], pw ^ 1u, abort_flag)) { ok = false; break; }
        // Thread (r, kk) of warp cw takes, four times, the 16-byte chunk (cw % 4) * 2 + kk of packed row r in k group
        // (j % 2) * 2 + cw / 4 of half j / 2: four words w(r, k .. k+3).  A word's even nibbles are channels
        // 8r + 0, 2, 4, 6 and its odd nibbles 8r + 1, 3, 5, 7 at one k: two masks give eight int8 that go, as one
        // 8-byte store, to bytes 8r .. 8r+7 of that k's 128-byte channel row.  Sixteen lanes fill a whole row.
        const uint8_t* src = smem_p + size_t(sp) * kPBytes + ld_off;
        uint8_t* dst = smem_w + size_t(sw) * kWBytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 w = *reinterpret_cast<const uint4*>(src + (j >> 1) * 8192 + (j & 1) * 4096);
          const uint32_t wd[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint2*>(dst + (st_off ^ (i << 4)) + i * 128 + (j >> 1) * 16384 + (j & 1) * 8192) =
                make_uint2(wd[i] & 0x0F0F0F0Fu, (wd[i] >> 4) & 0x0F0F0F0Fu);
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) { ptx::mbar_arrive(&sh->w_full[sw]); ptx::mbar_arrive(&sh->p_empty[sp]); }
        if (++sp == kPStages) { sp = 0; pp ^= 1u; }
        if (++sw == kWStages) { sw = 0; pw ^= 1u; }
      }
    }
  } else {
    // ---- promotion and epilogue: thread = output channel (one of each half), registers = tokens ----------------------
    ptx::setmaxnreg_inc<kRegsPromo>();
    // TMEM lane 8r + b of a half holds channel 8r + 2b (b < 4) or 8r + 2(b - 4) + 1: the converters keep a word's even
    // and odd nibbles together
    const int q = warp & 3, tl_lane = q * 32 + lane;
    const int c = (tl_lane & ~7) + ((tl_lane & 3) << 1) + ((tl_lane >> 2) & 1);
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    int as = 0, sr = 0, epi_n = 0;
    uint32_t pacc = 0;
    bool ok = true;
    for (int t = first; ok && t < total_tiles; t += step) {
      const Tile8 tl = decode_tile8(sh, p, t, num_ct);
      int n0, n1;
      half_ch(tl, n0, n1);
      const bool second = n1 < p.N;
      const int ch0 = n0 + c, ch1 = second ? n1 + c : ch0;
      float acc0[kChunk], acc1[kChunk];
#pragma unroll
      for (int m = 0; m < kChunk; ++m) { acc0[m] = 0.f; acc1[m] = 0.f; }
      // K loop and epilogue exist once per number of 16-token blocks, so that the code a tile runs is short and straight
      // (a single version unrolled for 64 tokens spent more time fetching instructions than executing them).
      auto tile_body = [&](auto nblocks) {
      constexpr int kBlocks = decltype(nblocks)::value;
      for (int kb = 0; kb < KB; ++kb) {
        // tmem_full alone: the MMAs of this K block were issued after x_full, which follows t_full, so the sums, the
        // scales and the (s4, z4) pairs of this stage are in place (acquire/release chain over the three barriers)
        if (!warp_wait(&sh->tmem_full[as], pacc, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t tcol = tmem_base + lane_base + static_cast<uint32_t>(as) * 128u;
        uint32_t d0[16], d1[16];                       // one 16-token block of each half; the next block's load is
        ptx::tmem_ld16(tcol, d0);                      // issued as soon as the registers have been consumed
        ptx::tmem_ld16(tcol + 64, d1);
        const uint32_t zs0 = sh->sz[sr][c], zs1 = sh->sz[sr][128 + c];
        const int s0 = static_cast<int8_t>(zs0 & 0xFFu), nz0 = -static_cast<int>(static_cast<int8_t>(zs0 >> 8));
        const int s1 = static_cast<int8_t>(zs1 & 0xFFu), nz1 = -static_cast<int>(static_cast<int8_t>(zs1 >> 8));
        const int4* rsp = reinterpret_cast<const int4*>(sh->rsum[sr]);
        const float4* tsp = reinterpret_cast<const float4*>(sh->tscale[sr]);
#pragma unroll
        for (int mb = 0; mb < kBlocks; ++mb) {
          {
            const bool more = mb + 1 < kBlocks;
            int4 rq[4];
            float4 tq[8];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) { rq[j4] = rsp[mb * 4 + j4]; tq[2 * j4] = tsp[mb * 8 + j4 * 2]; tq[2 * j4 + 1] = tsp[mb * 8 + j4 * 2 + 1]; }
            tmem_ld_wait16(d0, d1);
            // exact integers: sum_k a_k (q_k - z) s = s (a.q - z sum_k a_k)
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const int4 r4 = rq[j4];
              const float4 ta = tq[2 * j4], tb = tq[2 * j4 + 1];
              const int rs[4] = {r4.x, r4.y, r4.z, r4.w};
              const float ts0[4] = {ta.x, ta.z, tb.x, tb.z};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int u0 = (static_cast<int>(d0[j4 * 4 + i]) + nz0 * rs[i]) * s0;
                acc0[mb * 16 + j4 * 4 + i] = fmaf(__int2float_rn(u0), ts0[i], acc0[mb * 16 + j4 * 4 + i]);
              }
            }
            if (more) ptx::tmem_ld16(tcol + (mb + 1) * 16, d0);
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const int4 r4 = rq[j4];
              const float4 ta = tq[2 * j4], tb = tq[2 * j4 + 1];
              const int rs[4] = {r4.x, r4.y, r4.z, r4.w};
              const float ts1[4] = {ta.y, ta.w, tb.y, tb.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int u1 = (static_cast<int>(d1[j4 * 4 + i]) + nz1 * rs[i]) * s1;
                acc1[mb * 16 + j4 * 4 + i] = fmaf(__int2float_rn(u1), ts1[i], acc1[mb * 16 + j4 * 4 + i]);
              }
            }
            if (more) ptx::tmem_ld16(tcol + 64 + (mb + 1) * 16, d1);
          }
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) { ptx::mbar_arrive(&sh->tmem_empty[as]); ptx::mbar_arrive(&sh->t_empty[sr]); }
        if (++as == kAccStages) { as = 0; pacc ^= 1u; }
        if (++sr == kTStages) sr = 0;
      }
      if (!ok) return;

      if (!p.fused) {
        const int esize = p.c_dtype == B200MOE_F32 ? 4 : 2;
        uint8_t* dst0 = static_cast<uint8_t*>(p.c) + static_cast<int64_t>(tl.m0) * p.c_stride + static_cast<int64_t>(ch0) * esize;
        uint8_t* dst1 = static_cast<uint8_t*>(p.c) + static_cast<int64_t>(tl.m0) * p.c_stride + static_cast<int64_t>(ch1) * esize;
        if (p.c_dtype == B200MOE_F32) {
#pragma unroll
          for (int m = 0; m < kBlocks * 16; ++m)
            if (m < tl.rows) {
              *reinterpret_cast<float*>(dst0 + m * p.c_stride) = acc0[m];
              if (second) *reinterpret_cast<float*>(dst1 + m * p.c_stride) = acc1[m];
            }
        } else if (p.c_dtype == B200MOE_BF16) {
#pragma unroll
          for (int m = 0; m < kBlocks * 16; ++m)
            if (m < tl.rows) {
              *reinterpret_cast<__nv_bfloat16*>(dst0 + m * p.c_stride) = __float2bfloat16_rn(acc0[m]);
              if (second) *reinterpret_cast<__nv_bfloat16*>(dst1 + m * p.c_stride) = __float2bfloat16_rn(acc1[m]);
            }
        } else {
#pragma unroll
          for (int m = 0; m < kBlocks * 16; ++m)
            if (m < tl.rows) {
              *reinterpret_cast<__half*>(dst0 + m * p.c_stride) = __float2half_rn(acc0[m]);
              if (second) *reinterpret_cast<__half*>(dst1 + m * p.c_stride) = __float2half_rn(acc1[m]);
            }
        }
      } else {
        // act(gate) * up with the roundings of the unfused chain (GEMM output, activation and product each rounded
        // to bf16; moe/group_gemm_kernel.py:120-235), then the int8 1x128 quantizer of
        // quantization/w4a8_kernel.py:145-168: s = amax / 127, y = floor(h / s + 0.5), s stored after an f16 rounding.
        // The products go through a [token][channel] bf16 stage in shared memory (exact: they are bf16 values), so
        // that a warp then owns whole tokens: maximum by shuffles, four channels per lane, one 128-byte row per store.
        const uint32_t par = static_cast<uint32_t>(epi_n & 1);
        if (!warp_wait(&sh->stage_free, par ^ 1u, abort_flag)) { ok = false; return; }     // previous tile's readers are done
#pragma unroll
        for (int m = 0; m < kBlocks * 16; ++m) {
          const float g = bf16r(acc0[m]);
          const float u = bf16r(acc1[m]);
          sh->hstage[m][c] = __float2bfloat16_rn(bf16r(gate_act(g, p.act)) * u);
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sh->stage_full);
        if (!warp_wait(&sh->stage_full, par, abort_flag)) { ok = false; return; }
        ++epi_n;
        for (int m = q; m < tl.rows; m += kPromoWarps) {
          const uint2 hv = *reinterpret_cast<const uint2*>(&sh->hstage[m][lane * 4]);
          const float h[4] = {__uint_as_float(hv.x << 16), __uint_as_float(hv.x & 0xFFFF0000u),
                              __uint_as_float(hv.y << 16), __uint_as_float(hv.y & 0xFFFF0000u)};
          float amax = fmaxf(fmaxf(fabsf(h[0]), fabsf(h[1])), fmaxf(fabsf(h[2]), fabsf(h[3])));
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          const float scale = __fdiv_rn(amax, 127.f);
          uint32_t packed = 0;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float rq = floorf(__fdiv_rn(h[i], scale) + 0.5f);
            packed |= (static_cast<uint32_t>(__float2int_rz(fminf(fmaxf(rq, -128.f), 127.f))) & 0xFFu) << (8 * i);
          }
          *reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(p.c) + static_cast<int64_t>(tl.m0 + m) * p.c_stride + tl.ct * 128 + lane * 4) = packed;
          if (lane == 0) p.c_s[static_cast<int64_t>(tl.m0 + m) * p.c_s_stride + tl.ct] = __half2float(__float2half_rn(scale));
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sh->stage_free);
      }
      };
      switch (tl.tn >> 4) {
        case 1: tile_body(std::integral_constant<int, 1>{}); break;
        case 2: tile_body(std::integral_constant<int, 2>{}); break;
        case 3: tile_body(std::integral_constant<int, 3>{}); break;
        default: tile_body(std::integral_constant<int, 4>{}); break;
      }
    }
  }

  // ---- teardown ------------------------------------------------------------------------------------------
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
  for (int i = 0; i < 3; ++i)
    if (int rc = cached_tensor_map_u8(&ma.m[i], a, static_cast<uint64_t>(M_total), static_cast<uint64_t>(K),
                                      static_cast<uint64_t>(a_row_stride_bytes), 16u << i)) return rc;
  ma.m[3] = ma.m[2];
  if (int rc = make_tensor_map_i32_plain(&mp, b_packed, static_cast<uint64_t>(num_weights) * (N / 8), static_cast<uint64_t>(K),
                                         static_cast<uint64_t>(K) * 4, 32, 16, true)) return rc;
  w4::Params8 p{a_s, a_s_row_stride, b_s, static_cast<const uint16_t*>(s4z4_t), c, c_row_stride_bytes, c_s, c_s_row_stride,
                seg_indptr, weight_indices, M_total, static_cast<int>(N), static_cast<int>(K), num_groups, c_dtype,
                epilogue != 0 ? 1 : 0, epilogue == 4 ? 1 : 0, status_word};
  cudaFuncSetAttribute(w4::gemm_w4a8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(w4::kSmem8));
  w4::gemm_w4a8_kernel<<<sms, w4::kThreads8, w4::kSmem8, as_stream(stream)>>>(ma, mp, p);
  return check_launch("gemm_w4a8_kernel");
}
