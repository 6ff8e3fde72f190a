// Top-k router: MoEGate.forward of moe/all2all_moe.py:60-118, one launch.
//
// Phase A computes f32 logits x . W^T for a tile of tokens into shared memory;
// phase B (one warp per token) applies sigmoid/softmax, the group-limited
// selection and the weight normalisation.  Ties always go to the lower expert
// id, so the output is a pure function of the scores.
//
//   E <= 32  : one warp per token, 128-bit loads of x, shuffle reductions
//              (HBM-bound: x is read once, W stays in L1/L2)
//   E <= 256 : 32-token x E register-tiled f32 GEMM through shared memory
#include "common.cuh"

namespace b200moe {

constexpr int kMaxE = 256;
constexpr int kMaxTopK = 32;

struct RouterParams {
  const float* w;      // [E,H]
  const float* bias;   // [E] or null
  int64_t T, H;
  int E, top_k, n_group, topk_group, scoring, norm;
  float scale;
  int64_t* topk_idx;
  float* topk_weight;
};

// Warp-wide argmax with "larger value, then lower index" order.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// Phase B for one token.  `logit` points at E f32 logits in shared memory, `sfc`
// at E floats of scratch (selection scores), both private to the calling warp.
__device__ void select_token(const RouterParams& p, int64_t t, float* logit, float* sfc) {
  const int lane = threadIdx.x & 31;
  const int E = p.E;
  // scores (kept in `logit`) and selection scores
  if (p.scoring == 1) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, logit[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float ex = expf(logit[e] - m); logit[e] = ex; sum += ex; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    for (int e = lane; e < E; e += 32) logit[e] = __fdiv_rn(logit[e], sum);
  } else {
    for (int e = lane; e < E; e += 32) logit[e] = __fdiv_rn(1.f, 1.f + expf(-logit[e]));
  }
  for (int e = lane; e < E; e += 32) sfc[e] = logit[e] + (p.bias ? p.bias[e] : 0.f);
  __syncwarp();

  if (p.n_group > 1) {
    // group score = sum of the two largest selection scores of the group
    const int gsz = E / p.n_group;
    uint32_t keep = 0;  // bit g set = group g survives (n_group <= 32)
    float gs = -INFINITY;
    if (lane < p.n_group) {
      float a = -INFINITY, b = -INFINITY;
      for (int j = 0; j < gsz; ++j) {
        const float v = sfc[lane * gsz + j];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gs = a + b;
    }
    for (int r = 0; r < p.topk_group; ++r) {
      float v = gs; int i = lane;
      warp_argmax(v, i);
      keep |= 1u << i;
      if (lane == i) gs = -INFINITY;
    }
    for (int e = lane; e < E; e += 32)
      if (!((keep >> (e / gsz)) & 1u)) sfc[e] = 0.0f;     // masked_fill(~mask, 0.0)
    __syncwarp();
  }

  // top-k over the selection scores
  float wsum = 0.f;
  float my_w = 0.f; int my_i = 0;   // lane r keeps the r-th pick
  for (int r = 0; r < p.top_k; ++r) {
    float v = -INFINITY; int i = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float s = sfc[e];
      if (s > v) { v = s; i = e; }        // ascending e: first maximum = lowest id
    }
    warp_argmax(v, i);
    if (i == 0x7fffffff) i = 0;           // all candidates NaN/-inf: degenerate input
    const float sc = logit[i];
    if (lane == r) { my_w = sc; my_i = i; }
    wsum += sc;
    if (lane == (i & 31)) sfc[i] = -INFINITY;
    __syncwarp();
  }
  if (lane < p.top_k) {
    float wv = my_w;
    if (p.top_k > 1 && p.norm) wv = __fdiv_rn(wv, wsum + 1e-20f);
    wv *= p.scale;
    p.topk_idx[t * p.top_k + lane] = my_i;
    p.topk_weight[t * p.top_k + lane] = wv;
  }
}

// ---- E <= 32: warp per token ------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) router_small_kernel(const T* __restrict__ x, RouterParams p) {
  __shared__ float s_logit[8][32];
  __shared__ float s_sfc[8][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  if (t >= p.T) return;
  const int E = p.E;
  float acc[32];
#pragma unroll
  for (int e = 0; e < 32; ++e) acc[e] = 0.f;
  const T* xr = x + t * p.H;
  for (int64_t h = lane * 8; h < p.H; h += 256) {
    float xv[8];
    load8(xr + h, xv);
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      if (e < E) {
        float wv[8];
        load8(p.w + e * p.H + h, wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[e] = fmaf(xv[k], wv[k], acc[e]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 32; ++e) {
    if (e < E) {
      float v = acc[e];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) s_logit[warp][e] = v;
    }
  }
  __syncwarp();
  select_token(p, t, s_logit[warp], s_sfc[warp]);
}

// ---- E <= 256: 32 tokens x E tile, K chunks of 32 through shared memory -----------
constexpr int kTM = 32;   // tokens per CTA
constexpr int kKC = 32;   // K chunk
constexpr int kLd = kKC + 4;

template <typename T>
__global__ void __launch_bounds__(256) router_tiled_kernel(const T* __restrict__ x, RouterParams p) {
  extern __shared__ __align__(16) float smem[];
  float* xs = smem;                       // [kTM][kLd]
  float* ws = xs + kTM * kLd;             // [kMaxE][kLd]
  float* lg = ws + kMaxE * kLd;           // [kTM][kMaxE] logits, later scores
  float* sf = lg + kTM * kMaxE;           // [8][kMaxE] per-warp selection scratch
  const int tid = threadIdx.x;
  const int tx = tid & 31, ty = tid >> 5;  // ty: 4 tokens each; tx: experts tx + 32 j
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * kTM;
  const int E = p.E;
  float acc[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[a][b] = 0.f;

  for (int64_t k0 = 0; k0 < p.H; k0 += kKC) {
    // x tile: 32 tokens x 32 k = 128 chunks of 8 -> threads 0..127
    if (tid < 128) {
      const int r = tid >> 2, c = (tid & 3) * 8;
      float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (t0 + r < p.T && k0 + c < p.H) load8(x + (t0 + r) * p.H + k0 + c, v);
      store8(xs + r * kLd + c, v);
    }
    // W tile: E x 32 k = E*4 chunks of 8
    for (int i = tid; i < E * 4; i += 256) {
      const int r = i >> 2, c = (i & 3) * 8;
      float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (k0 + c < p.H) load8(p.w + static_cast<int64_t>(r) * p.H + k0 + c, v);
      store8(ws + r * kLd + c, v);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kKC; kk += 4) {
      float4 xv[4], wv[8];
#pragma unroll
      for (int a = 0; a < 4; ++a) xv[a] = *reinterpret_cast<const float4*>(xs + (ty * 4 + a) * kLd + kk);
#pragma unroll
      for (int b = 0; b < 8; ++b)
        wv[b] = (tx + 32 * b < E) ? *reinterpret_cast<const float4*>(ws + (tx + 32 * b) * kLd + kk)
                                  : make_float4(0, 0, 0, 0);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          acc[a][b] = fmaf(xv[a].x, wv[b].x, acc[a][b]);
          acc[a][b] = fmaf(xv[a].y, wv[b].y, acc[a][b]);
          acc[a][b] = fmaf(xv[a].z, wv[b].z, acc[a][b]);
          acc[a][b] = fmaf(xv[a].w, wv[b].w, acc[a][b]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b)
      if (tx + 32 * b < E) lg[(ty * 4 + a) * kMaxE + tx + 32 * b] = acc[a][b];
  __syncthreads();
  for (int a = 0; a < 4; ++a) {
    const int64_t t = t0 + ty * 4 + a;
    if (t < p.T) select_token(p, t, lg + (ty * 4 + a) * kMaxE, sf + ty * kMaxE);
    __syncwarp();
  }
}

// ---- selection from precomputed logits (tensor-core path) ----------------------------------
__global__ void __launch_bounds__(256) router_select_kernel(const float* __restrict__ partials,
                                                            int nsplit, int64_t row_stride, RouterParams p) {
  extern __shared__ __align__(16) float smem[];   // [8 warps][2][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  if (t >= p.T) return;
  float* lg = smem + warp * 2 * p.E;
  float* sf = lg + p.E;
  for (int e = lane; e < p.E; e += 32) {
    float v = 0.f;
    for (int s = 0; s < nsplit; ++s) v += partials[(static_cast<int64_t>(s) * p.T + t) * row_stride + e];
    lg[e] = v;
  }
  __syncwarp();
  select_token(p, t, lg, sf);
}

constexpr size_t kTiledSmem = sizeof(float) * (kTM * kLd + kMaxE * kLd + kTM * kMaxE + 8 * kMaxE);

template <typename T>
static int launch_router(const T* x, const RouterParams& p, cudaStream_t st) {
  if (p.E <= 32) {
    const unsigned grid = static_cast<unsigned>((p.T + 7) / 8);
    router_small_kernel<T><<<grid, 256, 0, st>>>(x, p);
  } else {
    // more than 48 KB of dynamic shared memory needs the opt-in (per device, cheap)
    cudaFuncSetAttribute(router_tiled_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(kTiledSmem));
    const unsigned grid = static_cast<unsigned>((p.T + kTM - 1) / kTM);
    router_tiled_kernel<T><<<grid, 256, kTiledSmem, st>>>(x, p);
  }
  return check_launch("router_topk");
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_router_topk(const void* x, int x_dtype, const float* w, const float* bias,
                                   int64_t T, int64_t H, int E, int top_k, int n_group,
                                   int topk_group, int scoring, int norm_topk_prob,
                                   float routed_scaling_factor, int64_t* topk_idx,
                                   float* topk_weight, void* stream) {
  B200MOE_REQUIRE(x && w && topk_idx && topk_weight, B200MOE_BAD_ARG, "router_topk: null pointer");
  B200MOE_REQUIRE(T >= 0 && H > 0 && H % 8 == 0, B200MOE_BAD_SHAPE, "router_topk: H=%lld must be a positive multiple of 8", (long long)H);
  B200MOE_REQUIRE(E >= 1 && E <= kMaxE, B200MOE_BAD_SHAPE, "router_topk: E=%d not in [1,%d]", E, kMaxE);
  B200MOE_REQUIRE(top_k >= 1 && top_k <= kMaxTopK && top_k <= E, B200MOE_BAD_SHAPE, "router_topk: top_k=%d", top_k);
  B200MOE_REQUIRE(n_group >= 1 && n_group <= 32 && E % n_group == 0, B200MOE_BAD_SHAPE,
                  "router_topk: n_group=%d must divide E=%d and be <= 32", n_group, E);
  B200MOE_REQUIRE(topk_group >= 1 && topk_group <= n_group, B200MOE_BAD_SHAPE, "router_topk: topk_group=%d", topk_group);
  B200MOE_REQUIRE(n_group == 1 || E / n_group >= 2, B200MOE_BAD_SHAPE,
                  "router_topk: groups of %d expert(s) cannot supply a top-2 sum", E / n_group);
  B200MOE_REQUIRE(scoring == 0 || scoring == 1, B200MOE_BAD_ARG,
                  "router_topk: insupportable scoring function for MoE gating: %d", scoring);
  B200MOE_REQUIRE(aligned(x, 16) && aligned(w, 16), B200MOE_BAD_ALIGN, "router_topk: x and w must be 16-byte aligned");
  if (T == 0) return B200MOE_OK;
  RouterParams p{w, bias, T, H, E, top_k, n_group, topk_group, scoring, norm_topk_prob,
                 routed_scaling_factor, topk_idx, topk_weight};
  cudaStream_t st = as_stream(stream);
  switch (x_dtype) {
    case B200MOE_F32: return launch_router(static_cast<const float*>(x), p, st);
    case B200MOE_F16: return launch_router(static_cast<const __half*>(x), p, st);
    case B200MOE_BF16: return launch_router(static_cast<const __nv_bfloat16*>(x), p, st);
    default: return fail(B200MOE_BAD_DTYPE, "router_topk: x dtype %d", x_dtype);
  }
}

extern "C" int b200moe_router_select(const float* partials, int nsplit, int64_t partials_row_stride,
                                     const float* bias, int64_t T, int E,
                                     int top_k, int n_group, int topk_group, int scoring,
                                     int norm_topk_prob, float routed_scaling_factor, int64_t* topk_idx,
                                     float* topk_weight, void* stream) {
  B200MOE_REQUIRE(partials && topk_idx && topk_weight, B200MOE_BAD_ARG, "router_select: null pointer");
  B200MOE_REQUIRE(nsplit >= 1 && T >= 0 && E >= 1 && E <= 1024 && partials_row_stride >= E, B200MOE_BAD_SHAPE,
                  "router_select: nsplit=%d E=%d row stride %lld", nsplit, E, (long long)partials_row_stride);
  B200MOE_REQUIRE(top_k >= 1 && top_k <= kMaxTopK && top_k <= E, B200MOE_BAD_SHAPE, "router_select: top_k=%d", top_k);
  B200MOE_REQUIRE(n_group >= 1 && n_group <= 32 && E % n_group == 0 && topk_group >= 1 && topk_group <= n_group &&
                  (n_group == 1 || E / n_group >= 2), B200MOE_BAD_SHAPE, "router_select: n_group=%d topk_group=%d", n_group, topk_group);
  B200MOE_REQUIRE(scoring == 0 || scoring == 1, B200MOE_BAD_ARG,
                  "router_select: insupportable scoring function for MoE gating: %d", scoring);
  if (T == 0) return B200MOE_OK;
  RouterParams p{nullptr, bias, T, 0, E, top_k, n_group, topk_group, scoring, norm_topk_prob,
                 routed_scaling_factor, topk_idx, topk_weight};
  const unsigned grid = static_cast<unsigned>((T + 7) / 8);
  const size_t smem = sizeof(float) * 8 * 2 * E;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(router_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  router_select_kernel<<<grid, 256, smem, as_stream(stream)>>>(partials, nsplit, partials_row_stride, p);
  return check_launch("router_select");
}
