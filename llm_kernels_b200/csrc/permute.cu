// Row movers of the MoE layer (all HBM-bound, 128-bit vectorised, one CTA per
// token or per permuted row):
//
//   pre_reorder        moe/group_gemm_kernel.py:81-117
//   permute_quant_fp8  pre_reorder fused with quantization/fp8_kernel.py:9-52
//   act_and_mul        moe/group_gemm_kernel.py:120-168 (silu), :176-235 (gelu)
//   post_reorder       moe/group_gemm_kernel.py:238-288 with the f32 accumulation
//                      of moe/all2all_moe.py:270-278
#include "common.cuh"

namespace b200moe {

constexpr int kMaxK = 32;

// Destination rows of the token's local slots, shared by the CTA.
__device__ __forceinline__ int load_slots(const int32_t* src2dst, const int64_t* topk_ids,
                                          int64_t t, int topk, int lo, int hi, int32_t* s_dst,
                                          int32_t* s_exp) {
  __shared__ int s_n;
  if (threadIdx.x == 0) {
    int n = 0;
    for (int j = 0; j < topk; ++j) {
      const int64_t e = topk_ids[t * topk + j];
      const int32_t d = src2dst[t * topk + j];
      if (e >= lo && e <= hi && d >= 0) { s_dst[n] = d; s_exp[n] = static_cast<int32_t>(e - lo) | (j << 16); ++n; }
    }
    s_n = n;
  }
  __syncthreads();
  return s_n;
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) pre_reorder_kernel(
    const TI* __restrict__ x, TO* __restrict__ out, const int32_t* __restrict__ src2dst,
    const int64_t* __restrict__ topk_ids, const float* __restrict__ a1_scales, int lo, int hi,
    int topk, int64_t H) {
  __shared__ int32_t s_dst[kMaxK], s_exp[kMaxK];
  const int64_t t = blockIdx.x;
  const int n = load_slots(src2dst, topk_ids, t, topk, lo, hi, s_dst, s_exp);
  if (n == 0) return;
  for (int64_t c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float v[8];
    load8(x + t * H + c, v);
    for (int j = 0; j < n; ++j) {
      float o[8];
      const float sc = a1_scales ? __fdiv_rn(1.0f, a1_scales[s_exp[j] & 0xffff]) : 1.0f;
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = v[k] * sc;
      if constexpr (sizeof(TO) == 1) {
        *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(out) + static_cast<int64_t>(s_dst[j]) * H + c) = pack8_e4m3(o);
      } else {
        store8(out + static_cast<int64_t>(s_dst[j]) * H + c, o);
      }
    }
  }
}

// One CTA per token; a thread owns 8 values, a half-warp one 128-value group.
template <typename TI>
__global__ void __launch_bounds__(256) permute_quant_fp8_kernel(
    const TI* __restrict__ x, const int32_t* __restrict__ src2dst,
    const int64_t* __restrict__ topk_ids, int lo, int hi, int topk, int64_t H,
    uint8_t* __restrict__ out_q, int64_t q_stride, float* __restrict__ out_s, int64_t s_stride) {
  __shared__ int32_t s_dst[kMaxK], s_exp[kMaxK];
  const int64_t t = blockIdx.x;
  const int n = load_slots(src2dst, topk_ids, t, topk, lo, hi, s_dst, s_exp);
  if (n == 0) return;
  const int64_t chunks = H / 8;                       // multiple of 16
  const int64_t padded = (chunks + 31) & ~int64_t(31);  // whole warps take part in the shuffles
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
    const uint2 packed = pack8_e4m3(q);
    const bool lead = (threadIdx.x & 15) == 0;
    for (int j = 0; j < n; ++j) {
      const int64_t d = s_dst[j];
      *reinterpret_cast<uint2*>(out_q + d * q_stride + i * 8) = packed;
      if (lead) out_s[d * s_stride + i / 16] = scale;
    }
  }
}

// Same with the int8 quantizer of quantization/w4a8_kernel.py:145-168 (rounding 1 = floor(v+0.5))
// or quantization/int8_kernel.py:9-31 (rounding 0 = half away from zero): s = amax/127 rounded to
// f16 as the reference stores it, written out as f32 next to the payload.
template <typename TI>
__global__ void __launch_bounds__(256) permute_quant_int8_kernel(
    const TI* __restrict__ x, const int32_t* __restrict__ src2dst,
    const int64_t* __restrict__ topk_ids, int lo, int hi, int topk, int64_t H,
    int8_t* __restrict__ out_q, int64_t q_stride, float* __restrict__ out_s, int64_t s_stride,
    int rounding) {
  __shared__ int32_t s_dst[kMaxK], s_exp[kMaxK];
  const int64_t t = blockIdx.x;
  const int n = load_slots(src2dst, topk_ids, t, topk, lo, hi, s_dst, s_exp);
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
    const float scale = __fdiv_rn(amax, 127.f);
    uint2 packed;
    int8_t* o8 = reinterpret_cast<int8_t*>(&packed);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float q = __fdiv_rn(v[k], scale);
      const float rq = rounding == 0 ? roundf(q) : floorf(q + 0.5f);
      o8[k] = static_cast<int8_t>(__float2int_rz(fminf(fmaxf(rq, -128.f), 127.f)));
    }
    const float stored = __half2float(__float2half_rn(scale));
    const bool lead = (threadIdx.x & 15) == 0;
    for (int j = 0; j < n; ++j) {
      const int64_t d = s_dst[j];
      *reinterpret_cast<uint2*>(out_q + d * q_stride + i * 8) = packed;
      if (lead) out_s[d * s_stride + i / 16] = stored;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) act_and_mul_kernel(
    const T* __restrict__ gateup, T* __restrict__ out, int64_t two_I,
    const int64_t* __restrict__ reorder_ids, const float* __restrict__ scales, int lo, int hi,
    int act) {
  const int64_t row = blockIdx.x;
  float sc = 1.f;
  if (reorder_ids) {
    const int64_t e = reorder_ids[row];
    if (e < lo || e > hi) return;
    if (scales) sc = round_to(__fdiv_rn(1.0f, scales[e - lo]), T());
  }
  const int64_t I = two_I / 2;
  const T* g = gateup + row * two_I;
  const T* u = g + I;
  for (int64_t c = threadIdx.x * 8; c < I; c += blockDim.x * 8) {
    float gv[8], uv[8], o[8];
    load8(g + c, gv);
    load8(u + c, uv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float a;
      if (act == 0) {
        a = gv[k] * __fdiv_rn(1.0f, 1.0f + expf(-gv[k]));
      } else {
        const float inner = 0.7978845608028654f * (gv[k] + 0.044715f * gv[k] * gv[k] * gv[k]);
        const float th = 2.f * __fdiv_rn(1.0f, 1.0f + expf(-2.f * inner)) - 1.f;
        a = 0.5f * gv[k] * (1.f + th);
      }
      a = round_to(a, T());
      float prod = round_to(a * uv[k], T());
      if (scales) prod = round_to(prod * sc, T());
      o[k] = prod;
    }
    store8(out + row * I + c, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) post_reorder_kernel(
    const T* __restrict__ down, T* __restrict__ out, const int32_t* __restrict__ src2dst,
    const int64_t* __restrict__ topk_ids, const float* __restrict__ w, int lo, int hi, int topk,
    int64_t H) {
  __shared__ int32_t s_dst[kMaxK], s_exp[kMaxK];
  __shared__ float s_w[kMaxK];
  const int64_t t = blockIdx.x;
  const int n = load_slots(src2dst, topk_ids, t, topk, lo, hi, s_dst, s_exp);
  if (threadIdx.x < n) s_w[threadIdx.x] = w[t * topk + (s_exp[threadIdx.x] >> 16)];
  __syncthreads();
  for (int64_t c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < n; ++j) {
      float v[8];
      load8(down + static_cast<int64_t>(s_dst[j]) * H + c, v);
      const float wj = s_w[j];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = fmaf(v[k], wj, acc[k]);
    }
    store8(out + t * H + c, acc);
  }
}

// dst row i <- src row row_map[i]; rows are row_bytes long (multiple of 16), one CTA per row.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint8_t* __restrict__ src,
                                                          uint8_t* __restrict__ dst,
                                                          const int32_t* __restrict__ row_map,
                                                          int64_t row_bytes) {
  const int64_t i = blockIdx.x;
  const int64_t s = row_map[i];
  if (s < 0) return;
  const uint4* in = reinterpret_cast<const uint4*>(src + s * row_bytes);
  uint4* out = reinterpret_cast<uint4*>(dst + i * row_bytes);
  for (int64_t c = threadIdx.x; c < row_bytes / 16; c += blockDim.x) out[c] = in[c];
}

static int pick_threads(int64_t chunks) {
  int th = 256;
  while (th > 32 && th / 2 >= chunks) th /= 2;
  return th;
}

}  // namespace b200moe

using namespace b200moe;

#define DISPATCH_16BIT_OR_F32(dtype, fn)                                            \
  switch (dtype) {                                                                  \
    case B200MOE_F32: fn(float); break;                                             \
    case B200MOE_F16: fn(__half); break;                                            \
    case B200MOE_BF16: fn(__nv_bfloat16); break;                                    \
    default: return fail(B200MOE_BAD_DTYPE, "%s: dtype %d", __func__, (int)(dtype)); \
  }

extern "C" int b200moe_pre_reorder(const void* x, int x_dtype, void* out, int out_dtype,
                                   const int32_t* src2dst, const int64_t* topk_ids,
                                   const float* a1_scales, int start_expert_id,
                                   int end_expert_id, int64_t T, int topk, int64_t H,
                                   void* stream) {
  B200MOE_REQUIRE(x && out && src2dst && topk_ids, B200MOE_BAD_ARG, "pre_reorder: null pointer");
  B200MOE_REQUIRE(T >= 0 && H > 0 && H % 8 == 0, B200MOE_BAD_SHAPE, "pre_reorder: hidden_size=%lld must be a multiple of 8", (long long)H);
  B200MOE_REQUIRE(topk >= 1 && topk <= kMaxK, B200MOE_BAD_SHAPE, "pre_reorder: topk=%d", topk);
  B200MOE_REQUIRE(aligned(x, 16) && aligned(out, 16), B200MOE_BAD_ALIGN, "pre_reorder: 16-byte alignment");
  B200MOE_REQUIRE(out_dtype == x_dtype || out_dtype == B200MOE_FP8_E4M3, B200MOE_BAD_DTYPE,
                  "pre_reorder: out dtype %d must equal the input dtype or be e4m3", out_dtype);
  if (T == 0) return B200MOE_OK;
  cudaStream_t st = as_stream(stream);
  const int th = pick_threads(H / 8);
  const unsigned grid = static_cast<unsigned>(T);
#define LAUNCH_PRE(TI)                                                                            \
  if (out_dtype == B200MOE_FP8_E4M3)                                                              \
    pre_reorder_kernel<TI, uint8_t><<<grid, th, 0, st>>>(static_cast<const TI*>(x), static_cast<uint8_t*>(out), src2dst, topk_ids, a1_scales, start_expert_id, end_expert_id, topk, H); \
  else                                                                                            \
    pre_reorder_kernel<TI, TI><<<grid, th, 0, st>>>(static_cast<const TI*>(x), static_cast<TI*>(out), src2dst, topk_ids, a1_scales, start_expert_id, end_expert_id, topk, H)
  DISPATCH_16BIT_OR_F32(x_dtype, LAUNCH_PRE)
#undef LAUNCH_PRE
  return check_launch("pre_reorder");
}

extern "C" int b200moe_permute_quant_fp8(const void* x, int x_dtype, const int32_t* src2dst,
                                         const int64_t* topk_ids, int start_expert_id,
                                         int end_expert_id, int64_t T, int topk, int64_t H,
                                         void* out_q, int64_t out_q_row_stride_bytes,
                                         float* out_s, int64_t out_s_row_stride, void* stream) {
  if (T == 0) return B200MOE_OK;      // an empty batch has no buffers to check
  B200MOE_REQUIRE(x && out_q && out_s && src2dst && topk_ids, B200MOE_BAD_ARG, "permute_quant_fp8: null pointer");
  B200MOE_REQUIRE(T >= 0 && H > 0 && H % 128 == 0, B200MOE_BAD_SHAPE,
                  "permute_quant_fp8: hidden_size=%lld must be divisible by block_size (block_size=128)", (long long)H);
  B200MOE_REQUIRE(topk >= 1 && topk <= kMaxK, B200MOE_BAD_SHAPE, "permute_quant_fp8: topk=%d", topk);
  B200MOE_REQUIRE(aligned(x, 16) && aligned(out_q, 8) && out_q_row_stride_bytes % 8 == 0 && aligned(out_s, 4),
                  B200MOE_BAD_ALIGN, "permute_quant_fp8: alignment");
  B200MOE_REQUIRE(out_q_row_stride_bytes >= H && out_s_row_stride >= H / 128, B200MOE_BAD_ARG,
                  "permute_quant_fp8: output strides smaller than a row");
  if (T == 0) return B200MOE_OK;
  cudaStream_t st = as_stream(stream);
  const int th = pick_threads(H / 8);
  const unsigned grid = static_cast<unsigned>(T);
#define LAUNCH_PQ(TI)                                                                           \
  permute_quant_fp8_kernel<TI><<<grid, th, 0, st>>>(static_cast<const TI*>(x), src2dst, topk_ids, \
      start_expert_id, end_expert_id, topk, H, static_cast<uint8_t*>(out_q),                     \
      out_q_row_stride_bytes, out_s, out_s_row_stride)
  DISPATCH_16BIT_OR_F32(x_dtype, LAUNCH_PQ)
#undef LAUNCH_PQ
  return check_launch("permute_quant_fp8");
}

extern "C" int b200moe_permute_quant_int8(const void* x, int x_dtype, const int32_t* src2dst,
                                          const int64_t* topk_ids, int start_expert_id,
                                          int end_expert_id, int64_t T, int topk, int64_t H,
                                          void* out_q, int64_t out_q_row_stride_bytes,
                                          float* out_s, int64_t out_s_row_stride, int rounding,
                                          void* stream) {
  B200MOE_REQUIRE(x && out_q && out_s && src2dst && topk_ids, B200MOE_BAD_ARG, "permute_quant_int8: null pointer");
  B200MOE_REQUIRE(T >= 0 && H > 0 && H % 128 == 0, B200MOE_BAD_SHAPE,
                  "permute_quant_int8: hidden_size=%lld must be divisible by block_size (block_size=128)", (long long)H);
  B200MOE_REQUIRE(topk >= 1 && topk <= kMaxK, B200MOE_BAD_SHAPE, "permute_quant_int8: topk=%d", topk);
  B200MOE_REQUIRE(rounding == 0 || rounding == 1, B200MOE_BAD_ARG, "permute_quant_int8: rounding %d", rounding);
  B200MOE_REQUIRE(aligned(x, 16) && aligned(out_q, 8) && out_q_row_stride_bytes % 8 == 0 && aligned(out_s, 4),
                  B200MOE_BAD_ALIGN, "permute_quant_int8: alignment");
  B200MOE_REQUIRE(out_q_row_stride_bytes >= H && out_s_row_stride >= H / 128, B200MOE_BAD_ARG,
                  "permute_quant_int8: output strides smaller than a row");
  if (T == 0) return B200MOE_OK;
  cudaStream_t st = as_stream(stream);
  const int th = pick_threads(H / 8);
  const unsigned grid = static_cast<unsigned>(T);
#define LAUNCH_PQ8(TI)                                                                           \
  permute_quant_int8_kernel<TI><<<grid, th, 0, st>>>(static_cast<const TI*>(x), src2dst, topk_ids, \
      start_expert_id, end_expert_id, topk, H, static_cast<int8_t*>(out_q),                       \
      out_q_row_stride_bytes, out_s, out_s_row_stride, rounding)
  DISPATCH_16BIT_OR_F32(x_dtype, LAUNCH_PQ8)
#undef LAUNCH_PQ8
  return check_launch("permute_quant_int8");
}

extern "C" int b200moe_gather_rows(const void* src, void* dst, const int32_t* row_map, int64_t n,
                                   int64_t row_bytes, void* stream) {
  B200MOE_REQUIRE(n >= 0 && row_bytes > 0 && row_bytes % 16 == 0, B200MOE_BAD_SHAPE,
                  "gather_rows: row_bytes=%lld must be a positive multiple of 16", (long long)row_bytes);
  if (n == 0) return B200MOE_OK;
  B200MOE_REQUIRE(src && dst && row_map, B200MOE_BAD_ARG, "gather_rows: null pointer");
  B200MOE_REQUIRE(aligned(src, 16) && aligned(dst, 16), B200MOE_BAD_ALIGN, "gather_rows: 16-byte alignment");
  gather_rows_kernel<<<static_cast<unsigned>(n), pick_threads(row_bytes / 16), 0, as_stream(stream)>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), row_map, row_bytes);
  return check_launch("gather_rows");
}

extern "C" int b200moe_act_and_mul(const void* gateup, int dtype, void* down_input, int out_dtype,
                                   int64_t rows, int64_t two_I, const int64_t* reorder_topk_ids,
                                   const float* scales, int start_expert_id, int end_expert_id,
                                   int act, void* stream) {
  B200MOE_REQUIRE(gateup && down_input, B200MOE_BAD_ARG, "act_and_mul: null pointer");
  B200MOE_REQUIRE(rows >= 0 && two_I > 0 && two_I % 16 == 0, B200MOE_BAD_SHAPE,
                  "act_and_mul: hidden_size=%lld must be a multiple of 16", (long long)two_I);
  B200MOE_REQUIRE(act == 0 || act == 1, B200MOE_BAD_ARG, "act_and_mul: act %d", act);
  B200MOE_REQUIRE(out_dtype == dtype, B200MOE_BAD_DTYPE, "act_and_mul: out dtype must equal in dtype");
  B200MOE_REQUIRE(scales == nullptr || reorder_topk_ids != nullptr, B200MOE_BAD_ARG,
                  "act_and_mul: per-expert scales need reorder_topk_ids");
  B200MOE_REQUIRE(aligned(gateup, 16) && aligned(down_input, 16), B200MOE_BAD_ALIGN, "act_and_mul: alignment");
  if (rows == 0) return B200MOE_OK;
  cudaStream_t st = as_stream(stream);
  const int th = pick_threads(two_I / 16);
  const unsigned grid = static_cast<unsigned>(rows);
#define LAUNCH_AM(TT)                                                                       \
  act_and_mul_kernel<TT><<<grid, th, 0, st>>>(static_cast<const TT*>(gateup), static_cast<TT*>(down_input), \
      two_I, reorder_topk_ids, scales, start_expert_id, end_expert_id, act)
  DISPATCH_16BIT_OR_F32(dtype, LAUNCH_AM)
#undef LAUNCH_AM
  return check_launch("act_and_mul");
}

extern "C" int b200moe_post_reorder(const void* down_output, int dtype, void* out,
                                    const int32_t* src2dst, const int64_t* topk_ids,
                                    const float* topk_weights, int start_expert_id,
                                    int end_expert_id, int64_t T, int topk, int64_t H,
                                    void* stream) {
  B200MOE_REQUIRE(down_output && out && src2dst && topk_ids && topk_weights, B200MOE_BAD_ARG, "post_reorder: null pointer");
  B200MOE_REQUIRE(T >= 0 && H > 0 && H % 8 == 0, B200MOE_BAD_SHAPE, "post_reorder: hidden_size=%lld must be a multiple of 8", (long long)H);
  B200MOE_REQUIRE(topk >= 1 && topk <= kMaxK, B200MOE_BAD_SHAPE, "post_reorder: topk=%d", topk);
  B200MOE_REQUIRE(aligned(down_output, 16) && aligned(out, 16), B200MOE_BAD_ALIGN, "post_reorder: alignment");
  if (T == 0) return B200MOE_OK;
  cudaStream_t st = as_stream(stream);
  const int th = pick_threads(H / 8);
  const unsigned grid = static_cast<unsigned>(T);
#define LAUNCH_POST(TT)                                                                      \
  post_reorder_kernel<TT><<<grid, th, 0, st>>>(static_cast<const TT*>(down_output), static_cast<TT*>(out), \
      src2dst, topk_ids, topk_weights, start_expert_id, end_expert_id, topk, H)
  DISPATCH_16BIT_OR_F32(dtype, LAUNCH_POST)
#undef LAUNCH_POST
  return check_launch("post_reorder");
}
