// Activation / weight quantizers (HBM-bound, 128-bit vectorised).
//
//   act_quant_fp8     quantization/fp8_kernel.py:9-52   1x128 groups, s = amax/448
//   weight_dequant    quantization/fp8_kernel.py:55-105 128x128 blocks
//   weight_quant_fp8  fp8 twin of quantization/int8_kernel.py:59-113
//   act_quant_int8    quantization/int8_kernel.py:9-56 and quantization/w4a8_kernel.py:145-193
#include "common.cuh"

namespace b200moe {

// One thread owns 8 consecutive values; the 16 lanes of a half-warp own one
// 128-value group and reduce its amax with xor-shuffles.
template <typename T>
__global__ void __launch_bounds__(256) act_quant_fp8_kernel(
    const T* __restrict__ x, int64_t rows, int64_t cols, uint8_t* __restrict__ y,
    int64_t y_stride, float* __restrict__ s, int64_t s_stride) {
  const int64_t chunks_per_row = cols / 8;
  const int64_t total = rows * chunks_per_row;
  // total is a multiple of 16, the grid is sized so whole half-warps are in or out
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool live = i < total;
  float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int64_t r = 0, c = 0;
  if (live) {
    r = i / chunks_per_row;
    c = (i - r * chunks_per_row) * 8;
    load8(x + r * cols + c, v);
  }
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = __fdiv_rn(amax, 448.f);
  if (live) {
    float q[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) q[k] = __fdiv_rn(v[k], scale);
    *reinterpret_cast<uint2*>(y + r * y_stride + c) = pack8_e4m3(q);
    if ((threadIdx.x & 15) == 0) s[r * s_stride + c / 128] = scale;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) weight_dequant_fp8_kernel(
    const uint8_t* __restrict__ x, const float* __restrict__ s, T* __restrict__ y, int64_t M,
    int64_t N) {
  const int64_t nb = (N + 127) / 128;
  const int64_t total = M * N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / N, c = i - r * N;
    const float v = e4m3_to_float(x[i]) * s[(r / 128) * nb + c / 128];
    y[i] = static_cast<T>(v);
  }
}

// One CTA per 128x128 block: pass 1 amax, pass 2 quantize.
template <typename T>
__global__ void __launch_bounds__(256) weight_quant_fp8_kernel(
    const T* __restrict__ w, uint8_t* __restrict__ y, float* __restrict__ s, int64_t M,
    int64_t N) {
  __shared__ float red[8];
  __shared__ float sh_scale;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 128;
  const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 128;
  float amax = 0.f;
  for (int e = threadIdx.x; e < 128 * 128; e += 256) {
    const int64_t r = r0 + e / 128, c = c0 + e % 128;
    if (r < M && c < N) amax = fmaxf(amax, fabsf(static_cast<float>(w[r * N + c])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
    for (int k = 1; k < 8; ++k) m = fmaxf(m, red[k]);
    sh_scale = __fdiv_rn(m, 448.f);
    s[blockIdx.y * gridDim.x + blockIdx.x] = sh_scale;
  }
  __syncthreads();
  const float scale = sh_scale;
  for (int e = threadIdx.x; e < 128 * 128; e += 256) {
    const int64_t r = r0 + e / 128, c = c0 + e % 128;
    if (r < M && c < N)
      y[r * N + c] = to_e4m3(__fdiv_rn(static_cast<float>(w[r * N + c]), scale));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) act_quant_int8_kernel(
    const T* __restrict__ x, int64_t total_chunks, int8_t* __restrict__ y,
    __half* __restrict__ s, int rounding) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool live = i < total_chunks;
  float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (live) load8(x + i * 8, v);
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = __fdiv_rn(amax, 127.f);
  if (live) {
    uint2 out;
    int8_t* o8 = reinterpret_cast<int8_t*>(&out);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float q = __fdiv_rn(v[k], scale);
      const float rq = rounding == 0 ? roundf(q) : floorf(q + 0.5f);
      // float -> int8 as the reference's .to(int8) does for in-range values; NaN -> 0
      o8[k] = static_cast<int8_t>(__float2int_rz(fminf(fmaxf(rq, -128.f), 127.f)));
    }
    *reinterpret_cast<uint2*>(y + i * 8) = out;
    if ((threadIdx.x & 15) == 0) s[i / 16] = __float2half_rn(scale);
  }
}

// Quantized all-reduce, middle step (quant_communication/quant_all2all_allreduce.py:73-80): the chunks received
// from the n_src ranks are dequantized, each rounded to the output dtype, summed in f32 in rank order and the
// sum rounded to the output dtype.  One thread owns 8 consecutive values of a row.
template <typename TO, typename TS, bool FP8>
__global__ void __launch_bounds__(256) dequant_sum_kernel(
    const uint8_t* __restrict__ q, int64_t q_row_stride, int64_t q_src_stride, const TS* __restrict__ s,
    int64_t s_row_stride, int64_t s_src_stride, int n_src, int64_t rows, int64_t cols, TO* __restrict__ out) {
  const int64_t chunks = cols / 8, total = rows * chunks;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / chunks, c = (i - r * chunks) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int src = 0; src < n_src; ++src) {
      const uint2 raw = *reinterpret_cast<const uint2*>(q + src * q_src_stride + r * q_row_stride + c);
      const float sc = static_cast<float>(s[src * s_src_stride + r * s_row_stride + c / 128]);
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        // an all-zero group has scale 0 and, by the quantizer's x / s, a NaN payload: it decodes to zero
        const float v = sc == 0.f ? 0.f : (FP8 ? e4m3_to_float(b[k]) : static_cast<float>(static_cast<int8_t>(b[k])));
        // the product is formed in the scale's dtype (exact in f32, then one rounding), then cast to the output dtype
        acc[k] += round_to(round_to(v * sc, TS()), TO());
      }
    }
    store8(out + r * cols + c, acc);
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_dequant_sum(const void* q, int q_dtype, int64_t q_row_stride_bytes, int64_t q_src_stride_bytes,
                                   const void* s, int s_dtype, int64_t s_row_stride, int64_t s_src_stride, int n_src,
                                   int64_t rows, int64_t cols, void* out, int out_dtype, void* stream) {
  B200MOE_REQUIRE(q && s && out, B200MOE_BAD_ARG, "dequant_sum: null pointer");
  B200MOE_REQUIRE(rows >= 0 && cols >= 0 && cols % 128 == 0 && n_src >= 1, B200MOE_BAD_SHAPE,
                  "dequant_sum: Last dimension size must be divisible by block_size (block_size=128), got %lld (%d sources)",
                  (long long)cols, n_src);
  B200MOE_REQUIRE((q_dtype == B200MOE_FP8_E4M3 && s_dtype == B200MOE_F32) || (q_dtype == B200MOE_I8 && s_dtype == B200MOE_F16),
                  B200MOE_BAD_DTYPE, "dequant_sum: payload %d with scales %d (e4m3 + f32 or int8 + f16)", q_dtype, s_dtype);
  B200MOE_REQUIRE(out_dtype == B200MOE_BF16 || out_dtype == B200MOE_F16, B200MOE_BAD_DTYPE, "dequant_sum: out dtype %d", out_dtype);
  B200MOE_REQUIRE(aligned(q, 8) && q_row_stride_bytes % 8 == 0 && q_src_stride_bytes % 8 == 0 && aligned(out, 16),
                  B200MOE_BAD_ALIGN, "dequant_sum: alignment");
  B200MOE_REQUIRE(q_row_stride_bytes >= cols && s_row_stride >= cols / 128, B200MOE_BAD_ARG, "dequant_sum: strides smaller than a row");
  if (rows == 0 || cols == 0) return B200MOE_OK;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((rows * (cols / 8) + 255) / 256, 148 * 16));
  cudaStream_t st = as_stream(stream);
  const uint8_t* q8 = static_cast<const uint8_t*>(q);
#define DQS(TO, TS, F8) dequant_sum_kernel<TO, TS, F8><<<grid, 256, 0, st>>>(q8, q_row_stride_bytes, q_src_stride_bytes, \
    static_cast<const TS*>(s), s_row_stride, s_src_stride, n_src, rows, cols, static_cast<TO*>(out))
  if (q_dtype == B200MOE_FP8_E4M3) {
    if (out_dtype == B200MOE_BF16) DQS(__nv_bfloat16, float, true); else DQS(__half, float, true);
  } else {
    if (out_dtype == B200MOE_BF16) DQS(__nv_bfloat16, __half, false); else DQS(__half, __half, false);
  }
#undef DQS
  return check_launch("dequant_sum");
}

extern "C" int b200moe_act_quant_fp8(const void* x, int x_dtype, int64_t rows, int64_t cols,
                                     void* y, int64_t y_row_stride_bytes, float* s,
                                     int64_t s_row_stride, void* stream) {
  B200MOE_REQUIRE(x && y && s, B200MOE_BAD_ARG, "act_quant_fp8: null pointer");
  B200MOE_REQUIRE(rows >= 0 && cols >= 0 && cols % 128 == 0, B200MOE_BAD_SHAPE,
                  "act_quant_fp8: Last dimension size must be divisible by block_size (block_size=128), got %lld",
                  (long long)cols);
  B200MOE_REQUIRE(aligned(x, 16) && aligned(y, 8) && y_row_stride_bytes % 8 == 0,
                  B200MOE_BAD_ALIGN, "act_quant_fp8: x must be 16-byte and y 8-byte aligned");
  B200MOE_REQUIRE(y_row_stride_bytes >= cols && s_row_stride >= cols / 128, B200MOE_BAD_ARG,
                  "act_quant_fp8: output strides smaller than a row");
  if (rows == 0 || cols == 0) return B200MOE_OK;
  const int64_t total = rows * (cols / 8);
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  uint8_t* y8 = static_cast<uint8_t*>(y);
  cudaStream_t st = as_stream(stream);
  switch (x_dtype) {
    case B200MOE_F32:
      act_quant_fp8_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), rows, cols, y8, y_row_stride_bytes, s, s_row_stride);
      break;
    case B200MOE_F16:
      act_quant_fp8_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), rows, cols, y8, y_row_stride_bytes, s, s_row_stride);
      break;
    case B200MOE_BF16:
      act_quant_fp8_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, cols, y8, y_row_stride_bytes, s, s_row_stride);
      break;
    default:
      return fail(B200MOE_BAD_DTYPE, "act_quant_fp8: x dtype %d", x_dtype);
  }
  return check_launch("act_quant_fp8");
}

extern "C" int b200moe_weight_dequant_fp8(const void* x, const float* s, void* y, int y_dtype,
                                          int64_t M, int64_t N, void* stream) {
  B200MOE_REQUIRE(x && s && y, B200MOE_BAD_ARG, "weight_dequant_fp8: null pointer");
  B200MOE_REQUIRE(M >= 0 && N >= 0, B200MOE_BAD_SHAPE, "weight_dequant_fp8: negative size");
  if (M == 0 || N == 0) return B200MOE_OK;
  const int64_t total = M * N;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148 * 16));
  cudaStream_t st = as_stream(stream);
  const uint8_t* x8 = static_cast<const uint8_t*>(x);
  switch (y_dtype) {
    case B200MOE_F32: weight_dequant_fp8_kernel<float><<<grid, 256, 0, st>>>(x8, s, static_cast<float*>(y), M, N); break;
    case B200MOE_F16: weight_dequant_fp8_kernel<__half><<<grid, 256, 0, st>>>(x8, s, static_cast<__half*>(y), M, N); break;
    case B200MOE_BF16: weight_dequant_fp8_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(x8, s, static_cast<__nv_bfloat16*>(y), M, N); break;
    default: return fail(B200MOE_BAD_DTYPE, "weight_dequant_fp8: y dtype %d", y_dtype);
  }
  return check_launch("weight_dequant_fp8");
}

extern "C" int b200moe_weight_quant_fp8(const void* w, int w_dtype, void* y, float* s,
                                        int64_t M, int64_t N, void* stream) {
  B200MOE_REQUIRE(w && y && s, B200MOE_BAD_ARG, "weight_quant_fp8: null pointer");
  B200MOE_REQUIRE(M >= 0 && N >= 0, B200MOE_BAD_SHAPE, "weight_quant_fp8: negative size");
  if (M == 0 || N == 0) return B200MOE_OK;
  const dim3 grid(static_cast<unsigned>((N + 127) / 128), static_cast<unsigned>((M + 127) / 128));
  B200MOE_REQUIRE(grid.y <= 65535, B200MOE_BAD_SHAPE, "weight_quant_fp8: M too large");
  cudaStream_t st = as_stream(stream);
  uint8_t* y8 = static_cast<uint8_t*>(y);
  switch (w_dtype) {
    case B200MOE_F32: weight_quant_fp8_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(w), y8, s, M, N); break;
    case B200MOE_F16: weight_quant_fp8_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(w), y8, s, M, N); break;
    case B200MOE_BF16: weight_quant_fp8_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(w), y8, s, M, N); break;
    default: return fail(B200MOE_BAD_DTYPE, "weight_quant_fp8: w dtype %d", w_dtype);
  }
  return check_launch("weight_quant_fp8");
}

extern "C" int b200moe_act_quant_int8(const void* x, int x_dtype, int64_t rows, int64_t cols,
                                      void* y, void* s_f16, int rounding, void* stream) {
  B200MOE_REQUIRE(x && y && s_f16, B200MOE_BAD_ARG, "act_quant_int8: null pointer");
  B200MOE_REQUIRE(rows >= 0 && cols >= 0 && cols % 128 == 0, B200MOE_BAD_SHAPE,
                  "act_quant_int8: Last dimension size must be divisible by block_size (block_size=128), got %lld",
                  (long long)cols);
  B200MOE_REQUIRE(rounding == 0 || rounding == 1, B200MOE_BAD_ARG, "act_quant_int8: rounding %d", rounding);
  B200MOE_REQUIRE(aligned(x, 16) && aligned(y, 8), B200MOE_BAD_ALIGN, "act_quant_int8: alignment");
  if (rows == 0 || cols == 0) return B200MOE_OK;
  const int64_t total = rows * (cols / 8);
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  cudaStream_t st = as_stream(stream);
  int8_t* y8 = static_cast<int8_t*>(y);
  __half* sh = static_cast<__half*>(s_f16);
  switch (x_dtype) {
    case B200MOE_F32: act_quant_int8_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), total, y8, sh, rounding); break;
    case B200MOE_F16: act_quant_int8_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), total, y8, sh, rounding); break;
    case B200MOE_BF16: act_quant_int8_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), total, y8, sh, rounding); break;
    default: return fail(B200MOE_BAD_DTYPE, "act_quant_int8: x dtype %d", x_dtype);
  }
  return check_launch("act_quant_int8");
}
