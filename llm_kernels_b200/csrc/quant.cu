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

}  // namespace b200moe

using namespace b200moe;

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
