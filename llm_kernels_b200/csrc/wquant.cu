// Offline weight quantizers (HBM-bound, one pass over the weight).
//
//   weight_quant_int8     quantization/int8_kernel.py:59-113   128x128 blocks, s = amax/127, round half away
//                         quantization/w4a8_kernel.py:196-225  same with s = amax/119, floor(v+0.5), clamp +-119
//   weight_dequant_int8   quantization/int8_kernel.py:116-170  y = x * s[bm, bn]
//   weight_quant_w4a8     quantization/w4a8_kernel.py:196-309  two levels: int8 per 128x128 block, then uint4 per
//                         (row, 128 columns) with int8 scale s4 and zero point z4; packed over rows
//                         (quantization/bitpack.py:9-36: word row r, nibble i = q[8r + i, c])
//   weight_quant_w4a16    asymmetric extension of fast_dequant/simple_marlin/utils.py:98-136: per (row, 128
//                         columns) scale = (max-min)/15 and zero = round(-min/scale) in bf16; packed over columns
//                         (quantization/bitpack.py:38-67: nibble i of word c = q[r, 8c + i])
//   marlin_pack           fast_dequant/simple_marlin/utils.py:53-95: 16x16 tiling, the fixed 1024-entry lane
//                         permutation with even/odd nibble interleave, 8 nibbles per int32; scale permutation
#include "common.cuh"
#include "marlin_perm.cuh"

namespace b200moe {

template <typename T>
__device__ __forceinline__ float block_amax_128(const T* __restrict__ w, int64_t r0, int64_t c0, int64_t M, int64_t N,
                                                float* red) {
  float amax = 0.f;
  for (int e = threadIdx.x; e < 128 * 128; e += 256) {
    const int64_t r = r0 + e / 128, c = c0 + e % 128;
    if (r < M && c < N) amax = fmaxf(amax, fabsf(static_cast<float>(w[r * N + c])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) m = fmaxf(m, red[k]);
  return m;
}

// float -> int8 as torch's / Triton's cast of an in-range integer-valued float; NaN -> 0
__device__ __forceinline__ int8_t f2i8(float v) {
  if (v != v) return 0;
  return static_cast<int8_t>(__float2int_rz(fminf(fmaxf(v, -128.f), 127.f)));
}

// mode 0: round half away from zero, no clamp (int8_kernel.py:82-84); mode 1: floor(v + 0.5) clamped to +-qmax
// (w4a8_kernel.py:218-221)
__device__ __forceinline__ float quant_level1(float x, float s, int mode, float qmax) {
  const float v = __fdiv_rn(x, s);
  if (v != v) return v;                       // 0/0 of an all-zero block stays NaN (stored as 0)
  return mode == 0 ? roundf(v) : fminf(fmaxf(floorf(v + 0.5f), -qmax), qmax);
}

// One CTA per 128x128 block.
template <typename T>
__global__ void __launch_bounds__(256) weight_quant_int8_kernel(const T* __restrict__ w, int8_t* __restrict__ y,
                                                                __half* __restrict__ s, int64_t M, int64_t N,
                                                                float qmax, int mode) {
  __shared__ float red[8];
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 128, c0 = static_cast<int64_t>(blockIdx.x) * 128;
  const float scale = __fdiv_rn(block_amax_128(w, r0, c0, M, N, red), qmax);
  if (threadIdx.x == 0) s[blockIdx.y * gridDim.x + blockIdx.x] = __float2half_rn(scale);
  for (int e = threadIdx.x; e < 128 * 128; e += 256) {
    const int64_t r = r0 + e / 128, c = c0 + e % 128;
    if (r < M && c < N) y[r * N + c] = f2i8(quant_level1(static_cast<float>(w[r * N + c]), scale, mode, qmax));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) weight_dequant_int8_kernel(const int8_t* __restrict__ x,
                                                                  const __half* __restrict__ s, T* __restrict__ y,
                                                                  int64_t M, int64_t N) {
  const int64_t nb = (N + 127) / 128, total = M * N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / N, c = i - r * N;
    y[i] = static_cast<T>(static_cast<float>(x[i]) * __half2float(s[(r / 128) * nb + c / 128]));
  }
}

// Two-level int4.  One CTA per 128x128 block; the block's int8 values live in shared memory between the levels.
// Level 2 gives every row of the block its own (s4, z4); 8 consecutive rows share a packed word.
template <typename T>
__global__ void __launch_bounds__(256) weight_quant_w4a8_kernel(const T* __restrict__ w, uint32_t* __restrict__ packed,
                                                                __half* __restrict__ s, int8_t* __restrict__ s4,
                                                                int8_t* __restrict__ z4, int64_t M, int64_t N) {
  __shared__ float red[8];
  __shared__ int8_t y8[128][128 + 4];     // level-1 values, overwritten in place by the level-2 nibbles
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 128, c0 = static_cast<int64_t>(blockIdx.x) * 128;
  const int64_t kg = N / 128;
  const float scale = __fdiv_rn(block_amax_128(w, r0, c0, M, N, red), 119.f);
  if (threadIdx.x == 0) s[blockIdx.y * gridDim.x + blockIdx.x] = __float2half_rn(scale);
  for (int e = threadIdx.x; e < 128 * 128; e += 256) {
    const int r = e / 128, c = e % 128;
    y8[r][c] = f2i8(quant_level1(static_cast<float>(w[(r0 + r) * N + c0 + c]), scale, 1, 119.f));
  }
  __syncthreads();
  // one warp per row, 16 rows per warp; lane l owns columns l, l+32, l+64, l+96
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < 128; r += 8) {
    float v[4], mx = -INFINITY, mn = INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[j] = static_cast<float>(y8[r][lane + 32 * j]); mx = fmaxf(mx, v[j]); mn = fminf(mn, v[j]); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    }
    __syncwarp();
    const float sc4 = floorf(__fdiv_rn(mx - mn, 15.f) + 0.5f);
    const float zp4 = floorf(__fdiv_rn(-mn, sc4) + 0.5f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float q = fminf(fmaxf(floorf(__fdiv_rn(v[j], sc4) + 0.5f) + zp4, 0.f), 15.f);
      y8[r][lane + 32 * j] = static_cast<int8_t>(__float2int_rz(q));         // NaN -> 0
    }
    if (lane == 0) {
      s4[(r0 + r) * kg + blockIdx.x] = f2i8(sc4);
      z4[(r0 + r) * kg + blockIdx.x] = f2i8(zp4);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 16 * 128; e += 256) {
    const int pr = e / 128, c = e % 128;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) word |= (static_cast<uint32_t>(y8[pr * 8 + i][c]) & 0xFu) << (4 * i);
    packed[(r0 / 8 + pr) * N + c0 + c] = word;
  }
}

// Asymmetric group-128 int4: one warp per (row, group); lane l owns 4 consecutive k, two lanes make a word.
template <typename T>
__global__ void __launch_bounds__(256) weight_quant_w4a16_kernel(const T* __restrict__ w, uint32_t* __restrict__ packed,
                                                                 __nv_bfloat16* __restrict__ scale,
                                                                 __nv_bfloat16* __restrict__ zero, int64_t rows,
                                                                 int64_t K) {
  const int64_t kg = K / 128, total = rows * kg;
  const int lane = threadIdx.x & 31;
  for (int64_t g = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; g < total;
       g += (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5) {
    const int64_t r = g / kg, kb = g - r * kg;
    const T* src = w + r * K + kb * 128 + lane * 4;
    float v[4], mx = -INFINITY, mn = INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[j] = static_cast<float>(src[j]); mx = fmaxf(mx, v[j]); mn = fminf(mn, v[j]); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    }
    const __nv_bfloat16 sc_b = __float2bfloat16_rn(fmaxf(__fdiv_rn(mx - mn, 15.f), 1e-8f));
    const float sc = __bfloat162float(sc_b);
    const __nv_bfloat16 zp_b = __float2bfloat16_rn(fminf(fmaxf(rintf(__fdiv_rn(-mn, sc)), 0.f), 15.f));
    const float zp = __bfloat162float(zp_b);
    uint32_t part = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float q = fminf(fmaxf(rintf(__fdiv_rn(v[j], sc)) + zp, 0.f), 15.f);
      part |= static_cast<uint32_t>(__float2int_rz(q)) << (4 * j);
    }
    const uint32_t hi = __shfl_down_sync(0xffffffffu, part, 1);
    if ((lane & 1) == 0) packed[r * (K / 8) + kb * 16 + lane / 2] = part | (hi << 16);
    if (lane == 0) { scale[g] = sc_b; zero[g] = zp_b; }
  }
}

// Marlin order: one thread builds one packed word (8 nibbles).
__global__ void __launch_bounds__(256) marlin_pack_kernel(const int32_t* __restrict__ q, uint32_t* __restrict__ packed,
                                                          int64_t K, int64_t N) {
  const int64_t words_per_row = N * 2, total = (K / 16) * words_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / words_per_row, j = i - r * words_per_row;
    uint32_t word = 0;
#pragma unroll
    for (int f = 0; f < 8; ++f) {
      const int64_t pcol = j * 8 + f;
      const int64_t c = (pcol / 1024) * 1024 + marlin_perm(static_cast<int>(pcol % 1024));
      const int64_t n = (c / 256) * 16 + (c % 16), k = r * 16 + (c % 256) / 16;
      word |= (static_cast<uint32_t>(q[k * N + n]) & 0xFu) << (4 * f);
    }
    packed[i] = word;
  }
}

// out[g, c] = scale[g, (c / L) * L + scale_perm[c % L]]   (utils.py:84-88)
__global__ void __launch_bounds__(256) marlin_scale_perm_kernel(const __half* __restrict__ s, __half* __restrict__ out,
                                                                int64_t total, int L) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int p = static_cast<int>(i % L);
    out[i] = s[i - p + (L == 64 ? marlin_scale_perm64(p) : marlin_scale_perm32(p))];
  }
}

}  // namespace b200moe

using namespace b200moe;

#define DISPATCH_W(dtype, CALL)                                                     \
  switch (dtype) {                                                                  \
    case B200MOE_F32: { using T = float; CALL; break; }                             \
    case B200MOE_F16: { using T = __half; CALL; break; }                            \
    case B200MOE_BF16: { using T = __nv_bfloat16; CALL; break; }                    \
    default: return fail(B200MOE_BAD_DTYPE, "%s: dtype %d", __func__, dtype);       \
  }

extern "C" int b200moe_weight_quant_int8(const void* w, int w_dtype, void* y_int8, void* s_f16, int64_t M, int64_t N,
                                         float qmax, int rounding, void* stream) {
  B200MOE_REQUIRE(w && y_int8 && s_f16, B200MOE_BAD_ARG, "weight_quant_int8: null pointer");
  B200MOE_REQUIRE(M >= 0 && N >= 0, B200MOE_BAD_SHAPE, "weight_quant_int8: negative size");
  B200MOE_REQUIRE(qmax > 0.f && qmax <= 127.f && (rounding == 0 || rounding == 1), B200MOE_BAD_ARG,
                  "weight_quant_int8: qmax %g rounding %d", qmax, rounding);
  if (M == 0 || N == 0) return B200MOE_OK;
  const dim3 grid(static_cast<unsigned>((N + 127) / 128), static_cast<unsigned>((M + 127) / 128));
  B200MOE_REQUIRE(grid.y <= 65535, B200MOE_BAD_SHAPE, "weight_quant_int8: M too large");
  cudaStream_t st = as_stream(stream);
  DISPATCH_W(w_dtype, (weight_quant_int8_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(w), static_cast<int8_t*>(y_int8),
                                                                        static_cast<__half*>(s_f16), M, N, qmax, rounding)));
  return check_launch("weight_quant_int8");
}

extern "C" int b200moe_weight_dequant_int8(const void* x_int8, const void* s_f16, void* y, int y_dtype, int64_t M,
                                           int64_t N, void* stream) {
  B200MOE_REQUIRE(x_int8 && s_f16 && y, B200MOE_BAD_ARG, "weight_dequant_int8: null pointer");
  B200MOE_REQUIRE(M >= 0 && N >= 0, B200MOE_BAD_SHAPE, "weight_dequant_int8: negative size");
  if (M == 0 || N == 0) return B200MOE_OK;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((M * N + 255) / 256, 148 * 16));
  cudaStream_t st = as_stream(stream);
  DISPATCH_W(y_dtype, (weight_dequant_int8_kernel<T><<<grid, 256, 0, st>>>(static_cast<const int8_t*>(x_int8),
                                                                          static_cast<const __half*>(s_f16),
                                                                          static_cast<T*>(y), M, N)));
  return check_launch("weight_dequant_int8");
}

extern "C" int b200moe_weight_quant_w4a8(const void* w, int w_dtype, void* packed_i32, void* s_f16, int8_t* s4,
                                         int8_t* z4, int64_t M, int64_t N, void* stream) {
  B200MOE_REQUIRE(w && packed_i32 && s_f16 && s4 && z4, B200MOE_BAD_ARG, "weight_quant_w4a8: null pointer");
  B200MOE_REQUIRE(M >= 0 && N >= 0 && M % 128 == 0 && N % 128 == 0, B200MOE_BAD_SHAPE,
                  "weight_quant_w4a8: Last dimension size must be divisible by block_size (block_size=128) and the row "
                  "count by 128, got [%lld, %lld]", (long long)M, (long long)N);
  if (M == 0 || N == 0) return B200MOE_OK;
  const dim3 grid(static_cast<unsigned>(N / 128), static_cast<unsigned>(M / 128));
  B200MOE_REQUIRE(grid.y <= 65535, B200MOE_BAD_SHAPE, "weight_quant_w4a8: M too large");
  cudaStream_t st = as_stream(stream);
  DISPATCH_W(w_dtype, (weight_quant_w4a8_kernel<T><<<grid, 256, 0, st>>>(
      static_cast<const T*>(w), static_cast<uint32_t*>(packed_i32), static_cast<__half*>(s_f16), s4, z4, M, N)));
  return check_launch("weight_quant_w4a8");
}

extern "C" int b200moe_weight_quant_w4a16(const void* w, int w_dtype, void* packed_i32, void* scale_bf16,
                                          void* zero_bf16, int64_t rows, int64_t K, void* stream) {
  B200MOE_REQUIRE(w && packed_i32 && scale_bf16 && zero_bf16, B200MOE_BAD_ARG, "weight_quant_w4a16: null pointer");
  B200MOE_REQUIRE(rows >= 0 && K > 0 && K % 128 == 0, B200MOE_BAD_SHAPE,
                  "weight_quant_w4a16: K=%lld must be a multiple of 128", (long long)K);
  if (rows == 0) return B200MOE_OK;
  const int64_t warps = rows * (K / 128);
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((warps + 7) / 8, 148 * 32));
  cudaStream_t st = as_stream(stream);
  DISPATCH_W(w_dtype, (weight_quant_w4a16_kernel<T><<<grid, 256, 0, st>>>(
      static_cast<const T*>(w), static_cast<uint32_t*>(packed_i32), static_cast<__nv_bfloat16*>(scale_bf16),
      static_cast<__nv_bfloat16*>(zero_bf16), rows, K)));
  return check_launch("weight_quant_w4a16");
}

extern "C" int b200moe_marlin_pack(const int32_t* q, void* packed_i32, const void* scales_f16, void* scales_out_f16,
                                   int64_t K, int64_t N, int64_t groupsize, void* stream) {
  B200MOE_REQUIRE(q && packed_i32 && scales_f16 && scales_out_f16, B200MOE_BAD_ARG, "marlin_pack: null pointer");
  B200MOE_REQUIRE(K > 0 && N > 0 && K % 16 == 0 && N % 64 == 0, B200MOE_BAD_SHAPE,
                  "marlin_pack: Matrix dimensions not compatible with Marlin kernel requirements (K=%lld N=%lld)",
                  (long long)K, (long long)N);
  B200MOE_REQUIRE(groupsize == -1 || (groupsize > 0 && K % groupsize == 0), B200MOE_BAD_SHAPE,
                  "marlin_pack: Weight shape must be divisible by groupsize (K=%lld, groupsize=%lld)", (long long)K,
                  (long long)groupsize);
  cudaStream_t st = as_stream(stream);
  const int64_t total = (K / 16) * N * 2;
  marlin_pack_kernel<<<static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148 * 32)), 256, 0, st>>>(
      q, static_cast<uint32_t*>(packed_i32), K, N);
  const int64_t ns = (groupsize == -1 ? 1 : K / groupsize) * N;
  marlin_scale_perm_kernel<<<static_cast<unsigned>(std::min<int64_t>((ns + 255) / 256, 148 * 32)), 256, 0, st>>>(
      static_cast<const __half*>(scales_f16), static_cast<__half*>(scales_out_f16), ns, groupsize == -1 ? 32 : 64);
  return check_launch("marlin_pack");
}
