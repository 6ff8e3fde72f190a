// int4 weight formats: expansion to the tensor-core operand types.
//
//   two-level int4 (quantization/w4a8_kernel.py:44-101, 196-309): packed int32 [N/8, K] (8 output
//   channels per word, quantization/bitpack.py:9-36), s4/z4 int8 [N, K/128]:
//       w8[n,k] = int8( (q[n,k] - z4[n,k/128]) * s4[n,k/128] )         (int8 wrap as the reference)
//   asymmetric group-128 int4 (extension of fast_dequant/simple_marlin/utils.py:98-136): packed
//   int32 [N, K/8] (8 consecutive k per word, quantization/bitpack.py:38-67), scale/zero bf16
//   [N, K/128]:  w[n,k] = bf16( (q - zero) * scale )
// Both are HBM-bound one-pass kernels over a stack of W matrices.
#include "common.cuh"
#include "marlin_perm.cuh"

namespace b200moe {

// one thread: 4 consecutive k of one packed row -> 8 rows x 4 int8
__global__ void __launch_bounds__(256) w4a8_expand_kernel(const uint32_t* __restrict__ packed,
                                                          const int8_t* __restrict__ s4,
                                                          const int8_t* __restrict__ z4,
                                                          int8_t* __restrict__ out, int64_t W,
                                                          int64_t N, int64_t K) {
  const int64_t k4 = K / 4, n8 = N / 8, kg = K / 128;
  const int64_t total = W * n8 * k4;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t kq = i % k4, r = (i / k4) % n8, w = i / (k4 * n8);
    const uint4 words = *reinterpret_cast<const uint4*>(packed + (w * n8 + r) * K + kq * 4);
    const uint32_t wv[4] = {words.x, words.y, words.z, words.w};
    const int64_t g = (kq * 4) / 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int64_t n = r * 8 + c;
      const int s = s4[(w * N + n) * kg + g], z = z4[(w * N + n) * kg + g];
      uint32_t o = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int qv = static_cast<int>((wv[j] >> (4 * c)) & 0xF);
        o |= (static_cast<uint32_t>((qv - z) * s) & 0xFFu) << (8 * j);
      }
      *reinterpret_cast<uint32_t*>(out + (w * N + n) * K + kq * 4) = o;
    }
  }
}

// one thread: one packed word = 8 consecutive k of one row -> 8 bf16
__global__ void __launch_bounds__(256) w4a16_expand_kernel(const uint32_t* __restrict__ packed,
                                                           const __nv_bfloat16* __restrict__ scale,
                                                           const __nv_bfloat16* __restrict__ zero,
                                                           __nv_bfloat16* __restrict__ out,
                                                           int64_t rows, int64_t K) {
  const int64_t k8 = K / 8, kg = K / 128;
  const int64_t total = rows * k8;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / k8, kw = i - r * k8;
    const uint32_t word = packed[i];
    const float sc = __bfloat162float(scale[r * kg + (kw * 8) / 128]);
    const float zp = __bfloat162float(zero[r * kg + (kw * 8) / 128]);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (static_cast<float>((word >> (4 * j)) & 0xF) - zp) * sc;
    store8(out + r * K + kw * 8, v);
  }
}

// Marlin-order symmetric int4 (fast_dequant/simple_marlin/utils.py:53-95): packed int32
// [K/16, N*16/8].  A packed row holds one 16-row k-tile, tiles of 16 x 16 flattened as
// n_tile*256 + k_in*16 + n_in, permuted in blocks of 1024 by `perm` (packed position i holds
// element perm[i]) and packed 8 nibbles per word.  Scales f16 [K/g, N] are permuted in blocks of
// 64 (grouped) or 32 (one group) columns; both permutations are closed forms (marlin_perm.cuh), so calls
// share no state.  One thread expands one word into
// out[n, k] = (q - 8) * s[k/g, n]  (f16, nn.Linear layout [N, K]).
__global__ void __launch_bounds__(256) marlin_expand_kernel(const uint32_t* __restrict__ packed,
                                                            const __half* __restrict__ s,
                                                            __half* __restrict__ out, int64_t K,
                                                            int64_t N, int64_t groupsize, int L) {
  const int64_t words_per_row = N * 2;
  const int64_t total = (K / 16) * words_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / words_per_row, j = i - r * words_per_row;
    const uint32_t word = packed[i];
#pragma unroll
    for (int f = 0; f < 8; ++f) {
      const int64_t pcol = j * 8 + f;
      const int64_t c = (pcol / 1024) * 1024 + marlin_perm(static_cast<int>(pcol % 1024));
      const int64_t n = (c / 256) * 16 + (c % 16);
      const int64_t k = r * 16 + (c % 256) / 16;
      const int64_t g = groupsize > 0 ? k / groupsize : 0;
      const float sc = __half2float(s[g * N + (n / L) * L + (L == 64 ? marlin_scale_inv64(static_cast<int>(n % L)) : marlin_scale_inv32(static_cast<int>(n % L)))]);
      const int q = static_cast<int>((word >> (4 * f)) & 0xF);
      out[n * K + k] = __float2half_rn(static_cast<float>(q - 8) * sc);
    }
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_marlin_expand_f16(const void* packed, const void* scales_f16, void* out_f16,
                                         int64_t K, int64_t N, int64_t groupsize, void* stream) {
  B200MOE_REQUIRE(packed && scales_f16 && out_f16, B200MOE_BAD_ARG, "marlin_expand_f16: null pointer");
  B200MOE_REQUIRE(K > 0 && N > 0 && K % 16 == 0 && N % 64 == 0 && (N * 16) % 1024 == 0, B200MOE_BAD_SHAPE,
                  "marlin_expand_f16: Matrix dimensions not compatible with Marlin kernel requirements (K=%lld N=%lld)",
                  (long long)K, (long long)N);
  B200MOE_REQUIRE(groupsize == -1 || (groupsize > 0 && K % groupsize == 0), B200MOE_BAD_SHAPE,
                  "marlin_expand_f16: K dimension not divisible by groupsize: K=%lld, groupsize=%lld", (long long)K, (long long)groupsize);
  cudaStream_t st = as_stream(stream);
  const int scale_perm_len = groupsize == -1 ? 32 : 64;
  const int64_t total = (K / 16) * N * 2;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148 * 32));
  marlin_expand_kernel<<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(packed), static_cast<const __half*>(scales_f16),
                                             static_cast<__half*>(out_f16), K, N, groupsize, scale_perm_len);
  return check_launch("marlin_expand_f16");
}

extern "C" int b200moe_w4a8_expand_int8(const void* packed, const int8_t* s4, const int8_t* z4, void* out,
                                        int64_t W, int64_t N, int64_t K, void* stream) {
  B200MOE_REQUIRE(packed && s4 && z4 && out, B200MOE_BAD_ARG, "w4a8_expand_int8: null pointer");
  B200MOE_REQUIRE(W >= 0 && N > 0 && K > 0 && N % 8 == 0 && K % 128 == 0, B200MOE_BAD_SHAPE,
                  "w4a8_expand_int8: N=%lld must be a multiple of 8 and K=%lld of 128", (long long)N, (long long)K);
  B200MOE_REQUIRE(aligned(packed, 16) && aligned(out, 4), B200MOE_BAD_ALIGN, "w4a8_expand_int8: alignment");
  if (W == 0) return B200MOE_OK;
  const int64_t total = W * (N / 8) * (K / 4);
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148 * 32));
  w4a8_expand_kernel<<<grid, 256, 0, as_stream(stream)>>>(static_cast<const uint32_t*>(packed), s4, z4,
                                                          static_cast<int8_t*>(out), W, N, K);
  return check_launch("w4a8_expand_int8");
}

extern "C" int b200moe_w4a16_expand_bf16(const void* packed, const void* scale_bf16, const void* zero_bf16,
                                         void* out_bf16, int64_t rows, int64_t K, void* stream) {
  B200MOE_REQUIRE(packed && scale_bf16 && zero_bf16 && out_bf16, B200MOE_BAD_ARG, "w4a16_expand_bf16: null pointer");
  B200MOE_REQUIRE(rows >= 0 && K > 0 && K % 128 == 0, B200MOE_BAD_SHAPE, "w4a16_expand_bf16: K=%lld must be a multiple of 128", (long long)K);
  B200MOE_REQUIRE(aligned(out_bf16, 16), B200MOE_BAD_ALIGN, "w4a16_expand_bf16: alignment");
  if (rows == 0) return B200MOE_OK;
  const int64_t total = rows * (K / 8);
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148 * 32));
  w4a16_expand_kernel<<<grid, 256, 0, as_stream(stream)>>>(static_cast<const uint32_t*>(packed),
                                                           static_cast<const __nv_bfloat16*>(scale_bf16),
                                                           static_cast<const __nv_bfloat16*>(zero_bf16),
                                                           static_cast<__nv_bfloat16*>(out_bf16), rows, K);
  return check_launch("w4a16_expand_bf16");
}
