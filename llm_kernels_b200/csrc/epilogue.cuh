// Epilogue helpers shared by the tcgen05 GEMM kernels: row stores and the fused gate activations.
#pragma once

#include "common.cuh"

namespace b200moe {

template <typename T>
__device__ __forceinline__ void store_row64(T* dst, const float* v);
template <>
__device__ __forceinline__ void store_row64<float>(float* dst, const float* v) {
#pragma unroll
  for (int j = 0; j < 64; j += 4)
    *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
}
template <>
__device__ __forceinline__ void store_row64<__nv_bfloat16>(__nv_bfloat16* dst, const float* v) {
#pragma unroll
  for (int j = 0; j < 64; j += 8) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[j + 2 * i], v[j + 2 * i + 1]);
    *reinterpret_cast<uint4*>(dst + j) = r;
  }
}
template <>
__device__ __forceinline__ void store_row64<__half>(__half* dst, const float* v) {
#pragma unroll
  for (int j = 0; j < 64; j += 8) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[j + 2 * i], v[j + 2 * i + 1]);
    *reinterpret_cast<uint4*>(dst + j) = r;
  }
}

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Activation of the fused "act(gate) * up" epilogues, evaluated in f32 on the bf16-rounded gate value:
// act 0 = SiLU (moe/group_gemm_kernel.py:158-162), act 1 = tanh-GELU with tanh(x) = 2 sigmoid(2x) - 1 (:176-224).
__device__ __forceinline__ float gate_act(float g, int act) {
  if (act == 0) return g * __fdividef(1.0f, 1.0f + __expf(-g));
  const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  const float th = 2.f * __fdividef(1.0f, 1.0f + __expf(-2.f * inner)) - 1.f;
  return 0.5f * g * (1.f + th);
}

}  // namespace b200moe
