// Host-side creation of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's
// driver entry point, so the library does not link libcuda).
#pragma once

#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace b200moe {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

inline EncodeFn get_tensor_map_encoder() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  }
  return fn;
}

// Byte matrix rows x cols with the given row stride; box = box_rows x 128 bytes, 128-byte swizzle,
// out-of-range elements read as zero.
inline int make_tensor_map_u8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols,
                              uint64_t row_stride, uint32_t box_rows) {
  EncodeFn enc = get_tensor_map_encoder();
  if (!enc) return fail(B200MOE_UNSUPPORTED_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                         box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200MOE_BAD_ARG, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return B200MOE_OK;
}

// Encoding a tensor map costs a few microseconds of host time and depends on nothing but its arguments, so the
// encoded maps are kept: the key is (base, rows, cols, row stride, box rows).  A layer's weights and workspaces
// keep their addresses from step to step, so every launch after the first finds its maps here.  The table is
// process-wide, mutex-protected, and simply cleared when it reaches 1024 entries.
struct TensorMapKey {
  const void* base; uint64_t rows, cols, stride; uint32_t box;
  bool operator==(const TensorMapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && stride == o.stride && box == o.box;
  }
};
struct TensorMapKeyHash {
  size_t operator()(const TensorMapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base);
    for (uint64_t v : {k.rows, k.cols, k.stride, static_cast<uint64_t>(k.box)}) h = (h ^ v) * 0x9E3779B97F4A7C15ull + (h >> 29);
    return static_cast<size_t>(h);
  }
};
inline int cached_tensor_map_u8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols,
                                uint64_t row_stride, uint32_t box_rows) {
  static std::mutex mu;
  static std::unordered_map<TensorMapKey, CUtensorMap, TensorMapKeyHash> table;
  const TensorMapKey key{base, rows, cols, row_stride, box_rows};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = table.find(key);
    if (it != table.end()) { *m = it->second; return B200MOE_OK; }
  }
  if (int rc = make_tensor_map_u8(m, base, rows, cols, row_stride, box_rows)) return rc;
  std::lock_guard<std::mutex> lock(mu);
  if (table.size() >= 1024) table.clear();
  table.emplace(key, *m);
  return B200MOE_OK;
}

// int32 matrix rows x cols (row stride in bytes); box = box_rows x box_cols words.  Without swizzle the tile lands
// in shared memory as plain [box_rows][box_cols] words; with it (box_cols must then be 32 words = 128 bytes) the
// 16-byte chunks of row r sit at chunk position (c ^ (r % 8)).
inline int make_tensor_map_i32_plain(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols,
                                     uint64_t row_stride, uint32_t box_cols, uint32_t box_rows, bool swizzle128 = false) {
  EncodeFn enc = get_tensor_map_encoder();
  if (!enc) return fail(B200MOE_UNSUPPORTED_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200MOE_BAD_ARG, "cuTensorMapEncodeTiled (int32) failed with %d", (int)r);
  return B200MOE_OK;
}

inline int require_sm100(int* sms) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(B200MOE_UNSUPPORTED_DEVICE, "no CUDA device");
  int major = 0;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev);
  if (major != 10)
    return fail(B200MOE_UNSUPPORTED_DEVICE, "tcgen05 kernels need compute capability 10.x, device has %d.x", major);
  return B200MOE_OK;
}

}  // namespace b200moe
