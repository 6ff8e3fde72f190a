// Bit packing of quantized weights: quantization/bitpack.py.
//   pack over rows  (:9-36, :228-293)   word r, field i  = w[e*r + i, c] << (nbits*i)
//   pack over cols  (:38-67, :84-149)   word c, field i  = w[r, e*c + i] << (nbits*i)
//   unpack          (:152-226, :296-373) inverse, to uint8
// e = width / nbits fields per word.  Offline, HBM-bound, one word per thread.
#include "common.cuh"

namespace b200moe {

template <typename W>
__global__ void __launch_bounds__(256) pack_kernel(const uint8_t* __restrict__ w, W* __restrict__ out,
                                                   int64_t out_rows, int64_t out_cols, int64_t C,
                                                   int nbits, int e, int over_rows) {
  const int64_t total = out_rows * out_cols;
  const uint32_t mask = (1u << nbits) - 1u;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / out_cols, c = i - r * out_cols;
    uint32_t word = 0;
    for (int f = 0; f < e; ++f) {
      const uint8_t v = over_rows ? w[(r * e + f) * C + c] : w[r * C + c * e + f];
      word |= (static_cast<uint32_t>(v) & mask) << (nbits * f);
    }
    out[i] = static_cast<W>(word);
  }
}

template <typename W>
__global__ void __launch_bounds__(256) unpack_kernel(const W* __restrict__ packed, uint8_t* __restrict__ out,
                                                     int64_t R, int64_t C, int nbits, int e,
                                                     int over_rows) {
  const int64_t total = R * C;
  const uint32_t mask = (1u << nbits) - 1u;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / C, c = i - r * C;
    uint32_t word; int f;
    if (over_rows) { word = static_cast<uint32_t>(packed[(r / e) * C + c]); f = static_cast<int>(r % e); }
    else { word = static_cast<uint32_t>(packed[r * (C / e) + c / e]); f = static_cast<int>(c % e); }
    out[i] = static_cast<uint8_t>((word >> (nbits * f)) & mask);
  }
}

static int check_bits(const char* who, int64_t R, int64_t C, int nbits, int width, int over_rows) {
  B200MOE_REQUIRE(nbits == 1 || nbits == 2 || nbits == 4 || nbits == 8, B200MOE_BAD_ARG, "%s: Unsuported nbits %d", who, nbits);
  B200MOE_REQUIRE(width == 8 || width == 16 || width == 32, B200MOE_BAD_ARG, "%s: Unsuported bitpacking width %d", who, width);
  B200MOE_REQUIRE(R >= 0 && C >= 0, B200MOE_BAD_SHAPE, "%s: negative size", who);
  const int e = width / nbits;
  B200MOE_REQUIRE((over_rows ? R : C) % e == 0, B200MOE_BAD_SHAPE, "%s: %s must be divisible by %d",
                  who, over_rows ? "rows" : "cols", e);
  return B200MOE_OK;
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_pack_bits(const uint8_t* w, void* out, int64_t R, int64_t C, int nbits,
                                 int width, int over_rows, void* stream) {
  if (int rc = check_bits("pack_bits", R, C, nbits, width, over_rows)) return rc;
  if (R == 0 || C == 0) return B200MOE_OK;
  B200MOE_REQUIRE(w && out, B200MOE_BAD_ARG, "pack_bits: null pointer");
  const int e = width / nbits;
  const int64_t orows = over_rows ? R / e : R, ocols = over_rows ? C : C / e;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((orows * ocols + 255) / 256, 148 * 32));
  cudaStream_t st = as_stream(stream);
  if (width == 8) pack_kernel<uint8_t><<<grid, 256, 0, st>>>(w, static_cast<uint8_t*>(out), orows, ocols, C, nbits, e, over_rows);
  else if (width == 16) pack_kernel<uint16_t><<<grid, 256, 0, st>>>(w, static_cast<uint16_t*>(out), orows, ocols, C, nbits, e, over_rows);
  else pack_kernel<uint32_t><<<grid, 256, 0, st>>>(w, static_cast<uint32_t*>(out), orows, ocols, C, nbits, e, over_rows);
  return check_launch("pack_bits");
}

extern "C" int b200moe_unpack_bits(const void* packed, uint8_t* out, int64_t R, int64_t C, int nbits,
                                   int width, int over_rows, void* stream) {
  if (int rc = check_bits("unpack_bits", R, C, nbits, width, over_rows)) return rc;
  if (R == 0 || C == 0) return B200MOE_OK;
  B200MOE_REQUIRE(packed && out, B200MOE_BAD_ARG, "unpack_bits: null pointer");
  const int e = width / nbits;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((R * C + 255) / 256, 148 * 32));
  cudaStream_t st = as_stream(stream);
  if (width == 8) unpack_kernel<uint8_t><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(packed), out, R, C, nbits, e, over_rows);
  else if (width == 16) unpack_kernel<uint16_t><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(packed), out, R, C, nbits, e, over_rows);
  else unpack_kernel<uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(packed), out, R, C, nbits, e, over_rows);
  return check_launch("unpack_bits");
}
