// The fixed permutations of the Marlin weight layout (fast_dequant/simple_marlin/utils.py:20-46), as functions:
// nothing is uploaded, so concurrent calls share no state.
#pragma once

namespace b200moe {

// Packed position i (0..1023) of a block of four 16x16 tiles holds element marlin_perm(i) of the block stored
// tile-major (tile * 256 + row * 16 + col).  Position i belongs to tensor-core lane i / 32, tile (i % 32) / 8; the
// eight nibbles of a word are the lane's values in the order [0, 2, 4, 6, 1, 3, 5, 7].
__host__ __device__ __forceinline__ int marlin_perm(int i) {
  const int lane = i >> 5, tile = (i >> 3) & 3, pos = i & 7;
  const int j = pos < 4 ? 2 * pos : 2 * (pos - 4) + 1;      // source slot of this nibble
  const int col = lane >> 2, quad = lane & 3;
  const int half = j >> 2, rr = j & 3;                      // rows of a lane: 2q, 2q+1, 2q+8, 2q+9
  const int row = 2 * quad + (rr & 1) + 8 * (rr >> 1);
  return 256 * tile + 16 * row + col + 8 * half;
}
// Scale columns are permuted in blocks of 64 (grouped) or 32 (one group): position p holds source column
// marlin_scale_perm*(p); marlin_scale_inv*(n) is the position that holds source column n.
__host__ __device__ __forceinline__ int marlin_scale_perm64(int p) { return (p >> 3) + 8 * (p & 7); }
__host__ __device__ __forceinline__ int marlin_scale_inv64(int n) { return 8 * (n & 7) + (n >> 3); }
__host__ __device__ __forceinline__ int marlin_scale_perm32(int p) {
  const int i = p >> 3, jj = p & 7;
  return 2 * i + 8 * (jj >> 1) + (jj & 1);
}
__host__ __device__ __forceinline__ int marlin_scale_inv32(int n) { return 8 * ((n & 7) >> 1) + 2 * (n >> 3) + (n & 1); }

}  // namespace b200moe
