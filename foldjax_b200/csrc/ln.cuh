// Layer norm of one 128-channel pair held in a K-major, 128-byte-swizzled
// operand tile (two 16 KiB slabs of 64 channels; row = pair). One thread owns
// one row: it reads its 256 bytes, computes the statistics in fp32 exactly as
// the reference does (mean, then mean of squared deviations, rsqrt(var + eps);
// src/foldjax/models/boltz2/models/primitives/_common.py:15-26), rounds the
// normalised value to bf16 before the affine step like the reference, and
// writes the result back in place, so the tile TMA delivered becomes the
// tensor-core operand without a second buffer.
#pragma once
#include "tc.cuh"

namespace b200 {

constexpr int SLAB_BYTES = 128 * 128;  // 128 rows x 64 bf16

// v[0..7] = slab 0 chunks, v[8..15] = slab 1 chunks (16 bytes = 8 channels each).
__device__ __forceinline__ void ln_load_row(const uint8_t* tile, int row, uint4 (&v)[16]) {
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int c = 0; c < 8; ++c) v[s * 8 + c] = *reinterpret_cast<const uint4*>(tile + s * SLAB_BYTES + sw128_offset(row, c));
}

__device__ __forceinline__ void ln_store_row(uint8_t* tile, int row, const uint4 (&v)[16]) {
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(tile + s * SLAB_BYTES + sw128_offset(row, c)) = v[s * 8 + c];
}

// In-register layer norm of the 128 bf16 values packed in v. gamma2/beta2 are
// the scale and bias as 64 packed bf16 pairs in shared memory (every thread
// reads the same address, a broadcast).
__device__ __forceinline__ void ln_rows_inplace(uint4 (&v)[16], const uint32_t* gamma2, const uint32_t* beta2,
                                                float eps) {
  uint32_t* w = reinterpret_cast<uint32_t*>(v);  // 64 words, 2 channels each
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 64; ++i) sum += bf16_lo(w[i]) + bf16_hi(w[i]);
  const float mean = sum * (1.0f / 128.0f);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    const float a = bf16_lo(w[i]) - mean, b = bf16_hi(w[i]) - mean;
    sq = fmaf(a, a, sq);
    sq = fmaf(b, b, sq);
  }
  const float rstd = rsqrtf(sq * (1.0f / 128.0f) + eps);
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    const float a = (bf16_lo(w[i]) - mean) * rstd;
    const float b = (bf16_hi(w[i]) - mean) * rstd;
    // normed.astype(bf16) * scale + bias, each step rounded to bf16
    w[i] = bf16x2_add(bf16x2_mul(pack_bf16x2(a, b), gamma2[i]), beta2[i]);
  }
}

// The same layer norm (same operations in the same order, so the same bits) as three
// sweeps over the row in shared memory - mean, variance, normalise - holding four words
// at a time instead of the whole row: for kernels whose other roles leave the
// layer-norm warps few registers.
__device__ __forceinline__ void ln_row_sweeps(uint8_t* tile, int row, const uint32_t* gamma2, const uint32_t* beta2,
                                              float eps) {
  float sum = 0.f;
#pragma unroll 4
  for (int c = 0; c < 16; ++c) {
    const uint4 v = *reinterpret_cast<const uint4*>(tile + (c >> 3) * SLAB_BYTES + sw128_offset(row, c & 7));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) sum += bf16_lo(w[e]) + bf16_hi(w[e]);
  }
  const float mean = sum * (1.0f / 128.0f);
  float sq = 0.f;
#pragma unroll 4
  for (int c = 0; c < 16; ++c) {
    const uint4 v = *reinterpret_cast<const uint4*>(tile + (c >> 3) * SLAB_BYTES + sw128_offset(row, c & 7));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = bf16_lo(w[e]) - mean, b = bf16_hi(w[e]) - mean;
      sq = fmaf(a, a, sq);
      sq = fmaf(b, b, sq);
    }
  }
  const float rstd = rsqrtf(sq * (1.0f / 128.0f) + eps);
#pragma unroll 4
  for (int c = 0; c < 16; ++c) {
    uint4* ptr = reinterpret_cast<uint4*>(tile + (c >> 3) * SLAB_BYTES + sw128_offset(row, c & 7));
    const uint4 v = *ptr;
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = (bf16_lo(w[e]) - mean) * rstd, b = (bf16_hi(w[e]) - mean) * rstd;
      w[e] = bf16x2_add(bf16x2_mul(pack_bf16x2(a, b), gamma2[4 * c + e]), beta2[4 * c + e]);
    }
    *ptr = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Two threads per row: lanes l and l ^ 16 of a warp share row (l & 15) of the warp's 16
// rows; `half` = l >> 4 takes the 64 channels of slab `half`, and the two partial sums
// meet through one shuffle each. Half the instructions and half the dependency chain
// per thread, and twice the warps: the layer norm is what a projection tile waits for.
// Must be called by all 32 lanes of the warp. Same rounding points as ln_rows_inplace;
// the fp32 statistics are summed in a different order (four partial sums per thread).
__device__ __forceinline__ void ln_row_two_threads(uint8_t* tile, int row, int half, const uint32_t* gamma2,
                                                   const uint32_t* beta2, float eps) {
  uint4 v[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const uint4*>(tile + half * SLAB_BYTES + sw128_offset(row, c));
  uint32_t* w = reinterpret_cast<uint32_t*>(v);  // 32 words, 2 channels each
  float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 32; ++i) s4[i & 3] += bf16_lo(w[i]) + bf16_hi(w[i]);
  float sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
  sum += __shfl_xor_sync(0xffffffffu, sum, 16);
  const float mean = sum * (1.0f / 128.0f);
  float q4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float a = bf16_lo(w[i]) - mean, b = bf16_hi(w[i]) - mean;
    q4[i & 3] = fmaf(a, a, q4[i & 3]);
    q4[i & 3] = fmaf(b, b, q4[i & 3]);
  }
  float sq = (q4[0] + q4[1]) + (q4[2] + q4[3]);
  sq += __shfl_xor_sync(0xffffffffu, sq, 16);
  const float rstd = rsqrtf(sq * (1.0f / 128.0f) + eps);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float a = (bf16_lo(w[i]) - mean) * rstd, b = (bf16_hi(w[i]) - mean) * rstd;
    w[i] = bf16x2_add(bf16x2_mul(pack_bf16x2(a, b), gamma2[half * 32 + i]), beta2[half * 32 + i]);
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(tile + half * SLAB_BYTES + sw128_offset(row, c)) = v[c];
}

}  // namespace b200
