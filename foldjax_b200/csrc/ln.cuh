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

}  // namespace b200
