// Small device-side repacking of the reference's parameter layouts into the
// K-major form the tensor-core kernels read. The reference stores linear
// kernels as [in, out] (x @ kernel); tcgen05 wants each output channel's 128
// input weights contiguous, i.e. [out, in].
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// dst[o * 128 + c] = src[c * src_ld + col0 + o] * scale   for o in [0, ncols), c in [0, 128).
void pack_transpose(const __nv_bfloat16* src, int src_ld, int col0, int ncols, __nv_bfloat16* dst,
                    cudaStream_t stream, float scale = 1.0f);
// Zero-fill `count` bf16 elements.
void pack_zero(__nv_bfloat16* dst, int count, cudaStream_t stream);
// Copy `nwords` 32-bit words device-to-device.
void pack_copy_words(const void* src, void* dst, int nwords, cudaStream_t stream);

}  // namespace b200
