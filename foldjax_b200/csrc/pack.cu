// Parameter repacking kernels (see pack.cuh).
#include "pack.cuh"

#include "host.cuh"

namespace b200 {

namespace {
__global__ void pack_transpose_kernel(const __nv_bfloat16* __restrict__ src, int src_ld, int col0, int ncols,
                                      __nv_bfloat16* __restrict__ dst, float scale) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= ncols * 128) return;
  const int o = idx >> 7, c = idx & 127;
  const float v = __bfloat162float(src[static_cast<long long>(c) * src_ld + col0 + o]);
  dst[idx] = (scale == 1.0f) ? src[static_cast<long long>(c) * src_ld + col0 + o] : __float2bfloat16_rn(v * scale);
}
__global__ void pack_zero_kernel(__nv_bfloat16* dst, int count) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < count) dst[idx] = __float2bfloat16_rn(0.f);
}
__global__ void pack_copy_words_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int n) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n) dst[idx] = src[idx];
}
}  // namespace

void pack_transpose(const __nv_bfloat16* src, int src_ld, int col0, int ncols, __nv_bfloat16* dst,
                    cudaStream_t stream, float scale) {
  const int total = ncols * 128;
  count_launch();
  pack_transpose_kernel<<<(total + 255) / 256, 256, 0, stream>>>(src, src_ld, col0, ncols, dst, scale);
}
void pack_zero(__nv_bfloat16* dst, int count, cudaStream_t stream) {
  count_launch();
  pack_zero_kernel<<<(count + 255) / 256, 256, 0, stream>>>(dst, count);
}
void pack_copy_words(const void* src, void* dst, int nwords, cudaStream_t stream) {
  count_launch();
  pack_copy_words_kernel<<<(nwords + 255) / 256, 256, 0, stream>>>(static_cast<const uint32_t*>(src),
                                                                   static_cast<uint32_t*>(dst), nwords);
}

}  // namespace b200
