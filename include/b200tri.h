/* libb200tri - C ABI of the B200 (sm_100a) triangle-op backend.
 *
 * Plain C: device pointers, sizes, POD argument structs, a CUDA stream and an
 * int status. No allocation happens inside any entry point: every call works in
 * a caller-provided workspace whose size the matching *_workspace_bytes()
 * reports. All entry points only enqueue work on `stream` (no host sync), so an
 * XLA FFI handler can forward to them directly.
 *
 * "Reference" below is eightmm/FoldJAX; paths are relative to its root.
 *
 * Layout conventions (device memory, bf16 unless noted):
 *   pair tensor  x[n, n, 128]   channel-last, dense
 *   mask         float32 [n, n] (1 keep / 0 drop), may be NULL (= ones)
 *   linear kernels in the reference's [in, out] layout, no biases
 *   layer-norm scale/bias [128]
 */
#ifndef B200TRI_H_
#define B200TRI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* b200tri_stream_t; /* == cudaStream_t */

enum {
  B200TRI_OK = 0,
  B200TRI_ERR_INVALID = 1,     /* bad argument (null pointer, alignment, size) */
  B200TRI_ERR_UNSUPPORTED = 2, /* shape/dtype this build has no kernel for    */
  B200TRI_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed           */
  B200TRI_ERR_TIMEOUT = 4,     /* a kernel gave up on a bounded device wait   */
  B200TRI_ERR_WORKSPACE = 5    /* workspace missing or too small              */
};

/* Library version (major*10000 + minor*100 + patch). */
int b200tri_version(void);
/* Message of the last failing call made by this thread. */
const char* b200tri_last_error(void);
/* Synchronises the current device, returns the device status word (0 = fine,
 * >100 = the role whose bounded wait ran out) and clears it. */
int b200tri_device_status(void);

/* ------------------------------------------------------------------------
 * Triangle multiplicative update.
 * Replaces: triangle_multiplication_forward,
 *   src/foldjax/models/boltz2/models/triangle/triangle.py:33-129, and the fused
 *   call it can dispatch to, cueq_triangle_multiplication_forward,
 *   src/foldjax/models/boltz2/models/triangle/triangle_cueq.py:72-102.
 * Computes  update = LN_out(contract(a, b)) @ p_out * sigmoid(LN_in(x) @ g_out)
 * with [a | b] = sigmoid(LN_in(x) @ g_in) * (LN_in(x) @ p_in) * mask,
 * outgoing: contract[i,j,d] = sum_k a[i,k,d] b[j,k,d]
 * incoming: contract[i,j,d] = sum_k a[k,i,d] b[k,j,d].
 * If `residual` is not NULL the kernel writes residual + update (the caller's
 * add at src/foldjax/models/boltz2/models/trunk_blocks/pairformer.py:133-142).
 * --------------------------------------------------------------------- */
typedef struct {
  int32_t n;        /* tokens */
  int32_t incoming; /* 0 = outgoing, 1 = incoming */
  float eps;        /* layer-norm epsilon (reference default 1e-5) */
  const void* x;    /* [n, n, 128] bf16 */
  const float* mask;
  const void* norm_in_scale;
  const void* norm_in_bias;
  const void* p_in;  /* [128, 256] */
  const void* g_in;  /* [128, 256] */
  const void* norm_out_scale;
  const void* norm_out_bias;
  const void* p_out; /* [128, 128] */
  const void* g_out; /* [128, 128] */
  const void* residual; /* optional [n, n, 128] */
  void* out;            /* [n, n, 128] */
  void* workspace;
  size_t workspace_bytes;
} b200tri_trimul_args;

size_t b200tri_trimul_workspace_bytes(int32_t n);
int b200tri_trimul_forward(const b200tri_trimul_args* args, b200tri_stream_t stream);

/* The three stages of the update, exposed so that the 2-D context-parallel
 * layer can exchange tiles between them (the reference's _cannon_contract,
 * triangle.py:132-212, sits between its projection and its output stage).
 *
 * project: reads a tile of x and writes a and b channel-major,
 *   a[d][o][t] with o in [0,n_outer), t in [0,n_inner), row pitch `ld`.
 *   The pair feeding (o,t) is x[o*xs_outer + t*xs_inner ...] (element strides),
 *   so the incoming direction is the same kernel with the two strides swapped.
 *   Rows are grouped in blocks of `rows_per_block`; element (d,o,t) lives at
 *   (o / rows_per_block) * block_stride + d * chan_stride + (o % rows_per_block) * ld + t.
 */
typedef struct {
  int32_t n_outer, n_inner;
  float eps;
  const void* x;
  int64_t xs_outer, xs_inner; /* element strides of x (multiples of 128) */
  const float* mask;          /* NULL = ones */
  int64_t ms_outer, ms_inner;
  const void* norm_in_scale;
  const void* norm_in_bias;
  const void* p_in;
  const void* g_in;
  void* a;
  void* b;
  int64_t ld, chan_stride, block_stride;
  int32_t rows_per_block;
  void* workspace; /* b200tri_trimul_project_workspace_bytes() */
  size_t workspace_bytes;
} b200tri_trimul_project_args;

size_t b200tri_trimul_project_workspace_bytes(void);
int b200tri_trimul_project(const b200tri_trimul_project_args* args, b200tri_stream_t stream);

/* contract: t[d][i][j] = sum over sources s and k of a[s][d][i][k] * b[s][d][j][k]
 * for 128 channels d, fp32 accumulation on the tensor cores. `acc_in` (fp32,
 * same indexing as the outputs) is added when not NULL; the result goes to
 * `out_f32` and/or `out_bf16` (rounded once). Replaces _chunked_triangle_einsum,
 * triangle.py:215-254. */
typedef struct {
  int32_t n_i, n_j, n_k, n_src;
  const void* a;
  int64_t a_ld, a_chan_stride, a_src_stride; /* elements */
  const void* b;
  int64_t b_ld, b_chan_stride, b_src_stride;
  const float* acc_in;
  float* out_f32;
  void* out_bf16;
  int64_t out_ld, out_chan_stride;
} b200tri_trimul_contract_args;

int b200tri_trimul_contract(const b200tri_trimul_contract_args* args, b200tri_stream_t stream);

/* finish: out[i][j][:] = LN_out(t[:, i, j]) @ p_out * sigmoid(LN_in(x[i][j]) @ g_out)
 * (+ residual). t is channel-major bf16 with row pitch t_ld. */
typedef struct {
  int32_t n_i, n_j;
  float eps;
  const void* t;
  int64_t t_ld, t_chan_stride;
  const void* x;
  int64_t xs_i, xs_j;
  const void* norm_in_scale;
  const void* norm_in_bias;
  const void* norm_out_scale;
  const void* norm_out_bias;
  const void* p_out;
  const void* g_out;
  const void* residual; /* optional, indexed like out */
  void* out;
  int64_t os_i, os_j; /* element strides of out / residual */
  void* workspace;
  size_t workspace_bytes;
} b200tri_trimul_finish_args;

size_t b200tri_trimul_finish_workspace_bytes(void);
int b200tri_trimul_finish(const b200tri_trimul_finish_args* args, b200tri_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200TRI_H_ */
