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

/* Element type of the pair tensor, the parameters and the result of the two triangle ops.
 * BF16 is the throughput mode (bf16 storage, float32 accumulation, the reference's bf16
 * trunk); F32 is the float32 trunk of the reference - every step in float32, the triangle
 * contraction as split-bf16 products accumulated in float32 on the tensor cores - and meets
 * its 1e-4 tolerance. */
enum { B200TRI_DTYPE_BF16 = 0, B200TRI_DTYPE_F32 = 1 };

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

/* Failure-detection self-test. Every wait inside the library's kernels (on an mbarrier
 * fed by TMA, by the tensor core or by another warp) is bounded: when it runs out, the
 * kernel records which role gave up in the device status word, drains, frees its tensor
 * memory and returns, so the context stays usable and the host learns of it from
 * b200tri_device_status(). This entry exercises that path on purpose and harmlessly: it
 * enqueues a one-warp kernel that waits, through the same code, on a barrier nothing ever
 * arrives at, for at most `limit_cycles` SM clock cycles (about 2e6 per millisecond). The
 * next b200tri_device_status() then reports code 110 and clears it. The reference's
 * counterpart is the host-side refusal of a half-delivered exchange
 * (src/foldjax/models/_cp.py:199-256); it has no device-side waits of its own. */
int b200tri_selftest_wait(int64_t limit_cycles, b200tri_stream_t stream);

/* Measurement aids (not on the data path).
 * b200tri_launch_count: kernels launched by this library in this process so far.
 * b200tri_timing_enable(1): from now on the library brackets each of its main
 *   kernels with CUDA events on the launching stream. b200tri_timing_read
 *   synchronises the device and returns, for a kernel name ("trimul_project",
 *   "trimul_contract", "trimul_finish", "triatt_project", "triatt_core",
 *   "triatt_finish", "pair_transition", "pair_bias"; "cp_exchange" = the tile-exchange groups of the
 *   context-parallel ops, timed on the exchange stream, and inside them "cp_ready" = the wait for
 *   the peers' tiles, "cp_copy" = the copies plus the closing token round), the summed duration in ms and the number of launches since
 *   the last b200tri_timing_reset. Off by default. */
uint64_t b200tri_launch_count(void);
/* The persistent kernels launch one CTA per SM. b200tri_set_sm_limit(n) makes
 * them use at most n SMs (0 = all) on the CURRENT device, which leaves SMs to a
 * communication library whose kernels run beside them (NCCL send/recv during a tile
 * exchange). The limit and the timing switch below are kept per device, so host threads
 * that each drive one device do not disturb one another. */
int b200tri_set_sm_limit(int32_t sms);
int b200tri_timing_enable(int32_t on);
int b200tri_timing_reset(void);
int b200tri_timing_read(const char* kernel, double* total_ms, int32_t* launches);
/* The same records one by one, in launch order: up to `capacity` durations into ms[], their
 * number into *count. */
int b200tri_timing_list(const char* kernel, double* ms, int32_t capacity, int32_t* count);

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
  int32_t dtype; /* B200TRI_DTYPE_*: type of x, mask excepted (always float32), of every
                    parameter, of residual and of out. 0 = bf16. */
  /* Channel counts, 0 = 128: x is [n, n, c_z]; p_in / g_in [c_z, 2 * c_hidden]; norm_out
   * [c_hidden]; p_out [c_hidden, c_z]; g_out [c_z, c_z]. c_z = c_hidden = 128 in bf16 runs the
   * tensor-core kernels end to end; any other shape (the template stacks' c_z = 64 with
   * c_hidden = 128, the 384-channel refiner) or float32 runs the general path: CUDA-core
   * stages around the tensor-core contraction. Multiples of 8, up to 1024. */
  int32_t c_z, c_hidden;
} b200tri_trimul_args;

size_t b200tri_trimul_workspace_bytes(int32_t n); /* bf16, 128 channels */
size_t b200tri_trimul_workspace_bytes_dtype(int32_t n, int32_t dtype); /* 128 channels */
size_t b200tri_trimul_workspace_bytes_shape(int32_t n, int32_t dtype, int32_t c_z, int32_t c_hidden);
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
  /* Optional row blocking (0 = one block): row i of an operand lives at
   * (i / rows_per_block) * block_stride + d * chan_stride + (i % rows_per_block) * ld.
   * Blocks keep the 128 channel planes of a tile close together in memory, which is
   * what the projection stage's stores want. a needs rows_per_block dividing or a
   * multiple of 128, b of 256. */
  int32_t a_rows_per_block, b_rows_per_block, out_rows_per_block;
  int64_t a_block_stride, b_block_stride, out_block_stride;
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
  int32_t t_rows_per_block; /* optional row blocking of t (0 = one block), as in contract */
  int64_t t_block_stride;
} b200tri_trimul_finish_args;

size_t b200tri_trimul_finish_workspace_bytes(void);
int b200tri_trimul_finish(const b200tri_trimul_finish_args* args, b200tri_stream_t stream);

/* ------------------------------------------------------------------------
 * Triangle attention (starting / ending node).
 * Replaces: triangle_attention_forward,
 *   src/foldjax/models/boltz2/models/triangle/triangle_attention.py:79-162,
 *   including _attention (:346-425) and the fused attention cores it can
 *   dispatch to: pallas_attention_core (triangle_attention_pallas.py:180),
 *   tokamax_attention_core (triangle_attention_tokamax.py:42) and
 *   cueq_attention_core (src/foldjax/models/_cueq.py:66-121).
 * Parameters in the reference's layout: layer_norm scale/bias [128]; `linear`
 * (pair bias) [128, 4]; linear_q/k/v/g [128, 128] with heads-major columns;
 * linear_o [128, 128] (other shapes: see c_z below). starting = 0 computes the ending node: the same
 * attention on the transposed pair tensor and mask, result transposed back.
 * If `residual` is not NULL the kernel writes residual + update.
 * --------------------------------------------------------------------- */
typedef struct {
  int32_t n;
  int32_t starting; /* 1 = starting node, 0 = ending node */
  int32_t heads;    /* 4 */
  int32_t head_dim; /* 32 */
  float inf;        /* mask constant (reference default 1e9) */
  float eps;
  const void* x; /* [n, n, 128] bf16 */
  const float* mask;
  const void* norm_scale;
  const void* norm_bias;
  const void* w_bias; /* params["linear"]["kernel"] */
  const void* w_q;
  const void* w_k;
  const void* w_v;
  const void* w_g;
  const void* w_o;
  const void* residual;
  void* out;
  void* workspace;
  size_t workspace_bytes;
  int32_t dtype; /* B200TRI_DTYPE_*, as in b200tri_trimul_args */
  /* 0 = 128. x is [n, n, c_z]; linear (w_bias) [c_z, heads]; linear_q/k/v/g [c_z, heads *
   * head_dim]; linear_o [heads * head_dim, c_z]. bf16 with c_z = 128 and 4 heads x 32 runs the
   * tensor-core kernels; other shapes (head widths 8, 16, 24, 32, 48, 64) or float32 run the
   * general CUDA-core path. */
  int32_t c_z;
} b200tri_triatt_args;

size_t b200tri_triatt_workspace_bytes(int32_t n); /* bf16, c_z = 128, 4 heads x 32 */
size_t b200tri_triatt_workspace_bytes_dtype(int32_t n, int32_t dtype);
size_t b200tri_triatt_workspace_bytes_shape(int32_t n, int32_t dtype, int32_t c_z, int32_t heads, int32_t head_dim);
int b200tri_triatt_forward(const b200tri_triatt_args* args, b200tri_stream_t stream);

/* Stages, exposed for the context-parallel ring (the reference's
 * ring_triangle_attention_2d, src/foldjax/models/_cp_attention.py:197-403, runs
 * between the projections and the output stage).
 *
 * project: pair (o, t) is read at x + o*xs_outer + t*xs_inner. Writes
 *   q, k   [n_outer][n_inner][128] bf16 (q already divided by sqrt(head_dim))
 *   vt     [n_outer][128][ld] fp16 (V transposed per row o)
 *   bias   [heads][n_outer][ld] bf16 at bias + h*bias_head_stride + o*ld + t
 */
typedef struct {
  int32_t n_outer, n_inner, heads, head_dim;
  float eps;
  const void* x;
  int64_t xs_outer, xs_inner;
  const void* norm_scale;
  const void* norm_bias;
  const void* w_q;
  const void* w_k;
  const void* w_v;
  const void* w_bias;
  void* q;
  void* k;
  void* vt;
  void* bias;
  int64_t ld, bias_head_stride;
  void* workspace;
  size_t workspace_bytes;
} b200tri_triatt_project_args;

size_t b200tri_triatt_project_workspace_bytes(void);
int b200tri_triatt_project(const b200tri_triatt_project_args* args, b200tri_stream_t stream);

/* core: o[i][j][h*32+d] = sum_k softmax_k(q[i,j,h].k[i,k,h] + inf*(mask[i,k]-1) + bias[h,j,k]) v[i,k,h,d]
 * for n_i rows, n_j queries, n_k keys (the operator the reference's attention
 * cores implement, with q pre-scaled). mask is read at mask + i*ms_i + k*ms_k,
 * NULL = ones. With row_max/row_sum not NULL the kernel also returns, per
 * (i, h, j), the offset m it subtracted and l = sum_k exp(S - m). */
typedef struct {
  int32_t n_i, n_j, n_k, heads, head_dim;
  const void* q;  /* [n_i][n_j][128] */
  const void* k;  /* [n_i][n_k][128] */
  const void* vt; /* [n_i][128][v_ld] fp16 */
  int64_t v_ld;
  const void* bias; /* [heads][n_j][bias_ld] */
  int64_t bias_ld, bias_head_stride;
  const float* mask;
  int64_t ms_i, ms_k;
  float inf;
  void* o;        /* [n_i][n_j][128] bf16 */
  float* row_max; /* optional [n_i][heads][n_j] */
  float* row_sum;
  int32_t unnormalized;
  void* workspace; /* b200tri_triatt_core_workspace_bytes(n_i, n_k) */
  size_t workspace_bytes;
  /* Continuing one softmax over several key tiles (ring attention): with
   * `unnormalized` the kernel leaves its running state - the fp32 numerator in
   * acc_o [n_i][n_j][128], the offset in row_max and the denominator in row_sum -
   * instead of writing o; with `resume` it starts from that state instead of from
   * nothing. First tile: unnormalized; middle tiles: resume + unnormalized; last
   * tile: resume only, which writes the normalised o. */
  float* acc_o;
  int32_t resume;
  /* 0: `mask` holds 1 (keep) / 0 (drop) and the kernel forms inf * (mask - 1), the way
   * triangle_attention_forward builds its mask bias (triangle_attention.py:138-142).
   * 1: `mask` already is the additive mask bias [n_i][n_k] the reference's attention-core
   * operators receive (0, a soft negative bias, -1e9 or -infinity); `inf` is ignored.
   * Either way a bias at or below -30000 drops the key. */
  int32_t mask_additive;
} b200tri_triatt_core_args;

size_t b200tri_triatt_core_workspace_bytes(int32_t n_i, int32_t n_k);
int b200tri_triatt_core(const b200tri_triatt_core_args* args, b200tri_stream_t stream);

/* core over several key tiles in ONE launch: the same softmax walks tiles[0..n_tiles) in
 * order, each tile with its own k, vt, bias and mask buffers (the peers' tiles of a
 * context-parallel ring, which live in separate receive buffers); q, the sizes, the
 * outputs, the flags and the workspace are taken from tiles[0]. All tiles have the same
 * n_k, a multiple of 64 when n_tiles > 1; at most 7 tiles per launch. The running state
 * stays on chip between tiles, which the one-launch-per-tile form has to spill to acc_o.
 * Replaces the per-hop update of local_ring, src/foldjax/models/_cp_attention.py:290-386. */
size_t b200tri_triatt_core_multi_workspace_bytes(int32_t n_i, int32_t n_k, int32_t n_tiles);
int b200tri_triatt_core_multi(const b200tri_triatt_core_args* tiles, int32_t n_tiles, b200tri_stream_t stream);

/* core, for callers that have no scratch memory to give and must not allocate.
 * This entry point has no counterpart in the reference. Some hosts of this
 * library cannot hand over a workspace: a custom-call handler inside a framework
 * that reserved the device's memory when it started and passes the handler only
 * the operand and result buffers it planned, or a service whose memory budget is
 * fixed at start-up. For them cudaMalloc inside the call may fail, stall or be
 * forbidden. This variant runs the same kernel as b200tri_triatt_core but keeps
 * its one scratch buffer (the additive mask-bias rows, n_i x round_up(n_k, 64)
 * floats) in a fixed array inside the library: B200TRI_TRIATT_CORE_STATIC_MAX_FLOATS
 * floats (4 MiB), resident on every GPU that loads the library until the process
 * exits. `workspace` / `workspace_bytes` of the argument struct are ignored.
 *
 * Limits and rules:
 *  - n_i * round_up(n_k, 64) must not exceed the maximum; larger problems are
 *    rejected with B200TRI_ERR_UNSUPPORTED (use b200tri_triatt_core instead).
 *  - The call allocates nothing (no cudaMalloc/cudaFree, no events): it is refused
 *    with B200TRI_ERR_INVALID while b200tri_timing_enable(1) is in effect, because
 *    that mode creates CUDA events.
 *  - The first call on a device looks up the array's device address (once per
 *    device, with that device current). Make that first call before any stream
 *    capture begins.
 *  - All calls on a device share the array. Every call rewrites the part it uses
 *    before reading it, so nothing has to be cleared; but two calls whose kernels
 *    overlap on the GPU (different streams) race on it. Keep them on one stream
 *    or order them with events. */
#define B200TRI_TRIATT_CORE_STATIC_MAX_FLOATS (1 << 20)
int b200tri_triatt_core_static(const b200tri_triatt_core_args* args, b200tri_stream_t stream);

/* finish: out = bf16(bf16(o * sigmoid(LN(x) @ w_g)) @ w_o) (+ residual); x and
 * out/residual are addressed through (outer, inner) strides. */
typedef struct {
  int32_t n_outer, n_inner;
  float eps;
  const void* o; /* [n_outer][n_inner][128] */
  const void* x;
  int64_t xs_outer, xs_inner;
  const void* norm_scale;
  const void* norm_bias;
  const void* w_g;
  const void* w_o;
  const void* residual;
  void* out;
  int64_t os_outer, os_inner;
  void* workspace;
  size_t workspace_bytes;
} b200tri_triatt_finish_args;

size_t b200tri_triatt_finish_workspace_bytes(void);
int b200tri_triatt_finish(const b200tri_triatt_finish_args* args, b200tri_stream_t stream);

/* ------------------------------------------------------------------------
 * 2-D context parallelism: the pair tensor tiled z[I_r, J_c] over an R x C grid of GPUs
 * (C a multiple of R: 1x2, 2x2, 2x4 on one 8-GPU box), one communicator per GPU.
 * Replaces: context_parallel / resolve_cp_layout, src/foldjax/models/_cp.py:162-187,259;
 *   _cannon_contract, src/foldjax/models/boltz2/models/triangle/triangle.py:132-212;
 *   ring_triangle_attention_2d, src/foldjax/models/_cp_attention.py:197-403 and its
 *   callers (boltz2 triangle_attention_cp.py:40-156, protenix triangle_attention_cp.py:33,
 *   openfold3 triangle_attention_cp.py:30).
 * rank = r * cols + c owns rows I_r (n / rows of them) and columns J_c (n / cols).
 * Tiles travel over NVLink as grouped ncclSend/ncclRecv on the communicator's own stream,
 * fenced against the caller's stream by events: every entry point below only enqueues.
 * NCCL (libnccl.so.2) is loaded on first use of this section.
 *
 * One process per GPU: rank 0 calls b200tri_comm_unique_id, the caller hands the 128 bytes
 * to every rank (any side channel), each rank makes its device current and calls
 * b200tri_comm_init. One process driving all GPUs (the reference's arrangement under
 * shard_map): b200tri_comm_init_all fills comms[0..world); calls for different devices come
 * from one host thread per device, or are wrapped in b200tri_comm_group_start/_end.
 * --------------------------------------------------------------------- */
#define B200TRI_COMM_ID_BYTES 128
typedef struct b200tri_comm b200tri_comm;

int b200tri_comm_unique_id(void* id128);
int b200tri_comm_init(b200tri_comm** comm, const void* id128, int32_t world, int32_t rank, int32_t rows, int32_t cols);
int b200tri_comm_init_all(b200tri_comm** comms, const int32_t* devices, int32_t world, int32_t rows, int32_t cols);
int b200tri_comm_destroy(b200tri_comm* comm);
int b200tri_comm_info(const b200tri_comm* comm, int32_t* world, int32_t* rank, int32_t* rows, int32_t* cols);
int b200tri_comm_group_start(void);
int b200tri_comm_group_end(void);

/* Optional: an exchange workspace owned by the communicator. Collective and host-synchronous
 * (set-up time: it allocates), every rank with the same size; *ptr is the rank's workspace.
 * With one process per GPU the peers' workspaces are mapped into this process through CUDA
 * IPC, and b200tri_trimul_cp / b200tri_triatt_cp called with workspace = NULL then move their
 * tiles between the workspaces with device-to-device copies on the copy engines (NCCL only
 * carries 4-byte tokens) instead of NCCL's send/receive kernels: by default every sender WRITES
 * its tiles into the receivers' workspaces (a "slot is free" token from each receiver before, a
 * "written" token after); b200tri_comm_configure(comm, push = 0, ...) makes every receiver READ
 * them out of the owners' workspaces instead ("ready" before, "consumed" after), and
 * copy_streams (1..4) spreads the copies of an exchange over that many streams; sm_reserve
 * (default 4) is the number of SMs the attention launch that runs while key tiles travel leaves
 * free, so that the token kernels are not held back until it ends. Every rank must configure
 * the same direction. b200tri_comm_pulls() tells whether the mapped-memory path is
 * active (it is not when a peer could not be mapped, or under b200tri_comm_init_all: one
 * process sees every device and keeps to sends and receives). A caller-provided workspace
 * always means sends and receives. Sizes: the larger of the two *_cp_workspace_bytes. */
int b200tri_comm_workspace(b200tri_comm* comm, size_t bytes, void** ptr);
int b200tri_comm_pulls(const b200tri_comm* comm);
int b200tri_comm_configure(b200tri_comm* comm, int32_t push, int32_t copy_streams, int32_t sm_reserve);

/* Mesh self-test, the counterpart of verify_mesh_exchange (src/foldjax/models/_cp.py:199-232):
 * every rank sends `bytes` from `shard` to every other rank and receives theirs into
 * gathered[src * bytes ...] through the very send/receive path the ops use. The caller stamps
 * the shards, copies `gathered` to the host and judges it there. */
int b200tri_comm_probe(b200tri_comm* comm, const void* shard, void* gathered, size_t bytes, b200tri_stream_t stream);

/* The exchange schedule, for inspection and tests: the global message list of an op on a
 * rows x cols grid. A message moves `what` (0 = a, 1 = b, 2 = K and V, 3 = pair bias) of rank
 * `src` - row block `block` of it, or all of it when block = -1 - into slot (slot0, slot1) of
 * rank `dst`'s panel; src == dst is a local copy. Returns the number of messages (writes at
 * most `capacity` of them to `out`, which may be NULL), or -1 on a bad grid / op. */
enum { B200TRI_CP_TRIMUL_OUTGOING = 0, B200TRI_CP_TRIMUL_INCOMING = 1, B200TRI_CP_TRIATT_STARTING = 2,
       B200TRI_CP_TRIATT_ENDING = 3 };
typedef struct { int32_t src, dst, what, block, slot0, slot1; } b200tri_cp_msg;
int b200tri_cp_plan(int32_t rows, int32_t cols, int32_t op, b200tri_cp_msg* out, int32_t capacity);
/* Order of the copies of one exchange: round[i] for message i of b200tri_cp_plan (-1 for a
 * local message or one whose `what` differs from the filter; what < 0 takes all). Within a
 * round every rank sends at most one tile and receives at most one; the ops issue their copies
 * round by round. Returns the number of messages, or -1 on a bad grid / op. No counterpart in
 * the reference, whose ring hops are scheduled by XLA. */
int b200tri_cp_rounds(int32_t rows, int32_t cols, int32_t op, int32_t what, int32_t* round, int32_t capacity);

/* Dry run of one context-parallel op, for checks on a machine without a GPU: what rank `rank`
 * of a rows x cols grid would do for `op` at n tokens - every copy it issues (the tiles it
 * writes into its peers' workspaces with push = 1, the ones it reads out of them with push = 0,
 * its local copies) and every launch it makes - without a CUDA or NCCL call. Offsets are bytes
 * from the start of a rank's exchange workspace (src_off in the sender's, dst_off in the
 * receiver's; off[0..2] of a launch in the rank's own) or from the start of its tile (off[3] of
 * an output stage). `group` numbers the exchange groups (and the launches they fence), `round`
 * the copy rounds inside a group. Returns the number of events (at most `capacity` are written),
 * or -1. b200tri_cp_layout gives the byte offsets of the arrays in the workspace:
 * tri-mult: {a slots, own a, b slots, own b, bytes of one block, blocks per a slot, t, total};
 * tri-attn: {q, k slots, vT slots, own bias, bias slots, bytes of a k tile, of a vT tile, of a
 * bias tile, key tiles, own tile index, total}. No counterpart in the reference (XLA schedules
 * its collective-permutes). */
enum { B200TRI_CP_EVENT_LOCAL_COPY = 0, B200TRI_CP_EVENT_COPY = 1, B200TRI_CP_EVENT_PROJECT = 2,
       B200TRI_CP_EVENT_CONTRACT = 3, B200TRI_CP_EVENT_OUTPUT = 4, B200TRI_CP_EVENT_CORE_TILE = 5 };
typedef struct {
  int32_t kind, group, round, src, dst, what, block, slot0, slot1, n_i, n_j, reserved;
  int64_t src_off, dst_off, bytes;
  int64_t off[4];
} b200tri_cp_event;
int b200tri_cp_dry_run(int32_t rows, int32_t cols, int32_t rank, int32_t n, int32_t op, int32_t push,
                       b200tri_cp_event* out, int32_t capacity);
int b200tri_cp_layout(int32_t rows, int32_t cols, int32_t rank, int32_t n, int32_t op, int64_t* out16);

/* Triangle multiplication on this rank's tile. x / residual / out are the rank's tile
 * [n / rows][n / cols][128] bf16; mask is the WHOLE [n][n] float32 mask (or NULL), replicated
 * on every rank; parameters as in b200tri_trimul_args. n must be a multiple of cols (pad
 * with zero pairs and mask 0, as the reference does, triangle.py:165-172). */
typedef struct {
  int32_t n;        /* tokens of the whole pair tensor */
  int32_t incoming;
  float eps;
  const void* x;
  const float* mask;
  const void* norm_in_scale;
  const void* norm_in_bias;
  const void* p_in;
  const void* g_in;
  const void* norm_out_scale;
  const void* norm_out_bias;
  const void* p_out;
  const void* g_out;
  const void* residual;
  void* out;
  void* workspace; /* b200tri_trimul_cp_workspace_bytes(comm, n), 1 KiB aligned; NULL = the communicator's own */
  size_t workspace_bytes;
} b200tri_trimul_cp_args;

size_t b200tri_trimul_cp_workspace_bytes(const b200tri_comm* comm, int32_t n);
int b200tri_trimul_cp(b200tri_comm* comm, const b200tri_trimul_cp_args* args, b200tri_stream_t stream);

/* Triangle attention on this rank's tile: the starting node rings over the key tiles of
 * the rank's grid row, the ending node over those of its grid column. One softmax is
 * continued over the key tiles (own tile first while the peers' K/V are in flight, then all
 * peer tiles in one launch). Rows without a valid key come out as the uniform average over
 * their keys (the convention of the dense path), not as the zeros of the reference's ring. */
typedef struct {
  int32_t n;
  int32_t starting;
  int32_t heads, head_dim; /* 4 x 32 */
  float inf, eps;
  const void* x;
  const float* mask; /* whole [n][n] or NULL */
  const void* norm_scale;
  const void* norm_bias;
  const void* w_bias;
  const void* w_q;
  const void* w_k;
  const void* w_v;
  const void* w_g;
  const void* w_o;
  const void* residual;
  void* out;
  void* workspace; /* b200tri_triatt_cp_workspace_bytes(comm, n), 1 KiB aligned; NULL = the communicator's own */
  size_t workspace_bytes;
} b200tri_triatt_cp_args;

size_t b200tri_triatt_cp_workspace_bytes(const b200tri_comm* comm, int32_t n);
int b200tri_triatt_cp(b200tri_comm* comm, const b200tri_triatt_cp_args* args, b200tri_stream_t stream);

/* ------------------------------------------------------------------------
 * Pair transition (the feed-forward that follows the triangle ops in a
 * Pairformer block).
 * Replaces: transition_forward,
 *   src/foldjax/models/boltz2/models/primitives/transition.py:41-127, as called
 *   on the pair tensor by src/foldjax/models/boltz2/models/pairformer.py:152-160
 *   (and its fused-GLU branch, glu_backend="tokamax", :101-105).
 * Computes  update = (silu(LN(x) @ fc1) * (LN(x) @ fc2)) @ fc3  per row of the
 * flattened [rows][128] tensor, with the reference's bf16 rounding points.
 * The op is row-local, so a context-parallel caller passes its own tile.
 * If `residual` is not NULL the kernel writes residual + update; residual may
 * alias x and out (the block's z += transition(z)). */
typedef struct {
  int64_t rows;          /* pairs: product of all leading axes */
  int32_t channels;      /* 128 */
  int32_t hidden;        /* width of fc1/fc2 outputs: a multiple of 64 (512 in the Pairformer) */
  float eps;
  const void* x;         /* bf16 [rows][128], contiguous */
  const void* norm_scale;
  const void* norm_bias; /* bf16 [128] */
  const void* fc1;       /* bf16 [128][hidden]  ([in, out], the reference's layout) */
  const void* fc2;       /* bf16 [128][hidden] */
  const void* fc3;       /* bf16 [hidden][128] */
  const void* residual;  /* bf16 [rows][128] or NULL */
  void* out;             /* bf16 [rows][128] */
  void* workspace;
  size_t workspace_bytes;
  /* Optional float32 [rows]: the update of row r is multiplied by row_mask[r] (rounded to
   * bf16) before the residual add - OpenFold3's masked transition, swiglu_transition(...,
   * mask=pair_mask), src/foldjax/models/openfold3/models/primitives.py:133-150 as called by
   * pair_block.py:174-183. NULL = no mask. */
  const float* row_mask;
} b200tri_pair_transition_args;

size_t b200tri_pair_transition_workspace_bytes(int32_t hidden);
int b200tri_pair_transition(const b200tri_pair_transition_args* args, b200tri_stream_t stream);

/* ------------------------------------------------------------------------
 * Single-representation attention with pair bias (the other reader of z in a
 * Pairformer block).
 * Replaces: attention_pair_bias_forward,
 *   src/foldjax/models/boltz2/models/primitives/attention.py:19-140, as called by
 *   src/foldjax/models/boltz2/models/trunk_blocks/pairformer.py:188-203 with s and z
 *   promoted to float32.
 * Computes  out = (sigmoid(s @ proj_g) * softmax_j(q_h . k_h / sqrt(d) + bias_h[i,j]
 *                  + (1 - mask_j) * -inf) v_h) @ proj_o
 * with q = s @ proj_q + proj_q_bias, k/v = k_in @ proj_k/proj_v and
 * bias = LN(z) @ proj_z. s, k_in, mask and out are fp32 (as in the reference); z and
 * all parameters are bf16 (the trunk dtype) and are promoted to fp32. Returns the
 * update (the caller adds the residual). `multiplicity` is 1. */
typedef struct {
  int32_t n;        /* tokens */
  int32_t c_s;      /* heads * 24 (384 in the Pairformer) */
  int32_t c_z;      /* 128 */
  int32_t heads;    /* <= 16 */
  float eps;        /* layer norm of z */
  float inf;        /* mask constant (1e6 in the reference) */
  const void* s;    /* fp32 [n][c_s], the caller's layer-normed single representation */
  const void* k_in; /* fp32 [n][c_s] or NULL (= s) */
  const void* z;    /* bf16 [n][n][128] */
  const void* mask; /* fp32 [n], 1 = valid token */
  const void* proj_q;      /* bf16 [c_s][c_s]  ([in, out]) */
  const void* proj_q_bias; /* bf16 [c_s] */
  const void* proj_k;
  const void* proj_v;
  const void* proj_g;
  const void* proj_z_norm_scale; /* bf16 [128] */
  const void* proj_z_norm_bias;
  const void* proj_z;      /* bf16 [128][heads] */
  const void* proj_o;      /* bf16 [c_s][c_s] */
  void* out;        /* fp32 [n][c_s] */
  void* workspace;
  size_t workspace_bytes;
} b200tri_attention_pair_bias_args;

size_t b200tri_attention_pair_bias_workspace_bytes(int32_t n, int32_t c_s, int32_t heads);
int b200tri_attention_pair_bias(const b200tri_attention_pair_bias_args* args, b200tri_stream_t stream);

/* ------------------------------------------------------------------------
 * One Pairformer block, or a stack of them (the trunk), as ONE call.
 * Replaces: pairformer_layer_forward, src/foldjax/models/boltz2/models/trunk_blocks/
 *   pairformer.py:100-206, and the lax.scan over stacked layer parameters around it
 *   (pairformer.py:30-100, src/foldjax/models/_stacking.py).
 * Per block:  z += tri_mul_out(z); z += tri_mul_in(z); z += tri_att_start(z);
 *   z += tri_att_end(z); z += transition_z(z);
 *   s += attention_pair_bias(LN(s), z, mask); s += transition_s(s).
 * z is bf16 [n][n][128]; s is float32 [n][c_s] (the reference promotes the single track to
 * float32, pairformer.py:182-206); every parameter is bf16 in the reference's layout.
 * s_in = NULL runs the pair track only. z_out may alias z_in, s_out may alias s_in.
 * `stacked` = 0: params points at n_blocks structs, one per block. `stacked` = 1: params
 * points at ONE struct whose pointers are the bases of leaves stacked with a leading layer
 * axis ([n_blocks, ...], what FoldJAX's scan carries); block l reads leaf l.
 * --------------------------------------------------------------------- */
typedef struct { const void *norm_in_scale, *norm_in_bias, *p_in, *g_in, *norm_out_scale, *norm_out_bias, *p_out, *g_out; } b200tri_trimul_params;
typedef struct { const void *norm_scale, *norm_bias, *w_bias, *w_q, *w_k, *w_v, *w_g, *w_o; } b200tri_triatt_params;
typedef struct { const void *norm_scale, *norm_bias, *fc1, *fc2, *fc3; int32_t hidden; } b200tri_transition_params;
typedef struct { const void *proj_q, *proj_q_bias, *proj_k, *proj_v, *proj_g, *proj_z_norm_scale, *proj_z_norm_bias, *proj_z, *proj_o; } b200tri_attention_params;
typedef struct {
  b200tri_trimul_params tri_mul_out, tri_mul_in;
  b200tri_triatt_params tri_att_start, tri_att_end;
  b200tri_transition_params transition_z;   /* 128 -> hidden -> 128 (hidden 512) */
  const void *pre_norm_s_scale, *pre_norm_s_bias; /* [c_s] */
  b200tri_attention_params attention;       /* heads_s heads of width 24 */
  b200tri_transition_params transition_s;   /* c_s -> hidden -> c_s */
} b200tri_pairformer_block_params;

typedef struct {
  int32_t n;        /* tokens */
  int32_t c_s;      /* 384 (0 with s_in = NULL) */
  int32_t heads_s;  /* 16 */
  int32_t n_blocks; /* 1 = one block, L = a trunk */
  int32_t stacked;
  float eps;        /* every layer norm (1e-5) */
  float tri_inf;    /* triangle-attention mask constant (1e9) */
  float att_inf;    /* single-track attention mask constant (1e6) */
  const b200tri_pairformer_block_params* params;
  const void* z_in;
  void* z_out;
  const float* s_in;
  float* s_out;
  const float* pair_mask; /* [n][n] or NULL (= ones) */
  const float* mask;      /* [n] or NULL (= ones) */
  void* workspace;        /* b200tri_pairformer_workspace_bytes, 1 KiB aligned */
  size_t workspace_bytes;
  /* Variants of the block in the other model families (all 0 = the Boltz-2 block):
   * pair_gate: z is multiplied by (pair_mask != 0) before the first update and after every
   *   update, and s by (mask != 0) after both single-track updates - Protenix's block,
   *   src/foldjax/models/protenix/models/trunk_blocks/pairformer.py:71-180 (pass mask = the
   *   diagonal of pair_mask, as it does).
   * mask_transition: the pair transition's update is multiplied by pair_mask before it is
   *   added - OpenFold3's _mask_trans default, openfold3/models/pair_block.py:174-183.
   * attention_first: the two attention updates run before the two multiplications
   *   (tri_mul_first = False of OpenFold3's template pair block, pair_block.py:151-171). */
  int32_t pair_gate;
  int32_t mask_transition;
  int32_t attention_first;
} b200tri_pairformer_args;

size_t b200tri_pairformer_workspace_bytes(int32_t n, int32_t c_s, int32_t heads_s, int32_t hidden_z, int32_t hidden_s);
int b200tri_pairformer_forward(const b200tri_pairformer_args* args, b200tri_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200TRI_H_ */
