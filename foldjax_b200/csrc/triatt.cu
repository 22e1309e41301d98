// Triangle attention, whole module on one GPU: projections -> core -> output
// stage in a caller-provided workspace. Replaces triangle_attention_forward,
// src/foldjax/models/boltz2/models/triangle/triangle_attention.py:79-162.
// The ending node is the starting node on swapped strides of x, mask and out
// (:128-130, :160-161); no transposed copy of the pair tensor is made.
#include "host.cuh"

namespace {

struct Plan {
  int64_t ld;
  size_t off_q, off_k, off_v, off_o, off_bias, off_proj, off_core, off_fin, total;
};

Plan plan_offsets(int32_t n) {
  Plan p;
  p.ld = b200::round_up(n, 64);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    off = (off + 1023) / 1024 * 1024;
    size_t r = off;
    off += bytes;
    return r;
  };
  const size_t pair = static_cast<size_t>(n) * n * 128 * 2;
  p.off_q = take(pair);
  p.off_k = take(pair);
  p.off_o = take(pair);
  p.off_v = take(static_cast<size_t>(n) * 128 * p.ld * 2);
  p.off_bias = take(static_cast<size_t>(4) * n * p.ld * 2);
  p.off_proj = take(b200tri_triatt_project_workspace_bytes());
  p.off_core = take(b200tri_triatt_core_workspace_bytes(n, n));
  p.off_fin = take(b200tri_triatt_finish_workspace_bytes());
  p.total = (off + 1023) / 1024 * 1024;
  return p;
}

}  // namespace

extern "C" size_t b200tri_triatt_workspace_bytes(int32_t n) {
  if (n <= 0) return 0;
  return plan_offsets(n).total;
}

static bool specialised(int32_t dtype, int32_t c_z, int32_t heads, int32_t head_dim) {
  return dtype == B200TRI_DTYPE_BF16 && c_z == 128 && heads == 4 && head_dim == 32;
}

extern "C" size_t b200tri_triatt_workspace_bytes_shape(int32_t n, int32_t dtype, int32_t c_z, int32_t heads,
                                                       int32_t head_dim) {
  c_z = c_z > 0 ? c_z : 128;
  if (dtype != B200TRI_DTYPE_BF16 && dtype != B200TRI_DTYPE_F32) return 0;
  if (specialised(dtype, c_z, heads, head_dim)) return b200tri_triatt_workspace_bytes(n);
  return b200::triatt_workspace_bytes_generic(n, c_z, heads, head_dim);
}

extern "C" size_t b200tri_triatt_workspace_bytes_dtype(int32_t n, int32_t dtype) {
  return b200tri_triatt_workspace_bytes_shape(n, dtype, 128, 4, 32);
}

extern "C" int b200tri_triatt_forward(const b200tri_triatt_args* a, b200tri_stream_t stream) {
  using namespace b200;
  B200_REQUIRE(a != nullptr, B200TRI_ERR_INVALID, "triatt: null args");
  B200_REQUIRE(a->n > 0, B200TRI_ERR_INVALID, "triatt: n must be positive (got %d)", a->n);
  B200_REQUIRE(a->x && a->out, B200TRI_ERR_INVALID, "triatt: x/out must not be null");
  B200_REQUIRE(a->dtype == B200TRI_DTYPE_BF16 || a->dtype == B200TRI_DTYPE_F32, B200TRI_ERR_UNSUPPORTED,
               "triatt: unknown dtype %d", a->dtype);
  const int c_z = a->c_z > 0 ? a->c_z : 128;
  B200_REQUIRE(a->heads >= 1 && a->heads <= 64 && a->head_dim >= 1, B200TRI_ERR_UNSUPPORTED,
               "triatt: 1 to 64 heads (got %d x %d)", a->heads, a->head_dim);
  B200_REQUIRE(c_z % 8 == 0 && c_z <= 1024, B200TRI_ERR_UNSUPPORTED,
               "triatt: c_z must be a multiple of 8 up to 1024 (got %d)", c_z);
  if (!specialised(a->dtype, c_z, a->heads, a->head_dim)) {
    const size_t need = triatt_workspace_bytes_generic(a->n, c_z, a->heads, a->head_dim);
    B200_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= need, B200TRI_ERR_WORKSPACE,
                 "triatt (general shapes): workspace of %zu bytes needed for n=%d, got %zu", need, a->n,
                 a->workspace_bytes);
    B200_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 1023) == 0, B200TRI_ERR_INVALID,
                 "triatt: workspace must be 1024-byte aligned");
    B200_REQUIRE(a->norm_scale && a->norm_bias && a->w_bias && a->w_q && a->w_k && a->w_v && a->w_g && a->w_o,
                 B200TRI_ERR_INVALID, "triatt: null parameter pointer");
    return triatt_forward_generic(a, c_z, reinterpret_cast<cudaStream_t>(stream));
  }
  const Plan pl = plan_offsets(a->n);
  B200_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= pl.total, B200TRI_ERR_WORKSPACE,
               "triatt: workspace of %zu bytes needed for n=%d, got %zu", pl.total, a->n, a->workspace_bytes);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 1023) == 0, B200TRI_ERR_INVALID,
               "triatt: workspace must be 1024-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  const int64_t n = a->n;
  // Attention frame (o = row i, t = column): the starting node reads x[o][t], the
  // ending node reads x[t][o].
  const int64_t s_outer = a->starting ? n * 128 : 128;
  const int64_t s_inner = a->starting ? 128 : n * 128;

  b200tri_triatt_project_args pa = {};
  pa.n_outer = pa.n_inner = a->n;
  pa.heads = a->heads;
  pa.head_dim = a->head_dim;
  pa.eps = a->eps;
  pa.x = a->x;
  pa.xs_outer = s_outer;
  pa.xs_inner = s_inner;
  pa.norm_scale = a->norm_scale;
  pa.norm_bias = a->norm_bias;
  pa.w_q = a->w_q;
  pa.w_k = a->w_k;
  pa.w_v = a->w_v;
  pa.w_bias = a->w_bias;
  pa.q = ws + pl.off_q;
  pa.k = ws + pl.off_k;
  pa.vt = ws + pl.off_v;
  pa.bias = ws + pl.off_bias;
  pa.ld = pl.ld;
  pa.bias_head_stride = n * pl.ld;
  pa.workspace = ws + pl.off_proj;
  pa.workspace_bytes = b200tri_triatt_project_workspace_bytes();
  int rc = b200tri_triatt_project(&pa, stream);
  if (rc) return rc;

  b200tri_triatt_core_args ca = {};
  ca.n_i = ca.n_j = ca.n_k = a->n;
  ca.heads = a->heads;
  ca.head_dim = a->head_dim;
  ca.q = pa.q;
  ca.k = pa.k;
  ca.vt = pa.vt;
  ca.v_ld = pl.ld;
  ca.bias = pa.bias;
  ca.bias_ld = pl.ld;
  ca.bias_head_stride = n * pl.ld;
  ca.mask = a->mask;
  ca.ms_i = a->starting ? n : 1;
  ca.ms_k = a->starting ? 1 : n;
  ca.inf = a->inf;
  ca.o = ws + pl.off_o;
  ca.workspace = ws + pl.off_core;
  ca.workspace_bytes = b200tri_triatt_core_workspace_bytes(a->n, a->n);
  rc = b200tri_triatt_core(&ca, stream);
  if (rc) return rc;

  b200tri_triatt_finish_args fa = {};
  fa.n_outer = fa.n_inner = a->n;
  fa.eps = a->eps;
  fa.o = ca.o;
  fa.x = a->x;
  fa.xs_outer = s_outer;
  fa.xs_inner = s_inner;
  fa.norm_scale = a->norm_scale;
  fa.norm_bias = a->norm_bias;
  fa.w_g = a->w_g;
  fa.w_o = a->w_o;
  fa.residual = a->residual;
  fa.out = a->out;
  fa.os_outer = s_outer;
  fa.os_inner = s_inner;
  fa.workspace = ws + pl.off_fin;
  fa.workspace_bytes = b200tri_triatt_finish_workspace_bytes();
  return b200tri_triatt_finish(&fa, stream);
}
