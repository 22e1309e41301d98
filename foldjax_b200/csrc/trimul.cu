// Triangle multiplicative update, whole module on one GPU: projection ->
// contraction -> output stage in a caller-provided workspace.
// Replaces triangle_multiplication_forward,
// src/foldjax/models/boltz2/models/triangle/triangle.py:33-129.
#include "host.cuh"

namespace {

// Intermediates are channel-major inside blocks of RPB rows: [block][128][RPB][ld].
// A tile of the projection then stores its 128 channel planes RPB*ld*2 bytes apart
// (384 KiB at N = 3072) instead of N*ld*2 (18 MiB), which is what its scattered
// 256-byte stores need to run at memory speed; the contraction's TMA boxes span
// two (a) or four (b) blocks.
constexpr int RPB = 64;

struct Plan {
  int64_t ld;           // row pitch of the intermediates
  int64_t chan_stride;  // elements between channels inside a block
  int64_t block_stride; // elements between row blocks
  size_t inter_elems;   // elements of one intermediate (a, b or t)
  size_t off_a, off_b, off_t, off_proj, off_fin, total;
};

}  // namespace

static Plan plan_offsets(int32_t n) {
  Plan p;
  p.ld = b200::round_up(n, 64);
  p.chan_stride = p.ld * RPB;
  p.block_stride = p.chan_stride * 128;
  p.inter_elems = static_cast<size_t>(p.block_stride) * ((n + RPB - 1) / RPB);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    off = (off + 1023) / 1024 * 1024;
    size_t r = off;
    off += bytes;
    return r;
  };
  p.off_a = take(p.inter_elems * 2);
  p.off_b = take(p.inter_elems * 2);
  p.off_t = take(p.inter_elems * 2);
  p.off_proj = take(b200tri_trimul_project_workspace_bytes());
  p.off_fin = take(b200tri_trimul_finish_workspace_bytes());
  p.total = (off + 1023) / 1024 * 1024;
  return p;
}

extern "C" size_t b200tri_trimul_workspace_bytes(int32_t n) {
  if (n <= 0) return 0;
  return plan_offsets(n).total;
}

static bool specialised(int32_t dtype, int32_t c_z, int32_t c_hidden) {
  return dtype == B200TRI_DTYPE_BF16 && c_z == 128 && c_hidden == 128;
}

extern "C" size_t b200tri_trimul_workspace_bytes_shape(int32_t n, int32_t dtype, int32_t c_z, int32_t c_hidden) {
  c_z = c_z > 0 ? c_z : 128;
  c_hidden = c_hidden > 0 ? c_hidden : 128;
  if (dtype != B200TRI_DTYPE_BF16 && dtype != B200TRI_DTYPE_F32) return 0;
  if (specialised(dtype, c_z, c_hidden)) return b200tri_trimul_workspace_bytes(n);
  return b200::trimul_workspace_bytes_generic(n, c_z, c_hidden, dtype);
}

extern "C" size_t b200tri_trimul_workspace_bytes_dtype(int32_t n, int32_t dtype) {
  return b200tri_trimul_workspace_bytes_shape(n, dtype, 128, 128);
}

extern "C" int b200tri_trimul_forward(const b200tri_trimul_args* a, b200tri_stream_t stream) {
  using namespace b200;
  B200_REQUIRE(a != nullptr, B200TRI_ERR_INVALID, "trimul: null args");
  B200_REQUIRE(a->n > 0, B200TRI_ERR_INVALID, "trimul: n must be positive (got %d)", a->n);
  B200_REQUIRE(a->x && a->out, B200TRI_ERR_INVALID, "trimul: x/out must not be null");
  B200_REQUIRE(a->dtype == B200TRI_DTYPE_BF16 || a->dtype == B200TRI_DTYPE_F32, B200TRI_ERR_UNSUPPORTED,
               "trimul: unknown dtype %d", a->dtype);
  const int c_z = a->c_z > 0 ? a->c_z : 128, c_hidden = a->c_hidden > 0 ? a->c_hidden : 128;
  B200_REQUIRE(c_z % 8 == 0 && c_z <= 1024 && c_hidden % 8 == 0 && c_hidden <= 1024, B200TRI_ERR_UNSUPPORTED,
               "trimul: channel counts must be multiples of 8 up to 1024 (got c_z %d, c_hidden %d)", c_z, c_hidden);
  if (!specialised(a->dtype, c_z, c_hidden)) {
    const size_t need = trimul_workspace_bytes_generic(a->n, c_z, c_hidden, a->dtype);
    B200_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= need, B200TRI_ERR_WORKSPACE,
                 "trimul (general shapes): workspace of %zu bytes needed for n=%d, got %zu", need, a->n,
                 a->workspace_bytes);
    B200_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 1023) == 0, B200TRI_ERR_INVALID,
                 "trimul: workspace must be 1024-byte aligned");
    B200_REQUIRE(a->norm_in_scale && a->norm_in_bias && a->p_in && a->g_in && a->norm_out_scale && a->norm_out_bias &&
                     a->p_out && a->g_out,
                 B200TRI_ERR_INVALID, "trimul: null parameter pointer");
    return trimul_forward_generic(a, c_z, c_hidden, reinterpret_cast<cudaStream_t>(stream));
  }
  const Plan pl = plan_offsets(a->n);
  B200_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= pl.total, B200TRI_ERR_WORKSPACE,
               "trimul: workspace of %zu bytes needed for n=%d, got %zu", pl.total, a->n, a->workspace_bytes);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 1023) == 0, B200TRI_ERR_INVALID,
               "trimul: workspace must be 1024-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  const int64_t n = a->n;

  b200tri_trimul_project_args pa = {};
  pa.n_outer = a->n;
  pa.n_inner = a->n;
  pa.eps = a->eps;
  pa.x = a->x;
  pa.mask = a->mask;
  if (!a->incoming) {  // a[i][k] from x[i][k]
    pa.xs_outer = n * 128;
    pa.xs_inner = 128;
    pa.ms_outer = n;
    pa.ms_inner = 1;
  } else {  // a'[i][k] = a[k][i] from x[k][i]
    pa.xs_outer = 128;
    pa.xs_inner = n * 128;
    pa.ms_outer = 1;
    pa.ms_inner = n;
  }
  pa.norm_in_scale = a->norm_in_scale;
  pa.norm_in_bias = a->norm_in_bias;
  pa.p_in = a->p_in;
  pa.g_in = a->g_in;
  pa.a = ws + pl.off_a;
  pa.b = ws + pl.off_b;
  pa.ld = pl.ld;
  pa.chan_stride = pl.chan_stride;
  pa.block_stride = pl.block_stride;
  pa.rows_per_block = RPB;
  pa.workspace = ws + pl.off_proj;
  pa.workspace_bytes = b200tri_trimul_project_workspace_bytes();
  int rc = b200tri_trimul_project(&pa, stream);
  if (rc) return rc;

  b200tri_trimul_contract_args ca = {};
  ca.n_i = ca.n_j = ca.n_k = a->n;
  ca.n_src = 1;
  ca.a = pa.a;
  ca.a_ld = pl.ld;
  ca.a_chan_stride = pl.chan_stride;
  ca.b = pa.b;
  ca.b_ld = pl.ld;
  ca.b_chan_stride = pl.chan_stride;
  ca.out_bf16 = ws + pl.off_t;
  ca.out_ld = pl.ld;
  ca.out_chan_stride = pl.chan_stride;
  ca.a_rows_per_block = ca.b_rows_per_block = ca.out_rows_per_block = RPB;
  ca.a_block_stride = ca.b_block_stride = ca.out_block_stride = pl.block_stride;
  rc = b200tri_trimul_contract(&ca, stream);
  if (rc) return rc;

  b200tri_trimul_finish_args fa = {};
  fa.n_i = fa.n_j = a->n;
  fa.eps = a->eps;
  fa.t = ws + pl.off_t;
  fa.t_ld = pl.ld;
  fa.t_chan_stride = pl.chan_stride;
  fa.t_rows_per_block = RPB;
  fa.t_block_stride = pl.block_stride;
  fa.x = a->x;
  fa.xs_i = n * 128;
  fa.xs_j = 128;
  fa.norm_in_scale = a->norm_in_scale;
  fa.norm_in_bias = a->norm_in_bias;
  fa.norm_out_scale = a->norm_out_scale;
  fa.norm_out_bias = a->norm_out_bias;
  fa.p_out = a->p_out;
  fa.g_out = a->g_out;
  fa.residual = a->residual;
  fa.out = a->out;
  fa.os_i = n * 128;
  fa.os_j = 128;
  fa.workspace = ws + pl.off_fin;
  fa.workspace_bytes = b200tri_trimul_finish_workspace_bytes();
  return b200tri_trimul_finish(&fa, stream);
}
