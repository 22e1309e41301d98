// One Pairformer block - or a whole stack of them - as a single call.
//
// Reference: pairformer_layer_forward, src/foldjax/models/boltz2/models/trunk_blocks/
// pairformer.py:100-206, and the lax.scan over stacked layer parameters that drives it
// (pairformer.py:30-100, src/foldjax/models/_stacking.py). Op order and residuals:
//
//   z += tri_mul_out(z);  z += tri_mul_in(z);  z += tri_att_start(z);  z += tri_att_end(z)
//   z += transition_z(z)
//   s += attention_pair_bias(LN(s), z, mask, k_in = LN(s));  s += transition_s(s)
//
// The pair track is bf16 on the tensor cores (the entry points of this library, residual adds
// fused into their output stages); the single track is float32, as the reference promotes it
// (pairformer.py:182-206), with bf16 parameters. One call per block removes the per-op host
// round trips; one call per trunk replaces the scan.
#include <cuda_bf16.h>

#include "host.cuh"

namespace b200 {
namespace {

// ---- single-track float32 helpers (rows of c_s channels; N x 384 values: tiny next to z)
// One warp per row: LN with bf16 scale/bias, float32 statistics (_common.py:15-26 with a
// float32 input: no intermediate rounding).
__global__ void ln_rows_kernel(const float* __restrict__ x, int rows, int c, const __nv_bfloat16* __restrict__ scale,
                               const __nv_bfloat16* __restrict__ bias, float eps, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const float* src = x + static_cast<long long>(row) * c;
  float s = 0.f;
  for (int i = lane; i < c; i += 32) s += src[i];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
  const float mean = s / c;
  float q = 0.f;
  for (int i = lane; i < c; i += 32) {
    const float v = src[i] - mean;
    q += v * v;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) q += __shfl_xor_sync(0xffffffffu, q, d);
  const float rstd = 1.0f / sqrtf(q / c + eps);
  float* dst = out + static_cast<long long>(row) * c;
  for (int i = lane; i < c; i += 32)
    dst[i] = (src[i] - mean) * rstd * __bfloat162float(scale[i]) + __bfloat162float(bias[i]);
}

// h = silu(a) * b, elementwise (transition.py:108)
__global__ void swiglu_kernel(const float* __restrict__ a, const float* __restrict__ b, long long total,
                              float* __restrict__ h) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float v = a[i];
  h[i] = v / (1.0f + expf(-v)) * b[i];
}

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, long long total,
                           float* __restrict__ out) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < total) out[i] = a[i] + b[i];
}

// dst[pair][:] = mask[pair] != 0 ? src[pair][:] : 0 for 128-channel bf16 pairs, one thread per
// 16-byte chunk. With src == dst only the dropped pairs are written. The pair gate of
// Protenix's block: z * pair_valid (protenix/models/trunk_blocks/pairformer.py:71-100).
__global__ void gate_pairs_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const float* __restrict__ mask,
                                  long long pairs) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= pairs * 16) return;
  const bool keep = mask[idx >> 4] != 0.f;
  if (!keep)
    dst[idx] = make_uint4(0u, 0u, 0u, 0u);
  else if (src != dst)
    dst[idx] = src[idx];
}

// s[row][:] = 0 where mask[row] == 0 (the single-track gate of the same block)
__global__ void gate_rows_kernel(float* __restrict__ s, const float* __restrict__ mask, int rows, int c) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx < static_cast<long long>(rows) * c && mask[idx / c] == 0.f) s[idx] = 0.f;
}

__global__ void fill_kernel(float* __restrict__ p, long long total, float v) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < total) p[i] = v;
}

struct Offsets {
  size_t off = 0;
  size_t take(size_t bytes) {
    off = (off + 1023) / 1024 * 1024;
    const size_t r = off;
    off += bytes;
    return r;
  }
  size_t total() const { return (off + 1023) / 1024 * 1024; }
};

struct Plan {
  size_t w, sub, sub_bytes, sn, upd, h1, h2, hs, ones, total;
};

Plan plan(int n, int c_s, int heads_s, int hidden_z, int hidden_s, bool single) {
  Plan p = {};
  Offsets o;
  p.w = o.take(static_cast<size_t>(n) * n * 128 * 2);
  size_t sub = b200tri_trimul_workspace_bytes(n);
  const size_t cand[3] = {b200tri_triatt_workspace_bytes(n), b200tri_pair_transition_workspace_bytes(hidden_z),
                          single ? b200tri_attention_pair_bias_workspace_bytes(n, c_s, heads_s) : 0};
  for (size_t c : cand) sub = c > sub ? c : sub;
  p.sub_bytes = sub;
  p.sub = o.take(sub);
  if (single) {
    const size_t act = static_cast<size_t>(n) * c_s * 4, hid = static_cast<size_t>(n) * hidden_s * 4;
    p.sn = o.take(act);
    p.upd = o.take(act);
    p.h1 = o.take(hid);
    p.h2 = o.take(hid);
    p.hs = o.take(hid);
    p.ones = o.take(static_cast<size_t>(n) * 4);
  }
  p.total = o.total();
  return p;
}

const void* leaf(const void* base, int layer, size_t elems) {
  return base ? static_cast<const uint8_t*>(base) + static_cast<size_t>(layer) * elems * 2 : nullptr;
}

// Block `layer` of parameters stacked leaf by leaf with a leading layer axis ([L, ...] bf16).
b200tri_pairformer_block_params unstack(const b200tri_pairformer_block_params& s, int layer, int c_s, int heads_s) {
  b200tri_pairformer_block_params p = s;
  auto mul = [&](b200tri_trimul_params& d, const b200tri_trimul_params& b) {
    d.norm_in_scale = leaf(b.norm_in_scale, layer, 128);
    d.norm_in_bias = leaf(b.norm_in_bias, layer, 128);
    d.p_in = leaf(b.p_in, layer, 128 * 256);
    d.g_in = leaf(b.g_in, layer, 128 * 256);
    d.norm_out_scale = leaf(b.norm_out_scale, layer, 128);
    d.norm_out_bias = leaf(b.norm_out_bias, layer, 128);
    d.p_out = leaf(b.p_out, layer, 128 * 128);
    d.g_out = leaf(b.g_out, layer, 128 * 128);
  };
  auto att = [&](b200tri_triatt_params& d, const b200tri_triatt_params& b) {
    d.norm_scale = leaf(b.norm_scale, layer, 128);
    d.norm_bias = leaf(b.norm_bias, layer, 128);
    d.w_bias = leaf(b.w_bias, layer, 128 * 4);
    d.w_q = leaf(b.w_q, layer, 128 * 128);
    d.w_k = leaf(b.w_k, layer, 128 * 128);
    d.w_v = leaf(b.w_v, layer, 128 * 128);
    d.w_g = leaf(b.w_g, layer, 128 * 128);
    d.w_o = leaf(b.w_o, layer, 128 * 128);
  };
  auto trn = [&](b200tri_transition_params& d, const b200tri_transition_params& b, size_t c) {
    d.norm_scale = leaf(b.norm_scale, layer, c);
    d.norm_bias = leaf(b.norm_bias, layer, c);
    d.fc1 = leaf(b.fc1, layer, c * b.hidden);
    d.fc2 = leaf(b.fc2, layer, c * b.hidden);
    d.fc3 = leaf(b.fc3, layer, c * b.hidden);
  };
  mul(p.tri_mul_out, s.tri_mul_out);
  mul(p.tri_mul_in, s.tri_mul_in);
  att(p.tri_att_start, s.tri_att_start);
  att(p.tri_att_end, s.tri_att_end);
  trn(p.transition_z, s.transition_z, 128);
  p.pre_norm_s_scale = leaf(s.pre_norm_s_scale, layer, c_s);
  p.pre_norm_s_bias = leaf(s.pre_norm_s_bias, layer, c_s);
  const size_t cc = static_cast<size_t>(c_s) * c_s;
  p.attention.proj_q = leaf(s.attention.proj_q, layer, cc);
  p.attention.proj_q_bias = leaf(s.attention.proj_q_bias, layer, c_s);
  p.attention.proj_k = leaf(s.attention.proj_k, layer, cc);
  p.attention.proj_v = leaf(s.attention.proj_v, layer, cc);
  p.attention.proj_g = leaf(s.attention.proj_g, layer, cc);
  p.attention.proj_z_norm_scale = leaf(s.attention.proj_z_norm_scale, layer, 128);
  p.attention.proj_z_norm_bias = leaf(s.attention.proj_z_norm_bias, layer, 128);
  p.attention.proj_z = leaf(s.attention.proj_z, layer, 128 * static_cast<size_t>(heads_s));
  p.attention.proj_o = leaf(s.attention.proj_o, layer, cc);
  trn(p.transition_s, s.transition_s, c_s);
  return p;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" size_t b200tri_pairformer_workspace_bytes(int32_t n, int32_t c_s, int32_t heads_s, int32_t hidden_z,
                                                     int32_t hidden_s) {
  if (n <= 0 || hidden_z <= 0) return 0;
  return plan(n, c_s, heads_s, hidden_z, hidden_s, c_s > 0).total + 1024;
}

extern "C" int b200tri_pairformer_forward(const b200tri_pairformer_args* a, b200tri_stream_t stream_) {
  B200_REQUIRE(a != nullptr && a->params != nullptr, B200TRI_ERR_INVALID, "pairformer: null args or params");
  B200_REQUIRE(a->n > 0 && a->n_blocks >= 1, B200TRI_ERR_INVALID, "pairformer: n and n_blocks must be positive");
  B200_REQUIRE(a->z_in && a->z_out, B200TRI_ERR_INVALID, "pairformer: z_in/z_out must not be null");
  const bool single = a->s_in != nullptr;
  B200_REQUIRE(!single || (a->s_out && a->c_s > 0 && a->heads_s > 0), B200TRI_ERR_INVALID,
               "pairformer: the single track needs s_out, c_s and heads_s");
  const b200tri_pairformer_block_params& first = a->params[0];
  const int hidden_z = first.transition_z.hidden, hidden_s = single ? first.transition_s.hidden : 0;
  B200_REQUIRE(hidden_z > 0 && (!single || hidden_s > 0), B200TRI_ERR_INVALID, "pairformer: transition widths missing");
  const Plan pl = plan(a->n, a->c_s, a->heads_s, hidden_z, hidden_s, single);
  B200_REQUIRE(a->workspace && a->workspace_bytes >= pl.total, B200TRI_ERR_WORKSPACE,
               "pairformer: workspace of %zu bytes needed, got %zu", pl.total, a->workspace_bytes);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 1023) == 0, B200TRI_ERR_INVALID,
               "pairformer: workspace must be 1024-byte aligned");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  void* w = ws + pl.w;
  const int n = a->n, c_s = a->c_s;
  const long long act = static_cast<long long>(n) * c_s;
  const float* token_mask = a->mask;
  if (single && !token_mask) {
    float* ones = reinterpret_cast<float*>(ws + pl.ones);
    count_launch();
    fill_kernel<<<(n + 255) / 256, 256, 0, stream>>>(ones, n, 1.0f);
    B200_CUDA_OK(cudaGetLastError());
    token_mask = ones;
  }

  const void* z_cur = a->z_in;
  const float* s_cur = a->s_in;
  const long long pairs = static_cast<long long>(n) * n;
  const bool gate = a->pair_gate != 0 && a->pair_mask != nullptr;
  auto gate_pairs = [&](const void* src, void* dst) -> int {
    count_launch();
    gate_pairs_kernel<<<static_cast<unsigned>((pairs * 16 + 255) / 256), 256, 0, stream>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), a->pair_mask, pairs);
    B200_CUDA_OK(cudaGetLastError());
    return B200TRI_OK;
  };
  auto gate_rows = [&](float* sv) -> int {
    count_launch();
    gate_rows_kernel<<<static_cast<unsigned>((act + 255) / 256), 256, 0, stream>>>(sv, token_mask, n, c_s);
    B200_CUDA_OK(cudaGetLastError());
    return B200TRI_OK;
  };
  for (int layer = 0; layer < a->n_blocks; ++layer) {
    const b200tri_pairformer_block_params P =
        a->stacked ? unstack(first, layer, c_s, a->heads_s) : a->params[layer];
    int rc;
    // ---- pair track: the four triangle updates ping-pong between z_out and w (the first one
    // reads the caller's z_in), residual adds fused; with the pair gate, dropped pairs are
    // zeroed before the first update and after every update
    if (gate && layer == 0) {
      if ((rc = gate_pairs(z_cur, a->z_out))) return rc;  // a gated copy, or in place when they alias
      z_cur = a->z_out;
    }
    for (int k = 0; k < 4; ++k) {
      // Boltz-2 / Protenix / OpenFold3 default: multiplications first; attention_first swaps the halves
      const int op = a->attention_first ? (k + 2) % 4 : k;  // 0 out, 1 in, 2 start, 3 end
      void* dst = z_cur == w ? a->z_out : w;
      if (op < 2) {
        const b200tri_trimul_params& m = op == 0 ? P.tri_mul_out : P.tri_mul_in;
        b200tri_trimul_args t = {};
        t.n = n;
        t.incoming = op;
        t.eps = a->eps;
        t.x = z_cur;
        t.mask = a->pair_mask;
        t.norm_in_scale = m.norm_in_scale;
        t.norm_in_bias = m.norm_in_bias;
        t.p_in = m.p_in;
        t.g_in = m.g_in;
        t.norm_out_scale = m.norm_out_scale;
        t.norm_out_bias = m.norm_out_bias;
        t.p_out = m.p_out;
        t.g_out = m.g_out;
        t.residual = t.x;
        t.out = dst;
        t.workspace = ws + pl.sub;
        t.workspace_bytes = pl.sub_bytes;
        if ((rc = b200tri_trimul_forward(&t, stream_))) return rc;
      } else {
        const b200tri_triatt_params& m = op == 2 ? P.tri_att_start : P.tri_att_end;
        b200tri_triatt_args t = {};
        t.n = n;
        t.starting = op == 2;
        t.heads = 4;
        t.head_dim = 32;
        t.inf = a->tri_inf;
        t.eps = a->eps;
        t.x = z_cur;
        t.mask = a->pair_mask;
        t.norm_scale = m.norm_scale;
        t.norm_bias = m.norm_bias;
        t.w_bias = m.w_bias;
        t.w_q = m.w_q;
        t.w_k = m.w_k;
        t.w_v = m.w_v;
        t.w_g = m.w_g;
        t.w_o = m.w_o;
        t.residual = t.x;
        t.out = dst;
        t.workspace = ws + pl.sub;
        t.workspace_bytes = pl.sub_bytes;
        if ((rc = b200tri_triatt_forward(&t, stream_))) return rc;
      }
      if (gate && (rc = gate_pairs(dst, dst))) return rc;
      z_cur = dst;
    }
    // four updates from z_in (or z_out) end in z_out
    {
      b200tri_pair_transition_args t = {};
      t.rows = static_cast<int64_t>(n) * n;
      t.channels = 128;
      t.hidden = P.transition_z.hidden;
      t.eps = a->eps;
      t.x = a->z_out;
      t.norm_scale = P.transition_z.norm_scale;
      t.norm_bias = P.transition_z.norm_bias;
      t.fc1 = P.transition_z.fc1;
      t.fc2 = P.transition_z.fc2;
      t.fc3 = P.transition_z.fc3;
      t.residual = a->z_out;
      t.out = a->z_out;  // row-local: in place
      t.workspace = ws + pl.sub;
      t.workspace_bytes = pl.sub_bytes;
      t.row_mask = a->mask_transition ? a->pair_mask : nullptr;
      if ((rc = b200tri_pair_transition(&t, stream_))) return rc;
      if (gate && (rc = gate_pairs(a->z_out, a->z_out))) return rc;
    }
    z_cur = a->z_out;
    if (!single) continue;

    // ---- single track, float32
    float* sn = reinterpret_cast<float*>(ws + pl.sn);
    float* upd = reinterpret_cast<float*>(ws + pl.upd);
    float* h1 = reinterpret_cast<float*>(ws + pl.h1);
    float* h2 = reinterpret_cast<float*>(ws + pl.h2);
    float* hs = reinterpret_cast<float*>(ws + pl.hs);
    count_launch();
    ln_rows_kernel<<<(n * 32 + 255) / 256, 256, 0, stream>>>(
        s_cur, n, c_s, static_cast<const __nv_bfloat16*>(P.pre_norm_s_scale),
        static_cast<const __nv_bfloat16*>(P.pre_norm_s_bias), a->eps, sn);
    B200_CUDA_OK(cudaGetLastError());
    b200tri_attention_pair_bias_args t = {};
    t.n = n;
    t.c_s = c_s;
    t.c_z = 128;
    t.heads = a->heads_s;
    t.eps = a->eps;
    t.inf = a->att_inf;
    t.s = sn;
    t.k_in = sn;
    t.z = a->z_out;
    t.mask = token_mask;
    t.proj_q = P.attention.proj_q;
    t.proj_q_bias = P.attention.proj_q_bias;
    t.proj_k = P.attention.proj_k;
    t.proj_v = P.attention.proj_v;
    t.proj_g = P.attention.proj_g;
    t.proj_z_norm_scale = P.attention.proj_z_norm_scale;
    t.proj_z_norm_bias = P.attention.proj_z_norm_bias;
    t.proj_z = P.attention.proj_z;
    t.proj_o = P.attention.proj_o;
    t.out = upd;
    t.workspace = ws + pl.sub;
    t.workspace_bytes = pl.sub_bytes;
    if ((rc = b200tri_attention_pair_bias(&t, stream_))) return rc;
    count_launch();
    add_kernel<<<static_cast<unsigned>((act + 255) / 256), 256, 0, stream>>>(s_cur, upd, act, a->s_out);
    B200_CUDA_OK(cudaGetLastError());
    if (gate && (rc = gate_rows(a->s_out))) return rc;
    // transition_s: LN -> fc1 | fc2 -> silu(fc1) * fc2 -> fc3, added to s (transition.py:99-112)
    const int hid = P.transition_s.hidden;
    count_launch(2);
    ln_rows_kernel<<<(n * 32 + 255) / 256, 256, 0, stream>>>(
        a->s_out, n, c_s, static_cast<const __nv_bfloat16*>(P.transition_s.norm_scale),
        static_cast<const __nv_bfloat16*>(P.transition_s.norm_bias), a->eps, sn);
    B200_CUDA_OK(cudaGetLastError());
    if ((rc = launch_linear_f32(sn, nullptr, P.transition_s.fc1, nullptr, n, c_s, hid, 0, nullptr, h1, stream))) return rc;
    if ((rc = launch_linear_f32(sn, nullptr, P.transition_s.fc2, nullptr, n, c_s, hid, 0, nullptr, h2, stream))) return rc;
    const long long hact = static_cast<long long>(n) * hid;
    swiglu_kernel<<<static_cast<unsigned>((hact + 255) / 256), 256, 0, stream>>>(h1, h2, hact, hs);
    B200_CUDA_OK(cudaGetLastError());
    if ((rc = launch_linear_f32(hs, nullptr, P.transition_s.fc3, nullptr, n, hid, c_s, 0, a->s_out, a->s_out, stream)))
      return rc;
    if (gate && (rc = gate_rows(a->s_out))) return rc;
    s_cur = a->s_out;
  }
  return B200TRI_OK;
}
