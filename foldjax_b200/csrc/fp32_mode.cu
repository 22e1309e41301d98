// float32 mode of the two triangle ops: float32 in, float32 parameters, float32 out.
//
// The reference's default contraction precision is float32 (triangle_multiplication_forward,
// src/foldjax/models/boltz2/models/triangle/triangle.py:95-96, casts the gated projections to
// float32 before the einsum) and a float32 trunk runs every step of both ops in float32. This
// file is that mode: a correctness mode with a 1e-4 bar, not a throughput mode.
//
//  * The triangle contraction, the one dense cubic step of the multiplicative update, stays on
//    the tensor cores: each float32 operand is split into three bf16 pieces (hi + mid + lo carry
//    24 significand bits) and the six products that matter - hi.hi, hi.mid, mid.hi, mid.mid,
//    hi.lo, lo.hi - are accumulated in float32 by the bf16 contraction kernel
//    (b200tri_trimul_contract, accumulate-in / float32-out), smallest terms first.
//  * Layer norms, the 128-wide projections, gates, the softmax and the attention products are
//    plain float32 CUDA-core kernels (IEEE expf, no fast-math forms): at the sizes this mode is
//    meant for (the N = 256 config) they are a few milliseconds.
#include <math.h>

#include "host.cuh"
#include "tc.cuh"

namespace b200 {
namespace {

constexpr int C = 128;

// ------------------------------------------------------------------ layer norm + gather
// xn[(o * n_inner + t)][:] = LN(x[o * xs_o + t * xs_i + :]); one warp per pair.
__global__ void ln_gather_f32_kernel(const float* __restrict__ x, long long xs_o, long long xs_i, int n_outer,
                                     int n_inner, const float* __restrict__ scale, const float* __restrict__ bias,
                                     float eps, float* __restrict__ xn) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long pairs = static_cast<long long>(n_outer) * n_inner;
  if (warp >= pairs) return;
  const int o = static_cast<int>(warp / n_inner), t = static_cast<int>(warp % n_inner);
  const float4 v = *reinterpret_cast<const float4*>(x + o * xs_o + t * xs_i + lane * 4);
  float s = v.x + v.y + v.z + v.w;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
  const float mean = s / C;
  const float4 c = make_float4(v.x - mean, v.y - mean, v.z - mean, v.w - mean);
  float q = c.x * c.x + c.y * c.y + c.z * c.z + c.w * c.w;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) q += __shfl_xor_sync(0xffffffffu, q, d);
  const float rstd = 1.0f / sqrtf(q / C + eps);
  const float4 g = *reinterpret_cast<const float4*>(scale + lane * 4);
  const float4 b = *reinterpret_cast<const float4*>(bias + lane * 4);
  float4 r;
  r.x = c.x * rstd * g.x + b.x;
  r.y = c.y * rstd * g.y + b.y;
  r.z = c.z * rstd * g.z + b.z;
  r.w = c.w * rstd * g.w + b.w;
  *reinterpret_cast<float4*>(xn + warp * C + lane * 4) = r;
}

// --------------------------------------------------------------------------- float32 GEMM
// out[row(m)][n] = sum_k a[m][k] * w[k][n] (+ res[row(m)][n]); a is [M][K] dense, w [K][N] dense.
// Output rows are addressed as (m / rows_inner) * s_outer + (m % rows_inner) * s_inner, which
// lets the last projection of the attention write straight through the caller's strides.
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ w, long long M, int K, int N,
                float* __restrict__ out, const float* __restrict__ res, int rows_inner, long long s_outer,
                long long s_inner) {
  __shared__ float as[16][64 + 1];
  __shared__ float ws[16][64];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const long long m0 = static_cast<long long>(blockIdx.y) * 64;
  const int n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int idx = threadIdx.x; idx < 64 * 16; idx += 256) {
      const int r = idx >> 4, c = idx & 15;
      const long long m = m0 + r;
      as[c][r] = (m < M && k0 + c < K) ? a[m * K + k0 + c] : 0.f;
    }
    for (int idx = threadIdx.x; idx < 16 * 64; idx += 256) {
      const int r = idx >> 6, c = idx & 63;
      ws[r][c] = (k0 + r < K && n0 + c < N) ? w[static_cast<long long>(k0 + r) * N + n0 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float av[4], bv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        av[e] = as[k][ty * 4 + e];
        bv[e] = ws[k][tx * 4 + e];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long m = m0 + ty * 4 + i;
    if (m >= M) continue;
    const long long row = (m / rows_inner) * s_outer + (m % rows_inner) * s_inner;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[row + n] = acc[i][j] + (res ? res[row + n] : 0.f);
    }
  }
}

int gemm_f32(const float* a, const float* w, long long M, int K, int N, float* out, cudaStream_t stream,
             const float* res = nullptr, int rows_inner = 0, long long s_outer = 0, long long s_inner = 0) {
  if (rows_inner <= 0) {  // dense [M][N]
    rows_inner = 1;
    s_outer = N;
    s_inner = 0;
  }
  dim3 grid(static_cast<unsigned>((N + 63) / 64), static_cast<unsigned>((M + 63) / 64));
  count_launch();
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(a, w, M, K, N, out, res, rows_inner, s_outer, s_inner);
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}

__device__ __forceinline__ float sigmoid_exact(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------- tri-mult: gate + split
// v = sigmoid(g) * p * mask for the 256 projected channels of a pair; channels 0..127 are a,
// 128..255 are b (triangle.py:102). Each value is written as three bf16 pieces into
// piece-major, channel-major planes [piece][channel][o][ld] - the layout the tensor-core
// contraction reads. One block = one row o and 32 consecutive t; shared memory turns the
// channel-contiguous reads into t-contiguous writes.
__global__ void __launch_bounds__(256)
glu_split_kernel(const float* __restrict__ p, const float* __restrict__ g, const float* __restrict__ mask,
                 long long ms_o, long long ms_i, int n_outer, int n_inner, int ld, __nv_bfloat16* __restrict__ a,
                 __nv_bfloat16* __restrict__ b) {
  __shared__ float tile[32][256 + 1];
  const int o = blockIdx.y, t0 = blockIdx.x * 32;
  for (int idx = threadIdx.x; idx < 32 * 256; idx += 256) {
    const int tt = idx >> 8, c = idx & 255;
    const int t = t0 + tt;
    float v = 0.f;
    if (t < n_inner) {
      const long long pair = static_cast<long long>(o) * n_inner + t;
      const float m = mask ? mask[o * ms_o + t * ms_i] : 1.0f;
      v = sigmoid_exact(g[pair * 256 + c]) * p[pair * 256 + c] * m;
    }
    tile[tt][c] = v;
  }
  __syncthreads();
  const long long plane = static_cast<long long>(n_outer) * ld;  // one channel
  const long long piece = 128 * plane;
  for (int idx = threadIdx.x; idx < 32 * 256; idx += 256) {
    const int c = idx >> 5, tt = idx & 31;
    const int t = t0 + tt;
    if (t >= ld) continue;
    const float v = t < n_inner ? tile[tt][c] : 0.f;  // pitch padding is zero: it is read as k
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
    __nv_bfloat16* dst = (c < 128 ? a : b) + static_cast<long long>(c & 127) * plane + static_cast<long long>(o) * ld + t;
    dst[0] = hi;
    dst[piece] = mid;
    dst[2 * piece] = lo;
  }
}

// ------------------------------------------------------------ tri-mult: LN of the contraction
// tn[(i * n + j)][:] = LN_out(t[:, i, j]) with t channel-major float32 [128][n][ld].
// One block = one row i and 32 consecutive j (a t-contiguous read per channel).
__global__ void __launch_bounds__(256)
ln_channel_major_kernel(const float* __restrict__ t, int n, int ld, const float* __restrict__ scale,
                        const float* __restrict__ bias, float eps, float* __restrict__ tn) {
  __shared__ float tile[128][32 + 1];
  const int i = blockIdx.y, j0 = blockIdx.x * 32;
  for (int idx = threadIdx.x; idx < 128 * 32; idx += 256) {
    const int c = idx >> 5, jj = idx & 31;
    const int j = j0 + jj;
    tile[c][jj] = j < n ? t[(static_cast<long long>(c) * n + i) * ld + j] : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int jj = warp; jj < 32; jj += 8) {
    const int j = j0 + jj;
    if (j >= n) continue;
    float v[4];
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[e] = tile[lane * 4 + e][jj];
      s += v[e];
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    const float mean = s / C;
    float q = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[e] -= mean;
      q += v[e] * v[e];
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) q += __shfl_xor_sync(0xffffffffu, q, d);
    const float rstd = 1.0f / sqrtf(q / C + eps);
    float4 r;
    r.x = v[0] * rstd * scale[lane * 4 + 0] + bias[lane * 4 + 0];
    r.y = v[1] * rstd * scale[lane * 4 + 1] + bias[lane * 4 + 1];
    r.z = v[2] * rstd * scale[lane * 4 + 2] + bias[lane * 4 + 2];
    r.w = v[3] * rstd * scale[lane * 4 + 3] + bias[lane * 4 + 3];
    *reinterpret_cast<float4*>(tn + (static_cast<long long>(i) * n + j) * C + lane * 4) = r;
  }
}

// out[i][j][c] = o[(i * n + j)][c] * sigmoid(gate[(gi * n + gj)][c]) (+ residual), where the gate
// rows live in the projection frame: (gi, gj) = (i, j), or (j, i) when that frame is transposed.
__global__ void gate_out_kernel(const float* __restrict__ o, const float* __restrict__ gate, int n, int transposed,
                                const float* __restrict__ residual, float* __restrict__ out) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(n) * n * C;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % C);
  const long long pair = idx / C;
  const int i = static_cast<int>(pair / n), j = static_cast<int>(pair % n);
  const long long gp = transposed ? static_cast<long long>(j) * n + i : pair;
  const float v = o[idx] * sigmoid_exact(gate[gp * C + c]);
  out[idx] = residual ? residual[idx] + v : v;
}

// in place: o[m][c] *= sigmoid(g[m][c])
__global__ void mul_sigmoid_kernel(float* __restrict__ o, const float* __restrict__ g, long long total) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx < total) o[idx] *= sigmoid_exact(g[idx]);
}

// ------------------------------------------------------------------- tri-attn: float32 core
// One block = (row o, head h, 128 queries); one thread per query; K and V of the row stream
// through shared memory 32 keys at a time. Scores follow the reference's order and precision
// (triangle_attention.py:449-455): (q.k + mask_bias) + tri_bias in float32, softmax in
// float32, P.v in float32. q is divided by sqrt(d) first (:399-400).
constexpr int AQ = 128, AK = 32, HD = 32;
__global__ void __launch_bounds__(AQ)
att_core_f32_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                    const float* __restrict__ bias, const float* __restrict__ mask, long long ms_o, long long ms_k,
                    float inf, int n_outer, int n, int heads, float* __restrict__ out) {
  __shared__ float ks[AK][HD], vs[AK][HD], mb[AK];
  const int o = blockIdx.z, h = blockIdx.y;
  const int j = blockIdx.x * AQ + threadIdx.x;
  const bool live = j < n;
  const int width = heads * HD;
  const float q_scale = sqrtf(static_cast<float>(HD));
  float qr[HD], acc[HD];
  const float* qrow = q + (static_cast<long long>(o) * n + (live ? j : 0)) * width + h * HD;
#pragma unroll
  for (int d = 0; d < HD; ++d) {
    qr[d] = qrow[d] / q_scale;
    acc[d] = 0.f;
  }
  float m_run = -INFINITY, l_run = 0.f;
  for (int k0 = 0; k0 < n; k0 += AK) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < AK * HD; idx += AQ) {
      const int r = idx / HD, d = idx % HD;
      const int kk = k0 + r;
      const long long src = (static_cast<long long>(o) * n + kk) * width + h * HD + d;
      ks[r][d] = kk < n ? k[src] : 0.f;
      vs[r][d] = kk < n ? v[src] : 0.f;
    }
    if (threadIdx.x < AK) {
      const int kk = k0 + threadIdx.x;
      mb[threadIdx.x] = kk < n ? (mask ? inf * (mask[o * ms_o + kk * ms_k] - 1.0f) : 0.0f) : -INFINITY;
    }
    __syncthreads();
    if (!live) continue;
    float sc[AK];
    float mx = m_run;
#pragma unroll
    for (int r = 0; r < AK; ++r) {
      float s = 0.f;
#pragma unroll
      for (int d = 0; d < HD; ++d) s = fmaf(qr[d], ks[r][d], s);
      const int kk = k0 + r;
      const float tb = kk < n ? bias[(static_cast<long long>(j) * n + kk) * heads + h] : 0.f;
      s = (s + mb[r]) + tb;
      sc[r] = s;
      mx = fmaxf(mx, s);
    }
    const float corr = expf(m_run - mx);  // 0 on the first tile
    l_run *= corr;
#pragma unroll
    for (int d = 0; d < HD; ++d) acc[d] *= corr;
#pragma unroll
    for (int r = 0; r < AK; ++r) {
      const float pexp = expf(sc[r] - mx);
      l_run += pexp;
#pragma unroll
      for (int d = 0; d < HD; ++d) acc[d] = fmaf(pexp, vs[r][d], acc[d]);
    }
    m_run = mx;
  }
  if (live) {
    float* dst = out + (static_cast<long long>(o) * n + j) * width + h * HD;
#pragma unroll
    for (int d = 0; d < HD; ++d) dst[d] = acc[d] / l_run;
  }
}

struct Carve {
  Carver c;
  explicit Carve(void* p) : c(p) {}
  float* f32(size_t n) { return c.take<float>(n); }
  __nv_bfloat16* bf16(size_t n) { return c.take<__nv_bfloat16>(n); }
};

size_t trimul_f32_bytes(int32_t n) {
  Carve w(nullptr);
  const size_t pairs = static_cast<size_t>(n) * n;
  const size_t ld = round_up(n, 64);
  w.f32(pairs * C);        // xn
  w.f32(pairs * 256);      // p
  w.f32(pairs * 256);      // g
  w.bf16(3 * 128 * n * ld);  // a pieces
  w.bf16(3 * 128 * n * ld);  // b pieces
  w.f32(128 * n * ld);     // contraction, channel-major
  w.f32(pairs * C);        // tn
  w.f32(pairs * C);        // o
  w.f32(pairs * C);        // gate
  return w.c.total() + 1024;
}

size_t triatt_f32_bytes(int32_t n) {
  Carve w(nullptr);
  const size_t pairs = static_cast<size_t>(n) * n;
  for (int i = 0; i < 6; ++i) w.f32(pairs * C);  // xn, q, k, v, gate, o
  w.f32(pairs * 4);                              // bias
  return w.c.total() + 1024;
}

}  // namespace

size_t trimul_workspace_bytes_f32(int32_t n) { return n > 0 ? trimul_f32_bytes(n) : 0; }
size_t triatt_workspace_bytes_f32(int32_t n) { return n > 0 ? triatt_f32_bytes(n) : 0; }

int trimul_forward_f32(const b200tri_trimul_args* a, cudaStream_t stream) {
  const int n = a->n;
  const long long pairs = static_cast<long long>(n) * n;
  const int ld = round_up(n, 64);
  Carve w(a->workspace);
  float* xn = w.f32(pairs * C);
  float* p = w.f32(pairs * 256);
  float* g = w.f32(pairs * 256);
  __nv_bfloat16* ap = w.bf16(static_cast<size_t>(3) * 128 * n * ld);
  __nv_bfloat16* bp = w.bf16(static_cast<size_t>(3) * 128 * n * ld);
  float* t = w.f32(static_cast<size_t>(128) * n * ld);
  float* tn = w.f32(pairs * C);
  float* o = w.f32(pairs * C);
  float* gate = w.f32(pairs * C);
  const float* x = static_cast<const float*>(a->x);
  // projection frame (o, t): the outgoing update reads x[o][t], the incoming one x[t][o], so
  // both contract over t (triangle.py:231, :239).
  const long long xs_o = a->incoming ? C : static_cast<long long>(n) * C;
  const long long xs_i = a->incoming ? static_cast<long long>(n) * C : C;
  const long long ms_o = a->incoming ? 1 : n, ms_i = a->incoming ? n : 1;
  count_launch();
  ln_gather_f32_kernel<<<static_cast<unsigned>((pairs * 32 + 255) / 256), 256, 0, stream>>>(
      x, xs_o, xs_i, n, n, static_cast<const float*>(a->norm_in_scale), static_cast<const float*>(a->norm_in_bias),
      a->eps, xn);
  B200_CUDA_OK(cudaGetLastError());
  int rc = gemm_f32(xn, static_cast<const float*>(a->p_in), pairs, C, 256, p, stream);
  if (rc) return rc;
  rc = gemm_f32(xn, static_cast<const float*>(a->g_in), pairs, C, 256, g, stream);
  if (rc) return rc;
  count_launch();
  glu_split_kernel<<<dim3(static_cast<unsigned>(ld / 32), static_cast<unsigned>(n)), 256, 0, stream>>>(
      p, g, a->mask, ms_o, ms_i, n, n, ld, ap, bp);
  B200_CUDA_OK(cudaGetLastError());
  // six bf16 products, float32 accumulation carried from call to call, smallest terms first
  const long long piece = static_cast<long long>(128) * n * ld;
  const int order[6][2] = {{2, 0}, {0, 2}, {1, 1}, {1, 0}, {0, 1}, {0, 0}};
  for (int s = 0; s < 6; ++s) {
    b200tri_trimul_contract_args ca = {};
    ca.n_i = ca.n_j = ca.n_k = n;
    ca.n_src = 1;
    ca.a = ap + order[s][0] * piece;
    ca.b = bp + order[s][1] * piece;
    ca.a_ld = ca.b_ld = ca.out_ld = ld;
    ca.a_chan_stride = ca.b_chan_stride = ca.out_chan_stride = static_cast<int64_t>(n) * ld;
    ca.a_src_stride = ca.b_src_stride = piece;
    ca.acc_in = s ? t : nullptr;
    ca.out_f32 = t;
    rc = b200tri_trimul_contract(&ca, reinterpret_cast<b200tri_stream_t>(stream));
    if (rc) return rc;
  }
  count_launch();
  ln_channel_major_kernel<<<dim3(static_cast<unsigned>((n + 31) / 32), static_cast<unsigned>(n)), 256, 0, stream>>>(
      t, n, ld, static_cast<const float*>(a->norm_out_scale), static_cast<const float*>(a->norm_out_bias), a->eps, tn);
  B200_CUDA_OK(cudaGetLastError());
  rc = gemm_f32(tn, static_cast<const float*>(a->p_out), pairs, C, C, o, stream);
  if (rc) return rc;
  rc = gemm_f32(xn, static_cast<const float*>(a->g_out), pairs, C, C, gate, stream);
  if (rc) return rc;
  count_launch();
  gate_out_kernel<<<static_cast<unsigned>((pairs * C + 255) / 256), 256, 0, stream>>>(
      o, gate, n, a->incoming ? 1 : 0, static_cast<const float*>(a->residual), static_cast<float*>(a->out));
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}

int triatt_forward_f32(const b200tri_triatt_args* a, cudaStream_t stream) {
  const int n = a->n;
  const long long pairs = static_cast<long long>(n) * n;
  Carve w(a->workspace);
  float* xn = w.f32(pairs * C);
  float* q = w.f32(pairs * C);
  float* k = w.f32(pairs * C);
  float* v = w.f32(pairs * C);
  float* gate = w.f32(pairs * C);
  float* o = w.f32(pairs * C);
  float* bias = w.f32(pairs * 4);
  const float* x = static_cast<const float*>(a->x);
  // attention frame (o = row, t = position inside the row): the ending node is the starting
  // node on the transposed pair tensor and mask (triangle_attention.py:128-130, :160-161)
  const long long s_o = a->starting ? static_cast<long long>(n) * C : C;
  const long long s_i = a->starting ? C : static_cast<long long>(n) * C;
  count_launch();
  ln_gather_f32_kernel<<<static_cast<unsigned>((pairs * 32 + 255) / 256), 256, 0, stream>>>(
      x, s_o, s_i, n, n, static_cast<const float*>(a->norm_scale), static_cast<const float*>(a->norm_bias), a->eps, xn);
  B200_CUDA_OK(cudaGetLastError());
  int rc;
  if ((rc = gemm_f32(xn, static_cast<const float*>(a->w_q), pairs, C, C, q, stream))) return rc;
  if ((rc = gemm_f32(xn, static_cast<const float*>(a->w_k), pairs, C, C, k, stream))) return rc;
  if ((rc = gemm_f32(xn, static_cast<const float*>(a->w_v), pairs, C, C, v, stream))) return rc;
  if ((rc = gemm_f32(xn, static_cast<const float*>(a->w_g), pairs, C, C, gate, stream))) return rc;
  if ((rc = gemm_f32(xn, static_cast<const float*>(a->w_bias), pairs, C, a->heads, bias, stream))) return rc;
  count_launch();
  att_core_f32_kernel<<<dim3(static_cast<unsigned>((n + AQ - 1) / AQ), static_cast<unsigned>(a->heads),
                             static_cast<unsigned>(n)),
                        AQ, 0, stream>>>(q, k, v, bias, a->mask, a->starting ? n : 1, a->starting ? 1 : n, a->inf, n, n,
                                         a->heads, o);
  B200_CUDA_OK(cudaGetLastError());
  count_launch();
  mul_sigmoid_kernel<<<static_cast<unsigned>((pairs * C + 255) / 256), 256, 0, stream>>>(o, gate, pairs * C);
  B200_CUDA_OK(cudaGetLastError());
  return gemm_f32(o, static_cast<const float*>(a->w_o), pairs, C, C, static_cast<float*>(a->out), stream,
                  static_cast<const float*>(a->residual), n, s_o, s_i);
}

}  // namespace b200
