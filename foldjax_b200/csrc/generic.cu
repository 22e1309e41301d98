// The two triangle ops for every shape and element type the tensor-core specialisation
// (c_z = c_hidden = 128, 4 heads x 32, bf16) does not cover:
//
//  * the float32 trunk of the reference at the specialised shape (a correctness mode with a
//    1e-4 bar: triangle_multiplication_forward's default contraction precision is float32,
//    src/foldjax/models/boltz2/models/triangle/triangle.py:95-96);
//  * other call sites of the same ops - the template stacks (c_z = 64 with c_hidden = 128,
//    which the cuEquivariance kernel rejects, src/foldjax/models/protenix/models/triangle/
//    triangle.py:131-137), the 384-channel / 12-head structural refiner
//    (src/foldjax/models/opendde/structural_refiner.py:62), other head counts and widths -
//    in bf16 or float32.
//
// Structure. Layer norms, projections, gates, softmax and P.V are plain CUDA-core kernels in
// float32 arithmetic. The triangle contraction, the one cubic step of the multiplicative
// update, stays on the tensor cores: in bf16 the operands are the bf16 values themselves; in
// float32 each operand is split into three bf16 pieces (hi + mid + lo carry 24 significand
// bits) and the six products that matter - hi.hi, hi.mid, mid.hi, mid.mid, hi.lo, lo.hi - are
// accumulated in float32 by the bf16 contraction kernel, smallest terms first.
//
// With a bf16 trunk every point where the reference's bf16 arrays round (after each matmul,
// the sigmoid, each elementwise product or sum, the two steps of the layer-norm affine,
// q / sqrt(d), the contraction and the attention output) is rounded here too (`Rb`), so the
// results follow the same recipe as the specialised kernels; with float32 nothing is rounded.
#include <cuda_bf16.h>
#include <math.h>

#include <type_traits>

#include "host.cuh"
#include "tc.cuh"

namespace b200 {
namespace {

// Rounding policy of the trunk dtype.
template <bool BF>
struct Rb {
  static __device__ __forceinline__ float r(float v) { return BF ? round_bf16(v) : v; }
};

__device__ __forceinline__ float sigmoid_exact(float x) { return 1.0f / (1.0f + expf(-x)); }

// bf16 or float32 array -> float32 (parameters and the pair tensor of a bf16 trunk)
__global__ void to_f32_kernel(const __nv_bfloat16* __restrict__ src, long long total, float* __restrict__ dst) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < total) dst[i] = __bfloat162float(src[i]);
}

// ------------------------------------------------------------------ layer norm + gather
// xn[(o * n_inner + t)][:] = LN(x[o * xs_o + t * xs_i + :]); one warp per pair, any width c.
// X is float or __nv_bfloat16 (the caller's pair tensor is read as it is stored).
template <bool BF, typename X>
__global__ void ln_gather_kernel(const X* __restrict__ x, long long xs_o, long long xs_i, int n_outer, int n_inner,
                                 int c, const float* __restrict__ scale, const float* __restrict__ bias, float eps,
                                 float* __restrict__ xn) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long pairs = static_cast<long long>(n_outer) * n_inner;
  if (warp >= pairs) return;
  const int o = static_cast<int>(warp / n_inner), t = static_cast<int>(warp % n_inner);
  const X* src = x + o * xs_o + t * xs_i;
  float s = 0.f;
  for (int i = lane; i < c; i += 32) s += static_cast<float>(src[i]);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
  const float mean = s / c;
  float q = 0.f;
  for (int i = lane; i < c; i += 32) {
    const float v = static_cast<float>(src[i]) - mean;
    q += v * v;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) q += __shfl_xor_sync(0xffffffffu, q, d);
  const float rstd = 1.0f / sqrtf(q / c + eps);
  float* dst = xn + warp * c;
  for (int i = lane; i < c; i += 32) {
    const float normed = Rb<BF>::r((static_cast<float>(src[i]) - mean) * rstd);  // cast before the affine step
    dst[i] = Rb<BF>::r(Rb<BF>::r(normed * scale[i]) + bias[i]);
  }
}

// --------------------------------------------------------------------------- float32 GEMM
// out[row(m)][n] = R(sum_k a[m][k] * w[k][n]) (+ res); a is [M][K] dense, w [K][N] dense.
// Output rows are addressed as (m / rows_inner) * s_outer + (m % rows_inner) * s_inner, which
// lets the last projection of the attention write straight through the caller's strides.
// O is the output element type (float, or __nv_bfloat16 for the final result of a bf16 trunk).
template <bool BF, typename O>
__global__ void __launch_bounds__(256)
gemm_kernel(const float* __restrict__ a, const float* __restrict__ w, long long M, int K, int N, O* __restrict__ out,
            const O* __restrict__ res, int rows_inner, long long s_outer, long long s_inner) {
  __shared__ float as[16][64 + 1];
  __shared__ float ws[16][64];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const long long m0 = static_cast<long long>(blockIdx.x) * 64;  // rows on x: the pair count exceeds 65535 * 64
  const int n0 = blockIdx.y * 64;
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
      if (n >= N) continue;
      float v = Rb<BF>::r(acc[i][j]);
      if (res) v = Rb<BF>::r(v + static_cast<float>(res[row + n]));  // the caller's z + update
      out[row + n] = static_cast<O>(v);
    }
  }
}

template <bool BF, typename O = float>
int gemm(const float* a, const float* w, long long M, int K, int N, O* out, cudaStream_t stream, const O* res = nullptr,
         int rows_inner = 0, long long s_outer = 0, long long s_inner = 0) {
  if (rows_inner <= 0) {  // dense [M][N]
    rows_inner = 1;
    s_outer = N;
    s_inner = 0;
  }
  dim3 grid(static_cast<unsigned>((M + 63) / 64), static_cast<unsigned>((N + 63) / 64));
  count_launch();
  gemm_kernel<BF, O><<<grid, 256, 0, stream>>>(a, w, M, K, N, out, res, rows_inner, s_outer, s_inner);
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}

// ------------------------------------------------------------------- tri-mult: gate + split
// v = R(R(R(sigmoid(g)) * p) * mask) for the 2 * c_h projected channels of a pair; the first
// c_h are a, the rest b (triangle.py:102). Written as bf16 pieces into piece-major,
// channel-major planes [piece][channel][o][ld] with the channel count padded to `planes` (a
// multiple of 128: the tensor-core contraction walks 128 channels per call; padding planes
// stay zero). One block = one row o and 32 consecutive t; shared memory turns the
// channel-contiguous reads into t-contiguous writes, 64 channels at a time.
template <bool BF>
__global__ void __launch_bounds__(256)
glu_split_kernel(const float* __restrict__ p, const float* __restrict__ g, const float* __restrict__ mask,
                 long long ms_o, long long ms_i, int n_outer, int n_inner, int ld, int c_h, int planes, int pieces,
                 __nv_bfloat16* __restrict__ a, __nv_bfloat16* __restrict__ b) {
  __shared__ float tile[32][64 + 1];
  const int o = blockIdx.y, t0 = blockIdx.x * 32;
  const int width = 2 * c_h;
  const long long plane = static_cast<long long>(n_outer) * ld;  // one channel
  const long long piece = static_cast<long long>(planes) * plane;
  for (int c0 = 0; c0 < width; c0 += 64) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < 32 * 64; idx += 256) {
      const int tt = idx >> 6, cc = idx & 63;
      const int t = t0 + tt, c = c0 + cc;
      float v = 0.f;
      if (t < n_inner && c < width) {
        const long long pair = static_cast<long long>(o) * n_inner + t;
        const float m = mask ? Rb<BF>::r(mask[o * ms_o + t * ms_i]) : 1.0f;
        const float gate = Rb<BF>::r(sigmoid_exact(g[pair * width + c]));
        v = Rb<BF>::r(Rb<BF>::r(gate * p[pair * width + c]) * m);
      }
      tile[tt][cc] = v;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 32 * 64; idx += 256) {
      const int cc = idx >> 5, tt = idx & 31;
      const int t = t0 + tt, c = c0 + cc;
      if (t >= ld || c >= width) continue;
      const float v = t < n_inner ? tile[tt][cc] : 0.f;  // pitch padding is zero: it is read as k
      const int chan = c < c_h ? c : c - c_h;
      __nv_bfloat16* dst = (c < c_h ? a : b) + static_cast<long long>(chan) * plane + static_cast<long long>(o) * ld + t;
      const __nv_bfloat16 hi = __float2bfloat16_rn(v);
      dst[0] = hi;
      if (pieces == 3) {
        const float r1 = v - __bfloat162float(hi);
        const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
        dst[piece] = mid;
        dst[2 * piece] = __float2bfloat16_rn(r1 - __bfloat162float(mid));
      }
    }
  }
}

// ------------------------------------------------------------ tri-mult: LN of the contraction
// tn[(i * n + j)][:] = LN_out(R(t[:, i, j])) with t channel-major float32 [planes][n][ld]; the
// contraction is rounded to the trunk dtype before the layer norm (triangle.py:124-126).
// One warp per pair.
template <bool BF>
__global__ void ln_channel_major_kernel(const float* __restrict__ t, int n, int ld, int c_h,
                                        const float* __restrict__ scale, const float* __restrict__ bias, float eps,
                                        float* __restrict__ tn) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long pairs = static_cast<long long>(n) * n;
  if (warp >= pairs) return;
  const int i = static_cast<int>(warp / n), j = static_cast<int>(warp % n);
  const float* src = t + static_cast<long long>(i) * ld + j;
  const long long plane = static_cast<long long>(n) * ld;
  float s = 0.f;
  for (int c = lane; c < c_h; c += 32) s += Rb<BF>::r(src[c * plane]);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
  const float mean = s / c_h;
  float q = 0.f;
  for (int c = lane; c < c_h; c += 32) {
    const float v = Rb<BF>::r(src[c * plane]) - mean;
    q += v * v;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) q += __shfl_xor_sync(0xffffffffu, q, d);
  const float rstd = 1.0f / sqrtf(q / c_h + eps);
  float* dst = tn + warp * c_h;
  for (int c = lane; c < c_h; c += 32) {
    const float normed = Rb<BF>::r((Rb<BF>::r(src[c * plane]) - mean) * rstd);
    dst[c] = Rb<BF>::r(Rb<BF>::r(normed * scale[c]) + bias[c]);
  }
}

// out[i][j][c] = R(o[(i * n + j)][c] * R(sigmoid(gate[(gi * n + gj)][c]))) (+ residual), where the
// gate rows live in the projection frame: (gi, gj) = (i, j), or (j, i) when that frame is
// transposed.
template <bool BF, typename O>
__global__ void gate_out_kernel(const float* __restrict__ o, const float* __restrict__ gate, int n, int c_z,
                                int transposed, const O* __restrict__ residual, O* __restrict__ out) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(n) * n * c_z;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % c_z);
  const long long pair = idx / c_z;
  const int i = static_cast<int>(pair / n), j = static_cast<int>(pair % n);
  const long long gp = transposed ? static_cast<long long>(j) * n + i : pair;
  float v = Rb<BF>::r(o[idx] * Rb<BF>::r(sigmoid_exact(gate[gp * c_z + c])));
  if (residual) v = Rb<BF>::r(static_cast<float>(residual[idx]) + v);
  out[idx] = static_cast<O>(v);
}

// in place: o[m][c] = R(o[m][c] * R(sigmoid(g[m][c])))
template <bool BF>
__global__ void mul_sigmoid_kernel(float* __restrict__ o, const float* __restrict__ g, long long total) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx < total) o[idx] = Rb<BF>::r(o[idx] * Rb<BF>::r(sigmoid_exact(g[idx])));
}

// ------------------------------------------------------------------- tri-attn: attention core
// One block = (row o, head h, 128 queries); one thread per query; K and V of the row stream
// through shared memory 32 keys at a time. Scores follow the reference's order and precision
// (triangle_attention.py:449-455): (q.k + mask_bias) + tri_bias in float32, softmax in float32,
// P.v in float32, cast to the trunk dtype. q is divided by sqrt(d), evaluated and rounded in
// the trunk dtype, first (:399-400).
constexpr int AQ = 128, AK = 32;
template <bool BF, int HD>
__global__ void __launch_bounds__(AQ)
att_core_kernel_f32(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                    const float* __restrict__ bias, const float* __restrict__ mask, long long ms_o, long long ms_k,
                    float inf, int n, int heads, float* __restrict__ out) {
  __shared__ float ks[AK][HD], vs[AK][HD], mb[AK];
  const int o = blockIdx.z, h = blockIdx.y;
  const int j = blockIdx.x * AQ + threadIdx.x;
  const bool live = j < n;
  const int width = heads * HD;
  const float q_scale = Rb<BF>::r(sqrtf(static_cast<float>(HD)));
  float qr[HD], acc[HD];
  const float* qrow = q + (static_cast<long long>(o) * n + (live ? j : 0)) * width + h * HD;
#pragma unroll
  for (int d = 0; d < HD; ++d) {
    qr[d] = Rb<BF>::r(qrow[d] / q_scale);
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
    for (int d = 0; d < HD; ++d) dst[d] = Rb<BF>::r(acc[d] / l_run);
  }
}

template <bool BF>
int launch_att_core(int head_dim, dim3 grid, cudaStream_t stream, const float* q, const float* k, const float* v,
                    const float* bias, const float* mask, long long ms_o, long long ms_k, float inf, int n, int heads,
                    float* out) {
  count_launch();
  switch (head_dim) {
#define B200_CASE(HD)                                                                                      \
  case HD:                                                                                                 \
    att_core_kernel_f32<BF, HD><<<grid, AQ, 0, stream>>>(q, k, v, bias, mask, ms_o, ms_k, inf, n, heads, out); \
    break;
    B200_CASE(8)
    B200_CASE(16)
    B200_CASE(24)
    B200_CASE(32)
    B200_CASE(48)
    B200_CASE(64)
#undef B200_CASE
    default:
      set_error("triatt: head widths 8, 16, 24, 32, 48 and 64 are built (got %d)", head_dim);
      return B200TRI_ERR_UNSUPPORTED;
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
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

int planes_for(int c_h) { return round_up(c_h, 128); }

struct TrimulPlan {
  size_t xn, p, g, ap, bp, t, tn, o, gate, params, total;
};

TrimulPlan trimul_plan(int n, int c_z, int c_h, bool f32) {
  TrimulPlan pl;
  Offsets w;
  const size_t pairs = static_cast<size_t>(n) * n, ld = round_up(n, 64), planes = planes_for(c_h);
  const int pieces = f32 ? 3 : 1;
  pl.xn = w.take(pairs * c_z * 4);
  pl.p = w.take(pairs * 2 * c_h * 4);
  pl.g = w.take(pairs * 2 * c_h * 4);
  pl.ap = w.take(pieces * planes * n * ld * 2);
  pl.bp = w.take(pieces * planes * n * ld * 2);
  pl.t = w.take(planes * n * ld * 4);
  pl.tn = w.take(pairs * c_h * 4);
  pl.o = w.take(pairs * c_z * 4);
  pl.gate = w.take(pairs * c_z * 4);
  // float32 copies of the parameters of a bf16 trunk
  pl.params = w.take((2 * static_cast<size_t>(c_z) + 2 * c_h + 2 * static_cast<size_t>(c_z) * 2 * c_h +
                      static_cast<size_t>(c_h) * c_z + static_cast<size_t>(c_z) * c_z) * 4 + 8 * 1024);
  pl.total = w.total();
  return pl;
}

struct TriattPlan {
  size_t xn, q, k, v, gate, o, bias, params, total;
};

TriattPlan triatt_plan(int n, int c_z, int heads, int head_dim) {
  TriattPlan pl;
  Offsets w;
  const size_t pairs = static_cast<size_t>(n) * n, hd = static_cast<size_t>(heads) * head_dim;
  pl.xn = w.take(pairs * c_z * 4);
  pl.q = w.take(pairs * hd * 4);
  pl.k = w.take(pairs * hd * 4);
  pl.v = w.take(pairs * hd * 4);
  pl.gate = w.take(pairs * hd * 4);
  pl.o = w.take(pairs * hd * 4);
  pl.bias = w.take(pairs * heads * 4);
  pl.params = w.take((2 * static_cast<size_t>(c_z) + static_cast<size_t>(c_z) * heads + 4 * c_z * hd + hd * c_z) * 4 +
                     10 * 1024);
  pl.total = w.total();
  return pl;
}

// A parameter as float32: the caller's array itself (float32 trunk), or a converted copy
// carved from `scratch` (bf16 trunk).
struct ParamStage {
  uint8_t* scratch;
  size_t off = 0;
  bool f32;
  cudaStream_t stream;
  int rc = B200TRI_OK;
  const float* get(const void* p, size_t count) {
    if (f32) return static_cast<const float*>(p);
    off = (off + 255) / 256 * 256;
    float* dst = reinterpret_cast<float*>(scratch + off);
    off += count * 4;
    count_launch();
    to_f32_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(p), static_cast<long long>(count), dst);
    if (cudaGetLastError() != cudaSuccess) rc = B200TRI_ERR_CUDA;
    return dst;
  }
};

template <bool BF>
int trimul_generic(const b200tri_trimul_args* a, int c_z, int c_h, cudaStream_t stream) {
  using O = typename std::conditional<BF, __nv_bfloat16, float>::type;
  const int n = a->n;
  const long long pairs = static_cast<long long>(n) * n;
  const int ld = round_up(n, 64), planes = planes_for(c_h), pieces = BF ? 1 : 3;
  const TrimulPlan pl = trimul_plan(n, c_z, c_h, !BF);
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  float* xn = reinterpret_cast<float*>(ws + pl.xn);
  float* p = reinterpret_cast<float*>(ws + pl.p);
  float* g = reinterpret_cast<float*>(ws + pl.g);
  __nv_bfloat16* ap = reinterpret_cast<__nv_bfloat16*>(ws + pl.ap);
  __nv_bfloat16* bp = reinterpret_cast<__nv_bfloat16*>(ws + pl.bp);
  float* t = reinterpret_cast<float*>(ws + pl.t);
  float* tn = reinterpret_cast<float*>(ws + pl.tn);
  float* o = reinterpret_cast<float*>(ws + pl.o);
  float* gate = reinterpret_cast<float*>(ws + pl.gate);
  ParamStage ps{ws + pl.params, 0, !BF, stream};
  const float* ln_in_s = ps.get(a->norm_in_scale, c_z);
  const float* ln_in_b = ps.get(a->norm_in_bias, c_z);
  const float* p_in = ps.get(a->p_in, static_cast<size_t>(c_z) * 2 * c_h);
  const float* g_in = ps.get(a->g_in, static_cast<size_t>(c_z) * 2 * c_h);
  const float* ln_out_s = ps.get(a->norm_out_scale, c_h);
  const float* ln_out_b = ps.get(a->norm_out_bias, c_h);
  const float* p_out = ps.get(a->p_out, static_cast<size_t>(c_h) * c_z);
  const float* g_out = ps.get(a->g_out, static_cast<size_t>(c_z) * c_z);
  if (ps.rc) return ps.rc;
  // projection frame (o, t): the outgoing update reads x[o][t], the incoming one x[t][o], so
  // both contract over t (triangle.py:231, :239).
  const long long xs_o = a->incoming ? c_z : static_cast<long long>(n) * c_z;
  const long long xs_i = a->incoming ? static_cast<long long>(n) * c_z : c_z;
  const long long ms_o = a->incoming ? 1 : n, ms_i = a->incoming ? n : 1;
  count_launch();
  ln_gather_kernel<BF, O><<<static_cast<unsigned>((pairs * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const O*>(a->x), xs_o, xs_i, n, n, c_z, ln_in_s, ln_in_b, a->eps, xn);
  B200_CUDA_OK(cudaGetLastError());
  int rc;
  if ((rc = gemm<BF>(xn, p_in, pairs, c_z, 2 * c_h, p, stream))) return rc;
  if ((rc = gemm<BF>(xn, g_in, pairs, c_z, 2 * c_h, g, stream))) return rc;
  if (planes != c_h) {  // padding channel planes must read as zero
    B200_CUDA_OK(cudaMemsetAsync(ap, 0, static_cast<size_t>(pieces) * planes * n * ld * 2, stream));
    B200_CUDA_OK(cudaMemsetAsync(bp, 0, static_cast<size_t>(pieces) * planes * n * ld * 2, stream));
  }
  count_launch();
  glu_split_kernel<BF><<<dim3(static_cast<unsigned>(ld / 32), static_cast<unsigned>(n)), 256, 0, stream>>>(
      p, g, a->mask, ms_o, ms_i, n, n, ld, c_h, planes, pieces, ap, bp);
  B200_CUDA_OK(cudaGetLastError());
  // bf16 products with float32 accumulation carried from call to call (smallest terms first
  // in float32 mode), 128 channel planes per call
  const long long plane = static_cast<long long>(n) * ld, piece = static_cast<long long>(planes) * plane;
  const int order3[6][2] = {{2, 0}, {0, 2}, {1, 1}, {1, 0}, {0, 1}, {0, 0}};
  const int n_terms = BF ? 1 : 6;
  for (int c0 = 0; c0 < planes; c0 += 128) {
    for (int s = 0; s < n_terms; ++s) {
      const int pa = BF ? 0 : order3[s][0], pb = BF ? 0 : order3[s][1];
      b200tri_trimul_contract_args ca = {};
      ca.n_i = ca.n_j = ca.n_k = n;
      ca.n_src = 1;
      ca.a = ap + pa * piece + c0 * plane;
      ca.b = bp + pb * piece + c0 * plane;
      ca.a_ld = ca.b_ld = ca.out_ld = ld;
      ca.a_chan_stride = ca.b_chan_stride = ca.out_chan_stride = plane;
      ca.a_src_stride = ca.b_src_stride = piece;
      ca.acc_in = s ? t + c0 * plane : nullptr;
      ca.out_f32 = t + c0 * plane;
      if ((rc = b200tri_trimul_contract(&ca, reinterpret_cast<b200tri_stream_t>(stream)))) return rc;
    }
  }
  count_launch();
  ln_channel_major_kernel<BF><<<static_cast<unsigned>((pairs * 32 + 255) / 256), 256, 0, stream>>>(
      t, n, ld, c_h, ln_out_s, ln_out_b, a->eps, tn);
  B200_CUDA_OK(cudaGetLastError());
  if ((rc = gemm<BF>(tn, p_out, pairs, c_h, c_z, o, stream))) return rc;
  if ((rc = gemm<BF>(xn, g_out, pairs, c_z, c_z, gate, stream))) return rc;
  count_launch();
  gate_out_kernel<BF, O><<<static_cast<unsigned>((pairs * c_z + 255) / 256), 256, 0, stream>>>(
      o, gate, n, c_z, a->incoming ? 1 : 0, static_cast<const O*>(a->residual), static_cast<O*>(a->out));
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}

template <bool BF>
int triatt_generic(const b200tri_triatt_args* a, int c_z, cudaStream_t stream) {
  using O = typename std::conditional<BF, __nv_bfloat16, float>::type;
  const int n = a->n, heads = a->heads, head_dim = a->head_dim, hd = heads * head_dim;
  const long long pairs = static_cast<long long>(n) * n;
  const TriattPlan pl = triatt_plan(n, c_z, heads, head_dim);
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  float* xn = reinterpret_cast<float*>(ws + pl.xn);
  float* q = reinterpret_cast<float*>(ws + pl.q);
  float* k = reinterpret_cast<float*>(ws + pl.k);
  float* v = reinterpret_cast<float*>(ws + pl.v);
  float* gate = reinterpret_cast<float*>(ws + pl.gate);
  float* o = reinterpret_cast<float*>(ws + pl.o);
  float* bias = reinterpret_cast<float*>(ws + pl.bias);
  ParamStage ps{ws + pl.params, 0, !BF, stream};
  const float* ln_s = ps.get(a->norm_scale, c_z);
  const float* ln_b = ps.get(a->norm_bias, c_z);
  const float* w_bias = ps.get(a->w_bias, static_cast<size_t>(c_z) * heads);
  const float* w_q = ps.get(a->w_q, static_cast<size_t>(c_z) * hd);
  const float* w_k = ps.get(a->w_k, static_cast<size_t>(c_z) * hd);
  const float* w_v = ps.get(a->w_v, static_cast<size_t>(c_z) * hd);
  const float* w_g = ps.get(a->w_g, static_cast<size_t>(c_z) * hd);
  const float* w_o = ps.get(a->w_o, static_cast<size_t>(hd) * c_z);
  if (ps.rc) return ps.rc;
  // attention frame (o = row, t = position inside the row): the ending node is the starting
  // node on the transposed pair tensor and mask (triangle_attention.py:128-130, :160-161)
  const long long s_o = a->starting ? static_cast<long long>(n) * c_z : c_z;
  const long long s_i = a->starting ? c_z : static_cast<long long>(n) * c_z;
  count_launch();
  ln_gather_kernel<BF, O><<<static_cast<unsigned>((pairs * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const O*>(a->x), s_o, s_i, n, n, c_z, ln_s, ln_b, a->eps, xn);
  B200_CUDA_OK(cudaGetLastError());
  int rc;
  if ((rc = gemm<BF>(xn, w_q, pairs, c_z, hd, q, stream))) return rc;
  if ((rc = gemm<BF>(xn, w_k, pairs, c_z, hd, k, stream))) return rc;
  if ((rc = gemm<BF>(xn, w_v, pairs, c_z, hd, v, stream))) return rc;
  if ((rc = gemm<BF>(xn, w_g, pairs, c_z, hd, gate, stream))) return rc;
  if ((rc = gemm<BF>(xn, w_bias, pairs, c_z, heads, bias, stream))) return rc;
  rc = launch_att_core<BF>(head_dim, dim3(static_cast<unsigned>((n + AQ - 1) / AQ), static_cast<unsigned>(heads),
                                          static_cast<unsigned>(n)),
                           stream, q, k, v, bias, a->mask, a->starting ? n : 1, a->starting ? 1 : n, a->inf, n, heads, o);
  if (rc) return rc;
  count_launch();
  mul_sigmoid_kernel<BF><<<static_cast<unsigned>((pairs * hd + 255) / 256), 256, 0, stream>>>(o, gate, pairs * hd);
  B200_CUDA_OK(cudaGetLastError());
  return gemm<BF, O>(o, w_o, pairs, hd, c_z, static_cast<O*>(a->out), stream, static_cast<const O*>(a->residual), n, s_o,
                     s_i);
}

}  // namespace

size_t trimul_workspace_bytes_generic(int32_t n, int32_t c_z, int32_t c_h, int32_t dtype) {
  if (n <= 0 || c_z <= 0 || c_h <= 0) return 0;
  return trimul_plan(n, c_z, c_h, dtype == B200TRI_DTYPE_F32).total + 1024;
}

size_t triatt_workspace_bytes_generic(int32_t n, int32_t c_z, int32_t heads, int32_t head_dim) {
  if (n <= 0 || c_z <= 0 || heads <= 0 || head_dim <= 0) return 0;
  return triatt_plan(n, c_z, heads, head_dim).total + 1024;
}

int trimul_forward_generic(const b200tri_trimul_args* a, int c_z, int c_h, cudaStream_t stream) {
  B200_REQUIRE(a->n <= 65535, B200TRI_ERR_UNSUPPORTED, "trimul (general shapes): n up to 65535");
  return a->dtype == B200TRI_DTYPE_F32 ? trimul_generic<false>(a, c_z, c_h, stream)
                                       : trimul_generic<true>(a, c_z, c_h, stream);
}

int triatt_forward_generic(const b200tri_triatt_args* a, int c_z, cudaStream_t stream) {
  B200_REQUIRE(a->n <= 65535, B200TRI_ERR_UNSUPPORTED, "triatt (general shapes): n up to 65535");
  return a->dtype == B200TRI_DTYPE_F32 ? triatt_generic<false>(a, c_z, stream) : triatt_generic<true>(a, c_z, stream);
}

}  // namespace b200
