// Single-representation attention with pair bias (the block's other consumer of z).
//
//   q = s @ Wq + bq,  g = sigmoid(s @ Wg),  k = k_in @ Wk,  v = k_in @ Wv
//   bias[h,i,j] = LN(z[i,j,:]) @ Wz[:,h]                      (z read once, in fp32)
//   out = (g * softmax_j(q_h . k_h / sqrt(d) + bias + (1 - mask_j) * -inf) v_h) @ Wo
//
// Reference: attention_pair_bias_forward,
// src/foldjax/models/boltz2/models/primitives/attention.py:19-140 (XLA branch
// :85-110, _attention_qblock :124-140), called from the Pairformer block with
// s and z in float32, src/foldjax/models/boltz2/models/trunk_blocks/pairformer.py:188-203.
// Everything here is fp32 arithmetic on fp32 s and bf16 z / weights (the trunk
// dtype), like the reference's promoted computation.
//
// The only part that scales with N^2 * c_z is the pair-bias pass over z
// (pair_bias_kernel, HBM-bound: 256 B read and 4 * heads B written per pair); the
// token attention itself is N^2 * c_s work (14 GFLOP at N = 3072) and runs on the
// fp32 pipes: at 16 heads x 24 channels it is far too small to be worth tensor-core
// tiles, and its operands are fp32.
#include "host.cuh"
#include "tc.cuh"

namespace b200 {

namespace {

constexpr int C_Z = 128;
constexpr int MAX_HEADS = 16;
constexpr int HD = 24;  // head width the token-attention kernel is built for

// ---------------------------------------------------------------- pair bias
// One thread per pair, 128 pairs per tile. With gamma folded into the projection,
//   bias_h = rstd * (sum_c x_c W'[c][h] - mean * sum_c W'[c][h]) + sum_c beta_c W[c][h],
// so the normalised row is never formed: one pass for the mean, one for the variance
// (two-pass, as the reference computes it), one pass of heads FMAs per channel. The tile is
// loaded with coalesced 16-byte loads into shared memory (16-byte chunks XOR-swizzled by the
// pair index, so that neither the row-major stores nor the thread-per-row reads conflict)
// and every pass reads it from there: the row never has to live in registers, and the
// projection runs two heads per instruction (fma.f32x2).
__global__ void __launch_bounds__(128, 4)
pair_bias_kernel(const __nv_bfloat16* __restrict__ z, long long n_pairs, int n, int ld, int heads,
                 const __nv_bfloat16* __restrict__ ln_scale, const __nv_bfloat16* __restrict__ ln_bias,
                 const __nv_bfloat16* __restrict__ wz, float eps, float* __restrict__ bias) {
  __shared__ __align__(16) float w[C_Z][MAX_HEADS];  // gamma_c * Wz[c][h]
  __shared__ float sw[MAX_HEADS], bw[MAX_HEADS];
  __shared__ __align__(16) uint4 tile_s[128 * 16];   // 128 pairs x 16 chunks of 8 channels
  for (int idx = threadIdx.x; idx < C_Z * MAX_HEADS; idx += blockDim.x) {
    const int c = idx / MAX_HEADS, h = idx % MAX_HEADS;
    w[c][h] = h < heads ? __bfloat162float(ln_scale[c]) * __bfloat162float(wz[c * heads + h]) : 0.f;
  }
  __syncthreads();
  if (threadIdx.x < MAX_HEADS) {
    const int h = threadIdx.x;
    float a = 0.f, b = 0.f;
    for (int c = 0; c < C_Z; ++c) {
      a += w[c][h];
      if (h < heads) b += __bfloat162float(ln_bias[c]) * __bfloat162float(wz[c * heads + h]);
    }
    sw[h] = a;
    bw[h] = b;
  }
  __syncthreads();
  const long long tiles = (n_pairs + 127) / 128;
  const int p = threadIdx.x, key = p & 15;
  for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const long long base = tile * 128;
    const long long left = n_pairs - base;  // pairs of this tile that exist (>= 1)
    const uint4* src = reinterpret_cast<const uint4*>(z + base * C_Z);
#pragma unroll 8
    for (int it = 0; it < 16; ++it) {
      const int idx = it * 128 + p;  // chunk idx of the tile: pair idx / 16, chunk idx % 16
      const int pr = idx >> 4, ch = idx & 15;
      const uint4 v = pr < left ? src[idx] : make_uint4(0u, 0u, 0u, 0u);
      tile_s[pr * 16 + (ch ^ (pr & 15))] = v;
    }
    __syncthreads();
    const uint4* row = tile_s + p * 16;
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const uint4 v = row[c ^ key];
      const uint32_t x4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) s4[e] += bf16_lo(x4[e]) + bf16_hi(x4[e]);
    }
    const float mean = ((s4[0] + s4[1]) + (s4[2] + s4[3])) * (1.0f / C_Z);
    float q4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const uint4 v = row[c ^ key];
      const uint32_t x4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a = bf16_lo(x4[e]) - mean, b = bf16_hi(x4[e]) - mean;
        q4[e] = fmaf(a, a, q4[e]);
        q4[e] = fmaf(b, b, q4[e]);
      }
    }
    const float rstd = rsqrtf(((q4[0] + q4[1]) + (q4[2] + q4[3])) * (1.0f / C_Z) + eps);
    float2 acc[MAX_HEADS / 2];
#pragma unroll
    for (int h = 0; h < MAX_HEADS / 2; ++h) acc[h] = make_float2(0.f, 0.f);
#pragma unroll 2
    for (int c = 0; c < 16; ++c) {
      const uint4 v = row[c ^ key];
      const uint32_t x4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ch = 8 * c + 2 * e;  // channels ch (low half) and ch + 1 (high half)
        const float a = bf16_lo(x4[e]), b = bf16_hi(x4[e]);
        const float2 a2 = make_float2(a, a), b2 = make_float2(b, b);
        const float4* wa = reinterpret_cast<const float4*>(w[ch]);
        const float4* wb = reinterpret_cast<const float4*>(w[ch + 1]);
#pragma unroll
        for (int h4 = 0; h4 < MAX_HEADS / 4; ++h4) {
          const float4 fa = wa[h4], fb = wb[h4];
          acc[2 * h4 + 0] = __ffma2_rn(b2, make_float2(fb.x, fb.y), __ffma2_rn(a2, make_float2(fa.x, fa.y), acc[2 * h4 + 0]));
          acc[2 * h4 + 1] = __ffma2_rn(b2, make_float2(fb.z, fb.w), __ffma2_rn(a2, make_float2(fa.z, fa.w), acc[2 * h4 + 1]));
        }
      }
    }
    const long long pair = base + p;
    if (pair < n_pairs) {
      const long long i = pair / n, j = pair % n;
#pragma unroll
      for (int h = 0; h < MAX_HEADS; ++h)
        if (h < heads)
          bias[(static_cast<long long>(h) * n + i) * ld + j] = rstd * ((h & 1 ? acc[h >> 1].y : acc[h >> 1].x) - mean * sw[h]) + bw[h];
    }
    __syncthreads();  // the tile is overwritten by the next round's loads
  }
}

// ------------------------------------------------------------------ linear
// out[M][N] = act(x[M][K] @ W[K][N] (+ b[N])) with fp32 x, bf16 W and b, fp32 out;
// optional elementwise gate on the input rows: x <- x * gate (the reference's g * out
// in front of the output projection). 64 x 64 tiles, 4 x 4 outputs per thread.
__global__ void __launch_bounds__(256)
linear_f32_kernel(const float* __restrict__ x, const float* __restrict__ gate, const __nv_bfloat16* __restrict__ w,
                  const __nv_bfloat16* __restrict__ b, int M, int K, int N, int sigmoid, float* __restrict__ out,
                  const float* __restrict__ res = nullptr) {
  __shared__ float xs[16][64 + 1];
  __shared__ float ws[16][64];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int idx = threadIdx.x; idx < 64 * 16; idx += 256) {
      const int r = idx >> 4, c = idx & 15;
      const int m = m0 + r, k = k0 + c;
      float v = 0.f;
      if (m < M && k < K) {
        v = x[static_cast<long long>(m) * K + k];
        if (gate) v *= gate[static_cast<long long>(m) * K + k];
      }
      xs[c][r] = v;
    }
    for (int idx = threadIdx.x; idx < 16 * 64; idx += 256) {
      const int r = idx >> 6, c = idx & 63;
      const int k = k0 + r, nn = n0 + c;
      ws[r][c] = (k < K && nn < N) ? __bfloat162float(w[static_cast<long long>(k) * N + nn]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float a[4], bb[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        a[e] = xs[k][ty * 4 + e];
        bb[e] = ws[k][tx * 4 + e];
      }
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(a[r], bb[c], acc[r][c]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int m = m0 + ty * 4 + r;
    if (m >= M) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int nn = n0 + tx * 4 + c;
      if (nn >= N) continue;
      float v = acc[r][c] + (b ? __bfloat162float(b[nn]) : 0.f);
      if (sigmoid) v = 1.0f / (1.0f + expf(-v));
      if (res) v += res[static_cast<long long>(m) * N + nn];
      out[static_cast<long long>(m) * N + nn] = v;
    }
  }
}

// --------------------------------------------------------- token attention
// One thread per (query i, head h); keys in tiles of 32 staged in shared memory.
// Online softmax in fp32; scores = q.k / sqrt(d) + bias + (1 - mask) * -inf, added in
// that order like the reference (attention.py:134-136).
constexpr int TQ = 64;  // queries per block
constexpr int TK = 32;  // keys per tile

__global__ void __launch_bounds__(TQ)
token_attention_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                       const float* __restrict__ bias, const float* __restrict__ mask, int n, int n_keys, int ld,
                       int c_s, float inf, float* __restrict__ out) {
  __shared__ float ks[TK][HD], vs[TK][HD], ms[TK];
  const int h = blockIdx.y;
  const int i = blockIdx.x * TQ + threadIdx.x;
  const bool live = i < n;
  const float inv_scale = 1.0f / sqrtf(static_cast<float>(HD));
  float qr[HD], acc[HD];
#pragma unroll
  for (int d = 0; d < HD; ++d) {
    qr[d] = live ? q[static_cast<long long>(i) * c_s + h * HD + d] : 0.f;
    acc[d] = 0.f;
  }
  float m_run = -INFINITY, l_run = 0.f;
  const float* brow = bias + (static_cast<long long>(h) * n + (live ? i : 0)) * ld;
  for (int j0 = 0; j0 < n_keys; j0 += TK) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < TK * HD; idx += TQ) {
      const int r = idx / HD, d = idx % HD;
      const int j = j0 + r;
      ks[r][d] = j < n_keys ? k[static_cast<long long>(j) * c_s + h * HD + d] : 0.f;
      vs[r][d] = j < n_keys ? v[static_cast<long long>(j) * c_s + h * HD + d] : 0.f;
    }
    if (threadIdx.x < TK) {
      const int j = j0 + threadIdx.x;
      ms[threadIdx.x] = j < n_keys ? (1.0f - mask[j]) * -inf : -INFINITY;  // keys past the end: no weight
    }
    __syncthreads();
    float sc[TK];
    float mx = m_run;
#pragma unroll
    for (int r = 0; r < TK; ++r) {
      float dot = 0.f;
#pragma unroll
      for (int d = 0; d < HD; ++d) dot = fmaf(qr[d], ks[r][d], dot);
      const float b = (j0 + r < n_keys) ? brow[j0 + r] : 0.f;
      sc[r] = (dot * inv_scale + b) + ms[r];
      mx = fmaxf(mx, sc[r]);
    }
    const float alpha = __expf(m_run - mx);  // 0 on the first tile
    l_run *= alpha;
#pragma unroll
    for (int d = 0; d < HD; ++d) acc[d] *= alpha;
#pragma unroll
    for (int r = 0; r < TK; ++r) {
      const float pr = __expf(sc[r] - mx);
      l_run += pr;
#pragma unroll
      for (int d = 0; d < HD; ++d) acc[d] = fmaf(pr, vs[r][d], acc[d]);
    }
    m_run = mx;
  }
  if (live) {
    const float inv = 1.0f / l_run;
#pragma unroll
    for (int d = 0; d < HD; ++d) out[static_cast<long long>(i) * c_s + h * HD + d] = acc[d] * inv;
  }
}

}  // namespace

int launch_linear_f32(const float* x, const float* gate, const void* w, const void* bias, int M, int K, int N,
                      int sigmoid, const float* res, float* out, cudaStream_t stream) {
  const dim3 grid((N + 63) / 64, (M + 63) / 64);
  count_launch();
  linear_f32_kernel<<<grid, 256, 0, stream>>>(x, gate, static_cast<const __nv_bfloat16*>(w),
                                              static_cast<const __nv_bfloat16*>(bias), M, K, N, sigmoid, out, res);
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}

}  // namespace b200

extern "C" size_t b200tri_attention_pair_bias_workspace_bytes(int32_t n, int32_t c_s, int32_t heads) {
  if (n <= 0 || c_s <= 0 || heads <= 0) return 0;
  const size_t ld = static_cast<size_t>(b200::round_up(n, 4));
  return (5 * static_cast<size_t>(n) * c_s + static_cast<size_t>(heads) * n * ld) * sizeof(float) + 8 * 1024;
}

extern "C" int b200tri_attention_pair_bias(const b200tri_attention_pair_bias_args* a, b200tri_stream_t stream_) {
  using namespace b200;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  B200_REQUIRE(a != nullptr, B200TRI_ERR_INVALID, "attention pair bias: null args");
  B200_REQUIRE(a->s && a->z && a->mask && a->out && a->proj_q && a->proj_q_bias && a->proj_k && a->proj_v && a->proj_g &&
                   a->proj_z_norm_scale && a->proj_z_norm_bias && a->proj_z && a->proj_o,
               B200TRI_ERR_INVALID, "attention pair bias: null pointer argument");
  B200_REQUIRE(a->n > 0, B200TRI_ERR_INVALID, "attention pair bias: n must be positive");
  B200_REQUIRE(a->c_z == C_Z, B200TRI_ERR_UNSUPPORTED, "attention pair bias: built for c_z = 128 (got %d)", a->c_z);
  B200_REQUIRE(a->heads >= 1 && a->heads <= MAX_HEADS && a->c_s == a->heads * HD, B200TRI_ERR_UNSUPPORTED,
               "attention pair bias: built for up to 16 heads of width 24 (got c_s %d, %d heads)", a->c_s, a->heads);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a->z) & 15) == 0, B200TRI_ERR_INVALID,
               "attention pair bias: z must be 16-byte aligned");
  const size_t need = b200tri_attention_pair_bias_workspace_bytes(a->n, a->c_s, a->heads);
  B200_REQUIRE(a->workspace && a->workspace_bytes >= need, B200TRI_ERR_WORKSPACE,
               "attention pair bias: workspace of %zu bytes needed", need);
  const int n = a->n, c_s = a->c_s, heads = a->heads;
  const int ld = round_up(n, 4);
  Carver ws(a->workspace);
  const size_t act = static_cast<size_t>(n) * c_s;
  float* q = ws.take<float>(act);
  float* g = ws.take<float>(act);
  float* k = ws.take<float>(act);
  float* v = ws.take<float>(act);
  float* ao = ws.take<float>(act);
  float* bias = ws.take<float>(static_cast<size_t>(heads) * n * ld);
  const float* s = static_cast<const float*>(a->s);
  const float* k_in = a->k_in ? static_cast<const float*>(a->k_in) : s;
  auto bf = [](const void* p) { return static_cast<const __nv_bfloat16*>(p); };
  const dim3 lin_grid((c_s + 63) / 64, (n + 63) / 64);
  count_launch(7);
  linear_f32_kernel<<<lin_grid, 256, 0, stream>>>(s, nullptr, bf(a->proj_q), bf(a->proj_q_bias), n, c_s, c_s, 0, q);
  linear_f32_kernel<<<lin_grid, 256, 0, stream>>>(s, nullptr, bf(a->proj_g), nullptr, n, c_s, c_s, 1, g);
  linear_f32_kernel<<<lin_grid, 256, 0, stream>>>(k_in, nullptr, bf(a->proj_k), nullptr, n, c_s, c_s, 0, k);
  linear_f32_kernel<<<lin_grid, 256, 0, stream>>>(k_in, nullptr, bf(a->proj_v), nullptr, n, c_s, c_s, 0, v);
  {
    TimedLaunch timed(K_PAIR_BIAS, stream);
    const long long n_pairs = static_cast<long long>(n) * n;
    const long long tiles = (n_pairs + 127) / 128;
    const long long blocks = tiles < 16LL * sm_count() ? tiles : 16LL * sm_count();
    pair_bias_kernel<<<static_cast<unsigned>(blocks), 128, 0, stream>>>(bf(a->z), n_pairs, n, ld, heads,
                                                                       bf(a->proj_z_norm_scale), bf(a->proj_z_norm_bias),
                                                                       bf(a->proj_z), a->eps, bias);
  }
  token_attention_kernel<<<dim3((n + TQ - 1) / TQ, heads), TQ, 0, stream>>>(q, k, v, bias, static_cast<const float*>(a->mask),
                                                                          n, n, ld, c_s, a->inf, ao);
  linear_f32_kernel<<<lin_grid, 256, 0, stream>>>(ao, g, bf(a->proj_o), nullptr, n, c_s, c_s, 0, static_cast<float*>(a->out));
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}
