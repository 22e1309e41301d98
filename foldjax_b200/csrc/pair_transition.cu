// Pair transition (SwiGLU feed-forward on every pair), fused into one pass over z.
//
//   xn     = LN(x)
//   a, b   = bf16(xn @ fc1), bf16(xn @ fc2)          128 -> hidden (512), twice
//   hidden = bf16(bf16(a * bf16(sigmoid(a))) * b)     silu(a) * b
//   out    = bf16(hidden @ fc3)   (+ residual)        hidden -> 128
//
// Reference: transition_forward,
// src/foldjax/models/boltz2/models/primitives/transition.py:41-127 (the
// unchunked XLA branch :108-112); called on the pair tensor from the Pairformer
// block, src/foldjax/models/boltz2/models/pairformer.py:152-160.
//
// One tile = 128 consecutive pairs (rows of the flattened [rows][128] tensor).
// The widened form (rows x 1024) never leaves the SM: the hidden dimension is
// walked in chunks of 64, each chunk's [a | b] accumulates in TMEM, is turned
// into 64 hidden values per pair by the activation warps, goes back to shared
// memory as the A operand of the second product and is consumed there.
// The weights (384 KiB as bf16) do not fit in shared memory; they stream from
// L2 through a 3-stage ring, one chunk (W1 rows, W2 rows, W3 columns: 48 KiB)
// per stage.
//
// Persistent, one CTA per SM:
//   warp 0        TMA producer (x tiles, weight chunks)
//   warp 1        MMA issuer: D1[chunk] = xn . [W1c ; W2c]^T, then OUT += h . W3c^T
//   warps 2-5     layer norm of the x tile in place (three register-light sweeps over
//                 shared memory); epilogue of OUT (+ residual)
//   warps 6-21    activation: four warpgroups, each turns 16 of the 64 [a | b] column
//                 pairs of every row into hidden values per chunk (four threads per
//                 pair). All of them must have stored their part before the second
//                 product of the chunk can start, so these warps carry no other duty.
// Bound: the activation (two MUFU operations per hidden unit: 1024 per pair) and
// the tensor pipe (393 kflop per pair) are within 25 % of each other; HBM moves
// 2 x 256 B per pair (x doubles as the residual when the caller adds in place).
#include "host.cuh"
#include "ln.cuh"
#include "tc.cuh"

namespace b200 {

namespace {

constexpr int HC = 64;  // hidden units per chunk
constexpr int WSTAGES = 3;
constexpr int XSTAGES = 2;
constexpr int TILE_BYTES = 2 * SLAB_BYTES;
constexpr int NWORK = 4;  // activation warpgroups
constexpr int THREADS = 64 + 128 + NWORK * 128;

struct Smem {
  uint8_t w12[WSTAGES][2 * SLAB_BYTES];  // rows 0-63: W1 chunk, 64-127: W2 chunk; [128][128 in] as two K slabs
  uint8_t w3[WSTAGES][SLAB_BYTES];       // [128 out][64 hidden]
  uint8_t x[XSTAGES][TILE_BYTES];
  uint8_t h[SLAB_BYTES];                 // [128 pairs][64 hidden]
  uint32_t gamma2[64], beta2[64];
  uint64_t w_full[WSTAGES], w_empty[WSTAGES], x_full[XSTAGES], xn_full[XSTAGES], x_empty[XSTAGES];
  uint64_t d1_full[2], d1_empty[2], h_full, h_empty, out_full[2], out_empty[2];
  uint32_t tmem_base;
};
static_assert(sizeof(Smem) <= 232448, "shared memory budget");

struct Params {
  long long rows, total_tiles;
  int nchunks;         // hidden / 64
  const uint32_t* ln;  // gamma, beta: 2 x 64 words
  const __nv_bfloat16* residual;
  const float* row_mask;
  __nv_bfloat16* out;
  float eps;
  int* status;
};

// bf16(bf16(a * bf16(sigmoid(a))) * b) for two hidden units; a and b arrive as the
// fp32 accumulators and are rounded to bf16 first, like the reference's matmul output.
__device__ __forceinline__ uint32_t swiglu_bf16x2(float a0, float a1, float b0, float b1) {
  const uint32_t a = pack_bf16x2(a0, a1);
  const float2 s = sigmoid_f32x2(make_float2(bf16_lo(a), bf16_hi(a)));
  return bf16x2_mul(bf16x2_mul(a, pack_bf16x2(s.x, s.y)), pack_bf16x2(b0, b1));
}

__global__ void __launch_bounds__(THREADS, 1)
pair_transition_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w12,
                       const __grid_constant__ CUtensorMap tm_w3, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, ST_OK, 900);
    return;
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_w12);
    tma_prefetch_desc(&tm_w3);
    for (int s = 0; s < WSTAGES; ++s) {
      mbar_init(&sm.w_full[s], 1);
      mbar_init(&sm.w_empty[s], 1);
    }
    for (int s = 0; s < XSTAGES; ++s) {
      mbar_init(&sm.x_full[s], 1);
      mbar_init(&sm.xn_full[s], 128);
      mbar_init(&sm.x_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sm.d1_full[a], 1);
      mbar_init(&sm.d1_empty[a], NWORK * 4);
      mbar_init(&sm.out_full[a], 1);
      mbar_init(&sm.out_empty[a], 4);  // the four warps of the warpgroup on epilogue duty
    }
    mbar_init(&sm.h_full, NWORK * 128);
    mbar_init(&sm.h_empty, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  if (threadIdx.x >= 64 && threadIdx.x < 128) {
    sm.gamma2[threadIdx.x - 64] = p.ln[threadIdx.x - 64];
    sm.beta2[threadIdx.x - 64] = p.ln[64 + threadIdx.x - 64];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;
  // TMEM: D1 (the chunk's [a | b], 128 columns) double-buffered at 0 and 128;
  // OUT (128 columns) double-buffered over tiles at 256 and 384.
  long long n_my = 0;
  for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) ++n_my;
  const int nchunks = p.nchunks;
  const long long total_n = n_my * nchunks;  // chunk steps of this CTA

  if (warp == 0) {
    if (elect_one()) {
      auto load_x = [&](long long it) -> bool {
        const int xs = static_cast<int>(it % XSTAGES);
        const uint32_t ph = static_cast<uint32_t>((it / XSTAGES) & 1);
        if (!mbar_wait(&sm.x_empty[xs], ph ^ 1, p.status, ST_TIMEOUT_PRODUCER)) return false;
        const long long tile = blockIdx.x + it * static_cast<long long>(gridDim.x);
        const int r0 = static_cast<int>(tile * 128);
        mbar_expect_tx(&sm.x_full[xs], TILE_BYTES);
        tma_load_2d(sm.x[xs], &tm_x, &sm.x_full[xs], 0, r0);
        tma_load_2d(sm.x[xs] + SLAB_BYTES, &tm_x, &sm.x_full[xs], 64, r0);
        return true;
      };
      bool alive = n_my > 0 && load_x(0);
      // The next tile's x is requested a few chunks into the current tile, when its
      // buffer (the previous tile's) has certainly been released.
      const int x_at = nchunks > WSTAGES ? WSTAGES : nchunks - 1;
      for (long long n = 0; n < total_n && alive; ++n) {
        const long long it = n / nchunks;
        const int c = static_cast<int>(n % nchunks);
        if (c == x_at && it + 1 < n_my && !load_x(it + 1)) break;
        const int ws = static_cast<int>(n % WSTAGES);
        const uint32_t ph = static_cast<uint32_t>((n / WSTAGES) & 1);
        if (!mbar_wait(&sm.w_empty[ws], ph ^ 1, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&sm.w_full[ws], 3 * SLAB_BYTES);
        tma_load_2d(sm.w12[ws], &tm_w12, &sm.w_full[ws], 0, c * 128);
        tma_load_2d(sm.w12[ws] + SLAB_BYTES, &tm_w12, &sm.w_full[ws], 64, c * 128);
        tma_load_2d(sm.w3[ws], &tm_w3, &sm.w_full[ws], c * HC, 0);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 128);
      for (long long n = 0; n <= total_n; ++n) {
        if (n < total_n) {  // first product of chunk step n
          const long long it = n / nchunks;
          const int c = static_cast<int>(n % nchunks);
          const int xs = static_cast<int>(it % XSTAGES);
          const int ws = static_cast<int>(n % WSTAGES);
          const uint32_t d = static_cast<uint32_t>(n & 1);
          if (c == 0 && !mbar_wait(&sm.xn_full[xs], static_cast<uint32_t>((it / XSTAGES) & 1), p.status, ST_TIMEOUT_MMA)) break;
          if (!mbar_wait(&sm.w_full[ws], static_cast<uint32_t>((n / WSTAGES) & 1), p.status, ST_TIMEOUT_MMA)) break;
          if (!mbar_wait(&sm.d1_empty[d], static_cast<uint32_t>(((n >> 1) & 1) ^ 1), p.status, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint64_t adesc = umma_desc_kmajor(smem_u32(sm.x[xs]) + s * SLAB_BYTES, 128);
            const uint64_t bdesc = umma_desc_kmajor(smem_u32(sm.w12[ws]) + s * SLAB_BYTES, 128);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16_ss(tmem_base + d * 128, umma_desc_advance(adesc, k * 32), umma_desc_advance(bdesc, k * 32), idesc,
                           (s | k) != 0);
          }
          umma_commit(&sm.d1_full[d]);
          if (c == nchunks - 1) umma_commit(&sm.x_empty[xs]);  // every first product of the tile has been issued
        }
        if (n > 0) {  // second product of chunk step n - 1
          const long long m = n - 1;
          const long long it = m / nchunks;
          const int c = static_cast<int>(m % nchunks);
          const int ws = static_cast<int>(m % WSTAGES);
          const uint32_t tb = static_cast<uint32_t>(it & 1);
          if (c == 0 && !mbar_wait(&sm.out_empty[tb], static_cast<uint32_t>(((it >> 1) & 1) ^ 1), p.status, ST_TIMEOUT_MMA)) break;
          if (!mbar_wait(&sm.h_full, static_cast<uint32_t>(m & 1), p.status, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
          const uint64_t adesc = umma_desc_kmajor(smem_u32(sm.h), 128);
          const uint64_t bdesc = umma_desc_kmajor(smem_u32(sm.w3[ws]), 128);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base + 256 + tb * 128, umma_desc_advance(adesc, k * 32), umma_desc_advance(bdesc, k * 32),
                         idesc, (c | k) != 0);
          umma_commit(&sm.w_empty[ws]);  // covers both products that read this stage
          umma_commit(&sm.h_empty);
          if (c == nchunks - 1) umma_commit(&sm.out_full[tb]);
        }
      }
    }
  } else {
    const bool act = warp >= 6;
    const int wg = act ? (warp - 6) >> 2 : 0;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // pair inside the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    bool alive = true;

    // Layer norm of one row in place (the register-light form).
    auto layer_norm_tile = [&](long long it) {
      const int xs = static_cast<int>(it % XSTAGES);
      if (!mbar_wait(&sm.x_full[xs], static_cast<uint32_t>((it / XSTAGES) & 1), p.status, ST_TIMEOUT_PROLOGUE)) {
        alive = false;
        return;
      }
      ln_row_sweeps(sm.x[xs], row, sm.gamma2, sm.beta2, p.eps);
      fence_proxy_async();
      mbar_arrive(&sm.xn_full[xs]);
    };

    auto epilogue_tile = [&](long long jt) {
      const uint32_t tb = static_cast<uint32_t>(jt & 1);
      if (!mbar_wait(&sm.out_full[tb], static_cast<uint32_t>((jt >> 1) & 1), p.status, ST_TIMEOUT_EPILOGUE)) {
        alive = false;
        return;
      }
      tc_fence_after();
      const long long r = (blockIdx.x + jt * static_cast<long long>(gridDim.x)) * 128 + row;
      const long long off = r * 128;
      // optional per-row mask on the update (before the residual add), rounded to the trunk dtype
      const float mkf = (p.row_mask && r < p.rows) ? p.row_mask[r] : 1.0f;
      const uint32_t mk2 = pack_bf16x2(mkf, mkf);
#pragma unroll 1
      for (int chunk = 0; chunk < 4; ++chunk) {
        uint32_t v[32];
        tmem_ld32(lane_addr + 256 + tb * 128 + chunk * 32, v);
        tmem_ld_wait();
        if (r < p.rows) {
          uint4* dst = reinterpret_cast<uint4*>(p.out + off + chunk * 32);
          const uint4* res = p.residual ? reinterpret_cast<const uint4*>(p.residual + off + chunk * 32) : nullptr;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t u[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              u[e] = pack_bf16x2(__uint_as_float(v[8 * q + 2 * e]), __uint_as_float(v[8 * q + 2 * e + 1]));
            if (p.row_mask) {
#pragma unroll
              for (int e = 0; e < 4; ++e) u[e] = bf16x2_mul(u[e], mk2);
            }
            if (res) {
              const uint4 rv = res[q];
              u[0] = bf16x2_add(rv.x, u[0]);
              u[1] = bf16x2_add(rv.y, u[1]);
              u[2] = bf16x2_add(rv.z, u[2]);
              u[3] = bf16x2_add(rv.w, u[3]);
            }
            dst[q] = make_uint4(u[0], u[1], u[2], u[3]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.out_empty[tb]);
    };

    if (!act) {
      // ---- layer norm of tile `it`, then the output epilogue of tile `it - 1`
      for (long long it = 0; it <= n_my && alive; ++it) {
        if (it < n_my) layer_norm_tile(it);
        if (it > 0 && alive) epilogue_tile(it - 1);
      }
    }
    for (long long n = 0; act && n < total_n; ++n) {
      // ---- activation: this thread's 16 columns of a and of b -> 16 hidden values
      const uint32_t d = static_cast<uint32_t>(n & 1);
      if (!mbar_wait(&sm.d1_full[d], static_cast<uint32_t>((n >> 1) & 1), p.status, ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      uint32_t a[16], b[16], hv[8];
      tmem_ld16(lane_addr + d * 128 + wg * 16, a);
      tmem_ld16(lane_addr + d * 128 + HC + wg * 16, b);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.d1_empty[d]);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        hv[e] = swiglu_bf16x2(__uint_as_float(a[2 * e]), __uint_as_float(a[2 * e + 1]), __uint_as_float(b[2 * e]),
                              __uint_as_float(b[2 * e + 1]));
      // the previous chunk's second product must have read h before it is overwritten
      if (!mbar_wait(&sm.h_empty, static_cast<uint32_t>((n & 1) ^ 1), p.status, ST_TIMEOUT_EPILOGUE)) break;
#pragma unroll
      for (int q = 0; q < 2; ++q)
        *reinterpret_cast<uint4*>(sm.h + sw128_offset(row, wg * 2 + q)) =
            make_uint4(hv[4 * q], hv[4 * q + 1], hv[4 * q + 2], hv[4 * q + 3]);
      fence_proxy_async();
      mbar_arrive(&sm.h_full);
    }
  }

  if (*reinterpret_cast<volatile int*>(p.status) != ST_OK)
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// Weight repacking (every call; a few microseconds). The reference stores linear
// kernels as [in, out]; the tensor core wants K-major rows.
// w12[(c * 128 + r) * 128 + k] = r < 64 ? fc1[k][c * 64 + r] : fc2[k][c * 64 + r - 64]
__global__ void pack_w12_kernel(const __nv_bfloat16* __restrict__ fc1, const __nv_bfloat16* __restrict__ fc2, int hidden,
                                __nv_bfloat16* __restrict__ dst) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= 2 * hidden * 128) return;
  const int k = idx & 127, rr = idx >> 7;
  const int c = rr >> 7, r = rr & 127;
  const __nv_bfloat16* src = r < HC ? fc1 : fc2;
  dst[idx] = src[static_cast<long long>(k) * hidden + c * HC + (r & (HC - 1))];
}
// w3[o * hidden + h] = fc3[h][o]
__global__ void pack_w3_kernel(const __nv_bfloat16* __restrict__ fc3, int hidden, __nv_bfloat16* __restrict__ dst) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= hidden * 128) return;
  const int h = idx % hidden, o = idx / hidden;
  dst[idx] = fc3[static_cast<long long>(h) * 128 + o];
}
__global__ void pack_ln_kernel(const uint32_t* __restrict__ scale, const uint32_t* __restrict__ bias,
                               uint32_t* __restrict__ dst) {
  const int idx = threadIdx.x;
  dst[idx] = idx < 64 ? scale[idx] : bias[idx - 64];
}

}  // namespace
}  // namespace b200

extern "C" size_t b200tri_pair_transition_workspace_bytes(int32_t hidden) {
  if (hidden <= 0) return 0;
  return static_cast<size_t>(3) * hidden * 128 * 2 + 3 * 1024 + 1024;
}

extern "C" int b200tri_pair_transition(const b200tri_pair_transition_args* a, b200tri_stream_t stream_) {
  using namespace b200;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  B200_REQUIRE(a != nullptr, B200TRI_ERR_INVALID, "pair transition: null args");
  B200_REQUIRE(a->x && a->out && a->norm_scale && a->norm_bias && a->fc1 && a->fc2 && a->fc3, B200TRI_ERR_INVALID,
               "pair transition: null pointer argument");
  B200_REQUIRE(a->rows > 0 && a->rows < (1ll << 31) - 256, B200TRI_ERR_INVALID,
               "pair transition: rows must be in [1, 2^31 - 256)");
  B200_REQUIRE(a->channels == 128, B200TRI_ERR_UNSUPPORTED, "pair transition: built for 128 channels (got %d)", a->channels);
  B200_REQUIRE(a->hidden > 0 && a->hidden % HC == 0 && a->hidden <= 4096, B200TRI_ERR_UNSUPPORTED,
               "pair transition: hidden width must be a positive multiple of 64 up to 4096 (got %d)", a->hidden);
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->out) |
                 reinterpret_cast<uintptr_t>(a->residual)) & 15) == 0,
               B200TRI_ERR_INVALID, "pair transition: x/out/residual must be 16-byte aligned");
  const size_t need = b200tri_pair_transition_workspace_bytes(a->hidden);
  B200_REQUIRE(a->workspace && a->workspace_bytes >= need, B200TRI_ERR_WORKSPACE,
               "pair transition: workspace of %zu bytes needed", need);
  int* status = device_status_word();
  B200_REQUIRE(status != nullptr, B200TRI_ERR_CUDA, "pair transition: no current CUDA device");

  Carver ws(a->workspace);
  __nv_bfloat16* w12 = ws.take<__nv_bfloat16>(static_cast<size_t>(2) * a->hidden * 128);
  __nv_bfloat16* w3 = ws.take<__nv_bfloat16>(static_cast<size_t>(a->hidden) * 128);
  uint32_t* ln = ws.take<uint32_t>(128, 256);
  {
    const int total = 2 * a->hidden * 128;
    count_launch(3);
    pack_w12_kernel<<<(total + 255) / 256, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(a->fc1),
                                                            static_cast<const __nv_bfloat16*>(a->fc2), a->hidden, w12);
    pack_w3_kernel<<<(a->hidden * 128 + 255) / 256, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(a->fc3), a->hidden, w3);
    pack_ln_kernel<<<1, 128, 0, stream>>>(static_cast<const uint32_t*>(a->norm_scale),
                                          static_cast<const uint32_t*>(a->norm_bias), ln);
    B200_CUDA_OK(cudaGetLastError());
  }

  CUtensorMap tm_x, tm_w12, tm_w3;
  {
    const uint64_t dims[2] = {128, (uint64_t)a->rows};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 128};
    int rc = make_tmap(&tm_x, a->x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {128, (uint64_t)2 * a->hidden};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 128};
    int rc = make_tmap(&tm_w12, w12, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)a->hidden, 128};
    const uint64_t str[1] = {(uint64_t)a->hidden * 2};
    const uint32_t box[2] = {64, 128};
    int rc = make_tmap(&tm_w3, w3, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  Params p;
  p.rows = a->rows;
  p.total_tiles = (a->rows + 127) / 128;
  p.nchunks = a->hidden / HC;
  p.ln = ln;
  p.residual = static_cast<const __nv_bfloat16*>(a->residual);
  p.row_mask = a->row_mask;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.eps = a->eps;
  p.status = status;

  {
    const int rc = ensure_smem_limit(reinterpret_cast<const void*>(pair_transition_kernel), (int)sizeof(Smem));
    if (rc) return rc;
  }
  const long long grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
  {
    TimedLaunch timed(K_PAIR_TRANSITION, stream);
    count_launch();
    pair_transition_kernel<<<static_cast<unsigned>(grid), THREADS, sizeof(Smem), stream>>>(tm_x, tm_w12, tm_w3, p);
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}
