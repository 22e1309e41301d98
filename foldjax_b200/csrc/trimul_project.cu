// Triangle multiplicative update, projection stage.
//
//   xn     = LN_in(x)
//   [a|b]  = sigmoid(xn @ g_in) * (xn @ p_in) * mask        (256 channels)
//
// written channel-major (a[d][o][t], b[d][o][t]) so the contraction stage can
// feed both operands to the tensor cores K-major. Reference:
// src/foldjax/models/boltz2/models/triangle/triangle.py:78-102.
//
// One tile = 128 consecutive pairs (o, t0..t0+127). The products are issued
// "transposed" - D[channel][pair] = W[channel][:] . xn[pair][:] - so a TMEM
// lane is an output channel and a thread of the epilogue owns 128 consecutive
// pairs of one channel, i.e. one contiguous 256-byte run of the output.
//
// Persistent kernel, one CTA per SM, 10 warps:
//   warp 0      TMA producer: weights once (128 KiB, resident), x tiles in a 3-stage ring
//   warp 1      MMA issuer: 4 groups (p_a, g_a, p_b, g_b) of 128x128x128 per tile
//   warps 2-9   layer norm, in place in the tile TMA delivered (two threads per pair)
//   warps 10-13 epilogue: TMEM -> sigmoid gate -> mask -> bf16 -> global
// TMEM: four 128-column accumulators; the a-half and the b-half are released
// separately so the MMAs of the next tile overlap the epilogue of this one.
//
// Bound: HBM (read x once, write a and b once: 3 * n*n*128*2 bytes).
#include "host.cuh"
#include "ln.cuh"
#include "pack.cuh"
#include "tc.cuh"

namespace b200 {

namespace {

constexpr int XSTAGES = 3;
constexpr int TILE_BYTES = 2 * SLAB_BYTES;  // 32 KiB: 128 pairs x 128 channels bf16
constexpr int W_BYTES = 8 * SLAB_BYTES;     // 128 KiB: 4 groups x 2 K-slabs
constexpr int MASK_SLOTS = 4;
constexpr int LN_WARPS = 8;  // two threads per pair
constexpr int THREADS = 64 + LN_WARPS * 32 + 128;

struct Smem {
  uint8_t w[W_BYTES];
  uint8_t x[XSTAGES][TILE_BYTES];
  __nv_bfloat16 mask[MASK_SLOTS][128];  // mask.astype(bf16), as the reference casts it
  uint32_t gamma2[64];
  uint32_t beta2[64];
  uint64_t w_full, x_full[XSTAGES], xn_full[XSTAGES], x_empty[XSTAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};
static_assert(sizeof(Smem) <= 232448, "shared memory budget");

struct ProjParams {
  int n_outer, n_inner, tiles_inner;
  long long total_tiles;
  const float* mask;
  long long ms_outer, ms_inner;
  const uint32_t* gamma2;
  const uint32_t* beta2;
  __nv_bfloat16* a;
  __nv_bfloat16* b;
  long long ld, chan_stride, block_stride;
  int rows_per_block;
  float eps;
  int* status;
};

__global__ void __launch_bounds__(THREADS, 1)
project_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
               const ProjParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if ((smem_u32(smem_raw) & 1023u) != 0) {  // operand tiles need 1 KiB alignment
    if (threadIdx.x == 0) atomicCAS(p.status, ST_OK, 900);
    return;
  }

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_w);
    mbar_init(&sm.w_full, 1);
    for (int s = 0; s < XSTAGES; ++s) {
      mbar_init(&sm.x_full[s], 1);
      mbar_init(&sm.xn_full[s], LN_WARPS * 32);
      mbar_init(&sm.x_empty[s], 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(&sm.acc_full[h], 1);
      mbar_init(&sm.acc_empty[h], 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  if (threadIdx.x >= 64 && threadIdx.x < 128) {
    sm.gamma2[threadIdx.x - 64] = p.gamma2[threadIdx.x - 64];
    sm.beta2[threadIdx.x - 64] = p.beta2[threadIdx.x - 64];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&sm.w_full, W_BYTES);
      for (int g = 0; g < 4; ++g)
        for (int s = 0; s < 2; ++s) tma_load_2d(sm.w + (g * 2 + s) * SLAB_BYTES, &tm_w, &sm.w_full, s * 64, g * 128);
      int stage = 0;
      uint32_t phase = 0;
      for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
        const int o = static_cast<int>(tile / p.tiles_inner);
        const int t0 = static_cast<int>(tile % p.tiles_inner) * 128;
        if (!mbar_wait(&sm.x_empty[stage], phase ^ 1, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&sm.x_full[stage], TILE_BYTES);
        tma_load_3d(sm.x[stage], &tm_x, &sm.x_full[stage], 0, t0, o);
        tma_load_3d(sm.x[stage] + SLAB_BYTES, &tm_x, &sm.x_full[stage], 64, t0, o);
        if (++stage == XSTAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 128);
      bool alive = mbar_wait(&sm.w_full, 0, p.status, ST_TIMEOUT_MMA);
      int stage = 0;
      uint32_t phase = 0, it = 0;
      for (long long tile = blockIdx.x; tile < p.total_tiles && alive; tile += gridDim.x, ++it) {
        if (!mbar_wait(&sm.xn_full[stage], phase, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t xs = smem_u32(sm.x[stage]);
        for (int half = 0; half < 2 && alive; ++half) {
          if (!mbar_wait(&sm.acc_empty[half], (it & 1) ^ 1, p.status, ST_TIMEOUT_MMA)) {
            alive = false;
            break;
          }
          tc_fence_after();
          for (int g = 0; g < 2; ++g) {
            const int group = half * 2 + g;
            const uint32_t d_tmem = tmem_base + group * 128;
#pragma unroll
            for (int s = 0; s < 2; ++s) {
              const uint64_t wdesc = umma_desc_kmajor(smem_u32(sm.w + (group * 2 + s) * SLAB_BYTES), 128);
              const uint64_t xdesc = umma_desc_kmajor(xs + s * SLAB_BYTES, 128);
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_bf16_ss(d_tmem, umma_desc_advance(wdesc, k * 32), umma_desc_advance(xdesc, k * 32), idesc,
                             (s | k) != 0);
            }
          }
          umma_commit(&sm.acc_full[half]);
        }
        if (alive) umma_commit(&sm.x_empty[stage]);
        if (++stage == XSTAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp < 2 + LN_WARPS) {
    // ---- layer norm, two threads per pair of the tile (lanes l and l ^ 16)
    const int r = (warp - 2) * 16 + (lane & 15);
    int stage = 0;
    uint32_t phase = 0, it = 0;
    for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
      const int o = static_cast<int>(tile / p.tiles_inner);
      const int t = static_cast<int>(tile % p.tiles_inner) * 128 + r;
      float mval = 0.f;
      if (t < p.n_inner) mval = p.mask ? p.mask[o * p.ms_outer + t * p.ms_inner] : 1.0f;
      if (!mbar_wait(&sm.x_full[stage], phase, p.status, ST_TIMEOUT_PROLOGUE)) break;
      ln_row_two_threads(sm.x[stage], r, lane >> 4, sm.gamma2, sm.beta2, p.eps);
      if (lane < 16) sm.mask[it & (MASK_SLOTS - 1)][r] = __float2bfloat16_rn(mval);
      fence_proxy_async();
      mbar_arrive(&sm.xn_full[stage]);
      if (++stage == XSTAGES) {
        stage = 0;
        phase ^= 1;
      }
    }
  } else {
    // ---- epilogue: thread = output channel (TMEM lane), columns = pairs
    const int quarter = warp & 3;
    const int chan = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    uint32_t it = 0;
    bool alive = true;
    for (long long tile = blockIdx.x; tile < p.total_tiles && alive; tile += gridDim.x, ++it) {
      const int o = static_cast<int>(tile / p.tiles_inner);
      const int t0 = static_cast<int>(tile % p.tiles_inner) * 128;
      const long long row_off = static_cast<long long>(o / p.rows_per_block) * p.block_stride +
                                static_cast<long long>(chan) * p.chan_stride +
                                static_cast<long long>(o % p.rows_per_block) * p.ld + t0;
      const uint32_t* mrow = reinterpret_cast<const uint32_t*>(sm.mask[it & (MASK_SLOTS - 1)]);
      for (int half = 0; half < 2; ++half) {
        if (!mbar_wait(&sm.acc_full[half], it & 1, p.status, ST_TIMEOUT_EPILOGUE)) {
          alive = false;
          break;
        }
        tc_fence_after();
        __nv_bfloat16* dst = (half ? p.b : p.a) + row_off;
#pragma unroll 1
        for (int chunk = 0; chunk < 4; ++chunk) {
          uint32_t pr[32], gr[32];
          tmem_ld32(lane_addr + half * 256 + chunk * 32, pr);
          tmem_ld32(lane_addr + half * 256 + 128 + chunk * 32, gr);
          tmem_ld_wait();
          // bf16 rounding after the two products, the sigmoid, the gating and the
          // mask, as on the reference's bf16 trunk.
          uint32_t packed[16];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 m = *reinterpret_cast<const uint4*>(mrow + chunk * 16 + 4 * q);
            const uint32_t mm[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int c = 8 * q + 2 * e;
              const uint32_t pv = pack_bf16x2(__uint_as_float(pr[c]), __uint_as_float(pr[c + 1]));
              const uint32_t sg = sigmoid_bf16x2(__uint_as_float(gr[c]), __uint_as_float(gr[c + 1]));
              packed[4 * q + e] = bf16x2_mul(bf16x2_mul(sg, pv), mm[e]);
            }
          }
          const int tc = t0 + chunk * 32;
          if (tc + 32 <= p.n_inner) {
            uint4* d4 = reinterpret_cast<uint4*>(dst + chunk * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              d4[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
          } else if (tc < p.n_inner) {
#pragma unroll
            for (int q = 0; q < 32; ++q)
              if (tc + q < p.n_inner) {
                const uint32_t w = packed[q >> 1];
                dst[chunk * 32 + q] = __ushort_as_bfloat16(static_cast<unsigned short>((q & 1) ? (w >> 16) : (w & 0xffffu)));
              }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.acc_empty[half]);
      }
    }
  }

  if (*reinterpret_cast<volatile int*>(p.status) != ST_OK)
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

}  // namespace b200

extern "C" size_t b200tri_trimul_project_workspace_bytes(void) {
  return 512 * 128 * 2 + 1024;  // packed weights + layer-norm parameters
}

extern "C" int b200tri_trimul_project(const b200tri_trimul_project_args* a, b200tri_stream_t stream_) {
  using namespace b200;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  B200_REQUIRE(a != nullptr, B200TRI_ERR_INVALID, "project: null args");
  B200_REQUIRE(a->x && a->a && a->b && a->p_in && a->g_in && a->norm_in_scale && a->norm_in_bias, B200TRI_ERR_INVALID,
               "project: null pointer argument");
  B200_REQUIRE(a->n_outer > 0 && a->n_inner > 0, B200TRI_ERR_INVALID, "project: sizes must be positive");
  B200_REQUIRE(a->xs_outer % 8 == 0 && a->xs_inner % 8 == 0, B200TRI_ERR_INVALID,
               "project: x strides must be multiples of 8 elements");
  B200_REQUIRE(a->ld % 8 == 0 && a->chan_stride % 8 == 0 && a->block_stride % 8 == 0 && a->rows_per_block > 0,
               B200TRI_ERR_INVALID, "project: output pitch/strides must be multiples of 8 elements");
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(a->a) | reinterpret_cast<uintptr_t>(a->b)) & 15) == 0, B200TRI_ERR_INVALID,
               "project: outputs must be 16-byte aligned");
  B200_REQUIRE(a->workspace && a->workspace_bytes >= b200tri_trimul_project_workspace_bytes(), B200TRI_ERR_WORKSPACE,
               "project: workspace of %zu bytes needed", b200tri_trimul_project_workspace_bytes());
  int* status = device_status_word();
  B200_REQUIRE(status != nullptr, B200TRI_ERR_CUDA, "project: no current CUDA device");

  Carver ws(a->workspace);
  __nv_bfloat16* wpk = ws.take<__nv_bfloat16>(512 * 128);
  uint32_t* gamma2 = ws.take<uint32_t>(64, 256);
  uint32_t* beta2 = ws.take<uint32_t>(64, 256);
  // Row groups of the packed weight: p_a, g_a, p_b, g_b (a = first 128 channels).
  const __nv_bfloat16* p_in = static_cast<const __nv_bfloat16*>(a->p_in);
  const __nv_bfloat16* g_in = static_cast<const __nv_bfloat16*>(a->g_in);
  pack_transpose(p_in, 256, 0, 128, wpk + 0 * 128 * 128, stream);
  pack_transpose(g_in, 256, 0, 128, wpk + 1 * 128 * 128, stream);
  pack_transpose(p_in, 256, 128, 128, wpk + 2 * 128 * 128, stream);
  pack_transpose(g_in, 256, 128, 128, wpk + 3 * 128 * 128, stream);
  pack_copy_words(a->norm_in_scale, gamma2, 64, stream);
  pack_copy_words(a->norm_in_bias, beta2, 64, stream);

  CUtensorMap tm_x, tm_w;
  {
    const uint64_t dims[3] = {128, (uint64_t)a->n_inner, (uint64_t)a->n_outer};
    const uint64_t str[2] = {(uint64_t)a->xs_inner * 2, (uint64_t)a->xs_outer * 2};
    const uint32_t box[3] = {64, 128, 1};
    int rc = make_tmap(&tm_x, a->x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {128, 512};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 128};
    int rc = make_tmap(&tm_w, wpk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  ProjParams p;
  p.n_outer = a->n_outer;
  p.n_inner = a->n_inner;
  p.tiles_inner = (a->n_inner + 127) / 128;
  p.total_tiles = static_cast<long long>(p.tiles_inner) * a->n_outer;
  p.mask = a->mask;
  p.ms_outer = a->ms_outer;
  p.ms_inner = a->ms_inner;
  p.gamma2 = gamma2;
  p.beta2 = beta2;
  p.a = static_cast<__nv_bfloat16*>(a->a);
  p.b = static_cast<__nv_bfloat16*>(a->b);
  p.ld = a->ld;
  p.chan_stride = a->chan_stride;
  p.block_stride = a->block_stride;
  p.rows_per_block = a->rows_per_block;
  p.eps = a->eps;
  p.status = status;

  {
    const int rc = ensure_smem_limit(reinterpret_cast<const void*>(project_kernel), (int)sizeof(Smem));
    if (rc) return rc;
  }
  const long long grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
  {
    TimedLaunch timed(K_TRIMUL_PROJECT, stream);
    count_launch();
    project_kernel<<<static_cast<unsigned>(grid), THREADS, sizeof(Smem), stream>>>(tm_x, tm_w, p);
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}
