// Triangle multiplicative update, output stage.
//
//   out[i][j][:] = LN_out(t[:, i, j]) @ p_out * sigmoid(LN_in(x[i][j]) @ g_out)  (+ residual)
//
// Reference: src/foldjax/models/boltz2/models/triangle/triangle.py:124-129.
// t is the contraction result, channel-major (t[d][i][j]); the kernel turns it
// back into channel-last while it normalises. The output gate is recomputed
// from x here instead of being stored by the projection stage: reading x costs
// the same bytes as reading a stored gate would, and saves writing it.
//
// One tile = 128 consecutive pairs (i, j0..j0+127). Persistent, one CTA per SM:
//   warp 0      TMA producer: two 128x128 weights once; per tile the x tile
//               (K-major, swizzled) and the t tile ([channel][pair], plain)
//   warp 1      MMA issuer: D1 = LN_in(x) . g_out^T, D2 = LN_out(t) . p_out^T
//   warps 2-5   layer norms, one thread per pair; the t tile is transposed into
//               operand layout in place (read column, mbarrier, write row)
//   warps 6-9   epilogue: D2 * sigmoid(D1) (+ residual) -> bf16 -> shared-memory tile -> TMA store
// TMEM: 2 x (D1, D2) so the epilogue overlaps the next tile's MMAs.
//
// Bound: HBM (read t and x, write out: 3 * n_i*n_j*128*2 bytes; + residual).
#include "host.cuh"
#include "ln.cuh"
#include "pack.cuh"
#include "tc.cuh"

namespace b200 {

namespace {

constexpr int STAGES = 2;
constexpr int TILE_BYTES = 2 * SLAB_BYTES;
constexpr int THREADS = 320;
constexpr int EPI_THREAD0 = 192;  // first thread of the epilogue warps
// 1: the epilogue stages the output tile in shared memory ([128 pairs][128 channels] as two
// swizzled slabs) and writes it with two TMA stores; 0: every thread stores its pair's row
// itself, 64 bytes at a time, so that a warp's store instruction touches 32 cache lines.
#ifndef B200_FIN_TMASTORE
#define B200_FIN_TMASTORE 1
#endif

struct Smem {
  uint8_t w[4 * SLAB_BYTES];  // g_out^T (2 slabs), p_out^T (2 slabs)
  uint8_t x[STAGES][TILE_BYTES];
  uint8_t t[STAGES][TILE_BYTES];
#if B200_FIN_TMASTORE
  uint8_t out[TILE_BYTES];
#endif
  uint32_t gamma_in[64], beta_in[64], gamma_out[64], beta_out[64];
  uint64_t w_full, in_full[STAGES], xn_full[STAGES], in_empty[STAGES], col_read[STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};
static_assert(sizeof(Smem) <= 232448, "shared memory budget");

struct FinishParams {
  int n_i, n_j, tiles_j;
  long long total_tiles;
  const uint32_t* ln;  // gamma_in, beta_in, gamma_out, beta_out: 4 x 64 words
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  long long os_i, os_j;
  float eps;
  int t_rpb;  // rows per block of t
  int* status;
};

__global__ void __launch_bounds__(THREADS, 1)
finish_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_t,
              const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_out,
              const FinishParams p) {
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
    tma_prefetch_desc(&tm_t);
    tma_prefetch_desc(&tm_w);
    mbar_init(&sm.w_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.in_full[s], 1);
      mbar_init(&sm.xn_full[s], 128);
      mbar_init(&sm.in_empty[s], 1);
      mbar_init(&sm.col_read[s], 128);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sm.acc_full[a], 1);
      mbar_init(&sm.acc_empty[a], 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  if (threadIdx.x >= 64 && threadIdx.x < 128) {
    const int q = threadIdx.x - 64;
    sm.gamma_in[q] = p.ln[q];
    sm.beta_in[q] = p.ln[64 + q];
    sm.gamma_out[q] = p.ln[128 + q];
    sm.beta_out[q] = p.ln[192 + q];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&sm.w_full, 4 * SLAB_BYTES);
      for (int g = 0; g < 2; ++g)
        for (int s = 0; s < 2; ++s) tma_load_2d(sm.w + (g * 2 + s) * SLAB_BYTES, &tm_w, &sm.w_full, s * 64, g * 128);
      int stage = 0;
      uint32_t phase = 0;
      for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
        const int i = static_cast<int>(tile / p.tiles_j);
        const int j0 = static_cast<int>(tile % p.tiles_j) * 128;
        if (!mbar_wait(&sm.in_empty[stage], phase ^ 1, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&sm.in_full[stage], 2 * TILE_BYTES);
        tma_load_3d(sm.x[stage], &tm_x, &sm.in_full[stage], 0, j0, i);
        tma_load_3d(sm.x[stage] + SLAB_BYTES, &tm_x, &sm.in_full[stage], 64, j0, i);
        tma_load_4d(sm.t[stage], &tm_t, &sm.in_full[stage], j0, i % p.t_rpb, 0, i / p.t_rpb);
        if (++stage == STAGES) {
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
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&sm.acc_empty[acc], acc_phase ^ 1, p.status, ST_TIMEOUT_MMA)) break;
        if (!mbar_wait(&sm.xn_full[stage], phase, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const uint32_t d_tmem = tmem_base + acc * 256 + g * 128;
          const uint32_t in = smem_u32(g == 0 ? sm.x[stage] : sm.t[stage]);
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint64_t adesc = umma_desc_kmajor(in + s * SLAB_BYTES, 128);
            const uint64_t bdesc = umma_desc_kmajor(smem_u32(sm.w + (g * 2 + s) * SLAB_BYTES), 128);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16_ss(d_tmem, umma_desc_advance(adesc, k * 32), umma_desc_advance(bdesc, k * 32), idesc,
                           (s | k) != 0);
          }
        }
        umma_commit(&sm.in_empty[stage]);
        umma_commit(&sm.acc_full[acc]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp < 6) {
    const int r = threadIdx.x - 64;
    int stage = 0;
    uint32_t phase = 0;
    for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
      if (!mbar_wait(&sm.in_full[stage], phase, p.status, ST_TIMEOUT_PROLOGUE)) break;
      uint4 v[16];
      // x tile: in-place layer norm of this thread's row.
      ln_load_row(sm.x[stage], r, v);
      ln_rows_inplace(v, sm.gamma_in, sm.beta_in, p.eps);
      ln_store_row(sm.x[stage], r, v);
      // t tile: gather this pair's column of the [channel][pair] tile.
      {
        const unsigned short* tcol = reinterpret_cast<const unsigned short*>(sm.t[stage]) + r;
        uint32_t* w = reinterpret_cast<uint32_t*>(v);
#pragma unroll
        for (int i = 0; i < 64; ++i)
          w[i] = static_cast<uint32_t>(tcol[(2 * i) * 128]) | (static_cast<uint32_t>(tcol[(2 * i + 1) * 128]) << 16);
      }
      ln_rows_inplace(v, sm.gamma_out, sm.beta_out, p.eps);
      // Rows may overwrite the tile only once every column has been read.
      mbar_arrive(&sm.col_read[stage]);
      if (!mbar_wait(&sm.col_read[stage], phase, p.status, ST_TIMEOUT_PROLOGUE)) break;
      ln_store_row(sm.t[stage], r, v);
      fence_proxy_async();
      mbar_arrive(&sm.xn_full[stage]);
      if (++stage == STAGES) {
        stage = 0;
        phase ^= 1;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int pr = quarter * 32 + lane;  // pair inside the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    uint32_t it = 0;
    for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
      const int i = static_cast<int>(tile / p.tiles_j);
      const int j = static_cast<int>(tile % p.tiles_j) * 128 + pr;
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
#if B200_FIN_TMASTORE
      // the previous tile must have left the staging buffer; the vote makes the outcome of the
      // bounded wait the same for all 128 threads, which meet at a barrier below
      if (threadIdx.x == EPI_THREAD0) tma_store_wait_read();
      if (!named_barrier_and(1, 128, mbar_wait(&sm.acc_full[acc], acc_phase, p.status, ST_TIMEOUT_EPILOGUE))) break;
#else
      if (!mbar_wait(&sm.acc_full[acc], acc_phase, p.status, ST_TIMEOUT_EPILOGUE)) break;
#endif
      tc_fence_after();
      const long long off = static_cast<long long>(i) * p.os_i + static_cast<long long>(j) * p.os_j;
#pragma unroll 1
      for (int chunk = 0; chunk < 4; ++chunk) {
        uint32_t g[32], o[32];
        tmem_ld32(lane_addr + acc * 256 + chunk * 32, g);
        tmem_ld32(lane_addr + acc * 256 + 128 + chunk * 32, o);
        tmem_ld_wait();
        if (j < p.n_j) {
#if !B200_FIN_TMASTORE
          uint4* dst = reinterpret_cast<uint4*>(p.out + off + chunk * 32);
#endif
          const uint4* res = p.residual ? reinterpret_cast<const uint4*>(p.residual + off + chunk * 32) : nullptr;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t u[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int c = 8 * q + 2 * e;
              const uint32_t ov = pack_bf16x2(__uint_as_float(o[c]), __uint_as_float(o[c + 1]));
              const uint32_t sg = sigmoid_bf16x2(__uint_as_float(g[c]), __uint_as_float(g[c + 1]));
              u[e] = bf16x2_mul(ov, sg);
            }
            if (res) {  // the caller's z + update, one more bf16 rounding
              const uint4 rv = res[q];
              u[0] = bf16x2_add(rv.x, u[0]);
              u[1] = bf16x2_add(rv.y, u[1]);
              u[2] = bf16x2_add(rv.z, u[2]);
              u[3] = bf16x2_add(rv.w, u[3]);
            }
#if B200_FIN_TMASTORE
            *reinterpret_cast<uint4*>(sm.out + (chunk >> 1) * SLAB_BYTES + sw128_offset(pr, (chunk & 1) * 4 + q)) =
                make_uint4(u[0], u[1], u[2], u[3]);
#else
            dst[q] = make_uint4(u[0], u[1], u[2], u[3]);
#endif
          }
        }
      }
#if B200_FIN_TMASTORE
      fence_proxy_async();
      named_barrier(1, 128);
      if (threadIdx.x == EPI_THREAD0) {  // rows past n_j are outside the tensor and are not written
        const int j0 = static_cast<int>(tile % p.tiles_j) * 128;
        tma_store_3d(&tm_out, sm.out, 0, j0, i);
        tma_store_3d(&tm_out, sm.out + SLAB_BYTES, 64, j0, i);
        tma_store_commit();
      }
#endif
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.acc_empty[acc]);
    }
  }

#if B200_FIN_TMASTORE
  if (threadIdx.x == EPI_THREAD0) tma_store_wait_all();
#endif
  if (*reinterpret_cast<volatile int*>(p.status) != ST_OK)
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

}  // namespace b200

extern "C" size_t b200tri_trimul_finish_workspace_bytes(void) { return 256 * 128 * 2 + 1024 + 1024; }

extern "C" int b200tri_trimul_finish(const b200tri_trimul_finish_args* a, b200tri_stream_t stream_) {
  using namespace b200;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  B200_REQUIRE(a != nullptr, B200TRI_ERR_INVALID, "finish: null args");
  B200_REQUIRE(a->t && a->x && a->out && a->p_out && a->g_out && a->norm_in_scale && a->norm_in_bias &&
                   a->norm_out_scale && a->norm_out_bias,
               B200TRI_ERR_INVALID, "finish: null pointer argument");
  B200_REQUIRE(a->n_i > 0 && a->n_j > 0, B200TRI_ERR_INVALID, "finish: sizes must be positive");
  B200_REQUIRE(a->t_ld % 8 == 0 && a->t_chan_stride % 8 == 0 && a->xs_i % 8 == 0 && a->xs_j % 8 == 0 &&
                   a->os_i % 8 == 0 && a->os_j % 8 == 0,
               B200TRI_ERR_INVALID, "finish: pitches and strides must be multiples of 8 elements");
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(a->out) | reinterpret_cast<uintptr_t>(a->residual)) & 15) == 0,
               B200TRI_ERR_INVALID, "finish: out/residual must be 16-byte aligned");
  B200_REQUIRE(a->workspace && a->workspace_bytes >= b200tri_trimul_finish_workspace_bytes(), B200TRI_ERR_WORKSPACE,
               "finish: workspace of %zu bytes needed", b200tri_trimul_finish_workspace_bytes());
  int* status = device_status_word();
  B200_REQUIRE(status != nullptr, B200TRI_ERR_CUDA, "finish: no current CUDA device");

  Carver ws(a->workspace);
  __nv_bfloat16* wpk = ws.take<__nv_bfloat16>(256 * 128);
  uint32_t* ln = ws.take<uint32_t>(256, 256);
  pack_transpose(static_cast<const __nv_bfloat16*>(a->g_out), 128, 0, 128, wpk, stream);
  pack_transpose(static_cast<const __nv_bfloat16*>(a->p_out), 128, 0, 128, wpk + 128 * 128, stream);
  pack_copy_words(a->norm_in_scale, ln, 64, stream);
  pack_copy_words(a->norm_in_bias, ln + 64, 64, stream);
  pack_copy_words(a->norm_out_scale, ln + 128, 64, stream);
  pack_copy_words(a->norm_out_bias, ln + 192, 64, stream);

  CUtensorMap tm_x, tm_t, tm_w, tm_out;
  {
    const uint64_t dims[3] = {128, (uint64_t)a->n_j, (uint64_t)a->n_i};
    const uint64_t str[2] = {(uint64_t)a->os_j * 2, (uint64_t)a->os_i * 2};
    const uint32_t box[3] = {64, 128, 1};
    int rc = make_tmap(&tm_out, a->out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  {
    const uint64_t dims[3] = {128, (uint64_t)a->n_j, (uint64_t)a->n_i};
    const uint64_t str[2] = {(uint64_t)a->xs_j * 2, (uint64_t)a->xs_i * 2};
    const uint32_t box[3] = {64, 128, 1};
    int rc = make_tmap(&tm_x, a->x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  {
    // (j, row in block, channel, block); one block when t is not row-blocked
    const bool blocked = a->t_rows_per_block > 0 && a->t_rows_per_block < a->n_i;
    const uint64_t rpb = blocked ? (uint64_t)a->t_rows_per_block : (uint64_t)a->n_i;
    const uint64_t blocks = (a->n_i + rpb - 1) / rpb;
    B200_REQUIRE(!blocked || a->t_block_stride % 8 == 0, B200TRI_ERR_INVALID, "finish: t_block_stride must be a multiple of 8");
    const uint64_t dims[4] = {(uint64_t)a->n_j, rpb, 128, blocks};
    const uint64_t str[3] = {(uint64_t)a->t_ld * 2, (uint64_t)a->t_chan_stride * 2,
                             (uint64_t)(blocked ? a->t_block_stride : a->t_chan_stride * 128) * 2};
    const uint32_t box[4] = {128, 1, 128, 1};
    int rc = make_tmap(&tm_t, a->t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, str, box, Swz::None);
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {128, 256};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 128};
    int rc = make_tmap(&tm_w, wpk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  FinishParams p;
  p.n_i = a->n_i;
  p.n_j = a->n_j;
  p.tiles_j = (a->n_j + 127) / 128;
  p.total_tiles = static_cast<long long>(p.tiles_j) * a->n_i;
  p.ln = ln;
  p.residual = static_cast<const __nv_bfloat16*>(a->residual);
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.os_i = a->os_i;
  p.os_j = a->os_j;
  p.eps = a->eps;
  p.t_rpb = (a->t_rows_per_block > 0 && a->t_rows_per_block < a->n_i) ? a->t_rows_per_block : a->n_i;
  p.status = status;

  {
    const int rc = ensure_smem_limit(reinterpret_cast<const void*>(finish_kernel), (int)sizeof(Smem));
    if (rc) return rc;
  }
  const long long grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
  {
    TimedLaunch timed(K_TRIMUL_FINISH, stream);
    count_launch();
    finish_kernel<<<static_cast<unsigned>(grid), THREADS, sizeof(Smem), stream>>>(tm_x, tm_t, tm_w, tm_out, p);
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}
