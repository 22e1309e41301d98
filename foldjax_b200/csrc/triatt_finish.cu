// Triangle attention, output stage.
//
//   g    = bf16(sigmoid(bf16(LN(x) @ Wg)))
//   out  = bf16(bf16(o * g) @ Wo)   (+ residual), written through caller strides so the
//          ending node lands transposed back in place
//
// Reference: src/foldjax/models/boltz2/models/triangle/triangle_attention.py
// :360-366 (gate projection), :421-425 (gating, output projection), :160-161.
// o is the attention core's output [n_outer][n_inner][128] in the attention
// frame; x and out are addressed as base + o*stride_outer + t*stride_inner.
//
// One tile = 128 consecutive pairs. Persistent, one CTA per SM:
//   warp 0      TMA producer (Wg, Wo once; x and o tiles, 2-stage ring)
//   warp 1      MMA issuer: G = LN(x).Wg^T, then OUT = (o*g).Wo^T
//   warps 2-5   layer norm of x in place, then the gating of o in place
//               (the o tile becomes the A operand of the second product)
//   warps 6-9   epilogue of OUT
// The gating of tile t is done after the layer norm of tile t+1, so the first
// product of the next tile runs while this tile is gated.
// Bound: HBM (read x and o, write out: 3 * n*n*128*2 bytes; + residual).
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
// swizzled slabs) and writes it with two TMA stores through the caller's strides; 0: every
// thread stores its pair's row itself, 64 bytes at a time (32 cache lines per warp store).
#ifndef B200_AFIN_TMASTORE
#define B200_AFIN_TMASTORE 1
#endif

struct Smem {
  uint8_t w[4 * SLAB_BYTES];  // Wg^T (2 slabs), Wo^T (2 slabs)
  uint8_t x[STAGES][TILE_BYTES];
  uint8_t o[STAGES][TILE_BYTES];
#if B200_AFIN_TMASTORE
  uint8_t out[TILE_BYTES];
#endif
  uint32_t gamma2[64], beta2[64];
  uint64_t w_full, in_full[STAGES], xn_full[STAGES], y_full[STAGES], in_empty[STAGES];
  uint64_t g_full[2], g_empty[2], out_full[2], out_empty[2];
  uint32_t tmem_base;
};
static_assert(sizeof(Smem) <= 232448, "shared memory budget");

struct Params {
  int n_outer, n_inner, tiles_inner;
  long long total_tiles;
  const uint32_t* ln;  // gamma, beta: 2 x 64 words
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  long long os_outer, os_inner;
  float eps;
  int* status;
};

__global__ void __launch_bounds__(THREADS, 1)
att_finish_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_o,
                  const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_out,
                  const Params p) {
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
    tma_prefetch_desc(&tm_o);
    tma_prefetch_desc(&tm_w);
    mbar_init(&sm.w_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.in_full[s], 1);
      mbar_init(&sm.xn_full[s], 128);
      mbar_init(&sm.y_full[s], 128);
      mbar_init(&sm.in_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sm.g_full[a], 1);
      mbar_init(&sm.g_empty[a], 4);
      mbar_init(&sm.out_full[a], 1);
      mbar_init(&sm.out_empty[a], 4);
    }
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
  // TMEM: buffer a (= tile parity): G at a*256, OUT at a*256 + 128.

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&sm.w_full, 4 * SLAB_BYTES);
      for (int g = 0; g < 2; ++g)
        for (int s = 0; s < 2; ++s) tma_load_2d(sm.w + (g * 2 + s) * SLAB_BYTES, &tm_w, &sm.w_full, s * 64, g * 128);
      int stage = 0;
      uint32_t phase = 0;
      for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
        const int o = static_cast<int>(tile / p.tiles_inner);
        const int t0 = static_cast<int>(tile % p.tiles_inner) * 128;
        if (!mbar_wait(&sm.in_empty[stage], phase ^ 1, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&sm.in_full[stage], 2 * TILE_BYTES);
        tma_load_3d(sm.x[stage], &tm_x, &sm.in_full[stage], 0, t0, o);
        tma_load_3d(sm.x[stage] + SLAB_BYTES, &tm_x, &sm.in_full[stage], 64, t0, o);
        tma_load_3d(sm.o[stage], &tm_o, &sm.in_full[stage], 0, t0, o);
        tma_load_3d(sm.o[stage] + SLAB_BYTES, &tm_o, &sm.in_full[stage], 64, t0, o);
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
      // Two products per tile; the second of tile t is issued after the first of
      // tile t+1, mirroring the order in which the gating warps deliver operands.
      auto product = [&](uint32_t d_tmem, uint32_t a_smem, int wgroup) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint64_t adesc = umma_desc_kmajor(a_smem + s * SLAB_BYTES, 128);
          const uint64_t bdesc = umma_desc_kmajor(smem_u32(sm.w + (wgroup * 2 + s) * SLAB_BYTES), 128);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(d_tmem, umma_desc_advance(adesc, k * 32), umma_desc_advance(bdesc, k * 32), idesc,
                         (s | k) != 0);
        }
      };
      long long n_my = 0;
      for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) ++n_my;
      for (long long it = 0; it <= n_my && alive; ++it) {
        if (it < n_my) {  // first product of tile `it`
          const int stage = static_cast<int>(it % STAGES);
          const uint32_t phase = static_cast<uint32_t>((it / STAGES) & 1);
          const uint32_t a = static_cast<uint32_t>(it & 1), aph = static_cast<uint32_t>((it >> 1) & 1);
          if (!mbar_wait(&sm.g_empty[a], aph ^ 1, p.status, ST_TIMEOUT_MMA)) break;
          if (!mbar_wait(&sm.xn_full[stage], phase, p.status, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
          product(tmem_base + a * 256, smem_u32(sm.x[stage]), 0);
          umma_commit(&sm.g_full[a]);
        }
        if (it > 0) {  // second product of tile `it - 1`
          const long long jt = it - 1;
          const int stage = static_cast<int>(jt % STAGES);
          const uint32_t phase = static_cast<uint32_t>((jt / STAGES) & 1);
          const uint32_t a = static_cast<uint32_t>(jt & 1), aph = static_cast<uint32_t>((jt >> 1) & 1);
          if (!mbar_wait(&sm.out_empty[a], aph ^ 1, p.status, ST_TIMEOUT_MMA)) break;
          if (!mbar_wait(&sm.y_full[stage], phase, p.status, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
          product(tmem_base + a * 256 + 128, smem_u32(sm.o[stage]), 1);
          umma_commit(&sm.in_empty[stage]);
          umma_commit(&sm.out_full[a]);
        }
      }
    }
  } else if (warp < 6) {
    const int r = threadIdx.x - 64;
    const int quarter = warp & 3;
    // This thread's TMEM lane must be its warp's quarter; rows are assigned so
    // that thread r handles tile row `row`.
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    (void)r;
    long long n_my = 0;
    for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) ++n_my;
    bool alive = true;
    for (long long it = 0; it <= n_my && alive; ++it) {
      if (it < n_my) {  // layer norm of tile `it`
        const int stage = static_cast<int>(it % STAGES);
        const uint32_t phase = static_cast<uint32_t>((it / STAGES) & 1);
        if (!mbar_wait(&sm.in_full[stage], phase, p.status, ST_TIMEOUT_PROLOGUE)) break;
        uint4 v[16];
        ln_load_row(sm.x[stage], row, v);
        ln_rows_inplace(v, sm.gamma2, sm.beta2, p.eps);
        ln_store_row(sm.x[stage], row, v);
        fence_proxy_async();
        mbar_arrive(&sm.xn_full[stage]);
      }
      if (it > 0) {  // gating of tile `it - 1`: o <- bf16(o * bf16(sigmoid(bf16(G))))
        const long long jt = it - 1;
        const int stage = static_cast<int>(jt % STAGES);
        const uint32_t a = static_cast<uint32_t>(jt & 1), aph = static_cast<uint32_t>((jt >> 1) & 1);
        if (!mbar_wait(&sm.g_full[a], aph, p.status, ST_TIMEOUT_PROLOGUE)) break;
        tc_fence_after();
        uint8_t* otile = sm.o[stage];
#pragma unroll 1
        for (int chunk = 0; chunk < 4; ++chunk) {  // 32 channels = 4 sixteen-byte chunks of one slab
          uint32_t g[32];
          tmem_ld32(lane_addr + a * 256 + chunk * 32, g);
          tmem_ld_wait();
          const int slab = chunk >> 1;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const int c = (chunk & 1) * 4 + c4;  // chunk index inside the slab
            uint4* ptr = reinterpret_cast<uint4*>(otile + slab * SLAB_BYTES + sw128_offset(row, c));
            uint4 ov = *ptr;
            ov.x = bf16x2_mul(ov.x, sigmoid_bf16x2(__uint_as_float(g[8 * c4 + 0]), __uint_as_float(g[8 * c4 + 1])));
            ov.y = bf16x2_mul(ov.y, sigmoid_bf16x2(__uint_as_float(g[8 * c4 + 2]), __uint_as_float(g[8 * c4 + 3])));
            ov.z = bf16x2_mul(ov.z, sigmoid_bf16x2(__uint_as_float(g[8 * c4 + 4]), __uint_as_float(g[8 * c4 + 5])));
            ov.w = bf16x2_mul(ov.w, sigmoid_bf16x2(__uint_as_float(g[8 * c4 + 6]), __uint_as_float(g[8 * c4 + 7])));
            *ptr = ov;
          }
        }
        tc_fence_before();
        fence_proxy_async();
        mbar_arrive(&sm.y_full[stage]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.g_empty[a]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    uint32_t it = 0;
    for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
      const int o = static_cast<int>(tile / p.tiles_inner);
      const int t = static_cast<int>(tile % p.tiles_inner) * 128 + row;
      const uint32_t a = it & 1, aph = (it >> 1) & 1;
#if B200_AFIN_TMASTORE
      // the previous tile must have left the staging buffer; the vote makes the outcome of the
      // bounded wait the same for all 128 threads, which meet at a barrier below
      if (threadIdx.x == EPI_THREAD0) tma_store_wait_read();
      if (!named_barrier_and(1, 128, mbar_wait(&sm.out_full[a], aph, p.status, ST_TIMEOUT_EPILOGUE))) break;
#else
      if (!mbar_wait(&sm.out_full[a], aph, p.status, ST_TIMEOUT_EPILOGUE)) break;
#endif
      tc_fence_after();
      const long long off = static_cast<long long>(o) * p.os_outer + static_cast<long long>(t) * p.os_inner;
#pragma unroll 1
      for (int chunk = 0; chunk < 4; ++chunk) {
        uint32_t v[32];
        tmem_ld32(lane_addr + a * 256 + 128 + chunk * 32, v);
        tmem_ld_wait();
        if (t < p.n_inner) {
#if !B200_AFIN_TMASTORE
          uint4* dst = reinterpret_cast<uint4*>(p.out + off + chunk * 32);
#endif
          const uint4* res = p.residual ? reinterpret_cast<const uint4*>(p.residual + off + chunk * 32) : nullptr;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t u[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              u[e] = pack_bf16x2(__uint_as_float(v[8 * q + 2 * e]), __uint_as_float(v[8 * q + 2 * e + 1]));
            if (res) {
              const uint4 rv = res[q];
              u[0] = bf16x2_add(rv.x, u[0]);
              u[1] = bf16x2_add(rv.y, u[1]);
              u[2] = bf16x2_add(rv.z, u[2]);
              u[3] = bf16x2_add(rv.w, u[3]);
            }
#if B200_AFIN_TMASTORE
            *reinterpret_cast<uint4*>(sm.out + (chunk >> 1) * SLAB_BYTES + sw128_offset(row, (chunk & 1) * 4 + q)) =
                make_uint4(u[0], u[1], u[2], u[3]);
#else
            dst[q] = make_uint4(u[0], u[1], u[2], u[3]);
#endif
          }
        }
      }
#if B200_AFIN_TMASTORE
      fence_proxy_async();
      named_barrier(1, 128);
      if (threadIdx.x == EPI_THREAD0) {  // rows past n_inner are outside the tensor and are not written
        const int t0 = static_cast<int>(tile % p.tiles_inner) * 128;
        tma_store_3d(&tm_out, sm.out, 0, t0, o);
        tma_store_3d(&tm_out, sm.out + SLAB_BYTES, 64, t0, o);
        tma_store_commit();
      }
#endif
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.out_empty[a]);
    }
  }

#if B200_AFIN_TMASTORE
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

extern "C" size_t b200tri_triatt_finish_workspace_bytes(void) { return 256 * 128 * 2 + 1024 + 1024; }

extern "C" int b200tri_triatt_finish(const b200tri_triatt_finish_args* a, b200tri_stream_t stream_) {
  using namespace b200;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  B200_REQUIRE(a != nullptr, B200TRI_ERR_INVALID, "att finish: null args");
  B200_REQUIRE(a->o && a->x && a->out && a->norm_scale && a->norm_bias && a->w_g && a->w_o, B200TRI_ERR_INVALID,
               "att finish: null pointer argument");
  B200_REQUIRE(a->n_outer > 0 && a->n_inner > 0, B200TRI_ERR_INVALID, "att finish: sizes must be positive");
  B200_REQUIRE(a->xs_outer % 8 == 0 && a->xs_inner % 8 == 0 && a->os_outer % 8 == 0 && a->os_inner % 8 == 0,
               B200TRI_ERR_INVALID, "att finish: strides must be multiples of 8 elements");
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(a->out) | reinterpret_cast<uintptr_t>(a->residual)) & 15) == 0,
               B200TRI_ERR_INVALID, "att finish: out/residual must be 16-byte aligned");
  B200_REQUIRE(a->workspace && a->workspace_bytes >= b200tri_triatt_finish_workspace_bytes(), B200TRI_ERR_WORKSPACE,
               "att finish: workspace of %zu bytes needed", b200tri_triatt_finish_workspace_bytes());
  int* status = device_status_word();
  B200_REQUIRE(status != nullptr, B200TRI_ERR_CUDA, "att finish: no current CUDA device");

  Carver ws(a->workspace);
  __nv_bfloat16* wpk = ws.take<__nv_bfloat16>(256 * 128);
  uint32_t* ln = ws.take<uint32_t>(128, 256);
  pack_transpose(static_cast<const __nv_bfloat16*>(a->w_g), 128, 0, 128, wpk, stream);
  pack_transpose(static_cast<const __nv_bfloat16*>(a->w_o), 128, 0, 128, wpk + 128 * 128, stream);
  pack_copy_words(a->norm_scale, ln, 64, stream);
  pack_copy_words(a->norm_bias, ln + 64, 64, stream);

  CUtensorMap tm_x, tm_o, tm_w, tm_out;
  {  // the result through the caller's strides (the ending node lands transposed back in place)
    const uint64_t dims[3] = {128, (uint64_t)a->n_inner, (uint64_t)a->n_outer};
    const uint64_t str[2] = {(uint64_t)a->os_inner * 2, (uint64_t)a->os_outer * 2};
    const uint32_t box[3] = {64, 128, 1};
    int rc = make_tmap(&tm_out, a->out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  {
    const uint64_t dims[3] = {128, (uint64_t)a->n_inner, (uint64_t)a->n_outer};
    const uint64_t str[2] = {(uint64_t)a->xs_inner * 2, (uint64_t)a->xs_outer * 2};
    const uint32_t box[3] = {64, 128, 1};
    int rc = make_tmap(&tm_x, a->x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  {
    const uint64_t dims[3] = {128, (uint64_t)a->n_inner, (uint64_t)a->n_outer};
    const uint64_t str[2] = {256, (uint64_t)a->n_inner * 256};
    const uint32_t box[3] = {64, 128, 1};
    int rc = make_tmap(&tm_o, a->o, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {128, 256};
    const uint64_t str[1] = {256};
    const uint32_t box[2] = {64, 128};
    int rc = make_tmap(&tm_w, wpk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  Params p;
  p.n_outer = a->n_outer;
  p.n_inner = a->n_inner;
  p.tiles_inner = (a->n_inner + 127) / 128;
  p.total_tiles = static_cast<long long>(p.tiles_inner) * a->n_outer;
  p.ln = ln;
  p.residual = static_cast<const __nv_bfloat16*>(a->residual);
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.os_outer = a->os_outer;
  p.os_inner = a->os_inner;
  p.eps = a->eps;
  p.status = status;

  {
    const int rc = ensure_smem_limit(reinterpret_cast<const void*>(att_finish_kernel), (int)sizeof(Smem));
    if (rc) return rc;
  }
  const long long grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
  {
    TimedLaunch timed(K_TRIATT_FINISH, stream);
    count_launch();
    att_finish_kernel<<<static_cast<unsigned>(grid), THREADS, sizeof(Smem), stream>>>(tm_x, tm_o, tm_w, tm_out, p);
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}
