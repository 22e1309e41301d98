// Triangle attention, projection stage.
//
//   xn   = LN(x)                                   (x is read through caller strides,
//                                                   so the ending node is the same
//                                                   kernel on swapped strides)
//   q    = bf16(bf16(xn @ Wq) / bf16(sqrt(32)))    [o][t][128]   heads-major channels
//   k    = bf16(xn @ Wk)                            [o][t][128]
//   vT   = fp16(bf16(xn @ Wv))                      [o][128][ld]  channel-major per row o
//   bias = bf16(xn @ Wb)                            [4][o][ld]    (tri_bias[h][j][k] of the
//                                                   reference with j = o, k = t)
//
// Reference: src/foldjax/models/boltz2/models/triangle/triangle_attention.py
// :132 (LN), :144-146 (bias), :360-382 (fused projections), :399-400 (q scale).
// The gate projection is not done here: the output stage recomputes it from x,
// which costs the same bytes as reading a stored gate and saves writing one.
//
// V is stored transposed and in fp16: the core kernel multiplies P (fp16, 11
// significand bits) by V on the tensor cores. A bf16-rounded value of magnitude in
// [2^-14, 65504] is exactly representable in fp16 (8 significand bits fit in 11); larger
// ones saturate, values in [2^-24, 2^-14) land on fp16 subnormals and lose significand
// bits (at most the absolute 2^-25), smaller ones flush to zero. V is a layer-normed
// projection of order one, so only the exact range matters in practice.
//
// One tile = 128 consecutive pairs (o, t0..t0+127). Persistent, one CTA per SM:
//   warp 0      TMA producer (weights once, x tiles in a 3-stage ring)
//   warp 1      MMA issuer: [q|k] = xn.[Wq|Wk]^T (N=256), bias = xn.Wb^T (N=16),
//               vT = Wv.xn^T ("transposed": a TMEM lane is a channel)
//   warps 2-9   layer norm in place (two threads per pair)
//   warps 10-13 epilogue
// TMEM: [q|k] 256 columns, vT 128, bias 16; each group is released on its own
// so the next tile's MMAs overlap this tile's epilogue.
// Bound: HBM (read x, write q, k, vT: 4 * n*n*128*2 bytes).
#include <cuda_fp16.h>

#include "host.cuh"
#include "ln.cuh"
#include "pack.cuh"
#include "tc.cuh"

namespace b200 {

namespace {

// 1: q, k and vT tiles are staged in shared memory and written with TMA stores (one elected
// thread, two 16 KiB boxes each); 0: every thread stores its row's 64-byte pieces itself, so a
// warp's store instruction touches 32 cache lines and the L1 pipe bounds the kernel.
#ifndef B200_APROJ_TMASTORE
#define B200_APROJ_TMASTORE 1
#endif
#if B200_APROJ_TMASTORE
constexpr int XSTAGES = 2;
#else
constexpr int XSTAGES = 3;
#endif
constexpr int TILE_BYTES = 2 * SLAB_BYTES;
constexpr int W_BYTES = 8 * SLAB_BYTES;  // rows 0..255 [Wq|Wk], 256..383 Wv, 384..399 Wb, rest zero
constexpr int LN_WARPS = 8;  // two threads per pair
constexpr int THREADS = 64 + LN_WARPS * 32 + 128;
constexpr int EPI_THREAD0 = 64 + LN_WARPS * 32;  // first thread of the epilogue warps
constexpr uint32_t TM_QK = 0, TM_V = 256, TM_B = 384;
enum { G_QK = 0, G_B = 1, G_V = 2 };

struct Smem {
  uint8_t w[W_BYTES];
  uint8_t x[XSTAGES][TILE_BYTES];
#if B200_APROJ_TMASTORE
  uint8_t out[TILE_BYTES];  // staging of one 32 KiB output tile (q, then k, then vT)
#endif
  uint32_t gamma2[64];
  uint32_t beta2[64];
  uint64_t w_full, x_full[XSTAGES], xn_full[XSTAGES], x_empty[XSTAGES], acc_full[3], acc_empty[3];
  uint32_t tmem_base;
};
static_assert(sizeof(Smem) <= 232448, "shared memory budget");

struct Params {
  int n_outer, n_inner, tiles_inner;
  long long total_tiles;
  const uint32_t* gamma2;
  const uint32_t* beta2;
  __nv_bfloat16* q;
  __nv_bfloat16* k;
  __half* vt;
  __nv_bfloat16* bias;
  long long ld;           // pitch of vT rows and of bias rows (elements)
  long long bias_head_stride;
  float q_scale;          // bf16(sqrt(head_dim))
  float eps;
  int* status;
};

__global__ void __launch_bounds__(THREADS, 1)
att_project_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                   const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_vt,
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
    tma_prefetch_desc(&tm_w);
    mbar_init(&sm.w_full, 1);
    for (int s = 0; s < XSTAGES; ++s) {
      mbar_init(&sm.x_full[s], 1);
      mbar_init(&sm.xn_full[s], LN_WARPS * 32);
      mbar_init(&sm.x_empty[s], 1);
    }
    for (int g = 0; g < 3; ++g) {
      mbar_init(&sm.acc_full[g], 1);
      mbar_init(&sm.acc_empty[g], 4);
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
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 256);
      constexpr uint32_t idesc_b = umma_idesc_bf16(128, 16);
      constexpr uint32_t idesc_v = umma_idesc_bf16(128, 128);
      bool alive = mbar_wait(&sm.w_full, 0, p.status, ST_TIMEOUT_MMA);
      int stage = 0;
      uint32_t phase = 0, it = 0;
      for (long long tile = blockIdx.x; tile < p.total_tiles && alive; tile += gridDim.x, ++it) {
        if (!mbar_wait(&sm.xn_full[stage], phase, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t xs = smem_u32(sm.x[stage]);
        const uint32_t ws = smem_u32(sm.w);
        // [q|k]: A = xn (rows = pairs), B = weight rows 0..255 (slabs 0..3: rows 0-127 s0,s1; rows 128-255 s0,s1)
        if (!mbar_wait(&sm.acc_empty[G_QK], (it & 1) ^ 1, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int half = 0; half < 2; ++half)  // N = 256 as two N = 128 halves (weight groups 0 and 1)
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint64_t adesc = umma_desc_kmajor(xs + s * SLAB_BYTES, 128);
            const uint64_t bdesc = umma_desc_kmajor(ws + (half * 2 + s) * SLAB_BYTES, 128);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16_ss(tmem_base + TM_QK + half * 128, umma_desc_advance(adesc, k * 32),
                           umma_desc_advance(bdesc, k * 32), idesc_v, (s | k) != 0);
          }
        umma_commit(&sm.acc_full[G_QK]);
        // bias: A = xn, B = weight rows 384..399 (group 3), N = 16
        if (!mbar_wait(&sm.acc_empty[G_B], (it & 1) ^ 1, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint64_t adesc = umma_desc_kmajor(xs + s * SLAB_BYTES, 128);
          const uint64_t bdesc = umma_desc_kmajor(ws + (3 * 2 + s) * SLAB_BYTES, 128);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base + TM_B, umma_desc_advance(adesc, k * 32), umma_desc_advance(bdesc, k * 32),
                         idesc_b, (s | k) != 0);
        }
        umma_commit(&sm.acc_full[G_B]);
        // vT: A = Wv (rows = channels, group 2), B = xn (rows = pairs)
        if (!mbar_wait(&sm.acc_empty[G_V], (it & 1) ^ 1, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint64_t adesc = umma_desc_kmajor(ws + (2 * 2 + s) * SLAB_BYTES, 128);
          const uint64_t bdesc = umma_desc_kmajor(xs + s * SLAB_BYTES, 128);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base + TM_V, umma_desc_advance(adesc, k * 32), umma_desc_advance(bdesc, k * 32),
                         idesc_v, (s | k) != 0);
        }
        umma_commit(&sm.acc_full[G_V]);
        umma_commit(&sm.x_empty[stage]);
        if (++stage == XSTAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      (void)idesc_qk;
    }
  } else if (warp < 2 + LN_WARPS) {
    const int r = (warp - 2) * 16 + (lane & 15);  // pair of the tile; lanes l and l ^ 16 share it
    int stage = 0;
    uint32_t phase = 0;
    for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
      if (!mbar_wait(&sm.x_full[stage], phase, p.status, ST_TIMEOUT_PROLOGUE)) break;
      ln_row_two_threads(sm.x[stage], r, lane >> 4, sm.gamma2, sm.beta2, p.eps);
      fence_proxy_async();
      mbar_arrive(&sm.xn_full[stage]);
      if (++stage == XSTAGES) {
        stage = 0;
        phase ^= 1;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // TMEM lane: a pair for q/k/bias, a channel for vT
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t qs = pack_bf16x2(p.q_scale, p.q_scale);
    const float q_inv = 1.0f / bf16_lo(qs);
    uint32_t it = 0;
    for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
      const int o = static_cast<int>(tile / p.tiles_inner);
      const int t0 = static_cast<int>(tile % p.tiles_inner) * 128;
      const int t = t0 + row;
#if !B200_APROJ_TMASTORE
      const long long pair_off = (static_cast<long long>(o) * p.n_inner + t) * 128;
#endif
      // ---- q and k: thread = pair, 128 + 128 channels
#if B200_APROJ_TMASTORE
      // (votes: the outcome of each bounded wait is made the same for all 128 threads, which
      // meet at named barriers around the staging buffer)
      if (!named_barrier_and(1, 128, mbar_wait(&sm.acc_full[G_QK], it & 1, p.status, ST_TIMEOUT_EPILOGUE))) break;
#else
      if (!mbar_wait(&sm.acc_full[G_QK], it & 1, p.status, ST_TIMEOUT_EPILOGUE)) break;
#endif
      tc_fence_after();
#if B200_APROJ_TMASTORE
#pragma unroll 1
      for (int part = 0; part < 2; ++part) {  // q, then k: one staged 32 KiB tile each
        if (threadIdx.x == EPI_THREAD0) tma_store_wait_read();
        named_barrier(1, 128);
#pragma unroll 1
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t r[32];
          tmem_ld32(lane_addr + TM_QK + (part * 4 + c4) * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4) {
            uint32_t u[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              uint32_t v2 = pack_bf16x2(__uint_as_float(r[8 * g4 + 2 * e]), __uint_as_float(r[8 * g4 + 2 * e + 1]));
              // q / sqrt(d) as the product with the rounded reciprocal: the same bf16 as the true
              // division for every bf16 q (the quotient is never within 1e-5 of a rounding boundary)
              if (part == 0) v2 = pack_bf16x2(bf16_lo(v2) * q_inv, bf16_hi(v2) * q_inv);
              u[e] = v2;
            }
            // row = pair, 16-byte chunk = 8 channels: channels 32*c4 + 8*g4 .. +7
            *reinterpret_cast<uint4*>(sm.out + (c4 >> 1) * SLAB_BYTES + sw128_offset(row, (c4 & 1) * 4 + g4)) =
                make_uint4(u[0], u[1], u[2], u[3]);
          }
        }
        fence_proxy_async();
        named_barrier(1, 128);
        if (threadIdx.x == EPI_THREAD0) {  // pairs past n_inner are outside the tensor and are not written
          const CUtensorMap* tm = part ? &tm_k : &tm_q;
          tma_store_3d(tm, sm.out, 0, t0, o);
          tma_store_3d(tm, sm.out + SLAB_BYTES, 64, t0, o);
          tma_store_commit();
        }
      }
#else
#pragma unroll 1
      for (int chunk = 0; chunk < 8; ++chunk) {
        uint32_t r[32];
        tmem_ld32(lane_addr + TM_QK + chunk * 32, r);
        tmem_ld_wait();
        if (t < p.n_inner) {
          __nv_bfloat16* base = (chunk < 4 ? p.q : p.k) + pair_off + (chunk & 3) * 32;
          uint4* dst = reinterpret_cast<uint4*>(base);
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4) {
            uint32_t u[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              uint32_t v2 = pack_bf16x2(__uint_as_float(r[8 * g4 + 2 * e]), __uint_as_float(r[8 * g4 + 2 * e + 1]));
              // q / sqrt(d): the quotient of two bf16 numbers, rounded to bf16. The divisor
              // is bf16(sqrt(32)) = 181/32 and q has an 8-bit significand, so the exact
              // quotient is a multiple of 1/181 of its ulp scale and never closer than
              // ~1e-5 (relative) to a bf16 rounding boundary: any fp32 value within 1e-6 of
              // it, such as the product with the rounded reciprocal, rounds to the same bf16
              // as the true division.
              if (chunk < 4) v2 = pack_bf16x2(bf16_lo(v2) * q_inv, bf16_hi(v2) * q_inv);
              u[e] = v2;
            }
            dst[g4] = make_uint4(u[0], u[1], u[2], u[3]);
          }
        }
      }
#endif
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.acc_empty[G_QK]);
      // ---- bias: thread = pair, 4 heads
#if B200_APROJ_TMASTORE
      if (!named_barrier_and(1, 128, mbar_wait(&sm.acc_full[G_B], it & 1, p.status, ST_TIMEOUT_EPILOGUE))) break;
#else
      if (!mbar_wait(&sm.acc_full[G_B], it & 1, p.status, ST_TIMEOUT_EPILOGUE)) break;
#endif
      tc_fence_after();
      {
        uint32_t r[16];
        tmem_ld16(lane_addr + TM_B, r);
        tmem_ld_wait();
        if (t < p.n_inner) {
#pragma unroll
          for (int h = 0; h < 4; ++h)
            p.bias[h * p.bias_head_stride + static_cast<long long>(o) * p.ld + t] =
                __float2bfloat16_rn(__uint_as_float(r[h]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.acc_empty[G_B]);
      // ---- vT: thread = channel, 128 pairs -> one contiguous run of the row
#if B200_APROJ_TMASTORE
      if (!named_barrier_and(1, 128, mbar_wait(&sm.acc_full[G_V], it & 1, p.status, ST_TIMEOUT_EPILOGUE))) break;
#else
      if (!mbar_wait(&sm.acc_full[G_V], it & 1, p.status, ST_TIMEOUT_EPILOGUE)) break;
#endif
      tc_fence_after();
#if B200_APROJ_TMASTORE
      if (threadIdx.x == EPI_THREAD0) tma_store_wait_read();
      named_barrier(1, 128);
#pragma unroll 1
      for (int chunk = 0; chunk < 4; ++chunk) {
        uint32_t r[32];
        tmem_ld32(lane_addr + TM_V + chunk * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) {
          uint32_t u[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = 8 * g4 + 2 * e;
            const uint32_t b2 = pack_bf16x2(__uint_as_float(r[c]), __uint_as_float(r[c + 1]));  // bf16(xn @ Wv)
            const __half2 h2 = __floats2half2_rn(bf16_lo(b2), bf16_hi(b2));
            u[e] = *reinterpret_cast<const uint32_t*>(&h2);
          }
          // row = channel, 16-byte chunk = 8 pairs: pairs 32*chunk + 8*g4 .. +7 of the tile
          *reinterpret_cast<uint4*>(sm.out + (chunk >> 1) * SLAB_BYTES + sw128_offset(row, (chunk & 1) * 4 + g4)) =
              make_uint4(u[0], u[1], u[2], u[3]);
        }
      }
      fence_proxy_async();
      named_barrier(1, 128);
      if (threadIdx.x == EPI_THREAD0) {
        tma_store_3d(&tm_vt, sm.out, t0, 0, o);
        if (t0 + 64 < p.n_inner) tma_store_3d(&tm_vt, sm.out + SLAB_BYTES, t0 + 64, 0, o);
        tma_store_commit();
      }
#else
      __half* vrow = p.vt + (static_cast<long long>(o) * 128 + row) * p.ld + t0;
#pragma unroll 1
      for (int chunk = 0; chunk < 4; ++chunk) {
        uint32_t r[32];
        tmem_ld32(lane_addr + TM_V + chunk * 32, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const uint32_t b2 = pack_bf16x2(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));  // bf16(xn @ Wv)
          const __half2 h2 = __floats2half2_rn(bf16_lo(b2), bf16_hi(b2));
          packed[e] = *reinterpret_cast<const uint32_t*>(&h2);
        }
        const int tc = t0 + chunk * 32;
        if (tc + 32 <= p.n_inner) {
          uint4* d4 = reinterpret_cast<uint4*>(vrow + chunk * 32);
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4)
            d4[g4] = make_uint4(packed[4 * g4], packed[4 * g4 + 1], packed[4 * g4 + 2], packed[4 * g4 + 3]);
        } else if (tc < p.n_inner) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (tc + e < p.n_inner) {
              const uint32_t w = packed[e >> 1];
              vrow[chunk * 32 + e] = __ushort_as_half(static_cast<unsigned short>((e & 1) ? (w >> 16) : (w & 0xffffu)));
            }
        }
      }
#endif
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.acc_empty[G_V]);
    }
  }

#if B200_APROJ_TMASTORE
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

extern "C" size_t b200tri_triatt_project_workspace_bytes(void) { return 512 * 128 * 2 + 1024; }

extern "C" int b200tri_triatt_project(const b200tri_triatt_project_args* a, b200tri_stream_t stream_) {
  using namespace b200;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  B200_REQUIRE(a != nullptr, B200TRI_ERR_INVALID, "att project: null args");
  B200_REQUIRE(a->x && a->q && a->k && a->vt && a->bias && a->norm_scale && a->norm_bias && a->w_q && a->w_k &&
                   a->w_v && a->w_bias,
               B200TRI_ERR_INVALID, "att project: null pointer argument");
  B200_REQUIRE(a->n_outer > 0 && a->n_inner > 0, B200TRI_ERR_INVALID, "att project: sizes must be positive");
  B200_REQUIRE(a->heads == 4 && a->head_dim == 32, B200TRI_ERR_UNSUPPORTED,
               "att project: built for 4 heads x 32 (got %d x %d)", a->heads, a->head_dim);
  B200_REQUIRE(a->xs_outer % 8 == 0 && a->xs_inner % 8 == 0 && a->ld % 8 == 0 && a->ld >= a->n_inner,
               B200TRI_ERR_INVALID, "att project: strides/pitch must be multiples of 8 elements, ld >= n_inner");
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) |
                 reinterpret_cast<uintptr_t>(a->vt) | reinterpret_cast<uintptr_t>(a->bias)) & 15) == 0,
               B200TRI_ERR_INVALID, "att project: outputs must be 16-byte aligned");
  B200_REQUIRE(a->workspace && a->workspace_bytes >= b200tri_triatt_project_workspace_bytes(), B200TRI_ERR_WORKSPACE,
               "att project: workspace of %zu bytes needed", b200tri_triatt_project_workspace_bytes());
  int* status = device_status_word();
  B200_REQUIRE(status != nullptr, B200TRI_ERR_CUDA, "att project: no current CUDA device");

  Carver ws(a->workspace);
  __nv_bfloat16* wpk = ws.take<__nv_bfloat16>(512 * 128);
  uint32_t* gamma2 = ws.take<uint32_t>(64, 256);
  uint32_t* beta2 = ws.take<uint32_t>(64, 256);
  pack_transpose(static_cast<const __nv_bfloat16*>(a->w_q), 128, 0, 128, wpk, stream);
  pack_transpose(static_cast<const __nv_bfloat16*>(a->w_k), 128, 0, 128, wpk + 128 * 128, stream);
  pack_transpose(static_cast<const __nv_bfloat16*>(a->w_v), 128, 0, 128, wpk + 256 * 128, stream);
  pack_zero(wpk + 384 * 128, 128 * 128, stream);
  pack_transpose(static_cast<const __nv_bfloat16*>(a->w_bias), 4, 0, 4, wpk + 384 * 128, stream);
  pack_copy_words(a->norm_scale, gamma2, 64, stream);
  pack_copy_words(a->norm_bias, beta2, 64, stream);

  CUtensorMap tm_x, tm_w, tm_q, tm_k, tm_vt;
  {  // q and k [n_outer][n_inner][128], written as tiles of [128 pairs][64 channels]
    const uint64_t dims[3] = {128, (uint64_t)a->n_inner, (uint64_t)a->n_outer};
    const uint64_t str[2] = {256, (uint64_t)a->n_inner * 256};
    const uint32_t box[3] = {64, 128, 1};
    int rc = make_tmap(&tm_q, a->q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B128);
    if (rc) return rc;
    rc = make_tmap(&tm_k, a->k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  {  // vT [n_outer][128][ld] fp16, written as tiles of [128 channels][64 pairs]
    const uint64_t dims[3] = {(uint64_t)a->n_inner, 128, (uint64_t)a->n_outer};
    const uint64_t str[2] = {(uint64_t)a->ld * 2, (uint64_t)a->ld * 2 * 128};
    const uint32_t box[3] = {64, 128, 1};
    int rc = make_tmap(&tm_vt, a->vt, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, dims, str, box, Swz::B128);
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
    const uint64_t dims[2] = {128, 512};
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
  p.gamma2 = gamma2;
  p.beta2 = beta2;
  p.q = static_cast<__nv_bfloat16*>(a->q);
  p.k = static_cast<__nv_bfloat16*>(a->k);
  p.vt = static_cast<__half*>(a->vt);
  p.bias = static_cast<__nv_bfloat16*>(a->bias);
  p.ld = a->ld;
  p.bias_head_stride = a->bias_head_stride;
  p.q_scale = __bfloat162float(__float2bfloat16_rn(sqrtf(static_cast<float>(a->head_dim))));
  p.eps = a->eps;
  p.status = status;

  {
    const int rc = ensure_smem_limit(reinterpret_cast<const void*>(att_project_kernel), (int)sizeof(Smem));
    if (rc) return rc;
  }
  const long long grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
  {
    TimedLaunch timed(K_TRIATT_PROJECT, stream);
    count_launch();
    att_project_kernel<<<static_cast<unsigned>(grid), THREADS, sizeof(Smem), stream>>>(tm_x, tm_w, tm_q, tm_k, tm_vt, p);
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}
