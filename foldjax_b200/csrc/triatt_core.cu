// Triangle attention, core: for every row i, head h and query j
//
//   S[k]  = q[i,j,h,:] . k[i,k,h,:] + mask_bias[i,k] + tri_bias[h,j,k]
//   o     = softmax_k(S) . v[i,k,h,:]
//
// Reference: _attention_block, src/foldjax/models/boltz2/models/triangle/
// triangle_attention.py:428-455 (scores = q k^T + mask_bias + tri_bias in fp32,
// softmax in fp32, P v, cast to the trunk dtype); the fused entry it replaces is
// pallas_attention_core, triangle_attention_pallas.py:180.
//
// Flash-style: scores never leave the SM. One work item = (head h, group of NWG
// consecutive rows i, tile of 128 queries j); each of the NWG softmax warpgroups
// owns one row i, and all of them share the tri_bias tile [128 j x 64 k] of the
// step, so the bias (the only operand that does not depend on i) crosses
// L2 -> shared memory once per NWG rows.
//
//   warp 0        (warps 0-3 form the control warpgroup; warp 3 idle) TMA producer: Q tiles per
//                 item; per 64-key step the bias tile and, per row, K [64x32], V^T [32x64] and
//                 the mask-bias row
//   warp 1        score issuer: S = bias . I + Q K^T into TMEM. The bias tile of the step is a
//                 K-major A operand itself; times a 64 x 64 identity it lands in the accumulator
//                 exactly, so the softmax threads never touch it (bf16, 128x64, 4 + 2 MMAs)
//   warp 2        P.V issuer: O += P V (fp16, 128x48x64) with P read from TMEM
//   warpgroups    softmax: one thread per query row. S from TMEM (+ the mask row where the step
//                 has dropped or soft-masked keys), running max with lazy rescale (the offset is
//                 an integer in log2 units and only moves when the max grew by more than 2^8,
//                 so O stays in TMEM, is rescaled rarely and by exact powers of two), the
//                 exponentials split between the MUFU unit and a cubic on the FMA pipe,
//                 P -> fp16 -> TMEM
// TMEM per warpgroup: S 64 columns, P 32 (fp16 pairs), O 32 + the row sum (column 128 of
// the group; rows 32..47 of every V tile are a row of ones and zero padding, so the
// tensor core accumulates sum_k P next to P.V). Registers are moved from the control warpgroup
// to the softmax warpgroups at start-up (setmaxnreg).
//
// Bound: not the tensor pipe and not HBM. Per score the SM issues about 7 instructions (3-input
// max, packed fma, ex2 or the cubic with its exponent insertion, clamp, half a cvt) against 128
// tensor flops, and the MUFU unit delivers 16 exponentials per clock and SM: the kernel runs
// at about 60 % of its issue slots with the tensor pipe under 40 % busy at head dim 32.
#include <cuda_fp16.h>

#include <mutex>

#include "host.cuh"
#include "tc.cuh"

namespace b200 {

namespace {

#ifndef B200_NWG
#define B200_NWG 3
#endif
#ifndef B200_TURNS
#define B200_TURNS 0
#endif
// 1: the pair bias is added by the tensor core (S = bias . I + Q . K^T); 0: by the softmax threads.
#ifndef B200_BIAS_MMA
#define B200_BIAS_MMA 1
#endif
// Of every 16 pairs of exponentials, this many are evaluated on the FMA pipe.
#ifndef B200_POLY
#define B200_POLY 8
#endif
// 1: registers are moved from the control warpgroup to the softmax warpgroups at start-up.
#ifndef B200_POLY_IMAD
#define B200_POLY_IMAD 0
#endif
#ifndef B200_SETMAXNREG
#define B200_SETMAXNREG 1
#endif
constexpr int NWG = B200_NWG;  // softmax warpgroups = rows i that share one bias tile
constexpr int KT = 64;
constexpr int STAGES = 3;
constexpr int THREADS = 128 + NWG * 128;  // warpgroup 0: producer, MMA issuer, 2 idle warps; then the softmax warpgroups
constexpr int Q_BYTES = 128 * 64;    // [128 j][32 d] bf16
constexpr int BIAS_BYTES = 128 * 128;  // [128 j][64 k] bf16
constexpr int K_BYTES = KT * 64;     // [64 k][32 d] bf16
constexpr int V_ROWS = 48;           // 32 head channels + a row of ones (row 32) + 15 zero rows
constexpr int V_BYTES = V_ROWS * 128;  // [48][64 k] fp16; TMA fills rows 0..31
constexpr int V_TMA_BYTES = 32 * 128;
constexpr uint32_t TM_S = 0, TM_P = 64, TM_O = 96, TM_L = 128, TM_WG = 160;  // O: 32 columns + the row sum in column 128
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units: P stays below 2^8.5
constexpr float LN2 = 0.6931471805599453f;
constexpr float EXP_MAGIC = 12582912.0f;  // 1.5 * 2^23: adding it leaves round(x) in the low mantissa bits
// A dropped key's score. The reference adds -1e9 in fp32, which absorbs q.k + bias
// (|q.k + bias| < 32 is below half an ulp of 1e9): every dropped key ends up with
// the same score, so a row with no valid key becomes a uniform average. Here a
// mask bias at or below MASKED_SCORE REPLACES the score with that constant, which
// has the same two effects (zero weight beside any valid key, uniform without one)
// while keeping the softmax offset small enough for a single fp32 fma per
// exponent. Smaller mask biases (soft masks) are added as they are.
constexpr float MASKED_SCORE = -30000.0f;

struct Smem {
  uint8_t q[NWG][Q_BYTES];
  uint8_t bias[STAGES][BIAS_BYTES];
#if B200_BIAS_MMA
  uint8_t ident[KT * 128];  // 64 x 64 bf16 identity, K-major rows of 128 B under the 128-byte swizzle
#endif
  uint8_t k[STAGES][NWG][K_BYTES];
  uint8_t v[STAGES][NWG][V_BYTES];
  float mb[STAGES][NWG][KT];
  uint64_t q_full, q_empty, st_full[STAGES], st_empty[STAGES], s_full[NWG], s_free[NWG], p_full[NWG], pv_done[NWG];
  uint64_t turn[NWG][4];  // whose exponentials run on each scheduler's MUFU unit
  uint32_t tmem_base;
};
static_assert(sizeof(Smem) <= 232448, "shared memory budget");
constexpr uint32_t STAGE_TX = BIAS_BYTES + NWG * (K_BYTES + V_TMA_BYTES + KT * 4);

// One launch can walk several key tiles (ring attention: the tiles of the peers, each in
// its own buffers): per tile one tensor map for K, V^T, the pair bias and the mask-bias rows.
constexpr int MAX_KEY_TILES = 7;
struct TileMaps {
  CUtensorMap k[MAX_KEY_TILES], v[MAX_KEY_TILES], b[MAX_KEY_TILES], m[MAX_KEY_TILES];
};

struct Params {
  int n_i, n_j, n_k;  // rows, queries, keys per key tile
  int steps_per_tile;
  int heads;
  int groups, tiles_j, steps;
  long long total_items;
  __nv_bfloat16* o;  // [n_i][n_j][128]
  float* row_max;    // optional [n_i][heads][n_j]: offset m used (natural log units)
  float* row_sum;    // optional: sum of exp(S - m)
  float* acc_o;      // fp32 running numerator [n_i][n_j][128] (ring attention)
  int normalize;     // 1: write o = O / l; 0: leave the running state in acc_o/row_max/row_sum
  int resume;        // 1: start from the running state instead of from nothing
  int* status;
};

__device__ __forceinline__ uint64_t desc_sw64(uint32_t saddr) { return umma_desc_kmajor(saddr, 64); }
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) { return umma_desc_kmajor(saddr, 128); }

__host__ __device__ constexpr uint32_t idesc_f16(int M, int N) {
  return (1u << 4) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// 2^(u * log2e - m2) for a pair of scores on the FMA pipe instead of the MUFU unit, m2 an
// integer: y = u * log2e + (magic - m2) holds n = round(t) in its low mantissa bits,
// f = u * log2e - m2 - n is formed with one more fma (|f| <= 0.5), a cubic gives 2^f to
// 2e-4 relative (below the fp16 rounding P gets anyway) and n is added to the exponent
// field. `u` must have been clamped so that t >= -125 (the caller does it): the exponent
// arithmetic has no underflow handling.
__device__ __forceinline__ float2 poly_exp2x2(float2 u, float2 log2e2, float2 magic_minus_m2) {
  const float2 y = __ffma2_rn(u, log2e2, magic_minus_m2);
  const float2 d = __ffma2_rn(y, make_float2(-1.0f, -1.0f), magic_minus_m2);  // -(m2 + n), exact
  const float2 f = __ffma2_rn(u, log2e2, d);
  float2 q = __ffma2_rn(make_float2(0.05286743f, 0.05286743f), f, make_float2(0.24215189f, 0.24215189f));
  q = __ffma2_rn(q, f, make_float2(0.69358677f, 0.69358677f));
  q = __ffma2_rn(q, f, make_float2(0.99996275f, 0.99996275f));
#if B200_POLY_IMAD
  // bits(q) + (bits(y) << 23) as one integer multiply-add per value (FMA pipe) instead of a
  // shift and an add on the ALU pipe, which the maxima and clamps already load.
  int rx, ry;
  asm("mad.lo.s32 %0, %1, 8388608, %2;" : "=r"(rx) : "r"(__float_as_int(y.x)), "r"(__float_as_int(q.x)));
  asm("mad.lo.s32 %0, %1, 8388608, %2;" : "=r"(ry) : "r"(__float_as_int(y.y)), "r"(__float_as_int(q.y)));
  return make_float2(__int_as_float(rx), __int_as_float(ry));
#else
  return make_float2(__int_as_float(__float_as_int(q.x) + (__float_as_int(y.x) << 23)),
                     __int_as_float(__float_as_int(q.y) + (__float_as_int(y.y) << 23)));
#endif
}

__global__ void __launch_bounds__(THREADS, 1)
att_core_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ TileMaps tm, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, ST_OK, 900);
    return;
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm.k[0]);
    tma_prefetch_desc(&tm.v[0]);
    tma_prefetch_desc(&tm.b[0]);
    tma_prefetch_desc(&tm.m[0]);
    mbar_init(&sm.q_full, 1);
    mbar_init(&sm.q_empty, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.st_full[s], 1);
      mbar_init(&sm.st_empty[s], 1 + NWG * 4);
    }
    for (int g = 0; g < NWG; ++g) {
      mbar_init(&sm.s_full[g], 1);
      mbar_init(&sm.s_free[g], 128);
      mbar_init(&sm.p_full[g], 128);
      mbar_init(&sm.pv_done[g], 1);
      for (int qr = 0; qr < 4; ++qr) mbar_init(&sm.turn[g][qr], 1);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  // Rows 32..47 of every V tile are constant and never touched by TMA: row 32 is
  // all ones, so column 32 of O accumulates the softmax row sum on the tensor core
  // (from the very P that multiplies V); rows 33..47 are zero padding to N = 48.
  for (int idx = threadIdx.x; idx < STAGES * NWG * (16 * 128 / 4); idx += blockDim.x) {
    const int tile = idx / (16 * 32), w = idx % (16 * 32);
    uint32_t* dst = reinterpret_cast<uint32_t*>(&sm.v[0][0][0] + tile * V_BYTES + V_TMA_BYTES);
    dst[w] = (w < 32) ? 0x3C003C00u : 0u;  // fp16 1.0 pairs in row 32
  }
#if B200_BIAS_MMA
  // The bias tile of a step is itself a K-major A operand ([128 queries][64 keys]); multiplied
  // by this identity it lands in the score accumulator exactly (bf16 x 1.0 in fp32), so the
  // softmax threads never touch the bias.
  for (int idx = threadIdx.x; idx < KT * 128 / 4; idx += blockDim.x) {
    const int row = idx / 32, w = idx % 32;          // 32-bit word w of the row = elements 2w, 2w+1
    const int chunk = (w >> 2) ^ (row & 7);          // undo the swizzle: logical 16-byte chunk
    const int e0 = chunk * 8 + (w & 3) * 2;          // logical element index of the low half
    uint32_t val = 0u;
    if (e0 == row) val = 0x00003F80u;                // bf16 1.0 in the low half
    if (e0 + 1 == row) val = 0x3F800000u;
    reinterpret_cast<uint32_t*>(sm.ident)[idx] = val;
  }
#endif
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;
  const int items_per_head = p.groups * p.tiles_j;

#if B200_SETMAXNREG
  // The control warpgroup needs few registers; the softmax warpgroups hold 64 scores per
  // thread and want more than the 128 an even split of the register file gives them.
#endif

  if (warp < 4) {
#if B200_SETMAXNREG
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
#endif
  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0, item_it = 0;
      bool alive = true;
      for (long long item = blockIdx.x; item < p.total_items && alive; item += gridDim.x, ++item_it) {
        const int h = static_cast<int>(item / items_per_head);
        const int rem = static_cast<int>(item % items_per_head);
        const int i0 = (rem / p.tiles_j) * NWG;
        const int j0 = (rem % p.tiles_j) * 128;
        if (!mbar_wait(&sm.q_empty, (item_it & 1) ^ 1, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&sm.q_full, NWG * Q_BYTES);
        for (int g = 0; g < NWG; ++g) tma_load_3d(sm.q[g], &tm_q, &sm.q_full, h * 32, j0, i0 + g);
        for (int t = 0; t < p.steps; ++t) {
          if (!mbar_wait(&sm.st_empty[stage], phase ^ 1, p.status, ST_TIMEOUT_PRODUCER)) {
            alive = false;
            break;
          }
          const int tile = t / p.steps_per_tile;
          const int k0 = (t - tile * p.steps_per_tile) * KT;
          mbar_expect_tx(&sm.st_full[stage], STAGE_TX);
          tma_load_3d(sm.bias[stage], &tm.b[tile], &sm.st_full[stage], k0, j0, h);
          for (int g = 0; g < NWG; ++g) {
            tma_load_3d(sm.k[stage][g], &tm.k[tile], &sm.st_full[stage], h * 32, k0, i0 + g);
            tma_load_3d(sm.v[stage][g], &tm.v[tile], &sm.st_full[stage], k0, h * 32, i0 + g);
            tma_load_2d(sm.mb[stage][g], &tm.m[tile], &sm.st_full[stage], k0, i0 + g);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- Q.K^T issuer: S[wg] = Q[wg] . K[stage][wg]^T as soon as the warpgroup has
    // taken the previous scores out of TMEM. Kept apart from the P.V issuer so that
    // neither product waits behind the other's barrier; both are single threads
    // competing with four softmax warps for issue slots on their sub-partition.
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, KT);
      int stage = 0;
      uint32_t phase = 0, item_it = 0, g = 0;  // g: global step counter
      bool alive = true;
      for (long long item = blockIdx.x; item < p.total_items && alive; item += gridDim.x, ++item_it) {
        if (!mbar_wait(&sm.q_full, item_it & 1, p.status, ST_TIMEOUT_MMA)) break;
        for (int t = 0; t < p.steps && alive; ++t, ++g) {
          if (!mbar_wait(&sm.st_full[stage], phase, p.status, ST_TIMEOUT_MMA)) {
            alive = false;
            break;
          }
          for (int wg = 0; wg < NWG; ++wg) {
            if (!mbar_wait(&sm.s_free[wg], (g & 1) ^ 1, p.status, ST_TIMEOUT_MMA)) {
              alive = false;
              break;
            }
            tc_fence_after();
            const uint64_t adesc = desc_sw64(smem_u32(sm.q[wg]));
            const uint64_t bdesc = desc_sw64(smem_u32(sm.k[stage][wg]));
            const uint32_t d = tmem_base + wg * TM_WG + TM_S;
#if B200_BIAS_MMA
            const uint64_t biasdesc = desc_sw128(smem_u32(sm.bias[stage]));
            const uint64_t identdesc = desc_sw128(smem_u32(sm.ident));
#pragma unroll
            for (int kk = 0; kk < KT / 16; ++kk)
              umma_bf16_ss(d, umma_desc_advance(biasdesc, kk * 32), umma_desc_advance(identdesc, kk * 32), idesc_qk,
                           kk != 0);
            umma_bf16_ss(d, adesc, bdesc, idesc_qk, 1);
#else
            umma_bf16_ss(d, adesc, bdesc, idesc_qk, 0);
#endif
            umma_bf16_ss(d, umma_desc_advance(adesc, 32), umma_desc_advance(bdesc, 32), idesc_qk, 1);
            umma_commit(&sm.s_full[wg]);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (alive) umma_commit(&sm.q_empty);  // every Q.K^T of the item has been issued
      }
    }
  } else if (warp == 2) {
    // ---- P.V issuer: O[wg] (+)= P[wg] . V[stage][wg], P read from TMEM.
    if (elect_one()) {
      constexpr uint32_t idesc_pv = idesc_f16(128, V_ROWS);
      int stage = 0;
      uint32_t phase = 0, g = 0;
      bool alive = true;
      for (long long item = blockIdx.x; item < p.total_items && alive; item += gridDim.x) {
        for (int t = 0; t < p.steps && alive; ++t, ++g) {
          // (already complete when P arrives; observed here so this thread's products
          // are ordered after the TMA writes of V)
          if (!mbar_wait(&sm.st_full[stage], phase, p.status, ST_TIMEOUT_MMA)) break;
          for (int wg = 0; wg < NWG; ++wg) {
            if (!mbar_wait(&sm.p_full[wg], g & 1, p.status, ST_TIMEOUT_MMA)) {
              alive = false;
              break;
            }
            tc_fence_after();
            const uint64_t vdesc = desc_sw128(smem_u32(sm.v[stage][wg]));
            const uint32_t d = tmem_base + wg * TM_WG + TM_O;
            const uint32_t a = tmem_base + wg * TM_WG + TM_P;
#pragma unroll
            for (int k = 0; k < KT / 16; ++k)
              umma_bf16_ts(d, a + k * 8, umma_desc_advance(vdesc, k * 32), idesc_pv, (t | k | p.resume) != 0);
            umma_commit(&sm.pv_done[wg]);
          }
          if (!alive) break;
          // K of this stage was consumed before the softmax saw its scores, V by the
          // products just issued: the stage is free once they complete.
          umma_commit(&sm.st_empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  }
  } else {
    // ------------------------------------------------------------- softmax
#if B200_SETMAXNREG
    asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
#endif
    const int wg = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // query inside the tile = TMEM lane
    const uint32_t t_wg = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + wg * TM_WG;
    int stage = 0;
    uint32_t phase = 0, g = 0;
    bool alive = true;
    for (long long item = blockIdx.x; item < p.total_items && alive; item += gridDim.x) {
      const int h = static_cast<int>(item / items_per_head);
      const int rem = static_cast<int>(item % items_per_head);
      const int i = (rem / p.tiles_j) * NWG + wg;
      const int j = (rem % p.tiles_j) * 128 + row;
      // The softmax offset, kept in log2 units and integer-valued: exp(s - m) is evaluated as
      // 2^(s * log2e - m2). An integer m2 lets the polynomial path fold it into its range
      // reduction exactly and makes every rescale factor an exact power of two.
      float m2_used = -INFINITY;
      const bool in_range = i < p.n_i && j < p.n_j;
      const long long si = (static_cast<long long>(i) * p.heads + h) * p.n_j + j;
      const long long oi = (static_cast<long long>(i) * p.n_j + j) * 128 + h * 32;
      if (p.resume) {
        // Continue the softmax of earlier key tiles: offset, denominator and fp32
        // numerator go back where the loop keeps them (registers and TMEM). The
        // previous item's O has been read out by this thread already, and the
        // first P.V of this item waits for this thread's P, so TMEM is free.
        uint32_t o[32], lcol[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) lcol[e] = 0u;
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = 0u;
        if (in_range) {
          m2_used = rintf(p.row_max[si] * LOG2E);
          lcol[0] = __float_as_uint(p.row_sum[si]);
          const float4* src = reinterpret_cast<const float4*>(p.acc_o + oi);
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4) {
            const float4 f = src[q4];
            o[4 * q4 + 0] = __float_as_uint(f.x);
            o[4 * q4 + 1] = __float_as_uint(f.y);
            o[4 * q4 + 2] = __float_as_uint(f.z);
            o[4 * q4 + 3] = __float_as_uint(f.w);
          }
        }
        tmem_st32(t_wg + TM_O, o);
        tmem_st16(t_wg + TM_L, lcol);
        tmem_st_wait();
        tc_fence_before();
      }
      for (int t = 0; t < p.steps; ++t, ++g) {
        if (!mbar_wait(&sm.st_full[stage], phase, p.status, ST_TIMEOUT_SOFTMAX) ||
            !mbar_wait(&sm.s_full[wg], g & 1, p.status, ST_TIMEOUT_SOFTMAX)) {
          alive = false;
          break;
        }
        tc_fence_after();
        // (fetched here, long before the vote that needs them)
        const float mk0 = sm.mb[stage][wg][lane], mk1 = sm.mb[stage][wg][lane + 32];
        // Scores, bias and mask travel as fp32 pairs: sm_100 adds/multiplies two
        // fp32 values per instruction (add/fma .f32x2), halving the softmax's ALU work.
        float2 u[KT / 2];
        {
#if B200_BIAS_MMA
          // q.k + bias arrives from the tensor core; both halves are requested at once.
          uint32_t r0[32], r1[32];
          tmem_ld32(t_wg + TM_S, r0);
          tmem_ld32(t_wg + TM_S + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            u[e] = make_float2(__uint_as_float(r0[2 * e]), __uint_as_float(r0[2 * e + 1]));
            u[16 + e] = make_float2(__uint_as_float(r1[2 * e]), __uint_as_float(r1[2 * e + 1]));
          }
#else
          // Two halves of 32 keys: the TMEM load of the second half and the bias
          // fetches overlap the adds of the first, and at most one raw half is live.
          const uint8_t* brow = sm.bias[stage];
          uint32_t r[32];
          uint4 b4[4];
          tmem_ld32(t_wg + TM_S, r);
#pragma unroll
          for (int c = 0; c < 4; ++c) b4[c] = *reinterpret_cast<const uint4*>(brow + sw128_offset(row, c));
          tmem_ld_wait();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint32_t w[4] = {b4[c].x, b4[c].y, b4[c].z, b4[c].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int q = 4 * c + e;  // pair inside this half: keys 32*half + 2q, +1
                u[16 * half + q] = __fadd2_rn(make_float2(__uint_as_float(r[2 * q]), __uint_as_float(r[2 * q + 1])),
                                              make_float2(bf16_lo(w[e]), bf16_hi(w[e])));
              }
            }
            if (half == 0) {
              tmem_ld32(t_wg + TM_S + 32, r);
#pragma unroll
              for (int c = 0; c < 4; ++c) b4[c] = *reinterpret_cast<const uint4*>(brow + sw128_offset(row, 4 + c));
              tmem_ld_wait();
            }
          }
#endif
          tc_fence_before();
          mbar_arrive(&sm.s_free[wg]);
        }
        const float* mrow = sm.mb[stage][wg];
        const bool masked = __any_sync(0xffffffffu, (mk0 != 0.f) || (mk1 != 0.f));
        if (masked) {
#pragma unroll
          for (int c = 0; c < KT / 4; ++c) {
            const float4 m4 = *reinterpret_cast<const float4*>(mrow + 4 * c);
            const float mv[4] = {m4.x, m4.y, m4.z, m4.w};
            float uu[4] = {u[2 * c].x, u[2 * c].y, u[2 * c + 1].x, u[2 * c + 1].y};
#pragma unroll
            for (int e = 0; e < 4; ++e) uu[e] = (mv[e] <= MASKED_SCORE) ? mv[e] : uu[e] + mv[e];
            u[2 * c] = make_float2(uu[0], uu[1]);
            u[2 * c + 1] = make_float2(uu[2], uu[3]);
            if ((c & 3) == 3) asm volatile("" ::: "memory");  // keep the loads from piling up in registers
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.st_empty[stage]);
        // P buffer free and O stable once the previous step's P.V has completed (it
        // was issued before this step's Q.K^T, so this wait does not stall).
        if (!mbar_wait(&sm.pv_done[wg], (g & 1) ^ 1, p.status, ST_TIMEOUT_SOFTMAX)) {
          alive = false;
          break;
        }
        tc_fence_after();
#if B200_TURNS
        // The exponentials of one warp keep a scheduler's MUFU unit busy by themselves,
        // while the rest of a step (loads, adds, maxima) needs issue slots but no MUFU.
        // Left alone, the three warps of a scheduler drift into the same phase and the
        // two resources are used one after the other. So the exponent phase is taken in
        // turns: warpgroup w runs it after warpgroup w - 1 (warpgroup 0 after the last
        // one's previous step), and the others' load/add/max work fills the issue slots.
        if (!mbar_wait(&sm.turn[wg][quarter], wg == 0 ? ((g & 1) ^ 1) : (g & 1), p.status, ST_TIMEOUT_SOFTMAX)) {
          alive = false;
          break;
        }
#endif
        // four independent chains, so the reduction is not one 32-deep dependency
        float mxa = fmaxf(u[0].x, u[0].y), mxb = fmaxf(u[1].x, u[1].y);
        float mxc = fmaxf(u[2].x, u[2].y), mxd = fmaxf(u[3].x, u[3].y);
#pragma unroll
        for (int e = 4; e < KT / 2; e += 4) {
          mxa = fmax3(mxa, u[e].x, u[e].y);
          mxb = fmax3(mxb, u[e + 1].x, u[e + 1].y);
          mxc = fmax3(mxc, u[e + 2].x, u[e + 2].y);
          mxd = fmax3(mxd, u[e + 3].x, u[e + 3].y);
        }
        const float mx2 = fmaxf(fmaxf(mxa, mxb), fmaxf(mxc, mxd)) * LOG2E;  // this step's maximum, log2 units
        // Lazy rescale: the offset only moves when this step's maximum exceeds it by more than
        // 2^8 (then it exceeds every earlier maximum too, which stayed within the threshold).
        const bool need = (mx2 - m2_used) > RESCALE_THRESHOLD;  // true on the first step (m2_used = -inf)
        float alpha = 1.f;
        if (need) {
          const float m2_new = rintf(mx2);
          alpha = fast_exp2(m2_used - m2_new);  // an exact power of two; 0 on the first step
          m2_used = m2_new;
        }
        const bool any_need = __any_sync(0xffffffffu, need);
        // exp(u - m) = 2^(u * log2e - m2): one fma per pair feeds the MUFU unit (|m2| < 2^17, so
        // the sum is exact to the last bit of the product and cancels exactly for the keys that
        // equal the offset). B200_POLY of every 16 pairs take the polynomial path instead: the
        // MUFU unit delivers 16 results per clock and SM and would otherwise be the one pipe
        // every exponential queues for, while the FMA pipe idles.
        // P goes to TMEM in two halves of 32 keys to keep the live registers down.
        {
          const float2 log2e2 = make_float2(LOG2E, LOG2E);
          const float2 nm2 = make_float2(-m2_used, -m2_used);
          const float2 mm2 = make_float2(EXP_MAGIC - m2_used, EXP_MAGIC - m2_used);
          const float u_min = (m2_used - 120.0f) * LN2;  // keeps the polynomial path's t above about -120
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t packed[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float2 ue = u[16 * half + e];
              float2 ex;
              if (((e + 1) * B200_POLY) / 16 != (e * B200_POLY) / 16) {  // spread evenly over the half
                ex = poly_exp2x2(make_float2(fmaxf(ue.x, u_min), fmaxf(ue.y, u_min)), log2e2, mm2);
              } else {
                const float2 t2 = __ffma2_rn(ue, log2e2, nm2);
                ex = make_float2(fast_exp2(t2.x), fast_exp2(t2.y));
              }
              // fp32 exponentials, rounded once to the fp16 pair the tensor core reads
              // (the packed fp16 ex2 costs more instructions than two fp32 ones here)
              const __half2 h2 = __floats2half2_rn(ex.x, ex.y);
              packed[e] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            tmem_st16(t_wg + TM_P + 16 * half, packed);
          }
        }
#if B200_TURNS
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.turn[(wg + 1) % NWG][quarter]);
#endif
        if ((t > 0 || p.resume) && any_need) {
          uint32_t o[32];
          tmem_ld32(t_wg + TM_O, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(t_wg + TM_O, o);
          uint32_t lcol[16];  // the row-sum column (and its zero padding) scales the same way
          tmem_ld16(t_wg + TM_L, lcol);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) lcol[e] = __float_as_uint(__uint_as_float(lcol[e]) * alpha);
          tmem_st16(t_wg + TM_L, lcol);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&sm.p_full[wg]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!alive) break;
      // ---- item epilogue: O / l -> bf16 -> o[i][j][h*32 ..]
      if (!mbar_wait(&sm.pv_done[wg], (g & 1) ^ 1, p.status, ST_TIMEOUT_SOFTMAX)) break;
      tc_fence_after();
      uint32_t o[32], lcol[16];
      tmem_ld32(t_wg + TM_O, o);
      tmem_ld16(t_wg + TM_L, lcol);
      tmem_ld_wait();
      tc_fence_before();
      const float l = __uint_as_float(lcol[0]);  // sum_k exp(S - m), accumulated by the P.V products
      if (in_range) {
        if (p.normalize) {
          const float inv = __fdividef(1.0f, l);
          uint4* dst = reinterpret_cast<uint4*>(p.o + oi);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              w[e] = pack_bf16x2(__uint_as_float(o[8 * q4 + 2 * e]) * inv, __uint_as_float(o[8 * q4 + 2 * e + 1]) * inv);
            dst[q4] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        } else {
          float4* dst = reinterpret_cast<float4*>(p.acc_o + oi);
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            dst[q4] = make_float4(__uint_as_float(o[4 * q4]), __uint_as_float(o[4 * q4 + 1]),
                                  __uint_as_float(o[4 * q4 + 2]), __uint_as_float(o[4 * q4 + 3]));
        }
        if (p.row_max) {
          p.row_max[si] = m2_used * LN2;  // natural-log units
          p.row_sum[si] = l;
        }
      }
    }
  }

  if (*reinterpret_cast<volatile int*>(p.status) != ST_OK)
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// mask_bias[i][k] = inf * (mask[i,k] - 1) for k < n_k, -infinity for the pitch
// padding (keys that do not exist), built in fp32 like the reference
// (triangle_attention.py:138-142).
__global__ void mask_bias_kernel(const float* __restrict__ mask, long long ms_i, long long ms_k, int n_i, int n_k,
                                 int ld, float inf, int additive, float* __restrict__ out) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(n_i) * ld) return;
  const int i = static_cast<int>(idx / ld), k = static_cast<int>(idx % ld);
  float v = -INFINITY;
  if (k < n_k && mask) {
    const float m = mask[i * ms_i + k * ms_k];
    // fmaxf drops a NaN operand, so a NaN bias would silently become "keep": map it to "drop"
    const float b = additive ? m : inf * (m - 1.0f);
    v = (b == b) ? fmaxf(b, MASKED_SCORE) : MASKED_SCORE;
  } else if (k < n_k) {
    v = 0.0f;
  }
  out[idx] = v;
}

}  // namespace
}  // namespace b200

extern "C" size_t b200tri_triatt_core_workspace_bytes(int32_t n_i, int32_t n_k) {
  if (n_i <= 0 || n_k <= 0) return 0;
  return static_cast<size_t>(n_i) * b200::round_up(n_k, 64) * sizeof(float) + 1024;
}

extern "C" size_t b200tri_triatt_core_multi_workspace_bytes(int32_t n_i, int32_t n_k, int32_t n_tiles) {
  if (n_tiles <= 0) return 0;
  return static_cast<size_t>(n_tiles) * b200tri_triatt_core_workspace_bytes(n_i, n_k);
}

namespace {
// `may_time` = false keeps the launch free of event creation whatever the timing switch
// says at that moment (the allocation-free entry point relies on it).
int core_launch(const b200tri_triatt_core_args* tiles, int n_tiles, b200tri_stream_t stream_, bool may_time);
}  // namespace

extern "C" int b200tri_triatt_core(const b200tri_triatt_core_args* a, b200tri_stream_t stream) {
  return core_launch(a, 1, stream, true);
}

extern "C" int b200tri_triatt_core_multi(const b200tri_triatt_core_args* tiles, int32_t n_tiles,
                                         b200tri_stream_t stream) {
  return core_launch(tiles, n_tiles, stream, true);
}

namespace {
int core_launch(const b200tri_triatt_core_args* tiles, int n_tiles, b200tri_stream_t stream_, bool may_time) {
  using namespace b200;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  B200_REQUIRE(tiles != nullptr, B200TRI_ERR_INVALID, "att core: null args");
  B200_REQUIRE(n_tiles >= 1 && n_tiles <= MAX_KEY_TILES, B200TRI_ERR_INVALID,
               "att core: 1..%d key tiles per launch (got %d)", MAX_KEY_TILES, n_tiles);
  const b200tri_triatt_core_args* a = tiles;  // queries, sizes, outputs and flags come from the first entry
  B200_REQUIRE(a->q && (a->o || a->unnormalized), B200TRI_ERR_INVALID, "att core: null pointer argument");
  B200_REQUIRE(a->n_i > 0 && a->n_j > 0 && a->n_k > 0, B200TRI_ERR_INVALID, "att core: sizes must be positive");
  B200_REQUIRE(a->heads == 4 && a->head_dim == 32, B200TRI_ERR_UNSUPPORTED,
               "att core: built for 4 heads x 32 (got %d x %d)", a->heads, a->head_dim);
  B200_REQUIRE((a->row_max == nullptr) == (a->row_sum == nullptr), B200TRI_ERR_INVALID,
               "att core: row_max and row_sum go together");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a->o) & 15) == 0, B200TRI_ERR_INVALID, "att core: o must be 16-byte aligned");
  B200_REQUIRE(!(a->unnormalized || a->resume) ||
                   (a->acc_o && a->row_max && a->row_sum && (reinterpret_cast<uintptr_t>(a->acc_o) & 15) == 0),
               B200TRI_ERR_INVALID, "att core: resume/unnormalized need acc_o (16-byte aligned), row_max and row_sum");
  B200_REQUIRE(n_tiles == 1 || a->n_k % KT == 0, B200TRI_ERR_INVALID,
               "att core: with several key tiles n_k must be a multiple of %d (got %d)", KT, a->n_k);
  const size_t need_one = b200tri_triatt_core_workspace_bytes(a->n_i, a->n_k);
  B200_REQUIRE(a->workspace && a->workspace_bytes >= need_one * n_tiles, B200TRI_ERR_WORKSPACE,
               "att core: workspace of %zu bytes needed", need_one * n_tiles);
  int* status = device_status_word();
  B200_REQUIRE(status != nullptr, B200TRI_ERR_CUDA, "att core: no current CUDA device");

  const int ldm = round_up(a->n_k, 64);
  TileMaps tm;
  for (int t = 0; t < n_tiles; ++t) {
    const b200tri_triatt_core_args* ti = tiles + t;
    B200_REQUIRE(ti->k && ti->vt && ti->bias, B200TRI_ERR_INVALID, "att core: null k/vt/bias in key tile %d", t);
    B200_REQUIRE(ti->n_k == a->n_k, B200TRI_ERR_INVALID, "att core: key tiles of one launch must have the same n_k");
    B200_REQUIRE(ti->v_ld % 8 == 0 && ti->bias_ld % 8 == 0 && ti->bias_head_stride % 8 == 0 && ti->v_ld >= a->n_k &&
                     ti->bias_ld >= a->n_k,
                 B200TRI_ERR_INVALID, "att core: pitches must be multiples of 8 elements and cover n_k");
    float* mb = reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) + need_one * t);
    {
      const long long total = static_cast<long long>(a->n_i) * ldm;
      count_launch();
      mask_bias_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
          ti->mask, ti->ms_i, ti->ms_k, a->n_i, a->n_k, ldm, ti->inf, ti->mask_additive ? 1 : 0, mb);
      B200_CUDA_OK(cudaGetLastError());
    }
    {
      const uint64_t dims[3] = {128, (uint64_t)a->n_k, (uint64_t)a->n_i};
      const uint64_t str[2] = {256, (uint64_t)a->n_k * 256};
      const uint32_t box[3] = {32, KT, 1};
      int rc = make_tmap(&tm.k[t], ti->k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B64);
      if (rc) return rc;
    }
    {
      const uint64_t dims[3] = {(uint64_t)a->n_k, 128, (uint64_t)a->n_i};
      const uint64_t str[2] = {(uint64_t)ti->v_ld * 2, (uint64_t)ti->v_ld * 2 * 128};
      const uint32_t box[3] = {KT, 32, 1};
      int rc = make_tmap(&tm.v[t], ti->vt, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, dims, str, box, Swz::B128);
      if (rc) return rc;
    }
    {
      const uint64_t dims[3] = {(uint64_t)a->n_k, (uint64_t)a->n_j, 4};
      const uint64_t str[2] = {(uint64_t)ti->bias_ld * 2, (uint64_t)ti->bias_head_stride * 2};
      const uint32_t box[3] = {KT, 128, 1};
      int rc = make_tmap(&tm.b[t], ti->bias, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B128);
      if (rc) return rc;
    }
    {
      const uint64_t dims[2] = {(uint64_t)ldm, (uint64_t)a->n_i};
      const uint64_t str[1] = {(uint64_t)ldm * 4};
      const uint32_t box[2] = {KT, 1};
      int rc = make_tmap(&tm.m[t], mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dims, str, box, Swz::None);
      if (rc) return rc;
    }
  }
  for (int t = n_tiles; t < MAX_KEY_TILES; ++t) {  // unused slots: valid descriptors, never read
    tm.k[t] = tm.k[0];
    tm.v[t] = tm.v[0];
    tm.b[t] = tm.b[0];
    tm.m[t] = tm.m[0];
  }
  CUtensorMap tm_q;
  {
    const uint64_t dims[3] = {128, (uint64_t)a->n_j, (uint64_t)a->n_i};
    const uint64_t str[2] = {256, (uint64_t)a->n_j * 256};
    const uint32_t box[3] = {32, 128, 1};
    int rc = make_tmap(&tm_q, a->q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, str, box, Swz::B64);
    if (rc) return rc;
  }
  Params p;
  p.n_i = a->n_i;
  p.n_j = a->n_j;
  p.n_k = a->n_k;
  p.heads = a->heads;
  p.groups = (a->n_i + NWG - 1) / NWG;
  p.tiles_j = (a->n_j + 127) / 128;
  p.steps_per_tile = (a->n_k + KT - 1) / KT;
  p.steps = p.steps_per_tile * n_tiles;
  p.total_items = static_cast<long long>(a->heads) * p.groups * p.tiles_j;
  p.o = static_cast<__nv_bfloat16*>(a->o);
  p.row_max = a->row_max;
  p.row_sum = a->row_sum;
  p.acc_o = a->acc_o;
  p.normalize = a->unnormalized ? 0 : 1;
  p.resume = a->resume ? 1 : 0;
  p.status = status;

  {
    const int rc = ensure_smem_limit(reinterpret_cast<const void*>(att_core_kernel), (int)sizeof(Smem));
    if (rc) return rc;
  }
  const long long grid = p.total_items < sm_count() ? p.total_items : sm_count();
  {
    TimedLaunch timed(K_TRIATT_CORE, stream, may_time);
    count_launch();
    att_core_kernel<<<static_cast<unsigned>(grid), THREADS, sizeof(Smem), stream>>>(tm_q, tm, p);
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}
}  // namespace

// ---------------------------------------------------------------------------
// Variant for callers that cannot provide scratch memory and must not allocate:
// the mask-bias rows live in a fixed array inside the library instead of the
// caller's workspace. Same kernel, same results as b200tri_triatt_core.
namespace {

// Host code may only use this name to ask the runtime for the device address
// (cudaGetSymbolAddress); it is not itself a device pointer.
// (+256 floats: the workspace carve-up of b200tri_triatt_core rounds its size up by 1 KiB)
static __device__ __align__(256) float g_core_static_scratch[B200TRI_TRIATT_CORE_STATIC_MAX_FLOATS + 256];

// Device address of the array on the current device, looked up once per device.
int core_static_scratch(float** out) {
  constexpr int kMaxDev = 64;
  static float* cache[kMaxDev] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  B200_CUDA_OK(cudaGetDevice(&dev));
  B200_REQUIRE(dev >= 0 && dev < kMaxDev, B200TRI_ERR_CUDA, "att core static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    float* ptr = nullptr;
    B200_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_core_static_scratch));
    B200_REQUIRE(ptr != nullptr, B200TRI_ERR_CUDA, "att core static: no device address for the scratch array");
    cache[dev] = ptr;
  }
  *out = cache[dev];
  return B200TRI_OK;
}

}  // namespace

extern "C" int b200tri_triatt_core_static(const b200tri_triatt_core_args* a, b200tri_stream_t stream) {
  using namespace b200;
  B200_REQUIRE(a != nullptr, B200TRI_ERR_INVALID, "att core static: null args");
  B200_REQUIRE(a->n_i > 0 && a->n_k > 0, B200TRI_ERR_INVALID, "att core static: sizes must be positive");
  const long long floats = static_cast<long long>(a->n_i) * round_up(a->n_k, 64);
  B200_REQUIRE(floats <= B200TRI_TRIATT_CORE_STATIC_MAX_FLOATS, B200TRI_ERR_UNSUPPORTED,
               "att core static: n_i * round_up(n_k, 64) = %lld floats exceeds the built-in scratch of %d floats; "
               "use b200tri_triatt_core with a workspace",
               floats, B200TRI_TRIATT_CORE_STATIC_MAX_FLOATS);
  B200_REQUIRE(!timing_enabled(), B200TRI_ERR_INVALID,
               "att core static: kernel timing is enabled (it creates CUDA events); disable it for this entry point");
  float* scratch = nullptr;
  int rc = core_static_scratch(&scratch);
  if (rc) return rc;
  b200tri_triatt_core_args local = *a;
  local.workspace = scratch;
  local.workspace_bytes = sizeof(float) * static_cast<size_t>(B200TRI_TRIATT_CORE_STATIC_MAX_FLOATS + 256);
  return core_launch(&local, 1, stream, false);
}
