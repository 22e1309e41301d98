// Triangle multiplicative update, contraction stage.
//
//   t[d][i][j] = sum_{s,k} a[s][d][i][k] * b[s][d][j][k]        d = 0..127
//
// 128 independent N x N x N matrix products with both operands K-major, the
// shape tcgen05.mma consumes directly. Persistent kernel, one CTA per SM:
//   warp 0      TMA producer   (A 128x64 and B 256x64 bf16 tiles, 4-stage ring)
//   warp 1      MMA issuer     (128x256x16 tcgen05.mma, fp32 accumulators in
//                               TMEM, two accumulators so the epilogue of one
//                               tile overlaps the main loop of the next)
//   warps 2..5  epilogue       (TMEM -> registers -> bf16/fp32 -> global)
// Tiles are walked channel by channel so the A_d/B_d panels of the channel in
// flight (2 * N*N*2 bytes) stay in L2 while all SMs work on them.
//
// Bound: tensor pipe. Algorithmic work 2*128*n_i*n_j*n_k*n_src flop.
#include "host.cuh"
#include "tc.cuh"

namespace b200 {

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // + slack for 1 KiB alignment
constexpr int THREADS = 192;

struct ContractParams {
  int n_i, n_j, n_src;
  int kb_per_src;  // ceil(n_k / BK)
  int tiles_m, tiles_n;
  long long total_tiles;
  const float* acc_in;
  float* out_f32;
  __nv_bfloat16* out_bf16;
  long long out_ld, out_chan_stride;
  int a_rpb, b_rpb, out_rpb;  // rows per block of the row-blocked layouts
  long long out_block_stride;
  int* status;
};

__global__ void __launch_bounds__(THREADS, 1)
contract_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                const ContractParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  const int k_iters = p.n_src * p.kb_per_src;
  const long long tiles_per_chan = static_cast<long long>(p.tiles_m) * p.tiles_n;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (long long tile = blockIdx.x; tile < p.total_tiles && alive; tile += gridDim.x) {
        const int d = static_cast<int>(tile / tiles_per_chan);
        const int rem = static_cast<int>(tile % tiles_per_chan);
        const int mi = rem / p.tiles_n, nj = rem % p.tiles_n;
        for (int s = 0; s < p.n_src && alive; ++s) {
          for (int kb = 0; kb < p.kb_per_src; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_PRODUCER)) {
              alive = false;
              break;
            }
            uint8_t* sa = smem + stage * STAGE_BYTES;
            mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
            // rows are (block, row in block): a tile starts at block row0 / rpb
            tma_load_5d(sa, &tm_a, &full_bar[stage], kb * BK, (mi * BM) % p.a_rpb, (mi * BM) / p.a_rpb, d, s);
            tma_load_5d(sa + A_BYTES, &tm_b, &full_bar[stage], kb * BK, (nj * BN) % p.b_rpb, (nj * BN) / p.b_rpb, d, s);
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;
      bool alive = true;
      for (long long tile = blockIdx.x; tile < p.total_tiles && alive; tile += gridDim.x, ++it) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int ki = 0; ki < k_iters; ++ki) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_MMA)) {
            alive = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t adesc = umma_desc_kmajor(sa, 128);
          const uint64_t bdesc = umma_desc_kmajor(sa + A_BYTES, 128);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16_ss(d_tmem, umma_desc_advance(adesc, k * 32), umma_desc_advance(bdesc, k * 32), idesc,
                         (ki | k) != 0);
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (alive) umma_commit(&acc_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t it = 0;
    for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
      const int d = static_cast<int>(tile / tiles_per_chan);
      const int rem = static_cast<int>(tile % tiles_per_chan);
      const int mi = rem / p.tiles_n, nj = rem % p.tiles_n;
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase, p.status, ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const int row = mi * BM + quarter * 32 + lane;
      const long long row_off = static_cast<long long>(row / p.out_rpb) * p.out_block_stride +
                                static_cast<long long>(d) * p.out_chan_stride +
                                static_cast<long long>(row % p.out_rpb) * p.out_ld;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int chunk = 0; chunk < BN / 32; ++chunk) {
        uint32_t r[32];
        tmem_ld32(taddr + chunk * 32, r);
        tmem_ld_wait();
        const int col0 = nj * BN + chunk * 32;
        if (row < p.n_i && col0 < p.n_j) {
          const long long off = row_off + col0;
          const bool full = (col0 + 32 <= p.n_j);
          if (p.acc_in) {
            if (full) {
              const float4* src = reinterpret_cast<const float4*>(p.acc_in + off);
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 v = src[q];
                r[4 * q + 0] = __float_as_uint(__uint_as_float(r[4 * q + 0]) + v.x);
                r[4 * q + 1] = __float_as_uint(__uint_as_float(r[4 * q + 1]) + v.y);
                r[4 * q + 2] = __float_as_uint(__uint_as_float(r[4 * q + 2]) + v.z);
                r[4 * q + 3] = __float_as_uint(__uint_as_float(r[4 * q + 3]) + v.w);
              }
            } else {
#pragma unroll
              for (int q = 0; q < 32; ++q)
                if (col0 + q < p.n_j) r[q] = __float_as_uint(__uint_as_float(r[q]) + p.acc_in[off + q]);
            }
          }
          if (p.out_f32) {
            if (full) {
              float4* dst = reinterpret_cast<float4*>(p.out_f32 + off);
#pragma unroll
              for (int q = 0; q < 8; ++q)
                dst[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                     __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
            } else {
#pragma unroll
              for (int q = 0; q < 32; ++q)
                if (col0 + q < p.n_j) p.out_f32[off + q] = __uint_as_float(r[q]);
            }
          }
          if (p.out_bf16) {
            if (full) {
              uint4* dst = reinterpret_cast<uint4*>(p.out_bf16 + off);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[8 * q + 0]), __uint_as_float(r[8 * q + 1]));
                v.y = pack_bf16x2(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3]));
                v.z = pack_bf16x2(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
                v.w = pack_bf16x2(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
                dst[q] = v;
              }
            } else {
#pragma unroll
              for (int q = 0; q < 32; ++q)
                if (col0 + q < p.n_j) p.out_bf16[off + q] = __float2bfloat16_rn(__uint_as_float(r[q]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
  }

  // Tear-down. After a timeout give in-flight bulk copies time to land first.
  if (*reinterpret_cast<volatile int*>(p.status) != ST_OK)
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

}  // namespace b200

extern "C" int b200tri_trimul_contract(const b200tri_trimul_contract_args* a, b200tri_stream_t stream) {
  using namespace b200;
  B200_REQUIRE(a != nullptr, B200TRI_ERR_INVALID, "contract: null args");
  B200_REQUIRE(a->a && a->b, B200TRI_ERR_INVALID, "contract: null operand");
  B200_REQUIRE(a->out_f32 || a->out_bf16, B200TRI_ERR_INVALID, "contract: no output buffer");
  B200_REQUIRE(a->n_i > 0 && a->n_j > 0 && a->n_k > 0 && a->n_src > 0, B200TRI_ERR_INVALID,
               "contract: sizes must be positive (n_i=%d n_j=%d n_k=%d n_src=%d)", a->n_i, a->n_j, a->n_k, a->n_src);
  B200_REQUIRE(a->a_ld % 8 == 0 && a->b_ld % 8 == 0 && a->out_ld % 8 == 0 && a->a_chan_stride % 8 == 0 &&
                   a->b_chan_stride % 8 == 0 && a->a_src_stride % 8 == 0 && a->b_src_stride % 8 == 0 &&
                   a->out_chan_stride % 8 == 0,
               B200TRI_ERR_INVALID, "contract: pitches and strides must be multiples of 8 elements");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a->out_bf16) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->out_f32) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(a->acc_in) & 15) == 0,
               B200TRI_ERR_INVALID, "contract: output pointers must be 16-byte aligned");
  int* status = device_status_word();
  B200_REQUIRE(status != nullptr, B200TRI_ERR_CUDA, "contract: no current CUDA device");

  // Row-blocked operands: rows_per_block 0 (or >= the row count) means one block.
  // A blocked operand needs blocks that tile the kernel's 128- / 256-row tiles.
  auto blocking = [](int32_t rpb, int32_t n, int tile, int* rows, uint32_t* box_r, uint32_t* box_b, uint64_t* blocks) {
    if (rpb <= 0 || rpb >= n) {
      *rows = n;
      *box_r = static_cast<uint32_t>(tile);
      *box_b = 1;
      *blocks = 1;
      return true;
    }
    if (rpb % tile != 0 && tile % rpb != 0) return false;
    *rows = rpb;
    *box_r = static_cast<uint32_t>(rpb < tile ? rpb : tile);
    *box_b = static_cast<uint32_t>(tile / static_cast<int>(*box_r));
    *blocks = static_cast<uint64_t>((n + rpb - 1) / rpb);
    return true;
  };
  int a_rows, b_rows;
  uint32_t a_box_r, a_box_b, b_box_r, b_box_b;
  uint64_t a_blocks, b_blocks;
  B200_REQUIRE(blocking(a->a_rows_per_block, a->n_i, BM, &a_rows, &a_box_r, &a_box_b, &a_blocks) &&
                   blocking(a->b_rows_per_block, a->n_j, BN, &b_rows, &b_box_r, &b_box_b, &b_blocks),
               B200TRI_ERR_INVALID, "contract: rows_per_block must divide or be a multiple of the tile rows (128 for a, 256 for b)");
  B200_REQUIRE(a->a_block_stride % 8 == 0 && a->b_block_stride % 8 == 0 && a->out_block_stride % 8 == 0,
               B200TRI_ERR_INVALID, "contract: block strides must be multiples of 8 elements");
  CUtensorMap tm_a, tm_b;
  {
    const uint64_t dims[5] = {(uint64_t)a->n_k, (uint64_t)a_rows, a_blocks, 128, (uint64_t)a->n_src};
    const uint64_t str[4] = {(uint64_t)a->a_ld * 2, (uint64_t)(a_blocks > 1 ? a->a_block_stride : a->a_chan_stride * 128) * 2,
                             (uint64_t)a->a_chan_stride * 2,
                             (uint64_t)(a->n_src > 1 ? a->a_src_stride : a->a_chan_stride * 128) * 2};
    const uint32_t box[5] = {BK, a_box_r, a_box_b, 1, 1};
    int rc = make_tmap(&tm_a, a->a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  {
    const uint64_t dims[5] = {(uint64_t)a->n_k, (uint64_t)b_rows, b_blocks, 128, (uint64_t)a->n_src};
    const uint64_t str[4] = {(uint64_t)a->b_ld * 2, (uint64_t)(b_blocks > 1 ? a->b_block_stride : a->b_chan_stride * 128) * 2,
                             (uint64_t)a->b_chan_stride * 2,
                             (uint64_t)(a->n_src > 1 ? a->b_src_stride : a->b_chan_stride * 128) * 2};
    const uint32_t box[5] = {BK, b_box_r, b_box_b, 1, 1};
    int rc = make_tmap(&tm_b, a->b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, dims, str, box, Swz::B128);
    if (rc) return rc;
  }
  ContractParams p;
  p.n_i = a->n_i;
  p.n_j = a->n_j;
  p.n_src = a->n_src;
  p.kb_per_src = (a->n_k + BK - 1) / BK;
  p.tiles_m = (a->n_i + BM - 1) / BM;
  p.tiles_n = (a->n_j + BN - 1) / BN;
  p.total_tiles = 128ll * p.tiles_m * p.tiles_n;
  p.acc_in = a->acc_in;
  p.out_f32 = a->out_f32;
  p.out_bf16 = static_cast<__nv_bfloat16*>(a->out_bf16);
  p.out_ld = a->out_ld;
  p.out_chan_stride = a->out_chan_stride;
  p.a_rpb = a_rows;
  p.b_rpb = b_rows;
  p.out_rpb = (a->out_rows_per_block > 0 && a->out_rows_per_block < a->n_i) ? a->out_rows_per_block : (a->n_i > 0 ? a->n_i : 1);
  p.out_block_stride = a->out_block_stride;
  p.status = status;

  {
    const int rc = ensure_smem_limit(reinterpret_cast<const void*>(contract_kernel), SMEM_BYTES);
    if (rc) return rc;
  }
  const long long grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
  {
    TimedLaunch timed(K_TRIMUL_CONTRACT, reinterpret_cast<cudaStream_t>(stream));
    count_launch();
    contract_kernel<<<static_cast<unsigned>(grid), THREADS, SMEM_BYTES, reinterpret_cast<cudaStream_t>(stream)>>>(
      tm_a, tm_b, p);
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}
