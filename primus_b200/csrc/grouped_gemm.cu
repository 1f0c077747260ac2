// Grouped (per-expert) bf16 GEMMs for MoE on tcgen05, with the expert schedule read from device memory
// (no host synchronisation on the routing result).
//
// Tokens are stored expert-major in a padded layout: expert e owns rows [row_start[e], row_start[e] +
// padded[e]) where padded[e] is its token count rounded up to 128 (padding rows are zero), so a 128-row
// tile never straddles two experts.  `mblock_expert[mb]` gives the expert of row block mb (-1 beyond the
// last used block): the persistent tile loop simply skips unused blocks.
//
//   fprop / dgrad : D[rows, N] = A[rows, K] . B[e]^T      B: [E, N, K]  (B_MN = 0)   or   [E, K, N]  (B_MN = 1)
//   wgrad         : D[e][N, K] (=|+=) A_e^T . B_e         A = dy [rows, N], B = x [rows, K]; reduction over the
//                                                          expert's rows; fp32 output (store or accumulate)
//
// Same pipeline as csrc/gemm_bf16.cu (TMA 128B-swizzled stages, one MMA-issuing thread, double-buffered
// TMEM accumulator, TMA store epilogue).  Replaces `pt.ops.grouped_gemm`
// (primus/backends/megatron/core/extensions/primus_turbo.py:2103-2218).
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BUF_BYTES = BM * 128;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * EPI_BUF_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 2 * BN;

enum { G_FPROP = 0, G_DGRAD = 1, G_WGRAD = 2 };

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (pb::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!pb::mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > PB_WAIT_CYCLES) return false;
  }
  return true;
}

PB_DEVICE void tma_reduce_add_3d(const CUtensorMap* m, const void* smem_src, int x, int y, int z) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(pb::smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

struct Tile {
  int valid;      // 0: skip
  int expert;
  int m0, n0;     // output tile origin (rows / cols of D, or of D[e] for wgrad)
  int k_begin;    // first reduction block (units of BK)
  int k_blocks;   // number of reduction blocks
};

// MODE fprop/dgrad: tiles = max_mblocks x num_n (m fastest inside a group of 8 row blocks)
// MODE wgrad      : tiles = E x num_m x num_n over D[e][N_out, K_out]
template <int MODE>
__device__ __forceinline__ Tile get_tile(int tile, int num_m, int num_n, int K, const int* __restrict__ mblock_expert,
                                         const int* __restrict__ row_start, const int* __restrict__ padded) {
  Tile t;
  if (MODE != G_WGRAD) {
    const int mb = tile % num_m, nb = tile / num_m;
    const int e = mblock_expert[mb];
    t.valid = e >= 0;
    t.expert = e;
    t.m0 = mb * BM;
    t.n0 = nb * BN;
    t.k_begin = 0;
    t.k_blocks = (K + BK - 1) / BK;
  } else {
    const int per_e = num_m * num_n;
    const int e = tile / per_e;
    const int r = tile - e * per_e;
    t.expert = e;
    t.m0 = (r % num_m) * BM;
    t.n0 = (r / num_m) * BN;
    t.k_begin = row_start[e] / BK;
    t.k_blocks = padded[e] / BK;
    t.valid = 1;  // experts without tokens still run the epilogue with an untouched (zero) accumulator
  }
  return t;
}

template <int MODE, int OUT_ADD>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmD, int num_m, int num_n, int num_tiles, int K,
                    const int* __restrict__ mblock_expert, const int* __restrict__ row_start,
                    const int* __restrict__ padded, int* status) {
  constexpr int A_MN = (MODE == G_WGRAD) ? 1 : 0;
  constexpr int B_MN = (MODE == G_FPROP) ? 0 : 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_ab = smem;
  uint8_t* smem_epi = smem + STAGES * STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(smem_epi + 2 * EPI_BUF_BYTES);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      pb::mbar_init(&bars->full[i], 1);
      pb::mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      pb::mbar_init(&bars->tmem_full[i], 1);
      pb::mbar_init(&bars->tmem_empty[i], EPI_THREADS);
    }
    bars->abort_flag = 0;
    pb::fence_barrier_init();
  }
  if (warp == 1) {
    pb::tmem_alloc<1>(&bars->tmem_base, TMEM_COLS);
    pb::tmem_relinquish<1>();
  }
  pb::tc_fence_before();
  __syncthreads();
  pb::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const Tile t = get_tile<MODE>(tile, num_m, num_n, K, mblock_expert, row_start, padded);
        if (!t.valid) continue;
        for (int kb = t.k_begin; kb < t.k_begin + t.k_blocks; ++kb) {
          if (!wait_or_abort(&bars->empty[stage], phase ^ 1, abort_flag)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_TMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem_ab + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          pb::mbar_expect_tx(&bars->full[stage], STAGE_BYTES);
          if (MODE == G_FPROP) {
            pb::tma_load_2d(sa, &tmA, &bars->full[stage], kb * BK, t.m0);
            pb::tma_load_3d(sb, &tmB, &bars->full[stage], kb * BK, t.n0, t.expert);
          } else if (MODE == G_DGRAD) {
            pb::tma_load_2d(sa, &tmA, &bars->full[stage], kb * BK, t.m0);
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              pb::tma_load_3d(sb + i * (BK * 128), &tmB, &bars->full[stage], t.n0 + i * 64, kb * BK, t.expert);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              pb::tma_load_2d(sa + i * (BK * 128), &tmA, &bars->full[stage], t.m0 + i * 64, kb * BK);
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              pb::tma_load_2d(sb + i * (BK * 128), &tmB, &bars->full[stage], t.n0 + i * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = pb::make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const Tile t = get_tile<MODE>(tile, num_m, num_n, K, mblock_expert, row_start, padded);
        if (!t.valid) continue;
        if (!wait_or_abort(&bars->tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          atomicCAS(status, 0, PB_ERR_TIMEOUT_MMA);
          bars->abort_flag = 1;
          break;
        }
        pb::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!wait_or_abort(&bars->full[stage], phase, abort_flag)) {
            if (!*abort_flag) atomicCAS(status, 0, PB_ERR_TIMEOUT_MMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          pb::tc_fence_after();
          const uint32_t sa = pb::smem_u32(smem_ab + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? pb::make_smem_desc(sa + k * (UMMA_K * 128), BK * 128, 1024, 2)
                                     : pb::make_smem_desc(sa + k * (UMMA_K * 2), 0, 1024, 2);
            const uint64_t db = B_MN ? pb::make_smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024, 2)
                                     : pb::make_smem_desc(sb + k * (UMMA_K * 2), 0, 1024, 2);
            pb::umma_f16_ss(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          pb::umma_commit(&bars->empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        pb::umma_commit(&bars->tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    const int et = threadIdx.x - 64;
    const int lane_grp = warp & 3;
    const int row = lane_grp * 32 + lane;
    constexpr int CHUNK_COLS = (MODE == G_WGRAD) ? 32 : 64;
    constexpr int NUM_CHUNKS = BN / CHUNK_COLS;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const Tile t = get_tile<MODE>(tile, num_m, num_n, K, mblock_expert, row_start, padded);
      if (!t.valid) continue;
      const bool empty_acc = (t.k_blocks == 0);  // wgrad of an expert without tokens: nothing was accumulated
      if (!wait_or_abort(&bars->tmem_full[acc], acc_phase, abort_flag)) {
        if (!*abort_flag) atomicCAS(status, 0, PB_ERR_TIMEOUT_EPILOGUE);
        bars->abort_flag = 1;
        ok = false;
        break;
      }
      pb::tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(lane_grp * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < NUM_CHUNKS; ++c) {
        uint32_t r[64];
        if (MODE != G_WGRAD) {
          pb::tmem_ld_32x32b_x32(t_row + c * 64, r);
          pb::tmem_ld_32x32b_x32(t_row + c * 64 + 32, r + 32);
        } else {
          pb::tmem_ld_32x32b_x32(t_row + c * 32, r);
        }
        pb::tmem_wait_ld();
        if (empty_acc) {
#pragma unroll
          for (int i = 0; i < 64; ++i) r[i] = 0u;
        }
        if (et == 0) pb::tma_store_wait_read<1>();
        pb::named_bar_sync(1, EPI_THREADS);
        uint8_t* stage_buf = smem_epi + buf * EPI_BUF_BYTES;
        uint8_t* my_row = stage_buf + row * 128;
        if (MODE != G_WGRAD) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 v;
            v.x = pb::pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            v.y = pb::pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            v.z = pb::pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            v.w = pb::pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            *reinterpret_cast<uint4*>(my_row + ((j ^ (row & 7)) << 4)) = v;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(my_row + ((j ^ (row & 7)) << 4)) =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
        pb::fence_proxy_async_smem();
        pb::named_bar_sync(1, EPI_THREADS);
        if (et == 0) {
          if (MODE != G_WGRAD) {
            pb::tma_store_2d(&tmD, stage_buf, t.n0 + c * CHUNK_COLS, t.m0);
          } else if (OUT_ADD) {
            tma_reduce_add_3d(&tmD, stage_buf, t.n0 + c * CHUNK_COLS, t.m0, t.expert);
          } else {
            pb::tma_store_3d(&tmD, stage_buf, t.n0 + c * CHUNK_COLS, t.m0, t.expert);
          }
          pb::tma_store_commit();
        }
        buf ^= 1;
      }
      pb::tc_fence_before();
      pb::mbar_arrive(&bars->tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (et == 0) pb::tma_store_wait_all<0>();
  }

  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  pb::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    pb::tc_fence_after();
    pb::tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

template <int MODE, int OUT_ADD>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tD, int num_m, int num_n, int num_tiles,
           int K, const int* mblock_expert, const int* row_start, const int* padded, int* status, cudaStream_t s) {
  auto kern = grouped_gemm_kernel<MODE, OUT_ADD>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int ctas = num_tiles < num_sms ? num_tiles : num_sms;
  kern<<<ctas, NUM_THREADS, SMEM_BYTES, s>>>(tA, tB, tD, num_m, num_n, num_tiles, K, mblock_expert, row_start, padded,
                                            status);
  return (int)cudaGetLastError();
}

// Builds the per-row-block expert table and the padded row offsets from per-expert token counts.
//   counts[E] -> padded[E] (multiple of 128), row_start[E], mblock_expert[max_mblocks] (-1 when unused),
//   total_rows[0].
__global__ void build_schedule_kernel(const int* __restrict__ counts, int E, int max_mblocks, int* __restrict__ padded,
                                      int* __restrict__ row_start, int* __restrict__ mblock_expert,
                                      int* __restrict__ total_rows) {
  __shared__ int s_start[1025];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      const int p = (counts[e] + BM - 1) / BM * BM;
      padded[e] = p;
      row_start[e] = acc;
      s_start[e] = acc;
      acc += p;
    }
    s_start[E] = acc;
    total_rows[0] = acc;
  }
  __syncthreads();
  for (int mb = threadIdx.x; mb < max_mblocks; mb += blockDim.x) {
    const int r = mb * BM;
    int e = -1;
    if (r < s_start[E]) {
      int lo = 0, hi = E - 1;  // last expert with start <= r
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_start[mid] <= r) lo = mid; else hi = mid - 1;
      }
      e = lo;
    }
    mblock_expert[mb] = e;
  }
}

}  // namespace

extern "C" {

int pb_moe_build_schedule(const int* counts, int E, int max_mblocks, int* padded, int* row_start, int* mblock_expert,
                          int* total_rows, cudaStream_t s) {
  if (E > 1024) return -2;
  build_schedule_kernel<<<1, 256, 0, s>>>(counts, E, max_mblocks, padded, row_start, mblock_expert, total_rows);
  return (int)cudaGetLastError();
}

// mode 0 fprop: A [rows_cap, K], B [E, N, K], D [rows_cap, N] bf16
// mode 1 dgrad: A [rows_cap, K_red], B [E, K_red, N], D [rows_cap, N] bf16   (K = K_red)
// mode 2 wgrad: A = dy [rows_cap, N_out], B = x [rows_cap, K_out], D [E, N_out, K_out] fp32 (accumulate != 0: +=);
//               here N := N_out rows of D[e], Kdim := K_out cols of D[e]
int pb_grouped_gemm(int mode, const void* A, const void* B, void* D, int rows_cap, int N, int K, int E,
                    const int* mblock_expert, const int* row_start, const int* padded, int accumulate, int* status,
                    cudaStream_t s) {
  if (rows_cap % BM || N % 8 || K % 8) return -2;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA, tB, tD;
  int rc;
  if (mode == G_FPROP) {
    if ((rc = pbh::make_tmap_2d(&tA, A, bf, 2, rows_cap, K, K, BM, BK, sw))) return rc;
    if ((rc = pbh::make_tmap_3d(&tB, B, bf, 2, E, N, K, K, (long)N * K, 1, BN, BK, sw))) return rc;
    if ((rc = pbh::make_tmap_2d(&tD, D, bf, 2, rows_cap, N, N, BM, 64, sw))) return rc;
    const int num_m = rows_cap / BM, num_n = (N + BN - 1) / BN;
    return launch<G_FPROP, 0>(tA, tB, tD, num_m, num_n, num_m * num_n, K, mblock_expert, row_start, padded, status, s);
  }
  if (mode == G_DGRAD) {
    if ((rc = pbh::make_tmap_2d(&tA, A, bf, 2, rows_cap, K, K, BM, BK, sw))) return rc;
    if ((rc = pbh::make_tmap_3d(&tB, B, bf, 2, E, K, N, N, (long)N * K, 1, BK, 64, sw))) return rc;
    if ((rc = pbh::make_tmap_2d(&tD, D, bf, 2, rows_cap, N, N, BM, 64, sw))) return rc;
    const int num_m = rows_cap / BM, num_n = (N + BN - 1) / BN;
    return launch<G_DGRAD, 0>(tA, tB, tD, num_m, num_n, num_m * num_n, K, mblock_expert, row_start, padded, status, s);
  }
  if (mode == G_WGRAD) {
    if ((rc = pbh::make_tmap_2d(&tA, A, bf, 2, rows_cap, N, N, BK, 64, sw))) return rc;
    if ((rc = pbh::make_tmap_2d(&tB, B, bf, 2, rows_cap, K, K, BK, 64, sw))) return rc;
    if ((rc = pbh::make_tmap_3d(&tD, D, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, E, N, K, K, (long)N * K, 1, BM, 32, sw)))
      return rc;
    const int num_m = (N + BM - 1) / BM, num_n = (K + BN - 1) / BN;
    const int tiles = E * num_m * num_n;
    if (accumulate)
      return launch<G_WGRAD, 1>(tA, tB, tD, num_m, num_n, tiles, K, mblock_expert, row_start, padded, status, s);
    return launch<G_WGRAD, 0>(tA, tB, tD, num_m, num_n, tiles, K, mblock_expert, row_start, padded, status, s);
  }
  return -3;
}

}  // extern "C"
