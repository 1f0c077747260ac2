// MXFP8 GEMM on CTA pairs (`cta_group::2`): one 256 x 256 output tile per 2-CTA cluster.
//
// Each CTA of the pair stages its own 128 rows of A and only *half* of B (128 of the 256 N columns) plus the
// scale blocks; one thread of the even CTA issues `tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale` with M = 256,
// which reads both CTAs' shared memory and writes 128 accumulator rows into each CTA's tensor memory.  Per CTA
// and K step the MMA reads 4 KB of A + 4 KB of B instead of 4 + 8 KB for a single-CTA 128 x 256 tile, which is
// what lifts the operand-bandwidth ceiling of the one-CTA kernel (csrc/gemm_mxfp8.cu).  No TMA load is multicast:
// each CTA fetches exactly the bytes it keeps.
//
// Synchronisation inside the pair (all waits bounded, errors through the status word):
//   full[stage]      lives in the even CTA: its producer arrives once expecting the bytes of BOTH CTAs; the odd
//                    CTA's TMA loads (`cta_group::2` form) count their bytes on that same barrier;
//   empty[stage]     in both CTAs, released by a multicast `tcgen05.commit` of the MMA thread;
//   tmem_full        in both CTAs, multicast commit after the last K step of a tile;
//   tmem_empty       in the even CTA, two arrivals: one elected epilogue thread per CTA (the odd one remotely).
// Tensor memory is allocated / freed with the `cta_group::2` forms by the same warp of both CTAs; a cluster
// barrier closes the kernel so that neither CTA exits while its peer may still touch its memory.
//
// Layout conventions and scale-block format as in csrc/gemm_mxfp8.cu / csrc/quant_mxfp8.cu; scale blocks are
// fetched with 3-D tensor maps ([mn block, k block, 512 bytes]) so that blocks past the edge read as zero.
#include "common.cuh"

namespace {

constexpr int BM = 128;            // rows per CTA (256 per pair)
constexpr int BN = 256;            // columns per pair; each CTA stages BN / 2 of B
constexpr int BK = 128;
constexpr int UMMA_K = 32;
constexpr int STAGES = 6;
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int GROUP_M = 8;         // in units of 256-row pair tiles
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = (BN / 2) * BK;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;      // 32 KiB
constexpr int SF_BYTES = 512 + 1024;                // A scales of this CTA's rows + B scales of all 256 columns
constexpr int SMEM_BYTES = STAGES * (STAGE_BYTES + SF_BYTES) + 1024 + 256;
constexpr int SFA_COL = BN;
constexpr int SFB_COL = BN + 4;
constexpr int TMEM_COLS = 512;
enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ADD = 2 };

struct Barriers {
  uint64_t full[STAGES];        // used in the even CTA: 1 arrival, transaction bytes of both CTAs
  uint64_t empty[STAGES];
  uint64_t tmem_full;
  uint64_t tmem_empty;          // used in the even CTA
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

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& mb, int& nb) {
  const int per_group = GROUP_M * num_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, num_m - first_m);
  const int r = tile - g * per_group;
  mb = first_m + r % gm;
  nb = r / gm;
}

template <int A_MN, int B_MN, int OUT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mxfp8_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                       void* __restrict__ Dv, long ldd, int M, int N, int K, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_ab = smem;
  uint8_t* smem_sf = smem + STAGES * STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(smem_sf + STAGES * SF_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = pb::cluster_ctarank();      // 0: even CTA (issues the MMAs), 1: odd CTA
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_m = (M + 2 * BM - 1) / (2 * BM);
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = K / BK;
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      pb::mbar_init(&bars->full[i], 1);
      pb::mbar_init(&bars->empty[i], 1);
    }
    pb::mbar_init(&bars->tmem_full, 1);
    pb::mbar_init(&bars->tmem_empty, 2);
    bars->abort_flag = 0;
    pb::fence_barrier_init();
    pb::prefetch_tmap(&tmA);
    pb::prefetch_tmap(&tmB);
    pb::prefetch_tmap(&tmSFA);
    pb::prefetch_tmap(&tmSFB);
  }
  if (warp == 1) {
    pb::tmem_alloc<2>(&bars->tmem_base, TMEM_COLS);
    pb::tmem_relinquish<2>();
  }
  pb::tc_fence_before();
  __syncthreads();
  pb::cluster_sync();          // barriers of both CTAs are initialised before any remote arrive / multicast commit
  pb::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int mb, nb;
        tile_coords(tile, num_m, num_n, mb, nb);
        const int mblk = mb * 2 + (int)cta;          // 128-row block of this CTA
        const int m0 = mblk * BM;
        const int n0 = nb * BN + (int)cta * (BN / 2);  // this CTA's half of the B tile
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->empty[stage], phase ^ 1, abort_flag)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_TMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem_ab + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          uint8_t* ssf = smem_sf + stage * SF_BYTES;
          if (cta == 0) pb::mbar_expect_tx(&bars->full[stage], 2 * (STAGE_BYTES + SF_BYTES));
          const uint32_t fb = pb::mapa_shared(&bars->full[stage], 0);   // the even CTA's barrier
          if (A_MN == 0) pb::tma_load_2d_pair(sa, &tmA, fb, kb * BK, m0);
          else pb::tma_load_2d_pair(sa, &tmA, fb, m0, kb * BK);
          if (B_MN == 0) pb::tma_load_2d_pair(sb, &tmB, fb, kb * BK, n0);
          else pb::tma_load_2d_pair(sb, &tmB, fb, n0, kb * BK);
          pb::tma_load_3d_pair(ssf, &tmSFA, fb, 0, kb, mblk);
          pb::tma_load_3d_pair(ssf + 512, &tmSFB, fb, 0, kb, nb * 2);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta == 0) {
      // ---------------------------------------------------------- MMA issuer (even CTA)
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t sfa_t = tmem_base + SFA_COL;
      const uint32_t sfb_t = tmem_base + SFB_COL;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!wait_or_abort(&bars->tmem_empty, acc_phase ^ 1, abort_flag)) {
          atomicCAS(status, 0, PB_ERR_TIMEOUT_MMA);
          bars->abort_flag = 1;
          break;
        }
        pb::tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->full[stage], phase, abort_flag)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_MMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          pb::tc_fence_after();
          const uint32_t sa = pb::smem_u32(smem_ab + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          const uint32_t ssf = pb::smem_u32(smem_sf + stage * SF_BYTES);
          pb::utccp_32x128b_warpx4_2cta(sfa_t, pb::make_smem_desc(ssf, 128, 128, 0));
          pb::utccp_32x128b_warpx4_2cta(sfb_t, pb::make_smem_desc(ssf + 512, 128, 128, 0));
          pb::utccp_32x128b_warpx4_2cta(sfb_t + 4, pb::make_smem_desc(ssf + 1024, 128, 128, 0));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? pb::make_smem_desc(sa + k * (UMMA_K * 128), BK * 128, 1024, 2)
                                     : pb::make_smem_desc(sa + k * UMMA_K, 0, 1024, 2);
            const uint64_t db = B_MN ? pb::make_smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024, 2)
                                     : pb::make_smem_desc(sb + k * UMMA_K, 0, 1024, 2);
            const uint32_t idesc = pb::make_idesc_mxf8(2 * BM, BN, A_MN, B_MN, k, k);
            pb::umma_mxf8_ss_2cta(tmem_base, da, db, idesc, sfa_t | (uint32_t(k) << 30), sfb_t | (uint32_t(k) << 30),
                                  (kb > 0 || k > 0) ? 1u : 0u);
          }
          pb::umma_commit_2cta(&bars->empty[stage], 3);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        pb::umma_commit_2cta(&bars->tmem_full, 3);
        acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, 128 rows each)
    const int et = threadIdx.x - 64;
    const int lane_grp = warp & 3;
    const int row = lane_grp * 32 + lane;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int mb, nb;
      tile_coords(tile, num_m, num_n, mb, nb);
      const int m = (mb * 2 + (int)cta) * BM + row, n0 = nb * BN;
      if (!wait_or_abort(&bars->tmem_full, acc_phase, abort_flag)) {
        atomicCAS(status, 0, PB_ERR_TIMEOUT_EPILOGUE);
        bars->abort_flag = 1;
        ok = false;
        break;
      }
      acc_phase ^= 1;
      pb::tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(lane_grp * 32) << 16);
      auto release = [&]() {
        pb::tc_fence_before();
        pb::named_bar_sync(1, EPI_THREADS);
        if (et == 0) {
          if (cta == 0) pb::mbar_arrive(&bars->tmem_empty);
          else pb::mbar_arrive_remote(pb::mapa_shared(&bars->tmem_empty, 0));
        }
      };
      if (OUT == OUT_BF16) {
        uint32_t packed[BN / 2];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          pb::tmem_ld_32x32b_x32(t_row + c * 32, r);
          pb::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            packed[c * 16 + j] = pb::pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        }
        release();
        if (m < M) {
          __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(Dv) + (long)m * ldd + n0;
#pragma unroll
          for (int j = 0; j < BN / 8; ++j)
            if (n0 + 8 * j < N)
              reinterpret_cast<uint4*>(d)[j] =
                  make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          pb::tmem_ld_32x32b_x32(t_row + c * 32, r);
          pb::tmem_wait_ld();
          const int n = n0 + c * 32;
          if (m < M && n < N) {
            float* d = reinterpret_cast<float*>(Dv) + (long)m * ldd + n;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (n + 4 * j < N) {
                if (OUT == OUT_F32) {
                  reinterpret_cast<uint4*>(d)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                } else {
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d + 4 * j),
                               "f"(__uint_as_float(r[4 * j])), "f"(__uint_as_float(r[4 * j + 1])),
                               "f"(__uint_as_float(r[4 * j + 2])), "f"(__uint_as_float(r[4 * j + 3]))
                               : "memory");
                }
              }
            }
          }
        }
        release();
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  pb::tc_fence_before();
  __syncthreads();
  pb::cluster_sync();          // the peer may still multicast into / read from this CTA until here
  if (warp == 1) {
    pb::tc_fence_after();
    pb::tmem_dealloc<2>(tmem_base, TMEM_COLS);
  }
}

int g_num_sms = 0;
int g_max_pairs_seen = 0;

template <int A_MN, int B_MN, int OUT>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tSFA, const CUtensorMap& tSFB, void* D,
           long ldd, int M, int N, int K, int* status, int max_ctas, cudaStream_t stream) {
  auto kern = gemm_mxfp8_2cta_kernel<A_MN, B_MN, OUT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // a persistent grid must not exceed the number of CTA pairs the device can keep resident at once (SMs pair up
  // inside a GPC, so this can be fewer than SMs / 2)
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cfg.gridDim = dim3(g_num_sms, 1, 1);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = g_num_sms / 2;
    }
    max_pairs = n;
    g_max_pairs_seen = n;
  }
  int pairs = max_pairs;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (tiles < pairs) pairs = tiles;
  if (pairs < 1) pairs = 1;
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.stream = stream;
  return (int)cudaLaunchKernelEx(&cfg, kern, tA, tB, tSFA, tSFB, D, ldd, M, N, K, status);
}

}  // namespace

// number of CTA pairs the last launch configuration could keep resident (0 before the first launch)
extern "C" int pb_gemm_mxfp8_2cta_resident_pairs() { return g_max_pairs_seen; }

// Same contract as pb_gemm_mxfp8 (csrc/gemm_mxfp8.cu); output tile 256 x 256 per CTA pair.
extern "C" int pb_gemm_mxfp8_2cta(const void* A, const void* SFA, const void* B, const void* SFB, void* D, int M, int N,
                                  int K, long lda, long ldb, long ldd, int a_mn, int b_mn, int out_mode, int max_ctas,
                                  int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % BK || (lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A) % 16) ||
      (reinterpret_cast<uintptr_t>(B) % 16) || (reinterpret_cast<uintptr_t>(D) % 16) ||
      (reinterpret_cast<uintptr_t>(SFA) % 16) || (reinterpret_cast<uintptr_t>(SFB) % 16))
    return -2;
  if (out_mode == 0 ? (ldd % 8 || N % 8) : (ldd % 4 || N % 4)) return -2;
  CUtensorMap tA, tB, tSFA, tSFB;
  int rc;
  const auto u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  if (!a_mn) rc = pbh::make_tmap_2d(&tA, A, u8, 1, M, K, lda, BM, BK, sw);
  else rc = pbh::make_tmap_2d(&tA, A, u8, 1, K, M, lda, BK, 128, sw);
  if (rc) return rc;
  if (!b_mn) rc = pbh::make_tmap_2d(&tB, B, u8, 1, N, K, ldb, BN / 2, BK, sw);
  else rc = pbh::make_tmap_2d(&tB, B, u8, 1, K, N, ldb, BK, 128, sw);
  if (rc) return rc;
  // scale blocks: [mn block][k block][128 x uint32]
  const int num_kb = K / BK;
  const auto u32 = CU_TENSOR_MAP_DATA_TYPE_UINT32;
  const auto nsw = CU_TENSOR_MAP_SWIZZLE_NONE;
  if ((rc = pbh::make_tmap_3d(&tSFA, SFA, u32, 4, (M + 127) / 128, num_kb, 128, 128, (uint64_t)num_kb * 128, 1, 1, 128, nsw)))
    return rc;
  if ((rc = pbh::make_tmap_3d(&tSFB, SFB, u32, 4, (N + 127) / 128, num_kb, 128, 128, (uint64_t)num_kb * 128, 2, 1, 128, nsw)))
    return rc;

#define PB_DISPATCH_OUT(AM, BMN)                                                                                  \
  switch (out_mode) {                                                                                             \
    case 0: return launch<AM, BMN, OUT_BF16>(tA, tB, tSFA, tSFB, D, ldd, M, N, K, status, max_ctas, stream);      \
    case 1: return launch<AM, BMN, OUT_F32>(tA, tB, tSFA, tSFB, D, ldd, M, N, K, status, max_ctas, stream);       \
    case 2: return launch<AM, BMN, OUT_F32_ADD>(tA, tB, tSFA, tSFB, D, ldd, M, N, K, status, max_ctas, stream);   \
    default: return -3;                                                                                           \
  }
  if (!a_mn && !b_mn) { PB_DISPATCH_OUT(0, 0) }
  else if (!a_mn && b_mn) { PB_DISPATCH_OUT(0, 1) }
  else if (a_mn && b_mn) { PB_DISPATCH_OUT(1, 1) }
  else { PB_DISPATCH_OUT(1, 0) }
  return -3;
}
