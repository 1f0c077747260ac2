// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   D[M,N] (=|+=) A[M,K] . B[N,K]^T          fp32 accumulation in tensor memory
//
// * operands are staged in shared memory by TMA (128-byte swizzle, no multicast),
// * one elected thread issues tcgen05.mma (128 x BN x 16 per instruction) into a
//   double-buffered TMEM accumulator, so the epilogue of tile i overlaps the main loop of tile i+1,
// * four epilogue warps read the accumulator with tcgen05.ld, convert, stage through swizzled
//   shared memory and write with TMA stores (or TMA reduce-add for the fp32 "+=" mode that
//   accumulates weight gradients straight into the fp32 main-grad buffer).
//
// Operand layouts (row-major storage):
//   A_MN = 0: A stored [M, K] (K contiguous)      A_MN = 1: A stored [K, M] (M contiguous)
//   B_MN = 0: B stored [N, K] (K contiguous)      B_MN = 1: B stored [K, N] (N contiguous)
// so the three GEMMs of a linear layer y = x W^T need no transposes:
//   fprop  y  = x . W^T      -> (A_MN=0, B_MN=0)   A = x [T,in],  B = W [out,in]
//   dgrad  dx = dy . W       -> (A_MN=0, B_MN=1)   A = dy [T,out], B = W stored [K=out, N=in]
//   wgrad  dW = dy^T . x     -> (A_MN=1, B_MN=1)   A = dy stored [K=T, M=out], B = x stored [K=T, N=in]
//
// Replaces the reference's library GEMM call sites (primus/backends/megatron/core/extensions/
// primus_turbo.py:1182-1189 `pt.ops.gemm`, and the Apex wgrad-accumulate
// primus/backends/megatron/core/tensor_parallel/layers.py:171-181).
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;  // warp0: TMA, warp1: MMA + TMEM alloc, warps 2-5: epilogue
constexpr int EPI_THREADS = 128;
constexpr int GROUP_M = 16;

enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ADD = 2 };

template <int BN>
struct Cfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BUF_BYTES = BM * 128;  // 128 rows x 128 B
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * EPI_BUF_BYTES + 1024 /*align*/ + 256;
  static constexpr int TMEM_COLS = 2 * BN;
};

struct Barriers {
  uint64_t full[8];
  uint64_t empty[8];
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

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& mb, int& nb) {
  const int per_group = GROUP_M * num_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, num_m - first_m);
  const int r = tile - g * per_group;
  mb = first_m + r % gm;
  nb = r / gm;
}

template <int BN, int A_MN, int B_MN, int OUT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, int M, int N, int K, int* status) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_ab = smem;
  uint8_t* smem_epi = smem + C::STAGES * C::STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(smem_epi + 2 * C::EPI_BUF_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BK - 1) / BK;
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::STAGES; ++i) {
      pb::mbar_init(&bars->full[i], 1);
      pb::mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      pb::mbar_init(&bars->tmem_full[i], 1);
      pb::mbar_init(&bars->tmem_empty[i], EPI_THREADS);
    }
    bars->abort_flag = 0;
    pb::fence_barrier_init();
    pb::prefetch_tmap(&tmA);
    pb::prefetch_tmap(&tmB);
    pb::prefetch_tmap(&tmD);
  }
  if (warp == 1) {
    pb::tmem_alloc<1>(&bars->tmem_base, C::TMEM_COLS);
    pb::tmem_relinquish<1>();
  }
  pb::tc_fence_before();
  __syncthreads();
  pb::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, num_m, num_n, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->empty[stage], phase ^ 1, abort_flag)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_TMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem_ab + stage * C::STAGE_BYTES;
          uint8_t* sb = sa + C::A_BYTES;
          pb::mbar_expect_tx(&bars->full[stage], C::STAGE_BYTES);
          if (A_MN == 0) {
            pb::tma_load_2d(sa, &tmA, &bars->full[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              pb::tma_load_2d(sa + i * (BK * 128), &tmA, &bars->full[stage], m0 + i * 64, kb * BK);
          }
          if (B_MN == 0) {
            pb::tma_load_2d(sb, &tmB, &bars->full[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              pb::tma_load_2d(sb + i * (BK * 128), &tmB, &bars->full[stage], n0 + i * 64, kb * BK);
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = pb::make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!wait_or_abort(&bars->tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          atomicCAS(status, 0, PB_ERR_TIMEOUT_MMA);
          bars->abort_flag = 1;
          break;
        }
        pb::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->full[stage], phase, abort_flag)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_MMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          pb::tc_fence_after();
          const uint32_t sa = pb::smem_u32(smem_ab + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? pb::make_smem_desc(sa + k * (UMMA_K * 128), BK * 128, 1024, 2)
                                     : pb::make_smem_desc(sa + k * (UMMA_K * 2), 0, 1024, 2);
            const uint64_t db = B_MN ? pb::make_smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024, 2)
                                     : pb::make_smem_desc(sb + k * (UMMA_K * 2), 0, 1024, 2);
            pb::umma_f16_ss(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          pb::umma_commit(&bars->empty[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == C::STAGES) {
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
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int et = threadIdx.x - 64;         // 0..127
    const int lane_grp = warp & 3;           // TMEM lane quarter this warp may access
    const int row = lane_grp * 32 + lane;    // row inside the 128-row tile
    constexpr int CHUNK_COLS = (OUT == OUT_BF16) ? 64 : 32;  // 128 bytes of output per row
    constexpr int NUM_CHUNKS = BN / CHUNK_COLS;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int mb, nb;
      tile_coords(tile, num_m, num_n, mb, nb);
      const int m0 = mb * BM, n0 = nb * BN;
      if (!wait_or_abort(&bars->tmem_full[acc], acc_phase, abort_flag)) {
        atomicCAS(status, 0, PB_ERR_TIMEOUT_EPILOGUE);
        bars->abort_flag = 1;
        ok = false;
        break;
      }
      pb::tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(lane_grp * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < NUM_CHUNKS; ++c) {
        uint32_t r[64];
        if (OUT == OUT_BF16) {
          pb::tmem_ld_32x32b_x32(t_row + c * 64, r);
          pb::tmem_ld_32x32b_x32(t_row + c * 64 + 32, r + 32);
        } else {
          pb::tmem_ld_32x32b_x32(t_row + c * 32, r);
        }
        pb::tmem_wait_ld();
        // the staging buffer written two chunks ago must have been read by its TMA store
        if (et == 0) pb::tma_store_wait_read<1>();
        pb::named_bar_sync(1, EPI_THREADS);
        uint8_t* stage_buf = smem_epi + buf * C::EPI_BUF_BYTES;
        uint8_t* my_row = stage_buf + row * 128;
        if (OUT == OUT_BF16) {
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
          for (int j = 0; j < 8; ++j) {
            uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            *reinterpret_cast<uint4*>(my_row + ((j ^ (row & 7)) << 4)) = v;
          }
        }
        pb::fence_proxy_async_smem();
        pb::named_bar_sync(1, EPI_THREADS);
        if (et == 0) {
          if (OUT == OUT_F32_ADD)
            pb::tma_reduce_add_2d(&tmD, stage_buf, n0 + c * CHUNK_COLS, m0);
          else
            pb::tma_store_2d(&tmD, stage_buf, n0 + c * CHUNK_COLS, m0);
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

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    // give copies that are still in flight time to land before shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  pb::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    pb::tc_fence_after();
    pb::tmem_dealloc<1>(tmem_base, C::TMEM_COLS);
  }
}

int g_num_sms = 0;

template <int BN, int A_MN, int B_MN, int OUT>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tD, int M, int N, int K,
           int* status, int max_ctas, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OUT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int ctas = g_num_sms;
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (tiles < ctas) ctas = tiles;
  kern<<<ctas, NUM_THREADS, C::SMEM_BYTES, stream>>>(tA, tB, tD, M, N, K, status);
  return (int)cudaGetLastError();
}

}  // namespace

// D[M,N] (=|+=) A . B^T.  lda/ldb/ldd are row pitches in elements of the *stored* matrices.
// out_mode: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate (D += ...).
// block_n: 256 or 128.  max_ctas: 0 = all SMs (smaller values leave SMs free for overlapped work).
// Returns 0 on success, a CUDA/driver error code otherwise; device-side timeouts are reported
// through *status (device int, must be zero-initialised by the caller).
extern "C" int pb_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long lda,
                            long ldb, long ldd, int a_mn, int b_mn, int out_mode, int block_n,
                            int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) % 16) ||
      (reinterpret_cast<uintptr_t>(B) % 16) || (reinterpret_cast<uintptr_t>(D) % 16))
    return -2;
  if (out_mode == 0 ? (ldd % 8) : (ldd % 4)) return -2;
  const int BN = (block_n == 128) ? 128 : 256;
  CUtensorMap tA, tB, tD;
  int rc;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  if (!a_mn)
    rc = pbh::make_tmap_2d(&tA, A, bf, 2, M, K, lda, BM, BK, sw);
  else
    rc = pbh::make_tmap_2d(&tA, A, bf, 2, K, M, lda, BK, 64, sw);
  if (rc) return rc;
  if (!b_mn)
    rc = pbh::make_tmap_2d(&tB, B, bf, 2, N, K, ldb, BN, BK, sw);
  else
    rc = pbh::make_tmap_2d(&tB, B, bf, 2, K, N, ldb, BK, 64, sw);
  if (rc) return rc;
  if (out_mode == 0)
    rc = pbh::make_tmap_2d(&tD, D, bf, 2, M, N, ldd, BM, 64, sw);
  else
    rc = pbh::make_tmap_2d(&tD, D, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldd, BM, 32, sw);
  if (rc) return rc;

#define PB_DISPATCH_OUT(BN_, AM, BMN)                                                           \
  switch (out_mode) {                                                                           \
    case 0: return launch<BN_, AM, BMN, OUT_BF16>(tA, tB, tD, M, N, K, status, max_ctas, stream); \
    case 1: return launch<BN_, AM, BMN, OUT_F32>(tA, tB, tD, M, N, K, status, max_ctas, stream);  \
    case 2: return launch<BN_, AM, BMN, OUT_F32_ADD>(tA, tB, tD, M, N, K, status, max_ctas, stream); \
    default: return -3;                                                                         \
  }
#define PB_DISPATCH_LAYOUT(BN_)                          \
  if (!a_mn && !b_mn) { PB_DISPATCH_OUT(BN_, 0, 0) }     \
  else if (!a_mn && b_mn) { PB_DISPATCH_OUT(BN_, 0, 1) } \
  else if (a_mn && b_mn) { PB_DISPATCH_OUT(BN_, 1, 1) }  \
  else { PB_DISPATCH_OUT(BN_, 1, 0) }
  if (BN == 256) { PB_DISPATCH_LAYOUT(256) } else { PB_DISPATCH_LAYOUT(128) }
  return -3;
}
