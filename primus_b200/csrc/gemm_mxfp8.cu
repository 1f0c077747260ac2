// Persistent, warp-specialised MXFP8 GEMM for sm_100a (tcgen05 block-scaled MMA).
//
//   D[M,N] (=|+=) (A . SFA)[M,K] . (B . SFB)[N,K]^T      E4M3 values, one UE8M0 scale per 32 elements of K,
//                                                        fp32 accumulation in tensor memory
//
// * values are staged by TMA (128 bytes = 128 elements of K per row, 128-byte swizzle, no multicast); the
//   scale blocks (512 bytes per 128 rows x 128 K, already in the TMEM layout, see csrc/quant_mxfp8.cu) arrive
//   by plain bulk copies on the same barrier,
// * per stage the MMA thread copies the scales shared memory -> tensor memory (`tcgen05.cp.32x128b.warpx4`)
//   and issues four `tcgen05.mma.kind::mxf8f6f4.block_scale` (128 x BN x 32), selecting the scale byte of
//   each K step through the instruction descriptor,
// * TMEM holds the accumulator(s) plus 4 + BN/32 scale columns: a 128 x 256 tile leaves room for one
//   accumulator only (the producer keeps prefetching the next tile while the epilogue drains it), a 128 x 128
//   tile is double buffered,
// * the epilogue reads the accumulator with tcgen05.ld and writes full lines per row straight from registers;
//   for bf16 output a thread first drains its whole row into packed registers and releases the accumulator, so
//   the global stores overlap the next tile's MMAs (fp32 store / fp32 `red.add` into a main-grad buffer go
//   32 columns at a time).
//
// Operand layouts as in csrc/gemm_bf16.cu: X_MN = 0 -> stored [MN, K] (K contiguous), X_MN = 1 -> stored
// [K, MN] (MN contiguous); the scale tensors are always indexed (mn, k / 32).
//
// Replaces `pt.ops.gemm_fp8` with the MXFP8 recipe / TE MXFP8 GEMMs
// (primus/backends/megatron/core/extensions/primus_turbo.py: float8 linear paths).
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 128;   // fp8 elements = bytes per swizzle row
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int GROUP_M = 16;
enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ADD = 2 };

template <int BN>
struct Cfg {
  static constexpr int ACC_BUFS = (BN == 256) ? 1 : 2;
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = BN * BK;
  static constexpr int SF_BYTES = 512 + (BN / 128) * 512;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;                 // multiple of 1024
  static constexpr int SMEM_BYTES = STAGES * (STAGE_BYTES + SF_BYTES) + 1024 + 256;
  static constexpr int SFA_COL = ACC_BUFS * BN;                         // TMEM column of the A scales
  static constexpr int SFB_COL = SFA_COL + 4;
  static constexpr int TMEM_COLS = 512;
};

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

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& mb, int& nb) {
  const int per_group = GROUP_M * num_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, num_m - first_m);
  const int r = tile - g * per_group;
  mb = first_m + r % gm;
  nb = r / gm;
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          pb::smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(pb::smem_u32(bar))
      : "memory");
}

template <int BN, int A_MN, int B_MN, int OUT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, void* __restrict__ Dv, long ldd,
                  int M, int N, int K, int* status) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_ab = smem;
  uint8_t* smem_sf = smem + STAGES * C::STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(smem_sf + STAGES * C::SF_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = K / BK;
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
    pb::prefetch_tmap(&tmA);
    pb::prefetch_tmap(&tmB);
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
          uint8_t* ssf = smem_sf + stage * C::SF_BYTES;
          pb::mbar_expect_tx(&bars->full[stage], C::STAGE_BYTES + C::SF_BYTES);
          if (A_MN == 0) pb::tma_load_2d(sa, &tmA, &bars->full[stage], kb * BK, m0);
          else pb::tma_load_2d(sa, &tmA, &bars->full[stage], m0, kb * BK);
          if (B_MN == 0) {
            pb::tma_load_2d(sb, &tmB, &bars->full[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 128; ++i)
              pb::tma_load_2d(sb + i * (BK * 128), &tmB, &bars->full[stage], n0 + i * 128, kb * BK);
          }
          bulk_g2s(ssf, sfa + ((long)mb * num_kb + kb) * 512, 512, &bars->full[stage]);
#pragma unroll
          for (int i = 0; i < BN / 128; ++i)
            bulk_g2s(ssf + 512 + i * 512, sfb + ((long)(nb * (BN / 128) + i) * num_kb + kb) * 512, 512,
                     &bars->full[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t sfa_t = tmem_base + C::SFA_COL;
      const uint32_t sfb_t = tmem_base + C::SFB_COL;
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
          const uint32_t ssf = pb::smem_u32(smem_sf + stage * C::SF_BYTES);
          // scales: 32 rows x 16 bytes per 128-row block, 8-row groups 128 bytes apart, no swizzle
          pb::utccp_32x128b_warpx4(sfa_t, pb::make_smem_desc(ssf, 128, 128, 0));
#pragma unroll
          for (int i = 0; i < BN / 128; ++i)
            pb::utccp_32x128b_warpx4(sfb_t + 4 * i, pb::make_smem_desc(ssf + 512 + i * 512, 128, 128, 0));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? pb::make_smem_desc(sa + k * (UMMA_K * 128), BK * 128, 1024, 2)
                                     : pb::make_smem_desc(sa + k * UMMA_K, 0, 1024, 2);
            const uint64_t db = B_MN ? pb::make_smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024, 2)
                                     : pb::make_smem_desc(sb + k * UMMA_K, 0, 1024, 2);
            const uint32_t idesc = pb::make_idesc_mxf8(BM, BN, A_MN, B_MN, k, k);
            pb::umma_mxf8_ss(d_tmem, da, db, idesc, sfa_t | (uint32_t(k) << 30), sfb_t | (uint32_t(k) << 30),
                             (kb > 0 || k > 0) ? 1u : 0u);
          }
          pb::umma_commit(&bars->empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        pb::umma_commit(&bars->tmem_full[acc]);
        if (++acc == C::ACC_BUFS) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    const int lane_grp = warp & 3;
    const int row = lane_grp * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int mb, nb;
      tile_coords(tile, num_m, num_n, mb, nb);
      const int m = mb * BM + row, n0 = nb * BN;
      if (!wait_or_abort(&bars->tmem_full[acc], acc_phase, abort_flag)) {
        atomicCAS(status, 0, PB_ERR_TIMEOUT_EPILOGUE);
        bars->abort_flag = 1;
        ok = false;
        break;
      }
      pb::tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(lane_grp * 32) << 16) + acc * BN;
      if (OUT == OUT_BF16) {
        // drain the whole row into registers as packed bf16 (BN / 2 registers), hand the accumulator back to the
        // MMA thread, and only then write to global memory: the next tile's MMAs overlap the stores
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
        pb::tc_fence_before();
        pb::mbar_arrive(&bars->tmem_empty[acc]);
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
        pb::tc_fence_before();
        pb::mbar_arrive(&bars->tmem_empty[acc]);
      }
      if (++acc == C::ACC_BUFS) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  if (*abort_flag) {
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
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const void* sfa, const void* sfb, void* D, long ldd, int M,
           int N, int K, int* status, int max_ctas, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = gemm_mxfp8_kernel<BN, A_MN, B_MN, OUT>;
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
  kern<<<ctas, NUM_THREADS, C::SMEM_BYTES, stream>>>(tA, tB, reinterpret_cast<const uint8_t*>(sfa),
                                                     reinterpret_cast<const uint8_t*>(sfb), D, ldd, M, N, K, status);
  return (int)cudaGetLastError();
}

}  // namespace

// D[M,N] (=|+=) A . B^T with E4M3 operands and UE8M0 block scales (scale tensors in the 512-byte block layout,
// allocated for M, N rounded up to 128).  lda / ldb: row pitch in bytes of the stored matrices; ldd in elements.
// M, N need no alignment beyond N % 8 (bf16 out) / N % 4 (fp32 out) but the *scale tensors and operand buffers*
// must cover whole 128-row blocks; K % 128 == 0.  out_mode: 0 bf16, 1 fp32, 2 fp32 +=.  block_n: 256 or 128.
extern "C" int pb_gemm_mxfp8(const void* A, const void* SFA, const void* B, const void* SFB, void* D, int M, int N,
                             int K, long lda, long ldb, long ldd, int a_mn, int b_mn, int out_mode, int block_n,
                             int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % BK || (lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A) % 16) ||
      (reinterpret_cast<uintptr_t>(B) % 16) || (reinterpret_cast<uintptr_t>(D) % 16))
    return -2;
  if (out_mode == 0 ? (ldd % 8 || N % 8) : (ldd % 4 || N % 4)) return -2;
  const int BN = (block_n == 128) ? 128 : 256;
  CUtensorMap tA, tB;
  int rc;
  const auto u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  if (!a_mn) rc = pbh::make_tmap_2d(&tA, A, u8, 1, M, K, lda, BM, BK, sw);
  else rc = pbh::make_tmap_2d(&tA, A, u8, 1, K, M, lda, BK, 128, sw);
  if (rc) return rc;
  if (!b_mn) rc = pbh::make_tmap_2d(&tB, B, u8, 1, N, K, ldb, BN, BK, sw);
  else rc = pbh::make_tmap_2d(&tB, B, u8, 1, K, N, ldb, BK, 128, sw);
  if (rc) return rc;

#define PB_DISPATCH_OUT(BN_, AM, BMN)                                                                         \
  switch (out_mode) {                                                                                         \
    case 0: return launch<BN_, AM, BMN, OUT_BF16>(tA, tB, SFA, SFB, D, ldd, M, N, K, status, max_ctas, stream); \
    case 1: return launch<BN_, AM, BMN, OUT_F32>(tA, tB, SFA, SFB, D, ldd, M, N, K, status, max_ctas, stream);  \
    case 2: return launch<BN_, AM, BMN, OUT_F32_ADD>(tA, tB, SFA, SFB, D, ldd, M, N, K, status, max_ctas, stream); \
    default: return -3;                                                                                       \
  }
#define PB_DISPATCH_LAYOUT(BN_)                          \
  if (!a_mn && !b_mn) { PB_DISPATCH_OUT(BN_, 0, 0) }     \
  else if (!a_mn && b_mn) { PB_DISPATCH_OUT(BN_, 0, 1) } \
  else if (a_mn && b_mn) { PB_DISPATCH_OUT(BN_, 1, 1) }  \
  else { PB_DISPATCH_OUT(BN_, 1, 0) }
  if (BN == 256) { PB_DISPATCH_LAYOUT(256) } else { PB_DISPATCH_LAYOUT(128) }
  return -3;
}
