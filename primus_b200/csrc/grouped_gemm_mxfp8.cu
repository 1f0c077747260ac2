// Grouped (per-expert) MXFP8 GEMMs for MoE on tcgen05 block-scaled MMAs, with the expert schedule read from
// device memory (no host synchronisation on the routing result).
//
// Token rows are stored expert-major and padded to 128 per expert as in csrc/grouped_gemm.cu (`row_start`,
// `padded`, `mblock_expert`), so neither a 128-row tile nor a 32-row scale block straddles two experts.
//
//   fprop : D[rows, N]   = A[rows, K]    . W[e]^T     A row-quantised, W [E, N, K] row-quantised (as [E*N, K])
//   dgrad : D[rows, N]   = A[rows, Kred] . W[e]       A row-quantised, W [E, Kred, N] column-quantised (as [E*Kred, N])
//   wgrad : D[e][No, Ko] (=|+=) dy_e^T . x_e          dy [rows, No] and x [rows, Ko] column-quantised (scales along
//                                                      the token dimension); reduction over the expert's rows; fp32
//
// Pipeline of csrc/gemm_mxfp8.cu: TMA 128B-swizzled value stages + bulk copies of 512-byte scale blocks on one
// barrier, `tcgen05.cp` of the scales into tensor memory, four `tcgen05.mma.kind::mxf8f6f4.block_scale`
// (128 x 256 x 32) per stage, one accumulator in tensor memory, register-resident epilogue.
//
// Replaces `pt.ops.grouped_gemm_fp8` (primus/backends/megatron/core/extensions/primus_turbo.py: grouped MLP
// float8 paths).
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = BN * BK;
constexpr int SF_BYTES = 512 + (BN / 128) * 512;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * (STAGE_BYTES + SF_BYTES) + 1024 + 256;
constexpr int SFA_COL = BN;
constexpr int SFB_COL = SFA_COL + 4;
constexpr int TMEM_COLS = 512;

enum { G_FPROP = 0, G_DGRAD = 1, G_WGRAD = 2 };

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full;
  uint64_t tmem_empty;
  uint32_t tmem_base;
  int abort_flag;
};

struct Args {
  const uint8_t* sfa;
  const uint8_t* sfb;
  void* D;
  long ldd;           // elements
  int num_m;          // fprop/dgrad: row blocks in the buffer; wgrad: ceil(No / 128)
  int num_n;          // ceil(N / 256)
  int num_tiles;
  int N;              // columns of D (of D[e] for wgrad)
  int Mrows;          // wgrad: No (rows of D[e]); fprop/dgrad: rows of the token buffer
  int k_blocks;       // fprop/dgrad: reduction blocks of 128
  int E;
  int n_blk128;       // ceil(N / 128): scale blocks per expert along N (fprop), along N (dgrad, wgrad)
  int red_per_e;      // fprop: N (rows of W per expert in the [E*N, K] view); dgrad: Kred; wgrad: unused
  int kb_total;       // wgrad: token row blocks in the buffer; dgrad: E * Kred / 128
  const int* mblock_expert;
  const int* row_start;
  const int* padded;
  int* status;
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

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          pb::smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(pb::smem_u32(bar))
      : "memory");
}

struct Tile {
  int valid;
  int expert;
  int mb, nb;        // output tile (128-row block, 256-column block)
  int k_begin;       // first reduction block (units of 128) in TMA row coordinates of the reduction dimension
  int k_blocks;
};

template <int MODE>
__device__ __forceinline__ Tile get_tile(int tile, const Args& a) {
  Tile t;
  if (MODE != G_WGRAD) {
    t.mb = tile % a.num_m;
    t.nb = tile / a.num_m;
    t.expert = a.mblock_expert[t.mb];
    t.valid = t.expert >= 0;
    t.k_begin = 0;
    t.k_blocks = a.k_blocks;
  } else {
    const int per_e = a.num_m * a.num_n;
    t.expert = tile / per_e;
    const int r = tile - t.expert * per_e;
    t.mb = r % a.num_m;
    t.nb = r / a.num_m;
    t.k_begin = a.row_start[t.expert] / BK;
    t.k_blocks = a.padded[t.expert] / BK;
    t.valid = 1;
  }
  return t;
}

template <int MODE, int OUT_ADD>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const Args a) {
  constexpr int A_MN = (MODE == G_WGRAD) ? 1 : 0;
  constexpr int B_MN = (MODE == G_FPROP) ? 0 : 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_ab = smem;
  uint8_t* smem_sf = smem + STAGES * STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(smem_sf + STAGES * SF_BYTES);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      pb::mbar_init(&bars->full[i], 1);
      pb::mbar_init(&bars->empty[i], 1);
    }
    pb::mbar_init(&bars->tmem_full, 1);
    pb::mbar_init(&bars->tmem_empty, EPI_THREADS);
    bars->abort_flag = 0;
    pb::fence_barrier_init();
    pb::prefetch_tmap(&tmA);
    pb::prefetch_tmap(&tmB);
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
      for (int tile = blockIdx.x; tile < a.num_tiles && ok; tile += gridDim.x) {
        const Tile t = get_tile<MODE>(tile, a);
        if (!t.valid) continue;
        const int m0 = t.mb * BM, n0 = t.nb * BN;
        // scale-block addressing: offset = (mn_block * stride + k_base + kb) * 512
        long sfa_row, sfb_row[BN / 128];
        int sf_kbase;
        if (MODE == G_FPROP) {
          sfa_row = (long)t.mb * a.k_blocks;
          sf_kbase = 0;
#pragma unroll
          for (int i = 0; i < BN / 128; ++i)
            sfb_row[i] = ((long)t.expert * a.n_blk128 + min(t.nb * (BN / 128) + i, a.n_blk128 - 1)) * a.k_blocks;
        } else if (MODE == G_DGRAD) {
          sfa_row = (long)t.mb * a.k_blocks;
          sf_kbase = 0;
#pragma unroll
          for (int i = 0; i < BN / 128; ++i)
            sfb_row[i] = (long)min(t.nb * (BN / 128) + i, a.n_blk128 - 1) * a.kb_total + (long)t.expert * a.k_blocks;
        } else {
          sfa_row = (long)t.mb * a.kb_total;
          sf_kbase = t.k_begin;
#pragma unroll
          for (int i = 0; i < BN / 128; ++i)
            sfb_row[i] = (long)min(t.nb * (BN / 128) + i, a.n_blk128 - 1) * a.kb_total;
        }
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!wait_or_abort(&bars->empty[stage], phase ^ 1, abort_flag)) {
            atomicCAS(a.status, 0, PB_ERR_TIMEOUT_TMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem_ab + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          uint8_t* ssf = smem_sf + stage * SF_BYTES;
          pb::mbar_expect_tx(&bars->full[stage], STAGE_BYTES + SF_BYTES);
          const int kr = (t.k_begin + kb) * BK;
          if (MODE == G_FPROP) {
            pb::tma_load_2d(sa, &tmA, &bars->full[stage], kr, m0);
            pb::tma_load_2d(sb, &tmB, &bars->full[stage], kr, t.expert * a.red_per_e + n0);
          } else if (MODE == G_DGRAD) {
            pb::tma_load_2d(sa, &tmA, &bars->full[stage], kr, m0);
#pragma unroll
            for (int i = 0; i < BN / 128; ++i)
              pb::tma_load_2d(sb + i * (BK * 128), &tmB, &bars->full[stage], n0 + i * 128,
                              t.expert * a.red_per_e + kr);
          } else {
            pb::tma_load_2d(sa, &tmA, &bars->full[stage], m0, kr);
#pragma unroll
            for (int i = 0; i < BN / 128; ++i)
              pb::tma_load_2d(sb + i * (BK * 128), &tmB, &bars->full[stage], n0 + i * 128, kr);
          }
          bulk_g2s(ssf, a.sfa + (sfa_row + sf_kbase + kb) * 512, 512, &bars->full[stage]);
#pragma unroll
          for (int i = 0; i < BN / 128; ++i)
            bulk_g2s(ssf + 512 + i * 512, a.sfb + (sfb_row[i] + sf_kbase + kb) * 512, 512, &bars->full[stage]);
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
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t sfa_t = tmem_base + SFA_COL;
      const uint32_t sfb_t = tmem_base + SFB_COL;
      for (int tile = blockIdx.x; tile < a.num_tiles && ok; tile += gridDim.x) {
        const Tile t = get_tile<MODE>(tile, a);
        if (!t.valid) continue;
        if (!wait_or_abort(&bars->tmem_empty, acc_phase ^ 1, abort_flag)) {
          if (!*abort_flag) atomicCAS(a.status, 0, PB_ERR_TIMEOUT_MMA);
          bars->abort_flag = 1;
          break;
        }
        pb::tc_fence_after();
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!wait_or_abort(&bars->full[stage], phase, abort_flag)) {
            if (!*abort_flag) atomicCAS(a.status, 0, PB_ERR_TIMEOUT_MMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          pb::tc_fence_after();
          const uint32_t sa = pb::smem_u32(smem_ab + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          const uint32_t ssf = pb::smem_u32(smem_sf + stage * SF_BYTES);
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
            pb::umma_mxf8_ss(tmem_base, da, db, idesc, sfa_t | (uint32_t(k) << 30), sfb_t | (uint32_t(k) << 30),
                             (kb > 0 || k > 0) ? 1u : 0u);
          }
          pb::umma_commit(&bars->empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        pb::umma_commit(&bars->tmem_full);
        acc_phase ^= 1;
      }
    }
  } else {
    const int lane_grp = warp & 3;
    const int row = lane_grp * 32 + lane;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < a.num_tiles && ok; tile += gridDim.x) {
      const Tile t = get_tile<MODE>(tile, a);
      if (!t.valid) continue;
      const int m = t.mb * BM + row, n0 = t.nb * BN;
      if (!wait_or_abort(&bars->tmem_full, acc_phase, abort_flag)) {
        if (!*abort_flag) atomicCAS(a.status, 0, PB_ERR_TIMEOUT_EPILOGUE);
        bars->abort_flag = 1;
        ok = false;
        break;
      }
      acc_phase ^= 1;
      pb::tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(lane_grp * 32) << 16);
      if (MODE != G_WGRAD) {
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
        pb::mbar_arrive(&bars->tmem_empty);
        if (m < a.Mrows) {
          __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(a.D) + (long)m * a.ldd + n0;
#pragma unroll
          for (int j = 0; j < BN / 8; ++j)
            if (n0 + 8 * j < a.N)
              reinterpret_cast<uint4*>(d)[j] =
                  make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
        }
      } else {
        const bool empty_acc = (t.k_blocks == 0);   // expert without tokens: the accumulator was never written
        float* dbase = reinterpret_cast<float*>(a.D) + (long)t.expert * a.Mrows * a.ldd;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          pb::tmem_ld_32x32b_x32(t_row + c * 32, r);
          pb::tmem_wait_ld();
          const int n = n0 + c * 32;
          if (m < a.Mrows && n < a.N && !(empty_acc && OUT_ADD)) {
            float* d = dbase + (long)m * a.ldd + n;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (n + 4 * j < a.N) {
                if (!OUT_ADD) {
                  reinterpret_cast<uint4*>(d)[j] = empty_acc ? make_uint4(0u, 0u, 0u, 0u)
                                                             : make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
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
        pb::mbar_arrive(&bars->tmem_empty);
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
    pb::tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

template <int MODE, int OUT_ADD>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const Args& a, cudaStream_t s) {
  auto kern = grouped_gemm_mxfp8_kernel<MODE, OUT_ADD>;
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
  const int ctas = a.num_tiles < num_sms ? a.num_tiles : num_sms;
  kern<<<ctas, NUM_THREADS, SMEM_BYTES, s>>>(tA, tB, a);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

// mode 0 fprop: A [rows_cap, K] e4m3 (row scales SFA), B [E, N, K] e4m3 (row scales SFB over the [E*N, K] view),
//               D [rows_cap, N] bf16
// mode 1 dgrad: A [rows_cap, K] e4m3 (row scales; K is the reduction = the layer's output width), B [E, K, N] e4m3 with
//               column scales over the [E*K, N] view (blocks of 32 along K), D [rows_cap, N] bf16
// mode 2 wgrad: A = dy [rows_cap, N] and B = x [rows_cap, K], both e4m3 with column scales (blocks of 32 rows),
//               D [E, N, K] fp32 (accumulate != 0: +=)
// rows_cap, N, K multiples of 128; every scale tensor in the 512-byte block layout of csrc/quant_mxfp8.cu.
int pb_grouped_gemm_mxfp8(int mode, const void* A, const void* SFA, const void* B, const void* SFB, void* D,
                          int rows_cap, int N, int K, int E, const int* mblock_expert, const int* row_start,
                          const int* padded, int accumulate, int* status, cudaStream_t s) {
  if (rows_cap <= 0 || N <= 0 || K <= 0 || E <= 0) return 0;
  if ((rows_cap % 128) || (N % 128) || (K % 128)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16) ||
      (reinterpret_cast<uintptr_t>(D) % 16))
    return -2;
  CUtensorMap tA, tB;
  const auto u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  int rc;
  Args a;
  a.sfa = reinterpret_cast<const uint8_t*>(SFA);
  a.sfb = reinterpret_cast<const uint8_t*>(SFB);
  a.D = D;
  a.E = E;
  a.mblock_expert = mblock_expert;
  a.row_start = row_start;
  a.padded = padded;
  a.status = status;
  if (mode == G_FPROP) {
    if ((rc = pbh::make_tmap_2d(&tA, A, u8, 1, rows_cap, K, K, BM, BK, sw))) return rc;
    if ((rc = pbh::make_tmap_2d(&tB, B, u8, 1, (long)E * N, K, K, BN, BK, sw))) return rc;
    a.ldd = N; a.N = N; a.Mrows = rows_cap;
    a.num_m = rows_cap / BM; a.num_n = (N + BN - 1) / BN; a.num_tiles = a.num_m * a.num_n;
    a.k_blocks = K / BK; a.n_blk128 = N / 128; a.red_per_e = N; a.kb_total = 0;
    return launch<G_FPROP, 0>(tA, tB, a, s);
  }
  if (mode == G_DGRAD) {
    if ((rc = pbh::make_tmap_2d(&tA, A, u8, 1, rows_cap, K, K, BM, BK, sw))) return rc;
    if ((rc = pbh::make_tmap_2d(&tB, B, u8, 1, (long)E * K, N, N, BK, 128, sw))) return rc;
    a.ldd = N; a.N = N; a.Mrows = rows_cap;
    a.num_m = rows_cap / BM; a.num_n = (N + BN - 1) / BN; a.num_tiles = a.num_m * a.num_n;
    a.k_blocks = K / BK; a.n_blk128 = N / 128; a.red_per_e = K; a.kb_total = E * (K / BK);
    return launch<G_DGRAD, 0>(tA, tB, a, s);
  }
  if (mode == G_WGRAD) {
    if ((rc = pbh::make_tmap_2d(&tA, A, u8, 1, rows_cap, N, N, BK, 128, sw))) return rc;
    if ((rc = pbh::make_tmap_2d(&tB, B, u8, 1, rows_cap, K, K, BK, 128, sw))) return rc;
    a.ldd = K; a.N = K; a.Mrows = N;
    a.num_m = N / BM; a.num_n = (K + BN - 1) / BN; a.num_tiles = E * a.num_m * a.num_n;
    a.k_blocks = 0; a.n_blk128 = K / 128; a.red_per_e = 0; a.kb_total = rows_cap / BK;
    return accumulate ? launch<G_WGRAD, 1>(tA, tB, a, s) : launch<G_WGRAD, 0>(tA, tB, a, s);
  }
  return -3;
}

}  // extern "C"
