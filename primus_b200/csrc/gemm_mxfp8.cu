// Persistent, warp-specialised MXFP8 GEMM for sm_100a (tcgen05 block-scaled MMA).
//
//   D[M,N] (=|+=) (A . SFA)[M,K] . (B . SFB)[N,K]^T      E4M3 values, one UE8M0 scale per 32 elements of K,
//                                                        fp32 accumulation in tensor memory
//
// Roles of the 14 warps of a CTA (one CTA per SM, 128 x BN output tiles, BK = 128):
//   warp 0        TMA producer: the fp8 values of A and B, 128 bytes of K per row, 128-byte swizzle, no multicast.
//   warp 1        MMA issuer: four `tcgen05.mma.kind::mxf8f6f4.block_scale` (128 x BN x 32) per stage; the scale
//                 byte of each K step is selected through the instruction descriptor.
//   warps 2..5    scale loaders: the 512-byte scale blocks (already in the tensor-memory layout, see
//                 csrc/quant_mxfp8.cu) go global memory -> registers -> tensor memory with `tcgen05.st`, one warp per
//                 TMEM lane quarter, into a ring of scale columns with one slot per pipeline stage.  The scales
//                 never pass through shared memory and no `tcgen05.cp` sits between the MMAs of two stages: in
//                 sustained runs that copy cost 10 % of the tensor pipe's time.
//   warps 6..13   epilogue: two warps per lane quarter, each draining half of the columns.  A thread reads its row
//                 with `tcgen05.ld`, hands the accumulator back, and only then converts / stages the values in
//                 shared memory (one 32-row x 128-byte swizzled box per warp) from where TMA stores them (or adds
//                 them: `cp.reduce.async.bulk.tensor ... add` into an fp32 main-grad buffer).  Whole 128-byte lines
//                 leave the SM; per-lane 16-byte global stores of the same data took 14 % of the kernel at K = 4096
//                 because they compete with the operand loads for the SM's path to L2.
// TMEM: ACC_BUFS accumulators of BN columns + 16 scale columns per stage.  A 128 x 256 tile has one accumulator (the
// MMAs of the next tile start as soon as the eight epilogue warps have read it), a 128 x 128 tile two.
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
constexpr int SF_WARPS = 4;
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 32 * (2 + SF_WARPS + EPI_WARPS);
constexpr int EPI_THREADS = 32 * EPI_WARPS;
constexpr int EPI_BUF_BYTES = 4096;      // per epilogue warp: 32 rows x 128 bytes
constexpr int SF_SLOT_COLS = 16;         // TMEM columns per stage: 4 (A) + up to 8 (B), padded
constexpr int GROUP_M = 16;
enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ADD = 2 };

template <int BN>
struct Cfg {
  static constexpr int ACC_BUFS = (BN == 256) ? 1 : 2;
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = BN * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;                 // multiple of 1024
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * EPI_BUF_BYTES + 1024 + 256;
  static constexpr int SF_COL = ACC_BUFS * BN;                          // first TMEM column of the scale ring
  static constexpr int TMEM_COLS = 512;
  static_assert(SF_COL + STAGES * SF_SLOT_COLS <= 512, "tensor memory");
};

struct Barriers {
  uint64_t full[STAGES];      // operand bytes of a stage have landed (TMA transaction count)
  uint64_t sf_full[STAGES];   // the stage's scales are in tensor memory (one arrival per scale warp)
  uint64_t empty[STAGES];     // the stage's MMAs have completed: shared memory and scale slot are free
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

// Warp-collective wait: lane 0 polls, the other lanes park at the shuffle (no issue slots, no shared-memory traffic).
__device__ __forceinline__ bool warp_wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane,
                                                   unsigned backoff_ns) {
  int got = 1;
  if (lane == 0 && !pb::mbar_try_wait(bar, parity)) {
    const long long t0 = clock64();
    while (!pb::mbar_try_wait(bar, parity)) {
      if (backoff_ns) __nanosleep(backoff_ns);
      if (*abort_flag || clock64() - t0 > PB_WAIT_CYCLES) {
        got = 0;
        break;
      }
    }
  }
  return __shfl_sync(0xffffffffu, got, 0) != 0;
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

__device__ __forceinline__ void tmem_st_x4(uint32_t taddr, const uint4& v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

template <int BN, int A_MN, int B_MN, int OUT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmD, const uint8_t* __restrict__ sfa,
                  const uint8_t* __restrict__ sfb, int M, int N, int K, int* status) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_ab = smem;
  uint8_t* smem_epi = smem + STAGES * C::STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(smem_epi + EPI_WARPS * EPI_BUF_BYTES);

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
      pb::mbar_init(&bars->sf_full[i], SF_WARPS);
      pb::mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      pb::mbar_init(&bars->tmem_full[i], 1);
      pb::mbar_init(&bars->tmem_empty[i], EPI_WARPS);
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
    // ---------------------------------------------------------------- TMA producer
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
          if (A_MN == 0) pb::tma_load_2d(sa, &tmA, &bars->full[stage], kb * BK, m0);
          else pb::tma_load_2d(sa, &tmA, &bars->full[stage], m0, kb * BK);
          if (B_MN == 0) {
            pb::tma_load_2d(sb, &tmB, &bars->full[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 128; ++i)
              pb::tma_load_2d(sb + i * (BK * 128), &tmB, &bars->full[stage], n0 + i * 128, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
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
          if (!wait_or_abort(&bars->full[stage], phase, abort_flag) ||
              !wait_or_abort(&bars->sf_full[stage], phase, abort_flag)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_MMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          pb::tc_fence_after();
          const uint32_t sa = pb::smem_u32(smem_ab + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
          const uint32_t sfa_t = tmem_base + C::SF_COL + stage * SF_SLOT_COLS;
          const uint32_t sfb_t = sfa_t + 4;
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
  } else if (warp < 2 + SF_WARPS) {
    // ---------------------------------------------------------------- scale loaders (one warp per TMEM lane quarter)
    // A 512-byte scale block holds, for 128 rows and 128 elements of K, 16 bytes per lane l: the four scale bytes
    // (K steps 0..3) of rows l, l + 32, l + 64, l + 96.  The same 16 bytes go to lane l of every lane quarter, columns
    // 0..3 of the slot for A and 4 + 4 i .. 7 + 4 i for the i-th 128-column block of B.
    constexpr int NB = BN / 128;
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    auto fetch = [&](int tile, int kb, uint4* v) {
      int mb, nb;
      tile_coords(tile, num_m, num_n, mb, nb);
      v[0] = __ldg(reinterpret_cast<const uint4*>(sfa + ((long)mb * num_kb + kb) * 512) + lane);
#pragma unroll
      for (int i = 0; i < NB; ++i)   // a 128-column block past N has no scales (its MMA columns are never stored)
        v[1 + i] = (nb * NB + i) * 128 < N
                       ? __ldg(reinterpret_cast<const uint4*>(sfb + ((long)(nb * NB + i) * num_kb + kb) * 512) + lane)
                       : make_uint4(0, 0, 0, 0);
    };
    // The loads run SF_AHEAD steps ahead of the stores (their latency is an L2 round trip under full load).  The step
    // loop is unrolled by the ring size so that every register set has a fixed role per unrolled position (a
    // register-to-register rotation would make every step wait for the load it has just issued).
    constexpr int SF_AHEAD = 6, SF_RING = SF_AHEAD + 1;
    uint4 v[SF_RING][1 + NB];
    const int my_tiles = (num_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const long total = (long)my_tiles * num_kb;
    int tf = blockIdx.x, kf = 0;     // position of the next fetch
    long gf = 0;                     // its step index
    auto fetch_next = [&](uint4* dst) {
      if (gf < total) fetch(tf, kf, dst);
      ++gf;
      if (++kf == num_kb) {
        kf = 0;
        tf += gridDim.x;
      }
    };
#pragma unroll
    for (int j = 0; j < SF_AHEAD; ++j) fetch_next(v[j]);
    for (long g0 = 0; g0 < total && ok; g0 += SF_RING) {
#pragma unroll
      for (int j = 0; j < SF_RING; ++j) {
        if (g0 + j >= total || !ok) break;
        fetch_next(v[(j + SF_AHEAD) % SF_RING]);
        if (!warp_wait_or_abort(&bars->empty[stage], phase ^ 1, abort_flag, lane, 0)) {
          atomicCAS(status, 0, PB_ERR_TIMEOUT_TMA);
          bars->abort_flag = 1;
          ok = false;
          break;
        }
        pb::tc_fence_after();
        const uint32_t slot = tmem_base + lane_addr + C::SF_COL + stage * SF_SLOT_COLS;
#pragma unroll
        for (int i = 0; i < 1 + NB; ++i) tmem_st_x4(slot + 4 * i, v[j][i]);
        pb::tmem_wait_st();
        pb::tc_fence_before();
        __syncwarp();
        if (lane == 0) pb::mbar_arrive(&bars->sf_full[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int ew = warp - 2 - SF_WARPS;         // 0..7
    const int lane_grp = warp & 3;              // TMEM lane quarter this warp may access
    const int half = ew >> 2;                   // column half of the tile (ew and ew + 4 share a lane quarter)
    constexpr int HC = BN / 2;                  // columns per thread
    constexpr int EB = (OUT == OUT_BF16) ? 2 : 4;
    constexpr int RC = 128 / EB;                // columns per staging round (one 128-byte row)
    uint8_t* ebuf = smem_epi + ew * EPI_BUF_BYTES;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int mb, nb;
      tile_coords(tile, num_m, num_n, mb, nb);
      const int m0 = mb * BM + lane_grp * 32, n0 = nb * BN + half * HC;
      // one lane polls (with a back-off: the wait spans a whole main loop), the others park at the warp barrier
      if (!warp_wait_or_abort(&bars->tmem_full[acc], acc_phase, abort_flag, lane, 128)) {
        atomicCAS(status, 0, PB_ERR_TIMEOUT_EPILOGUE);
        bars->abort_flag = 1;
        ok = false;
        break;
      }
      pb::tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(lane_grp * 32) << 16) + acc * BN + half * HC;
      auto stage_and_store = [&](const uint4* chunks, int n) {
        // chunks: the 8 16-byte pieces of this thread's 128-byte row of the box
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(ebuf + lane * 128 + ((c ^ (lane & 7)) << 4)) = chunks[c];
        pb::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && m0 < M && n < N) {
          if (OUT == OUT_F32_ADD) pb::tma_reduce_add_2d(&tmD, ebuf, n, m0);
          else pb::tma_store_2d(&tmD, ebuf, n, m0);
          pb::tma_store_commit();
          pb::tma_store_wait_read<0>();    // the staging buffer may be overwritten by the next round
        }
        __syncwarp();
      };
      if (OUT == OUT_BF16) {
        uint4 packed[HC / 8];
#pragma unroll
        for (int c = 0; c < HC / 64; ++c) {
          uint32_t r[64];
          pb::tmem_ld_32x32b_x32(t_row + c * 64, r);
          pb::tmem_ld_32x32b_x32(t_row + c * 64 + 32, r + 32);
          pb::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            packed[c * 8 + j] = make_uint4(pb::pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                                           pb::pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                                           pb::pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                                           pb::pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
        }
        pb::tc_fence_before();
        __syncwarp();
        if (lane == 0) pb::mbar_arrive(&bars->tmem_empty[acc]);
#pragma unroll
        for (int c = 0; c < HC / RC; ++c) stage_and_store(packed + c * 8, n0 + c * RC);
      } else {
        // fp32: 64 columns (two boxes of 32) per load round; the accumulator is handed back once the last round's
        // values are in registers
#pragma unroll
        for (int c = 0; c < HC / 64; ++c) {
          uint32_t r[64];
          pb::tmem_ld_32x32b_x32(t_row + c * 64, r);
          pb::tmem_ld_32x32b_x32(t_row + c * 64 + 32, r + 32);
          pb::tmem_wait_ld();
          if (c == HC / 64 - 1) {
            pb::tc_fence_before();
            __syncwarp();
            if (lane == 0) pb::mbar_arrive(&bars->tmem_empty[acc]);
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint4 ch[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              ch[j] = make_uint4(r[h * 32 + 4 * j], r[h * 32 + 4 * j + 1], r[h * 32 + 4 * j + 2], r[h * 32 + 4 * j + 3]);
            stage_and_store(ch, n0 + c * 64 + h * 32);
          }
        }
      }
      if (++acc == C::ACC_BUFS) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) pb::tma_store_wait_all<0>();   // all stores of this warp are complete before the CTA exits
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
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tD, const void* sfa, const void* sfb,
           int M, int N, int K, int* status, int max_ctas, cudaStream_t stream) {
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
  kern<<<ctas, NUM_THREADS, C::SMEM_BYTES, stream>>>(tA, tB, tD, reinterpret_cast<const uint8_t*>(sfa),
                                                     reinterpret_cast<const uint8_t*>(sfb), M, N, K, status);
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
      (reinterpret_cast<uintptr_t>(B) % 16) || (reinterpret_cast<uintptr_t>(D) % 16) ||
      (reinterpret_cast<uintptr_t>(SFA) % 16) || (reinterpret_cast<uintptr_t>(SFB) % 16))
    return -2;
  if (out_mode == 0 ? (ldd % 8 || N % 8) : (ldd % 4 || N % 4)) return -2;
  const int BN = (block_n == 128) ? 128 : 256;
  CUtensorMap tA, tB, tD;
  int rc;
  const auto u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  if (!a_mn) rc = pbh::make_tmap_2d(&tA, A, u8, 1, M, K, lda, BM, BK, sw);
  else rc = pbh::make_tmap_2d(&tA, A, u8, 1, K, M, lda, BK, 128, sw);
  if (rc) return rc;
  if (!b_mn) rc = pbh::make_tmap_2d(&tB, B, u8, 1, N, K, ldb, BN, BK, sw);
  else rc = pbh::make_tmap_2d(&tB, B, u8, 1, K, N, ldb, BK, 128, sw);
  if (rc) return rc;
  // output boxes: 32 rows x 128 bytes (64 bf16 / 32 fp32 columns); rows and columns past M, N are clipped by TMA
  if (out_mode == 0) rc = pbh::make_tmap_2d(&tD, D, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldd, 32, 64, sw);
  else rc = pbh::make_tmap_2d(&tD, D, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldd, 32, 32, sw);
  if (rc) return rc;

#define PB_DISPATCH_OUT(BN_, AM, BMN)                                                                      \
  switch (out_mode) {                                                                                      \
    case 0: return launch<BN_, AM, BMN, OUT_BF16>(tA, tB, tD, SFA, SFB, M, N, K, status, max_ctas, stream); \
    case 1: return launch<BN_, AM, BMN, OUT_F32>(tA, tB, tD, SFA, SFB, M, N, K, status, max_ctas, stream);  \
    case 2: return launch<BN_, AM, BMN, OUT_F32_ADD>(tA, tB, tD, SFA, SFB, M, N, K, status, max_ctas, stream); \
    default: return -3;                                                                                    \
  }
#define PB_DISPATCH_LAYOUT(BN_)                          \
  if (!a_mn && !b_mn) { PB_DISPATCH_OUT(BN_, 0, 0) }     \
  else if (!a_mn && b_mn) { PB_DISPATCH_OUT(BN_, 0, 1) } \
  else if (a_mn && b_mn) { PB_DISPATCH_OUT(BN_, 1, 1) }  \
  else { PB_DISPATCH_OUT(BN_, 1, 0) }
  if (BN == 256) { PB_DISPATCH_LAYOUT(256) } else { PB_DISPATCH_LAYOUT(128) }
  return -3;
}
