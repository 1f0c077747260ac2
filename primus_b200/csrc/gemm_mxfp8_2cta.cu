// MXFP8 GEMM on CTA pairs (`cta_group::2`): one 256 x 256 output tile per 2-CTA cluster.
//
// Each CTA of the pair stages its own 128 rows of A and only *half* of B (128 of the 256 N columns); one thread of the
// even CTA issues `tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale` with M = 256, which reads both CTAs' shared
// memory and writes 128 accumulator rows into each CTA's tensor memory.  Per CTA and K step the MMA reads 4 KB of A +
// 4 KB of B instead of 4 + 8 KB for a single-CTA 128 x 256 tile: the one-CTA kernel (csrc/gemm_mxfp8.cu) is bound by
// those shared-memory operand reads (12 KB at 64 B / clk = 192 clk per MMA against 131 clk of tensor-pipe time: at most
// 68 % tensor utilisation, 64.6 % measured), the pair needs 128 clk.  No TMA load is multicast: each CTA fetches
// exactly the bytes it keeps.
//
// Warp roles are those of the one-CTA kernel, in both CTAs: warp 0 TMA producer, warp 1 MMA issuer (even CTA only),
// warps 2..5 scale loaders (global -> registers -> `tcgen05.st`: each CTA writes the scales of its own 128 rows of A
// and of all 256 columns of B into its own tensor memory), warps 6..13 epilogue (each CTA drains its 128 rows through
// swizzled staging boxes and TMA stores / reduce-adds).
//
// Synchronisation inside the pair (all waits bounded, errors through the status word):
//   full[stage]      lives in the even CTA: its producer arrives once expecting the bytes of BOTH CTAs; the odd
//                    CTA's TMA loads (`cta_group::2` form) count their bytes on that same barrier;
//   sf_full[slot]    in the even CTA: one arrival per scale warp of both CTAs (the odd CTA's arrive remotely, with a
//                    CTA-scope release: a cluster-scope release per arrival cost ~1000 cycles and halved the kernel).
//                    A slot of the scale ring holds TWO K steps and the ring is 12 K steps deep, twice the operand
//                    ring, because its hand-over crosses the pair twice;
//   sf_empty[slot]   in both CTAs, multicast commit after the slot's second K step;
//   empty[stage]     in both CTAs, released by a multicast `tcgen05.commit` of the MMA thread: frees the stage's
//                    shared memory;
//   tmem_full        in both CTAs, multicast commit after the last K step of a tile;
//   tmem_empty       in the even CTA: one arrival per epilogue warp of both CTAs, as soon as the warp holds its part
//                    of the accumulator in registers (conversion and stores overlap the next tile's MMAs).
// Tensor memory is allocated / freed with the `cta_group::2` forms by the same warp of both CTAs; a cluster
// barrier closes the kernel so that neither CTA exits while its peer may still touch its memory.
//
// Layout conventions and scale-block format as in csrc/gemm_mxfp8.cu / csrc/quant_mxfp8.cu.
#include "common.cuh"

namespace {

constexpr int BM = 128;            // rows per CTA (256 per pair)
constexpr int BN = 256;            // columns per pair; each CTA stages BN / 2 of B
constexpr int BK = 128;
constexpr int UMMA_K = 32;
constexpr int STAGES = 6;
constexpr int SF_WARPS = 4;
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 32 * (2 + SF_WARPS + EPI_WARPS);
constexpr int EPI_BUF_BYTES = 4096;      // per epilogue warp: 32 rows x 128 bytes
constexpr int SF_STEP_COLS = 16;         // TMEM columns per K step: 4 (A) + 8 (B), padded
constexpr int SF_SLOT_COLS = 2 * SF_STEP_COLS;   // a slot of the scale ring holds two K steps: one hand-over
                                         // (wait, tcgen05.st, fence, arrival) per 256 elements of K keeps the scale
                                         // warps ahead of a tensor pipe that needs a K step every ~520 cycles
constexpr int SF_SLOTS = 6;              // the ring is deeper than the operand ring in K steps (12 vs 6): a slot's
                                         // hand-over crosses the pair twice (multicast commit out, remote arrival back)
constexpr int GROUP_M = 8;               // in units of 256-row pair tiles
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = (BN / 2) * BK;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;      // 32 KiB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * EPI_BUF_BYTES + 1024 + 256;
constexpr int SF_COL = BN;               // first TMEM column of the scale ring (one accumulator of BN columns)
constexpr int TMEM_COLS = 512;
static_assert(SF_COL + SF_SLOTS * SF_SLOT_COLS <= TMEM_COLS, "tensor memory");
enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ADD = 2 };

struct Barriers {
  uint64_t full[STAGES];        // used in the even CTA: 1 arrival, transaction bytes of both CTAs
  uint64_t sf_full[SF_SLOTS];   // used in the even CTA: one arrival per scale warp of both CTAs
  uint64_t sf_empty[SF_SLOTS];  // both CTAs (multicast commit): the slot's scales have been consumed
  uint64_t empty[STAGES];       // both CTAs (multicast commit)
  uint64_t tmem_full;           // both CTAs (multicast commit)
  uint64_t tmem_empty;          // used in the even CTA: 2 x EPI_WARPS arrivals
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

// arrival on a barrier of the even CTA from either CTA of the pair
__device__ __forceinline__ void arrive_on_even(uint64_t* bar, uint32_t cta) {
  if (cta == 0) pb::mbar_arrive(bar);
  else pb::mbar_arrive_remote(pb::mapa_shared(bar, 0));
}

template <int A_MN, int B_MN, int OUT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mxfp8_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmD, const uint8_t* __restrict__ sfa,
                       const uint8_t* __restrict__ sfb, int M, int N, int K, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_ab = smem;
  uint8_t* smem_epi = smem + STAGES * STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(smem_epi + EPI_WARPS * EPI_BUF_BYTES);

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
    for (int i = 0; i < SF_SLOTS; ++i) {
      pb::mbar_init(&bars->sf_full[i], 2 * SF_WARPS);
      pb::mbar_init(&bars->sf_empty[i], 1);
    }
    pb::mbar_init(&bars->tmem_full, 1);
    pb::mbar_init(&bars->tmem_empty, 2 * EPI_WARPS);
    bars->abort_flag = 0;
    pb::fence_barrier_init();
    pb::prefetch_tmap(&tmA);
    pb::prefetch_tmap(&tmB);
    pb::prefetch_tmap(&tmD);
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
        const int m0 = (mb * 2 + (int)cta) * BM;         // 128-row block of this CTA
        const int n0 = nb * BN + (int)cta * (BN / 2);    // this CTA's half of the B tile
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->empty[stage], phase ^ 1, abort_flag)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_TMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem_ab + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (cta == 0) pb::mbar_expect_tx(&bars->full[stage], 2 * STAGE_BYTES);
          const uint32_t fb = pb::mapa_shared(&bars->full[stage], 0);   // the even CTA's barrier
          if (A_MN == 0) pb::tma_load_2d_pair(sa, &tmA, fb, kb * BK, m0);
          else pb::tma_load_2d_pair(sa, &tmA, fb, m0, kb * BK);
          if (B_MN == 0) pb::tma_load_2d_pair(sb, &tmB, fb, kb * BK, n0);
          else pb::tma_load_2d_pair(sb, &tmB, fb, n0, kb * BK);
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
      int stage = 0, slot = 0;
      uint32_t phase = 0, sphase = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!wait_or_abort(&bars->tmem_empty, acc_phase ^ 1, abort_flag)) {
          atomicCAS(status, 0, PB_ERR_TIMEOUT_MMA);
          bars->abort_flag = 1;
          break;
        }
        pb::tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->full[stage], phase, abort_flag) ||
              ((kb & 1) == 0 && !wait_or_abort(&bars->sf_full[slot], sphase, abort_flag))) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_MMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          pb::tc_fence_after();
          const uint32_t sa = pb::smem_u32(smem_ab + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          const uint32_t sfa_t = tmem_base + SF_COL + slot * SF_SLOT_COLS + (kb & 1) * SF_STEP_COLS;
          const uint32_t sfb_t = sfa_t + 4;
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
          if ((kb & 1) || kb == num_kb - 1) {        // second K step of the slot (or the tile's odd last step)
            pb::umma_commit_2cta(&bars->sf_empty[slot], 3);
            if (++slot == SF_SLOTS) {
              slot = 0;
              sphase ^= 1;
            }
          }
        }
        if (!ok) break;
        pb::umma_commit_2cta(&bars->tmem_full, 3);
        acc_phase ^= 1;
      }
    }
  } else if (warp < 2 + SF_WARPS) {
    // ------------------------------------------------------------ scale loaders (both CTAs, one warp per lane quarter)
    // Slot layout per stage: columns 0..3 the scales of this CTA's 128 rows of A, 4..7 and 8..11 those of the two
    // 128-column blocks of B (all 256 columns, in both CTAs).  See csrc/gemm_mxfp8.cu for the block format.
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    int stage = 0;           // here: the scale slot
    uint32_t phase = 0;
    bool ok = true;
    // per-tile base pointers of the three scale-block rows (null: the block lies past M / N), recomputed only when the
    // fetch position moves to another tile: the tile decomposition costs two integer divisions
    const uint4 *pa = nullptr, *pb0 = nullptr, *pb1 = nullptr;
    auto set_tile = [&](int tile) {
      int mb, nb;
      tile_coords(tile, num_m, num_n, mb, nb);
      const int mblk = mb * 2 + (int)cta;
      pa = mblk * 128 < M ? reinterpret_cast<const uint4*>(sfa + (long)mblk * num_kb * 512) + lane : nullptr;
      pb0 = (nb * 2) * 128 < N ? reinterpret_cast<const uint4*>(sfb + (long)(nb * 2) * num_kb * 512) + lane : nullptr;
      pb1 = (nb * 2 + 1) * 128 < N ? reinterpret_cast<const uint4*>(sfb + (long)(nb * 2 + 1) * num_kb * 512) + lane : nullptr;
    };
    auto fetch = [&](int kb, uint4* v) {
      const uint4 z = make_uint4(0, 0, 0, 0);
      v[0] = pa ? __ldg(pa + kb * 32) : z;
      v[1] = pb0 ? __ldg(pb0 + kb * 32) : z;
      v[2] = pb1 ? __ldg(pb1 + kb * 32) : z;
    };
    // One iteration handles a slot = two K steps (the second one is empty at the odd end of a tile).  The loads run
    // SF_AHEAD slots ahead of the stores; the loop is unrolled over the register ring (see csrc/gemm_mxfp8.cu).
    constexpr int SF_AHEAD = 2, SF_RING = SF_AHEAD + 1;
    uint4 v[SF_RING][6];
    const int my_tiles = (num_tiles - pair + num_pairs - 1) / num_pairs;
    const int slots_per_tile = (num_kb + 1) / 2;
    const long total = (long)my_tiles * slots_per_tile;
    int tf = pair, sf_ = 0;          // position of the next fetch: tile, slot inside the tile
    long gf = 0;                     // its index
    if (total > 0) set_tile(tf);
    auto fetch_next = [&](uint4* dst) {
      if (gf < total) {
        fetch(2 * sf_, dst);
        if (2 * sf_ + 1 < num_kb) fetch(2 * sf_ + 1, dst + 3);
      }
      ++gf;
      if (++sf_ == slots_per_tile) {
        sf_ = 0;
        tf += num_pairs;
        if (gf < total) set_tile(tf);
      }
    };
#pragma unroll
    for (int j = 0; j < SF_AHEAD; ++j) fetch_next(v[j]);
    for (long g0 = 0; g0 < total && ok; g0 += SF_RING) {
#pragma unroll
      for (int j = 0; j < SF_RING; ++j) {
        if (g0 + j >= total || !ok) break;
        fetch_next(v[(j + SF_AHEAD) % SF_RING]);
        if (!warp_wait_or_abort(&bars->sf_empty[stage], phase ^ 1, abort_flag, lane, 0)) {
          atomicCAS(status, 0, PB_ERR_TIMEOUT_TMA);
          bars->abort_flag = 1;
          ok = false;
          break;
        }
        pb::tc_fence_after();
        const uint32_t slot = tmem_base + lane_addr + SF_COL + stage * SF_SLOT_COLS;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          tmem_st_x4(slot + 4 * i, v[j][i]);
          tmem_st_x4(slot + SF_STEP_COLS + 4 * i, v[j][3 + i]);
        }
        pb::tmem_wait_st();
        pb::tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_on_even(&bars->sf_full[stage], cta);
        if (++stage == SF_SLOTS) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, 128 rows each)
    const int ew = warp - 2 - SF_WARPS;         // 0..7
    const int lane_grp = warp & 3;              // TMEM lane quarter this warp may access
    const int half = ew >> 2;                   // column half of the tile (ew and ew + 4 share a lane quarter)
    constexpr int HC = BN / 2;                  // columns per thread
    constexpr int EB = (OUT == OUT_BF16) ? 2 : 4;
    constexpr int RC = 128 / EB;                // columns per staging round (one 128-byte row)
    uint8_t* ebuf = smem_epi + ew * EPI_BUF_BYTES;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int mb, nb;
      tile_coords(tile, num_m, num_n, mb, nb);
      const int m0 = (mb * 2 + (int)cta) * BM + lane_grp * 32, n0 = nb * BN + half * HC;
      if (!warp_wait_or_abort(&bars->tmem_full, acc_phase, abort_flag, lane, 128)) {
        atomicCAS(status, 0, PB_ERR_TIMEOUT_EPILOGUE);
        bars->abort_flag = 1;
        ok = false;
        break;
      }
      acc_phase ^= 1;
      pb::tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(lane_grp * 32) << 16) + half * HC;
      auto stage_and_store = [&](const uint4* chunks, int n) {
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
        if (lane == 0) arrive_on_even(&bars->tmem_empty, cta);
#pragma unroll
        for (int c = 0; c < HC / RC; ++c) stage_and_store(packed + c * 8, n0 + c * RC);
      } else {
#pragma unroll
        for (int c = 0; c < HC / 64; ++c) {
          uint32_t r[64];
          pb::tmem_ld_32x32b_x32(t_row + c * 64, r);
          pb::tmem_ld_32x32b_x32(t_row + c * 64 + 32, r + 32);
          pb::tmem_wait_ld();
          if (c == HC / 64 - 1) {
            pb::tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_on_even(&bars->tmem_empty, cta);
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
    }
    if (lane == 0) pb::tma_store_wait_all<0>();   // all stores of this warp are complete before the CTA exits
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
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tD, const void* SFA, const void* SFB,
           int M, int N, int K, int* status, int max_ctas, cudaStream_t stream) {
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
  return (int)cudaLaunchKernelEx(&cfg, kern, tA, tB, tD, reinterpret_cast<const uint8_t*>(SFA),
                                 reinterpret_cast<const uint8_t*>(SFB), M, N, K, status);
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
  CUtensorMap tA, tB, tD;
  int rc;
  const auto u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  if (!a_mn) rc = pbh::make_tmap_2d(&tA, A, u8, 1, M, K, lda, BM, BK, sw);
  else rc = pbh::make_tmap_2d(&tA, A, u8, 1, K, M, lda, BK, 128, sw);
  if (rc) return rc;
  if (!b_mn) rc = pbh::make_tmap_2d(&tB, B, u8, 1, N, K, ldb, BN / 2, BK, sw);
  else rc = pbh::make_tmap_2d(&tB, B, u8, 1, K, N, ldb, BK, 128, sw);
  if (rc) return rc;
  // output boxes: 32 rows x 128 bytes (64 bf16 / 32 fp32 columns); rows and columns past M, N are clipped by TMA
  if (out_mode == 0) rc = pbh::make_tmap_2d(&tD, D, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldd, 32, 64, sw);
  else rc = pbh::make_tmap_2d(&tD, D, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldd, 32, 32, sw);
  if (rc) return rc;

#define PB_DISPATCH_OUT(AM, BMN)                                                                                  \
  switch (out_mode) {                                                                                             \
    case 0: return launch<AM, BMN, OUT_BF16>(tA, tB, tD, SFA, SFB, M, N, K, status, max_ctas, stream);            \
    case 1: return launch<AM, BMN, OUT_F32>(tA, tB, tD, SFA, SFB, M, N, K, status, max_ctas, stream);             \
    case 2: return launch<AM, BMN, OUT_F32_ADD>(tA, tB, tD, SFA, SFB, M, N, K, status, max_ctas, stream);         \
    default: return -3;                                                                                           \
  }
  if (!a_mn && !b_mn) { PB_DISPATCH_OUT(0, 0) }
  else if (!a_mn && b_mn) { PB_DISPATCH_OUT(0, 1) }
  else if (a_mn && b_mn) { PB_DISPATCH_OUT(1, 1) }
  else { PB_DISPATCH_OUT(1, 0) }
  return -3;
}
