// Tensor-parallel GEMMs fused with their collective over NVSwitch peer memory — one persistent kernel each.
//
//   MODE_AG  (all-gather -> GEMM):   out[T, N] = concat_r(x_r[T/tp, K]) . W[N, K]^T
//   MODE_RS  (GEMM -> reduce-scatter): out[T/tp, N] = sum_r (x_r[T, K] . W_r[N, K]^T)[rows of this rank]
//
// The grid is split into `comm_ctas` communication CTAs and GEMM CTAs that run concurrently:
//
//  AG: communication CTAs pull the peers' activation shards with plain 16-byte P2P loads into a *local*
//      gather buffer, one source rank after the other (own shard first, then rank+1, ...), and publish a
//      per-chunk counter.  GEMM CTAs walk the output tiles in the same chunk order; their TMA producer
//      waits (bounded) for the chunk counter and then loads A tiles from local memory, so every remote
//      byte crosses NVLink exactly once and the transfer of chunk k+1 overlaps the math of chunk k.
//  RS: GEMM CTAs compute the partial product tile by tile in destination order (rank+1 first, own rows
//      last) and write it with TMA into a local symmetric partial buffer; the CTA that completes the
//      last tile of a chunk raises a flag in the destination rank's memory.  Communication CTAs of the
//      destination wait for those flags, pull the peers' partial rows over NVLink as they become ready,
//      accumulate in fp32 and finally add their own partial and write the bf16 result.
//
// No TMA load ever targets peer memory with cluster multicast (none is used at all); peer data is
// moved by ordinary loads of the communication CTAs.  Every wait (mbarrier, chunk counter, peer flag)
// is bounded and reports through the status word.  Flags and counters are epoch based (monotonic), so
// nothing has to be cleared between calls.
//
// Replaces `fused_all_gather_matmul` / `fused_matmul_reduce_scatter`
// (primus/backends/transformer_engine/transformer_engine_torch/comm_overlap.py:408-504) and the plain
// all-gather / reduce-scatter + GEMM pairs of primus/backends/megatron/core/tensor_parallel/layers.py:67-74,158-167.
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int GEMM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BUF_BYTES = BM * 128;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * EPI_BUF_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 2 * BN;
enum { MODE_AG = 0, MODE_RS = 1 };
constexpr int MAX_TP = 8;
constexpr int RS_RING_BYTES = STAGES * STAGE_BYTES + 2 * EPI_BUF_BYTES;  // copy CTAs of the reduce-scatter: ring of slots
constexpr int RS_MAX_SLOTS = 16;                                        // + their barriers in the 256 spare bytes

struct TpArgs {
  int mode, tp, rank, epoch;
  int comm_ctas;
  int rs_group;         // reduce-scatter: sources added per pass (1 .. 4)
  int rows_per_chunk;   // T / tp
  int M, N, K;          // GEMM problem of this rank: A [M, K] (K contiguous), B [N, K] or [K, N]
  // AG: peers' shards [rows_per_chunk, K] and the local gather buffer [M, K]
  const __nv_bfloat16* peer_x[MAX_TP];
  __nv_bfloat16* gather;
  // RS: peers' partial buffers [M, N], fp32 accumulator [rows_per_chunk, N], output [rows_per_chunk, N]
  const __nv_bfloat16* peer_partial[MAX_TP];
  float* acc;
  __nv_bfloat16* out;
  // local monotonic counters: [0,tp) chunk progress (AG: copy CTAs done; RS: tiles done, own slot: copy CTAs whose
  // share of the accumulator is final), [tp,2tp) reads done
  int* counters;
  int tiles_per_chunk;
  // symmetric flags: slot r = "rank r's data is ready for me", slot tp + r = "rank r finished reading mine"
  int* peer_flags[MAX_TP];
  int* local_flags;
  int* status;
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

__device__ __forceinline__ bool wait_counter_geq(const int* ctr, int value) {
  const long long t0 = clock64();
  int v;
  do {
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= value) return true;
  } while (clock64() - t0 < PB_WAIT_CYCLES);
  return false;
}

// chunk processed k-th by this rank
__device__ __forceinline__ int chunk_at(const TpArgs& a, int k) {
  return (a.mode == MODE_AG) ? (a.rank + k) % a.tp : (a.rank + 1 + k) % a.tp;
}

// tile -> (chunk, m-block, n-block): chunk-major, inside a chunk m fastest (A tiles of one n sweep stay in L2)
__device__ __forceinline__ void tile_coords(const TpArgs& a, int tile, int num_n, int& chunk, int& mb, int& nb) {
  const int k = tile / a.tiles_per_chunk;
  const int t = tile - k * a.tiles_per_chunk;
  const int mbc = a.rows_per_chunk / BM;
  chunk = chunk_at(a, k);
  mb = chunk * mbc + t % mbc;
  nb = t / mbc;
}

// ------------------------------------------------------------------------------------------------
// Communication CTAs.  Data moves in 16 KiB pieces through a ring of shared-memory buffers with
// non-multicast bulk async copies (one elected thread keeps up to COMM_NBUF loads in flight, which is
// what hides the NVLink round trip): peer / local global memory -> shared -> local global memory.
constexpr int COMM_PIECE = 16384;
constexpr int COMM_NBUF = 12;
constexpr int COMM_LAG = 3;

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          pb::smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(pb::smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(pb::smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

__device__ void comm_main(const TpArgs& a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* bufs = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(bufs + COMM_NBUF * COMM_PIECE);
  __shared__ int s_ok;
  const int cta = blockIdx.x;
  const int tid = threadIdx.x;
  const int nthr = blockDim.x;
  if (tid == 0) {
    s_ok = 1;
    if (a.mode == MODE_AG) {  // the reduce-scatter lays its own ring (and barriers) over this memory
      for (int i = 0; i < COMM_NBUF; ++i) pb::mbar_init(&bars[i], 1);
      pb::fence_barrier_init();
    }
  }
  __syncthreads();
  // announce: everything this rank produced before the launch is ready for its peers
  if (cta == 0 && tid < a.tp && tid != a.rank && a.mode == MODE_AG) {
    __threadfence_system();
    pb::set_flag_release(a.peer_flags[tid] + a.rank, a.epoch);
  }
  long g = 0;  // running piece index of this CTA (ring slot = g % NBUF, barrier parity = (g / NBUF) & 1)
  if (a.mode == MODE_AG) {
    const long chunk_bytes = (long)a.rows_per_chunk * a.K * 2;
    const long pieces = (chunk_bytes + COMM_PIECE - 1) / COMM_PIECE;
    const long mine = (pieces - cta + a.comm_ctas - 1) / a.comm_ctas;  // pieces cta, cta + comm_ctas, ...
    if (tid == 0) {
      // remote chunks first (the GEMM reads this rank's own shard in place); the own chunk is copied into
      // the gather buffer last, only so that callers get a complete gathered tensor for the weight gradient
      for (int kk = 1; kk <= a.tp; ++kk) {
        const int k = kk % a.tp;
        const int c = chunk_at(a, k);
        if (c != a.rank && !pb::wait_flag_geq(a.local_flags + c, a.epoch)) {
          atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
          break;
        }
        const uint8_t* src = reinterpret_cast<const uint8_t*>(a.peer_x[c]);
        uint8_t* dst = reinterpret_cast<uint8_t*>(a.gather) + (long)c * chunk_bytes;
        auto piece_off = [&](long i) { return ((long)cta + i * a.comm_ctas) * COMM_PIECE; };
        auto piece_len = [&](long i) {
          const long off = piece_off(i);
          return (uint32_t)((chunk_bytes - off) < COMM_PIECE ? (chunk_bytes - off) : COMM_PIECE);
        };
        long issued = 0;
        bool ok = true;
        for (; issued < mine && issued < COMM_NBUF; ++issued) {
          const int slot = (int)((g + issued) % COMM_NBUF);
          pb::mbar_expect_tx(&bars[slot], piece_len(issued));
          bulk_g2s(bufs + slot * COMM_PIECE, src + piece_off(issued), piece_len(issued), &bars[slot]);
        }
        for (long done = 0; done < mine; ++done) {
          const long gi = g + done;
          const int slot = (int)(gi % COMM_NBUF);
          if (!pb::mbar_wait(&bars[slot], (uint32_t)((gi / COMM_NBUF) & 1))) {
            atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
            ok = false;
            break;
          }
          bulk_s2g(dst + piece_off(done), bufs + slot * COMM_PIECE, piece_len(done));
          pb::tma_store_commit();
          pb::tma_store_wait_read<COMM_LAG>();
          if (issued < mine && done >= COMM_LAG) {
            const int fslot = (int)((g + issued) % COMM_NBUF);  // == slot of piece (done - COMM_LAG): its store has read it
            pb::mbar_expect_tx(&bars[fslot], piece_len(issued));
            bulk_g2s(bufs + fslot * COMM_PIECE, src + piece_off(issued), piece_len(issued), &bars[fslot]);
            ++issued;
          }
        }
        if (!ok) break;
        // ring smaller than the lag window: issue what is left (only when mine < NBUF + LAG edge cases)
        pb::tma_store_wait_all<0>();
        g += mine;
        __threadfence();
        atomicAdd(a.counters + c, 1);  // chunk c: one more copy CTA done
        if (c != a.rank) {
          const int fin = atomicAdd(a.counters + a.tp + c, 1) + 1;
          if (fin == a.epoch * a.comm_ctas) pb::set_flag_release(a.peer_flags[c] + a.tp + a.rank, a.epoch);
        }
      }
    }
  } else {
    // reduce-scatter: my rows are [rank * rows_per_chunk, +rows_per_chunk) of every rank's partial buffer.  The copy
    // CTAs add the REMOTE partials into the fp32 accumulator while the GEMM runs; this rank's own tiles of those rows
    // come last in its tile order, and their epilogue adds the accumulator and writes the bf16 result, so nothing
    // is left to do once the GEMM has finished.  The sources are taken in arrival order (rank-1 finishes my rows
    // first) in groups of up to `rs_group` (<= 4): per piece a ring slot receives one bulk copy per source of the group
    // (plus the accumulator piece from the second group on), the threads add them in fp32 and store the sums with
    // ordinary coalesced stores.  tp <= 5 needs one pass, tp = 8 two.
    constexpr int RS_MAXG = 4;
    const int nsrc = a.tp - 1;
    int G = a.rs_group < 1 ? 1 : (a.rs_group > RS_MAXG ? RS_MAXG : a.rs_group);
    if (G > nsrc) G = nsrc;
    const bool multi = nsrc > G;  // several passes: the accumulator piece travels through the slot as well
    const int PIECE = (G == 1) ? 32768 : ((G == 2) ? 16384 : 8192);
    const int slot_bytes = G * PIECE + (multi ? 2 * PIECE : 0);
    int nslot = RS_RING_BYTES / slot_bytes;
    if (nslot > RS_MAX_SLOTS) nslot = RS_MAX_SLOTS;
    uint64_t* rbars = reinterpret_cast<uint64_t*>(bufs + RS_RING_BYTES);
    if (tid == 0) {
      for (int i = 0; i < nslot; ++i) pb::mbar_init(&rbars[i], 1);
      pb::fence_barrier_init();
    }
    __syncthreads();
    const long total_bytes = (long)a.rows_per_chunk * a.N * 2;
    const long row_off_bytes = (long)a.rank * total_bytes;
    const long pieces = (total_bytes + PIECE - 1) / PIECE;
    const long mine = (pieces - cta + a.comm_ctas - 1) / a.comm_ctas;
    auto piece_off = [&](long i) { return ((long)cta + i * a.comm_ctas) * PIECE; };
    auto piece_len = [&](long i) {
      const long off = piece_off(i);
      return (uint32_t)((total_bytes - off) < PIECE ? (total_bytes - off) : PIECE);
    };
    uint8_t* accg = reinterpret_cast<uint8_t*>(a.acc);
    for (int k0 = 1; k0 <= nsrc; k0 += G) {
      const int cnt = (k0 + G - 1 <= nsrc) ? G : (nsrc - k0 + 1);
      const bool has_acc = k0 > 1;
      const uint8_t* srcs[RS_MAXG];
#pragma unroll
      for (int j = 0; j < RS_MAXG; ++j) {
        const int p = (a.rank - (k0 + (j < cnt ? j : 0)) + 2 * a.tp) % a.tp;
        srcs[j] = reinterpret_cast<const uint8_t*>(a.peer_partial[p]) + row_off_bytes;
      }
      if (tid == 0) {
        for (int j = 0; j < cnt; ++j) {
          const int p = (a.rank - (k0 + j) + 2 * a.tp) % a.tp;
          if (!pb::wait_flag_geq(a.local_flags + p, a.epoch)) {
            atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
            s_ok = 0;
            break;
          }
        }
      }
      __syncthreads();
      if (!s_ok) break;
      auto issue_load = [&](long i) {
        const int slot = (int)((g + i) % nslot);
        const uint32_t len = piece_len(i);
        uint8_t* sb = bufs + slot * slot_bytes;
        pb::mbar_expect_tx(&rbars[slot], cnt * len + (has_acc ? 2 * len : 0));
        for (int j = 0; j < cnt; ++j) bulk_g2s(sb + j * PIECE, srcs[j] + piece_off(i), len, &rbars[slot]);
        if (has_acc) bulk_g2s(sb + G * PIECE, accg + 2 * piece_off(i), 2 * len, &rbars[slot]);
      };
      long issued = 0;
      if (tid == 0) {
        asm volatile("fence.proxy.async;" ::: "memory");  // accumulator pieces of the previous pass: ordinary stores
        for (; issued < mine && issued < nslot; ++issued) issue_load(issued);
      }
      for (long done = 0; done < mine; ++done) {
        const long gi = g + done;
        const int slot = (int)(gi % nslot);
        if (!pb::mbar_wait(&rbars[slot], (uint32_t)((gi / nslot) & 1))) {
          atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
          s_ok = 0;
        }
        __syncthreads();
        if (!s_ok) break;
        const int nvec = piece_len(done) / 16;
        const uint8_t* sb = bufs + slot * slot_bytes;
        const float4* sacc = reinterpret_cast<const float4*>(sb + G * PIECE);
        float4* gout = reinterpret_cast<float4*>(accg + 2 * piece_off(done));
        for (int i = tid; i < nvec; i += nthr) {
          float f[8];
          if (has_acc) {
            const float4 a0 = sacc[2 * i], a1 = sacc[2 * i + 1];
            f[0] = a0.x; f[1] = a0.y; f[2] = a0.z; f[3] = a0.w;
            f[4] = a1.x; f[5] = a1.y; f[6] = a1.z; f[7] = a1.w;
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = 0.f;
          }
          for (int sj = 0; sj < cnt; ++sj) {
            const uint4 v = reinterpret_cast<const uint4*>(sb + sj * PIECE)[i];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 t = __bfloat1622float2(h[j]);
              f[2 * j] += t.x;
              f[2 * j + 1] += t.y;
            }
          }
          gout[2 * i] = make_float4(f[0], f[1], f[2], f[3]);
          gout[2 * i + 1] = make_float4(f[4], f[5], f[6], f[7]);
        }
        __syncthreads();  // every thread has read the slot: it can take the next piece
        if (tid == 0 && issued < mine) {
          issue_load(issued);
          ++issued;
        }
      }
      if (!s_ok) break;
      g += mine;
      __threadfence();
      asm volatile("fence.proxy.async;" ::: "memory");  // the next pass reads these sums with bulk copies
      __syncthreads();
      if (tid == 0) {
        for (int j = 0; j < cnt; ++j) {
          const int p = (a.rank - (k0 + j) + 2 * a.tp) % a.tp;
          const int fin = atomicAdd(a.counters + a.tp + p, 1) + 1;
          if (fin == a.epoch * a.comm_ctas) pb::set_flag_release(a.peer_flags[p] + a.tp + a.rank, a.epoch);
        }
      }
    }
    // this CTA's share of the accumulator is final: the epilogue of this rank's own tiles may add it
    __syncthreads();
    if (tid == 0 && s_ok) {
      __threadfence();
      atomicAdd(a.counters + a.rank, 1);
    }
  }
  // leave only when every peer has finished reading this rank's buffers (they may be reused right after)
  if (cta == 0 && tid < a.tp && tid != a.rank) {
    if (!pb::wait_flag_geq(a.local_flags + a.tp + tid, a.epoch)) atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
  }
}

// ------------------------------------------------------------------------------------------------
template <int B_MN>
__global__ void __launch_bounds__(256, 1)
gemm_tp_fused_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmAown,
                     const __grid_constant__ TpArgs a) {
  if (blockIdx.x < a.comm_ctas) {
    comm_main(a);
    return;
  }
  if (threadIdx.x >= GEMM_THREADS) return;  // GEMM CTAs use 6 warps; the block size is shared with comm CTAs
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_ab = smem;
  uint8_t* smem_epi = smem + STAGES * STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(smem_epi + 2 * EPI_BUF_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int gemm_cta = blockIdx.x - a.comm_ctas;
  const int num_gemm = gridDim.x - a.comm_ctas;
  const int num_n = (a.N + BN - 1) / BN;
  const int num_tiles = a.tp * a.tiles_per_chunk;
  const int num_kb = (a.K + BK - 1) / BK;
  volatile int* abort_flag = &bars->abort_flag;
  int* status = a.status;

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
  // named barrier over the 192 GEMM threads (the extra 64 threads of the block have returned)
  pb::named_bar_sync(2, GEMM_THREADS);
  pb::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ready_chunk = -1;
      for (int tile = gemm_cta; tile < num_tiles && ok; tile += num_gemm) {
        int chunk, mb, nb;
        tile_coords(a, tile, num_n, chunk, mb, nb);
        const bool own_chunk = (a.mode == MODE_AG && chunk == a.rank);
        if (a.mode == MODE_AG && chunk != ready_chunk && !own_chunk) {
          if (!wait_counter_geq(a.counters + chunk, a.epoch * a.comm_ctas)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_FLAG);
            bars->abort_flag = 1;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");  // gathered rows were written by ordinary stores
          ready_chunk = chunk;
        }
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->empty[stage], phase ^ 1, abort_flag)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_TMA);
            bars->abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem_ab + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          pb::mbar_expect_tx(&bars->full[stage], STAGE_BYTES);
          if (own_chunk) pb::tma_load_2d(sa, &tmAown, &bars->full[stage], kb * BK, m0 - a.rank * a.rows_per_chunk);
          else pb::tma_load_2d(sa, &tmA, &bars->full[stage], kb * BK, m0);
          if (B_MN == 0) {
            pb::tma_load_2d(sb, &tmB, &bars->full[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              pb::tma_load_2d(sb + i * (BK * 128), &tmB, &bars->full[stage], n0 + i * 64, kb * BK);
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
      constexpr uint32_t idesc = pb::make_idesc_bf16(BM, BN, 0, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = gemm_cta; tile < num_tiles && ok; tile += num_gemm) {
        if (!wait_or_abort(&bars->tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          atomicCAS(status, 0, PB_ERR_TIMEOUT_MMA);
          bars->abort_flag = 1;
          break;
        }
        pb::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
            const uint64_t da = pb::make_smem_desc(sa + k * (UMMA_K * 2), 0, 1024, 2);
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
    constexpr int NUM_CHUNKS = BN / 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    bool ok = true;
    bool acc_ready = false;
    for (int tile = gemm_cta; tile < num_tiles && ok; tile += num_gemm) {
      int chunk, mb, nb;
      tile_coords(a, tile, num_n, chunk, mb, nb);
      const int m0 = mb * BM, n0 = nb * BN;
      // reduce-scatter, this rank's own rows: add the sum of the remote partials and write the final result
      const bool fin = (a.mode == MODE_RS && chunk == a.rank);
      if (fin && !acc_ready) {
        if (et == 0 && !wait_counter_geq(a.counters + a.rank, a.epoch * a.comm_ctas)) {
          atomicCAS(status, 0, PB_ERR_TIMEOUT_FLAG);
          bars->abort_flag = 1;
        }
        pb::named_bar_sync(1, EPI_THREADS);
        if (*abort_flag) break;
        acc_ready = true;
      }
      const float4* acc_row =
          fin ? reinterpret_cast<const float4*>(a.acc + (size_t)(m0 - a.rank * a.rows_per_chunk + row) * a.N + n0) : nullptr;
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
        pb::tmem_ld_32x32b_x32(t_row + c * 64, r);
        pb::tmem_ld_32x32b_x32(t_row + c * 64 + 32, r + 32);
        const bool add = fin && (n0 + c * 64 < a.N);
        float4 av[16];
        if (add) {
#pragma unroll
          for (int j = 0; j < 16; ++j) av[j] = __ldcg(acc_row + c * 16 + j);
        }
        pb::tmem_wait_ld();
        if (add) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            r[4 * j + 0] = __float_as_uint(__uint_as_float(r[4 * j + 0]) + av[j].x);
            r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + av[j].y);
            r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + av[j].z);
            r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + av[j].w);
          }
        }
        if (et == 0) pb::tma_store_wait_read<1>();
        pb::named_bar_sync(1, EPI_THREADS);
        uint8_t* stage_buf = smem_epi + buf * EPI_BUF_BYTES;
        uint8_t* my_row = stage_buf + row * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 v;
          v.x = pb::pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
          v.y = pb::pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
          v.z = pb::pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
          v.w = pb::pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
          *reinterpret_cast<uint4*>(my_row + ((j ^ (row & 7)) << 4)) = v;
        }
        pb::fence_proxy_async_smem();
        pb::named_bar_sync(1, EPI_THREADS);
        if (et == 0) {
          if (fin) pb::tma_store_2d(&tmAown, stage_buf, n0 + c * 64, m0 - a.rank * a.rows_per_chunk);
          else pb::tma_store_2d(&tmD, stage_buf, n0 + c * 64, m0);
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
      if (a.mode == MODE_RS && et == 0 && !fin) {
        // the tile's rows must be complete in global memory before the destination is told about them
        pb::tma_store_wait_all<0>();
        __threadfence_system();
        const int done = atomicAdd(a.counters + chunk, 1) + 1;
        if (done == a.epoch * a.tiles_per_chunk)
          pb::set_flag_release(a.peer_flags[chunk] + a.rank, a.epoch);
      }
    }
    if (et == 0) pb::tma_store_wait_all<0>();
  }

  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  pb::tc_fence_before();
  pb::named_bar_sync(2, GEMM_THREADS);
  if (warp == 1) {
    pb::tc_fence_after();
    pb::tmem_dealloc<1>(tmem_base, TMEM_COLS);
  }
}

}  // namespace

// Host launcher. Pointer tables have `tp` valid entries.
//  mode 0 (AG): A = gather buffer [M = tp*rows_per_chunk, K] (local), D = out [M, N].
//  mode 1 (RS): A = x [M, K] (local), D = this rank's partial buffer [M, N] (symmetric), out = [rows_per_chunk, N].
// b_mn: B stored [K, N].  counters: int[2*tp] local, zero-initialised once.  epoch: 1, 2, 3, ... per buffer set.
extern "C" int pb_gemm_tp_fused(int mode, int tp, int rank, int epoch, int comm_ctas, const void* A, const void* B,
                                void* D, int M, int N, int K, long ldb, int b_mn, const long* peer_x,
                                void* gather, const long* peer_partial, float* acc, void* out, int* counters,
                                const long* peer_flags, int* local_flags, int* status, cudaStream_t stream) {
  if (tp < 2 || tp > MAX_TP || M % tp || (M / tp) % BM || K % 8 || N % 8) return -2;
  TpArgs a;
  memset(&a, 0, sizeof(a));
  a.mode = mode; a.tp = tp; a.rank = rank; a.epoch = epoch; a.comm_ctas = comm_ctas;
  {
    const char* e = getenv("PRIMUS_B200_RS_GROUP");
    a.rs_group = e ? atoi(e) : 4;
  }
  a.rows_per_chunk = M / tp;
  a.M = M; a.N = N; a.K = K;
  for (int r = 0; r < tp; ++r) {
    if (peer_x) a.peer_x[r] = reinterpret_cast<const __nv_bfloat16*>(peer_x[r]);
    if (peer_partial) a.peer_partial[r] = reinterpret_cast<const __nv_bfloat16*>(peer_partial[r]);
    a.peer_flags[r] = reinterpret_cast<int*>(peer_flags[r]);
  }
  a.gather = reinterpret_cast<__nv_bfloat16*>(gather);
  a.acc = acc;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.counters = counters;
  a.local_flags = local_flags;
  a.status = status;
  const int num_n = (N + BN - 1) / BN;
  a.tiles_per_chunk = (a.rows_per_chunk / BM) * num_n;

  CUtensorMap tA, tB, tD;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  int rc;
  if ((rc = pbh::make_tmap_2d(&tA, A, bf, 2, M, K, K, BM, BK, sw))) return rc;
  if (!b_mn) rc = pbh::make_tmap_2d(&tB, B, bf, 2, N, K, ldb, BN, BK, sw);
  else rc = pbh::make_tmap_2d(&tB, B, bf, 2, K, N, ldb, BK, 64, sw);
  if (rc) return rc;
  if ((rc = pbh::make_tmap_2d(&tD, D, bf, 2, M, N, N, BM, 64, sw))) return rc;
  CUtensorMap tAown = tA;
  if (mode == MODE_AG && (rc = pbh::make_tmap_2d(&tAown, reinterpret_cast<const void*>(peer_x[rank]), bf, 2, M / tp, K, K, BM,
                                                  BK, sw)))
    return rc;
  // reduce-scatter: the fourth map is the output [M / tp, N], written by the epilogue of this rank's own tiles
  if (mode == MODE_RS && (rc = pbh::make_tmap_2d(&tAown, out, bf, 2, M / tp, N, N, BM, 64, sw))) return rc;

  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  static bool attr_set[2] = {false, false};
  auto k0 = gemm_tp_fused_kernel<0>;
  auto k1 = gemm_tp_fused_kernel<1>;
  if (!attr_set[b_mn ? 1 : 0]) {
    cudaError_t e = cudaFuncSetAttribute(b_mn ? k1 : k0, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[b_mn ? 1 : 0] = true;
  }
  int gemm_ctas = num_sms - comm_ctas;
  const int tiles = tp * a.tiles_per_chunk;
  if (tiles < gemm_ctas) gemm_ctas = tiles;
  const int grid = comm_ctas + gemm_ctas;
  if (b_mn) k1<<<grid, 256, SMEM_BYTES, stream>>>(tA, tB, tD, tAown, a);
  else k0<<<grid, 256, SMEM_BYTES, stream>>>(tA, tB, tD, tAown, a);
  return (int)cudaGetLastError();
}
