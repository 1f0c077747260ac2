// Tensor-parallel GEMMs fused with their collective over NVSwitch peer memory — one persistent kernel each.
//
//   MODE_AG  (all-gather -> GEMM):   out[T, N] = concat_r(x_r[T/tp, K]) . W[N, K]^T
//   MODE_RS  (GEMM -> reduce-scatter): out[T/tp, N] = sum_r (x_r[T, K] . W_r[N, K]^T)[rows of this rank]
//
// The grid is split into `comm_ctas` communication CTAs and GEMM CTAs that run concurrently:
//
//  AG: communication CTAs pull the peers' activation shards with non-multicast bulk copies (peer global ->
//      shared ring -> local global) into a *local* gather buffer, one source rank after the other (own shard
//      first, then rank+1, ...), and publish a per-chunk counter.  GEMM CTAs walk the output tiles in the same chunk order; their TMA producer
//      waits (bounded) for the chunk counter and then loads A tiles from local memory, so every remote
//      byte crosses NVLink exactly once and the transfer of chunk k+1 overlaps the math of chunk k.
//  RS: GEMM CTAs compute the partial product tile by tile in destination order (rank+1 first, own rows
//      last) and write it with TMA into a local symmetric partial buffer; the CTA that completes the
//      last tile of a chunk raises a flag in the destination rank's memory.  Communication CTAs of the
//      destination wait for those flags, pull the peers' partial rows over NVLink in arrival order, sum
//      them (fp32 in registers, pairs of sources per pass) into a bf16 accumulator that is handed over per
//      128-row block, and the GEMM epilogue of the own tiles adds it by TMA and writes the bf16 result.
//
// No TMA load ever targets peer memory with cluster multicast (none is used at all); peer data is
// moved by the communication CTAs (bulk copies without multicast, plain loads for the summing passes).  Every wait (mbarrier, chunk counter, peer flag)
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
constexpr int RS_MAX_SLOTS = 16;
constexpr int MAX_RB = 256;                                             // 128-row blocks per chunk (rows / tp <= 32768)                                        // + their barriers in the 256 spare bytes

struct TpArgs {
  int mode, tp, rank, epoch;
  int comm_ctas;
  int rs_test_repeat;   // test hook (tp = 2 only): the peer's partial product is added twice, in two passes
  int rows_per_chunk;   // T / tp
  int M, N, K;          // GEMM problem of this rank: A [M, K] (K contiguous), B [N, K] or [K, N]
  // AG: peers' shards [rows_per_chunk, K] and the local gather buffer [M, K]
  const __nv_bfloat16* peer_x[MAX_TP];
  __nv_bfloat16* gather;
  // RS: peers' partial buffers [M, N], fp32 accumulator [rows_per_chunk, N], output [rows_per_chunk, N]
  const __nv_bfloat16* peer_partial[MAX_TP];
  __nv_bfloat16* acc;
  __nv_bfloat16* out;
  // local monotonic counters: [0,tp) chunk progress (AG: copy CTAs done; RS: tiles done, own slot: copy CTAs whose
  // share of the accumulator is final), [tp,2tp) reads done
  int* counters;
  int tiles_per_chunk;
  // reduce-scatter, per 128-row block (monotonic over epochs): rb_ready[b] = accumulator pieces of my row block b that are
  // complete; rb_tiles[chunk * MAX_RB + b] = finished tiles of row block b of a remote chunk; published[chunk] = row blocks
  // of that chunk announced to its owner, (epoch - 1) * blocks_per_chunk + count
  int* rb_ready;
  int* rb_tiles;
  int* published;
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
  uint64_t acc_full;   // reduce-scatter: accumulator tile of an own tile has landed in the staging buffer
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

// reduce-scatter: bytes per accumulator piece (one bulk copy per source) for a tensor-parallel size
__host__ __device__ __forceinline__ int rs_piece_bytes(int tp) {
  const int g = tp - 1;
  (void)g;
  return 16384;
}

// chunk processed k-th by this rank
__device__ __forceinline__ int chunk_at(const TpArgs& a, int k) {
  return (a.mode == MODE_AG) ? (a.rank + k) % a.tp : (a.rank + 1 + k) % a.tp;
}

// tile -> (chunk, m-block, n-block): chunk-major; all-gather: inside a chunk m fastest (A tiles of one n sweep stay in L2)
__device__ __forceinline__ void tile_coords(const TpArgs& a, int tile, int num_n, int& chunk, int& mb, int& nb) {
  const int k = tile / a.tiles_per_chunk;
  const int t = tile - k * a.tiles_per_chunk;
  const int mbc = a.rows_per_chunk / BM;
  chunk = chunk_at(a, k);
  if (a.mode == MODE_RS) {  // row-block major: the 128-row blocks of a chunk finish in order and are handed on one by one
    mb = chunk * mbc + t / num_n;
    nb = t - (t / num_n) * num_n;
    return;
  }
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
    // CTAs add the REMOTE partials of those rows into the bf16 accumulator while the GEMM runs; this rank's own tiles of
    // the rows come last in its tile order, and their epilogue adds the accumulator tile and writes the result, so
    // nothing is left to do once the GEMM has finished.  Everything moves in row-block (128 rows) order: a source
    // publishes how many row blocks of my rows it has finished, a piece is fetched as soon as its sources have
    // published its row block, and the epilogue of an own tile waits only for the accumulator pieces of its row block.
    // The sources finish my rows one after the other (rank-1 first, rank+1 after (tp-2)/tp of its GEMM), so they are
    // added in that order, `gs` sources per pass: per piece a ring slot receives one bulk copy per source of the pass
    // plus, from the second pass on, the accumulator piece of the pass before; the threads add them in fp32 into the
    // first copy (a single input needs no arithmetic) and the sum leaves by a bulk store.  Only the last pass -- the
    // last source's share -- is left when the own tiles begin.
    const bool selftest = a.rs_test_repeat && a.tp == 2;   // test hook: the peer's partial is added twice, in two passes
    const int n_in = selftest ? 2 : a.tp - 1;
    const int gs = selftest ? 1 : 2;
    const int PIECE = rs_piece_bytes(a.tp);
    const int max_inputs = (n_in < gs ? n_in : gs) + (n_in > gs ? 1 : 0);
    const int slot_bytes = max_inputs * PIECE;
    int nslot = RS_RING_BYTES / slot_bytes;
    if (nslot > RS_MAX_SLOTS) nslot = RS_MAX_SLOTS;
    uint64_t* rbars = reinterpret_cast<uint64_t*>(bufs + RS_RING_BYTES);
    if (tid == 0) {
      for (int i = 0; i < nslot; ++i) pb::mbar_init(&rbars[i], 1);
      pb::fence_barrier_init();
    }
    __syncthreads();
    const long total_bytes = (long)a.rows_per_chunk * a.N * 2;
    const long rb_bytes = (long)BM * a.N * 2;           // a multiple of PIECE (N % 128 == 0)
    const int mbc = a.rows_per_chunk / BM;
    const int flag_base = (a.epoch - 1) * mbc;
    const long row_off_bytes = (long)a.rank * total_bytes;
    const long pieces = total_bytes / PIECE;
    const long mine = (pieces - cta + a.comm_ctas - 1) / a.comm_ctas;
    auto piece_off = [&](long i) { return ((long)cta + i * a.comm_ctas) * PIECE; };
    uint8_t* accg = reinterpret_cast<uint8_t*>(a.acc);
    const uint8_t* srcs[MAX_TP];
    int src_rank[MAX_TP];
#pragma unroll
    for (int j = 0; j < MAX_TP; ++j) {
      // arrival order: rank-1 does my rows first
      const int p = selftest ? (a.rank ^ 1) : (a.rank - 1 - (j < n_in ? j : 0) + 2 * a.tp) % a.tp;
      src_rank[j] = p;
      srcs[j] = reinterpret_cast<const uint8_t*>(a.peer_partial[p]) + row_off_bytes;
    }
    constexpr int STORE_LAG = 2;
    long gp = 0;  // pieces this CTA has put through the ring in earlier passes (slot and barrier phase continue)
    for (int k0 = 0; k0 < n_in && s_ok; k0 += gs) {
      const int cnt = (k0 + gs <= n_in) ? gs : (n_in - k0);
      const bool has_acc = k0 > 0;
      const bool last = k0 + cnt >= n_in;
      const int n_inputs = cnt + (has_acc ? 1 : 0);
      int rb_known = -1;  // the sources of this pass have published row blocks <= rb_known (thread 0 only)
      // 0: issued; 1: a source has not published the row block yet (only when !blocking); 2: gave up waiting
      auto issue_load = [&](long i, bool blocking) -> int {
        const long off = piece_off(i);
        const int rb = (int)(off / rb_bytes);
        if (rb > rb_known) {
          for (int j = 0; j < cnt; ++j) {
            const int* f = a.local_flags + src_rank[k0 + j];
            if (blocking) {
              if (!pb::wait_flag_geq(f, flag_base + rb + 1)) return 2;
            } else {
              int v;
              asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
              if (v < flag_base + rb + 1) return 1;
            }
          }
          rb_known = rb;
          asm volatile("fence.proxy.async;" ::: "memory");  // the rows were written by the source's TMA stores
        }
        const int slot = (int)((gp + i) % nslot);
        uint8_t* sb = bufs + slot * slot_bytes;
        pb::mbar_expect_tx(&rbars[slot], (uint32_t)(n_inputs * PIECE));
        for (int j = 0; j < cnt; ++j) bulk_g2s(sb + j * PIECE, srcs[k0 + j] + off, PIECE, &rbars[slot]);
        if (has_acc) bulk_g2s(sb + cnt * PIECE, accg + off, PIECE, &rbars[slot]);
        return 0;
      };
      // last pass: accumulator pieces whose bulk store has completed are announced to the epilogue (counter per row
      // block, batched: one fence + one atomic when this CTA's pieces move on to the next row block)
      int ann_rb = -1, ann_cnt = 0;
      auto announce_flush = [&]() {
        if (ann_cnt) {
          __threadfence();
          atomicAdd(a.rb_ready + ann_rb, ann_cnt);
        }
        ann_cnt = 0;
      };
      auto announce = [&](long i) {
        const int rb = (int)(piece_off(i) / rb_bytes);
        if (rb != ann_rb) announce_flush();
        ann_rb = rb;
        ++ann_cnt;
      };
      long issued = 0;
      // issue what the ring can take (the slot of piece i is free once the store of piece i - nslot has read it, i.e.
      // i <= last_read + nslot); wait for a source only if piece `needed` would otherwise not be in flight
      auto top_up = [&](long last_read, long needed) {
        while (issued < mine && issued <= last_read + nslot) {
          const int rc = issue_load(issued, issued <= needed);
          if (rc == 1) break;
          if (rc == 2) {
            atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
            s_ok = 0;
            break;
          }
          ++issued;
        }
      };
      if (tid == 0) top_up(-1, 0);
      __syncthreads();
      // thread 0: store the finished piece, announce older ones, refill the ring
      auto finish_piece = [&](long done, uint8_t* sb) {
        bulk_s2g(accg + piece_off(done), sb, PIECE);
        pb::tma_store_commit();
        pb::tma_store_wait_all<STORE_LAG>();   // stores of pieces <= done - STORE_LAG are complete in global memory
        if (last && done >= STORE_LAG) announce(done - STORE_LAG);
        pb::tma_store_wait_read<1>();          // the stores of pieces <= done - 1 have read their slots
        top_up(done - 1, done + 1);
      };
      if (n_inputs == 1) {
        // a single input: the accumulator is a copy; thread 0 runs the ring alone
        if (tid == 0) {
          for (long done = 0; done < mine && s_ok; ++done) {
            const long gi = gp + done;
            const int slot = (int)(gi % nslot);
            if (!pb::mbar_wait(&rbars[slot], (uint32_t)((gi / nslot) & 1))) {
              atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
              s_ok = 0;
              break;
            }
            finish_piece(done, bufs + slot * slot_bytes);
          }
        }
      } else {
        for (long done = 0; done < mine; ++done) {
          const long gi = gp + done;
          const int slot = (int)(gi % nslot);
          uint8_t* sb = bufs + slot * slot_bytes;
          if (!pb::mbar_wait(&rbars[slot], (uint32_t)((gi / nslot) & 1))) {
            atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
            s_ok = 0;
          }
          __syncthreads();
          if (!s_ok) break;   // uniform: s_ok is only written before this barrier
          uint4* s0 = reinterpret_cast<uint4*>(sb);
          for (int i = tid; i < PIECE / 16; i += nthr) {
            float f[8];
            const uint4 v0 = s0[i];
            {
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v0);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 t = __bfloat1622float2(h[j]);
                f[2 * j] = t.x;
                f[2 * j + 1] = t.y;
              }
            }
            for (int sj = 1; sj < n_inputs; ++sj) {
              const uint4 v = reinterpret_cast<const uint4*>(sb + sj * PIECE)[i];
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 t = __bfloat1622float2(h[j]);
                f[2 * j] += t.x;
                f[2 * j + 1] += t.y;
              }
            }
            uint4 o;
            o.x = pb::pack_bf16x2(f[0], f[1]);
            o.y = pb::pack_bf16x2(f[2], f[3]);
            o.z = pb::pack_bf16x2(f[4], f[5]);
            o.w = pb::pack_bf16x2(f[6], f[7]);
            s0[i] = o;
          }
          pb::fence_proxy_async_smem();
          __syncthreads();
          if (tid == 0) finish_piece(done, sb);
        }
      }
      __syncthreads();
      if (tid == 0) {
        pb::tma_store_wait_all<0>();   // the next pass reads these accumulator pieces back
        if (s_ok && last) {
          for (long i = (mine > STORE_LAG ? mine - STORE_LAG : 0); i < mine; ++i) announce(i);
          announce_flush();
        }
      }
      gp += mine;
      __syncthreads();
    }
    if (tid == 0 && s_ok) {
      for (int j = 0; j < a.tp - 1; ++j) {   // every load from the sources has landed: they may reuse their buffers
        const int p = (a.rank - 1 - j + 2 * a.tp) % a.tp;
        const int fin = atomicAdd(a.counters + a.tp + p, 1) + 1;
        if (fin == a.epoch * a.comm_ctas) pb::set_flag_release(a.peer_flags[p] + a.tp + a.rank, a.epoch);
      }
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
                     const __grid_constant__ CUtensorMap tmAcc, const __grid_constant__ TpArgs a) {
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
    pb::mbar_init(&bars->acc_full, 1);
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
    uint32_t acc_full_phase = 0;
    for (int tile = gemm_cta; tile < num_tiles && ok; tile += num_gemm) {
      int chunk, mb, nb;
      tile_coords(a, tile, num_n, chunk, mb, nb);
      const int m0 = mb * BM, n0 = nb * BN;
      // reduce-scatter, this rank's own rows: add the sum of the remote partials (accumulator tile, fetched by TMA into
      // the staging buffer) and write the final result.  Only the accumulator pieces of this row block must be there.
      const bool fin = (a.mode == MODE_RS && chunk == a.rank);
      if (fin) {
        if (et == 0) {
          const int rb = mb - a.rank * (a.rows_per_chunk / BM);
          const int want = a.epoch * (int)(((long)BM * a.N * 2) / rs_piece_bytes(a.tp));
          if (!wait_counter_geq(a.rb_ready + rb, want)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_FLAG);
            bars->abort_flag = 1;
          }
          asm volatile("fence.proxy.async;" ::: "memory");  // the pieces were written by other SMs' bulk stores
        }
        pb::named_bar_sync(1, EPI_THREADS);
        if (*abort_flag) break;
      }
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
        pb::tmem_wait_ld();
        uint8_t* stage_buf = smem_epi + buf * EPI_BUF_BYTES;
        uint8_t* my_row = stage_buf + row * 128;
        const bool add = fin && (n0 + c * 64 < a.N);
        if (et == 0) {
          pb::tma_store_wait_read<1>();
          if (add) {  // the accumulator tile lands where the result is staged (same 128-byte swizzle)
            pb::mbar_expect_tx(&bars->acc_full, EPI_BUF_BYTES);
            pb::tma_load_2d(stage_buf, &tmAcc, &bars->acc_full, n0 + c * 64, m0 - a.rank * a.rows_per_chunk);
          }
        }
        pb::named_bar_sync(1, EPI_THREADS);
        if (add) {
          if (!wait_or_abort(&bars->acc_full, acc_full_phase, abort_flag)) {
            if (!*abort_flag) atomicCAS(status, 0, PB_ERR_TIMEOUT_EPILOGUE);
            bars->abort_flag = 1;
            ok = false;
          }
          acc_full_phase ^= 1;
          if (ok) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint4 v = *reinterpret_cast<const uint4*>(my_row + ((j ^ (row & 7)) << 4));
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float2 t = __bfloat1622float2(h[u]);
                r[8 * j + 2 * u] = __float_as_uint(__uint_as_float(r[8 * j + 2 * u]) + t.x);
                r[8 * j + 2 * u + 1] = __float_as_uint(__uint_as_float(r[8 * j + 2 * u + 1]) + t.y);
              }
            }
          }
        }
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
        const int mbc = a.rows_per_chunk / BM;
        const int rb = mb - chunk * mbc;
        int* tiles_done = a.rb_tiles + chunk * MAX_RB;
        const int full = a.epoch * num_n;
        if (atomicAdd(tiles_done + rb, 1) + 1 == full) {
          // a row block is complete: extend the published prefix over every complete block that follows it (whoever
          // completes a later block first leaves it to the thread that closes the gap).  Two threads that complete
          // neighbouring blocks at the same time must not both miss the other's count: sequentially consistent fence
          // between the count and the reads below.
          asm volatile("fence.sc.gpu;" ::: "memory");
          const int base = (a.epoch - 1) * mbc;
          for (;;) {
            int p, t;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(p) : "l"(a.published + chunk) : "memory");
            const int k = p - base;
            if (k >= mbc) break;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(t) : "l"(tiles_done + k) : "memory");
            if (t < full) break;
            if (atomicCAS(a.published + chunk, p, p + 1) == p) {
              __threadfence_system();
              asm volatile("red.release.sys.global.max.s32 [%0], %1;" ::"l"(a.peer_flags[chunk] + a.rank), "r"(p + 1)
                           : "memory");
            }
          }
        }
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
// b_mn: B stored [K, N].  counters: int[3 * 8 + 256 + 8 * 256] local, zero-initialised once
// (chunk progress, reads done, published row-block prefixes, accumulator row-block counts, tiles done per row block).  epoch: 1, 2, 3, ... per buffer set.
extern "C" int pb_gemm_tp_fused(int mode, int tp, int rank, int epoch, int comm_ctas, const void* A, const void* B,
                                void* D, int M, int N, int K, long ldb, int b_mn, const long* peer_x,
                                void* gather, const long* peer_partial, void* acc, void* out, int* counters,
                                const long* peer_flags, int* local_flags, int* status, cudaStream_t stream) {
  if (tp < 2 || tp > MAX_TP || M % tp || (M / tp) % BM || K % 8 || N % 8) return -2;
  TpArgs a;
  memset(&a, 0, sizeof(a));
  a.mode = mode; a.tp = tp; a.rank = rank; a.epoch = epoch; a.comm_ctas = comm_ctas;
  {
    static const int rs_test_repeat = [] {          // read once per process: a test hook, not a tuning knob
      const char* e = getenv("PRIMUS_B200_RS_TEST_REPEAT");
      return (e && e[0] == '1') ? 1 : 0;
    }();
    a.rs_test_repeat = rs_test_repeat;
  }
  a.rows_per_chunk = M / tp;
  a.M = M; a.N = N; a.K = K;
  for (int r = 0; r < tp; ++r) {
    if (peer_x) a.peer_x[r] = reinterpret_cast<const __nv_bfloat16*>(peer_x[r]);
    if (peer_partial) a.peer_partial[r] = reinterpret_cast<const __nv_bfloat16*>(peer_partial[r]);
    a.peer_flags[r] = reinterpret_cast<int*>(peer_flags[r]);
  }
  a.gather = reinterpret_cast<__nv_bfloat16*>(gather);
  a.acc = reinterpret_cast<__nv_bfloat16*>(acc);
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.counters = counters;
  a.published = counters + 2 * MAX_TP;
  a.rb_ready = counters + 3 * MAX_TP;
  a.rb_tiles = counters + 3 * MAX_TP + MAX_RB;
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
  // reduce-scatter: the fourth map is the output [M / tp, N], written by the epilogue of this rank's own tiles, the
  // fifth the bf16 accumulator of the same shape, read by it
  CUtensorMap tAcc = tA;
  if (mode == MODE_RS) {
    if (N % 128 || (M / tp) / BM > MAX_RB) return -2;
    if ((rc = pbh::make_tmap_2d(&tAown, out, bf, 2, M / tp, N, N, BM, 64, sw))) return rc;
    if ((rc = pbh::make_tmap_2d(&tAcc, acc, bf, 2, M / tp, N, N, BM, 64, sw))) return rc;
  }

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
  if (b_mn) k1<<<grid, 256, SMEM_BYTES, stream>>>(tA, tB, tD, tAown, tAcc, a);
  else k0<<<grid, 256, SMEM_BYTES, stream>>>(tA, tB, tD, tAown, tAcc, a);
  return (int)cudaGetLastError();
}
