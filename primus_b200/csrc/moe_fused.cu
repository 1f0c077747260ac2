// Expert-parallel MoE stages fused with their all-to-all over NVSwitch peer memory.
//
//   dispatch + GEMM  : A_local[row] = x_{peer(row)}[token(row)]   (rows pulled from the owners' token buffers)
//                      D[rows, N]   = A_local . W[expert(row block)]^T
//   GEMM + combine   : D[rows, N]   = A . W[e]^T  written to a symmetric buffer; as soon as a 128-row block is
//                      complete a flag is raised in every peer's memory and the token owners pull their
//                      rows into a local buffer laid out by (token, top-k slot) order.
//
// Both are ONE persistent kernel whose grid is split into communication CTAs and GEMM CTAs:
//  * communication CTAs walk a list of row copies in 128-row chunks.  One elected thread keeps a ring of
//    non-multicast bulk async copies in flight (peer global -> shared -> local global), which is what hides
//    the NVLink round trip; padding rows are written as zeros.  In dispatch mode a finished chunk is
//    published through a per-row-block word that the GEMM CTAs' TMA producer waits on (bounded); in combine
//    mode a copy is issued only after the owner of the source row has raised that row block's flag.
//  * GEMM CTAs run the grouped tcgen05 pipeline of csrc/grouped_gemm.cu with row blocks visited in
//    order (n fastest), so that the copies of block k+1 overlap the math of block k.
// Every wait (mbarrier, block word, peer flag) is bounded and reports through the status word; flags
// are epoch based (monotonic) so nothing is cleared between calls.
//
// The routing plan is built on the device without a host round trip (pb_moe_plan_count / pb_moe_plan_assign):
// per-expert counts are exchanged with P2P stores, every source rank then derives the destination row of each
// of its token copies and writes (source rank, token) and the routing probability into the destination's map.
//
// Replaces `fused_mega_moe_stage1/2`, DeepEP dispatch / combine and the all-to-all token dispatcher
// (primus/backends/megatron/core/extensions/primus_turbo.py:2331-2343,
//  primus/backends/megatron/patches/moe_patches/moe_alltoall_dtoh_patches.py:22-85).
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
constexpr int MAX_EP = 8;

// communication CTAs reuse the GEMM CTAs' shared-memory budget: ring | zero row | barriers
constexpr int RING_BYTES = STAGES * STAGE_BYTES;   // 192 KiB
constexpr int ZERO_BYTES = 16384;                  // largest supported row (8192 bf16)
constexpr int MAX_SLOTS = 48;
constexpr int READ_LAG = 4;        // bulk stores that may still be reading their ring slot
constexpr int PUBLISH_LAG = 12;    // stores between the last row of a chunk and its publication
constexpr int MAX_WORKERS = 4;     // copy workers (elected threads with a private ring slice) per communication CTA
constexpr int CHUNK_ROWS = 128;

struct MoeArgs {
  int gather;        // 1: dispatch + GEMM, 0: GEMM + combine
  int ep, rank, epoch, comm_ctas;
  int rows_cap, N, K, num_mb;
  const int* mblock_expert;            // [num_mb] expert of each row block, -1 when unused
  // row-copy list
  int list_len;                        // dispatch: rows_cap (entry i -> local row i); combine: T*k (entry i -> local row i)
  const int* list_src;                 // (peer << 24) | source row, -1: no source (zero row)
  const uint8_t* peer_src[MAX_EP];
  uint8_t* dst;
  int row_bytes;
  // combine only: one float per source row gathered alongside (gradient of the routing probability)
  const float* peer_aux[MAX_EP];
  float* aux_dst;
  int* mb_words;                       // dispatch: [num_mb] epoch of the last completed gather of the block
                                       // combine : [num_mb] tiles finished for the block (returns to 0)
  int* peer_ready[MAX_EP];             // combine: peers' ready tables, [ep][ready_stride]
  const int* local_ready;
  int ready_stride;
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

__device__ __forceinline__ bool wait_word_geq(const int* w, int value) {
  const long long t0 = clock64();
  int v;
  do {
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(w) : "memory");
    if (v >= value) return true;
  } while (clock64() - t0 < PB_WAIT_CYCLES);
  return false;
}

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

// Walks the chunks first, first + stride, ... of the copy list, skipping chunks of unused row blocks.
struct RowCursor {
  int chunk, row, end;  // current chunk, current list index, one past the chunk's last index
  int stride;
  bool valid;
};
__device__ __forceinline__ void cursor_seek(const MoeArgs& a, RowCursor& c) {
  const int chunks = (a.list_len + CHUNK_ROWS - 1) / CHUNK_ROWS;
  while (c.chunk < chunks && a.gather && a.mblock_expert[c.chunk] < 0) c.chunk += c.stride;
  c.valid = c.chunk < chunks;
  c.row = c.chunk * CHUNK_ROWS;
  c.end = min(c.row + CHUNK_ROWS, a.list_len);
}
__device__ __forceinline__ void cursor_next(const MoeArgs& a, RowCursor& c) {
  if (++c.row < c.end) return;
  c.chunk += c.stride;
  cursor_seek(a, c);
}

// One copy worker = one elected thread with a private slice of the ring.  `worker` / `num_workers` number the
// workers of the whole grid; chunk c of the list is handled by worker c % num_workers, so chunks are started
// in list order across the grid.
__device__ void copy_worker(const MoeArgs& a, uint8_t* ring, int nslot, int slot_bytes, uint64_t* bars,
                            const uint8_t* zero, int worker, int num_workers) {
  RowCursor ic{worker, 0, 0, num_workers, false}, rc{worker, 0, 0, num_workers, false};
  cursor_seek(a, ic);
  cursor_seek(a, rc);
  long issued = 0, retired = 0;
  uint64_t phase_mask = 0;
  int ready_key = -1;          // (peer, row block) whose flag was seen last
  bool ok = true;
  // chunks whose last store has been committed but not yet published: (chunk, index of that store)
  int pend_chunk[4];
  long pend_q[4];
  int pend_n = 0;

  auto issue_one = [&]() {
    const int s = a.list_src[ic.row];
    if (s >= 0) {
      const int p = s >> 24, row = s & 0xffffff;
      if (!a.gather) {
        const int key = p * a.ready_stride + (row >> 7);
        if (key != ready_key) {
          if (!pb::wait_flag_geq(a.local_ready + key, a.epoch)) {
            atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
            ok = false;
            return;
          }
          ready_key = key;
        }
      }
      const int slot = (int)(issued % nslot);
      pb::mbar_expect_tx(&bars[slot], a.row_bytes);
      bulk_g2s(ring + (long)slot * slot_bytes, a.peer_src[p] + (long)row * a.row_bytes, a.row_bytes, &bars[slot]);
    }
    ++issued;
    cursor_next(a, ic);
  };
  auto publish = [&](long completed_upto) {  // stores with index <= completed_upto are complete
    int kept = 0;
    for (int i = 0; i < pend_n; ++i) {
      if (pend_q[i] <= completed_upto) {
        __threadfence();
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(a.mb_words + pend_chunk[i]), "r"(a.epoch) : "memory");
      } else {
        pend_chunk[kept] = pend_chunk[i];
        pend_q[kept] = pend_q[i];
        ++kept;
      }
    }
    pend_n = kept;
  };

  // slot reuse needs the store of row (issued - nslot) to have *read* its slot: keep READ_LAG stores unwaited
  const int depth = nslot - READ_LAG - 1;
  while (ok && ic.valid && issued < depth) issue_one();
  while (ok && rc.valid) {
    const int s = a.list_src[rc.row];
    const int slot = (int)(retired % nslot);
    uint8_t* gdst = a.dst + (long)rc.row * a.row_bytes;
    if (s >= 0) {
      if (!pb::mbar_wait(&bars[slot], (uint32_t)((phase_mask >> slot) & 1))) {
        atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
        ok = false;
        break;
      }
      phase_mask ^= (uint64_t(1) << slot);
      bulk_s2g(gdst, ring + (long)slot * slot_bytes, a.row_bytes);
    } else {
      bulk_s2g(gdst, zero, a.row_bytes);
    }
    pb::tma_store_commit();
    pb::tma_store_wait_read<READ_LAG>();
    const long q = retired++;
    if (a.gather) {
      if (rc.row + 1 == rc.end) {
        if (pend_n == 4) {  // only with chunks shorter than the publish lag; drain to stay correct
          pb::tma_store_wait_all<0>();
          publish(q);
        }
        pend_chunk[pend_n] = rc.chunk;
        pend_q[pend_n] = q;
        ++pend_n;
      }
      // a chunk is published PUBLISH_LAG stores after its last one: by then the wait for full completion is free
      if (pend_n && q - pend_q[0] >= PUBLISH_LAG) {
        pb::tma_store_wait_all<PUBLISH_LAG>();
        publish(q - PUBLISH_LAG);
      }
    }
    cursor_next(a, rc);
    if (ic.valid) issue_one();
  }
  pb::tma_store_wait_all<0>();
  if (a.gather && ok) publish(retired);
}

__device__ void comm_main(const MoeArgs& a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* zero = ring + RING_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(zero + ZERO_BYTES);
  const int cta = blockIdx.x;
  const int tid = threadIdx.x;
  const int slot_bytes = (a.row_bytes + 1023) & ~1023;
  // several independent copy workers per CTA when the rows are small (one per warp 0..W-1)
  const int W = max(1, min(MAX_WORKERS, RING_BYTES / (slot_bytes * 12)));
  const int nslot = min(MAX_SLOTS, (RING_BYTES / W) / slot_bytes);
  for (int i = tid; i < a.row_bytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(zero)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    for (int i = 0; i < W * MAX_SLOTS; ++i) pb::mbar_init(&bars[i], 1);
    pb::fence_barrier_init();
  }
  pb::fence_proxy_async_smem();
  __syncthreads();

  const int warp = tid >> 5, lane = tid & 31;
  if (warp < W && lane == 0) {
    copy_worker(a, ring + (long)warp * (RING_BYTES / W), nslot, slot_bytes, bars + warp * MAX_SLOTS, zero,
                cta * W + warp, a.comm_ctas * W);
  } else if (warp == MAX_WORKERS && !a.gather && a.aux_dst != nullptr) {
    // per-row float (probability gradient) of the same copy list, one row per lane
    const int chunks = (a.list_len + CHUNK_ROWS - 1) / CHUNK_ROWS;
    for (int chunk = cta; chunk < chunks; chunk += a.comm_ctas) {
      const int end = min((chunk + 1) * CHUNK_ROWS, a.list_len);
      for (int i = chunk * CHUNK_ROWS + lane; i < end; i += 32) {
        const int s = a.list_src[i];
        float v = 0.f;
        if (s >= 0) {
          const int p = s >> 24, row = s & 0xffffff;
          if (!pb::wait_flag_geq(a.local_ready + p * a.ready_stride + (row >> 7), a.epoch)) {
            atomicCAS(a.status, 0, PB_ERR_TIMEOUT_FLAG);
            break;
          }
          asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(a.peer_aux[p] + row) : "memory");
        }
        a.aux_dst[i] = v;
      }
    }
  }
}


// ------------------------------------------------------------------------------------------------
// B_MN = 0: B [E, N, K] (forward).  B_MN = 1: B [E, K, N] (data gradient).
template <int B_MN>
__global__ void __launch_bounds__(256, 1)
moe_fused_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, const __grid_constant__ MoeArgs a) {
  if (blockIdx.x < a.comm_ctas) {
    comm_main(a);
    return;
  }
  if (threadIdx.x >= GEMM_THREADS) return;
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
  const int num_tiles = a.num_mb * num_n;
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
  pb::named_bar_sync(2, GEMM_THREADS);
  pb::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // tile -> (row block, column block): row blocks in order, n fastest
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ready_mb = -1;
      for (int tile = gemm_cta; tile < num_tiles && ok; tile += num_gemm) {
        const int mb = tile / num_n, nb = tile - mb * num_n;
        const int e = a.mblock_expert[mb];
        if (e < 0) continue;
        if (a.gather && mb != ready_mb) {
          if (!wait_word_geq(a.mb_words + mb, a.epoch)) {
            atomicCAS(status, 0, PB_ERR_TIMEOUT_FLAG);
            bars->abort_flag = 1;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");  // gathered rows were written by bulk stores of other CTAs
          ready_mb = mb;
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
          pb::tma_load_2d(sa, &tmA, &bars->full[stage], kb * BK, m0);
          if (B_MN == 0) {
            pb::tma_load_3d(sb, &tmB, &bars->full[stage], kb * BK, n0, e);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              pb::tma_load_3d(sb + i * (BK * 128), &tmB, &bars->full[stage], n0 + i * 64, kb * BK, e);
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
        const int mb = tile / num_n;
        if (a.mblock_expert[mb] < 0) continue;
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
    for (int tile = gemm_cta; tile < num_tiles && ok; tile += num_gemm) {
      const int mb = tile / num_n, nb = tile - mb * num_n;
      if (a.mblock_expert[mb] < 0) continue;
      const int m0 = mb * BM, n0 = nb * BN;
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
          pb::tma_store_2d(&tmD, stage_buf, n0 + c * 64, m0);
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
      if (!a.gather && et == 0) {
        // the tile must be complete in global memory before the token owners are told about its row block
        pb::tma_store_wait_all<0>();
        __threadfence_system();
        const int done = atomicAdd(a.mb_words + mb, 1) + 1;
        if (done == num_n) {
          atomicExch(a.mb_words + mb, 0);
          __threadfence_system();
          for (int p = 0; p < a.ep; ++p)
            pb::set_flag_release(a.peer_ready[p] + a.rank * a.ready_stride + mb, a.epoch);
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

// ------------------------------------------------------------------------------------------------
// Routing plan.
//
// pb_moe_plan_count : histogram of this rank's expert choices, stored into row `rank` of every peer's
//                     [ep, E] count table; the local source map is reset to -1.
// pb_moe_plan_assign: (after a barrier) one CTA per global expert e.  With all counts known, the destination
//                     rank's padded layout is a pure function of the table, so the source rank computes the
//                     destination row of each of its copies itself:
//                       row = row_start_dest(e) + sum_{src < rank} count[src][e] + (rank of the copy among
//                             this rank's copies of e, in token order)
//                     and writes (rank << 24 | token) and the probability into the destination's map, and
//                     the pull list / inverse permutation used by the combine side locally.  Deterministic:
//                     no atomics decide an order.
constexpr int PLAN_SEG = 2048;   // routing entries per segment (one CTA of the count kernel)

// grid: [0, n_seg) histogram one segment each; the rest reset the source map.  The CTA that finishes last
// publishes the totals to the peers and clears the scratch for the next call.
__global__ void __launch_bounds__(256)
moe_plan_count_kernel(const int* __restrict__ idx, int TK, int E, int ep, int rank, int n_seg,
                      int* __restrict__ seg_counts, int* __restrict__ scratch /* [E + 1] zero */,
                      int* const* peer_counts, int* __restrict__ src_map, int rows_cap) {
  if ((int)blockIdx.x >= n_seg) {
    const int nb = gridDim.x - n_seg;
    for (int i = (blockIdx.x - n_seg) * blockDim.x + threadIdx.x; i < rows_cap; i += nb * blockDim.x) src_map[i] = -1;
    return;
  }
  __shared__ int hist[1024];
  __shared__ int s_last;
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int lo = blockIdx.x * PLAN_SEG, hi = min(lo + PLAN_SEG, TK);
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const int e = idx[i];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    seg_counts[blockIdx.x * E + e] = hist[e];
    if (hist[e]) atomicAdd(scratch + e, hist[e]);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(scratch + E, 1) == n_seg - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int c = atomicExch(scratch + e, 0);
    for (int p = 0; p < ep; ++p) peer_counts[p][rank * E + e] = c;
  }
  if (threadIdx.x == 0) scratch[E] = 0;
}

__device__ __forceinline__ int block_sum_256(int v, int* red) {
  v = __reduce_add_sync(0xffffffffu, v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  int t = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) t += red[i];
  return t;
}

// grid (E, n_seg): CTA (e, seg) places this rank's copies of expert e that lie in segment seg.
__global__ void __launch_bounds__(256)
moe_plan_assign_kernel(const int* __restrict__ idx, const float* __restrict__ probs, int TK, int k, int E, int ep,
                       int rank, const int* __restrict__ counts_all, const int* __restrict__ seg_counts,
                       int* const* peer_src_map, float* const* peer_prob, int rows_cap, int* __restrict__ pull_src,
                       int* __restrict__ inv_order, int* __restrict__ tok_sorted, int* __restrict__ counts_local,
                       int* status) {
  __shared__ int red[8];
  __shared__ int warp_cnt[8];
  const int e = blockIdx.x, seg = blockIdx.y;
  const int e_local = E / ep;
  const int d = e / e_local, le = e - d * e_local;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  int tot_e = 0, base_me = 0;
  for (int s = 0; s < ep; ++s) {
    const int c = counts_all[s * E + e];
    tot_e += c;
    if (s < rank) base_me += c;
  }
  if (seg_counts[seg * E + e] == 0 && !(seg == 0 && d == rank)) return;  // nothing of e in this segment

  int part = 0;
  for (int l2 = tid; l2 < le; l2 += 256) {
    int tot = 0;
    for (int s = 0; s < ep; ++s) tot += counts_all[s * E + d * e_local + l2];
    part += (tot + BM - 1) / BM * BM;
  }
  const int row_start = block_sum_256(part, red);
  part = 0;
  for (int e2 = tid; e2 < e; e2 += 256) part += counts_all[rank * E + e2];
  for (int s2 = tid; s2 < seg; s2 += 256) part += seg_counts[s2 * E + e];
  const int sorted_base = block_sum_256(part, red);     // copies of earlier experts + of e in earlier segments
  part = 0;
  for (int s2 = tid; s2 < seg; s2 += 256) part += seg_counts[s2 * E + e];
  const int seg_base = block_sum_256(part, red);        // copies of e in earlier segments
  const bool fits = row_start + (tot_e + BM - 1) / BM * BM <= rows_cap;
  if (!fits && tid == 0) atomicCAS(status, 0, PB_ERR_CAPACITY);
  if (d == rank && seg == 0 && tid == 0) counts_local[le] = fits ? tot_e : 0;

  int* dst_map = peer_src_map[d];
  float* dst_prob = peer_prob[d];
  int running = 0;
  const int lo = seg * PLAN_SEG, hi = min(lo + PLAN_SEG, TK);
  for (int base = lo; base < hi; base += 256) {
    const int i = base + tid;
    const bool f = (i < hi) && (idx[i] == e);
    const unsigned bal = __ballot_sync(0xffffffffu, f);
    if (lane == 0) warp_cnt[warp] = __popc(bal);
    __syncthreads();
    int woff = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int c = warp_cnt[w];
      if (w < warp) woff += c;
      total += c;
    }
    if (f) {
      const int r = running + woff + __popc(bal & ((1u << lane) - 1u));
      const int row = row_start + base_me + seg_base + r;
      const int s = sorted_base + r;
      const int tok = i / k;
      if (fits) {
        dst_map[row] = (rank << 24) | tok;
        dst_prob[row] = probs[i];
        pull_src[s] = (d << 24) | row;
      } else {
        pull_src[s] = -1;
      }
      inv_order[i] = s;
      tok_sorted[s] = tok;
    }
    running += total;
    __syncthreads();
  }
}

}  // namespace

extern "C" {

int pb_moe_plan_num_segments(int TK) { return (TK + PLAN_SEG - 1) / PLAN_SEG; }

// peer_counts_dev: device array of `ep` pointers (int [ep * E] tables, one per rank).
// seg_counts: int [n_seg * E]; scratch: int [E + 1], zero-initialised once (the kernel leaves it zero).
int pb_moe_plan_count(const int* idx, int TK, int E, int ep, int rank, int* seg_counts, int* scratch,
                      int* const* peer_counts_dev, int* src_map, int rows_cap, cudaStream_t s) {
  if (E > 1024 || ep < 1 || ep > MAX_EP || E % ep || TK < 1) return -2;
  const int n_seg = pb_moe_plan_num_segments(TK);
  moe_plan_count_kernel<<<n_seg + 32, 256, 0, s>>>(idx, TK, E, ep, rank, n_seg, seg_counts, scratch, peer_counts_dev,
                                                   src_map, rows_cap);
  return (int)cudaGetLastError();
}

// peer_src_map_dev / peer_prob_dev: device arrays of `ep` pointers.
int pb_moe_plan_assign(const int* idx, const float* probs, int TK, int k, int E, int ep, int rank,
                       const int* counts_all, const int* seg_counts, int* const* peer_src_map_dev,
                       float* const* peer_prob_dev, int rows_cap, int* pull_src, int* inv_order, int* tok_sorted,
                       int* counts_local, int* status, cudaStream_t s) {
  if (E > 1024 || ep < 1 || ep > MAX_EP || E % ep || rows_cap >= (1 << 24) || TK / k >= (1 << 24)) return -2;
  const int n_seg = pb_moe_plan_num_segments(TK);
  if (n_seg > 65535) return -2;
  moe_plan_assign_kernel<<<dim3(E, n_seg), 256, 0, s>>>(idx, probs, TK, k, E, ep, rank, counts_all, seg_counts,
                                                       peer_src_map_dev, peer_prob_dev, rows_cap, pull_src, inv_order,
                                                       tok_sorted, counts_local, status);
  return (int)cudaGetLastError();
}

// Host launcher of the fused stage.  Pointer tables are host arrays with `ep` valid entries.
//  gather = 1: A = local gather buffer [rows_cap, K] (filled by the kernel from peer_src rows of K bf16),
//              list_src = source map [rows_cap], dst = A, mb_words = int[num_mb] (zero-initialised once).
//  gather = 0: D = this rank's symmetric output [rows_cap, N]; list_src = pull list [list_len]; peer_src = peers'
//              outputs; dst = local [list_len, N]; mb_words = int[num_mb] tile counters (zero between calls).
//  b_mn: B stored [E, K, N] (data gradient) instead of [E, N, K].  epoch: 1, 2, 3, ... per workspace.
int pb_moe_fused(int gather, int b_mn, int ep, int rank, int epoch, int comm_ctas, const void* A, const void* B,
                 void* D, int rows_cap, int N, int K, int E_local, const int* mblock_expert, int list_len,
                 const int* list_src, const long* peer_src, void* dst, const long* peer_aux, float* aux_dst,
                 int* mb_words, const long* peer_ready, const int* local_ready, int ready_stride, int* status,
                 cudaStream_t stream) {
  if (ep < 1 || ep > MAX_EP || rows_cap % BM || K % 8 || N % 8 || comm_ctas < 1) return -2;
  MoeArgs a;
  memset(&a, 0, sizeof(a));
  a.gather = gather; a.ep = ep; a.rank = rank; a.epoch = epoch; a.comm_ctas = comm_ctas;
  a.rows_cap = rows_cap; a.N = N; a.K = K; a.num_mb = rows_cap / BM;
  a.mblock_expert = mblock_expert;
  a.list_len = list_len; a.list_src = list_src;
  a.dst = reinterpret_cast<uint8_t*>(dst);
  a.row_bytes = (gather ? K : N) * 2;
  if (a.row_bytes > ZERO_BYTES || a.row_bytes % 16) return -2;
  for (int r = 0; r < ep; ++r) {
    a.peer_src[r] = reinterpret_cast<const uint8_t*>(peer_src[r]);
    if (peer_aux) a.peer_aux[r] = reinterpret_cast<const float*>(peer_aux[r]);
    if (peer_ready) a.peer_ready[r] = reinterpret_cast<int*>(peer_ready[r]);
  }
  a.aux_dst = peer_aux ? aux_dst : nullptr;
  a.mb_words = mb_words;
  a.local_ready = local_ready;
  a.ready_stride = ready_stride;
  a.status = status;
  if (!gather && a.num_mb > ready_stride) return -2;

  CUtensorMap tA, tB, tD;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  int rc;
  if ((rc = pbh::make_tmap_2d(&tA, A, bf, 2, rows_cap, K, K, BM, BK, sw))) return rc;
  if (!b_mn) rc = pbh::make_tmap_3d(&tB, B, bf, 2, E_local, N, K, K, (long)N * K, 1, BN, BK, sw);
  else rc = pbh::make_tmap_3d(&tB, B, bf, 2, E_local, K, N, N, (long)N * K, 1, BK, 64, sw);
  if (rc) return rc;
  if ((rc = pbh::make_tmap_2d(&tD, D, bf, 2, rows_cap, N, N, BM, 64, sw))) return rc;

  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  static bool attr_set[2] = {false, false};
  auto k0 = moe_fused_kernel<0>;
  auto k1 = moe_fused_kernel<1>;
  if (!attr_set[b_mn ? 1 : 0]) {
    cudaError_t e = cudaFuncSetAttribute(b_mn ? k1 : k0, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[b_mn ? 1 : 0] = true;
  }
  if (comm_ctas > num_sms / 2) comm_ctas = a.comm_ctas = num_sms / 2;
  const int num_n = (N + BN - 1) / BN;
  int gemm_ctas = num_sms - comm_ctas;
  const int tiles = a.num_mb * num_n;
  if (tiles < gemm_ctas) gemm_ctas = tiles;
  const int grid = comm_ctas + gemm_ctas;
  if (b_mn) k1<<<grid, 256, SMEM_BYTES, stream>>>(tA, tB, tD, a);
  else k0<<<grid, 256, SMEM_BYTES, stream>>>(tA, tB, tD, a);
  return (int)cudaGetLastError();
}

}  // extern "C"
