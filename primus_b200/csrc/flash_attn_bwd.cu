// Flash-attention backward for sm_100a.
//
// One templated kernel runs in two modes that share all plumbing:
//   MODE_DKDV: a CTA owns 128 KV rows of one KV head (resident tiles X1 = K, X2 = V) and streams
//              64-row tiles of Q / dO (Y1, Y2) of every query head of the group;
//              S^T = K Q^T, dP^T = V dO^T  ->  P^T, dS^T  ->  dV += P^T dO,  dK += dS^T Q.
//   MODE_DQ  : a CTA owns 128 query rows of one head (X1 = Q, X2 = dO) and streams 64-row tiles of
//              K / V;  S = Q K^T, dP = dO V^T  ->  dS  ->  dQ += dS K.
// In both modes the accumulators live in tensor memory for the whole loop (no atomics, results are
// bit-reproducible), the S / dP tiles are double-buffered in TMEM where capacity allows, and the
// streamed tiles are used twice from one shared-memory copy (K-major operand for the first GEMM,
// MN-major operand for the second).  The softmax threads turn S / dP into bf16 P / dS *in tensor memory*:
// a thread overwrites the first 8 of its own 16 S (dP) columns with the packed pair values, and the second
// GEMM takes its A operand from there (`tcgen05.mma` with A in TMEM), one 16-wide K step per column group.
// Nothing but mbarriers goes through shared memory between the two GEMMs of a step.  The per-step chain of
// a softmax thread (TMEM load -> exp2 / multiply -> TMEM store -> arrive) is latency bound, so two teams of
// 128 threads work on alternating steps (each thread owns one row and all 64 columns of its step) while
// the MMA thread runs two steps ahead.
//
// Replaces the backward of `flash_attn_func` (primus/backends/megatron/core/extensions/
// primus_turbo.py:812-823); deterministic by construction (cf. the `deterministic=` flag there, :805).
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int BR = 128;  // resident rows
constexpr int BC = 64;   // streamed rows per step
constexpr int BW_THREADS = 320;   // warp0 TMA, warp1 MMA, warps 2..9: two softmax teams of 128 threads
constexpr int BW_COMPUTE = 256;
constexpr int BW_TEAMS = 2;       // team t handles steps i = t (mod 2): one thread per resident row, all 64 columns
constexpr int XATOM = 128 * 128;  // bytes of a [128 rows x 64 bf16] atom
constexpr int YATOM = 64 * 128;   // bytes of a [64 rows x 64 bf16] atom
enum { MODE_DKDV = 0, MODE_DQ = 1 };

template <int DQK, int DV, int MODE>
struct BwCfg {
  static constexpr int ACC_COLS = (MODE == MODE_DKDV) ? (DQK + DV) : DQK;
  // S / dP buffers in tensor memory: 3 when they fit next to the accumulators and (MODE_DQ) the TMEM copies of the
  // resident tiles, else 2, else 1.  For the dQ pass of 128-wide heads two buffers + the TMEM operands measured
  // faster (2.217 ms for the whole backward at seq 8192) than three buffers without them (2.260 ms).
  static constexpr int XA_COLS = (MODE == MODE_DQ) ? (DQK / 2 + DV / 2) : 0;
  static constexpr int SBUF = (ACC_COLS + 384 + XA_COLS <= 512) ? 3 : ((ACC_COLS + 256 <= 512) ? 2 : 1);
  // barrier of step i: one per buffer when there are three (steps i and i + 2 of a team can both be in flight), else
  // one per softmax team
  __host__ __device__ static constexpr int bar_idx(int i) { return SBUF == 3 ? i % 3 : (i & 1); }
  __host__ __device__ static constexpr uint32_t bar_parity(int i) { return SBUF == 3 ? ((i / 3) & 1) : ((i >> 1) & 1); }
  // MODE_DQ: when tensor memory has room, the resident tiles (Q, dO) are also kept there as packed bf16 and the first
  // GEMMs of a step (S = Q K^T, dP = dO V^T) take their A operand from tensor memory: a both-operands-in-shared-memory
  // MMA with a 64-wide N tile re-reads 128 x 16 A elements per 32 clocks, three times what shared memory delivers
  static constexpr bool XA = (MODE == MODE_DQ) && (ACC_COLS + SBUF * 128 + DQK / 2 + DV / 2 <= 512);
  static constexpr int XA1_COL = ACC_COLS + SBUF * 128;
  static constexpr int XA2_COL = XA1_COL + DQK / 2;
  static constexpr int X1_BYTES = BR * DQK * 2;
  static constexpr int X2_BYTES = BR * DV * 2;
  static constexpr int Y1_BYTES = BC * DQK * 2;
  static constexpr int Y2_BYTES = BC * DV * 2;
  static constexpr int STAT_BYTES = 512;  // 64 lse + 64 delta
  static constexpr int FIXED_BYTES = X1_BYTES + X2_BYTES + 1024 + 512;
  static constexpr int STAGE_BYTES = Y1_BYTES + Y2_BYTES + STAT_BYTES;
  static constexpr int NS_FIT = (232448 - FIXED_BYTES) / STAGE_BYTES;
  // streamed-tile ring depth: a stage is held from the first GEMM (S/dP) to the last (dK/dQ) of its
  // step, so at least three stages are needed to keep a load in flight behind the running step
  static constexpr int NS = NS_FIT >= 4 ? 4 : (NS_FIT >= 3 ? 3 : 2);
  static constexpr int SMEM_BYTES = FIXED_BYTES + NS * STAGE_BYTES;
};

struct BwBars {
  uint64_t x_full;
  uint64_t y_full[4], y_empty[4];
  uint64_t s_full[3];
  uint64_t p_ready[3]; // per team: P / dS of its current step are in tensor memory (one arrival per warp)
  uint64_t acc_done;   // all MMAs of the CTA have completed
  uint64_t xa_ready;   // resident tiles copied into tensor memory (one arrival per softmax warp)
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ bool bw_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (pb::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!pb::mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > PB_WAIT_CYCLES) return false;
  }
  return true;
}
#define BW_WAIT(bar, parity, code)             \
  if (!bw_wait((bar), (parity), abort_flag)) { \
    atomicCAS(status, 0, (code));              \
    bars->abort_flag = 1;                      \
    ok = false;                                \
    break;                                     \
  }

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          pb::smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(pb::smem_u32(bar))
      : "memory");
}

template <int DQK, int DV, int MODE, bool WIN>
__global__ void __launch_bounds__(BW_THREADS, 1)
flash_attn_bwd_kernel(const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
                      const __grid_constant__ CUtensorMap tmY1, const __grid_constant__ CUtensorMap tmY2,
                      const __grid_constant__ CUtensorMap tmO1, const __grid_constant__ CUtensorMap tmO2,
                      const float* __restrict__ lse, const float* __restrict__ delta, int seq, int seq_k, int q_off,
                      int hq, int hkv, float scale, int causal, int window_arg, float softcap_arg, int* status) {
  const int window = WIN ? window_arg : 0;   // the instantiation without a window carries no code for it
  // softcap > 0: scores were softcap * tanh(scale * s / softcap) in the forward pass
  const float softcap = WIN ? softcap_arg : 0.f;
  const float cap_a = (WIN && softcap > 0.f) ? scale / softcap : 0.f;
  const float cap_b = (WIN && softcap > 0.f) ? softcap / scale : 0.f;
  // seq: query rows per sequence, seq_k: key rows per sequence, q_off: key position of query row 0 (multiple of 128);
  // window > 0 (causal self-attention only): a query sees its last `window` keys, itself included
  using C = BwCfg<DQK, DV, MODE>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* x1_smem = smem;
  uint8_t* x2_smem = x1_smem + C::X1_BYTES;
  uint8_t* y1_smem = x2_smem + C::X2_BYTES;           // NS stages
  uint8_t* y2_smem = y1_smem + C::NS * C::Y1_BYTES;   // NS stages
  float* stat_smem = reinterpret_cast<float*>(y2_smem + C::NS * C::Y2_BYTES);  // NS stages x (64 lse, 64 delta)
  BwBars* bars = reinterpret_cast<BwBars*>(reinterpret_cast<uint8_t*>(stat_smem) + C::NS * C::STAT_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = hq / hkv;
  const int seq_x = (MODE == MODE_DKDV) ? seq_k : seq;   // stationary operand (K, V | Q, dO)
  const int seq_y = (MODE == MODE_DKDV) ? seq : seq_k;   // streamed operand (Q, dO | K, V)
  const int num_rb = seq_x / BR;
  const int num_c = seq_y / BC;
  const int qo = q_off / BC;                              // offset in streamed-tile units
  // grid (heads * batch, row blocks): blocks are issued x-fastest, so all heads of the longest row block start
  // first and the short ones fill the tail (work per block is proportional to the number of streamed tiles)
  const int rb = (MODE == MODE_DKDV) ? blockIdx.y : (num_rb - 1 - blockIdx.y);
  const int nxh = (MODE == MODE_DKDV) ? hkv : hq;
  const int xhead = blockIdx.x % nxh;  // MODE_DKDV: kv head; MODE_DQ: query head
  const int batch = blockIdx.x / nxh;
  const int tok0 = batch * seq_x;
  const int toky0 = batch * seq_y;
  // streamed-tile schedule: MODE_DKDV streams the query tiles at or after this key block, MODE_DQ the key tiles at or
  // before this query block (query row i sits at key position q_off + i)
  const int c_start = (MODE == MODE_DKDV) ? (causal ? max(0, 2 * rb - qo) : 0)
                                          : (window > 0 ? max(0, rb * BR + q_off - window + 1) / BC : 0);
  const int c_end = (MODE == MODE_DKDV)
                        ? (window > 0 ? min(num_c, (rb * BR + BR - 1 + window - 1 - q_off) / BC + 1) : num_c)
                        : (causal ? min(num_c, 2 * rb + 2 + qo) : num_c);
  const int n_per_head = max(0, c_end - c_start);
  const int n_iter = (MODE == MODE_DKDV) ? g * n_per_head : n_per_head;
  volatile int* abort_flag = &bars->abort_flag;
  const float sl2 = scale * 1.4426950408889634f;

  if (threadIdx.x == 0) {
    pb::mbar_init(&bars->x_full, 1);
    for (int i = 0; i < 4; ++i) {
      pb::mbar_init(&bars->y_full[i], 1);
      pb::mbar_init(&bars->y_empty[i], 1);
    }
    for (int i = 0; i < 3; ++i) pb::mbar_init(&bars->s_full[i], 1);
    for (int i = 0; i < 3; ++i) pb::mbar_init(&bars->p_ready[i], BW_COMPUTE / BW_TEAMS / 32);
    pb::mbar_init(&bars->acc_done, 1);
    pb::mbar_init(&bars->xa_ready, BW_COMPUTE / 32);
    bars->abort_flag = 0;
    pb::fence_barrier_init();
  }
  if (warp == 1) {
    pb::tmem_alloc<1>(&bars->tmem_base, 512);
    pb::tmem_relinquish<1>();
  }
  pb::tc_fence_before();
  __syncthreads();
  pb::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_sbuf = tmem_base + C::ACC_COLS;  // [buf][S 64 | dP 64]

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      pb::mbar_expect_tx(&bars->x_full, C::X1_BYTES + C::X2_BYTES);
#pragma unroll
      for (int a = 0; a < DQK / 64; ++a)
        pb::tma_load_3d(x1_smem + a * XATOM, &tmX1, &bars->x_full, a * 64, xhead, tok0 + rb * BR);
#pragma unroll
      for (int a = 0; a < DV / 64; ++a)
        pb::tma_load_3d(x2_smem + a * XATOM, &tmX2, &bars->x_full, a * 64, xhead, tok0 + rb * BR);
      for (int i = 0; i < n_iter && ok; ++i) {
        const int st = i % C::NS;
        const int yhead = (MODE == MODE_DKDV) ? (xhead * g + i / n_per_head) : (xhead / g);
        const int cs = c_start + i % n_per_head;
        BW_WAIT(&bars->y_empty[st], ((i / C::NS) & 1) ^ 1, PB_ERR_TIMEOUT_TMA);
        const uint32_t bytes = C::Y1_BYTES + C::Y2_BYTES + (MODE == MODE_DKDV ? C::STAT_BYTES : 0);
        pb::mbar_expect_tx(&bars->y_full[st], bytes);
#pragma unroll
        for (int a = 0; a < DQK / 64; ++a)
          pb::tma_load_3d(y1_smem + st * C::Y1_BYTES + a * YATOM, &tmY1, &bars->y_full[st], a * 64, yhead,
                          toky0 + cs * BC);
#pragma unroll
        for (int a = 0; a < DV / 64; ++a)
          pb::tma_load_3d(y2_smem + st * C::Y2_BYTES + a * YATOM, &tmY2, &bars->y_full[st], a * 64, yhead,
                          toky0 + cs * BC);
        if (MODE == MODE_DKDV) {
          const long off = ((long)batch * hq + yhead) * seq + cs * BC;
          bulk_load_1d(stat_smem + st * 128, lse + off, 256, &bars->y_full[st]);
          bulk_load_1d(stat_smem + st * 128 + 64, delta + off, 256, &bars->y_full[st]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = pb::make_idesc_bf16(BR, BC, 0, 0);
      constexpr uint32_t idesc_a1 = pb::make_idesc_bf16(BR, DQK, 0, 1);  // acc(DQK) += dS . Y1
      constexpr uint32_t idesc_a2 = pb::make_idesc_bf16(BR, DV, 0, 1);   // acc(DV)  += P  . Y2
      const uint32_t x1a = pb::smem_u32(x1_smem), x2a = pb::smem_u32(x2_smem);
      bool ok = true;
      auto issue_sdp = [&](int i) {
        const int st = i % C::NS;
        const uint32_t y1a = pb::smem_u32(y1_smem + st * C::Y1_BYTES);
        const uint32_t y2a = pb::smem_u32(y2_smem + st * C::Y2_BYTES);
        const uint32_t ts = tmem_sbuf + (i % C::SBUF) * 128;
        if (C::XA) {
#pragma unroll
          for (int k = 0; k < DQK / 16; ++k)
            pb::umma_f16_ts(ts, tmem_base + C::XA1_COL + 8 * k,
                            pb::make_smem_desc(y1a + (k / 4) * YATOM + (k % 4) * 32, 0, 1024, 2), idesc_s, k > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < DV / 16; ++k)
            pb::umma_f16_ts(ts + 64, tmem_base + C::XA2_COL + 8 * k,
                            pb::make_smem_desc(y2a + (k / 4) * YATOM + (k % 4) * 32, 0, 1024, 2), idesc_s, k > 0 ? 1u : 0u);
        } else {
#pragma unroll
          for (int k = 0; k < DQK / 16; ++k)
            pb::umma_f16_ss(ts, pb::make_smem_desc(x1a + (k / 4) * XATOM + (k % 4) * 32, 0, 1024, 2),
                            pb::make_smem_desc(y1a + (k / 4) * YATOM + (k % 4) * 32, 0, 1024, 2), idesc_s,
                            k > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < DV / 16; ++k)
            pb::umma_f16_ss(ts + 64, pb::make_smem_desc(x2a + (k / 4) * XATOM + (k % 4) * 32, 0, 1024, 2),
                            pb::make_smem_desc(y2a + (k / 4) * YATOM + (k % 4) * 32, 0, 1024, 2), idesc_s,
                            k > 0 ? 1u : 0u);
        }
        pb::umma_commit(&bars->s_full[C::bar_idx(i)]);
      };
      // The S / dP GEMMs run SBUF steps ahead.  Step i + SBUF reuses the TMEM buffer of step i; it is issued after
      // the second GEMMs of step i (same thread: the tensor pipe keeps the order), which themselves wait for the
      // softmax threads to have replaced S / dP of step i by P / dS.
      do {
        BW_WAIT(&bars->x_full, 0, PB_ERR_TIMEOUT_MMA);
        if (C::XA) {
          BW_WAIT(&bars->xa_ready, 0, PB_ERR_TIMEOUT_MMA);
          pb::tc_fence_after();
        }
        for (int j = 0; j < C::SBUF && j < n_iter && ok; ++j) {
          BW_WAIT(&bars->y_full[j % C::NS], (j / C::NS) & 1, PB_ERR_TIMEOUT_MMA);
          pb::tc_fence_after();
          issue_sdp(j);
        }
      } while (false);
      for (int i = 0; i < n_iter && ok; ++i) {
        const int st = i % C::NS;
        BW_WAIT(&bars->p_ready[C::bar_idx(i)], C::bar_parity(i), PB_ERR_TIMEOUT_MMA);
        pb::tc_fence_after();
        const uint32_t y1a = pb::smem_u32(y1_smem + st * C::Y1_BYTES);
        const uint32_t y2a = pb::smem_u32(y2_smem + st * C::Y2_BYTES);
        const uint32_t ts = tmem_sbuf + (i % C::SBUF) * 128;
        if (MODE == MODE_DKDV) {
#pragma unroll
          for (int k = 0; k < BC / 16; ++k)   // acc(DV) += P . Y2, A = packed P of K step k (TMEM columns 16k .. 16k+7)
            pb::umma_f16_ts(tmem_base + DQK, ts + 16 * k, pb::make_smem_desc(y2a + k * 2048, YATOM, 1024, 2), idesc_a2,
                            (i > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BC / 16; ++k)     // acc(DQK) += dS . Y1
          pb::umma_f16_ts(tmem_base, ts + 64 + 16 * k, pb::make_smem_desc(y1a + k * 2048, YATOM, 1024, 2), idesc_a1,
                          (i > 0 || k > 0) ? 1u : 0u);
        pb::umma_commit(&bars->y_empty[st]);
        if (i + C::SBUF < n_iter) {
          const int in = i + C::SBUF;
          BW_WAIT(&bars->y_full[in % C::NS], (in / C::NS) & 1, PB_ERR_TIMEOUT_MMA);
          pb::tc_fence_after();
          issue_sdp(in);
        }
      }
      if (ok) pb::umma_commit(&bars->acc_done);
    }
  } else {
    // ------------------------------------------------------------------ softmax-gradient threads
    const int wq = warp & 3;              // TMEM lane quarter of this warp
    const int team = (warp - 2) >> 2;     // 0 / 1: even / odd steps
    const int row = wq * 32 + lane;
    const uint32_t lane_addr = uint32_t(wq * 32) << 16;
    const int row_g = rb * BR + row;
    float lse2_row = 0.f, delta_row = 0.f;
    if (MODE == MODE_DQ) {
      const long off = ((long)batch * hq + xhead) * seq + row_g;
      lse2_row = lse[off];  // already in log2 units
      delta_row = delta[off];
    }
    bool ok = true;
    if (C::XA) {
      // team 0 copies its row of X1 (Q), team 1 its row of X2 (dO) from the 128-byte-swizzled shared tiles into
      // tensor memory: word w of a row (elements 2w, 2w + 1) goes to column w, the layout of a TMEM A operand
      do {
        BW_WAIT(&bars->x_full, 0, PB_ERR_TIMEOUT_EPILOGUE);
        const uint8_t* xs = team == 0 ? x1_smem : x2_smem;
        const int natoms = (team == 0 ? DQK : DV) / 64;
        const uint32_t dst = tmem_base + lane_addr + (team == 0 ? C::XA1_COL : C::XA2_COL);
        for (int a = 0; a < natoms; ++a) {
          uint32_t wds[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 v = *reinterpret_cast<const uint4*>(xs + a * XATOM + row * 128 + ((c ^ (row & 7)) << 4));
            wds[4 * c] = v.x; wds[4 * c + 1] = v.y; wds[4 * c + 2] = v.z; wds[4 * c + 3] = v.w;
          }
          pb::tmem_st_32x32b_x32(dst + 32 * a, wds);
        }
        pb::tmem_wait_st();
        pb::tc_fence_before();
        __syncwarp();
        if (lane == 0) pb::mbar_arrive(&bars->xa_ready);
      } while (false);
    }
    for (int i = team; i < n_iter && ok; i += BW_TEAMS) {
      const int sb = i % C::SBUF;
      const int st = i % C::NS;
      const int cs = c_start + i % n_per_head;
      BW_WAIT(&bars->s_full[C::bar_idx(i)], C::bar_parity(i), PB_ERR_TIMEOUT_EPILOGUE);
      if (MODE == MODE_DKDV) {
        BW_WAIT(&bars->y_full[st], (i / C::NS) & 1, PB_ERR_TIMEOUT_EPILOGUE);  // lse / delta tile visible
      }
      pb::tc_fence_after();
      const uint32_t ts = tmem_sbuf + lane_addr + sb * 128;
      const int cs_rel = (MODE == MODE_DKDV) ? cs + qo : cs - qo;   // streamed tile index in the stationary block's frame
      // largest (query position - key position) inside this tile pair: beyond the window -> element-wise mask
      const int max_diff = (MODE == MODE_DKDV) ? (cs_rel * BC + BC - 1 - rb * BR) : (rb * BR + BR - 1 - cs_rel * BC);
      const bool diag = (causal && (cs_rel >= 2 * rb) && (cs_rel <= 2 * rb + 1)) || (window > 0 && max_diff >= window);
      const float* st_lse = stat_smem + st * 128;
      const float* st_delta = st_lse + 64;
      uint32_t s[BC], dp[BC];
      pb::tmem_ld_32x32b_x32(ts, s);
      pb::tmem_ld_32x32b_x32(ts + 32, s + 32);
      pb::tmem_ld_32x32b_x32(ts + 64, dp);
      pb::tmem_ld_32x32b_x32(ts + 96, dp + 32);
      pb::tmem_wait_ld();
      auto body = [&](auto diag_tag) {
        constexpr bool DIAG = decltype(diag_tag)::value;
#pragma unroll
        for (int kk = 0; kk < BC / 16; ++kk) {   // one 16-wide K step of the second GEMM at a time
          uint32_t pk[8], dsk[8];
#pragma unroll
          for (int e4 = 0; e4 < 16; e4 += 4) {
            const int c = kk * 16 + e4;
            float4 l4 = make_float4(lse2_row, lse2_row, lse2_row, lse2_row);
            float4 d4 = make_float4(delta_row, delta_row, delta_row, delta_row);
            if (MODE == MODE_DKDV) {
              l4 = *reinterpret_cast<const float4*>(st_lse + c);
              d4 = *reinterpret_cast<const float4*>(st_delta + c);
            }
            const float l2[4] = {l4.x, l4.y, l4.z, l4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
            float pv[4], dv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              float sv = __uint_as_float(s[c + u]);
              float dcap = 1.f;
              if (WIN && softcap > 0.f) {
                const float t = pb::fast_tanh(sv * cap_a);
                sv = t * cap_b;                  // = softcap * tanh(scale * s / softcap) / scale
                dcap = 1.f - t * t;              // derivative of the capped score with respect to scale * s
              }
              float p = pb::fast_exp2(fmaf(sv, sl2, -l2[u]));
              if (DIAG) {
                const int col_g = cs_rel * BC + c + u;
                const int diff = (MODE == MODE_DKDV) ? (col_g - row_g) : (row_g - col_g);   // query - key position
                if (diff < 0 || (window > 0 && diff >= window)) p = 0.f;
              }
              pv[u] = p;
              dv[u] = p * (__uint_as_float(dp[c + u]) - dl[u]) * scale * dcap;
            }
            pk[e4 / 2] = pb::pack_bf16x2(pv[0], pv[1]);
            pk[e4 / 2 + 1] = pb::pack_bf16x2(pv[2], pv[3]);
            dsk[e4 / 2] = pb::pack_bf16x2(dv[0], dv[1]);
            dsk[e4 / 2 + 1] = pb::pack_bf16x2(dv[2], dv[3]);
          }
          // P / dS (bf16 pairs) replace the first 8 of the 16 S / dP columns of this K step
          if (MODE == MODE_DKDV) pb::tmem_st_32x32b_x8(ts + 16 * kk, pk);
          pb::tmem_st_32x32b_x8(ts + 64 + 16 * kk, dsk);
        }
      };
      if (diag) body(std::true_type{}); else body(std::false_type{});
      pb::tmem_wait_st();
      pb::tc_fence_before();
      __syncwarp();
      if (lane == 0) pb::mbar_arrive(&bars->p_ready[C::bar_idx(i)]);   // one arrival per warp
    }
    // ---- epilogue: accumulators -> bf16 -> (dead) resident tiles -> TMA store
    do {
      if (!ok) break;
      BW_WAIT(&bars->acc_done, 0, PB_ERR_TIMEOUT_EPILOGUE);
      pb::tc_fence_after();
      auto drain = [&](uint32_t tcol, int ncols, uint8_t* dst) {
#pragma unroll 1
        for (int c = team; c < ncols / 32; c += BW_TEAMS) {
          uint32_t r[32];
          pb::tmem_ld_32x32b_x32(tmem_base + lane_addr + tcol + c * 32, r);
          pb::tmem_wait_ld();
          uint8_t* atom = dst + (c >> 1) * XATOM + row * 128;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 v;
            v.x = pb::pack_bf16x2(__uint_as_float(r[8 * q4 + 0]), __uint_as_float(r[8 * q4 + 1]));
            v.y = pb::pack_bf16x2(__uint_as_float(r[8 * q4 + 2]), __uint_as_float(r[8 * q4 + 3]));
            v.z = pb::pack_bf16x2(__uint_as_float(r[8 * q4 + 4]), __uint_as_float(r[8 * q4 + 5]));
            v.w = pb::pack_bf16x2(__uint_as_float(r[8 * q4 + 6]), __uint_as_float(r[8 * q4 + 7]));
            const int chunk = (c & 1) * 4 + q4;
            *reinterpret_cast<uint4*>(atom + ((chunk ^ (row & 7)) << 4)) = v;
          }
        }
      };
      drain(0, DQK, x1_smem);
      if (MODE == MODE_DKDV) drain(DQK, DV, x2_smem);
      pb::fence_proxy_async_smem();
      pb::named_bar_sync(1, BW_COMPUTE);
      if (threadIdx.x == 64) {
#pragma unroll
        for (int a = 0; a < DQK / 64; ++a)
          pb::tma_store_3d(&tmO1, x1_smem + a * XATOM, a * 64, xhead, tok0 + rb * BR);
        if (MODE == MODE_DKDV) {
#pragma unroll
          for (int a = 0; a < DV / 64; ++a)
            pb::tma_store_3d(&tmO2, x2_smem + a * XATOM, a * 64, xhead, tok0 + rb * BR);
        }
        pb::tma_store_commit();
        pb::tma_store_wait_all<0>();
      }
    } while (false);
  }

  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  pb::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    pb::tc_fence_after();
    pb::tmem_dealloc<1>(tmem_base, 512);
  }
}

// delta[b, h, s] = sum_d dO * O ;  lse2 = lse * log2(e) (so the main kernels need no per-element multiply).
// One thread per (batch, head, position), position fastest: a thread streams its 2 * dv bf16 values with 16-byte
// loads (many loads in flight per thread) and the per-row results are written coalesced.
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                  const float* __restrict__ lse, float* __restrict__ delta, float* __restrict__ lse2, int seq, int hq,
                  int dv, long o_row, long do_row, long total_rows) {
  const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
  if (i >= total_rows * hq) return;
  const long pos = i % seq;
  const int h = (int)((i / seq) % hq);
  const long b = i / ((long)seq * hq);
  const long t = b * seq + pos;
  const uint4* op = reinterpret_cast<const uint4*>(o + t * o_row + (long)h * dv);
  const uint4* dp = reinterpret_cast<const uint4*>(d_o + t * do_row + (long)h * dv);
  float s = 0.f;
#pragma unroll 4
  for (int v = 0; v < dv / 8; ++v) {
    const uint4 x = op[v], y = dp[v];
    const __nv_bfloat162* xa = reinterpret_cast<const __nv_bfloat162*>(&x);
    const __nv_bfloat162* ya = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float2 a = __bfloat1622float2(xa[u]), c = __bfloat1622float2(ya[u]);
      s += a.x * c.x + a.y * c.y;
    }
  }
  delta[i] = s;
  lse2[i] = lse[i] * 1.4426950408889634f;
}

struct BwdArgs {
  const void *d_o, *q, *k, *v, *o;
  const float* lse;
  float* delta;
  void *dq, *dk, *dv;
  int batch, seq, seq_k, q_off, window, hq, hkv;
  float softcap;
  long q_row, k_row, v_row, o_row, do_row, dq_row, dk_row, dv_row;
  float scale;
  int causal;
  int* status;
  cudaStream_t stream;
};

template <int DQK, int DV>
int launch_bwd(const BwdArgs& a) {
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  const long T = (long)a.batch * a.seq;
  {
    const int threads = 256;
    const long blocks = (T * a.hq + threads - 1) / threads;
    attn_delta_kernel<<<(unsigned)blocks, threads, 0, a.stream>>>(
        (const __nv_bfloat16*)a.o, (const __nv_bfloat16*)a.d_o, a.lse, a.delta, a.delta + (long)a.batch * a.hq * a.seq,
        a.seq, a.hq, DV, a.o_row, a.do_row, T);
  }
  int rc;
  CUtensorMap q128, do128, k128, v128, q64, do64, k64, v64, dq_m, dk_m, dv_m;
  const long TK = (long)a.batch * a.seq_k;
#define MK(m, p, rows, heads, d, row, br) \
  if ((rc = pbh::make_tmap_3d(&m, p, bf, 2, rows, heads, d, d, row, br, 1, 64, sw))) return rc;
  MK(q128, a.q, T, a.hq, DQK, a.q_row, 128) MK(do128, a.d_o, T, a.hq, DV, a.do_row, 128)
  MK(k128, a.k, TK, a.hkv, DQK, a.k_row, 128) MK(v128, a.v, TK, a.hkv, DV, a.v_row, 128)
  MK(q64, a.q, T, a.hq, DQK, a.q_row, 64) MK(do64, a.d_o, T, a.hq, DV, a.do_row, 64)
  MK(k64, a.k, TK, a.hkv, DQK, a.k_row, 64) MK(v64, a.v, TK, a.hkv, DV, a.v_row, 64)
  MK(dq_m, a.dq, T, a.hq, DQK, a.dq_row, 128) MK(dk_m, a.dk, TK, a.hkv, DQK, a.dk_row, 128)
  MK(dv_m, a.dv, TK, a.hkv, DV, a.dv_row, 128)
#undef MK
  {
    using C = BwCfg<DQK, DV, MODE_DKDV>;
    auto kern = (a.window > 0 || a.softcap > 0.f) ? flash_attn_bwd_kernel<DQK, DV, MODE_DKDV, true> : flash_attn_bwd_kernel<DQK, DV, MODE_DKDV, false>;
    static bool attr_set[2] = {false, false};
    if (!attr_set[a.window > 0 || a.softcap > 0.f]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      attr_set[a.window > 0 || a.softcap > 0.f] = true;
    }
    dim3 grid(a.hkv * a.batch, a.seq_k / BR, 1);
    kern<<<grid, BW_THREADS, C::SMEM_BYTES, a.stream>>>(k128, v128, q64, do64, dk_m, dv_m,
                                                       a.delta + (long)a.batch * a.hq * a.seq, a.delta, a.seq, a.seq_k,
                                                       a.q_off, a.hq, a.hkv, a.scale, a.causal, a.window, a.softcap, a.status);
  }
  {
    using C = BwCfg<DQK, DV, MODE_DQ>;
    auto kern = (a.window > 0 || a.softcap > 0.f) ? flash_attn_bwd_kernel<DQK, DV, MODE_DQ, true> : flash_attn_bwd_kernel<DQK, DV, MODE_DQ, false>;
    static bool attr_set[2] = {false, false};
    if (!attr_set[a.window > 0 || a.softcap > 0.f]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      attr_set[a.window > 0 || a.softcap > 0.f] = true;
    }
    dim3 grid(a.hq * a.batch, a.seq / BR, 1);
    kern<<<grid, BW_THREADS, C::SMEM_BYTES, a.stream>>>(q128, do128, k64, v64, dq_m, dq_m,
                                                       a.delta + (long)a.batch * a.hq * a.seq, a.delta, a.seq, a.seq_k,
                                                       a.q_off, a.hq, a.hkv, a.scale, a.causal, a.window, a.softcap, a.status);
  }
  return (int)cudaGetLastError();
}

}  // namespace

// Layouts as in pb_flash_attn_fwd_ex (q / o / d_o / dq: batch*seq rows; k / v / dk / dv: batch*seq_k rows).
// delta: fp32 scratch [2, batch, hq, seq] (written here: row sums of dO*O, then the log-sum-exp in log2 units).
extern "C" int pb_flash_attn_bwd_cap(const void* d_o, const void* q, const void* k, const void* v, const void* o,
                                     const float* lse, float* delta, void* dq, void* dk, void* dv, int batch, int seq,
                                     int seq_k, int q_off, int hq, int hkv, int d_qk, int d_v, long q_row, long k_row,
                                     long v_row, long o_row, long do_row, long dq_row, long dk_row, long dv_row,
                                     float scale, int causal, int window, float softcap, int* status,
                                     cudaStream_t stream) {
  if (seq % 128 || seq_k % 128 || q_off % 128 || q_off < 0 || hq % hkv) return -2;
  if (causal ? (q_off + seq != seq_k) : (q_off != 0)) return -2;
  if (window < 0 || (window > 0 && (!causal || q_off != 0)) || softcap < 0.f) return -2;
  if ((q_row | k_row | v_row | o_row | do_row | dq_row | dk_row | dv_row) % 8) return -2;
  BwdArgs a{d_o, q, k, v, o, lse, delta, dq, dk, dv, batch, seq, seq_k, q_off, window, hq, hkv, softcap, q_row, k_row,
            v_row, o_row, do_row, dq_row, dk_row, dv_row, scale, causal, status, stream};
  if (d_qk == 128 && d_v == 128) return launch_bwd<128, 128>(a);
  if (d_qk == 192 && d_v == 128) return launch_bwd<192, 128>(a);
  if (d_qk == 64 && d_v == 64) return launch_bwd<64, 64>(a);
  return -3;
}

extern "C" int pb_flash_attn_bwd_win(const void* d_o, const void* q, const void* k, const void* v, const void* o,
                                     const float* lse, float* delta, void* dq, void* dk, void* dv, int batch, int seq,
                                     int seq_k, int q_off, int hq, int hkv, int d_qk, int d_v, long q_row, long k_row,
                                     long v_row, long o_row, long do_row, long dq_row, long dk_row, long dv_row,
                                     float scale, int causal, int window, int* status, cudaStream_t stream) {
  return pb_flash_attn_bwd_cap(d_o, q, k, v, o, lse, delta, dq, dk, dv, batch, seq, seq_k, q_off, hq, hkv, d_qk, d_v,
                               q_row, k_row, v_row, o_row, do_row, dq_row, dk_row, dv_row, scale, causal, window, 0.f,
                               status, stream);
}

extern "C" int pb_flash_attn_bwd_ex(const void* d_o, const void* q, const void* k, const void* v, const void* o,
                                    const float* lse, float* delta, void* dq, void* dk, void* dv, int batch, int seq,
                                    int seq_k, int q_off, int hq, int hkv, int d_qk, int d_v, long q_row, long k_row,
                                    long v_row, long o_row, long do_row, long dq_row, long dk_row, long dv_row,
                                    float scale, int causal, int* status, cudaStream_t stream) {
  return pb_flash_attn_bwd_win(d_o, q, k, v, o, lse, delta, dq, dk, dv, batch, seq, seq_k, q_off, hq, hkv, d_qk, d_v,
                               q_row, k_row, v_row, o_row, do_row, dq_row, dk_row, dv_row, scale, causal, 0, status,
                               stream);
}

extern "C" int pb_flash_attn_bwd(const void* d_o, const void* q, const void* k, const void* v, const void* o,
                                 const float* lse, float* delta, void* dq, void* dk, void* dv, int batch, int seq,
                                 int hq, int hkv, int d_qk, int d_v, long q_row, long k_row, long v_row, long o_row,
                                 long do_row, long dq_row, long dk_row, long dv_row, float scale, int causal,
                                 int* status, cudaStream_t stream) {
  return pb_flash_attn_bwd_ex(d_o, q, k, v, o, lse, delta, dq, dk, dv, batch, seq, seq, 0, hq, hkv, d_qk, d_v, q_row,
                              k_row, v_row, o_row, do_row, dq_row, dk_row, dv_row, scale, causal, status, stream);
}
