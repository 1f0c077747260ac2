// Flash-attention forward for sm_100a (causal or full, GQA / MQA / MLA head shapes).
//
// One CTA owns two 128-row query tiles of one head and walks the KV sequence in blocks of 128:
//   warp 0       : TMA producer (both Q tiles once, then K / V blocks through mbarrier rings)
//   warp 1       : tcgen05 issuer:  S_t = Q_t K^T  and  O_t += P_t V  for both tiles t
//   warps 2..5   : softmax warpgroup of tile 0        warps 6..9 : softmax warpgroup of tile 1
// One thread owns one query row: it reads S from tensor memory (tcgen05.ld), keeps the running
// max / sum, and writes P = exp2(.) back as packed bf16 *into the same TMEM columns* (tcgen05.st);
// the P.V MMA takes its A operand straight from tensor memory, so P never touches shared memory.
// The two tiles ping-pong: while one warpgroup does softmax, the tensor core runs the other tile's
// P.V and the next Q K^T, and both tiles share every K / V block that is loaded.
// O is rescaled in tensor memory only when the running max grew by more than 2^8.
// V is consumed straight from its [kv, d] row-major tile through an MN-major descriptor, so no
// transposes are needed.  All waits are bounded.
//
// Replaces `flash_attn_func` call sites of the reference
// (primus/backends/megatron/core/extensions/primus_turbo.py:812-823, 888-990); MLA shape
// d_qk = 192 / d_v = 128 as in primus/configs/models/megatron/deepseek_v2_lite.yaml:10-33.
#include "common.cuh"

namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int ATOM_BYTES = 128 * 128;  // 128 rows x 64 bf16
constexpr int FA_THREADS = 320;

template <int DQK, int DV>
struct FaCfg {
  static constexpr int KS = 2;                      // K stages
  static constexpr int VS = (DQK > 128) ? 1 : 2;    // V stages
  static constexpr int Q_BYTES = BQ * DQK * 2;      // one tile
  static constexpr int K_BYTES = BKV * DQK * 2;
  static constexpr int V_BYTES = BKV * DV * 2;
  static constexpr int SMEM_BYTES = 2 * Q_BYTES + KS * K_BYTES + VS * V_BYTES + 1024 + 256;
};

struct FaBars {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2];
  uint64_t v_full[2], v_empty[2];
  uint64_t s_full[2];   // per tile
  uint64_t p_full[2];   // per tile
  uint64_t pv_done[2];  // per tile
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ bool fa_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (pb::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!pb::mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > PB_WAIT_CYCLES) return false;
  }
  return true;
}

#define FA_WAIT(bar, parity, code)                 \
  if (!fa_wait((bar), (parity), abort_flag)) {     \
    atomicCAS(status, 0, (code));                  \
    bars->abort_flag = 1;                          \
    ok = false;                                    \
    break;                                         \
  }

template <int DQK, int DV, bool WIN>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                      float* __restrict__ lse, int seq, int seq_k, int q_off_blocks, int hq, int hkv,
                      float scale_log2, int causal, int window_arg, const float* __restrict__ sinks_arg, float softcap_arg,
                      int* status) {
  // WIN = false: the plain instantiation carries no code for windows or sinks
  const int window = WIN ? window_arg : 0;
  const float* sinks = WIN ? sinks_arg : nullptr;
  // softcap > 0: scores become softcap * tanh(scale * s / softcap) before the softmax
  const float softcap = WIN ? softcap_arg : 0.f;
  // seq: query rows per sequence; seq_k: key rows per sequence; query row i sits at key position
  // q_off_blocks * 128 + i (causal masking is relative to that position).  window > 0 (causal only): a query attends
  // to its last `window` keys, itself included.  sinks: optional per-query-head logit (natural-log units) that only
  // adds exp(sink) to the softmax denominator.
  using C = FaCfg<DQK, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;  // two tiles
  uint8_t* k_smem = q_smem + 2 * C::Q_BYTES;
  uint8_t* v_smem = k_smem + C::KS * C::K_BYTES;
  FaBars* bars = reinterpret_cast<FaBars*>(v_smem + C::VS * C::V_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_q128 = seq / BQ;
  const int num_pairs = (num_q128 + 1) / 2;
  // grid (heads * batch, pairs): x-fastest issue order starts all heads of the heaviest (longest KV range) pair first
  const int pair = num_pairs - 1 - blockIdx.y;
  const int head = blockIdx.x % hq;
  const int batch = blockIdx.x / hq;
  const int kv_head = head / (hq / hkv);
  const int tok0 = batch * seq;
  const int tokk0 = batch * seq_k;
  const int qt[2] = {2 * pair, 2 * pair + 1};  // 128-row query tile indices
  const bool active1 = qt[1] < num_q128;
  const int n_kv = seq_k / BKV;
  // first key block any row of this CTA can see (both tiles stream from there; the later tile masks what lies
  // before its own window)
  const int j_lo = (window > 0) ? max(0, (qt[0] + q_off_blocks) * BQ - window + 1) / BKV : 0;
  const int nb[2] = {(causal ? min(n_kv, qt[0] + q_off_blocks + 1) : n_kv) - j_lo,
                     active1 ? (causal ? min(n_kv, qt[1] + q_off_blocks + 1) : n_kv) - j_lo : 0};
  const int n_max = nb[0] > nb[1] ? nb[0] : nb[1];
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    pb::mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      pb::mbar_init(&bars->k_full[i], 1);
      pb::mbar_init(&bars->k_empty[i], 1);
      pb::mbar_init(&bars->v_full[i], 1);
      pb::mbar_init(&bars->v_empty[i], 1);
      pb::mbar_init(&bars->s_full[i], 1);
      pb::mbar_init(&bars->p_full[i], 4);   // one arrival per softmax warp of the tile
      pb::mbar_init(&bars->pv_done[i], 1);
    }
    bars->abort_flag = 0;
    pb::fence_barrier_init();
    pb::prefetch_tmap(&tmQ);
    pb::prefetch_tmap(&tmK);
    pb::prefetch_tmap(&tmV);
    pb::prefetch_tmap(&tmO);
  }
  if (warp == 1) {
    pb::tmem_alloc<1>(&bars->tmem_base, 512);
    pb::tmem_relinquish<1>();
  }
  pb::tc_fence_before();
  __syncthreads();
  pb::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  // TMEM columns: S_0 [0,128)  S_1 [128,256)  O_0 [256,256+DV)  O_1 [384,384+DV);  P_t aliases S_t[0,64)

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      pb::mbar_expect_tx(&bars->q_full, (active1 ? 2 : 1) * C::Q_BYTES);
      for (int t = 0; t < (active1 ? 2 : 1); ++t) {
#pragma unroll
        for (int a = 0; a < DQK / 64; ++a)
          pb::tma_load_3d(q_smem + t * C::Q_BYTES + a * ATOM_BYTES, &tmQ, &bars->q_full, a * 64, head,
                          tok0 + qt[t] * BQ);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int ks = j % C::KS, vs = j % C::VS;
        FA_WAIT(&bars->k_empty[ks], ((j / C::KS) & 1) ^ 1, PB_ERR_TIMEOUT_TMA);
        pb::mbar_expect_tx(&bars->k_full[ks], C::K_BYTES);
#pragma unroll
        for (int a = 0; a < DQK / 64; ++a)
          pb::tma_load_3d(k_smem + ks * C::K_BYTES + a * ATOM_BYTES, &tmK, &bars->k_full[ks], a * 64,
                          kv_head, tokk0 + (j + j_lo) * BKV);
        FA_WAIT(&bars->v_empty[vs], ((j / C::VS) & 1) ^ 1, PB_ERR_TIMEOUT_TMA);
        pb::mbar_expect_tx(&bars->v_full[vs], C::V_BYTES);
#pragma unroll
        for (int a = 0; a < DV / 64; ++a)
          pb::tma_load_3d(v_smem + vs * C::V_BYTES + a * ATOM_BYTES, &tmV, &bars->v_full[vs], a * 64,
                          kv_head, tokk0 + (j + j_lo) * BKV);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = pb::make_idesc_bf16(BQ, BKV, 0, 0);
      constexpr uint32_t idesc_o = pb::make_idesc_bf16(BQ, DV, 0, 1);
      bool ok = true;
      auto issue_s = [&](int t, int j) {
        const uint32_t qa = pb::smem_u32(q_smem + t * C::Q_BYTES);
        const uint32_t ka = pb::smem_u32(k_smem + (j % C::KS) * C::K_BYTES);
        const uint32_t d = tmem_base + t * 128;
#pragma unroll
        for (int k = 0; k < DQK / 16; ++k) {
          const uint32_t off = (k / 4) * ATOM_BYTES + (k % 4) * 32;
          pb::umma_f16_ss(d, pb::make_smem_desc(qa + off, 0, 1024, 2), pb::make_smem_desc(ka + off, 0, 1024, 2),
                          idesc_s, k > 0 ? 1u : 0u);
        }
        pb::umma_commit(&bars->s_full[t]);
      };
      do {
        FA_WAIT(&bars->q_full, 0, PB_ERR_TIMEOUT_MMA);
        FA_WAIT(&bars->k_full[0], 0, PB_ERR_TIMEOUT_MMA);
        pb::tc_fence_after();
        issue_s(0, 0);
        if (active1) issue_s(1, 0);
        pb::umma_commit(&bars->k_empty[0]);
      } while (false);
      for (int j = 0; j < n_max && ok; ++j) {
        const bool has_next = j + 1 < n_max;
        bool next_k_ready = false;
        FA_WAIT(&bars->v_full[j % C::VS], (j / C::VS) & 1, PB_ERR_TIMEOUT_MMA);
        const uint32_t va = pb::smem_u32(v_smem + (j % C::VS) * C::V_BYTES);
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= nb[t]) continue;
          FA_WAIT(&bars->p_full[t], j & 1, PB_ERR_TIMEOUT_MMA);
          pb::tc_fence_after();
          const uint32_t d = tmem_base + 256 + t * 128;
          const uint32_t pa = tmem_base + t * 128;  // P_t: packed bf16, 8 columns per 16-wide k step
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            const uint64_t db = pb::make_smem_desc(va + k * 2048, ATOM_BYTES, 1024, 2);
            pb::umma_f16_ts(d, pa + k * 8, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
          }
          pb::umma_commit(&bars->pv_done[t]);
          if (j + 1 < nb[t]) {
            if (!next_k_ready) {
              FA_WAIT(&bars->k_full[(j + 1) % C::KS], ((j + 1) / C::KS) & 1, PB_ERR_TIMEOUT_MMA);
              pb::tc_fence_after();
              next_k_ready = true;
            }
            issue_s(t, j + 1);
          }
        }
        if (!ok) break;
        pb::umma_commit(&bars->v_empty[j % C::VS]);
        if (has_next) pb::umma_commit(&bars->k_empty[(j + 1) % C::KS]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int t = (warp - 2) >> 2;  // tile / warpgroup
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const uint32_t lane_addr = uint32_t(wq * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + t * 128;
    const uint32_t t_o = tmem_base + lane_addr + 256 + t * 128;
    const int n_blocks = nb[t];
    float m_ref = -1e30f;
    float l = 0.f;
    float l_scale = 1.f;
    bool ok = true;
    for (int j = 0; j < n_blocks && ok; ++j) {
      FA_WAIT(&bars->s_full[t], j & 1, PB_ERR_TIMEOUT_EPILOGUE);
      pb::tc_fence_after();
      const bool diag = causal && (j + j_lo == qt[t] + q_off_blocks);
      // keys of this block older than the window of this row: columns [0, lim)
      const int lim = (window > 0) ? (qt[t] + q_off_blocks) * BQ + row - window + 1 - (j + j_lo) * BKV : 0;
      const bool edge = __any_sync(0xffffffffu, lim > 0);
      // the whole S row (128 fp32) is read once and stays in registers for both passes
      uint32_t sr[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) pb::tmem_ld_32x32b_x32(t_s + c * 32, sr + c * 32);
      pb::tmem_wait_ld();
      if (WIN && softcap > 0.f) {
        // keep the later `s * scale_log2` form: store softcap * tanh(scale * s / softcap) / scale
        const float scale = scale_log2 * 0.6931471805599453f;
        const float a = scale / softcap, b = softcap / scale;
#pragma unroll
        for (int i = 0; i < 128; ++i) sr[i] = __float_as_uint(b * pb::fast_tanh(__uint_as_float(sr[i]) * a));
      }
      if (diag) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i > row) sr[i] = 0xff800000u;  // -inf: masked out of max and exp
      }
      if (edge) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i < lim) sr[i] = 0xff800000u;
      }
      // pass 1: row maximum (four independent chains)
      float mx4[4] = {-1e30f, -1e30f, -1e30f, -1e30f};
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(mx4[u], __uint_as_float(sr[i + u]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_ref, mx * scale_log2);
      const bool grow = m_new > m_ref + 8.f;
      const bool any = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      if (any) {
        alpha = exp2f(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
      }
      if (j > 0 && any) {
        FA_WAIT(&bars->pv_done[t], (j - 1) & 1, PB_ERR_TIMEOUT_EPILOGUE);
        pb::tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < DV / 32; ++c) {
          uint32_t r[32];
          pb::tmem_ld_32x32b_x32(t_o + c * 32, r);
          pb::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          pb::tmem_st_32x32b_x32(t_o + c * 32, r);
        }
      }
      // pass 2: P = exp2(S * scale - m) as packed bf16, written over the (already read) S columns
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float e0 = pb::fast_exp2(fmaf(__uint_as_float(sr[c * 32 + i]), scale_log2, -m_ref));
          const float e1 = pb::fast_exp2(fmaf(__uint_as_float(sr[c * 32 + i + 1]), scale_log2, -m_ref));
          l4[(i >> 1) & 3] += e0 + e1;
          pk[i >> 1] = pb::pack_bf16x2(e0, e1);
        }
        pb::tmem_st_32x32b_x16(t_s + c * 16, pk);
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      pb::tmem_wait_st();
      pb::tc_fence_before();
      __syncwarp();
      if (lane == 0) pb::mbar_arrive(&bars->p_full[t]);   // 128 arrivals on one mbarrier would serialise
    }
    // epilogue: O / l -> bf16 -> shared (the tile's dead Q buffer) -> TMA store; log-sum-exp
    do {
      if (!ok || n_blocks == 0) break;
      FA_WAIT(&bars->pv_done[t], (n_blocks - 1) & 1, PB_ERR_TIMEOUT_EPILOGUE);
      pb::tc_fence_after();
      if (sinks != nullptr) {   // the sink joins the denominator only
        const float s2 = sinks[head] * 1.4426950408889634f;
        const float m_fin = fmaxf(m_ref, s2);
        const float a = exp2f(m_ref - m_fin);
        l = l * a + exp2f(s2 - m_fin);
        l_scale = a;
        m_ref = m_fin;
      }
      const float inv = l_scale / l;
      uint8_t* stage = q_smem + t * C::Q_BYTES;
      uint8_t* orow = stage + row * 128;
#pragma unroll 1
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t r[32];
        pb::tmem_ld_32x32b_x32(t_o + c * 32, r);
        pb::tmem_wait_ld();
        uint8_t* atom = orow + (c >> 1) * ATOM_BYTES;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 v;
          v.x = pb::pack_bf16x2(__uint_as_float(r[8 * i + 0]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
          v.y = pb::pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
          v.z = pb::pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
          v.w = pb::pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
          const int chunk = (c & 1) * 4 + i;
          *reinterpret_cast<uint4*>(atom + ((chunk ^ (row & 7)) << 4)) = v;
        }
      }
      lse[((long)batch * hq + head) * seq + qt[t] * BQ + row] = (m_ref + log2f(l)) * 0.6931471805599453f;
      pb::fence_proxy_async_smem();
      pb::named_bar_sync(1 + t, 128);
      if ((threadIdx.x & 127) == 64) {  // one thread per warpgroup (first lane of warps 2 and 6)
#pragma unroll
        for (int a = 0; a < DV / 64; ++a)
          pb::tma_store_3d(&tmO, stage + a * ATOM_BYTES, a * 64, head, tok0 + qt[t] * BQ);
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

template <int DQK, int DV>
int launch_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq, int seq_k,
               int q_off, int hq, int hkv, long q_row, long k_row, long v_row, long o_row, float scale, int causal,
               int window, const float* sinks, float softcap, int* status, cudaStream_t stream) {
  using C = FaCfg<DQK, DV>;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  const long T = (long)batch * seq;
  const long TK = (long)batch * seq_k;
  CUtensorMap tq, tk, tv, to;
  int rc;
  if ((rc = pbh::make_tmap_3d(&tq, q, bf, 2, T, hq, DQK, DQK, q_row, BQ, 1, 64, sw))) return rc;
  if ((rc = pbh::make_tmap_3d(&tk, k, bf, 2, TK, hkv, DQK, DQK, k_row, BKV, 1, 64, sw))) return rc;
  if ((rc = pbh::make_tmap_3d(&tv, v, bf, 2, TK, hkv, DV, DV, v_row, BKV, 1, 64, sw))) return rc;
  if ((rc = pbh::make_tmap_3d(&to, o, bf, 2, T, hq, DV, DV, o_row, BQ, 1, 64, sw))) return rc;
  const bool win = window > 0 || sinks != nullptr || softcap > 0.f;
  auto kern = win ? flash_attn_fwd_kernel<DQK, DV, true> : flash_attn_fwd_kernel<DQK, DV, false>;
  static bool attr_set[2] = {false, false};
  if (!attr_set[win]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[win] = true;
  }
  dim3 grid(hq * batch, (seq / BQ + 1) / 2, 1);
  kern<<<grid, FA_THREADS, C::SMEM_BYTES, stream>>>(tq, tk, tv, to, lse, seq, seq_k, q_off / BQ, hq, hkv,
                                                   scale * 1.4426950408889634f, causal, window, sinks, softcap, status);
  return (int)cudaGetLastError();
}

}  // namespace

// q: [batch*seq, hq, d_qk] (row pitch q_row elements, heads contiguous), k: [batch*seq_k, hkv, d_qk],
// v: [batch*seq_k, hkv, d_v], o: [batch*seq, hq, d_v]; lse: [batch, hq, seq] fp32 (natural log).  seq, seq_k and q_off
// are multiples of 128.  Query row i of a sequence sits at key position q_off + i: with `causal` it attends to keys
// [0, q_off + i] (the last `window` of them when window > 0) and q_off + seq must equal seq_k (the layout of a
// sequence chunk attending to the gathered prefix).  sinks: null or one fp32 logit per query head.
extern "C" int pb_flash_attn_fwd_cap(const void* q, const void* k, const void* v, void* o, float* lse, int batch,
                                     int seq, int seq_k, int q_off, int hq, int hkv, int d_qk, int d_v, long q_row,
                                     long k_row, long v_row, long o_row, float scale, int causal, int window,
                                     const float* sinks, float softcap, int* status, cudaStream_t stream) {
  if (seq % 128 || seq_k % 128 || q_off % 128 || q_off < 0 || hq % hkv || (q_row % 8) || (k_row % 8) || (v_row % 8) ||
      (o_row % 8))
    return -2;
  if (causal ? (q_off + seq != seq_k) : (q_off != 0)) return -2;
  if (window < 0 || (window > 0 && (!causal || q_off != 0)) || softcap < 0.f) return -2;
  if (d_qk == 128 && d_v == 128)
    return launch_fwd<128, 128>(q, k, v, o, lse, batch, seq, seq_k, q_off, hq, hkv, q_row, k_row, v_row, o_row, scale,
                                causal, window, sinks, softcap, status, stream);
  if (d_qk == 192 && d_v == 128)
    return launch_fwd<192, 128>(q, k, v, o, lse, batch, seq, seq_k, q_off, hq, hkv, q_row, k_row, v_row, o_row, scale,
                                causal, window, sinks, softcap, status, stream);
  if (d_qk == 64 && d_v == 64)
    return launch_fwd<64, 64>(q, k, v, o, lse, batch, seq, seq_k, q_off, hq, hkv, q_row, k_row, v_row, o_row, scale,
                              causal, window, sinks, softcap, status, stream);
  return -3;
}

// No logit soft-capping.
extern "C" int pb_flash_attn_fwd_win(const void* q, const void* k, const void* v, void* o, float* lse, int batch,
                                     int seq, int seq_k, int q_off, int hq, int hkv, int d_qk, int d_v, long q_row,
                                     long k_row, long v_row, long o_row, float scale, int causal, int window,
                                     const float* sinks, int* status, cudaStream_t stream) {
  return pb_flash_attn_fwd_cap(q, k, v, o, lse, batch, seq, seq_k, q_off, hq, hkv, d_qk, d_v, q_row, k_row, v_row, o_row,
                               scale, causal, window, sinks, 0.f, status, stream);
}

// No sliding window, no sinks.
extern "C" int pb_flash_attn_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse, int batch,
                                    int seq, int seq_k, int q_off, int hq, int hkv, int d_qk, int d_v, long q_row,
                                    long k_row, long v_row, long o_row, float scale, int causal, int* status,
                                    cudaStream_t stream) {
  return pb_flash_attn_fwd_win(q, k, v, o, lse, batch, seq, seq_k, q_off, hq, hkv, d_qk, d_v, q_row, k_row, v_row, o_row,
                               scale, causal, 0, nullptr, status, stream);
}

// Self-attention form: seq_k = seq, q_off = 0.
extern "C" int pb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch,
                                 int seq, int hq, int hkv, int d_qk, int d_v, long q_row, long k_row, long v_row,
                                 long o_row, float scale, int causal, int* status, cudaStream_t stream) {
  return pb_flash_attn_fwd_ex(q, k, v, o, lse, batch, seq, seq, 0, hq, hkv, d_qk, d_v, q_row, k_row, v_row, o_row,
                              scale, causal, status, stream);
}
