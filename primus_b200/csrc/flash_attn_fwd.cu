// Flash-attention forward for sm_100a (causal or full, GQA / MQA / MLA head shapes).
//
// One CTA owns 128 query rows of one head and walks the KV sequence in blocks of 128:
//   warp 0      : TMA producer (Q once, then K / V blocks through mbarrier rings)
//   warp 1      : tcgen05 issuer:  S = Q K^T  (into one of two TMEM S buffers)  and  O += P V
//   warps 2..5  : softmax, one thread per query row: S is read with tcgen05.ld, P = exp2(..) is
//                 written as bf16 into 128B-swizzled shared memory (the A operand of the PV MMA),
//                 O is rescaled in tensor memory only when the running max grew by more than 2^8.
// S is double-buffered so that Q K^T of block j+1 runs while softmax works on block j.
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
constexpr int FA_THREADS = 192;

template <int DQK, int DV>
struct FaCfg {
  static constexpr int KS = 2;                      // K stages
  static constexpr int VS = (DQK > 128) ? 1 : 2;    // V stages
  static constexpr int Q_BYTES = BQ * DQK * 2;
  static constexpr int K_BYTES = BKV * DQK * 2;
  static constexpr int V_BYTES = BKV * DV * 2;
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int SMEM_BYTES = Q_BYTES + KS * K_BYTES + VS * V_BYTES + P_BYTES + 1024 + 256;
};

struct FaBars {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2];
  uint64_t v_full[2], v_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full;
  uint64_t pv_done;
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

template <int DQK, int DV>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                      float* __restrict__ lse, int seq, int hq, int hkv, float scale_log2, int causal,
                      int* status) {
  using C = FaCfg<DQK, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;
  uint8_t* k_smem = q_smem + C::Q_BYTES;
  uint8_t* v_smem = k_smem + C::KS * C::K_BYTES;
  uint8_t* p_smem = v_smem + C::VS * C::V_BYTES;
  FaBars* bars = reinterpret_cast<FaBars*>(p_smem + C::P_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_qb = seq / BQ;
  const int qb = num_qb - 1 - blockIdx.x;  // heaviest (longest KV range) blocks first
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / (hq / hkv);
  const int tok0 = batch * seq;
  const int n_blocks = causal ? (qb + 1) : (seq / BKV);
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    pb::mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      pb::mbar_init(&bars->k_full[i], 1);
      pb::mbar_init(&bars->k_empty[i], 1);
      pb::mbar_init(&bars->v_full[i], 1);
      pb::mbar_init(&bars->v_empty[i], 1);
      pb::mbar_init(&bars->s_full[i], 1);
      pb::mbar_init(&bars->s_empty[i], 128);
    }
    pb::mbar_init(&bars->p_full, 128);
    pb::mbar_init(&bars->pv_done, 1);
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
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      pb::mbar_expect_tx(&bars->q_full, C::Q_BYTES);
#pragma unroll
      for (int a = 0; a < DQK / 64; ++a)
        pb::tma_load_3d(q_smem + a * ATOM_BYTES, &tmQ, &bars->q_full, a * 64, head, tok0 + qb * BQ);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int ks = j % C::KS, vs = j % C::VS;
        FA_WAIT(&bars->k_empty[ks], ((j / C::KS) & 1) ^ 1, PB_ERR_TIMEOUT_TMA);
        pb::mbar_expect_tx(&bars->k_full[ks], C::K_BYTES);
#pragma unroll
        for (int a = 0; a < DQK / 64; ++a)
          pb::tma_load_3d(k_smem + ks * C::K_BYTES + a * ATOM_BYTES, &tmK, &bars->k_full[ks], a * 64,
                          kv_head, tok0 + j * BKV);
        FA_WAIT(&bars->v_empty[vs], ((j / C::VS) & 1) ^ 1, PB_ERR_TIMEOUT_TMA);
        pb::mbar_expect_tx(&bars->v_full[vs], C::V_BYTES);
#pragma unroll
        for (int a = 0; a < DV / 64; ++a)
          pb::tma_load_3d(v_smem + vs * C::V_BYTES + a * ATOM_BYTES, &tmV, &bars->v_full[vs], a * 64,
                          kv_head, tok0 + j * BKV);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = pb::make_idesc_bf16(BQ, BKV, 0, 0);
      constexpr uint32_t idesc_o = pb::make_idesc_bf16(BQ, DV, 0, 1);
      const uint32_t qa = pb::smem_u32(q_smem);
      const uint32_t pa = pb::smem_u32(p_smem);
      bool ok = true;
      auto issue_s = [&](int j) {
        const uint32_t ka = pb::smem_u32(k_smem + (j % C::KS) * C::K_BYTES);
        const uint32_t d = tmem_base + (j & 1) * 128;
#pragma unroll
        for (int k = 0; k < DQK / 16; ++k) {
          const uint32_t off = (k / 4) * ATOM_BYTES + (k % 4) * 32;
          pb::umma_f16_ss(d, pb::make_smem_desc(qa + off, 0, 1024, 2), pb::make_smem_desc(ka + off, 0, 1024, 2),
                          idesc_s, k > 0 ? 1u : 0u);
        }
        pb::umma_commit(&bars->k_empty[j % C::KS]);
        pb::umma_commit(&bars->s_full[j & 1]);
      };
      do {
        FA_WAIT(&bars->q_full, 0, PB_ERR_TIMEOUT_MMA);
        FA_WAIT(&bars->k_full[0], 0, PB_ERR_TIMEOUT_MMA);
        pb::tc_fence_after();
        issue_s(0);
      } while (false);
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks) {
          const int jn = j + 1;
          FA_WAIT(&bars->k_full[jn % C::KS], (jn / C::KS) & 1, PB_ERR_TIMEOUT_MMA);
          FA_WAIT(&bars->s_empty[jn & 1], ((jn >> 1) & 1) ^ 1, PB_ERR_TIMEOUT_MMA);
          pb::tc_fence_after();
          issue_s(jn);
        }
        FA_WAIT(&bars->v_full[j % C::VS], (j / C::VS) & 1, PB_ERR_TIMEOUT_MMA);
        FA_WAIT(&bars->p_full, j & 1, PB_ERR_TIMEOUT_MMA);
        pb::tc_fence_after();
        const uint32_t va = pb::smem_u32(v_smem + (j % C::VS) * C::V_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint64_t da = pb::make_smem_desc(pa + (k / 4) * ATOM_BYTES + (k % 4) * 32, 0, 1024, 2);
          const uint64_t db = pb::make_smem_desc(va + k * 2048, ATOM_BYTES, 1024, 2);
          pb::umma_f16_ss(tmem_o, da, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        pb::umma_commit(&bars->v_empty[j % C::VS]);
        pb::umma_commit(&bars->pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const uint32_t lane_addr = uint32_t(wq * 32) << 16;
    float m_ref = -1e30f;
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int b = j & 1;
      FA_WAIT(&bars->s_full[b], (j >> 1) & 1, PB_ERR_TIMEOUT_EPILOGUE);
      pb::tc_fence_after();
      const uint32_t t_s = tmem_base + lane_addr + b * 128;
      const bool diag = causal && (j == qb);
      // pass 1: row maximum
      float mx = -1e30f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        pb::tmem_ld_32x32b_x32(t_s + c * 32, r);
        pb::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float v = __uint_as_float(r[i]);
          if (!diag || (c * 32 + i) <= row) mx = fmaxf(mx, v);
        }
      }
      const float m_new = fmaxf(m_ref, mx * scale_log2);
      const bool grow = m_new > m_ref + 8.f;
      const bool any = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      if (any) {
        alpha = exp2f(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
      }
      if (j > 0) {
        FA_WAIT(&bars->pv_done, (j - 1) & 1, PB_ERR_TIMEOUT_EPILOGUE);
        pb::tc_fence_after();
        if (any) {
          const uint32_t t_o = tmem_o + lane_addr;
#pragma unroll 1
          for (int c = 0; c < DV / 32; ++c) {
            uint32_t r[32];
            pb::tmem_ld_32x32b_x32(t_o + c * 32, r);
            pb::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            pb::tmem_st_32x32b_x32(t_o + c * 32, r);
          }
          pb::tmem_wait_st();
        }
      }
      // pass 2: probabilities -> bf16 -> swizzled shared memory (K-major A operand of P.V)
      uint8_t* prow = p_smem + row * 128;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        pb::tmem_ld_32x32b_x32(t_s + c * 32, r);
        pb::tmem_wait_ld();
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = pb::fast_exp2(fmaf(__uint_as_float(r[i]), scale_log2, -m_ref));
          if (diag && (c * 32 + i) > row) e = 0.f;
          p[i] = e;
          l += e;
        }
        uint8_t* atom = prow + (c >> 1) * ATOM_BYTES;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 v;
          v.x = pb::pack_bf16x2(p[8 * i + 0], p[8 * i + 1]);
          v.y = pb::pack_bf16x2(p[8 * i + 2], p[8 * i + 3]);
          v.z = pb::pack_bf16x2(p[8 * i + 4], p[8 * i + 5]);
          v.w = pb::pack_bf16x2(p[8 * i + 6], p[8 * i + 7]);
          const int chunk = (c & 1) * 4 + i;
          *reinterpret_cast<uint4*>(atom + ((chunk ^ (row & 7)) << 4)) = v;
        }
      }
      pb::tc_fence_before();
      pb::mbar_arrive(&bars->s_empty[b]);
      pb::fence_proxy_async_smem();
      pb::mbar_arrive(&bars->p_full);
    }
    // epilogue: O / l -> bf16 -> shared -> TMA store; log-sum-exp for the backward pass
    do {
      if (!ok) break;
      FA_WAIT(&bars->pv_done, (n_blocks - 1) & 1, PB_ERR_TIMEOUT_EPILOGUE);
      pb::tc_fence_after();
      const float inv = 1.f / l;
      const uint32_t t_o = tmem_o + lane_addr;
      uint8_t* orow = p_smem + row * 128;  // P is dead: reuse it as the output staging tile
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
      lse[((long)batch * hq + head) * seq + qb * BQ + row] = (m_ref + log2f(l)) * 0.6931471805599453f;
      pb::fence_proxy_async_smem();
      pb::named_bar_sync(1, 128);
      if (threadIdx.x == 64) {
#pragma unroll
        for (int a = 0; a < DV / 64; ++a)
          pb::tma_store_3d(&tmO, p_smem + a * ATOM_BYTES, a * 64, head, tok0 + qb * BQ);
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
int launch_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq, int hq,
               int hkv, long q_row, long k_row, long v_row, long o_row, float scale, int causal, int* status,
               cudaStream_t stream) {
  using C = FaCfg<DQK, DV>;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  const long T = (long)batch * seq;
  CUtensorMap tq, tk, tv, to;
  int rc;
  if ((rc = pbh::make_tmap_3d(&tq, q, bf, 2, T, hq, DQK, DQK, q_row, BQ, 1, 64, sw))) return rc;
  if ((rc = pbh::make_tmap_3d(&tk, k, bf, 2, T, hkv, DQK, DQK, k_row, BKV, 1, 64, sw))) return rc;
  if ((rc = pbh::make_tmap_3d(&tv, v, bf, 2, T, hkv, DV, DV, v_row, BKV, 1, 64, sw))) return rc;
  if ((rc = pbh::make_tmap_3d(&to, o, bf, 2, T, hq, DV, DV, o_row, BQ, 1, 64, sw))) return rc;
  auto kern = flash_attn_fwd_kernel<DQK, DV>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid(seq / BQ, hq, batch);
  kern<<<grid, FA_THREADS, C::SMEM_BYTES, stream>>>(tq, tk, tv, to, lse, seq, hq, hkv,
                                                   scale * 1.4426950408889634f, causal, status);
  return (int)cudaGetLastError();
}

}  // namespace

// q: [batch*seq, hq, d_qk] (row pitch q_row elements, heads contiguous), k: [.., hkv, d_qk], v: [.., hkv, d_v],
// o: [.., hq, d_v]; lse: [batch, hq, seq] fp32 (natural log). seq must be a multiple of 128.
extern "C" int pb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch,
                                 int seq, int hq, int hkv, int d_qk, int d_v, long q_row, long k_row, long v_row,
                                 long o_row, float scale, int causal, int* status, cudaStream_t stream) {
  if (seq % 128 || hq % hkv || (q_row % 8) || (k_row % 8) || (v_row % 8) || (o_row % 8)) return -2;
  if (d_qk == 128 && d_v == 128)
    return launch_fwd<128, 128>(q, k, v, o, lse, batch, seq, hq, hkv, q_row, k_row, v_row, o_row, scale, causal,
                                status, stream);
  if (d_qk == 192 && d_v == 128)
    return launch_fwd<192, 128>(q, k, v, o, lse, batch, seq, hq, hkv, q_row, k_row, v_row, o_row, scale, causal,
                                status, stream);
  if (d_qk == 64 && d_v == 64)
    return launch_fwd<64, 64>(q, k, v, o, lse, batch, seq, hq, hkv, q_row, k_row, v_row, o_row, scale, causal,
                              status, stream);
  return -3;
}
