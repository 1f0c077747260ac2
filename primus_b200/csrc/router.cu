// Fused MoE router: score function + (group-limited) top-k + probability normalisation + per-expert token
// counts in one pass over the logits, and the matching backward.  One warp per token; the token's scores
// live in shared memory (E <= 1024).
//
//   softmax, pre_softmax  : full = softmax(l); choose on full;  p_j = full[i_j]
//   softmax, post         : full = softmax(l); choose on l;     p   = softmax(l[i_1..i_k])
//   sigmoid (+ bias)      : full = sigmoid(l); choose on full + bias; p_j = full[i_j] / (sum_j full[i_j] + 1e-20) (k > 1)
//   group-limited         : experts are split into G groups, only the best `group_topk` groups stay eligible
//                           (group score = max, or the sum of the two best entries when a bias is used)
//   p *= scaling_factor;  counts[e] += 1 for every selected expert.
// `full` (fp32 [T, E]) is written for the load-balancing losses and the backward.
//
// Replaces `fused_group_topk_routing_with_aux_score` and the router's softmax / top-k op chain
// (primus/backends/megatron/core/transformer/moe/router.py:24-134).
#include "common.cuh"

namespace {

constexpr int WARPS = 8;

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax warp_argmax(float v, int i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  }
  return {v, i};
}

template <typename TIn>
__device__ __forceinline__ float to_f(TIn x);
template <>
__device__ __forceinline__ float to_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename TIn>
__global__ void __launch_bounds__(WARPS * 32)
router_fwd_kernel(const TIn* __restrict__ logits, const float* __restrict__ bias, int T, int E, int k, int sigmoid,
                  int pre_softmax, int num_groups, int group_topk, float scale, float* __restrict__ probs,
                  int* __restrict__ idx, float* __restrict__ full, int* __restrict__ counts) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WARPS + warp;
  if (t >= T) return;
  float* sc = smem + warp * 2 * E;  // [0,E): full scores, [E,2E): selection scores
  float* ch = sc + E;
  const TIn* lrow = logits + (long)t * E;

  float m = -INFINITY;
  for (int e = lane; e < E; e += 32) {
    const float l = to_f<TIn>(lrow[e]);
    ch[e] = l;
    m = fmaxf(m, l);
  }
  m = pb::warp_max(m);
  if (!sigmoid) {
    float s = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float ex = __expf(ch[e] - m);
      sc[e] = ex;
      s += ex;
    }
    s = pb::warp_sum(s);
    const float inv = 1.f / s;
    for (int e = lane; e < E; e += 32) {
      const float f = sc[e] * inv;
      sc[e] = f;
      if (pre_softmax) ch[e] = f;
    }
  } else {
    for (int e = lane; e < E; e += 32) {
      const float f = 1.f / (1.f + __expf(-ch[e]));
      sc[e] = f;
      ch[e] = bias ? f + bias[e] : f;
    }
  }
  for (int e = lane; e < E; e += 32) full[(long)t * E + e] = sc[e];
  __syncwarp();

  if (num_groups > 1 && group_topk > 0 && group_topk < num_groups) {
    // lane g owns groups g, g + 32, ... (num_groups <= 64 in practice)
    const int gs = E / num_groups;
    float gscore[2] = {-INFINITY, -INFINITY};
    for (int gi = 0; gi < 2; ++gi) {
      const int g = lane + gi * 32;
      if (g < num_groups) {
        float b1 = -INFINITY, b2 = -INFINITY;
        for (int j = 0; j < gs; ++j) {
          const float v = ch[g * gs + j];
          if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
        }
        gscore[gi] = (bias && gs > 1) ? b1 + b2 : b1;
      }
    }
    unsigned long long keep = 0ull;  // bit g: group stays eligible
    for (int it = 0; it < group_topk; ++it) {
      float v = gscore[0];
      int i = lane;
      if (gscore[1] > v) { v = gscore[1]; i = lane + 32; }
      const ArgMax am = warp_argmax(v, i);
      keep |= 1ull << am.i;
      if ((am.i & 31) == lane) gscore[am.i >> 5] = -INFINITY;
    }
    for (int e = lane; e < E; e += 32)
      if (!((keep >> (e / gs)) & 1ull)) ch[e] = -INFINITY;
    __syncwarp();
  }

  float sel_p = 0.f;   // lane j < k keeps the j-th selection
  int sel_i = 0;
  for (int j = 0; j < k; ++j) {
    float v = -INFINITY;
    int i = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float c = ch[e];
      if (c > v) { v = c; i = e; }
    }
    const ArgMax am = warp_argmax(v, i);
    if (lane == j) {
      sel_i = am.i;
      sel_p = (!sigmoid && !pre_softmax) ? am.v : sc[am.i];
    }
    if (lane == (am.i & 31)) ch[am.i] = -INFINITY;
    __syncwarp();
  }
  const bool act = lane < k;
  if (!sigmoid && !pre_softmax) {
    // softmax over the selected logits
    float mm = act ? sel_p : -INFINITY;
    mm = pb::warp_max(mm);
    const float ex = act ? __expf(sel_p - mm) : 0.f;
    const float s = pb::warp_sum(ex);
    sel_p = ex / s;
  } else if (sigmoid && k > 1) {
    const float s = pb::warp_sum(act ? sel_p : 0.f);
    sel_p = sel_p / (s + 1e-20f);
  }
  if (act) {
    probs[(long)t * k + lane] = sel_p * scale;
    idx[(long)t * k + lane] = sel_i;
    if (counts) atomicAdd(counts + sel_i, 1);
  }
}

// dlogits [T, E] fp32 from dprobs [T, k], dfull [T, E] (may be null), saved full / idx / probs.
__global__ void __launch_bounds__(WARPS * 32)
router_bwd_kernel(const float* __restrict__ dprobs, const float* __restrict__ dfull, const float* __restrict__ full,
                  const int* __restrict__ idx, const float* __restrict__ probs, int T, int E, int k, int sigmoid,
                  int pre_softmax, float scale, float* __restrict__ dlogits) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WARPS + warp;
  if (t >= T) return;
  float* g = smem + warp * E;  // gradient w.r.t. the full scores
  for (int e = lane; e < E; e += 32) g[e] = dfull ? dfull[(long)t * E + e] : 0.f;
  __syncwarp();
  const bool act = lane < k;
  const int my_i = act ? idx[(long)t * k + lane] : 0;
  const float dp = act ? dprobs[(long)t * k + lane] * scale : 0.f;   // gradient w.r.t. the unscaled probability
  const float p = act ? probs[(long)t * k + lane] / scale : 0.f;
  const float* frow = full + (long)t * E;
  float* drow = dlogits + (long)t * E;
  if (!sigmoid) {
    float extra = 0.f;  // direct logit gradient of the selected entries (post-softmax normalisation)
    if (pre_softmax) {
      if (act) g[my_i] += dp;
    } else {
      const float dot = pb::warp_sum(dp * p);
      extra = p * (dp - dot);
    }
    __syncwarp();
    float dot = 0.f;
    for (int e = lane; e < E; e += 32) dot += g[e] * frow[e];
    dot = pb::warp_sum(dot);
    for (int e = lane; e < E; e += 32) g[e] = frow[e] * (g[e] - dot);
    __syncwarp();
    if (!pre_softmax && act) g[my_i] += extra;
    __syncwarp();
    for (int e = lane; e < E; e += 32) drow[e] = g[e];
  } else {
    const float f = act ? frow[my_i] : 0.f;
    float df = dp;
    if (k > 1) {
      const float S = pb::warp_sum(f) + 1e-20f;
      const float dot = pb::warp_sum(dp * f);
      df = dp / S - dot / (S * S);
    }
    if (act) g[my_i] += df;
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
      const float fe = frow[e];
      drow[e] = g[e] * fe * (1.f - fe);
    }
  }
}

}  // namespace

extern "C" {

// logits: [T, E] bf16 (in_bf16 != 0) or fp32.  bias: fp32 [E] or null.  counts: int [E] accumulated (may be null).
int pb_router_fwd(const void* logits, int in_bf16, const float* bias, int T, int E, int k, int sigmoid, int pre_softmax,
                  int num_groups, int group_topk, float scale, float* probs, int* idx, float* full, int* counts,
                  cudaStream_t s) {
  if (E > 1024 || k > 32 || k < 1 || k > E || (num_groups > 1 && (E % num_groups || num_groups > 64))) return -2;
  const int blocks = (T + WARPS - 1) / WARPS;
  const size_t smem = (size_t)WARPS * 2 * E * sizeof(float);
  if (smem > 48 * 1024) {
    static bool set_b = false, set_f = false;
    bool& flag = in_bf16 ? set_b : set_f;
    if (!flag) {
      cudaError_t e = in_bf16 ? cudaFuncSetAttribute(router_fwd_kernel<__nv_bfloat16>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024)
                              : cudaFuncSetAttribute(router_fwd_kernel<float>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
      if (e != cudaSuccess) return (int)e;
      flag = true;
    }
  }
  if (in_bf16)
    router_fwd_kernel<__nv_bfloat16><<<blocks, WARPS * 32, smem, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits), bias, T, E, k, sigmoid, pre_softmax, num_groups, group_topk,
        scale, probs, idx, full, counts);
  else
    router_fwd_kernel<float><<<blocks, WARPS * 32, smem, s>>>(reinterpret_cast<const float*>(logits), bias, T, E, k,
                                                              sigmoid, pre_softmax, num_groups, group_topk, scale, probs,
                                                              idx, full, counts);
  return (int)cudaGetLastError();
}

int pb_router_bwd(const float* dprobs, const float* dfull, const float* full, const int* idx, const float* probs, int T,
                  int E, int k, int sigmoid, int pre_softmax, float scale, float* dlogits, cudaStream_t s) {
  if (E > 1024 || k > 32) return -2;
  const int blocks = (T + WARPS - 1) / WARPS;
  router_bwd_kernel<<<blocks, WARPS * 32, (size_t)WARPS * E * sizeof(float), s>>>(
      dprobs, dfull, full, idx, probs, T, E, k, sigmoid, pre_softmax, scale, dlogits);
  return (int)cudaGetLastError();
}

}  // extern "C"
