// Data-parallel distributed optimizer fused with its collectives over NVSwitch peer memory.
//
// The gradient buffers and the bf16 parameter buffers of all data-parallel ranks are symmetric
// allocations, so the two collectives of a ZeRO-1 step collapse into the two kernels that touch the
// shard anyway:
//
//   pb_dp_reduce_scatter : for the shard this rank owns, load the fp32 gradients of every rank straight
//                          from peer memory, sum, scale (1/dp), store the reduced fp32 shard locally and
//                          produce the shard's sum of squares (for the global-norm clip)     [= reduce-scatter
//                          + cast/scale + L2-norm partial in one pass]
//   pb_dp_adamw_allgather: AdamW on the shard (fp32 master / moments, device-side clip coefficient and
//                          skip flag) and store the updated bf16 parameters into *every* rank's
//                          parameter buffer                                                 [= update + all-gather]
//
// Ordering across ranks uses the bounded flag barrier of csrc/symm_mem.cu, issued on the same stream
// before the reduce (all gradients final), between the kernels (everybody has read my gradients before
// they are zeroed) and after the update (all parameter shards have landed).
//
// Replaces the bucket reduce-scatter + FusedAdam + parameter all-gather sequence of the reference's
// distributed optimizer (primus/backends/megatron/core/distributed/finalize_model_grad.py:35-38,
// primus/backends/megatron/patches/torch_fused_adam_patches.py:40-88,
// primus/backends/megatron/core/distributed/sdma_param_gather.py:126-243).
#include "common.cuh"

namespace {

constexpr int MAX_DP = 8;

struct PeerPtrs {
  const float* grad[MAX_DP];
  __nv_bfloat16* param[MAX_DP];
};

// out[i] = scale * sum_r grad_r[offset + i];  partial[b] = sum of out^2 handled by block b
__global__ void __launch_bounds__(512)
dp_reduce_scatter_kernel(const __grid_constant__ PeerPtrs pp, int dp, int rank, long offset, long n,
                         float* __restrict__ out, float scale, float* __restrict__ partial) {
  __shared__ float red[16];
  float ss = 0.f;
  const long nvec = n / 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 v[MAX_DP];
#pragma unroll
    for (int r = 0; r < MAX_DP; ++r) {
      if (r < dp) {
        const int src = (rank + r) % dp;  // rotate so that the ranks do not all hit one peer first
        v[r] = reinterpret_cast<const float4*>(pp.grad[src] + offset)[i];
      }
    }
#pragma unroll
    for (int r = 0; r < MAX_DP; ++r) {
      if (r < dp) {
        acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w;
      }
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(out)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  ss = pb::warp_sum(ss);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = ss;
  __syncthreads();
  if (w == 0) {
    float r = (l < 16) ? red[l] : 0.f;
    r = pb::warp_sum(r);
    if (l == 0) partial[blockIdx.x] = r;
  }
}

__global__ void __launch_bounds__(512)
dp_sumsq_final_kernel(const float* __restrict__ partial, int P, float* __restrict__ out, int accumulate) {
  __shared__ float red[16];
  float s = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s += partial[i];
  s = pb::warp_sum(s);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = s;
  __syncthreads();
  if (w == 0) {
    float r = (l < 16) ? red[l] : 0.f;
    r = pb::warp_sum(r);
    if (l == 0) out[0] = accumulate ? out[0] + r : r;
  }
}

__global__ void __launch_bounds__(256)
dp_adamw_allgather_kernel(const __grid_constant__ PeerPtrs pp, int dp, int rank, long offset, long n,
                          float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                          const float* __restrict__ grad, float lr, float beta1, float beta2, float eps,
                          float wd, float bc1, float bc2, const float* __restrict__ grad_scale,
                          const int* __restrict__ skip) {
  const bool do_skip = skip && *skip;
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long nvec = n / 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float p[4] = {p4.x, p4.y, p4.z, p4.w};
    if (!do_skip) {
      const float4 m4 = reinterpret_cast<float4*>(m)[i], v4 = reinterpret_cast<float4*>(v)[i];
      const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
      float mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w}, g[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gg = g[j] * gs;
        mm[j] = beta1 * mm[j] + (1.f - beta1) * gg;
        vv[j] = beta2 * vv[j] + (1.f - beta2) * gg * gg;
        p[j] = p[j] * (1.f - lr * wd) - lr * (mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
      }
      reinterpret_cast<float4*>(master)[i] = make_float4(p[0], p[1], p[2], p[3]);
      reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
      reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    }
    uint2 packed;
    packed.x = pb::pack_bf16x2(p[0], p[1]);
    packed.y = pb::pack_bf16x2(p[2], p[3]);
#pragma unroll
    for (int r = 0; r < MAX_DP; ++r) {
      if (r < dp) {
        const int dst = (rank + r) % dp;
        reinterpret_cast<uint2*>(pp.param[dst] + offset)[i] = packed;  // P2P store: the all-gather
      }
    }
  }
}

PeerPtrs make_ptrs(const long* grad_ptrs, const long* param_ptrs, int dp) {
  PeerPtrs p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < dp; ++r) {
    if (grad_ptrs) p.grad[r] = reinterpret_cast<const float*>(grad_ptrs[r]);
    if (param_ptrs) p.param[r] = reinterpret_cast<__nv_bfloat16*>(param_ptrs[r]);
  }
  return p;
}

}  // namespace

extern "C" {

int pb_dp_num_partials() { return 1184; }

// grad_ptrs[r]: base of rank r's flat fp32 gradient buffer; [offset, offset+n) is this rank's shard (n % 4 == 0).
// out: local fp32 [n] (may alias this rank's own buffer at offset); sumsq_out[0] (+)= sum(out^2).
int pb_dp_reduce_scatter(const long* grad_ptrs, int dp, int rank, long offset, long n, float* out, float scale,
                         float* partial, float* sumsq_out, int accumulate, cudaStream_t s) {
  if (dp < 1 || dp > MAX_DP || n % 4 || offset % 4) return -2;
  if (n == 0) return 0;
  const PeerPtrs p = make_ptrs(grad_ptrs, nullptr, dp);
  const int P = pb_dp_num_partials();
  dp_reduce_scatter_kernel<<<P, 512, 0, s>>>(p, dp, rank, offset, n, out, scale, partial);
  dp_sumsq_final_kernel<<<1, 512, 0, s>>>(partial, P, sumsq_out, accumulate);
  return (int)cudaGetLastError();
}

int pb_dp_adamw_allgather(const long* param_ptrs, int dp, int rank, long offset, long n, float* master, float* m,
                          float* v, const float* grad, float lr, float beta1, float beta2, float eps, float wd,
                          float bc1, float bc2, const float* grad_scale, const int* skip, cudaStream_t s) {
  if (dp < 1 || dp > MAX_DP || n % 4 || offset % 4) return -2;
  if (n == 0) return 0;
  const PeerPtrs p = make_ptrs(nullptr, param_ptrs, dp);
  long blocks = (n / 4 + 255) / 256;
  const long cap = (long)pbh::sm_count() * 8;      // 8 resident CTAs of 256 threads per SM
  if (blocks > cap) blocks = cap;
  dp_adamw_allgather_kernel<<<(int)blocks, 256, 0, s>>>(p, dp, rank, offset, n, master, m, v, grad, lr, beta1, beta2,
                                                       eps, wd, bc1, bc2, grad_scale, skip);
  return (int)cudaGetLastError();
}

}  // extern "C"
