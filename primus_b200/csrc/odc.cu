// On-demand communication (ODC) primitives over symmetric memory.
//
// ODC replaces the two collectives of a sharded data-parallel step by point-to-point traffic that every rank issues
// on its own schedule, so that ranks only meet once per mini-batch instead of at every collective:
//
//   pb_odc_scatter_accumulate : "reduce-scatter by pushes".  A rank adds its gradient of every shard straight into
//                               the shard owner's fp32 accumulator (`red.global.add.v4.f32` on peer memory over
//                               NVLink), whenever its own backward pass has produced it.  No rank waits for another.
//   pb_odc_gather             : "all-gather by pulls".  A rank copies the parameter shards of the other owners from
//                               their buffers into its own (peer loads, 16-byte vectors), when it needs them.
//
// Ordering is the caller's job and needs one device-side barrier per mini-batch (parallel/odc.py): accumulators are
// double buffered by mini-batch parity, so a fast rank may already push the next mini-batch while a slow owner still
// reads the previous one.  The sums are fp32 atomics: their order, and so the last bits of the result, can differ
// from run to run (the reference guards the same effect with `odc_grad_spike_threshold`).
//
// Counterparts in the reference: primus/core/odc/primitives/scatter_accumulate.py:36-431 (owner-side accumulate),
// primus/core/odc/primitives/gather.py:48-244 (GET-based gather); there on rocSHMEM / MORI, here on CUDA IPC mappings.
#include "common.cuh"

namespace {

constexpr int ODC_MAX_DP = 8;

struct OdcPtrs {
  float* acc[ODC_MAX_DP];                 // owner r's accumulator of this bucket (peer-mapped)
  const __nv_bfloat16* param[ODC_MAX_DP]; // rank r's parameter buffer (peer-mapped)
};

// grad: this rank's gradients of the whole bucket, dp shards of shard_n elements, owner-major.
__global__ void __launch_bounds__(512)
odc_scatter_accumulate_kernel(const __grid_constant__ OdcPtrs pp, int dp, int rank, const float* __restrict__ grad,
                              long shard_n, float scale) {
  const long nvec = shard_n / 4;
  const long total = nvec * dp;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    // consecutive blocks of work go to different owners first (rotated by rank) so that the ranks do not all
    // push to the same peer at the same time
    const int r = (int)(i / nvec);
    const long v = i - (long)r * nvec;
    const int owner = (rank + r) % dp;
    const float4 g = reinterpret_cast<const float4*>(grad + (long)owner * shard_n)[v];
    float* dst = pp.acc[owner] + 4 * v;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(g.x * scale), "f"(g.y * scale),
                 "f"(g.z * scale), "f"(g.w * scale)
                 : "memory");
  }
}

// out[owner's shard] = rank `owner`'s parameters of that shard, for every owner but this rank.
__global__ void __launch_bounds__(512)
odc_gather_kernel(const __grid_constant__ OdcPtrs pp, int dp, int rank, long offset, long shard_n,
                  __nv_bfloat16* __restrict__ local) {
  const long nvec = shard_n / 8;
  const long total = nvec * (dp - 1);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int r = (int)(i / nvec) + 1;
    const long v = i - (long)(r - 1) * nvec;
    const int owner = (rank + r) % dp;
    const long at = offset + (long)owner * shard_n;
    reinterpret_cast<uint4*>(local + at)[v] = reinterpret_cast<const uint4*>(pp.param[owner] + at)[v];
  }
}

}  // namespace

extern "C" {

// acc_ptrs[r]: base of owner r's accumulator for this bucket (shard_n floats); grad: local fp32 [dp * shard_n].
int pb_odc_scatter_accumulate(const long* acc_ptrs, int dp, int rank, const float* grad, long shard_n, float scale,
                              cudaStream_t s) {
  if (dp < 1 || dp > ODC_MAX_DP || shard_n % 4 || (reinterpret_cast<uintptr_t>(grad) % 16)) return -2;
  if (shard_n == 0) return 0;
  OdcPtrs p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < dp; ++r) {
    if (acc_ptrs[r] % 16) return -2;
    p.acc[r] = reinterpret_cast<float*>(acc_ptrs[r]);
  }
  long blocks = (shard_n / 4 * dp + 511) / 512;
  if (blocks > 1184) blocks = 1184;
  odc_scatter_accumulate_kernel<<<(int)blocks, 512, 0, s>>>(p, dp, rank, grad, shard_n, scale);
  return (int)cudaGetLastError();
}

// param_ptrs[r]: base of rank r's bf16 parameter buffer; the bucket's shards start at `offset` (elements) and have
// shard_n elements each; local: this rank's parameter buffer (same layout).
int pb_odc_gather(const long* param_ptrs, int dp, int rank, long offset, long shard_n, void* local, cudaStream_t s) {
  if (dp < 1 || dp > ODC_MAX_DP || shard_n % 8 || offset % 8) return -2;
  if (shard_n == 0 || dp == 1) return 0;
  OdcPtrs p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < dp; ++r) p.param[r] = reinterpret_cast<const __nv_bfloat16*>(param_ptrs[r]);
  long blocks = (shard_n / 8 * (dp - 1) + 511) / 512;
  if (blocks > 1184) blocks = 1184;
  odc_gather_kernel<<<(int)blocks, 512, 0, s>>>(p, dp, rank, offset, shard_n, reinterpret_cast<__nv_bfloat16*>(local));
  return (int)cudaGetLastError();
}

}  // extern "C"
