// Multi-tensor apply: one launch over a list of tensors (L2 norm, scale with overflow check, axpby).
//
// The host flattens the tensor list into a table of chunks (pointer triplet, element count, tensor index);
// one CTA processes one chunk.  Reductions are deterministic: every chunk writes its partial sum of squares,
// a second kernel adds the partials of each tensor (and the total) in chunk order.
//
// Replaces the Apex / TE multi-tensor kernels (`multi_tensor_l2norm`, `multi_tensor_scale`,
// `multi_tensor_axpby`) used by the reference's optimizer and gradient clipping
// (primus/backends/megatron/patches/torch_fused_adam_patches.py:40-88).
#include "common.cuh"

namespace {

struct Chunk {
  const void* a;
  const void* b;
  void* out;
  int n;
  int tensor;
};

template <typename T>
__device__ __forceinline__ float ld(const void* p, long i) {
  return static_cast<float>(reinterpret_cast<const T*>(p)[i]);
}
template <>
__device__ __forceinline__ float ld<__nv_bfloat16>(const void* p, long i) {
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
template <typename T>
__device__ __forceinline__ void st(void* p, long i, float v) {
  reinterpret_cast<T*>(p)[i] = static_cast<T>(v);
}
template <>
__device__ __forceinline__ void st<__nv_bfloat16>(void* p, long i, float v) {
  reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
}

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float red[8];
  v = pb::warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = 0.f;
  if (threadIdx.x == 0)
    for (int i = 0; i < 8; ++i) r += red[i];
  return r;  // valid on thread 0
}

template <typename TA>
__global__ void __launch_bounds__(256) mt_l2norm_kernel(const Chunk* chunks, float* partial) {
  const Chunk c = chunks[blockIdx.x];
  float s = 0.f;
  for (int i = threadIdx.x; i < c.n; i += 256) {
    const float v = ld<TA>(c.a, i);
    s += v * v;
  }
  s = block_sum(s);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// per_tensor[t] = sum of the partials of tensor t's chunks (chunks of a tensor are contiguous); total[0] = sum of all
__global__ void mt_l2norm_final_kernel(const Chunk* chunks, const float* partial, int n_chunks, float* per_tensor,
                                       int n_tensors, float* total) {
  __shared__ float s_total[256];
  float tot = 0.f;
  // thread t handles tensors t, t + 256, ...: find its chunk range by a scan over the (sorted) table
  for (int t = threadIdx.x; t < n_tensors; t += blockDim.x) {
    int lo = 0, hi = n_chunks;  // first chunk with tensor >= t
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (chunks[mid].tensor < t) lo = mid + 1; else hi = mid;
    }
    float s = 0.f;
    for (int i = lo; i < n_chunks && chunks[i].tensor == t; ++i) s += partial[i];
    if (per_tensor) per_tensor[t] = s;
    tot += s;
  }
  s_total[threadIdx.x] = tot;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = 0.f;
    for (int i = 0; i < blockDim.x; ++i) r += s_total[i];
    total[0] = r;
  }
}

template <typename TA, typename TO>
__global__ void __launch_bounds__(256) mt_scale_kernel(const Chunk* chunks, float scale, int* found_inf) {
  const Chunk c = chunks[blockIdx.x];
  bool bad = false;
  for (int i = threadIdx.x; i < c.n; i += 256) {
    const float v = ld<TA>(c.a, i);
    if (!isfinite(v)) bad = true;
    st<TO>(c.out, i, v * scale);
  }
  if (bad && found_inf) *found_inf = 1;
}

template <typename TA, typename TB, typename TO>
__global__ void __launch_bounds__(256) mt_axpby_kernel(const Chunk* chunks, float a, float b) {
  const Chunk c = chunks[blockIdx.x];
  for (int i = threadIdx.x; i < c.n; i += 256) st<TO>(c.out, i, a * ld<TA>(c.a, i) + b * ld<TB>(c.b, i));
}

}  // namespace

extern "C" {

int pb_mt_chunk_bytes() { return (int)sizeof(Chunk); }

// dtype codes: 0 fp32, 1 bf16
int pb_mt_l2norm(const void* chunks, int n_chunks, int dtype_a, float* partial, float* per_tensor, int n_tensors,
                 float* total, cudaStream_t s) {
  if (n_chunks <= 0) return (int)cudaMemsetAsync(total, 0, sizeof(float), s);
  const Chunk* c = reinterpret_cast<const Chunk*>(chunks);
  if (dtype_a == 0) mt_l2norm_kernel<float><<<n_chunks, 256, 0, s>>>(c, partial);
  else mt_l2norm_kernel<__nv_bfloat16><<<n_chunks, 256, 0, s>>>(c, partial);
  mt_l2norm_final_kernel<<<1, 256, 0, s>>>(c, partial, n_chunks, per_tensor, n_tensors, total);
  return (int)cudaGetLastError();
}

int pb_mt_scale(const void* chunks, int n_chunks, int dtype_a, int dtype_o, float scale, int* found_inf,
                cudaStream_t s) {
  if (n_chunks <= 0) return 0;
  const Chunk* c = reinterpret_cast<const Chunk*>(chunks);
  if (dtype_a == 0 && dtype_o == 0) mt_scale_kernel<float, float><<<n_chunks, 256, 0, s>>>(c, scale, found_inf);
  else if (dtype_a == 0) mt_scale_kernel<float, __nv_bfloat16><<<n_chunks, 256, 0, s>>>(c, scale, found_inf);
  else if (dtype_o == 0) mt_scale_kernel<__nv_bfloat16, float><<<n_chunks, 256, 0, s>>>(c, scale, found_inf);
  else mt_scale_kernel<__nv_bfloat16, __nv_bfloat16><<<n_chunks, 256, 0, s>>>(c, scale, found_inf);
  return (int)cudaGetLastError();
}

// out = a * x + b * y; x, y share `dtype_in`
int pb_mt_axpby(const void* chunks, int n_chunks, int dtype_in, int dtype_o, float a, float b, cudaStream_t s) {
  if (n_chunks <= 0) return 0;
  const Chunk* c = reinterpret_cast<const Chunk*>(chunks);
  if (dtype_in == 0 && dtype_o == 0) mt_axpby_kernel<float, float, float><<<n_chunks, 256, 0, s>>>(c, a, b);
  else if (dtype_in == 0) mt_axpby_kernel<float, float, __nv_bfloat16><<<n_chunks, 256, 0, s>>>(c, a, b);
  else if (dtype_o == 0) mt_axpby_kernel<__nv_bfloat16, __nv_bfloat16, float><<<n_chunks, 256, 0, s>>>(c, a, b);
  else mt_axpby_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16><<<n_chunks, 256, 0, s>>>(c, a, b);
  return (int)cudaGetLastError();
}

}  // extern "C"
