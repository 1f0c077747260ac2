// Memory-bound training ops for sm_100a: RMSNorm (fwd/bwd, optional fused residual add), RoPE,
// SwiGLU (plain / routing-prob weighted / clamped), cross-entropy (fused softmax + gradient,
// vocab-parallel capable), AdamW on flat buffers, L2-norm / scale helpers.
//
// All kernels move 16 bytes per thread per access and keep fp32 math in registers; each is one
// pass over its operands except where a row statistic forces a second read (which hits L1/L2).
//
// Reference call sites these replace: rmsnorm / fused residual norm
// (primus/backends/megatron/core/extensions/primus_turbo.py:1697-1700, fused_residual_rmsnorm.py),
// TE fused RoPE and bias-SwiGLU (primus/backends/megatron/patches/te_patches/
// fused_bias_swiglu_patches.py:21), swiglu_with_probs (primus_turbo.py:1954-1980), clamped SwiGLU
// (primus/backends/megatron/core/fusions/fused_bias_swiglu.py:25-100), TE cross-entropy fusion
// and FusedAdam (primus/backends/megatron/patches/torch_fused_adam_patches.py:40-88).
#include "common.cuh"

namespace {

struct alignas(16) Bf8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void bf8_to_f(const Bf8& b, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(b.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ Bf8 f_to_bf8(const float* f) {
  Bf8 b;
#pragma unroll
  for (int i = 0; i < 4; ++i) b.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return b;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = pb::warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = (l < THREADS / 32) ? red[l] : 0.f;
  r = pb::warp_sum(r);
  return r;
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = pb::warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = (l < THREADS / 32) ? red[l] : -INFINITY;
  r = pb::warp_max(r);
  return r;
}

// ------------------------------------------------------------------ RMSNorm forward
// y = (x [+ res]) * rstd * w ; optionally writes the summed residual stream to xsum.
constexpr int RN_THREADS = 256;
// One row per CTA; VPT 16-byte vectors per thread stay in registers between the sum-of-squares pass and the scaling
// pass, so every operand is read from memory exactly once.
template <int VPT>
__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ xsum, float* __restrict__ rstd_out, int H, long ldx,
                   long ldy, float eps) {
  __shared__ float red[32];
  const long row = blockIdx.x;
  const Bf8* xr = reinterpret_cast<const Bf8*>(x + row * ldx);
  const Bf8* rr = res ? reinterpret_cast<const Bf8*>(res + row * ldx) : nullptr;
  Bf8* sr = xsum ? reinterpret_cast<Bf8*>(xsum + row * ldx) : nullptr;
  const int nv = H / 8;
  float f[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * RN_THREADS;
    if (i < nv) {
      bf8_to_f(xr[i], f[k]);
      if (rr) {
        float g[8];
        bf8_to_f(rr[i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[k][j] += g[j];
        Bf8 s = f_to_bf8(f[k]);
        sr[i] = s;
        bf8_to_f(s, f[k]);  // normalise exactly what later layers will read
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[k][j] * f[k][j];
    }
  }
  ss = block_sum<RN_THREADS>(ss, red);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  const Bf8* wr = reinterpret_cast<const Bf8*>(w);
  Bf8* yr = reinterpret_cast<Bf8*>(y + row * ldy);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * RN_THREADS;
    if (i < nv) {
      float g[8];
      bf8_to_f(wr[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[k][j] = f[k][j] * rstd * g[j];
      yr[i] = f_to_bf8(f[k]);
    }
  }
}

template <typename... Args>
void launch_rmsnorm_fwd(long rows, int H, cudaStream_t s, Args... args) {
  const int vpt = (H / 8 + RN_THREADS - 1) / RN_THREADS;
  if (vpt <= 1) rmsnorm_fwd_kernel<1><<<(unsigned)rows, RN_THREADS, 0, s>>>(args...);
  else if (vpt == 2) rmsnorm_fwd_kernel<2><<<(unsigned)rows, RN_THREADS, 0, s>>>(args...);
  else if (vpt <= 4) rmsnorm_fwd_kernel<4><<<(unsigned)rows, RN_THREADS, 0, s>>>(args...);
  else rmsnorm_fwd_kernel<8><<<(unsigned)rows, RN_THREADS, 0, s>>>(args...);
}

// ------------------------------------------------------------------ RMSNorm backward
// dx = rstd * (dy*w) - x * rstd^3 * mean(dy*w*x)  (+ dres when given)
// dw partial sums per CTA go to `partial` [gridDim.x, H]; rmsnorm_dw_reduce_kernel folds them.
// A CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; VPT 16-byte vectors per thread per row.  The next row's
// operands are fetched into registers before the current row's block reduction, so the reduction's two barriers
// overlap the loads instead of serialising with them.
template <int VPT>
__global__ void __launch_bounds__(RN_THREADS, (VPT <= 2) ? 2 : 1)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ partial, int rows, int H, long ldx, long lddy) {
  __shared__ float red[32];
  const int nv = H / 8;
  float wreg[VPT][8];
  float dw[VPT][8];
  const Bf8* wr = reinterpret_cast<const Bf8*>(w);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * RN_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[k][j] = 0.f;
    if (i < nv) bf8_to_f(wr[i], wreg[k]);
  }
  Bf8 nx[VPT], ng[VPT], nr[VPT];
  float nrs = 0.f;
  auto fetch = [&](long row) {
    const Bf8* dyr = reinterpret_cast<const Bf8*>(dy + row * lddy);
    const Bf8* xr = reinterpret_cast<const Bf8*>(x + row * ldx);
    const Bf8* drr = dres ? reinterpret_cast<const Bf8*>(dres + row * ldx) : nullptr;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * RN_THREADS;
      if (i < nv) {
        nx[k] = xr[i];
        ng[k] = dyr[i];
        if (drr) nr[k] = drr[i];
      }
    }
    nrs = rstd[row];
  };
  long row = blockIdx.x;
  if (row < rows) fetch(row);
  for (; row < rows; row += gridDim.x) {
    float fx[VPT][8], fg[VPT][8], fr[VPT][8];
    const float rs = nrs;
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * RN_THREADS;
      if (i < nv) {
        bf8_to_f(nx[k], fx[k]);
        bf8_to_f(ng[k], fg[k]);
        if (dres) bf8_to_f(nr[k], fr[k]);
      }
    }
    if (row + gridDim.x < rows) fetch(row + gridDim.x);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * RN_THREADS;
      if (i < nv) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dw[k][j] += fg[k][j] * fx[k][j] * rs;
          fg[k][j] *= wreg[k][j];
          dot += fg[k][j] * fx[k][j];
        }
      }
    }
    dot = block_sum<RN_THREADS>(dot, red);
    const float c = dot * rs * rs * rs / H;
    Bf8* dxr = reinterpret_cast<Bf8*>(dx + row * ldx);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * RN_THREADS;
      if (i < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = fg[k][j] * rs - fx[k][j] * c;
        if (dres) {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += fr[k][j];
        }
        dxr[i] = f_to_bf8(o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * RN_THREADS;
    if (i < nv) {
      float* p = partial + (long)blockIdx.x * H + (long)i * 8;
      *reinterpret_cast<float4*>(p) = make_float4(dw[k][0], dw[k][1], dw[k][2], dw[k][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(dw[k][4], dw[k][5], dw[k][6], dw[k][7]);
    }
  }
}

// Rows wider than 8192 elements (up to 16384): 8 vectors per thread; the weight is re-read per row (L1-resident) and
// nothing is prefetched, which keeps the kernel inside the register file.
__global__ void __launch_bounds__(RN_THREADS, 1)
rmsnorm_bwd_wide_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                        const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                        float* __restrict__ partial, int rows, int H, long ldx, long lddy) {
  constexpr int VPT = 8;
  __shared__ float red[32];
  const int nv = H / 8;
  float dw[VPT][8];
  const Bf8* wr = reinterpret_cast<const Bf8*>(w);
#pragma unroll
  for (int k = 0; k < VPT; ++k)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[k][j] = 0.f;
  for (long row = blockIdx.x; row < rows; row += gridDim.x) {
    const Bf8* dyr = reinterpret_cast<const Bf8*>(dy + row * lddy);
    const Bf8* xr = reinterpret_cast<const Bf8*>(x + row * ldx);
    const float rs = rstd[row];
    float fx[VPT][8], fg[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * RN_THREADS;
      if (i < nv) {
        float wv[8];
        bf8_to_f(xr[i], fx[k]);
        bf8_to_f(dyr[i], fg[k]);
        bf8_to_f(wr[i], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dw[k][j] += fg[k][j] * fx[k][j] * rs;
          fg[k][j] *= wv[j];
          dot += fg[k][j] * fx[k][j];
        }
      }
    }
    dot = block_sum<RN_THREADS>(dot, red);
    const float c = dot * rs * rs * rs / H;
    Bf8* dxr = reinterpret_cast<Bf8*>(dx + row * ldx);
    const Bf8* drr = dres ? reinterpret_cast<const Bf8*>(dres + row * ldx) : nullptr;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * RN_THREADS;
      if (i < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = fg[k][j] * rs - fx[k][j] * c;
        if (drr) {
          float r[8];
          bf8_to_f(drr[i], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        dxr[i] = f_to_bf8(o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * RN_THREADS;
    if (i < nv) {
      float* p = partial + (long)blockIdx.x * H + (long)i * 8;
      *reinterpret_cast<float4*>(p) = make_float4(dw[k][0], dw[k][1], dw[k][2], dw[k][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(dw[k][4], dw[k][5], dw[k][6], dw[k][7]);
    }
  }
}

template <typename... Args>
void launch_rmsnorm_bwd(int P, int H, cudaStream_t s, Args... args) {
  const int vpt = (H / 8 + RN_THREADS - 1) / RN_THREADS;
  if (vpt <= 1) rmsnorm_bwd_kernel<1><<<P, RN_THREADS, 0, s>>>(args...);
  else if (vpt == 2) rmsnorm_bwd_kernel<2><<<P, RN_THREADS, 0, s>>>(args...);
  else if (vpt <= 4) rmsnorm_bwd_kernel<4><<<P, RN_THREADS, 0, s>>>(args...);
  else rmsnorm_bwd_wide_kernel<<<P, RN_THREADS, 0, s>>>(args...);
}

// dw[h] (+)= sum_p partial[p, h].  A CTA owns 32 columns; its 16 thread rows each add every 16th partial (coalesced
// 128-byte reads) and a fixed-order tree in shared memory folds them, so the result does not depend on scheduling.
constexpr int DWR_COLS = 32, DWR_ROWS = 16;
__global__ void __launch_bounds__(DWR_COLS * DWR_ROWS)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int P, int H, int accumulate) {
  __shared__ float red[DWR_ROWS][DWR_COLS + 1];
  const int c = threadIdx.x % DWR_COLS, g = threadIdx.x / DWR_COLS;
  const int h = blockIdx.x * DWR_COLS + c;
  float s = 0.f;
  if (h < H)
    for (int p = g; p < P; p += DWR_ROWS) s += partial[(long)p * H + h];
  red[g][c] = s;
  __syncthreads();
#pragma unroll
  for (int step = DWR_ROWS / 2; step > 0; step >>= 1) {
    if (g < step) red[g][c] += red[g + step][c];
    __syncthreads();
  }
  if (g == 0 && h < H) dw[h] = accumulate ? dw[h] + red[0][c] : red[0][c];
}

// ------------------------------------------------------------------ logit soft-capping
// forward: y = cap * tanh(x / cap) (in place when y == x); backward: dx = dy * (1 - (y / cap)^2) from the saved output.
// Replaces the reference's Triton `fused_softcap_kernel` (primus/backends/megatron/core/extensions/logits_processor.py:13-37).
__global__ void softcap_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long nvec,
                                   float cap, float inv_cap) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float f[8];
    bf8_to_f(reinterpret_cast<const Bf8*>(x)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = cap * tanhf(f[j] * inv_cap);
    reinterpret_cast<Bf8*>(y)[i] = f_to_bf8(f);
  }
}
__global__ void softcap_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ dx, long nvec, float inv_cap) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float g[8], f[8];
    bf8_to_f(reinterpret_cast<const Bf8*>(dy)[i], g);
    bf8_to_f(reinterpret_cast<const Bf8*>(y)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float t = f[j] * inv_cap;
      g[j] *= (1.f - t * t);
    }
    reinterpret_cast<Bf8*>(dx)[i] = f_to_bf8(g);
  }
}

// ------------------------------------------------------------------ RoPE (rotate-half), in place
// x: [T, heads, d] with row pitch ld; rotates the first rot_dim channels of every head.
// pos[t] selects the row of the cos/sin tables ([max_pos, rot_dim/2] fp32). sign=-1 for backward.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, long T,
                            int heads, int d, int rot_dim, long ld, float sign) {
  const int half = rot_dim / 2;
  const int vec_per_head = half / 8;
  const long total = T * heads * vec_per_head;
  for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total;
       idx += (long)gridDim.x * blockDim.x) {
    const int v = idx % vec_per_head;
    const long th = idx / vec_per_head;
    const int h = th % heads;
    const long t = th / heads;
    const int p = pos ? pos[t] : (int)t;
    __nv_bfloat16* base = x + t * ld + (long)h * d + v * 8;
    Bf8 a = *reinterpret_cast<Bf8*>(base);
    Bf8 b = *reinterpret_cast<Bf8*>(base + half);
    float fa[8], fb[8], c[8], s[8];
    bf8_to_f(a, fa);
    bf8_to_f(b, fb);
    const float* cp = cos_t + (long)p * half + v * 8;
    const float* sp = sin_t + (long)p * half + v * 8;
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cp);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cp + 4);
    *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(sp);
    *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(sp + 4);
    float oa[8], ob[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sn = s[j] * sign;
      oa[j] = fa[j] * c[j] - fb[j] * sn;
      ob[j] = fb[j] * c[j] + fa[j] * sn;
    }
    *reinterpret_cast<Bf8*>(base) = f_to_bf8(oa);
    *reinterpret_cast<Bf8*>(base + half) = f_to_bf8(ob);
  }
}

// gated-unit activations: kind 0 = SiLU (SwiGLU), 1 = tanh-approximated GELU (GEGLU)
__device__ __forceinline__ float gate_act(float g, int kind, float& dact) {
  if (kind == 0) {
    const float sig = pb::fast_sigmoid(g);
    dact = sig * (1.f + g * (1.f - sig));
    return g * sig;
  }
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (g + k1 * g * g * g));
  dact = 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
  return 0.5f * g * (1.f + t);
}

// ------------------------------------------------------------------ SwiGLU
// in: [T, 2I] = [gate | up]; out[T, I] = silu(min(g,clamp)) * clip(u,+-clamp) * prob[t]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in, const float* __restrict__ probs,
                                  __nv_bfloat16* __restrict__ out, long T, int I, float clamp, int kind) {
  const int vec_per_row = I / 8;
  const long total = T * vec_per_row;
  for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total;
       idx += (long)gridDim.x * blockDim.x) {
    const long t = idx / vec_per_row;
    const int v = idx % vec_per_row;
    const __nv_bfloat16* g = in + t * 2L * I + v * 8;
    float fg[8], fu[8], o[8];
    bf8_to_f(*reinterpret_cast<const Bf8*>(g), fg);
    bf8_to_f(*reinterpret_cast<const Bf8*>(g + I), fu);
    const float p = probs ? probs[t] : 1.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gg = fg[j], uu = fu[j];
      if (clamp > 0.f) {
        gg = fminf(gg, clamp);
        uu = fminf(fmaxf(uu, -clamp), clamp);
      }
      if (kind == 0) {
        const float sig = pb::fast_sigmoid(gg);
        o[j] = gg * sig * uu * p;
      } else {
        float unused;
        o[j] = gate_act(gg, kind, unused) * uu * p;
      }
    }
    *reinterpret_cast<Bf8*>(out + t * (long)I + v * 8) = f_to_bf8(o);
  }
}

// din[T,2I] from dy[T,I]; dprobs[t] = sum_i dy * silu(g) * u (one warp per row when probs given)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ in,
                                  const float* __restrict__ probs, __nv_bfloat16* __restrict__ din,
                                  float* __restrict__ dprobs, long T, int I, float clamp, int kind) {
  const int vec_per_row = I / 8;
  const int lane = threadIdx.x & 31;
  const long warp_global = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const long num_warps = ((long)gridDim.x * blockDim.x) >> 5;
  for (long t = warp_global; t < T; t += num_warps) {
    const float p = probs ? probs[t] : 1.f;
    float dp = 0.f;
    for (int v = lane; v < vec_per_row; v += 32) {
      const __nv_bfloat16* g = in + t * 2L * I + v * 8;
      float fg[8], fu[8], fd[8], og[8], ou[8];
      bf8_to_f(*reinterpret_cast<const Bf8*>(g), fg);
      bf8_to_f(*reinterpret_cast<const Bf8*>(g + I), fu);
      bf8_to_f(*reinterpret_cast<const Bf8*>(dy + t * (long)I + v * 8), fd);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float gg = fg[j], uu = fu[j];
        float gmask = 1.f, umask = 1.f;
        if (clamp > 0.f) {
          if (gg > clamp) { gg = clamp; gmask = 0.f; }
          if (uu > clamp) { uu = clamp; umask = 0.f; }
          if (uu < -clamp) { uu = -clamp; umask = 0.f; }
        }
        float sl, dsl;
        if (kind == 0) {
          const float sig = pb::fast_sigmoid(gg);
          sl = gg * sig;
          dsl = sig * (1.f + gg * (1.f - sig));
        } else {
          sl = gate_act(gg, kind, dsl);
        }
        dp += fd[j] * sl * uu;
        const float d = fd[j] * p;
        og[j] = d * uu * dsl * gmask;
        ou[j] = d * sl * umask;
      }
      __nv_bfloat16* o = din + t * 2L * I + v * 8;
      *reinterpret_cast<Bf8*>(o) = f_to_bf8(og);
      *reinterpret_cast<Bf8*>(o + I) = f_to_bf8(ou);
    }
    if (dprobs) {
      dp = pb::warp_sum(dp);
      if (lane == 0) dprobs[t] = dp;
    }
  }
}

// ------------------------------------------------------------------ cross entropy
// Phase 1: per-row local max, sum(exp(x - max)) and the target logit when the label falls into
// this rank's vocabulary slice [vocab_start, vocab_start + V).
constexpr int CE_THREADS = 1024;
__global__ void __launch_bounds__(CE_THREADS)
ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, const long* __restrict__ labels,
                float* __restrict__ row_max, float* __restrict__ row_sumexp,
                float* __restrict__ tgt_logit, int V, long ld, int vocab_start) {
  __shared__ float red[32];
  const long row = blockIdx.x;
  const Bf8* lr = reinterpret_cast<const Bf8*>(logits + row * ld);
  const int nv = V / 8;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nv; i += CE_THREADS) {
    float f[8];
    bf8_to_f(lr[i], f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  const float gm = block_max<CE_THREADS>(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = block_sum<CE_THREADS>(s, red);
  if (threadIdx.x == 0) {
    row_max[row] = gm;
    row_sumexp[row] = s;
    const long lab = labels[row] - vocab_start;
    tgt_logit[row] = (lab >= 0 && lab < V) ? __bfloat162float(logits[row * ld + lab]) : 0.f;
  }
}

// Phase 2: logits <- (softmax - onehot) * gscale[row]  (in place), given the global log-sum-exp.
__global__ void __launch_bounds__(CE_THREADS)
ce_grad_kernel(__nv_bfloat16* __restrict__ logits, const long* __restrict__ labels,
               const float* __restrict__ lse, const float* __restrict__ gscale, int V, long ld,
               int vocab_start) {
  const long row = blockIdx.x;
  Bf8* lr = reinterpret_cast<Bf8*>(logits + row * ld);
  const int nv = V / 8;
  const float l = lse[row];
  const float sc = gscale[row];
  const long lab = labels[row] - vocab_start;
  for (int i = threadIdx.x; i < nv; i += CE_THREADS) {
    float f[8];
    bf8_to_f(lr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - l);
      if ((long)i * 8 + j == lab) p -= 1.f;
      f[j] = p * sc;
    }
    lr[i] = f_to_bf8(f);
  }
}

// Single-rank fused form: loss[row] = lse - target, gradient written in place.
__global__ void __launch_bounds__(CE_THREADS)
ce_fused_kernel(__nv_bfloat16* __restrict__ logits, const long* __restrict__ labels,
                const float* __restrict__ gscale, float* __restrict__ loss, int V, long ld) {
  __shared__ float red[32];
  const long row = blockIdx.x;
  Bf8* lr = reinterpret_cast<Bf8*>(logits + row * ld);
  const int nv = V / 8;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nv; i += CE_THREADS) {
    float f[8];
    bf8_to_f(lr[i], f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  const float gm = block_max<CE_THREADS>(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = block_sum<CE_THREADS>(s, red);
  const float l = gm + __logf(s);
  const long lab = labels[row];
  if (threadIdx.x == 0) {
    const float t = (lab >= 0 && lab < V) ? __bfloat162float(logits[row * ld + lab]) : l;
    loss[row] = l - t;
  }
  __syncthreads();  // the target logit must be read before it is overwritten
  const float sc = gscale[row];
  for (int i = threadIdx.x; i < nv; i += CE_THREADS) {
    float f[8];
    bf8_to_f(lr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - l);
      if ((long)i * 8 + j == lab) p -= 1.f;
      f[j] = p * sc;
    }
    lr[i] = f_to_bf8(f);
  }
}

// ------------------------------------------------------------------ optimizer / flat-buffer helpers
// AdamW over a flat shard. grads are multiplied by *grad_scale (device scalar: clip coefficient x
// 1/loss-scale). When *skip != 0 (non-finite gradients found) nothing is updated.
__device__ __forceinline__ void load4(const float* p, float* o) {
  *reinterpret_cast<float4*>(o) = *reinterpret_cast<const float4*>(p);
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* o) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(p);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float* o) {
  *reinterpret_cast<float4*>(p) = *reinterpret_cast<const float4*>(o);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float* o) {
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(p);
  h[0] = __floats2bfloat162_rn(o[0], o[1]);
  h[1] = __floats2bfloat162_rn(o[2], o[3]);
}
__device__ __forceinline__ void store1(float* p, float o) { *p = o; }
__device__ __forceinline__ void store1(__nv_bfloat16* p, float o) { *p = __float2bfloat16(o); }

// GradT: fp32 or bf16 gradients; StateT: fp32 or bf16 moments (precision-aware optimizer: the moments can be kept in
// bf16 to halve their memory; the arithmetic is fp32 either way and the master weights stay fp32).
template <typename GradT, typename StateT>
__global__ void adamw_kernel(float* __restrict__ master, StateT* __restrict__ m, StateT* __restrict__ v,
                             const GradT* __restrict__ grad, __nv_bfloat16* __restrict__ param_out,
                             long n, float lr, float beta1, float beta2, float eps, float wd,
                             float bc1, float bc2, const float* __restrict__ grad_scale,
                             const int* __restrict__ skip) {
  if (skip && *skip) return;
  const float gs = grad_scale ? *grad_scale : 1.f;
  for (long i = (blockIdx.x * (long)blockDim.x + threadIdx.x) * 4; i < n;
       i += (long)gridDim.x * blockDim.x * 4) {
    float p[4], mm[4], vv[4], g[4];
    const bool full = i + 4 <= n;
    if (full) {
      load4(master + i, p);
      load4(m + i, mm);
      load4(v + i, vv);
      load4(grad + i, g);
    } else {
      for (int j = 0; j < 4; ++j) {
        const bool in = i + j < n;
        p[j] = in ? master[i + j] : 0.f;
        mm[j] = in ? (float)m[i + j] : 0.f;
        vv[j] = in ? (float)v[i + j] : 0.f;
        g[j] = in ? (float)grad[i + j] : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gg = g[j] * gs;
      mm[j] = beta1 * mm[j] + (1.f - beta1) * gg;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gg * gg;
      const float mh = mm[j] / bc1;
      const float vh = vv[j] / bc2;
      p[j] = p[j] * (1.f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
    }
    if (full) {
      store4(master + i, p);
      store4(m + i, mm);
      store4(v + i, vv);
      if (param_out) store4(param_out + i, p);
    } else {
      for (int j = 0; j < 4 && i + j < n; ++j) {
        master[i + j] = p[j];
        store1(m + i + j, mm[j]);
        store1(v + i + j, vv[j]);
        if (param_out) param_out[i + j] = __float2bfloat16(p[j]);
      }
    }
  }
}

// partial[b] = sum of squares handled by block b (deterministic two-stage reduction)
template <typename T>
__global__ void __launch_bounds__(512) sumsq_partial_kernel(const T* __restrict__ x, long n,
                                                           float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float f = (float)x[i];
    s += f * f;
  }
  s = block_sum<512>(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// out[0] (+)= sum(partial); nonfinite[0] |= !isfinite(sum)
__global__ void __launch_bounds__(512) sumsq_final_kernel(const float* __restrict__ partial, int P,
                                                         float* __restrict__ out, int accumulate,
                                                         int* __restrict__ nonfinite) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s += partial[i];
  s = block_sum<512>(s, red);
  if (threadIdx.x == 0) {
    const float r = accumulate ? out[0] + s : s;
    out[0] = r;
    if (nonfinite && !isfinite(r)) *nonfinite = 1;
  }
}
// coef = min(1, max_norm / (sqrt(sumsq) + 1e-6)) * extra
__global__ void clip_coef_kernel(const float* sumsq, float max_norm, float extra, float* coef,
                                 float* norm_out) {
  const float nrm = sqrtf(sumsq[0]);
  if (norm_out) norm_out[0] = nrm;
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (nrm + 1e-6f));
  coef[0] = c * extra;
}

__global__ void scale_f32_kernel(float* __restrict__ x, long n, float s) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    x[i] *= s;
}
__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long n) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16(x[i]);
}
// dst(fp32) += src(bf16)   (flat; used to fold bf16 gradients into fp32 main grads)
__global__ void add_bf16_into_f32_kernel(float* __restrict__ dst, const __nv_bfloat16* __restrict__ src, long n) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    dst[i] += __bfloat162float(src[i]);
}
// embedding backward: dW[token[t], :] += dy[t, :]  (fp32 atomics)
__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const long* __restrict__ tokens,
                                     float* __restrict__ dw, long T, int H, int vocab_start, int vocab) {
  const long total = T * (H / 2);
  for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total;
       idx += (long)gridDim.x * blockDim.x) {
    const long t = idx / (H / 2);
    const int c = (idx % (H / 2)) * 2;
    const long tok = tokens[t] - vocab_start;
    if (tok < 0 || tok >= vocab) continue;
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dy + t * H + c));
    atomicAdd(dw + tok * H + c, g.x);
    atomicAdd(dw + tok * H + c + 1, g.y);
  }
}

inline int grid_for(long work_items, int threads, int cap = 148 * 16) {
  long g = (work_items + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return (int)g;
}

}  // namespace

#define PB_CHECK_LAUNCH() return (int)cudaGetLastError()

extern "C" {

int pb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* xsum, float* rstd,
                   long rows, int H, long ldx, long ldy, float eps, cudaStream_t s) {
  if (H % 8 || ldx % 8 || ldy % 8 || H > 8 * 8 * RN_THREADS) return -2;
  if (rows == 0) return 0;
  launch_rmsnorm_fwd(rows, H, s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,
                     (__nv_bfloat16*)y, (__nv_bfloat16*)xsum, rstd, H, ldx, ldy, eps);
  PB_CHECK_LAUNCH();
}

// Number of CTAs (= rows of the [P, H] fp32 scratch) the backward uses for a given row count.
int pb_rmsnorm_bwd_num_partials(long rows) { return (int)(rows < 592 ? (rows < 1 ? 1 : rows) : 592); }

// scratch: fp32 [pb_rmsnorm_bwd_num_partials(rows), H]. dw_accumulate: 1 -> dw += result.
int pb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                   void* dx, float* dw, float* scratch, long rows, int H, long ldx, long lddy,
                   int dw_accumulate, cudaStream_t s) {
  if (H % 8 || ldx % 8 || lddy % 8 || H > 16384 || rows < 0 || rows > 2147483647L) return -2;   // 32-bit row indices
  if (rows == 0) return 0;
  const int P = pb_rmsnorm_bwd_num_partials(rows);
  launch_rmsnorm_bwd(P, H, s, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,
                     (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, scratch, (int)rows, H, ldx, lddy);
  rmsnorm_dw_reduce_kernel<<<(H + DWR_COLS - 1) / DWR_COLS, DWR_COLS * DWR_ROWS, 0, s>>>(scratch, dw, P, H, dw_accumulate);
  PB_CHECK_LAUNCH();
}

int pb_rope(void* x, const int* pos, const float* cos_t, const float* sin_t, long T, int heads, int d,
            int rot_dim, long ld, int backward, cudaStream_t s) {
  if (rot_dim % 16 || ld % 8 || d % 8) return -2;
  const long total = T * heads * (rot_dim / 16);
  if (total == 0) return 0;
  rope_kernel<<<grid_for(total, 256), 256, 0, s>>>((__nv_bfloat16*)x, pos, cos_t, sin_t, T, heads, d,
                                                  rot_dim, ld, backward ? -1.f : 1.f);
  PB_CHECK_LAUNCH();
}

int pb_softcap_fwd(const void* x, void* y, long n, float cap, cudaStream_t s) {
  if (n % 8 || cap <= 0.f) return -2;
  if (n == 0) return 0;
  softcap_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n / 8, cap,
                                                         1.f / cap);
  PB_CHECK_LAUNCH();
}

int pb_softcap_bwd(const void* dy, const void* y, void* dx, long n, float cap, cudaStream_t s) {
  if (n % 8 || cap <= 0.f) return -2;
  if (n == 0) return 0;
  softcap_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)y,
                                                         (__nv_bfloat16*)dx, n / 8, 1.f / cap);
  PB_CHECK_LAUNCH();
}

// kind: 0 SiLU gate (SwiGLU), 1 tanh-GELU gate (GEGLU)
int pb_swiglu_fwd(const void* in, const float* probs, void* out, long T, int I, float clamp, int kind, cudaStream_t s) {
  if (I % 8) return -2;
  if (T == 0) return 0;
  swiglu_fwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, s>>>((const __nv_bfloat16*)in, probs,
                                                              (__nv_bfloat16*)out, T, I, clamp, kind);
  PB_CHECK_LAUNCH();
}

int pb_swiglu_bwd(const void* dy, const void* in, const float* probs, void* din, float* dprobs, long T,
                  int I, float clamp, int kind, cudaStream_t s) {
  if (I % 8) return -2;
  if (T == 0) return 0;
  swiglu_bwd_kernel<<<grid_for(T * 32, 256), 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)in,
                                                         probs, (__nv_bfloat16*)din, dprobs, T, I, clamp, kind);
  PB_CHECK_LAUNCH();
}

int pb_ce_stats(const void* logits, const long* labels, float* row_max, float* row_sumexp, float* tgt,
                long rows, int V, long ld, int vocab_start, cudaStream_t s) {
  if (V % 8 || ld % 8) return -2;
  if (rows == 0) return 0;
  ce_stats_kernel<<<(unsigned)rows, CE_THREADS, 0, s>>>((const __nv_bfloat16*)logits, labels, row_max,
                                                       row_sumexp, tgt, V, ld, vocab_start);
  PB_CHECK_LAUNCH();
}

int pb_ce_grad(void* logits, const long* labels, const float* lse, const float* gscale, long rows, int V,
               long ld, int vocab_start, cudaStream_t s) {
  if (V % 8 || ld % 8) return -2;
  if (rows == 0) return 0;
  ce_grad_kernel<<<(unsigned)rows, CE_THREADS, 0, s>>>((__nv_bfloat16*)logits, labels, lse, gscale, V, ld,
                                                      vocab_start);
  PB_CHECK_LAUNCH();
}

int pb_ce_fused(void* logits, const long* labels, const float* gscale, float* loss, long rows, int V,
                long ld, cudaStream_t s) {
  if (V % 8 || ld % 8) return -2;
  if (rows == 0) return 0;
  ce_fused_kernel<<<(unsigned)rows, CE_THREADS, 0, s>>>((__nv_bfloat16*)logits, labels, gscale, loss, V, ld);
  PB_CHECK_LAUNCH();
}

// state_is_bf16: the moments m, v are bf16 tensors (else fp32).
int pb_adamw_ex(float* master, void* m, void* v, const void* grad, int grad_is_bf16, int state_is_bf16,
                void* param_out, long n, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                const float* grad_scale, const int* skip, cudaStream_t s) {
  if (n == 0) return 0;
  const int g = grid_for((n + 3) / 4, 256, 148 * 8);
  __nv_bfloat16* po = (__nv_bfloat16*)param_out;
#define PB_ADAMW(GT, ST)                                                                                          \
  adamw_kernel<GT, ST><<<g, 256, 0, s>>>(master, (ST*)m, (ST*)v, (const GT*)grad, po, n, lr, beta1, beta2, eps, wd, \
                                         bc1, bc2, grad_scale, skip)
  if (grad_is_bf16 && state_is_bf16) PB_ADAMW(__nv_bfloat16, __nv_bfloat16);
  else if (grad_is_bf16) PB_ADAMW(__nv_bfloat16, float);
  else if (state_is_bf16) PB_ADAMW(float, __nv_bfloat16);
  else PB_ADAMW(float, float);
#undef PB_ADAMW
  PB_CHECK_LAUNCH();
}

int pb_adamw(float* master, float* m, float* v, const void* grad, int grad_is_bf16, void* param_out,
             long n, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
             const float* grad_scale, const int* skip, cudaStream_t s) {
  return pb_adamw_ex(master, m, v, grad, grad_is_bf16, 0, param_out, n, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale,
                     skip, s);
}

int pb_sumsq_num_partials() { return 1184; }

// out[0] (+)= sum(x^2). scratch: fp32 [pb_sumsq_num_partials()].
int pb_sumsq(const void* x, int is_bf16, long n, float* scratch, float* out, int accumulate,
             int* nonfinite, cudaStream_t s) {
  const int P = pb_sumsq_num_partials();
  if (is_bf16)
    sumsq_partial_kernel<__nv_bfloat16><<<P, 512, 0, s>>>((const __nv_bfloat16*)x, n, scratch);
  else
    sumsq_partial_kernel<float><<<P, 512, 0, s>>>((const float*)x, n, scratch);
  sumsq_final_kernel<<<1, 512, 0, s>>>(scratch, P, out, accumulate, nonfinite);
  PB_CHECK_LAUNCH();
}

int pb_clip_coef(const float* sumsq, float max_norm, float extra, float* coef, float* norm_out,
                 cudaStream_t s) {
  clip_coef_kernel<<<1, 1, 0, s>>>(sumsq, max_norm, extra, coef, norm_out);
  PB_CHECK_LAUNCH();
}

int pb_scale_f32(float* x, long n, float sc, cudaStream_t s) {
  if (n == 0) return 0;
  scale_f32_kernel<<<grid_for(n, 256), 256, 0, s>>>(x, n, sc);
  PB_CHECK_LAUNCH();
}
int pb_cast_f32_bf16(const float* x, void* y, long n, cudaStream_t s) {
  if (n == 0) return 0;
  cast_f32_bf16_kernel<<<grid_for(n, 256), 256, 0, s>>>(x, (__nv_bfloat16*)y, n);
  PB_CHECK_LAUNCH();
}
int pb_add_bf16_into_f32(float* dst, const void* src, long n, cudaStream_t s) {
  if (n == 0) return 0;
  add_bf16_into_f32_kernel<<<grid_for(n, 256), 256, 0, s>>>(dst, (const __nv_bfloat16*)src, n);
  PB_CHECK_LAUNCH();
}
int pb_embedding_bwd(const void* dy, const long* tokens, float* dw, long T, int H, int vocab_start,
                     int vocab, cudaStream_t s) {
  if (H % 2) return -2;
  if (T == 0) return 0;
  embedding_bwd_kernel<<<grid_for(T * (H / 2), 256), 256, 0, s>>>((const __nv_bfloat16*)dy, tokens, dw, T, H,
                                                                 vocab_start, vocab);
  PB_CHECK_LAUNCH();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of pb_rmsnorm_bwd (declared in primus_b200_noalloc.h).
//
// For callers that cannot allocate at the call site (a host application that owns every cudaMalloc,
// a pre-planned memory arena, a latency-critical loop): the partial weight gradients go to a fixed
// array in this library's device image rather than to caller-provided scratch.  Host code must not
// pass the array's name to a kernel (on the host that name is only a stand-in for the symbol); its
// device address is looked up once per device with cudaGetSymbolAddress, with that device current.
#include "primus_b200_noalloc.h"

namespace {
static __device__ __align__(256) float g_noalloc_rmsnorm_partials[(long)PB_NOALLOC_MAX_PARTIALS * PB_NOALLOC_MAX_H];
constexpr int kMaxDevices = 64;
float* g_noalloc_scratch_ptr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" int pb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                      const void* dres, void* dx, float* dw, long rows, int H, long ldx,
                                      long lddy, int dw_accumulate, cudaStream_t s) {
  // the kernels index rows with 32-bit integers: more than INT_MAX rows are rejected rather than truncated
  if (H <= 0 || H % 8 || ldx % 8 || lddy % 8 || rows < 0 || rows > 2147483647L) return PB_NOALLOC_ERR_BAD_ARG;
  if (H > PB_NOALLOC_MAX_H) return PB_NOALLOC_ERR_TOO_LARGE;  // the built-in scratch holds rows of <= 8192 floats
  if (rows == 0) return 0;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return PB_NOALLOC_ERR_BAD_ARG;
  if (!g_noalloc_scratch_ptr[dev]) {
    // once per device: device address of the scratch array of the image loaded on *this* device
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_rmsnorm_partials);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_scratch_ptr[dev] = p;
  }
  float* scratch = g_noalloc_scratch_ptr[dev];
  const int P = (int)(rows < PB_NOALLOC_MAX_PARTIALS ? rows : PB_NOALLOC_MAX_PARTIALS);
  // every one of the P partial rows is fully written by its CTA before the reduction reads it
  launch_rmsnorm_bwd(P, H, s, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,
                     (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, scratch, (int)rows, H, ldx, lddy);
  rmsnorm_dw_reduce_kernel<<<(H + DWR_COLS - 1) / DWR_COLS, DWR_COLS * DWR_ROWS, 0, s>>>(scratch, dw, P, H, dw_accumulate);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// MoE token movement.
//   moe_gather_rows : out[r, :] = x[src[r], :] (* scale[r])   (src[r] < 0 -> zero row: expert padding)
//   moe_combine_rows: out[t, :] = sum_k y[pos[t, k], :]        (pos < 0 skipped)  -- the un-weighted top-k
//                     combine (routing probabilities are applied inside the expert activation) and, read
//                     the other way round, the backward of the gather.
// One warp moves one row with 16-byte accesses.  Replaces the permutation kernels of
// primus/backends/transformer_engine/pytorch/common/triton/permutation.py:189-305.
namespace {

__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src,
                                       const float* __restrict__ scale, __nv_bfloat16* __restrict__ out, long R,
                                       int H, const int* __restrict__ limit_rows) {
  const int lane = threadIdx.x & 31;
  const long warp_global = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const long num_warps = ((long)gridDim.x * blockDim.x) >> 5;
  const long lim = limit_rows ? (long)limit_rows[0] : R;
  const int nv = H / 8;
  for (long r = warp_global; r < R && r < lim; r += num_warps) {
    const int s = src[r];
    Bf8* o = reinterpret_cast<Bf8*>(out + r * H);
    if (s < 0) {
      Bf8 z;
#pragma unroll
      for (int i = 0; i < 4; ++i) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
      for (int v = lane; v < nv; v += 32) o[v] = z;
      continue;
    }
    const Bf8* in = reinterpret_cast<const Bf8*>(x + (long)s * H);
    if (scale) {
      const float sc = scale[r];
      for (int v = lane; v < nv; v += 32) {
        float f[8];
        bf8_to_f(in[v], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= sc;
        o[v] = f_to_bf8(f);
      }
    } else {
      for (int v = lane; v < nv; v += 32) o[v] = in[v];
    }
  }
}

__global__ void moe_combine_rows_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos,
                                        __nv_bfloat16* __restrict__ out, long T, int topk, int H) {
  const int lane = threadIdx.x & 31;
  const long warp_global = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const long num_warps = ((long)gridDim.x * blockDim.x) >> 5;
  const int nv = H / 8;
  for (long t = warp_global; t < T; t += num_warps) {
    Bf8* o = reinterpret_cast<Bf8*>(out + t * H);
    for (int v = lane; v < nv; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < topk; ++k) {
        const int p = pos[t * topk + k];
        if (p < 0) continue;
        float f[8];
        bf8_to_f(reinterpret_cast<const Bf8*>(y + (long)p * H)[v], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
      o[v] = f_to_bf8(acc);
    }
  }
}

}  // namespace

extern "C" int pb_moe_gather_rows(const void* x, const int* src, const float* scale, void* out, long R, int H,
                                  const int* limit_rows, cudaStream_t s) {
  if (H % 8) return -2;
  if (R == 0) return 0;
  moe_gather_rows_kernel<<<grid_for(R * 32, 256), 256, 0, s>>>((const __nv_bfloat16*)x, src, scale,
                                                              (__nv_bfloat16*)out, R, H, limit_rows);
  return (int)cudaGetLastError();
}

extern "C" int pb_moe_combine_rows(const void* y, const int* pos, void* out, long T, int topk, int H,
                                   cudaStream_t s) {
  if (H % 8) return -2;
  if (T == 0) return 0;
  moe_combine_rows_kernel<<<grid_for(T * 32, 256), 256, 0, s>>>((const __nv_bfloat16*)y, pos, (__nv_bfloat16*)out, T,
                                                               topk, H);
  return (int)cudaGetLastError();
}
