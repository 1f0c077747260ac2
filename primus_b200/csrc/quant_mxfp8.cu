// MXFP8 quantisation: bf16 [R, C] -> E4M3 values with one UE8M0 (power-of-two) scale per 32 elements, in one
// pass for both directions a training GEMM needs:
//   row-wise : blocks of 32 along C (operand reduced over C: forward / data-gradient inputs)
//   col-wise : blocks of 32 along R (operand reduced over R: weight-gradient inputs, transposed use)
// Values keep the [R, C] layout in both cases.  Scales are written directly in the layout tcgen05 block-scaled
// MMAs consume from TMEM: the operand's non-reduced dimension MN and reduced dimension K are tiled in
// 128 x 128-element blocks of 512 bytes, block (mn / 128, k / 128) stored K-fastest, and inside a block
//   offset(mn, kb) = (mn % 32) * 16 + ((mn % 128) / 32) * 4 + kb            (kb = (k % 128) / 32)
// so a block is exactly what one `tcgen05.cp.32x128b.warpx4` moves from shared memory into 4 TMEM columns.
//
// Scale: e = ceil(log2(amax / 448)) (rounded up so that nothing saturates), stored biased by 127;
// value = RN-even E4M3 of x * 2^-e.
//
// Replaces the Turbo / Transformer-Engine MXFP8 cast kernels
// (primus/backends/megatron/core/extensions/primus_turbo.py: `pt.ops.quantize` users, float8 recipe mxfp8).
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

constexpr int TILE = 128;
constexpr int PITCH = TILE + 8;  // bf16 elements per shared-memory row (272 B: conflict-free 16-byte row reads)

__device__ __forceinline__ int e8m0_from_amax(float amax) {
  const float v = amax * (1.0f / 448.0f);
  const uint32_t b = __float_as_uint(v);
  int e = (int)((b >> 23) & 0xff);        // biased exponent of v
  if (b & 0x7fffff) e += 1;               // ceil for non powers of two
  if (e < 0) e = 0;
  if (e > 254) e = 254;
  return (amax == 0.f) ? 0 : e;           // biased UE8M0
}
__device__ __forceinline__ float inv_scale_from_e8m0(int biased) {
  int f = 254 - biased;                   // exponent field of 2^-(biased - 127)
  if (f < 1) f = 1;
  return __uint_as_float((uint32_t)f << 23);
}
__device__ __forceinline__ uint16_t cvt2(float a, float b) {
  return (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}

// MXFP4 numerics on the FP8 data path: the block exponent leaves the block maximum at or below 6 (the largest E2M1
// magnitude), values are rounded to E2M1 (RN-even, saturating) and stored as the E4M3 byte of the same number (every
// E2M1 value is exact in E4M3), so the block-scaled FP8 GEMM consumes them unchanged.
__device__ __forceinline__ int e8m0_from_amax_fp4(float amax) {
  const float v = amax * (1.0f / 6.0f);
  const uint32_t b = __float_as_uint(v);
  int e = (int)((b >> 23) & 0xff);
  if (b & 0x7fffff) e += 1;
  if (e < 0) e = 0;
  if (e > 254) e = 254;
  return (amax == 0.f) ? 0 : e;
}
__device__ __forceinline__ uint16_t cvt2_fp4(float a, float b) {
  const uint32_t packed = (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(a, b), __NV_E2M1, cudaRoundNearest);
  // E2M1 code (sign, 3 magnitude bits: 0, 0.5, 1, 1.5, 2, 3, 4, 6) -> E4M3 byte of the same value
  constexpr unsigned long long lut = 0x4C4844403C383000ull;
  const uint32_t c0 = packed & 0xf, c1 = (packed >> 4) & 0xf;
  const uint32_t b0 = (uint32_t)((lut >> (8 * (c0 & 7))) & 0xff) | ((c0 & 8) << 4);
  const uint32_t b1 = (uint32_t)((lut >> (8 * (c1 & 7))) & 0xff) | ((c1 & 8) << 4);
  return (uint16_t)(b0 | (b1 << 8));
}
template <bool FP4>
__device__ __forceinline__ uint16_t cvt2_sel(float a, float b) {
  return FP4 ? cvt2_fp4(a, b) : cvt2(a, b);
}
template <bool FP4>
__device__ __forceinline__ int e8m0_sel(float amax) {
  return FP4 ? e8m0_from_amax_fp4(amax) : e8m0_from_amax(amax);
}

__device__ __forceinline__ long sf_offset(int mn, int k_blk32, int k_groups) {
  // block (mn / 128, k_blk32 / 4), K-fastest
  return ((long)(mn >> 7) * k_groups + (k_blk32 >> 2)) * 512 + (mn & 31) * 16 + ((mn & 127) >> 5) * 4 + (k_blk32 & 3);
}

constexpr int QUANT_SMEM = TILE * PITCH * 2;   // one staged bf16 tile; the fp8 results go from registers to global

// Quantises the 128 x 128 bf16 tile staged in `tile` (row pitch PITCH) whose origin in the [R, C] tensor is
// (row0, col0).  Called by all threads of a 256-thread CTA after the tile is complete (caller synchronises before).
// Results are written straight from registers: 64 contiguous bytes per thread in the row direction, 8 bytes per row
// (64 contiguous bytes per 8 lanes) in the column direction -- whole 32-byte sectors either way.
// MODE selects where a block of 32 takes its scale exponent from:
//   SCALE_BLOCK32 its own maximum (MXFP8);
//   SCALE_FIXED   `fixed_e` for every block (one power-of-two scale for the tensor, or for this 128 x 128 tile);
//   SCALE_VEC128  `e_rowv[r]` for the blocks of tile row r (row direction) and `e_colv[c]` for those of tile column c
//                 (column direction): one scale per 1 x 128 / 128 x 1 vector, written into its four 32-blocks.
enum { SCALE_BLOCK32 = 0, SCALE_FIXED = 1, SCALE_VEC128 = 2 };
template <int MODE = SCALE_BLOCK32, bool FP4 = false>
__device__ __forceinline__ void quantize_staged_tile(const __nv_bfloat16* tile, int R, int C,
                                                     int row0, int col0, uint8_t* __restrict__ q_row,
                                                     uint8_t* __restrict__ sf_row, uint8_t* __restrict__ q_col,
                                                     uint8_t* __restrict__ sf_col, int fixed_e = 0,
                                                     const uint8_t* e_rowv = nullptr, const uint8_t* e_colv = nullptr) {
  const int tid = threadIdx.x;
  if (q_row) {
    // thread -> (row r, two 32-element blocks): 64 contiguous bytes of the row
    const int r = tid & 127, half = tid >> 7;
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
      const int j = half * 2 + jj;
      float f[32];
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const uint4 d = *reinterpret_cast<const uint4*>(&tile[r * PITCH + j * 32 + v * 8]);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 t = __bfloat1622float2(h[u]);
          f[v * 8 + 2 * u] = t.x;
          f[v * 8 + 2 * u + 1] = t.y;
        }
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(f[i]));
      const int e = MODE == SCALE_FIXED ? fixed_e : (MODE == SCALE_VEC128 ? (int)e_rowv[r] : e8m0_sel<FP4>(amax));
      const float inv = inv_scale_from_e8m0(e);
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        w[i] = (uint32_t)cvt2_sel<FP4>(f[4 * i] * inv, f[4 * i + 1] * inv) |
               ((uint32_t)cvt2_sel<FP4>(f[4 * i + 2] * inv, f[4 * i + 3] * inv) << 16);
      uint4* dst = reinterpret_cast<uint4*>(q_row + (long)(row0 + r) * C + col0 + j * 32);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
      sf_row[sf_offset(row0 + r, (col0 >> 5) + j, C >> 7)] = (uint8_t)e;
    }
  }
  if (q_col) {
    // warp -> (64-column half, 32-row block); lane -> (8-column group cg, row subset sub): rows 4*sub + j and
    // 16 + 4*sub + j (j < 4), so that the two subsets sharing a shared-memory wavefront sit 64 bytes apart in the
    // banks.  One 16-byte load and one 8-byte store per row; the column maxima are reduced across the four subsets
    // with two shuffles on packed bf16 pairs.
    const int lane = tid & 31, warp = tid >> 5;
    const int cg = lane & 7, sub = lane >> 3;
    const int cbase = (warp & 1) * 64 + cg * 8;
    const int ib = warp >> 1;
    uint4 d[8];
    __nv_bfloat162 m[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) m[u] = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = ib * 32 + (i >> 2) * 16 + sub * 4 + (i & 3);
      d[i] = *reinterpret_cast<const uint4*>(&tile[r * PITCH + cbase]);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&d[i]);
#pragma unroll
      for (int u = 0; u < 4; ++u) m[u] = __hmax2(m[u], __habs2(h[u]));
    }
    float inv[8];
    int e[8];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t w = *reinterpret_cast<uint32_t*>(&m[u]);
      uint32_t o = __shfl_xor_sync(0xffffffffu, w, 8);
      m[u] = __hmax2(m[u], *reinterpret_cast<__nv_bfloat162*>(&o));
      w = *reinterpret_cast<uint32_t*>(&m[u]);
      o = __shfl_xor_sync(0xffffffffu, w, 16);
      m[u] = __hmax2(m[u], *reinterpret_cast<__nv_bfloat162*>(&o));
      const float2 a = __bfloat1622float2(m[u]);
      e[2 * u] = MODE == SCALE_FIXED ? fixed_e : (MODE == SCALE_VEC128 ? (int)e_colv[cbase + 2 * u] : e8m0_sel<FP4>(a.x));
      e[2 * u + 1] =
          MODE == SCALE_FIXED ? fixed_e : (MODE == SCALE_VEC128 ? (int)e_colv[cbase + 2 * u + 1] : e8m0_sel<FP4>(a.y));
      inv[2 * u] = inv_scale_from_e8m0(e[2 * u]);
      inv[2 * u + 1] = inv_scale_from_e8m0(e[2 * u + 1]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = ib * 32 + (i >> 2) * 16 + sub * 4 + (i & 3);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&d[i]);
      uint32_t w[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const float2 t0 = __bfloat1622float2(h[2 * u]), t1 = __bfloat1622float2(h[2 * u + 1]);
        w[u] = (uint32_t)cvt2_sel<FP4>(t0.x * inv[4 * u], t0.y * inv[4 * u + 1]) |
               ((uint32_t)cvt2_sel<FP4>(t1.x * inv[4 * u + 2], t1.y * inv[4 * u + 3]) << 16);
      }
      *reinterpret_cast<uint2*>(q_col + (long)(row0 + r) * C + col0 + cbase) = make_uint2(w[0], w[1]);
    }
    // every lane of a column group holds the 8 scales; subset s writes those of columns 2s and 2s + 1
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (sub == u) {
        sf_col[sf_offset(col0 + cbase + 2 * u, (row0 >> 5) + ib, R >> 7)] = (uint8_t)e[2 * u];
        sf_col[sf_offset(col0 + cbase + 2 * u + 1, (row0 >> 5) + ib, R >> 7)] = (uint8_t)e[2 * u + 1];
      }
    }
  }
}

template <bool FP4>
__global__ void __launch_bounds__(256, 4)
quant_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, int R, int C, uint8_t* __restrict__ q_row,
                   uint8_t* __restrict__ sf_row, uint8_t* __restrict__ q_col, uint8_t* __restrict__ sf_col) {
  extern __shared__ __align__(16) uint8_t smem_q[];
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_q);
  const int row0 = blockIdx.y * TILE, col0 = blockIdx.x * TILE;
  const int tid = threadIdx.x;
  // load 128 x 128 bf16 (16 vectors of 16 B per row)
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int v = tid + it * 256;
    const int r = v >> 4, c8 = (v & 15) * 8;
    const uint4 d = *reinterpret_cast<const uint4*>(x + (long)(row0 + r) * C + col0 + c8);
    *reinterpret_cast<uint4*>(&tile[r * PITCH + c8]) = d;
  }
  __syncthreads();
  quantize_staged_tile<SCALE_BLOCK32, FP4>(tile, R, C, row0, col0, q_row, sf_row, q_col, sf_col);
}

// Tensor-wise FP8 ("current scaling" with a power-of-two scale): one scale 2^e for the whole tensor,
// e = ceil(log2(amax / 448)) from the tensor maximum `tensor_amax` (device, written by amax_bf16_kernel).  The output has
// the MXFP8 layout with that exponent in every block, so the block-scaled GEMM consumes it unchanged.  The behaviour
// of the reference's tensor-wise quantiser (primus_turbo_cpp_extension::quantize_fp8_tensorwise, called from
// primus/backends/megatron/core/extensions/primus_turbo_float8_local.py:66-70).
__global__ void __launch_bounds__(256, 4)
quant_tensorwise_kernel(const __nv_bfloat16* __restrict__ x, int R, int C, const float* __restrict__ tensor_amax,
                        const float* __restrict__ fallback_amax, uint8_t* __restrict__ q_row,
                        uint8_t* __restrict__ sf_row, uint8_t* __restrict__ q_col, uint8_t* __restrict__ sf_col) {
  extern __shared__ __align__(16) uint8_t smem_q[];
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_q);
  const int row0 = blockIdx.y * TILE, col0 = blockIdx.x * TILE;
  const int tid = threadIdx.x;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int v = tid + it * 256;
    const int r = v >> 4, c8 = (v & 15) * 8;
    const uint4 d = *reinterpret_cast<const uint4*>(x + (long)(row0 + r) * C + col0 + c8);
    *reinterpret_cast<uint4*>(&tile[r * PITCH + c8]) = d;
  }
  // delayed scaling passes the maximum its history predicts as `tensor_amax` and this step's measured maximum as
  // `fallback_amax`, which is used while the history is still empty (0)
  float a = *tensor_amax;
  if (a == 0.f && fallback_amax != nullptr) a = *fallback_amax;
  const int fixed_e = e8m0_from_amax(a);
  __syncthreads();
  quantize_staged_tile<SCALE_FIXED>(tile, R, C, row0, col0, q_row, sf_row, q_col, sf_col, fixed_e);
}

// Block-wise FP8 (blocks of 128): activations and gradients take one power-of-two scale per 1 x 128 vector along the
// reduced dimension (row direction: 128 consecutive columns of a row; column direction: 128 consecutive rows of a
// column), weights (TILEWISE) one per 128 x 128 tile.  Stored in the MXFP8 layout with the exponent repeated in the
// four 32-blocks it covers, so the block-scaled GEMM consumes it unchanged.  Granularity of the reference's
// "blockwise" recipe (primus/backends/megatron/core/extensions/primus_turbo.py: Float8QuantConfig with
// ScalingGranularity.BLOCKWISE, block_size 128), with scales restricted to powers of two.
template <bool TILEWISE>
__global__ void __launch_bounds__(256, 4)
quant_blockwise_kernel(const __nv_bfloat16* __restrict__ x, int R, int C, uint8_t* __restrict__ q_row,
                       uint8_t* __restrict__ sf_row, uint8_t* __restrict__ q_col, uint8_t* __restrict__ sf_col) {
  extern __shared__ __align__(16) uint8_t smem_q[];
  __shared__ uint8_t e_rowv[TILE], e_colv[TILE];
  __shared__ float warp_max[4];
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_q);
  const int row0 = blockIdx.y * TILE, col0 = blockIdx.x * TILE;
  const int tid = threadIdx.x;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int v = tid + it * 256;
    const int r = v >> 4, c8 = (v & 15) * 8;
    const uint4 d = *reinterpret_cast<const uint4*>(x + (long)(row0 + r) * C + col0 + c8);
    *reinterpret_cast<uint4*>(&tile[r * PITCH + c8]) = d;
  }
  __syncthreads();
  // threads 0..127: maximum of tile row tid; threads 128..255: maximum of tile column tid - 128
  float m = 0.f;
  if (tid < TILE) {
    __nv_bfloat162 mm = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
    for (int v = 0; v < 16; ++v) {
      const uint4 d = *reinterpret_cast<const uint4*>(&tile[tid * PITCH + v * 8]);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
      for (int u = 0; u < 4; ++u) mm = __hmax2(mm, __habs2(h[u]));
    }
    const float2 f = __bfloat1622float2(mm);
    m = fmaxf(f.x, f.y);
  } else if (!TILEWISE) {
    const int c = tid - TILE;
#pragma unroll 8
    for (int r = 0; r < TILE; ++r) m = fmaxf(m, fabsf(__bfloat162float(tile[r * PITCH + c])));
  }
  if (TILEWISE) {
    float v = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (tid < TILE && (tid & 31) == 0) warp_max[tid >> 5] = v;
    __syncthreads();
    const int fixed_e = e8m0_from_amax(fmaxf(fmaxf(warp_max[0], warp_max[1]), fmaxf(warp_max[2], warp_max[3])));
    quantize_staged_tile<SCALE_FIXED>(tile, R, C, row0, col0, q_row, sf_row, q_col, sf_col, fixed_e);
  } else {
    if (tid < TILE) e_rowv[tid] = (uint8_t)e8m0_from_amax(m);
    else e_colv[tid - TILE] = (uint8_t)e8m0_from_amax(m);
    __syncthreads();
    quantize_staged_tile<SCALE_VEC128>(tile, R, C, row0, col0, q_row, sf_row, q_col, sf_col, 0, e_rowv, e_colv);
  }
}

// max |x| over n bf16 values (n a multiple of 8) into *out, which the caller zeroes first (non-negative floats order
// like their bit patterns, so the cross-CTA step is an integer atomicMax)
__global__ void __launch_bounds__(256)
amax_bf16_kernel(const __nv_bfloat16* __restrict__ x, long n8, float* __restrict__ out) {
  __nv_bfloat162 m = __floats2bfloat162_rn(0.f, 0.f);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const uint4 d = reinterpret_cast<const uint4*>(x)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
    for (int u = 0; u < 4; ++u) m = __hmax2(m, __habs2(h[u]));
  }
  const float2 f = __bfloat1622float2(m);
  float v = fmaxf(f.x, f.y);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __shared__ float s[8];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) v = fmaxf(v, s[i]);
    if (v != v) v = __uint_as_float(0x7f800000u);   // NaN in the input: report +inf
    atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(v));
  }
}

__device__ __forceinline__ void bf8_load(const __nv_bfloat16* p, float* f) {
  const uint4 d = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const float2 t = __bfloat1622float2(h[u]);
    f[2 * u] = t.x;
    f[2 * u + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 bf8_pack(const float* f) {
  uint4 o;
  o.x = pb::pack_bf16x2(f[0], f[1]);
  o.y = pb::pack_bf16x2(f[2], f[3]);
  o.z = pb::pack_bf16x2(f[4], f[5]);
  o.w = pb::pack_bf16x2(f[6], f[7]);
  return o;
}

// SwiGLU forward fused with the quantisation of its output: h1 [T, 2I] = [gate | up] -> MXFP8 of
// act[T, I] = silu(gate) * up (rounded to bf16 first, so the values equal quantising the un-fused kernel's output).
__global__ void __launch_bounds__(256, 4)
swiglu_quant_mxfp8_kernel(const __nv_bfloat16* __restrict__ h1, int T, int I, float clamp, uint8_t* __restrict__ q_row,
                          uint8_t* __restrict__ sf_row, uint8_t* __restrict__ q_col, uint8_t* __restrict__ sf_col) {
  extern __shared__ __align__(16) uint8_t smem_q[];
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_q);
  const int row0 = blockIdx.y * TILE, col0 = blockIdx.x * TILE;
  const int tid = threadIdx.x;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int v = tid + it * 256;
    const int r = v >> 4, c8 = (v & 15) * 8;
    const __nv_bfloat16* g = h1 + (long)(row0 + r) * 2 * I + col0 + c8;
    float fg[8], fu[8], o[8];
    bf8_load(g, fg);
    bf8_load(g + I, fu);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gg = fg[j], uu = fu[j];
      if (clamp > 0.f) {
        gg = fminf(gg, clamp);
        uu = fminf(fmaxf(uu, -clamp), clamp);
      }
      const float sig = pb::fast_sigmoid(gg);
      o[j] = gg * sig * uu * 1.f;
    }
    *reinterpret_cast<uint4*>(&tile[r * PITCH + c8]) = bf8_pack(o);
  }
  __syncthreads();
  quantize_staged_tile(tile, T, I, row0, col0, q_row, sf_row, q_col, sf_col);
}

// SwiGLU backward fused with the quantisation of its output: (h1 [T, 2I], dact [T, I]) -> MXFP8 (both directions) of
// dh1 [T, 2I] = [dgate | dup].  One CTA per 128 x 128 tile of the activation: it reads gate, up and dact once, stages
// the dgate and the dup tile, and quantises one after the other.
constexpr int QUANT_SMEM_BWD = 2 * TILE * PITCH * 2;
__global__ void __launch_bounds__(256, 3)
swiglu_bwd_quant_mxfp8_kernel(const __nv_bfloat16* __restrict__ h1, const __nv_bfloat16* __restrict__ dact, int T, int I,
                              float clamp, uint8_t* __restrict__ q_row, uint8_t* __restrict__ sf_row,
                              uint8_t* __restrict__ q_col, uint8_t* __restrict__ sf_col) {
  extern __shared__ __align__(16) uint8_t smem_q[];
  __nv_bfloat16* tile_g = reinterpret_cast<__nv_bfloat16*>(smem_q);
  __nv_bfloat16* tile_u = tile_g + TILE * PITCH;
  const int row0 = blockIdx.y * TILE, col0 = blockIdx.x * TILE;
  const int tid = threadIdx.x;
#pragma unroll 2
  for (int it = 0; it < 8; ++it) {
    const int v = tid + it * 256;
    const int r = v >> 4, c8 = (v & 15) * 8;
    const __nv_bfloat16* g = h1 + (long)(row0 + r) * 2 * I + col0 + c8;
    float fg[8], fu[8], fd[8], og[8], ou[8];
    bf8_load(g, fg);
    bf8_load(g + I, fu);
    bf8_load(dact + (long)(row0 + r) * I + col0 + c8, fd);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gg = fg[j], uu = fu[j];
      float gmask = 1.f, umask = 1.f;
      if (clamp > 0.f) {
        if (gg > clamp) { gg = clamp; gmask = 0.f; }
        if (uu > clamp) { uu = clamp; umask = 0.f; }
        if (uu < -clamp) { uu = -clamp; umask = 0.f; }
      }
      const float sig = pb::fast_sigmoid(gg);
      const float sl = gg * sig;
      const float d = fd[j] * 1.f;
      const float dsl = sig * (1.f + gg * (1.f - sig));
      og[j] = d * uu * dsl * gmask;
      ou[j] = d * sl * umask;
    }
    *reinterpret_cast<uint4*>(&tile_g[r * PITCH + c8]) = bf8_pack(og);
    *reinterpret_cast<uint4*>(&tile_u[r * PITCH + c8]) = bf8_pack(ou);
  }
  __syncthreads();
  quantize_staged_tile(tile_g, T, 2 * I, row0, col0, q_row, sf_row, q_col, sf_col);
  quantize_staged_tile(tile_u, T, 2 * I, row0, I + col0, q_row, sf_row, q_col, sf_col);
}

// value [R, C] fp8 + scales (operand layout with MN = R or C) -> fp32 [R, C]; test / debugging helper
__global__ void dequant_mxfp8_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf, int R, int C,
                                     int colwise, float* __restrict__ out) {
  const long n = (long)R * C;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const int r = (int)(i / C), c = (int)(i - (long)r * C);
    const int e = colwise ? sf[sf_offset(c, r >> 5, R >> 7)] : sf[sf_offset(r, c >> 5, C >> 7)];
    const __nv_fp8_e4m3 v = *reinterpret_cast<const __nv_fp8_e4m3*>(q + i);
    out[i] = float(v) * exp2f((float)(e - 127));
  }
}

}  // namespace

extern "C" {

// Any of the two outputs may be null.  R and C must be multiples of 128.
// sf_row: R * C / 32 bytes, sf_col: R * C / 32 bytes.
int pb_quant_mxfp8(const void* x, int R, int C, void* q_row, void* sf_row, void* q_col, void* sf_col, cudaStream_t s) {
  if (R % TILE || C % TILE || R <= 0 || C <= 0) return -2;
  dim3 grid(C / TILE, R / TILE);
  constexpr int SMEM = QUANT_SMEM;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(quant_mxfp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  quant_mxfp8_kernel<false><<<grid, 256, SMEM, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), R, C,
                                                reinterpret_cast<uint8_t*>(q_row), reinterpret_cast<uint8_t*>(sf_row),
                                                reinterpret_cast<uint8_t*>(q_col), reinterpret_cast<uint8_t*>(sf_col));
  return (int)cudaGetLastError();
}

// MXFP4 numerics in FP8 storage: E2M1 values (as E4M3 bytes) with one UE8M0 scale per 32 elements; outputs and
// constraints as pb_quant_mxfp8.
int pb_quant_mxfp4_as_fp8(const void* x, int R, int C, void* q_row, void* sf_row, void* q_col, void* sf_col,
                          cudaStream_t s) {
  if (R % TILE || C % TILE || R <= 0 || C <= 0) return -2;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(quant_mxfp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, QUANT_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  quant_mxfp8_kernel<true><<<dim3(C / TILE, R / TILE), 256, QUANT_SMEM, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), R, C, reinterpret_cast<uint8_t*>(q_row),
      reinterpret_cast<uint8_t*>(sf_row), reinterpret_cast<uint8_t*>(q_col), reinterpret_cast<uint8_t*>(sf_col));
  return (int)cudaGetLastError();
}

// Tensor-wise FP8 of x [R, C] (multiples of 128): amax[0] receives max |x|; outputs as pb_quant_mxfp8.
int pb_quant_fp8_tensorwise(const void* x, int R, int C, float* amax, void* q_row, void* sf_row, void* q_col, void* sf_col,
                            cudaStream_t s) {
  if (R % TILE || C % TILE || R <= 0 || C <= 0) return -2;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(quant_tensorwise_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, QUANT_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  cudaError_t e = cudaMemsetAsync(amax, 0, sizeof(float), s);
  if (e != cudaSuccess) return (int)e;
  const long n8 = (long)R * C / 8;
  const int blocks = (int)((n8 + 2047) / 2048 < 1184 ? (n8 + 2047) / 2048 : 1184);
  amax_bf16_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), n8, amax);
  quant_tensorwise_kernel<<<dim3(C / TILE, R / TILE), 256, QUANT_SMEM, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), R, C, amax, nullptr, reinterpret_cast<uint8_t*>(q_row),
      reinterpret_cast<uint8_t*>(sf_row), reinterpret_cast<uint8_t*>(q_col), reinterpret_cast<uint8_t*>(sf_col));
  return (int)cudaGetLastError();
}

// Delayed-scaling FP8 of x [R, C]: the scale comes from scale_amax[0] (the maximum predicted from the history of
// earlier steps; 0 = no history yet, then this call's own maximum is used), and max |x| is folded into amax_now[0]
// with an atomic maximum -- the caller zeroes amax_now when it rolls the history, so several calls between two rolls
// (micro-batches) record their overall maximum.  Values above the predicted range saturate at +-448.
int pb_quant_fp8_delayed(const void* x, int R, int C, float* amax_now, const float* scale_amax, void* q_row,
                         void* sf_row, void* q_col, void* sf_col, cudaStream_t s) {
  if (R % TILE || C % TILE || R <= 0 || C <= 0) return -2;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(quant_tensorwise_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, QUANT_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const long n8 = (long)R * C / 8;
  const int blocks = (int)((n8 + 2047) / 2048 < 1184 ? (n8 + 2047) / 2048 : 1184);
  amax_bf16_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), n8, amax_now);
  quant_tensorwise_kernel<<<dim3(C / TILE, R / TILE), 256, QUANT_SMEM, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), R, C, scale_amax, amax_now, reinterpret_cast<uint8_t*>(q_row),
      reinterpret_cast<uint8_t*>(sf_row), reinterpret_cast<uint8_t*>(q_col), reinterpret_cast<uint8_t*>(sf_col));
  return (int)cudaGetLastError();
}

// Block-wise FP8 of x [R, C] (multiples of 128): one power-of-two scale per 1 x 128 vector (tilewise = 0:
// activations, gradients) or per 128 x 128 tile (tilewise = 1: weights); outputs as pb_quant_mxfp8.
int pb_quant_fp8_blockwise(const void* x, int R, int C, int tilewise, void* q_row, void* sf_row, void* q_col,
                           void* sf_col, cudaStream_t s) {
  if (R % TILE || C % TILE || R <= 0 || C <= 0) return -2;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(quant_blockwise_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         QUANT_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(quant_blockwise_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, QUANT_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const dim3 grid(C / TILE, R / TILE);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  uint8_t *qr = reinterpret_cast<uint8_t*>(q_row), *sr = reinterpret_cast<uint8_t*>(sf_row);
  uint8_t *qc = reinterpret_cast<uint8_t*>(q_col), *sc = reinterpret_cast<uint8_t*>(sf_col);
  if (tilewise) quant_blockwise_kernel<true><<<grid, 256, QUANT_SMEM, s>>>(xp, R, C, qr, sr, qc, sc);
  else quant_blockwise_kernel<false><<<grid, 256, QUANT_SMEM, s>>>(xp, R, C, qr, sr, qc, sc);
  return (int)cudaGetLastError();
}

static int set_quant_smem(const void* kern) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, QUANT_SMEM);
  return (int)e;
}

// act = silu(gate) * up of h1 [T, 2I] (T, I multiples of 128) quantised to MXFP8; either output pair may be null.
int pb_swiglu_quant_mxfp8(const void* h1, int T, int I, float clamp, void* q_row, void* sf_row, void* q_col,
                          void* sf_col, cudaStream_t s) {
  if (T % TILE || I % TILE || T <= 0 || I <= 0) return -2;
  static bool attr_set = false;
  if (!attr_set) {
    int rc = set_quant_smem(reinterpret_cast<const void*>(swiglu_quant_mxfp8_kernel));
    if (rc) return rc;
    attr_set = true;
  }
  swiglu_quant_mxfp8_kernel<<<dim3(I / TILE, T / TILE), 256, QUANT_SMEM, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(h1), T, I, clamp, reinterpret_cast<uint8_t*>(q_row),
      reinterpret_cast<uint8_t*>(sf_row), reinterpret_cast<uint8_t*>(q_col), reinterpret_cast<uint8_t*>(sf_col));
  return (int)cudaGetLastError();
}

// dh1 [T, 2I] = swiglu backward of (h1, dact) quantised to MXFP8 (outputs sized for [T, 2I]).
int pb_swiglu_bwd_quant_mxfp8(const void* h1, const void* dact, int T, int I, float clamp, void* q_row, void* sf_row,
                              void* q_col, void* sf_col, cudaStream_t s) {
  if (T % TILE || I % TILE || T <= 0 || I <= 0) return -2;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(swiglu_bwd_quant_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         QUANT_SMEM_BWD);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  swiglu_bwd_quant_mxfp8_kernel<<<dim3(I / TILE, T / TILE), 256, QUANT_SMEM_BWD, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(h1), reinterpret_cast<const __nv_bfloat16*>(dact), T, I, clamp,
      reinterpret_cast<uint8_t*>(q_row), reinterpret_cast<uint8_t*>(sf_row), reinterpret_cast<uint8_t*>(q_col),
      reinterpret_cast<uint8_t*>(sf_col));
  return (int)cudaGetLastError();
}

int pb_dequant_mxfp8(const void* q, const void* sf, int R, int C, int colwise, float* out, cudaStream_t s) {
  if (R % TILE || C % TILE) return -2;
  dequant_mxfp8_kernel<<<1184, 256, 0, s>>>(reinterpret_cast<const uint8_t*>(q), reinterpret_cast<const uint8_t*>(sf), R,
                                           C, colwise, out);
  return (int)cudaGetLastError();
}

}  // extern "C"
