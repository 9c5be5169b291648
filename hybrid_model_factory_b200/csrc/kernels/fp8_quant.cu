// Row-wise scaled float8 quantisation for the fp8 linear layers (bf16 -> e4m3 / e5m2 with one fp32 scale per row of
// the GEMM operand).  A GEMM operand is always stored K-major, so an operand that is contracted over the ROWS of the
// source matrix (the weight in the input-gradient GEMM, both operands of the weight-gradient GEMM) is quantised per
// source COLUMN and written transposed in the same pass.
//
//   quant_rows   : x [R, C] -> q [R, C],  scale[r] = amax_c |x[r, c]| / fmax           (one block per row)
//   col_amax     : x [R, C] -> amax[c] = max_r |x[r, c]|                               (atomic max on the float bits)
//   quant_cols_t : x [R, C], amax[C] -> q_t [C, R], scale[c] = amax[c] / fmax          (64 x 64 tiles through shared memory)
#include <cuda_fp8.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace fp8q {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float fmt_max(int fmt) { return fmt == 0 ? 448.f : 57344.f; }
__device__ __forceinline__ uint8_t to_fp8(float v, int fmt) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, fmt == 0 ? __NV_E4M3 : __NV_E5M2);
}

__global__ void quant_rows_kernel(const bf16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                                  float* __restrict__ scale, int C, int fmt) {
  const long long r = blockIdx.x;
  const bf16* row = x + r * ldx;
  __shared__ float red[32];
  float m = 0.f;
  for (int c = threadIdx.x * 8; c < C; c += blockDim.x * 8) {
    if (c + 8 <= C) {
      const uint4 u = *reinterpret_cast<const uint4*>(row + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    } else {
      for (int i = c; i < C; ++i) m = fmaxf(m, fabsf(__bfloat162float(row[i])));
    }
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_max(v);
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  const float amax = red[0];
  const float sc = amax > 0.f ? amax / fmt_max(fmt) : 1.f;
  const float inv = 1.f / sc;
  if (threadIdx.x == 0) scale[r] = sc;
  uint8_t* out = q + r * ldq;
  for (int c = threadIdx.x * 8; c < C; c += blockDim.x * 8) {
    if (c + 8 <= C) {
      const uint4 u = *reinterpret_cast<const uint4*>(row + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
      uint8_t b[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        b[2 * i] = to_fp8(f.x * inv, fmt);
        b[2 * i + 1] = to_fp8(f.y * inv, fmt);
      }
      *reinterpret_cast<uint2*>(out + c) = *reinterpret_cast<const uint2*>(b);
    } else {
      for (int i = c; i < C; ++i) out[i] = to_fp8(__bfloat162float(row[i]) * inv, fmt);
    }
  }
}

// grid (ceil(C / 64), ceil(R / 256)), block (64, 4): thread (tx, ty) walks rows ty, ty + 4, ... of its 256-row slab
__global__ void col_amax_kernel(const bf16* __restrict__ x, long long ldx, float* __restrict__ amax, long long R, int C) {
  const int c = blockIdx.x * 64 + threadIdx.x;
  const long long r0 = (long long)blockIdx.y * 256;
  float m = 0.f;
  if (c < C) {
    const long long r1 = r0 + 256 < R ? r0 + 256 : R;
    for (long long r = r0 + threadIdx.y; r < r1; r += 4) m = fmaxf(m, fabsf(__bfloat162float(x[r * ldx + c])));
  }
  __shared__ float red[4][64];
  red[threadIdx.y][threadIdx.x] = m;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
    m = fmaxf(fmaxf(red[0][threadIdx.x], red[1][threadIdx.x]), fmaxf(red[2][threadIdx.x], red[3][threadIdx.x]));
    atomicMax(reinterpret_cast<int*>(amax + c), __float_as_int(m));        // non-negative floats order like ints
  }
}

// grid (ceil(C / 64), ceil(R / 64)), block (64, 4)
__global__ void quant_cols_t_kernel(const bf16* __restrict__ x, long long ldx, const float* __restrict__ amax,
                                    uint8_t* __restrict__ qt, long long ldq, float* __restrict__ scale, long long R,
                                    int C, int fmt) {
  __shared__ uint8_t tile[64][65];
  const int c0 = blockIdx.x * 64;
  const long long r0 = (long long)blockIdx.y * 64;
  {
    const int c = c0 + threadIdx.x;
    float inv = 0.f;
    if (c < C) {
      const float a = amax[c];
      const float sc = a > 0.f ? a / fmt_max(fmt) : 1.f;
      inv = 1.f / sc;
      if (blockIdx.y == 0 && threadIdx.y == 0) scale[c] = sc;
    }
    for (int i = threadIdx.y; i < 64; i += 4) {
      const long long r = r0 + i;
      const float v = (c < C && r < R) ? __bfloat162float(x[r * ldx + c]) * inv : 0.f;
      tile[i][threadIdx.x] = to_fp8(v, fmt);
    }
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 64; j += 4) {     // output row = source column c0 + j, 64 consecutive source rows
    const int c = c0 + j;
    const long long r = r0 + threadIdx.x;
    if (c < C && r < R) qt[(long long)c * ldq + r] = tile[threadIdx.x][j];
  }
}

}  // namespace fp8q
}  // namespace hmf

// x [R, C] bf16 (row stride ldx) -> q [R, C] fp8 (row stride ldq bytes), scale [R] fp32.  fmt 0 = e4m3, 1 = e5m2.
HMF_API int hmf_fp8_quant_rows(const void* x, long long ldx, void* q, long long ldq, float* scale, long long R, int C,
                               int fmt, cudaStream_t st) {
  using namespace hmf;
  HMF_REQUIRE(x && q && scale && R > 0 && C > 0, "fp8_quant_rows: bad arguments");
  HMF_REQUIRE(ldx % 8 == 0 && ldq % 8 == 0, "fp8_quant_rows: row strides must be multiples of 8");
  fp8q::quant_rows_kernel<<<(unsigned)R, 256, 0, st>>>((const fp8q::bf16*)x, ldx, (uint8_t*)q, ldq, scale, C, fmt);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// x [R, C] bf16 -> q_t [C, R] fp8 (row stride ldq bytes), scale [C] fp32 (one scale per source column);
// amax: fp32 scratch [C].
HMF_API int hmf_fp8_quant_cols_t(const void* x, long long ldx, void* qt, long long ldq, float* scale, float* amax,
                                 long long R, int C, int fmt, cudaStream_t st) {
  using namespace hmf;
  HMF_REQUIRE(x && qt && scale && amax && R > 0 && C > 0, "fp8_quant_cols_t: bad arguments");
  HMF_CHECK_CUDA(cudaMemsetAsync(amax, 0, sizeof(float) * C, st));
  dim3 blk(64, 4);
  fp8q::col_amax_kernel<<<dim3((C + 63) / 64, (unsigned)((R + 255) / 256)), blk, 0, st>>>((const fp8q::bf16*)x, ldx, amax, R, C);
  HMF_CHECK_CUDA(cudaGetLastError());
  fp8q::quant_cols_t_kernel<<<dim3((C + 63) / 64, (unsigned)((R + 63) / 64)), blk, 0, st>>>(
      (const fp8q::bf16*)x, ldx, amax, (uint8_t*)qt, ldq, scale, R, C, fmt);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
