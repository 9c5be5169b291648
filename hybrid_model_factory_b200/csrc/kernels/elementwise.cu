// Memory-bound kernels (bf16 activations, fp32 math): RMSNorm, gated RMSNorm, SwiGLU, RoPE,
// depthwise causal conv1d + SiLU, softmax cross-entropy over logit chunks, fused AdamW and
// gradient-norm reduction.  Every kernel moves 16 bytes per thread per access and keeps its
// reductions in registers / shuffles; the only scratch is what the caller passes.
#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace ew {

using bf16 = __nv_bfloat16;

struct alignas(16) Vec8 {
  bf16 v[8];
};

__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------------------------
// RMSNorm: one warp per row. D % 8 == 0.
//   y = x * rstd * (w or 1+w); optional fused residual add: r = x + res (stored), y = norm(r)
// ------------------------------------------------------------------------------------
__global__ void rms_norm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                                    const bf16* __restrict__ w, bf16* __restrict__ y,
                                    bf16* __restrict__ res_out, float* __restrict__ rstd_out, long long N,
                                    int D, float eps, int zero_centered) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= N) return;
  const bf16* xr = x + row * D;
  float ss = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    float f[8];
    load8(xr + c, f);
    if (res != nullptr) {
      float r[8];
      load8(res + row * D + c, r);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] + r[i]));
      store8(res_out + row * D + c, f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / D + eps);
  if (lane == 0 && rstd_out) rstd_out[row] = rstd;
  const bf16* src = (res != nullptr) ? (res_out + row * D) : xr;
  for (int c = lane * 8; c < D; c += 256) {
    float f[8], g[8];
    load8(src + c, f);
    if (w) {
      load8(w + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * (zero_centered ? 1.f + g[i] : g[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd;
    }
    store8(y + row * D + c, f);
  }
}

// Few rows (decode steps): one 256-thread block per row, the row held in registers between the sum and the scaling
// (D <= 8192), so a row costs one read and one write and its latency is spread over eight warps.
__global__ void __launch_bounds__(256)
rms_norm_fwd_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res, const bf16* __restrict__ w,
                         bf16* __restrict__ y, bf16* __restrict__ res_out, float* __restrict__ rstd_out, int D,
                         float eps, int zero_centered) {
  __shared__ float s_part[8];
  const long long row = blockIdx.x;
  const int t = threadIdx.x;
  float f[4][8];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int c = (u * 256 + t) * 8;
    if (c < D) {
      load8(x + row * D + c, f[u]);
      if (res != nullptr) {
        float r[8];
        load8(res + row * D + c, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[u][i] = __bfloat162float(__float2bfloat16(f[u][i] + r[i]));
        store8(res_out + row * D + c, f[u]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[u][i] * f[u][i];
    }
  }
  ss = warp_sum(ss);
  if ((t & 31) == 0) s_part[t >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += s_part[i];
  const float rstd = rsqrtf(tot / D + eps);
  if (t == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int c = (u * 256 + t) * 8;
    if (c < D) {
      if (w) {
        float g[8];
        load8(w + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[u][i] = f[u][i] * rstd * (zero_centered ? 1.f + g[i] : g[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[u][i] *= rstd;
      }
      store8(y + row * D + c, f[u]);
    }
  }
}

// backward, input gradient: dx = rstd * (w dy - xhat * mean(w dy xhat)); one warp per row.
__global__ void rms_norm_bwd_dx_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                       const bf16* __restrict__ dy, const float* __restrict__ rstd,
                                       bf16* __restrict__ dx, long long N, int D, int zero_centered) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= N) return;
  const float rs = rstd[row];
  float dot = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    float xf[8], gf[8], wf[8];
    load8(x + row * D + c, xf);
    load8(dy + row * D + c, gf);
    if (w) load8(w + c, wf);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float ww = w ? (zero_centered ? 1.f + wf[i] : wf[i]) : 1.f;
      dot += gf[i] * ww * xf[i] * rs;
    }
  }
  dot = warp_sum(dot) / D;
  for (int c = lane * 8; c < D; c += 256) {
    float xf[8], gf[8], wf[8], o[8];
    load8(x + row * D + c, xf);
    load8(dy + row * D + c, gf);
    if (w) load8(w + c, wf);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float ww = w ? (zero_centered ? 1.f + wf[i] : wf[i]) : 1.f;
      const float xh = xf[i] * rs;
      o[i] = rs * (gf[i] * ww - xh * dot);
    }
    store8(dx + row * D + c, o);
  }
}

// backward, weight gradient partials: dw_part[slab, c] = sum over the slab's rows of dy * x * rstd.
// block = 256 threads = CT column threads (8 columns each) x RL row lanes; grid = (col blocks, slabs).
__global__ void rms_norm_bwd_dw_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy,
                                       const float* __restrict__ rstd, float* __restrict__ dw_part,
                                       long long N, int D, long long rows_per_slab, int CT) {
  __shared__ float red[256 * 8];
  const int RL = 256 / CT;
  const int ct = threadIdx.x % CT, rl = threadIdx.x / CT;
  const int c = (blockIdx.x * CT + ct) * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_slab;
  const long long r1 = min(N, r0 + rows_per_slab);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (c < D) {
    for (long long row = r0 + rl; row < r1; row += RL) {
      float xf[8], gf[8];
      load8(x + row * D + c, xf);
      load8(dy + row * D + c, gf);
      const float rs = rstd[row];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += gf[i] * xf[i] * rs;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[threadIdx.x * 8 + i] = acc[i];
  __syncthreads();
  if (rl == 0 && c < D) {
    for (int r = 1; r < RL; ++r)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += red[(r * CT + ct) * 8 + i];
#pragma unroll
    for (int i = 0; i < 8; ++i) dw_part[(size_t)blockIdx.y * D + c + i] = acc[i];
  }
}

// column sum of partials [P, D] -> out[D] (bf16 or fp32 by flag)
__global__ void colsum_kernel(const float* __restrict__ part, int P, int D, float* __restrict__ out_f,
                              bf16* __restrict__ out_b) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += part[(size_t)p * D + c];
  if (out_f) out_f[c] = s;
  if (out_b) out_b[c] = __float2bfloat16(s);
}

// ------------------------------------------------------------------------------------
// Gated RMSNorm over head_dim rows (D <= 256, D % 8 == 0); 32/(D/8) ... one warp handles
// WARP_ROWS = 256/D rows at once (D=128 -> 2 rows of 16 lanes; D=64 -> 4 rows of 8 lanes).
//   mode 0 (norm_before_gate): y = x*rstd*w * silu(g)
//   mode 1:                    y = (x*silu(g)) * rstd' * w   with rstd' over x*silu(g)
// weight row = (row % H) when per-head weights (w_rows = H) else 0.
// ------------------------------------------------------------------------------------
template <int D>
__global__ void gated_norm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gate,
                                      const bf16* __restrict__ w, bf16* __restrict__ y,
                                      float* __restrict__ rstd_out, long long N, int w_rows, float eps,
                                      int mode) {
  constexpr int LPR = D / 8;       // lanes per row
  constexpr int RPW = 32 / LPR;    // rows per warp
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long row = wid * RPW + lane / LPR;
  const int c = (lane % LPR) * 8;
  const bool ok = row < N;
  float xf[8], gf[8], wf[8];
  if (ok) {
    load8(x + row * D + c, xf);
    load8(gate + row * D + c, gf);
    load8(w + (size_t)(w_rows > 1 ? row % w_rows : 0) * D + c, wf);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) xf[i] = gf[i] = wf[i] = 0.f;
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (mode == 1) xf[i] *= silu_f(gf[i]);
    ss += xf[i] * xf[i];
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rstd = rsqrtf(ss / D + eps);
  if (!ok) return;
  if (rstd_out && (lane % LPR) == 0) rstd_out[row] = rstd;
  float o8[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float v = xf[i] * rstd * wf[i];
    if (mode == 0) v *= silu_f(gf[i]);
    o8[i] = v;
  }
  store8(y + row * D + c, o8);
}

template <int D>
__global__ void gated_norm_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gate,
                                      const bf16* __restrict__ w, const bf16* __restrict__ dy,
                                      const float* __restrict__ rstd_in, bf16* __restrict__ dx,
                                      bf16* __restrict__ dgate, float* __restrict__ dw_acc, long long N,
                                      int w_rows, int mode, long long rows_per_block) {
  // dw_acc: [w_rows, D] fp32, atomically accumulated (zeroed by the caller)
  constexpr int LPR = D / 8;
  constexpr int RPW = 32 / LPR;
  extern __shared__ float s_dw[];  // [w_rows * D]
  const int wtot = (w_rows > 1 ? w_rows : 1) * D;
  for (int i = threadIdx.x; i < wtot; i += blockDim.x) s_dw[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int c = (lane % LPR) * 8;
  const long long r0 = (long long)blockIdx.x * rows_per_block;
  const long long r1 = min(N, r0 + rows_per_block);
  for (long long base = r0 + (long long)warp * RPW; base < r1; base += (long long)nwarp * RPW) {
    const long long row = base + lane / LPR;
    const bool ok = row < r1;
    float xf[8], gf[8], wf[8], dyf[8];
    int wrow = 0;
    if (ok) {
      wrow = w_rows > 1 ? (int)(row % w_rows) : 0;
      load8(x + row * D + c, xf);
      load8(gate + row * D + c, gf);
      load8(w + (size_t)wrow * D + c, wf);
      load8(dy + row * D + c, dyf);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) xf[i] = gf[i] = wf[i] = dyf[i] = 0.f;
    }
    const float rs = ok ? rstd_in[row] : 0.f;
    float sg[8], sig[8], z[8], dzn[8];  // z: normalised input (x or x*silu(g)); dzn: grad wrt z*rstd
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sig[i] = sigmoid_f(gf[i]);
      sg[i] = gf[i] * sig[i];
      z[i] = (mode == 1) ? xf[i] * sg[i] : xf[i];
      const float up = (mode == 0) ? dyf[i] * sg[i] : dyf[i];  // grad wrt (zhat * w)
      dzn[i] = up * wf[i];
      dot += dzn[i] * z[i] * rs;
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    dot /= D;
    float dxo[8], dgo[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float zh = z[i] * rs;
      const float dz = rs * (dzn[i] - zh * dot);
      const float dsilu = sig[i] * (1.f + gf[i] * (1.f - sig[i]));
      if (mode == 0) {
        dxo[i] = dz;
        dgo[i] = dyf[i] * zh * wf[i] * dsilu;
      } else {
        dxo[i] = dz * sg[i];
        dgo[i] = dz * xf[i] * dsilu;
      }
      if (ok) {
        const float up = (mode == 0) ? dyf[i] * sg[i] : dyf[i];
        atomicAdd(&s_dw[wrow * D + c + i], up * zh);
      }
    }
    if (ok) {
      store8(dx + row * D + c, dxo);
      store8(dgate + row * D + c, dgo);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < wtot; i += blockDim.x)
    if (s_dw[i] != 0.f) atomicAdd(&dw_acc[i], s_dw[i]);
}

// ------------------------------------------------------------------------------------
// SwiGLU
// ------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ g, const bf16* __restrict__ u,
                                  bf16* __restrict__ y, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float gf[8], uf[8], o[8];
    load8(g + i * 8, gf);
    load8(u + i * 8, uf);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = silu_f(gf[k]) * uf[k];
    store8(y + i * 8, o);
  }
}
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ g, const bf16* __restrict__ u,
                                  const bf16* __restrict__ dy, bf16* __restrict__ dg,
                                  bf16* __restrict__ du, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    float gf[8], uf[8], df[8], og[8], ou[8];
    load8(g + i * 8, gf);
    load8(u + i * 8, uf);
    load8(dy + i * 8, df);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = sigmoid_f(gf[k]);
      og[k] = df[k] * uf[k] * s * (1.f + gf[k] * (1.f - s));
      ou[k] = df[k] * gf[k] * s;
    }
    store8(dg + i * 8, og);
    store8(du + i * 8, ou);
  }
}

// ------------------------------------------------------------------------------------
// RoPE (rotate-half) on x[B*T, H, D] with cos/sin [B*T, R]; R <= D, R % 16 == 0.
// sign = +1 forward, -1 backward (transpose of the rotation).
// One thread handles 8 consecutive elements of the first half and their partners.
// ------------------------------------------------------------------------------------
__global__ void rope_kernel(const bf16* __restrict__ x, const bf16* __restrict__ cs,
                            const bf16* __restrict__ sn, bf16* __restrict__ y, long long rows, int H, int D,
                            int R, float sign, long long x_row_stride) {
  const int half = R / 2;
  const int per_head = half / 8 + (D - R) / 8;  // work items per (row, head)
  const long long total = rows * H * per_head;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int item = (int)(i % per_head);
    const long long rh = i / per_head;
    const int h = (int)(rh % H);
    const long long row = rh / H;
    const bf16* xp = x + row * x_row_stride + (size_t)h * D;
    bf16* yp = y + (row * H + h) * (long long)D;
    if (item < half / 8) {
      const int c = item * 8;
      float a[8], b[8], cf[8], sf[8], c2[8], s2[8], oa[8], ob[8];
      load8(xp + c, a);
      load8(xp + c + half, b);
      load8(cs + row * R + c, cf);
      load8(sn + row * R + c, sf);
      load8(cs + row * R + c + half, c2);
      load8(sn + row * R + c + half, s2);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        // forward: out1 = x1 c1 - x2 s1 ; out2 = x2 c2 + x1 s2.  backward: transpose.
        if (sign > 0.f) {
          oa[k] = a[k] * cf[k] - b[k] * sf[k];
          ob[k] = b[k] * c2[k] + a[k] * s2[k];
        } else {
          oa[k] = a[k] * cf[k] + b[k] * s2[k];
          ob[k] = b[k] * c2[k] - a[k] * sf[k];
        }
      }
      store8(yp + c, oa);
      store8(yp + c + half, ob);
    } else {
      const int c = R + (item - half / 8) * 8;
      float a[8];
      load8(xp + c, a);
      store8(yp + c, a);
    }
  }
}

// ------------------------------------------------------------------------------------
// Depthwise causal conv1d (K = 4 taps, channels-last [B, T, C]) + optional SiLU.
// grid: (ceil(C/8/CX), ceil(T/TT), B); block: CX threads, each 8 channels, walks TT tokens.
// init [B, K-1, C] supplies tokens before t=0 (zeros if null).
// ------------------------------------------------------------------------------------
constexpr int CONV_K = 4;
constexpr int CONV_TT = 64;

__global__ void conv1d_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                  const bf16* __restrict__ bias, const bf16* __restrict__ init,
                                  bf16* __restrict__ y, bf16* __restrict__ final_state, int T, int C,
                                  int act) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * CONV_TT;
  const int t1 = min(T, t0 + CONV_TT);
  float wf[8][CONV_K], bf[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int j = 0; j < CONV_K; ++j) wf[i][j] = __bfloat162float(w[(size_t)(c + i) * CONV_K + j]);
    bf[i] = bias ? __bfloat162float(bias[c + i]) : 0.f;
  }
  float win[CONV_K - 1][8];
#pragma unroll
  for (int j = 0; j < CONV_K - 1; ++j) {
    const int t = t0 - (CONV_K - 1) + j;
    if (t >= 0) {
      load8(x + ((size_t)b * T + t) * C + c, win[j]);
    } else if (init) {
      load8(init + ((size_t)b * (CONV_K - 1) + (t + CONV_K - 1)) * C + c, win[j]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) win[j][i] = 0.f;
    }
  }
  for (int t = t0; t < t1; ++t) {
    float cur[8], o[8];
    load8(x + ((size_t)b * T + t) * C + c, cur);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float s = bf[i] + wf[i][0] * win[0][i] + wf[i][1] * win[1][i] + wf[i][2] * win[2][i] +
                wf[i][3] * cur[i];
      o[i] = act ? silu_f(s) : s;
      win[0][i] = win[1][i];
      win[1][i] = win[2][i];
      win[2][i] = cur[i];
    }
    store8(y + ((size_t)b * T + t) * C + c, o);
  }
  if (final_state && t1 == T) {
    // last K-1 inputs (window after the loop holds x[T-3..T-1], including init when T < 3)
#pragma unroll
    for (int j = 0; j < CONV_K - 1; ++j)
      store8(final_state + ((size_t)b * (CONV_K - 1) + j) * C + c, win[j]);
  }
}

// backward: recomputes the pre-activation; dx, dinit, and per-block partial dw/dbias reduced by atomics.
__global__ void conv1d_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                  const bf16* __restrict__ bias, const bf16* __restrict__ init,
                                  const bf16* __restrict__ dy, bf16* __restrict__ dx,
                                  float* __restrict__ dinit, float* __restrict__ dw,
                                  float* __restrict__ dbias, int T, int C, int act) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * CONV_TT;
  const int t1 = min(T, t0 + CONV_TT);
  float wf[8][CONV_K], bf[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int j = 0; j < CONV_K; ++j) wf[i][j] = __bfloat162float(w[(size_t)(c + i) * CONV_K + j]);
    bf[i] = bias ? __bfloat162float(bias[c + i]) : 0.f;
  }
  auto load_x = [&](int t, float (&dst)[8]) {
    if (t >= 0 && t < T) {
      load8(x + ((size_t)b * T + t) * C + c, dst);
    } else if (t < 0 && init && t >= -(CONV_K - 1)) {
      load8(init + ((size_t)b * (CONV_K - 1) + (t + CONV_K - 1)) * C + c, dst);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[i] = 0.f;
    }
  };
  // dpre for tokens t0 .. t1+2 (lookahead needed by dx); window of inputs x[t-3..t]
  float xw[CONV_K][8];
  for (int j = 0; j < CONV_K - 1; ++j) load_x(t0 - (CONV_K - 1) + j, xw[j]);
  float dp_hist[CONV_K - 1][8];  // dpre[t-1], dpre[t-2], dpre[t-3] relative to current
#pragma unroll
  for (int j = 0; j < CONV_K - 1; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) dp_hist[j][i] = 0.f;
  float dwacc[8][CONV_K], dbacc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    dbacc[i] = 0.f;
#pragma unroll
    for (int j = 0; j < CONV_K; ++j) dwacc[i][j] = 0.f;
  }
  // walk t from t0 to t1+2; at step t we know dpre[t], and can emit dx[t-3]
  // dx[s] = sum_j w[j] * dpre[s + 3 - j]  (j = 0..3) -> needs dpre[s .. s+3]
  // Tokens s in [t0-3, t0) belong to the previous tile (or to init): contributions from this tile's
  // dpre are added there by that tile's lookahead, so here we only emit s in [t0, t1) and use
  // lookahead dpre up to t1+2 (recomputed locally).
  for (int t = t0; t < t1 + CONV_K - 1; ++t) {
    float dpre[8];
    load_x(t, xw[CONV_K - 1]);
    if (t < T) {
      float g[8];
      load8(dy + ((size_t)b * T + t) * C + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float s = bf[i] + wf[i][0] * xw[0][i] + wf[i][1] * xw[1][i] + wf[i][2] * xw[2][i] +
                        wf[i][3] * xw[3][i];
        float d = g[i];
        if (act) {
          const float sg = sigmoid_f(s);
          d *= sg * (1.f + s * (1.f - sg));
        }
        dpre[i] = d;
        if (t < t1) {  // parameter grads: each token counted once (by its own tile)
          dbacc[i] += d;
          dwacc[i][0] += d * xw[0][i];
          dwacc[i][1] += d * xw[1][i];
          dwacc[i][2] += d * xw[2][i];
          dwacc[i][3] += d * xw[3][i];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) dpre[i] = 0.f;
    }
    const int s = t - (CONV_K - 1);  // dx index now complete: needs dpre[s..s+3] = hist[2],hist[1],hist[0],dpre
    if (s >= t0) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        o[i] = wf[i][3] * dp_hist[2][i] + wf[i][2] * dp_hist[1][i] + wf[i][1] * dp_hist[0][i] +
               wf[i][0] * dpre[i];
      store8(dx + ((size_t)b * T + s) * C + c, o);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      dp_hist[2][i] = dp_hist[1][i];
      dp_hist[1][i] = dp_hist[0][i];
      dp_hist[0][i] = dpre[i];
      xw[0][i] = xw[1][i];
      xw[1][i] = xw[2][i];
      xw[2][i] = xw[3][i];
    }
  }
  // dinit: tokens s = -3..-1 receive sum_j w[j] dpre[s+3-j] for s+3-j in [0, T): only the first tile
  if (dinit && blockIdx.y == 0) {
    // recompute dpre[0..2] quickly
    float xs[CONV_K + 2][8];
    for (int j = 0; j < CONV_K + 2; ++j) load_x(j - (CONV_K - 1), xs[j]);
    float dp[CONV_K - 1][8];
    for (int t = 0; t < CONV_K - 1; ++t) {
      float g[8];
      if (t < T) load8(dy + ((size_t)b * T + t) * C + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (t >= T) { dp[t][i] = 0.f; continue; }
        const float s = bf[i] + wf[i][0] * xs[t][i] + wf[i][1] * xs[t + 1][i] + wf[i][2] * xs[t + 2][i] +
                        wf[i][3] * xs[t + 3][i];
        float d = g[i];
        if (act) {
          const float sg = sigmoid_f(s);
          d *= sg * (1.f + s * (1.f - sg));
        }
        dp[t][i] = d;
      }
    }
    // init slot m (0..2) is token s = m-3; dpre[t] uses x[t-3+j] -> token s pairs with j = s - t + 3
#pragma unroll
    for (int m = 0; m < CONV_K - 1; ++m) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int t = 0; t < CONV_K - 1; ++t) {
          const int j = (m - 3) - t + 3;
          if (j >= 0 && j < CONV_K) acc += wf[i][j] * dp[t][i];
        }
        dinit[((size_t)b * (CONV_K - 1) + m) * C + c + i] = acc;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (dbias) atomicAdd(&dbias[c + i], dbacc[i]);
#pragma unroll
    for (int j = 0; j < CONV_K; ++j) atomicAdd(&dw[(size_t)(c + i) * CONV_K + j], dwacc[i][j]);
  }
}

// single-token update: x [B, C], state [B, K-1, C] (updated in place), y [B, C]
__global__ void conv1d_update_kernel(const bf16* __restrict__ x, bf16* __restrict__ state,
                                     const bf16* __restrict__ w, const bf16* __restrict__ bias,
                                     bf16* __restrict__ y, const int* __restrict__ slots, int C, int act) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int b = blockIdx.y;
  const long long sb = slots ? slots[b] : b;
  float s0[8], s1[8], s2[8], cur[8], o[8];
  bf16* st = state + (size_t)sb * (CONV_K - 1) * C;
  load8(st + c, s0);
  load8(st + C + c, s1);
  load8(st + 2 * (size_t)C + c, s2);
  load8(x + (size_t)b * C + c, cur);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const bf16* wr = w + (size_t)(c + i) * CONV_K;
    float s = (bias ? __bfloat162float(bias[c + i]) : 0.f) + __bfloat162float(wr[0]) * s0[i] +
              __bfloat162float(wr[1]) * s1[i] + __bfloat162float(wr[2]) * s2[i] +
              __bfloat162float(wr[3]) * cur[i];
    o[i] = act ? silu_f(s) : s;
  }
  store8(y + (size_t)b * C + c, o);
  store8(st + c, s1);
  store8(st + C + c, s2);
  store8(st + 2 * (size_t)C + c, cur);
}

// ------------------------------------------------------------------------------------
// Softmax cross-entropy over one chunk of bf16 logits [n, V]: per row loss (fp32) and in-place
// gradient dlogits = (softmax - onehot) for valid labels, 0 for ignored rows. One block per row.
// ------------------------------------------------------------------------------------
__global__ void ce_fwd_bwd_kernel(bf16* __restrict__ logits, const long long* __restrict__ labels,
                                  float* __restrict__ loss_sum, int* __restrict__ n_valid, int V,
                                  long long ld, long long ignore_index) {
  const long long row = blockIdx.x;
  bf16* lr = logits + row * ld;
  const long long label = labels[row];
  __shared__ float red[32];
  __shared__ float s_max, s_sum;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int V8 = V & ~7;
  if (label == ignore_index) {
    for (int c = threadIdx.x * 8; c < V8; c += blockDim.x * 8)
      *reinterpret_cast<uint4*>(lr + c) = make_uint4(0, 0, 0, 0);
    for (int c = V8 + threadIdx.x; c < V; c += blockDim.x) lr[c] = __float2bfloat16(0.f);
    return;
  }
  float m = -INFINITY;
  for (int c = threadIdx.x * 8; c < V8; c += blockDim.x * 8) {
    float f[8];
    load8(lr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, f[i]);
  }
  for (int c = V8 + threadIdx.x; c < V; c += blockDim.x) m = fmaxf(m, __bfloat162float(lr[c]));
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  if (warp == 0) {
    float v = lane < nwarp ? red[lane] : -INFINITY;
    v = warp_max(v);
    if (lane == 0) s_max = v;
  }
  __syncthreads();
  m = s_max;
  float s = 0.f;
  for (int c = threadIdx.x * 8; c < V8; c += blockDim.x * 8) {
    float f[8];
    load8(lr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += __expf(f[i] - m);
  }
  for (int c = V8 + threadIdx.x; c < V; c += blockDim.x) s += __expf(__bfloat162float(lr[c]) - m);
  s = warp_sum(s);
  __syncthreads();
  if (lane == 0) red[warp] = s;
  __syncthreads();
  if (warp == 0) {
    float v = lane < nwarp ? red[lane] : 0.f;
    v = warp_sum(v);
    if (lane == 0) s_sum = v;
  }
  __syncthreads();
  s = s_sum;
  const float inv = 1.f / s;
  if (threadIdx.x == 0) {
    const float lab = __bfloat162float(lr[label]);
    atomicAdd(loss_sum, __logf(s) + m - lab);
    atomicAdd(n_valid, 1);
  }
  __syncthreads();
  for (int c = threadIdx.x * 8; c < V8; c += blockDim.x * 8) {
    float f[8];
    load8(lr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      f[i] = __expf(f[i] - m) * inv;
      if (c + i == label) f[i] -= 1.f;
    }
    store8(lr + c, f);
  }
  for (int c = V8 + threadIdx.x; c < V; c += blockDim.x) {
    float p = __expf(__bfloat162float(lr[c]) - m) * inv;
    if (c == label) p -= 1.f;
    lr[c] = __float2bfloat16(p);
  }
}

// ------------------------------------------------------------------------------------
// Sum of squares (gradient norm) and fused AdamW over flat buffers.
// ------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16(v); }

template <typename G>
__global__ void sumsq_kernel(const G* __restrict__ g, long long n, float* __restrict__ out) {
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = to_f<G>(g[i]);
    s += v * v;
  }
  __shared__ float red[32];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) atomicAdd(out, v);
  }
}

// p, g: parameter / gradient; m, v: moments (type S); optional fp32 master copy.
// clip: grad scale = min(1, max_norm / (sqrt(*norm_sq) + 1e-6)) when norm_sq != null and max_norm > 0.
template <typename P, typename G, typename S>
__global__ void adamw_kernel(P* __restrict__ p, const G* __restrict__ g, S* __restrict__ m,
                             S* __restrict__ v, float* __restrict__ master, long long n, float lr,
                             float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ norm_sq, float max_norm, float grad_scale) {
  float scale = grad_scale;
  if (norm_sq != nullptr && max_norm > 0.f) {
    const float nrm = sqrtf(*norm_sq) * grad_scale;
    scale *= fminf(1.f, max_norm / (nrm + 1e-6f));
  }
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gi = to_f<G>(g[i]) * scale;
    float pi = master ? master[i] : to_f<P>(p[i]);
    float mi = to_f<S>(m[i]) * beta1 + (1.f - beta1) * gi;
    float vi = to_f<S>(v[i]) * beta2 + (1.f - beta2) * gi * gi;
    const float mh = mi / bc1, vh = vi / bc2;
    pi = pi * (1.f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
    m[i] = from_f<S>(mi);
    v[i] = from_f<S>(vi);
    if (master) master[i] = pi;
    p[i] = from_f<P>(pi);
  }
}

}  // namespace ew
}  // namespace hmf

using namespace hmf;
using namespace hmf::ew;

static inline int grid_for(long long work, int block, int cap_mult = 8) {
  long long g = (work + block - 1) / block;
  const long long cap = (long long)sm_count() * cap_mult;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

HMF_API int hmf_rms_norm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out,
                             float* rstd, long long N, int D, float eps, int zero_centered,
                             cudaStream_t st) {
  HMF_REQUIRE(D % 8 == 0 && D > 0, "rms_norm: D=%d must be a positive multiple of 8", D);
  if (N == 0) return HMF_OK;
  if (N <= 1024 && D >= 1024 && D <= 8192) {          // too few rows to fill the GPU with one warp each
    rms_norm_fwd_rows_kernel<<<(unsigned)N, 256, 0, st>>>((const bf16*)x, (const bf16*)res, (const bf16*)w, (bf16*)y,
                                                         (bf16*)res_out, rstd, D, eps, zero_centered);
    HMF_CHECK_CUDA(cudaGetLastError());
    return HMF_OK;
  }
  const int warps = 8;
  const long long blocks = (N + warps - 1) / warps;
  rms_norm_fwd_kernel<<<(unsigned)blocks, warps * 32, 0, st>>>((const bf16*)x, (const bf16*)res,
                                                             (const bf16*)w, (bf16*)y, (bf16*)res_out,
                                                             rstd, N, D, eps, zero_centered);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// dw_part must hold hmf_rms_norm_bwd_blocks(N) * D floats (ignored when w is null).
HMF_API int hmf_rms_norm_bwd_blocks(long long N) {
  long long b = (N + 255) / 256;
  const long long cap = (long long)sm_count() * 2;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}
HMF_API int hmf_rms_norm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                             float* dw_part, void* dw_out, int dw_is_bf16, long long N, int D,
                             int zero_centered, cudaStream_t st) {
  HMF_REQUIRE(D % 8 == 0 && D > 0, "rms_norm_bwd: D=%d unsupported", D);
  if (N == 0) return HMF_OK;
  const int warps = 8;
  const long long blocks = (N + warps - 1) / warps;
  rms_norm_bwd_dx_kernel<<<(unsigned)blocks, warps * 32, 0, st>>>(
      (const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, N, D, zero_centered);
  HMF_CHECK_CUDA(cudaGetLastError());
  if (w && dw_part && dw_out) {
    const int slabs = hmf_rms_norm_bwd_blocks(N);
    const long long rps = (N + slabs - 1) / slabs;
    int CT = D / 8;
    if (CT > 256) CT = 256;
    // CT must divide 256: round down to a power of two
    int p2 = 1;
    while (p2 * 2 <= CT) p2 *= 2;
    CT = p2;
    dim3 grid((D / 8 + CT - 1) / CT, slabs);
    rms_norm_bwd_dw_kernel<<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)dy, rstd, dw_part, N, D, rps,
                                                 CT);
    HMF_CHECK_CUDA(cudaGetLastError());
    colsum_kernel<<<(D + 255) / 256, 256, 0, st>>>(dw_part, slabs, D, dw_is_bf16 ? nullptr : (float*)dw_out,
                                                   dw_is_bf16 ? (bf16*)dw_out : nullptr);
    HMF_CHECK_CUDA(cudaGetLastError());
  }
  return HMF_OK;
}

HMF_API int hmf_gated_norm_fwd(const void* x, const void* gate, const void* w, void* y, float* rstd,
                               long long N, int D, int w_rows, float eps, int mode, cudaStream_t st) {
  HMF_REQUIRE(D == 64 || D == 128 || D == 256, "gated_norm: head dim %d unsupported (64/128/256)", D);
  if (N == 0) return HMF_OK;
  const int rpw = 256 / D, warps = 8;
  const long long blocks = (N + (long long)rpw * warps - 1) / ((long long)rpw * warps);
#define LAUNCH(DD)                                                                                   \
  gated_norm_fwd_kernel<DD><<<(unsigned)blocks, warps * 32, 0, st>>>(                                  \
      (const bf16*)x, (const bf16*)gate, (const bf16*)w, (bf16*)y, rstd, N, w_rows, eps, mode)
  if (D == 64) LAUNCH(64); else if (D == 128) LAUNCH(128); else LAUNCH(256);
#undef LAUNCH
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_gated_norm_bwd(const void* x, const void* gate, const void* w, const void* dy,
                               const float* rstd, void* dx, void* dgate, float* dw_acc, long long N,
                               int D, int w_rows, int mode, cudaStream_t st) {
  HMF_REQUIRE(D == 64 || D == 128 || D == 256, "gated_norm_bwd: head dim %d unsupported", D);
  HMF_REQUIRE((long long)(w_rows > 1 ? w_rows : 1) * D * 4 <= 160 * 1024, "gated_norm_bwd: weight too large");
  if (N == 0) return HMF_OK;
  long long blocks = (N + 255) / 256;
  const long long cap = (long long)sm_count() * 4;
  if (blocks > cap) blocks = cap;
  long long rpb = (N + blocks - 1) / blocks;
  const int rpw = 256 / D;
  rpb = (rpb + rpw * 8 - 1) / (rpw * 8) * (rpw * 8);
  blocks = (N + rpb - 1) / rpb;
  const size_t smem = (size_t)(w_rows > 1 ? w_rows : 1) * D * sizeof(float);
#define LAUNCH(DD)                                                                                   \
  do {                                                                                               \
    if (smem > 48 * 1024)                                                                            \
      HMF_CHECK_CUDA(cudaFuncSetAttribute(gated_norm_bwd_kernel<DD>,                                  \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));  \
    gated_norm_bwd_kernel<DD><<<(unsigned)blocks, 256, smem, st>>>(                                   \
        (const bf16*)x, (const bf16*)gate, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx,          \
        (bf16*)dgate, dw_acc, N, w_rows, mode, rpb);                                                  \
  } while (0)
  if (D == 64) LAUNCH(64); else if (D == 128) LAUNCH(128); else LAUNCH(256);
#undef LAUNCH
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_swiglu_fwd(const void* g, const void* u, void* y, long long n, cudaStream_t st) {
  HMF_REQUIRE(n % 8 == 0, "swiglu: element count %lld must be a multiple of 8", n);
  if (n == 0) return HMF_OK;
  swiglu_fwd_kernel<<<grid_for(n / 8, 256, 16), 256, 0, st>>>((const bf16*)g, (const bf16*)u, (bf16*)y, n / 8);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
HMF_API int hmf_swiglu_bwd(const void* g, const void* u, const void* dy, void* dg, void* du, long long n,
                           cudaStream_t st) {
  HMF_REQUIRE(n % 8 == 0, "swiglu_bwd: element count %lld must be a multiple of 8", n);
  if (n == 0) return HMF_OK;
  swiglu_bwd_kernel<<<grid_for(n / 8, 256, 16), 256, 0, st>>>((const bf16*)g, (const bf16*)u,
                                                            (const bf16*)dy, (bf16*)dg, (bf16*)du, n / 8);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_rope(const void* x, const void* cos_t, const void* sin_t, void* y, long long rows, int H,
                     int D, int R, int backward, long long x_row_stride, cudaStream_t st) {
  HMF_REQUIRE(R % 16 == 0 && R <= D && D % 8 == 0, "rope: R=%d D=%d unsupported", R, D);
  HMF_REQUIRE(x_row_stride % 8 == 0, "rope: row stride %lld must be a multiple of 8", x_row_stride);
  if (rows == 0) return HMF_OK;
  const long long items = rows * H * (R / 16 + (D - R) / 8);
  rope_kernel<<<grid_for(items, 256, 16), 256, 0, st>>>((const bf16*)x, (const bf16*)cos_t,
                                                      (const bf16*)sin_t, (bf16*)y, rows, H, D, R,
                                                      backward ? -1.f : 1.f, x_row_stride);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_conv1d_fwd(const void* x, const void* w, const void* bias, const void* init, void* y,
                           void* final_state, int B, int T, int C, int K, int act, cudaStream_t st) {
  HMF_REQUIRE(K == CONV_K, "conv1d: kernel size %d unsupported (4)", K);
  HMF_REQUIRE(C % 8 == 0, "conv1d: channels %d must be a multiple of 8", C);
  if (B == 0 || T == 0) return HMF_OK;
  const int cx = 128;
  dim3 grid((C / 8 + cx - 1) / cx, (T + CONV_TT - 1) / CONV_TT, B);
  conv1d_fwd_kernel<<<grid, cx, 0, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)bias,
                                         (const bf16*)init, (bf16*)y, (bf16*)final_state, T, C, act);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
// dw [C,K] and dbias [C] are fp32 and must be zeroed by the caller; dinit [B,K-1,C] fp32 (or null).
HMF_API int hmf_conv1d_bwd(const void* x, const void* w, const void* bias, const void* init,
                           const void* dy, void* dx, float* dinit, float* dw, float* dbias, int B, int T,
                           int C, int K, int act, cudaStream_t st) {
  HMF_REQUIRE(K == CONV_K, "conv1d_bwd: kernel size %d unsupported (4)", K);
  HMF_REQUIRE(C % 8 == 0, "conv1d_bwd: channels %d must be a multiple of 8", C);
  if (B == 0 || T == 0) return HMF_OK;
  const int cx = 64;
  dim3 grid((C / 8 + cx - 1) / cx, (T + CONV_TT - 1) / CONV_TT, B);
  conv1d_bwd_kernel<<<grid, cx, 0, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)bias,
                                         (const bf16*)init, (const bf16*)dy, (bf16*)dx, dinit, dw, dbias,
                                         T, C, act);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
HMF_API int hmf_conv1d_update(const void* x, void* state, const void* w, const void* bias, void* y,
                              const int* slots, int B, int C, int K, int act, cudaStream_t st) {
  HMF_REQUIRE(K == CONV_K && C % 8 == 0, "conv1d_update: K=%d C=%d unsupported", K, C);
  if (B == 0) return HMF_OK;
  dim3 grid((C / 8 + 127) / 128, B);
  conv1d_update_kernel<<<grid, 128, 0, st>>>((const bf16*)x, (bf16*)state, (const bf16*)w,
                                             (const bf16*)bias, (bf16*)y, slots, C, act);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_ce_fwd_bwd(void* logits, const long long* labels, float* loss_sum, int* n_valid,
                           long long n, int V, long long ld, long long ignore_index, cudaStream_t st) {
  HMF_REQUIRE(ld % 8 == 0, "cross entropy: row stride %lld must be a multiple of 8", ld);
  if (n == 0) return HMF_OK;
  ce_fwd_bwd_kernel<<<(unsigned)n, 1024, 0, st>>>((bf16*)logits, labels, loss_sum, n_valid, V, ld,
                                                  ignore_index);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_sumsq(const void* g, int g_is_bf16, long long n, float* out, cudaStream_t st) {
  if (n == 0) return HMF_OK;
  const int grid = grid_for(n, 512, 8);
  if (g_is_bf16) sumsq_kernel<bf16><<<grid, 512, 0, st>>>((const bf16*)g, n, out);
  else sumsq_kernel<float><<<grid, 512, 0, st>>>((const float*)g, n, out);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// dtype codes: 0 = bf16, 1 = fp32 for params (p), grads (g) and moments (s).
HMF_API int hmf_adamw(void* p, const void* g, void* m, void* v, float* master, long long n, int p_dt,
                      int g_dt, int s_dt, float lr, float beta1, float beta2, float eps, float wd,
                      float bc1, float bc2, const float* norm_sq, float max_norm, float grad_scale,
                      cudaStream_t st) {
  if (n == 0) return HMF_OK;
  const int grid = grid_for(n, 512, 8);
#define ADAMW(P, G, S)                                                                              \
  adamw_kernel<P, G, S><<<grid, 512, 0, st>>>((P*)p, (const G*)g, (S*)m, (S*)v, master, n, lr, beta1, \
                                              beta2, eps, wd, bc1, bc2, norm_sq, max_norm, grad_scale)
  const int code = p_dt * 4 + g_dt * 2 + s_dt;
  switch (code) {
    case 0: ADAMW(bf16, bf16, bf16); break;
    case 1: ADAMW(bf16, bf16, float); break;
    case 2: ADAMW(bf16, float, bf16); break;
    case 3: ADAMW(bf16, float, float); break;
    case 4: ADAMW(float, bf16, bf16); break;
    case 5: ADAMW(float, bf16, float); break;
    case 6: ADAMW(float, float, bf16); break;
    case 7: ADAMW(float, float, float); break;
    default: set_last_error("adamw: bad dtype codes"); return HMF_ERR_BAD_ARG;
  }
#undef ADAMW
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// ------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared and documented in no_alloc.h).
// ------------------------------------------------------------------------------------------
#include <mutex>

#include "no_alloc.h"

// Workspace for the per-slab partial sums of the weight gradient: [MAX_SLABS][MAX_D] floats.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_noalloc_rmsnorm_ws[HMF_NOALLOC_RMSNORM_MAX_SLABS * HMF_NOALLOC_RMSNORM_MAX_D];

static int noalloc_workspace(float** out) {
  static float* table[64] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  HMF_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_last_error("rms_norm_bwd_noalloc: device index %d out of range", dev);
    return HMF_ERR_BAD_ARG;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (table[dev] == nullptr) {
    float* p = nullptr;
    // resolved once per device, with that device current
    HMF_CHECK_CUDA(cudaGetSymbolAddress((void**)&p, g_noalloc_rmsnorm_ws));
    table[dev] = p;
  }
  *out = table[dev];
  return HMF_OK;
}

HMF_API int hmf_rms_norm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                                     void* dw_out, int dw_is_bf16, long long N, int D, int zero_centered,
                                     cudaStream_t st) {
  HMF_REQUIRE(x && dy && rstd && dx, "rms_norm_bwd_noalloc: null tensor");
  HMF_REQUIRE(D > 0 && D % 8 == 0, "rms_norm_bwd_noalloc: D=%d must be a positive multiple of 8", D);
  if (D > HMF_NOALLOC_RMSNORM_MAX_D) {
    set_last_error("rms_norm_bwd_noalloc: D=%d exceeds the built-in workspace limit of %d columns; "
                   "use hmf_rms_norm_bwd with a caller-provided buffer", D, HMF_NOALLOC_RMSNORM_MAX_D);
    return HMF_ERR_TOO_LARGE;
  }
  if (N == 0) return HMF_OK;
  float* ws = nullptr;
  int rc = noalloc_workspace(&ws);
  if (rc != HMF_OK) return rc;
  const int warps = 8;
  const long long blocks = (N + warps - 1) / warps;
  rms_norm_bwd_dx_kernel<<<(unsigned)blocks, warps * 32, 0, st>>>(
      (const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, N, D, zero_centered);
  HMF_CHECK_CUDA(cudaGetLastError());
  if (w && dw_out) {
    int slabs = hmf_rms_norm_bwd_blocks(N);
    if (slabs > HMF_NOALLOC_RMSNORM_MAX_SLABS) slabs = HMF_NOALLOC_RMSNORM_MAX_SLABS;
    const long long rps = (N + slabs - 1) / slabs;
    int CT = D / 8;
    if (CT > 256) CT = 256;
    int p2 = 1;
    while (p2 * 2 <= CT) p2 *= 2;
    CT = p2;
    dim3 grid((D / 8 + CT - 1) / CT, slabs);
    // every word of ws[0 .. slabs*D) is written by this launch before colsum reads it
    rms_norm_bwd_dw_kernel<<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)dy, rstd, ws, N, D, rps, CT);
    HMF_CHECK_CUDA(cudaGetLastError());
    colsum_kernel<<<(D + 255) / 256, 256, 0, st>>>(ws, slabs, D, dw_is_bf16 ? nullptr : (float*)dw_out,
                                                   dw_is_bf16 ? (bf16*)dw_out : nullptr);
    HMF_CHECK_CUDA(cudaGetLastError());
  }
  return HMF_OK;
}
