// Fused glue kernels of the decode step (one token per request).  They remove the small per-head
// launches between the GEMMs of a layer:
//   * hmf_qkv_norm_rope_append: packed QKV row -> per-head RMSNorm (q, k) -> RoPE -> q buffer and paged K/V cache
//   * hmf_swiglu_packed:        [R, 2F] = [gate | up] -> silu(gate) * up
//   * hmf_ssd_decode_packed:    Mamba2 state update reading x / B / C / dt straight from the packed projection and
//                               convolution outputs (softplus(dt + bias) and A = -exp(A_log) computed in place)
#include <math.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace decode_fused {

using bf16 = __nv_bfloat16;

// grid (R, Hq + 2 Hkv), 128 threads (= head dim): thread t <-> element t of the head.
__global__ void __launch_bounds__(128)
qkv_norm_rope_append_kernel(const bf16* __restrict__ qkv, long long ld, const bf16* __restrict__ qw,
                            const bf16* __restrict__ kw, float eps, int zero_centered, const bf16* __restrict__ cs,
                            const bf16* __restrict__ sn, int rot, bf16* __restrict__ q_out, bf16* __restrict__ kc,
                            bf16* __restrict__ vc, const long long* __restrict__ slot_map, int Hq, int Hkv) {
  constexpr int D = 128;
  const int r = blockIdx.x, hh = blockIdx.y, t = threadIdx.x;
  __shared__ float s_x[D];
  __shared__ float s_red[4];
  const bool is_q = hh < Hq, is_k = !is_q && hh < Hq + Hkv;
  float x = __bfloat162float(qkv[(size_t)r * ld + (size_t)hh * D + t]);
  const long long slot = slot_map[r];
  if (!is_q && !is_k) {   // V: plain append
    if (slot >= 0) vc[(size_t)slot * Hkv * D + (size_t)(hh - Hq - Hkv) * D + t] = __float2bfloat16(x);
    return;
  }
  const bf16* w = is_q ? qw : kw;
  if (w != nullptr) {
    const float ss = warp_sum(x * x);
    if ((t & 31) == 0) s_red[t >> 5] = ss;
    __syncthreads();
    const float tot = s_red[0] + s_red[1] + s_red[2] + s_red[3];
    float wv = __bfloat162float(w[t]);
    if (zero_centered) wv += 1.f;
    x = x * rsqrtf(tot / D + eps) * wv;
    x = __bfloat162float(__float2bfloat16(x));   // the unfused path rounds between the norm and the rotation
  }
  s_x[t] = x;
  __syncthreads();
  float y = x;
  if (t < rot) {
    const int half = rot / 2;
    const float c = __bfloat162float(cs[(size_t)r * rot + t]), s = __bfloat162float(sn[(size_t)r * rot + t]);
    const float partner = t < half ? -s_x[t + half] : s_x[t - half];
    y = x * c + partner * s;
  }
  if (is_q) {
    q_out[((size_t)r * Hq + hh) * D + t] = __float2bfloat16(y);
  } else if (slot >= 0) {
    kc[(size_t)slot * Hkv * D + (size_t)(hh - Hq) * D + t] = __float2bfloat16(y);
  }
}

// Mamba2 decode glue: one pass over the convolution input row [x | B | C] (heads of 128 channels): x heads are copied,
// B and C heads get their per-head RMSNorm and the rotary embedding; the result is a contiguous row for the
// convolution update (replaces split + two norms + two rotations + concatenation + copy).
__global__ void __launch_bounds__(128)
heads_norm_rope_kernel(const bf16* __restrict__ in, long long ld_in, bf16* __restrict__ out, long long ld_out, int h_plain,
                       int h_b, const bf16* __restrict__ wb, const bf16* __restrict__ wc, float eps, int zero_centered,
                       const bf16* __restrict__ cs, const bf16* __restrict__ sn, int rot) {
  constexpr int D = 128;
  const int r = blockIdx.x, hh = blockIdx.y, t = threadIdx.x;
  __shared__ float s_x[D];
  __shared__ float s_red[4];
  float x = __bfloat162float(in[(size_t)r * ld_in + (size_t)hh * D + t]);
  bf16* dst = out + (size_t)r * ld_out + (size_t)hh * D + t;
  if (hh < h_plain) {
    *dst = __float2bfloat16(x);
    return;
  }
  const bf16* w = hh < h_plain + h_b ? wb : wc;
  if (w != nullptr) {
    const float ss = warp_sum(x * x);
    if ((t & 31) == 0) s_red[t >> 5] = ss;
    __syncthreads();
    const float tot = s_red[0] + s_red[1] + s_red[2] + s_red[3];
    float wv = __bfloat162float(w[t]);
    if (zero_centered) wv += 1.f;
    x = x * rsqrtf(tot / D + eps) * wv;
    x = __bfloat162float(__float2bfloat16(x));   // the unfused path rounds between the norm and the rotation
  }
  s_x[t] = x;
  __syncthreads();
  float y = x;
  if (t < rot) {
    const int half = rot / 2;
    const float c = __bfloat162float(cs[(size_t)r * rot + t]), s = __bfloat162float(sn[(size_t)r * rot + t]);
    const float partner = t < half ? -s_x[t + half] : s_x[t - half];
    y = x * c + partner * s;
  }
  *dst = __float2bfloat16(y);
}

__global__ void swiglu_packed_kernel(const bf16* __restrict__ gu, bf16* __restrict__ y, long long rows, int F8,
                                     long long ld) {
  const long long total = rows * F8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / F8;
    const int c = (int)(i % F8) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + row * ld + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + row * ld + (size_t)F8 * 8 + c);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(gp[j]), u = __bfloat1622float2(up[j]);
      op[j] = pack_bf16x2(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(y + row * (size_t)F8 * 8 + c) = o4;
  }
}

// Mamba2 step, state [slots, H, P, N] fp32, N = 128 * NG.  One warp per state row, 8 warps, 4 rows in flight.
//   x  = xbc + r * ld_xbc + x_off  [Hx, P]      B = ... + b_off [Hb, N]      C = ... + c_off [H, N]
//   dt = softplus(dt_raw[r * ld_dt + h] + dt_bias[h]),  A = -exp(A_log[h])
template <int NG>
__global__ void __launch_bounds__(256)
ssd_decode_packed_kernel(const bf16* __restrict__ xbc, long long ld_xbc, int x_off, int b_off, int c_off,
                         const bf16* __restrict__ dt_raw, long long ld_dt, const float* __restrict__ dt_bias,
                         const float* __restrict__ A_log, const float* __restrict__ Dp, float* __restrict__ state,
                         const int* __restrict__ slots, bf16* __restrict__ y, int H, int Hx, int Hb, int P) {
  constexpr int N = NG * 128;
  const int r = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hx = h / (H / Hx), hb = h / (H / Hb);
  const bf16* row = xbc + (size_t)r * ld_xbc;
  float bv[NG][4], cv[NG][4];
#pragma unroll
  for (int j = 0; j < NG; ++j) {
    const uint2 ub = *reinterpret_cast<const uint2*>(row + b_off + (size_t)hb * N + j * 128 + lane * 4);
    const uint2 uc = *reinterpret_cast<const uint2*>(row + c_off + (size_t)h * N + j * 128 + lane * 4);
    const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ub.x));
    const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ub.y));
    const float2 c0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uc.x));
    const float2 c1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uc.y));
    bv[j][0] = b0.x; bv[j][1] = b0.y; bv[j][2] = b1.x; bv[j][3] = b1.y;
    cv[j][0] = c0.x; cv[j][1] = c0.y; cv[j][2] = c1.x; cv[j][3] = c1.y;
  }
  const float z = __bfloat162float(dt_raw[(size_t)r * ld_dt + h]) + dt_bias[h];
  const float dtv = z > 20.f ? z : log1pf(__expf(z));
  const float a = __expf(-dtv * __expf(A_log[h]));
  const float dcoef = Dp ? Dp[h] : 0.f;
  float* S = state + ((size_t)slots[r] * H + h) * P * N;
  constexpr int RU = 4;
  for (int p0 = warp * RU; p0 < P; p0 += 8 * RU) {
    float4 sv[RU][NG];
    float xv[RU];
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const int pr = min(p0 + u, P - 1);
      xv[u] = __bfloat162float(row[x_off + (size_t)hx * P + pr]);
#pragma unroll
      for (int j = 0; j < NG; ++j) sv[u][j] = *reinterpret_cast<const float4*>(S + (size_t)pr * N + j * 128 + lane * 4);
    }
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      if (p0 + u >= P) break;
      const float dx = dtv * xv[u];
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < NG; ++j) {
        float4 s4 = sv[u][j];
        s4.x = fmaf(s4.x, a, dx * bv[j][0]);
        s4.y = fmaf(s4.y, a, dx * bv[j][1]);
        s4.z = fmaf(s4.z, a, dx * bv[j][2]);
        s4.w = fmaf(s4.w, a, dx * bv[j][3]);
        acc += s4.x * cv[j][0] + s4.y * cv[j][1] + s4.z * cv[j][2] + s4.w * cv[j][3];
        *reinterpret_cast<float4*>(S + (size_t)(p0 + u) * N + j * 128 + lane * 4) = s4;
      }
      acc = warp_sum(acc);
      if (lane == 0) y[((size_t)r * H + h) * P + p0 + u] = __float2bfloat16(acc + dcoef * xv[u]);
    }
  }
}

}  // namespace decode_fused
}  // namespace hmf

using namespace hmf;
using namespace hmf::decode_fused;

// qkv [R, ld] = [q (Hq*128) | k (Hkv*128) | v (Hkv*128)] bf16; q_weight / k_weight [128] or null (no QK norm);
// cos / sin [R, rot] bf16; q_out [R, Hq, 128]; caches [num_blocks * block_size, Hkv, 128]; slot_map [R] int64.
HMF_API int hmf_qkv_norm_rope_append(const void* qkv, long long ld, const void* q_weight, const void* k_weight,
                                     float eps, int zero_centered, const void* cos_t, const void* sin_t, int rot,
                                     void* q_out, void* kc, void* vc, const long long* slot_map, int R, int Hq, int Hkv,
                                     int D, cudaStream_t st) {
  HMF_REQUIRE(D == 128, "qkv_norm_rope_append: head dim %d unsupported (128)", D);
  HMF_REQUIRE(rot % 2 == 0 && rot <= D, "qkv_norm_rope_append: rotary dim %d unsupported", rot);
  if (R == 0) return HMF_OK;
  dim3 grid(R, Hq + 2 * Hkv);
  qkv_norm_rope_append_kernel<<<grid, 128, 0, st>>>((const bf16*)qkv, ld, (const bf16*)q_weight, (const bf16*)k_weight,
                                                    eps, zero_centered, (const bf16*)cos_t, (const bf16*)sin_t, rot,
                                                    (bf16*)q_out, (bf16*)kc, (bf16*)vc, slot_map, Hq, Hkv);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// in [R, ld_in] bf16 (h_plain + h_b + h_c heads of 128 channels), out [R, ld_out] bf16; wb / wc [128] or null (no norm);
// cos / sin [R, rot] bf16 (rot = 0: no rotation).
HMF_API int hmf_heads_norm_rope(const void* in, long long ld_in, void* out, long long ld_out, int h_plain, int h_b, int h_c,
                                const void* wb, const void* wc, float eps, int zero_centered, const void* cos_t,
                                const void* sin_t, int rot, int R, cudaStream_t st) {
  HMF_REQUIRE(rot % 2 == 0 && rot <= 128 && (rot == 0 || (cos_t && sin_t)), "heads_norm_rope: rotary dim %d unsupported", rot);
  HMF_REQUIRE((wb == nullptr) == (wc == nullptr), "heads_norm_rope: both norm weights or none");
  if (R == 0) return HMF_OK;
  dim3 grid(R, h_plain + h_b + h_c);
  heads_norm_rope_kernel<<<grid, 128, 0, st>>>((const bf16*)in, ld_in, (bf16*)out, ld_out, h_plain, h_b, (const bf16*)wb,
                                               (const bf16*)wc, eps, zero_centered, (const bf16*)cos_t,
                                               (const bf16*)sin_t, rot);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_swiglu_packed(const void* gu, void* y, long long rows, int F, long long ld, cudaStream_t st) {
  HMF_REQUIRE(F % 8 == 0 && ld % 8 == 0, "swiglu_packed: F=%d ld=%lld must be multiples of 8", F, ld);
  if (rows == 0) return HMF_OK;
  const long long items = rows * (F / 8);
  const int grid = (int)((items + 255) / 256 < 4096 ? (items + 255) / 256 : 4096);
  swiglu_packed_kernel<<<grid, 256, 0, st>>>((const bf16*)gu, (bf16*)y, rows, F / 8, ld);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_ssd_decode_packed(const void* xbc, long long ld_xbc, int x_off, int b_off, int c_off,
                                  const void* dt_raw, long long ld_dt, const float* dt_bias, const float* A_log,
                                  const float* Dp, float* state, const int* slots, void* y, int R, int H, int Hx,
                                  int Hb, int P, int N, cudaStream_t st) {
  HMF_REQUIRE(N == 128 || N == 256, "ssd_decode_packed: N=%d unsupported (128, 256)", N);
  HMF_REQUIRE(H % Hx == 0 && H % Hb == 0, "ssd_decode_packed: head counts do not divide H=%d", H);
  HMF_REQUIRE(b_off % 4 == 0 && c_off % 4 == 0 && ld_xbc % 4 == 0, "ssd_decode_packed: offsets must be multiples of 4");
  if (R == 0) return HMF_OK;
  dim3 grid(R, H);
  if (N == 128)
    ssd_decode_packed_kernel<1><<<grid, 256, 0, st>>>((const bf16*)xbc, ld_xbc, x_off, b_off, c_off, (const bf16*)dt_raw,
                                                      ld_dt, dt_bias, A_log, Dp, state, slots, (bf16*)y, H, Hx, Hb, P);
  else
    ssd_decode_packed_kernel<2><<<grid, 256, 0, st>>>((const bf16*)xbc, ld_xbc, x_off, b_off, c_off, (const bf16*)dt_raw,
                                                      ld_dt, dt_bias, A_log, Dp, state, slots, (bf16*)y, H, Hx, Hb, P);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// ------------------------------------------------------------------------------------
// Gated KalmaNet decode step, fully fused (one CTA per (request, head), 128 threads, head dim 128):
//   q, k <- x / (|x| + eps);  k, v <- (beta + eps) k, v  (optional)
//   H_kk <- e^{gk} H_kk + k k^T            (thread t keeps row t of the symmetric matrix in registers)
//   lambda = ridge * |H_kk|_F ;  num_iter Chebyshev steps on (H_kk + lambda I) x = q
//   q' = q + alpha (x - q)  (or x);  H_kv <- e^{g} H_kv + k v^T ;  o = scale * H_kv^T q'
// States [slots, H, 128, 128] fp32, indexed through slots[r].
// ------------------------------------------------------------------------------------
namespace hmf {
namespace decode_fused {

__device__ __forceinline__ float block_sum_128(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}

__global__ void __launch_bounds__(128)
gka_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                  const float* __restrict__ g, const float* __restrict__ beta, const float* __restrict__ alpha,
                  float* __restrict__ h_kk, float* __restrict__ h_kv, const int* __restrict__ slots,
                  bf16* __restrict__ o, int H, int Hq, int Hk, int Hv, float scale, float ridge, int num_iter,
                  int use_gk) {
  constexpr int D = 128;
  const int r = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
  __shared__ float s_x[D], s_k[D], s_red[4];
  const int hq = h / (H / Hq), hk = h / (H / Hk), hv = h / (H / Hv);
  float qv = __bfloat162float(q[((size_t)r * Hq + hq) * D + t]);
  float kv = __bfloat162float(k[((size_t)r * Hk + hk) * D + t]);
  float vv = __bfloat162float(v[((size_t)r * Hv + hv) * D + t]);
  const float eps = 1e-6f;
  qv = qv / (sqrtf(block_sum_128(qv * qv, s_red)) + eps);
  kv = kv / (sqrtf(block_sum_128(kv * kv, s_red)) + eps);
  if (beta != nullptr) {
    const float b = beta[(size_t)r * H + h] + eps;
    kv *= b;
    vv *= b;
  }
  const float gv = g[(size_t)r * H + h];
  const size_t sbase = (((size_t)slots[r] * H + h) * D) * D;
  // ---- covariance state update, row t in registers ----
  s_k[t] = kv;
  __syncthreads();
  float row[D];
  const float dkk = use_gk ? __expf(gv) : 1.f;
  float* Hrow = h_kk + sbase + (size_t)t * D;
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < D; j += 4) {
    float4 h4 = *reinterpret_cast<const float4*>(Hrow + j);
    h4.x = fmaf(h4.x, dkk, kv * s_k[j]);
    h4.y = fmaf(h4.y, dkk, kv * s_k[j + 1]);
    h4.z = fmaf(h4.z, dkk, kv * s_k[j + 2]);
    h4.w = fmaf(h4.w, dkk, kv * s_k[j + 3]);
    *reinterpret_cast<float4*>(Hrow + j) = h4;
    row[j] = h4.x; row[j + 1] = h4.y; row[j + 2] = h4.z; row[j + 3] = h4.w;
    ss += h4.x * h4.x + h4.y * h4.y + h4.z * h4.z + h4.w * h4.w;
  }
  float xq = qv;     // value of q' for this feature
  if (num_iter > 0) {
    const float fro = sqrtf(block_sum_128(ss, s_red));
    const float lam = ridge * fro;
    float denom = 2.f * lam + fro;
    if (denom == 0.f) denom = 1.f;
    const float step = 2.f / denom;
    const float c = (fro / denom * 0.5f) * (fro / denom * 0.5f);
    float x_prev = 0.f, x = step * qv, omega = 2.f;
    for (int it = 0; it < num_iter; ++it) {
      __syncthreads();
      s_x[t] = x;
      __syncthreads();
      float hx = 0.f;
#pragma unroll
      for (int j = 0; j < D; ++j) hx = fmaf(row[j], s_x[j], hx);
      omega = 1.f / (1.f - c * omega);
      const float upd = step * omega * (hx + lam * x - qv) + (omega - 1.f) * x_prev;
      x_prev = x;
      x = omega * x - upd;
    }
    xq = (alpha != nullptr) ? qv + alpha[(size_t)r * H + h] * (x - qv) : x;
  }
  // ---- key-value state update and read-out: thread t owns column t of H_kv [Dk, Dv] ----
  __syncthreads();
  s_x[t] = xq * scale;
  __syncthreads();
  const float dkv = __expf(gv);
  float* S = h_kv + sbase;
  float out = 0.f;
#pragma unroll 8
  for (int d = 0; d < D; ++d) {
    const float sv = fmaf(S[(size_t)d * D + t], dkv, s_k[d] * vv);
    S[(size_t)d * D + t] = sv;
    out = fmaf(sv, s_x[d], out);
  }
  o[((size_t)r * H + h) * D + t] = __float2bfloat16(out);
}

}  // namespace decode_fused
}  // namespace hmf

// q [R, Hq, 128], k [R, Hk, 128], v [R, Hv, 128] bf16 (after the convolution); g [R, H] fp32 log decay;
// beta / alpha [R, H] fp32 (already through the sigmoid) or null; states [slots, H, 128, 128] fp32.
HMF_API int hmf_gka_decode(const void* q, const void* k, const void* v, const float* g, const float* beta,
                           const float* alpha, float* h_kk, float* h_kv, const int* slots, void* o, int R, int H,
                           int Hq, int Hk, int Hv, int D, float scale, float ridge, int num_iter, int use_gk,
                           cudaStream_t st) {
  HMF_REQUIRE(D == 128, "gka_decode: head dim %d unsupported (128)", D);
  HMF_REQUIRE(H % Hq == 0 && H % Hk == 0 && H % Hv == 0, "gka_decode: head counts do not divide H=%d", H);
  if (R == 0) return HMF_OK;
  dim3 grid(R, H);
  hmf::decode_fused::gka_decode_kernel<<<grid, 128, 0, st>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, g, beta, alpha, h_kk, h_kv, slots,
      (__nv_bfloat16*)o, H, Hq, Hk, Hv, scale, ridge, num_iter, use_gk);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
