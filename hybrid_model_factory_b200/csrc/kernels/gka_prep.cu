// Gated KalmaNet input preparation in one pass (and its backward):
//   qn = q / (|q| + eps),   kn = (beta + eps) k / (|k| + eps),   vn = (beta + eps) v
// q, k, v: rows [N, D] bf16 with a row stride (N = batch x time x heads, D = head dimension, a multiple of 8 up to
// 256); beta [N] fp32 or null (no beta gate: the factor is 1).  One warp per row; the three tensors of a row are read
// once and written once, where the unfused formulation makes about ten full-size passes in fp32.
// The forward keeps |q| and |k| for the backward:
//   dq = g/(n+eps) - q <g, q> / (n (n+eps)^2)                                    with n = |q|, g = dqn
//   dk = c (g/(n+eps) - k <g, k> / (n (n+eps)^2)),  dv = c dvn                   with c = beta + eps
//   dbeta = <dkn, k> / (n+eps) + <dvn, v>
// Reference: the eager formulation of `layers/gated_kalmanet/gka.py:575-600` in the reference project.
#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace gka_prep {

using bf16 = __nv_bfloat16;

// sum over the `group` consecutive lanes that share a row (group = 8, 16 or 32)
__device__ __forceinline__ float group_sum_f(float v, int group) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    if (o < group) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void ld8(const bf16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ void st8(bf16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// lane l holds elements [8 l, 8 l + 8) of a row (D <= 256)
__global__ void __launch_bounds__(256)
fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
           const float* __restrict__ beta, bf16* __restrict__ qn, bf16* __restrict__ kn, bf16* __restrict__ vn,
           float* __restrict__ nq, float* __restrict__ nk, long long N, int D, long long sq, long long sk,
           long long sv, float eps, int group) {
  // `group` lanes per row: a warp covers 32 / group rows, so narrow heads still use every lane
  const int lane = threadIdx.x & 31, sub = lane % group, c = sub * 8;
  const long long row = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * (32 / group) + lane / group;
  const bool on = row < N && c < D;
  float a[8], b[8], d[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = b[i] = d[i] = 0.f;
  if (on) {
    ld8(q + row * sq + c, a);
    ld8(k + row * sk + c, b);
    ld8(v + row * sv + c, d);
  }
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s1 = fmaf(a[i], a[i], s1);
    s2 = fmaf(b[i], b[i], s2);
  }
  const float n1 = sqrtf(group_sum_f(s1, group)), n2 = sqrtf(group_sum_f(s2, group));
  if (row >= N) return;
  const float cf = beta ? beta[row] + eps : 1.f;
  const float r1 = 1.f / (n1 + eps), r2 = cf / (n2 + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    a[i] *= r1;
    b[i] *= r2;
    d[i] *= cf;
  }
  if (on) {
    st8(qn + row * D + c, a);
    st8(kn + row * D + c, b);
    st8(vn + row * D + c, d);
  }
  if (sub == 0) {
    nq[row] = n1;
    nk[row] = n2;
  }
}

__global__ void __launch_bounds__(256)
bwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
           const float* __restrict__ beta, const float* __restrict__ nq, const float* __restrict__ nk,
           const bf16* __restrict__ gq, const bf16* __restrict__ gk, const bf16* __restrict__ gv,
           bf16* __restrict__ dq, bf16* __restrict__ dk, bf16* __restrict__ dv, float* __restrict__ dbeta,
           long long N, int D, long long sq, long long sk, long long sv, float eps, int group) {
  const int lane = threadIdx.x & 31, sub = lane % group, c = sub * 8;
  const long long row = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * (32 / group) + lane / group;
  const bool on = row < N && c < D;
  float a[8], b[8], d[8], ga[8], gb[8], gd[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = b[i] = d[i] = ga[i] = gb[i] = gd[i] = 0.f;
  if (on) {
    ld8(q + row * sq + c, a);
    ld8(k + row * sk + c, b);
    ld8(v + row * sv + c, d);
    ld8(gq + row * D + c, ga);
    ld8(gk + row * D + c, gb);
    ld8(gv + row * D + c, gd);
  }
  float dot_q = 0.f, dot_k = 0.f, dot_v = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    dot_q = fmaf(ga[i], a[i], dot_q);
    dot_k = fmaf(gb[i], b[i], dot_k);
    dot_v = fmaf(gd[i], d[i], dot_v);
  }
  dot_q = group_sum_f(dot_q, group);
  dot_k = group_sum_f(dot_k, group);
  dot_v = group_sum_f(dot_v, group);
  if (row >= N) return;
  const float n1 = nq[row], n2 = nk[row];
  const float cf = beta ? beta[row] + eps : 1.f;
  const float r1 = 1.f / (n1 + eps), r2 = 1.f / (n2 + eps);
  // x <g, x> / (n (n+eps)^2): zero rows have zero gradient through the norm
  const float t1 = n1 > 0.f ? dot_q * r1 * r1 / n1 : 0.f;
  const float t2 = n2 > 0.f ? dot_k * r2 * r2 / n2 : 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    a[i] = ga[i] * r1 - a[i] * t1;
    b[i] = cf * (gb[i] * r2 - b[i] * t2);
    d[i] = cf * gd[i];
  }
  if (on) {
    st8(dq + row * D + c, a);
    st8(dk + row * D + c, b);
    st8(dv + row * D + c, d);
  }
  if (dbeta && sub == 0) dbeta[row] = dot_k * r2 + dot_v;
}

}  // namespace gka_prep
}  // namespace hmf

using namespace hmf;

// q, k, v: [N, D] bf16 with row strides sq / sk / sv (elements, multiples of 8); outputs contiguous [N, D];
// nq, nk [N] fp32 receive the row norms.
HMF_API int hmf_gka_prep_fwd(const void* q, const void* k, const void* v, const float* beta, void* qn, void* kn,
                             void* vn, float* nq, float* nk, long long N, int D, long long sq, long long sk,
                             long long sv, float eps, cudaStream_t st) {
  HMF_REQUIRE(D % 8 == 0 && D > 0 && D <= 256, "gka_prep: head dimension %d unsupported (multiple of 8 up to 256)", D);
  HMF_REQUIRE(sq % 8 == 0 && sk % 8 == 0 && sv % 8 == 0, "gka_prep: row strides must be multiples of 8 elements");
  if (N == 0) return HMF_OK;
  const int group = D <= 64 ? 8 : (D <= 128 ? 16 : 32);
  const long long rows_per_block = 8 * (32 / group);
  gka_prep::fwd_kernel<<<(unsigned)((N + rows_per_block - 1) / rows_per_block), 256, 0, st>>>(
      (const gka_prep::bf16*)q, (const gka_prep::bf16*)k, (const gka_prep::bf16*)v, beta, (gka_prep::bf16*)qn,
      (gka_prep::bf16*)kn, (gka_prep::bf16*)vn, nq, nk, N, D, sq, sk, sv, eps, group);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// gq, gk, gv: gradients of qn, kn, vn (contiguous [N, D]); dq, dk, dv contiguous [N, D]; dbeta [N] fp32 or null.
HMF_API int hmf_gka_prep_bwd(const void* q, const void* k, const void* v, const float* beta, const float* nq,
                             const float* nk, const void* gq, const void* gk, const void* gv, void* dq, void* dk,
                             void* dv, float* dbeta, long long N, int D, long long sq, long long sk, long long sv,
                             float eps, cudaStream_t st) {
  HMF_REQUIRE(D % 8 == 0 && D > 0 && D <= 256, "gka_prep: head dimension %d unsupported (multiple of 8 up to 256)", D);
  HMF_REQUIRE(sq % 8 == 0 && sk % 8 == 0 && sv % 8 == 0, "gka_prep: row strides must be multiples of 8 elements");
  if (N == 0) return HMF_OK;
  const int group = D <= 64 ? 8 : (D <= 128 ? 16 : 32);
  const long long rows_per_block = 8 * (32 / group);
  gka_prep::bwd_kernel<<<(unsigned)((N + rows_per_block - 1) / rows_per_block), 256, 0, st>>>(
      (const gka_prep::bf16*)q, (const gka_prep::bf16*)k, (const gka_prep::bf16*)v, beta, nq, nk,
      (const gka_prep::bf16*)gq, (const gka_prep::bf16*)gk, (const gka_prep::bf16*)gv, (gka_prep::bf16*)dq,
      (gka_prep::bf16*)dk, (gka_prep::bf16*)dv, dbeta, N, D, sq, sk, sv, eps, group);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
