// Backward of the Gated DeltaNet chunk preparation, one CTA per (chunk of 64 tokens, head).
//
// Forward (per chunk): qn = scale q/|q|, kn = k/|k|, G = cumsum(g), D_ij = e^{G_i - G_j} (i >= j),
//   A = strict_lower(beta_i (kn_i.kn_j) D_ij), Tm = (I + A)^-1, u = Tm (beta v), w = Tm (beta e^G kn),
//   P = (qn kn^T) o D, qt = qn e^G, kt = kn e^{G_last - G}, glast = G_last.
// Given d_u, d_w, d_qt, d_kt, d_P, d_glast this kernel produces dq, dk, dv, dg, dbeta.  It replaces about fifty
// memory-bound PyTorch passes over [tokens, heads, 128] fp32 tensors by one kernel that keeps the chunk in shared
// memory; the twelve small products (64x64x128, 64x128x64, 64^3) run on the fp32 pipes with register tiling, the
// 64x64 triangular inverse by forward substitution (one column per thread).
// `gla` mode (plain gated linear attention: w = 0, u = v) skips everything that involves A.
#include <math.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace gdn_prep_bwd {

using bf16 = __nv_bfloat16;
constexpr int C = 64, D = 128, NT = 256;
constexpr int LD = D + 4;      // padded leading dimension of [C, D] fp32 tiles
constexpr int LB = D + 8;      // padded leading dimension of [C, D] bf16 tiles
constexpr int LC = C + 1;      // padded leading dimension of [C, C] tiles
constexpr int OFF_QN = 0;
constexpr int OFF_KN = OFF_QN + C * LD * 4;
constexpr int OFF_DKN = OFF_KN + C * LD * 4;
constexpr int OFF_R = OFF_DKN + C * LD * 4;                 // bf16 v | d_u | d_w   then   fp32 dqn
constexpr int R_BYTES = 3 * C * LB * 2;
constexpr int OFF_CC = OFF_R + R_BYTES;                     // KD | Tm | dT | X1
constexpr int OFF_SMALL = OFF_CC + 4 * C * LC * 4;
constexpr int SMEM_BYTES = OFF_SMALL + 12 * C * 4;
static_assert(C * LD * 4 <= R_BYTES, "dqn must fit the region of v / d_u / d_w");

struct Params {
  const bf16 *q, *k, *v;            // [B, T, H, D] with element strides (batch, token, head)
  const float *g, *beta;            // [B, T, H]
  const bf16* dvnT;                 // d_u^T  [BH, N, D, C]
  const bf16 *d_w, *d_qt, *d_kt;    // [BH, N, C, D]
  const float* d_P;                 // [BH, N, C, C] (lower triangular part is read)
  const float* d_gl;                // [BH, N]
  bf16 *dq, *dk, *dv;               // [B, T, H, D] contiguous
  float *dg, *dbeta;                // [B, T, H]
  long long q_sb, q_st, q_sh, k_sb, k_st, k_sh, v_sb, v_st, v_sh;
  int B, T, H, N;
  float scale;
  int l2norm, gla;
};

// acc(i, j) = sum_k A(i, k) B(k, j) for an M x N result; 256 threads as a 16 x 16 grid, thread (ti, tj) owns rows
// ti + 16 r and columns tj + 16 c.  TA: A is stored [K][M]; TB: B is stored [N][K].  epi(i, j, value) consumes it.
template <int M, int N, bool TA, bool TB, typename AT, typename BT, typename Epi>
__device__ __forceinline__ void mm(const AT* A, int lda, const BT* Bm, int ldb, int K, Epi epi) {
  constexpr int RM = M / 16, RN = N / 16;
  const int ti = threadIdx.x >> 4, tj = threadIdx.x & 15;
  float acc[RM][RN];
#pragma unroll
  for (int r = 0; r < RM; ++r)
#pragma unroll
    for (int c = 0; c < RN; ++c) acc[r][c] = 0.f;
#pragma unroll 4
  for (int kk = 0; kk < K; ++kk) {
    float a[RM], b[RN];
#pragma unroll
    for (int r = 0; r < RM; ++r) {
      const int i = ti + 16 * r;
      a[r] = (float)(TA ? A[kk * lda + i] : A[i * lda + kk]);
    }
#pragma unroll
    for (int c = 0; c < RN; ++c) {
      const int j = tj + 16 * c;
      b[c] = (float)(TB ? Bm[j * ldb + kk] : Bm[kk * ldb + j]);
    }
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
      for (int c = 0; c < RN; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
  }
#pragma unroll
  for (int r = 0; r < RM; ++r)
#pragma unroll
    for (int c = 0; c < RN; ++c) epi(ti + 16 * r, tj + 16 * c, acc[r][c]);
}

__global__ void __launch_bounds__(NT, 1) gdn_prep_bwd_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* s_qn = reinterpret_cast<float*>(smem + OFF_QN);
  float* s_kn = reinterpret_cast<float*>(smem + OFF_KN);
  float* s_dkn = reinterpret_cast<float*>(smem + OFF_DKN);
  bf16* s_v = reinterpret_cast<bf16*>(smem + OFF_R);
  bf16* s_du = s_v + C * LB;
  bf16* s_dw = s_du + C * LB;
  float* s_dqn = reinterpret_cast<float*>(smem + OFF_R);          // aliases v / d_u / d_w once they are dead
  float* s_KD = reinterpret_cast<float*>(smem + OFF_CC);
  float* s_Tm = s_KD + C * LC;
  float* s_dT = s_Tm + C * LC;
  float* s_X1 = s_dT + C * LC;
  float* sm = reinterpret_cast<float*>(smem + OFF_SMALL);
  float *s_G = sm, *s_eG = sm + C, *s_eR = sm + 2 * C, *s_beta = sm + 3 * C, *s_rq = sm + 4 * C, *s_rk = sm + 5 * C,
        *s_dG = sm + 6 * C, *s_dbeta = sm + 7 * C;

  const int n = blockIdx.x, bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = n * C;
  const size_t chunk = (size_t)bh * p.N + n;

  // ---- gates ----
  if (tid < C) {
    const int t = t0 + tid;
    s_G[tid] = t < p.T ? p.g[((size_t)b * p.T + t) * p.H + h] : 0.f;
    s_beta[tid] = (!p.gla && t < p.T) ? p.beta[((size_t)b * p.T + t) * p.H + h] : (p.gla ? 1.f : 0.f);
    s_dG[tid] = 0.f;
    s_dbeta[tid] = 0.f;
  }
  __syncthreads();
  if (tid == 0) {
    float run = 0.f;
    for (int i = 0; i < C; ++i) { run += s_G[i]; s_G[i] = run; }
  }
  __syncthreads();
  if (tid < C) {
    s_eG[tid] = __expf(s_G[tid]);
    s_eR[tid] = __expf(s_G[C - 1] - s_G[tid]);
  }
  // ---- rows of q, k (normalised), v, d_u, d_w into shared memory: warp w handles rows w, w + 8, ... ----
  for (int i = warp; i < C; i += 8) {
    const int t = t0 + i;
    float qv[4] = {0.f, 0.f, 0.f, 0.f}, kv[4] = {0.f, 0.f, 0.f, 0.f};
    if (t < p.T) {
      const uint2 uq = *reinterpret_cast<const uint2*>(p.q + (size_t)b * p.q_sb + (size_t)t * p.q_st + (size_t)h * p.q_sh + lane * 4);
      const uint2 uk = *reinterpret_cast<const uint2*>(p.k + (size_t)b * p.k_sb + (size_t)t * p.k_st + (size_t)h * p.k_sh + lane * 4);
      const float2 q0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uq.x));
      const float2 q1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uq.y));
      const float2 k0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uk.x));
      const float2 k1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uk.y));
      qv[0] = q0.x; qv[1] = q0.y; qv[2] = q1.x; qv[3] = q1.y;
      kv[0] = k0.x; kv[1] = k0.y; kv[2] = k1.x; kv[3] = k1.y;
    }
    float rq = 1.f, rk = 1.f;
    if (p.l2norm) {
      rq = rsqrtf(warp_sum(qv[0] * qv[0] + qv[1] * qv[1] + qv[2] * qv[2] + qv[3] * qv[3]) + 1e-6f);
      rk = rsqrtf(warp_sum(kv[0] * kv[0] + kv[1] * kv[1] + kv[2] * kv[2] + kv[3] * kv[3]) + 1e-6f);
    }
    if (lane == 0) { s_rq[i] = rq; s_rk[i] = rk; }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      s_qn[i * LD + lane * 4 + e] = qv[e] * rq * p.scale;
      s_kn[i * LD + lane * 4 + e] = kv[e] * rk;
    }
    uint2 uv = make_uint2(0u, 0u), uw = make_uint2(0u, 0u);
    if (t < p.T) uv = *reinterpret_cast<const uint2*>(p.v + (size_t)b * p.v_sb + (size_t)t * p.v_st + (size_t)h * p.v_sh + lane * 4);
    if (!p.gla) uw = *reinterpret_cast<const uint2*>(p.d_w + (chunk * C + i) * D + lane * 4);
    *reinterpret_cast<uint2*>(s_v + i * LB + lane * 4) = uv;
    *reinterpret_cast<uint2*>(s_dw + i * LB + lane * 4) = uw;
  }
  // d_u arrives transposed ([D, C]): element (i, d) = dvnT[d * C + i]
  for (int e = tid; e < C * D; e += NT) {
    const int d = e / C, i = e % C;
    s_du[i * LB + d] = p.dvnT[chunk * (size_t)(D * C) + e];
  }
  __syncthreads();

  const bf16* g_dqt = p.d_qt + chunk * (size_t)(C * D);
  const bf16* g_dkt = p.d_kt + chunk * (size_t)(C * D);
  auto out_row = [&](int i) -> size_t { return (((size_t)b * p.T + t0 + i) * p.H + h) * D; };

  if (!p.gla) {
    // ---- KD = strict_lower((kn kn^T) o D) ----
    mm<C, C, false, true>(s_kn, LD, s_kn, LD, D, [&](int i, int j, float a) {
      s_KD[i * LC + j] = i > j ? a * __expf(s_G[i] - s_G[j]) : 0.f;
    });
    __syncthreads();
    // ---- Tm = (I + beta KD)^-1 by forward substitution, thread c owns column c ----
    if (tid < C) {
      float x[C];
#pragma unroll
      for (int i = 0; i < C; ++i) {
        float acc = (i == tid) ? 1.f : 0.f;
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < C; ++j)
          if (j < i) dot = fmaf(s_KD[i * LC + j], x[j], dot);
        x[i] = acc - s_beta[i] * dot;
        s_Tm[i * LC + tid] = x[i];
      }
    }
    __syncthreads();
    // ---- dT = d_u (beta v)^T + d_w (beta e^G kn)^T ----
    mm<C, C, false, true>(s_du, LB, s_v, LB, D, [&](int i, int j, float a) { s_dT[i * LC + j] = a * s_beta[j]; });
    mm<C, C, false, true>(s_dw, LB, s_kn, LD, D, [&](int i, int j, float a) {
      s_dT[i * LC + j] += a * s_beta[j] * s_eG[j];
    });
    // ---- dbv = Tm^T d_u: dv = beta dbv, dbeta += dbv . v ----
    mm<C, D, true, false>(s_Tm, LC, s_du, LB, C, [&](int j, int d, float a) {
      if (t0 + j < p.T) p.dv[out_row(j) + d] = __float2bfloat16(a * s_beta[j]);
      atomicAdd(&s_dbeta[j], a * __bfloat162float(s_v[j * LB + d]));
    });
    // ---- dbk = Tm^T d_w: dkn = beta e^G dbk, x = e^G dbk . kn -> dbeta, dG ----
    mm<C, D, true, false>(s_Tm, LC, s_dw, LB, C, [&](int j, int d, float a) {
      s_dkn[j * LD + d] = a * s_beta[j] * s_eG[j];
      const float x = a * s_kn[j * LD + d] * s_eG[j];
      atomicAdd(&s_dbeta[j], x);
      atomicAdd(&s_dG[j], x * s_beta[j]);
    });
    __syncthreads();
    // ---- dA = -strict_lower(Tm^T dT Tm^T) ----
    mm<C, C, true, false>(s_Tm, LC, s_dT, LC, C, [&](int i, int j, float a) { s_X1[i * LC + j] = a; });
    __syncthreads();
    mm<C, C, false, true>(s_X1, LC, s_Tm, LC, C, [&](int i, int j, float a) { s_dT[i * LC + j] = i > j ? -a : 0.f; });
    __syncthreads();
    // ---- gate / beta gradients through A, and Mm = dA o D o beta_i ----
    for (int e = tid; e < C * C; e += NT) {
      const int i = e / C, j = e % C;
      float m = 0.f;
      if (i > j) {
        const float dA = s_dT[i * LC + j], kd = s_KD[i * LC + j];
        const float sA = dA * kd * s_beta[i];
        atomicAdd(&s_dG[i], sA);
        atomicAdd(&s_dG[j], -sA);
        atomicAdd(&s_dbeta[i], dA * kd);
        m = dA * __expf(s_G[i] - s_G[j]) * s_beta[i];
      }
      s_X1[i * LC + j] = m;
    }
    __syncthreads();
    // ---- dkn += Mm kn + Mm^T kn ----
    mm<C, D, false, false>(s_X1, LC, s_kn, LD, C, [&](int i, int d, float a) { s_dkn[i * LD + d] += a; });
    __syncthreads();
    mm<C, D, true, false>(s_X1, LC, s_kn, LD, C, [&](int i, int d, float a) { s_dkn[i * LD + d] += a; });
    __syncthreads();
  } else {
    // plain gated linear attention: u = v, so dv = d_u; no contribution to dkn yet
    for (int e = tid; e < C * D; e += NT) {
      const int i = e / D, d = e % D;
      if (t0 + i < p.T) p.dv[out_row(i) + d] = s_du[i * LB + d];
      s_dkn[i * LD + d] = 0.f;
    }
    __syncthreads();
  }

  // ---- intra-chunk scores: Nm = d_P o D (lower, diagonal included) into s_dT; s_P = Nm o (qn kn^T) feeds dG ----
  const float* g_dP = p.d_P + chunk * (size_t)(C * C);
  for (int e = tid; e < C * C; e += NT) {
    const int i = e / C, j = e % C;
    s_dT[i * LC + j] = i >= j ? g_dP[e] * __expf(s_G[i] - s_G[j]) : 0.f;
  }
  __syncthreads();
  mm<C, C, false, true>(s_qn, LD, s_kn, LD, D, [&](int i, int j, float a) {
    if (i >= j) {
      const float sP = s_dT[i * LC + j] * a;
      atomicAdd(&s_dG[i], sP);
      atomicAdd(&s_dG[j], -sP);
    }
  });
  // ---- dqn = Nm kn + e^G d_qt (v / d_u / d_w are dead: their region now holds dqn) ----
  __syncthreads();
  mm<C, D, false, false>(s_dT, LC, s_kn, LD, C, [&](int i, int d, float a) {
    const float dqt = __bfloat162float(g_dqt[i * D + d]);
    s_dqn[i * LD + d] = a + dqt * s_eG[i];
    atomicAdd(&s_dG[i], dqt * s_qn[i * LD + d] * s_eG[i]);
  });
  // ---- dkn += Nm^T qn + e^{G_last - G} d_kt ----
  mm<C, D, true, false>(s_dT, LC, s_qn, LD, C, [&](int i, int d, float a) {
    const float dkt = __bfloat162float(g_dkt[i * D + d]);
    s_dkn[i * LD + d] += a + dkt * s_eR[i];
    const float tt = dkt * s_kn[i * LD + d] * s_eR[i];
    atomicAdd(&s_dG[i], -tt);
    atomicAdd(&s_dG[C - 1], tt);
  });
  __syncthreads();
  if (tid == 0) s_dG[C - 1] += p.d_gl[chunk];
  // ---- back through the L2 normalisation, rows by warps; outputs in the [B, T, H, D] layout ----
  for (int i = warp; i < C; i += 8) {
    if (t0 + i >= p.T) continue;
    float dq[4], dk[4], qn[4], kn[4];
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int d = lane * 4 + e;
      dq[e] = s_dqn[i * LD + d]; qn[e] = s_qn[i * LD + d];
      dk[e] = s_dkn[i * LD + d]; kn[e] = s_kn[i * LD + d];
      sq += dq[e] * qn[e];
      sk += dk[e] * kn[e];
    }
    float oq[4], ok[4];
    if (p.l2norm) {
      sq = warp_sum(sq) / (p.scale * p.scale);
      sk = warp_sum(sk);
      const float aq = s_rq[i] * p.scale, ak = s_rk[i];
#pragma unroll
      for (int e = 0; e < 4; ++e) { oq[e] = (dq[e] - qn[e] * sq) * aq; ok[e] = (dk[e] - kn[e] * sk) * ak; }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) { oq[e] = dq[e] * p.scale; ok[e] = dk[e]; }
    }
    uint2 wq, wk;
    wq.x = pack_bf16x2(oq[0], oq[1]); wq.y = pack_bf16x2(oq[2], oq[3]);
    wk.x = pack_bf16x2(ok[0], ok[1]); wk.y = pack_bf16x2(ok[2], ok[3]);
    *reinterpret_cast<uint2*>(p.dq + out_row(i) + lane * 4) = wq;
    *reinterpret_cast<uint2*>(p.dk + out_row(i) + lane * 4) = wk;
  }
  __syncthreads();
  // ---- dg = reverse cumulative sum of dG; dbeta ----
  if (tid == 0) {
    float run = 0.f;
    for (int i = C - 1; i >= 0; --i) { run += s_dG[i]; s_dG[i] = run; }
  }
  __syncthreads();
  if (tid < C && t0 + tid < p.T) {
    const size_t o = ((size_t)b * p.T + t0 + tid) * p.H + h;
    p.dg[o] = s_dG[tid];
    if (!p.gla && p.dbeta != nullptr) p.dbeta[o] = s_dbeta[tid];
  }
}

}  // namespace gdn_prep_bwd
}  // namespace hmf

using namespace hmf;
using namespace hmf::gdn_prep_bwd;

// q, k, v: [B, T, H, 128] bf16 views (element strides batch / token / head, unit inner stride, already expanded to H
// heads); g, beta: [B, T, H] fp32 contiguous; dvnT [B*H, N, 128, 64] bf16; d_w, d_qt, d_kt [B*H, N, 64, 128] bf16
// (d_w may be null in gla mode); d_P [B*H, N, 64, 64] fp32; d_gl [B*H, N] fp32.
// Outputs dq, dk, dv [B, T, H, 128] bf16 contiguous; dg, dbeta [B, T, H] fp32 (dbeta may be null in gla mode).
HMF_API int hmf_gdn_prep_bwd(const void* q, const void* k, const void* v, const float* g, const float* beta,
                             const void* dvnT, const void* d_w, const void* d_qt, const void* d_kt, const float* d_P,
                             const float* d_gl, void* dq, void* dk, void* dv, float* dg, float* dbeta, int B, int T,
                             int H, int N, long long q_sb, long long q_st, long long q_sh, long long k_sb,
                             long long k_st, long long k_sh, long long v_sb, long long v_st, long long v_sh,
                             float scale, int l2norm, int gla, cudaStream_t st) {
  HMF_REQUIRE(q && k && v && g && dvnT && d_qt && d_kt && d_P && d_gl && dq && dk && dv && dg, "gdn_prep_bwd: null tensor");
  HMF_REQUIRE(gla || (beta && d_w), "gdn_prep_bwd: beta and d_w are required outside gla mode");
  HMF_REQUIRE(q_st % 4 == 0 && q_sh % 4 == 0 && k_st % 4 == 0 && k_sh % 4 == 0 && v_st % 4 == 0 && v_sh % 4 == 0,
              "gdn_prep_bwd: strides must be multiples of 4 elements");
  HMF_REQUIRE(N == (T + C - 1) / C && (long long)B * H <= 65535, "gdn_prep_bwd: bad chunk count or batch * heads");
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(gdn_prep_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  Params p;
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.v = (const bf16*)v; p.g = g; p.beta = beta;
  p.dvnT = (const bf16*)dvnT; p.d_w = (const bf16*)d_w; p.d_qt = (const bf16*)d_qt; p.d_kt = (const bf16*)d_kt;
  p.d_P = d_P; p.d_gl = d_gl;
  p.dq = (bf16*)dq; p.dk = (bf16*)dk; p.dv = (bf16*)dv; p.dg = dg; p.dbeta = dbeta;
  p.q_sb = q_sb; p.q_st = q_st; p.q_sh = q_sh; p.k_sb = k_sb; p.k_st = k_st; p.k_sh = k_sh;
  p.v_sb = v_sb; p.v_st = v_st; p.v_sh = v_sh;
  p.B = B; p.T = T; p.H = H; p.N = N; p.scale = scale; p.l2norm = l2norm; p.gla = gla;
  dim3 grid(N, B * H);
  gdn_prep_bwd_kernel<<<grid, NT, SMEM_BYTES, st>>>(p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
