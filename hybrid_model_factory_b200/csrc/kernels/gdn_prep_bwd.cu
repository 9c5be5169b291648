// Backward of the Gated DeltaNet chunk preparation, one CTA per (chunk of 64 tokens, head).
//
// Forward (per chunk): qn = scale q/|q|, kn = k/|k|, G = cumsum(g), D_ij = e^{G_i - G_j} (i >= j),
//   A = strict_lower(beta_i (kn_i.kn_j) D_ij), Tm = (I + A)^-1, u = Tm (beta v), w = Tm (beta e^G kn),
//   P = (qn kn^T) o D, qt = qn e^G, kt = kn e^{G_last - G}, glast = G_last.
// Given d_u, d_w, d_qt, d_kt, d_P, d_glast this kernel produces dq, dk, dv, dg, dbeta.  It replaces about fifty
// memory-bound PyTorch passes over [tokens, heads, 128] fp32 tensors by one kernel that keeps the chunk in shared
// memory; the twelve small products (64x64x128, 64x128x64, 64^3) run as warp-level bf16 tensor-core MMAs with fp32
// accumulation (operands are the same bf16 tiles the forward kernels use), row reductions by warps, the 64x64
// triangular inverse by forward substitution (one column per thread).
// `gla` mode (plain gated linear attention: w = 0, u = v) skips everything that involves A.
#include <math.h>
#include <mma.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace gdn_prep_bwd {

using bf16 = __nv_bfloat16;
using namespace nvcuda;
constexpr int C = 64, D = 128, NT = 256;
constexpr int LD = D + 4;      // fp32 [C, D] tiles (row stride a multiple of 16 bytes)
constexpr int LB = D + 8;      // bf16 [C, D] operand tiles (row stride a multiple of 16 bytes)
constexpr int LCF = C + 4;     // fp32 [C, C] tiles
constexpr int LCB = C + 8;     // bf16 [C, C] operand tiles
constexpr int SZ_B = C * LB * 2, SZ_F = C * LD * 4, SZ_CF = C * LCF * 4, SZ_CB = C * LCB * 2;
constexpr int OFF_QN = 0, OFF_KN = SZ_B, OFF_V = 2 * SZ_B, OFF_DU = 3 * SZ_B, OFF_DW = 4 * SZ_B;
constexpr int OFF_T1 = 5 * SZ_B;               // fp32 [C, D] product tile (its head doubles as a [C, C] scratch)
constexpr int OFF_DKN = OFF_T1 + SZ_F;
constexpr int OFF_S = OFF_DKN + SZ_F;          // fp32 [C, C] scratch
constexpr int OFF_KD = OFF_S + SZ_CF;          // fp32 [C, C]  strict_lower((kn kn^T) o D)
constexpr int OFF_M1 = OFF_KD + SZ_CF;         // bf16 [C, C]  Tm
constexpr int OFF_M2 = OFF_M1 + SZ_CB;         // bf16 [C, C]  dT / X1 / Mm / Nm
constexpr int OFF_SMALL = OFF_M2 + SZ_CB;
constexpr int SMEM_BYTES = OFF_SMALL + 12 * C * 4;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");

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

// Cs[M, N] (fp32, row-major, ldc) (+)= A . B on the tensor cores (warp-level bf16 MMA, fp32 accumulate).
// TA: A is stored [K][M]; TB: B is stored [N][K].  The 16x16 output tiles are dealt round-robin to the 8 warps.
template <int M, int N, bool TA, bool TB, bool ACC>
__device__ __forceinline__ void mmw(float* Cs, int ldc, const bf16* A, int lda, const bf16* Bm, int ldb, int K) {
  const int warp = threadIdx.x >> 5;
  constexpr int TN = N / 16, TILES = (M / 16) * TN;
  for (int t = warp; t < TILES; t += NT / 32) {
    const int tm = t / TN, tn = t % TN;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> c;
    float* cp = Cs + tm * 16 * ldc + tn * 16;
    if (ACC) wmma::load_matrix_sync(c, cp, ldc, wmma::mem_row_major);
    else wmma::fill_fragment(c, 0.f);
    for (int k0 = 0; k0 < K; k0 += 16) {
      if constexpr (TA) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::col_major> a;
        wmma::load_matrix_sync(a, A + k0 * lda + tm * 16, lda);
        if constexpr (TB) {
          wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> b;
          wmma::load_matrix_sync(b, Bm + tn * 16 * ldb + k0, ldb);
          wmma::mma_sync(c, a, b, c);
        } else {
          wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> b;
          wmma::load_matrix_sync(b, Bm + k0 * ldb + tn * 16, ldb);
          wmma::mma_sync(c, a, b, c);
        }
      } else {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
        wmma::load_matrix_sync(a, A + tm * 16 * lda + k0, lda);
        if constexpr (TB) {
          wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> b;
          wmma::load_matrix_sync(b, Bm + tn * 16 * ldb + k0, ldb);
          wmma::mma_sync(c, a, b, c);
        } else {
          wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> b;
          wmma::load_matrix_sync(b, Bm + k0 * ldb + tn * 16, ldb);
          wmma::mma_sync(c, a, b, c);
        }
      }
    }
    wmma::store_matrix_sync(cp, c, ldc, wmma::mem_row_major);
  }
}

__device__ __forceinline__ void load4(const bf16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
  uint2 u;
  u.x = pack_bf16x2(v[0], v[1]);
  u.y = pack_bf16x2(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = u;
}

__global__ void __launch_bounds__(NT, 1) gdn_prep_bwd_kernel(const Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* b_qn = reinterpret_cast<bf16*>(smem + OFF_QN);
  bf16* b_kn = reinterpret_cast<bf16*>(smem + OFF_KN);
  bf16* b_v = reinterpret_cast<bf16*>(smem + OFF_V);
  bf16* b_du = reinterpret_cast<bf16*>(smem + OFF_DU);
  bf16* b_dw = reinterpret_cast<bf16*>(smem + OFF_DW);
  float* f_T1 = reinterpret_cast<float*>(smem + OFF_T1);
  float* f_S2 = f_T1;                                             // [C, C] scratch inside the T1 region
  float* f_dkn = reinterpret_cast<float*>(smem + OFF_DKN);
  float* f_S = reinterpret_cast<float*>(smem + OFF_S);
  float* f_KD = reinterpret_cast<float*>(smem + OFF_KD);
  bf16* b_M1 = reinterpret_cast<bf16*>(smem + OFF_M1);
  bf16* b_M2 = reinterpret_cast<bf16*>(smem + OFF_M2);
  float* sm = reinterpret_cast<float*>(smem + OFF_SMALL);
  float *s_G = sm, *s_eG = sm + C, *s_eR = sm + 2 * C, *s_beta = sm + 3 * C, *s_rq = sm + 4 * C, *s_rk = sm + 5 * C,
        *s_dG = sm + 6 * C, *s_dbeta = sm + 7 * C, *s_t = sm + 8 * C, *s_colsum = sm + 9 * C;

  const int n = blockIdx.x, bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = n * C;
  const size_t chunk = (size_t)bh * p.N + n;
  const int d4 = lane * 4;

  // ---- gates ----
  if (tid < C) {
    const int t = t0 + tid;
    s_G[tid] = t < p.T ? p.g[((size_t)b * p.T + t) * p.H + h] : 0.f;
    s_beta[tid] = p.gla ? 1.f : (t < p.T ? p.beta[((size_t)b * p.T + t) * p.H + h] : 0.f);
    s_dG[tid] = 0.f;
    s_dbeta[tid] = 0.f;
    s_t[tid] = 0.f;
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
  // ---- operand tiles (bf16): normalised q, k; v; d_u; d_w.  Warp w handles rows w, w + 8, ... ----
  for (int i = warp; i < C; i += 8) {
    const int t = t0 + i;
    float qv[4] = {0.f, 0.f, 0.f, 0.f}, kv[4] = {0.f, 0.f, 0.f, 0.f}, vv[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
    if (t < p.T) {
      load4(p.q + (size_t)b * p.q_sb + (size_t)t * p.q_st + (size_t)h * p.q_sh + d4, qv);
      load4(p.k + (size_t)b * p.k_sb + (size_t)t * p.k_st + (size_t)h * p.k_sh + d4, kv);
      load4(p.v + (size_t)b * p.v_sb + (size_t)t * p.v_st + (size_t)h * p.v_sh + d4, vv);
    }
    if (!p.gla) load4(p.d_w + (chunk * C + i) * D + d4, wv);
    float rq = 1.f, rk = 1.f;
    if (p.l2norm) {
      rq = rsqrtf(warp_sum(qv[0] * qv[0] + qv[1] * qv[1] + qv[2] * qv[2] + qv[3] * qv[3]) + 1e-6f);
      rk = rsqrtf(warp_sum(kv[0] * kv[0] + kv[1] * kv[1] + kv[2] * kv[2] + kv[3] * kv[3]) + 1e-6f);
    }
    if (lane == 0) { s_rq[i] = rq; s_rk[i] = rk; }
#pragma unroll
    for (int e = 0; e < 4; ++e) { qv[e] *= rq * p.scale; kv[e] *= rk; }
    store4(b_qn + i * LB + d4, qv);
    store4(b_kn + i * LB + d4, kv);
    store4(b_v + i * LB + d4, vv);
    store4(b_dw + i * LB + d4, wv);
  }
  // d_u arrives transposed ([D, C]): element (i, d) = dvnT[d * C + i]
  for (int e = tid; e < C * D; e += NT) {
    const int d = e / C, i = e % C;
    b_du[i * LB + d] = p.dvnT[chunk * (size_t)(D * C) + e];
  }
  __syncthreads();

  const bf16* g_dqt = p.d_qt + chunk * (size_t)(C * D);
  const bf16* g_dkt = p.d_kt + chunk * (size_t)(C * D);
  const float* g_dP = p.d_P + chunk * (size_t)(C * C);
  auto out_row = [&](int i) -> size_t { return (((size_t)b * p.T + t0 + i) * p.H + h) * D; };

  if (!p.gla) {
    // ---- KD = strict_lower((kn kn^T) o D) ----
    mmw<C, C, false, true, false>(f_S, LCF, b_kn, LB, b_kn, LB, D);
    __syncthreads();
    for (int e = tid; e < C * C; e += NT) {
      const int i = e / C, j = e % C;
      f_KD[i * LCF + j] = i > j ? f_S[i * LCF + j] * __expf(s_G[i] - s_G[j]) : 0.f;
    }
    __syncthreads();
    // ---- Tm = (I + beta KD)^-1 by forward substitution, thread c owns column c ----
    if (tid < C) {
      float x[C];
#pragma unroll
      for (int i = 0; i < C; ++i) {
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < C; ++j)
          if (j < i) dot = fmaf(f_KD[i * LCF + j], x[j], dot);
        x[i] = ((i == tid) ? 1.f : 0.f) - s_beta[i] * dot;
        b_M1[i * LCB + tid] = __float2bfloat16(x[i]);
      }
    }
    // ---- dT = d_u (beta v)^T + d_w (beta e^G kn)^T ----
    mmw<C, C, false, true, false>(f_S, LCF, b_du, LB, b_v, LB, D);
    mmw<C, C, false, true, false>(f_S2, LCF, b_dw, LB, b_kn, LB, D);
    __syncthreads();
    for (int e = tid; e < C * C; e += NT) {
      const int i = e / C, j = e % C;
      b_M2[i * LCB + j] = __float2bfloat16(s_beta[j] * (f_S[i * LCF + j] + s_eG[j] * f_S2[i * LCF + j]));
    }
    __syncthreads();
    // ---- dbv = Tm^T d_u: dv = beta dbv, dbeta += dbv . v ----
    mmw<C, D, true, false, false>(f_T1, LD, b_M1, LCB, b_du, LB, C);
    __syncthreads();
    for (int j = warp; j < C; j += 8) {
      float a[4], vv[4], o[4];
      load4(b_v + j * LB + d4, vv);
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        a[e] = f_T1[j * LD + d4 + e];
        o[e] = a[e] * s_beta[j];
        dot += a[e] * vv[e];
      }
      dot = warp_sum(dot);
      if (t0 + j < p.T) store4(p.dv + out_row(j) + d4, o);
      if (lane == 0) s_dbeta[j] += dot;
    }
    __syncthreads();
    // ---- dbk = Tm^T d_w: dkn = beta e^G dbk, x = e^G dbk . kn -> dbeta, dG ----
    mmw<C, D, true, false, false>(f_T1, LD, b_M1, LCB, b_dw, LB, C);
    __syncthreads();
    for (int j = warp; j < C; j += 8) {
      float kk[4];
      load4(b_kn + j * LB + d4, kk);
      float dot = 0.f;
      const float sc = s_beta[j] * s_eG[j];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a = f_T1[j * LD + d4 + e];
        f_dkn[j * LD + d4 + e] = a * sc;
        dot += a * kk[e];
      }
      dot = warp_sum(dot) * s_eG[j];
      if (lane == 0) { s_dbeta[j] += dot; s_dG[j] += dot * s_beta[j]; }
    }
    // ---- X1 = Tm^T dT ; dA = -strict_lower(X1 Tm^T) ----
    mmw<C, C, true, false, false>(f_S, LCF, b_M1, LCB, b_M2, LCB, C);
    __syncthreads();
    for (int e = tid; e < C * C; e += NT) b_M2[(e / C) * LCB + (e % C)] = __float2bfloat16(f_S[(e / C) * LCF + (e % C)]);
    __syncthreads();
    mmw<C, C, false, true, false>(f_S, LCF, b_M2, LCB, b_M1, LCB, C);
    __syncthreads();
    // f_S <- sA = dA o A (for the gate sums), f_S2 <- dA o KD (for dbeta), b_M2 <- Mm = dA o D o beta_i
    for (int e = tid; e < C * C; e += NT) {
      const int i = e / C, j = e % C;
      float sA = 0.f, dk_ = 0.f, m = 0.f;
      if (i > j) {
        const float dA = -f_S[i * LCF + j], kd = f_KD[i * LCF + j];
        dk_ = dA * kd;
        sA = dk_ * s_beta[i];
        m = dA * __expf(s_G[i] - s_G[j]) * s_beta[i];
      }
      f_S[i * LCF + j] = sA;
      f_S2[i * LCF + j] = dk_;
      b_M2[i * LCB + j] = __float2bfloat16(m);
    }
    __syncthreads();
    if (tid < C) {                      // row sums
      float rs = 0.f, rb = 0.f;
      for (int j = 0; j < C; ++j) { rs += f_S[tid * LCF + j]; rb += f_S2[tid * LCF + j]; }
      s_dG[tid] += rs;
      s_dbeta[tid] += rb;
    } else if (tid < 2 * C) {           // column sums
      const int j = tid - C;
      float cs = 0.f;
      for (int i = 0; i < C; ++i) cs += f_S[i * LCF + j];
      s_colsum[j] = cs;
    }
    __syncthreads();
    if (tid < C) s_dG[tid] -= s_colsum[tid];
    // ---- dkn += Mm kn + Mm^T kn ----
    mmw<C, D, false, false, true>(f_dkn, LD, b_M2, LCB, b_kn, LB, C);
    __syncthreads();
    mmw<C, D, true, false, true>(f_dkn, LD, b_M2, LCB, b_kn, LB, C);
    __syncthreads();
  } else {
    // plain gated linear attention: u = v, so dv = d_u; dkn starts at zero
    for (int i = warp; i < C; i += 8) {
      float a[4];
      load4(b_du + i * LB + d4, a);
      if (t0 + i < p.T) store4(p.dv + out_row(i) + d4, a);
#pragma unroll
      for (int e = 0; e < 4; ++e) f_dkn[i * LD + d4 + e] = 0.f;
    }
    __syncthreads();
  }

  // ---- intra-chunk scores: Nm = d_P o D (lower, diagonal included); s_P = Nm o (qn kn^T) feeds dG ----
  mmw<C, C, false, true, false>(f_S, LCF, b_qn, LB, b_kn, LB, D);
  for (int e = tid; e < C * C; e += NT) {
    const int i = e / C, j = e % C;
    const float nm = i >= j ? g_dP[e] * __expf(s_G[i] - s_G[j]) : 0.f;
    b_M2[i * LCB + j] = __float2bfloat16(nm);
    f_KD[i * LCF + j] = nm;                       // KD is dead: reuse as the fp32 copy of Nm
  }
  __syncthreads();
  if (tid < C) {
    float rs = 0.f;
    for (int j = 0; j <= tid; ++j) rs += f_KD[tid * LCF + j] * f_S[tid * LCF + j];
    s_dG[tid] += rs;
  } else if (tid < 2 * C) {
    const int j = tid - C;
    float cs = 0.f;
    for (int i = j; i < C; ++i) cs += f_KD[i * LCF + j] * f_S[i * LCF + j];
    s_colsum[j] = cs;
  }
  __syncthreads();
  if (tid < C) s_dG[tid] -= s_colsum[tid];
  // ---- dqn = Nm kn + e^G d_qt, then straight through the L2 normalisation of q ----
  mmw<C, D, false, false, false>(f_T1, LD, b_M2, LCB, b_kn, LB, C);
  __syncthreads();
  for (int i = warp; i < C; i += 8) {
    float qn[4], dqt[4], dq[4], o[4];
    load4(b_qn + i * LB + d4, qn);
    load4(g_dqt + i * D + d4, dqt);
    float dot_g = 0.f, dot_n = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      dq[e] = f_T1[i * LD + d4 + e] + dqt[e] * s_eG[i];
      dot_g += dqt[e] * qn[e];
      dot_n += dq[e] * qn[e];
    }
    dot_g = warp_sum(dot_g);
    if (lane == 0) s_dG[i] += dot_g * s_eG[i];
    if (p.l2norm) {
      dot_n = warp_sum(dot_n) / (p.scale * p.scale);
      const float aq = s_rq[i] * p.scale;
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = (dq[e] - qn[e] * dot_n) * aq;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = dq[e] * p.scale;
    }
    if (t0 + i < p.T) store4(p.dq + out_row(i) + d4, o);
  }
  // ---- dkn += Nm^T qn + e^{G_last - G} d_kt, then through the L2 normalisation of k ----
  mmw<C, D, true, false, true>(f_dkn, LD, b_M2, LCB, b_qn, LB, C);
  __syncthreads();
  for (int i = warp; i < C; i += 8) {
    float kn[4], dkt[4], dk[4], o[4];
    load4(b_kn + i * LB + d4, kn);
    load4(g_dkt + i * D + d4, dkt);
    float dot_t = 0.f, dot_n = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      dk[e] = f_dkn[i * LD + d4 + e] + dkt[e] * s_eR[i];
      dot_t += dkt[e] * kn[e];
      dot_n += dk[e] * kn[e];
    }
    dot_t = warp_sum(dot_t) * s_eR[i];
    if (lane == 0) { s_dG[i] -= dot_t; s_t[i] = dot_t; }
    if (p.l2norm) {
      dot_n = warp_sum(dot_n);
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = (dk[e] - kn[e] * dot_n) * s_rk[i];
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = dk[e];
    }
    if (t0 + i < p.T) store4(p.dk + out_row(i) + d4, o);
  }
  __syncthreads();
  // ---- dg = reverse cumulative sum of dG (with the G_last terms); dbeta ----
  if (tid == 0) {
    float tl = p.d_gl[chunk];
    for (int i = 0; i < C; ++i) tl += s_t[i];
    s_dG[C - 1] += tl;
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
