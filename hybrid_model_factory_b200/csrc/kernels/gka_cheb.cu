// Gated KalmaNet: chunked Chebyshev ridge solve, forward.  One CTA per (chunk of 64 tokens, head).
//
// Token i of a chunk sees the decayed key covariance  H_i = e^{G_i} Hs + sum_{j<=i} e^{G_i - G_j} k_j k_j^T
// (Hs: state at the chunk start, G: inclusive cumulative log-decay inside the chunk) and solves
//   (H_i + lam_i I) x_i = q_i,   lam_i = ridge_ratio * |H_i|_F,
// by `num_iter` steps of the Chebyshev semi-iteration.  In chunk form one step is
//   Hx = (x o e^G) Hs + ((x k^T) o m) k,     m_ij = e^{G_i - G_j} [j <= i]
//   upd = step w (Hx + lam x - q) + (w - 1) x_prev ;  x_prev = x ;  x = w x - upd ;  w <- 1 / (1 - c w)
// with per-token scalars step = 2 / (2 lam + |H|_F), c = (|H|_F / (2 (2 lam + |H|_F)))^2.
// The whole solve of a chunk stays on chip: Hs, k and the iterate live in shared memory (bf16 operands, fp32
// accumulation on the tensor cores, as the reference's kernel does by casting x to the operand dtype); x, x_prev and q
// are fp32 registers; |H_i|_F comes from the closed form
//   |H_i|_F^2 = sum_{j,l<=i} m_ij m_il (k_j.k_l)^2 + e^{2 G_i} |Hs|_F^2 + 2 e^{G_i} sum_{j<=i} m_ij k_j^T Hs k_j .
// Replaces `num_iter` rounds of batched library GEMMs plus a dozen elementwise passes per round over
// [tokens, heads, 128] fp32 tensors.
#include <math.h>
#include <mma.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace gka_cheb {

using bf16 = __nv_bfloat16;
using namespace nvcuda;
constexpr int C = 64, D = 128, NT = 512, RPT = C * D / NT;   // 16 warps; RPT elements of the iterate per thread
constexpr int LB = D + 8;      // bf16 rows of D
constexpr int LY = D + 4;      // fp32 rows of D
constexpr int LS = C + 4;      // fp32 rows of C
constexpr int LP = C + 8;      // bf16 rows of C
constexpr int OFF_HS = 0;                               // bf16 [D][LB]
constexpr int OFF_K = OFF_HS + D * LB * 2;              // bf16 [C][LB]
constexpr int OFF_X = OFF_K + C * LB * 2;               // bf16 [C][LB]   iterate
constexpr int OFF_XE = OFF_X + C * LB * 2;              // bf16 [C][LB]   iterate scaled by e^G (rows)
constexpr int OFF_Y = OFF_XE + C * LB * 2;              // fp32 [C][LY]   Hx; its head doubles as S [C][LS]
constexpr int OFF_P = OFF_Y + C * LY * 4;               // bf16 [C][LP]   (x k^T) o m; before the loop: fp32 m [C][LS] spans P + M
constexpr int OFF_SMALL = OFF_P + C * LS * 4;
constexpr int SMEM_BYTES = OFF_SMALL + 10 * C * 4 + 128;
static_assert(C * LS * 4 >= C * LP * 2, "m scratch must cover P");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");

struct Params {
  const bf16 *q, *k;        // [B, T, H, D] views (element strides)
  const float* gk;          // [B, T, H] log-decay per token (null: no decay)
  const float* hs;          // [B, H, hs_chunks, D, D] chunk-start states, fp32 (hs_chunks >= N)
  float* x;                 // [B, T, H, D] fp32 contiguous
  long long q_sb, q_st, q_sh, k_sb, k_st, k_sh;
  int B, T, H, N, hs_chunks, num_iter;
  float ridge_ratio;
};

// S[C, C] = A[C, D] . B[C, D]^T : 16 tiles, one per warp; two accumulators over alternating k-steps halve the
// dependent MMA chain.
__device__ __forceinline__ void mm_abt(float* S, const bf16* A, const bf16* Bm) {
  const int warp = threadIdx.x >> 5;
  const int tm = warp >> 2, tn = warp & 3;
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> c0, c1;
  wmma::fill_fragment(c0, 0.f);
  wmma::fill_fragment(c1, 0.f);
  wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a0, a1;
  wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> b0, b1;
  for (int k0 = 0; k0 < D; k0 += 32) {
    wmma::load_matrix_sync(a0, A + tm * 16 * LB + k0, LB);
    wmma::load_matrix_sync(b0, Bm + tn * 16 * LB + k0, LB);
    wmma::load_matrix_sync(a1, A + tm * 16 * LB + k0 + 16, LB);
    wmma::load_matrix_sync(b1, Bm + tn * 16 * LB + k0 + 16, LB);
    wmma::mma_sync(c0, a0, b0, c0);
    wmma::mma_sync(c1, a1, b1, c1);
  }
#pragma unroll
  for (int e = 0; e < c0.num_elements; ++e) c0.x[e] += c1.x[e];
  wmma::store_matrix_sync(S + tm * 16 * LS + tn * 16, c0, LS, wmma::mem_row_major);
}

// Y[C, D] = XE[C, D] . Hs[D, D] (+ P[C, C] . K[C, D] when P is given).  Warp w owns the column block w % 8 of the row
// blocks w / 8 and w / 8 + 2: the B fragments are shared by its two tiles, whose MMA chains are independent.
__device__ __forceinline__ void mm_hx(float* Y, const bf16* XE, const bf16* Hs, const bf16* P, const bf16* K) {
  const int warp = threadIdx.x >> 5;
  const int tn = warp & 7, tm0 = warp >> 3, tm1 = tm0 + 2;
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> c0, c1;
  wmma::fill_fragment(c0, 0.f);
  wmma::fill_fragment(c1, 0.f);
  wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a0, a1;
  wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> b;
  for (int k0 = 0; k0 < D; k0 += 16) {
    wmma::load_matrix_sync(b, Hs + k0 * LB + tn * 16, LB);
    wmma::load_matrix_sync(a0, XE + tm0 * 16 * LB + k0, LB);
    wmma::load_matrix_sync(a1, XE + tm1 * 16 * LB + k0, LB);
    wmma::mma_sync(c0, a0, b, c0);
    wmma::mma_sync(c1, a1, b, c1);
  }
  if (P != nullptr) {
    for (int k0 = 0; k0 < C; k0 += 16) {
      wmma::load_matrix_sync(b, K + k0 * LB + tn * 16, LB);
      wmma::load_matrix_sync(a0, P + tm0 * 16 * LP + k0, LP);
      wmma::load_matrix_sync(a1, P + tm1 * 16 * LP + k0, LP);
      wmma::mma_sync(c0, a0, b, c0);
      wmma::mma_sync(c1, a1, b, c1);
    }
  }
  wmma::store_matrix_sync(Y + tm0 * 16 * LY + tn * 16, c0, LY, wmma::mem_row_major);
  wmma::store_matrix_sync(Y + tm1 * 16 * LY + tn * 16, c1, LY, wmma::mem_row_major);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

static_assert(NT == 512, "tile-to-warp maps assume 16 warps");

__global__ void __launch_bounds__(NT, 1) gka_cheb_fwd_kernel(const Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* s_hs = reinterpret_cast<bf16*>(smem + OFF_HS);
  bf16* s_k = reinterpret_cast<bf16*>(smem + OFF_K);
  bf16* s_x = reinterpret_cast<bf16*>(smem + OFF_X);
  bf16* s_xe = reinterpret_cast<bf16*>(smem + OFF_XE);
  float* s_y = reinterpret_cast<float*>(smem + OFF_Y);
  float* s_s = s_y;                                     // [C][LS], dead before Hx is written
  bf16* s_p = reinterpret_cast<bf16*>(smem + OFF_P);
  float* s_m = reinterpret_cast<float*>(smem + OFF_P);  // [C][LS], only before the iteration
  float* small = reinterpret_cast<float*>(smem + OFF_SMALL);
  float* s_G = small;                // [C]
  float* s_eg = small + C;
  float* s_lam = small + 2 * C;
  float* s_step = small + 3 * C;
  float* s_c = small + 4 * C;
  float* s_om = small + 5 * C;       // [2][C]
  float* s_khk = small + 7 * C;
  float* s_fro = small + 8 * C;
  float* s_red = small + 9 * C;      // [16] warp partials + result

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int t0 = n * C;

  // ---- loads: k -> bf16 smem, q -> registers (element e = tid + NT r <-> (i = e / 128, d = e % 128)) ----
  float q[RPT], x[RPT], xp[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int e = tid + NT * r, i = e >> 7, d = e & 127;
    const bool ok = t0 + i < p.T;
    const bf16 kv = ok ? p.k[(size_t)b * p.k_sb + (size_t)(t0 + i) * p.k_st + (size_t)h * p.k_sh + d] : __float2bfloat16(0.f);
    s_k[i * LB + d] = kv;
    q[r] = ok ? __bfloat162float(p.q[(size_t)b * p.q_sb + (size_t)(t0 + i) * p.q_st + (size_t)h * p.q_sh + d]) : 0.f;
  }
  // chunk-start state: fp32 -> bf16 operand, Frobenius norm on the way
  const float* hs = p.hs + (((size_t)b * p.H + h) * p.hs_chunks + n) * D * D;
  float hsq = 0.f;
  for (int e = tid; e < D * D / 4; e += NT) {
    const float4 v = reinterpret_cast<const float4*>(hs)[e];
    const int row = (e * 4) >> 7, col = (e * 4) & 127;
    hsq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    uint2 u;
    u.x = pack_bf16x2(v.x, v.y);
    u.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(s_hs + row * LB + col) = u;
  }
  hsq = warp_sum(hsq);
  if (lane == 0) s_red[warp] = hsq;
  // inclusive cumulative log-decay of the chunk (one warp, two tokens per lane)
  if (warp == 0) {
    float g0 = 0.f, g1 = 0.f;
    if (p.gk != nullptr) {
      if (t0 + lane < p.T) g0 = p.gk[((size_t)b * p.T + t0 + lane) * p.H + h];
      if (t0 + 32 + lane < p.T) g1 = p.gk[((size_t)b * p.T + t0 + 32 + lane) * p.H + h];
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float a0 = __shfl_up_sync(0xffffffffu, g0, o), a1 = __shfl_up_sync(0xffffffffu, g1, o);
      if (lane >= o) { g0 += a0; g1 += a1; }
    }
    g1 += __shfl_sync(0xffffffffu, g0, 31);
    s_G[lane] = g0;
    s_G[32 + lane] = g1;
    s_eg[lane] = __expf(g0);
    s_eg[32 + lane] = __expf(g1);
  }
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int w = 0; w < NT / 32; ++w) t += s_red[w];
    s_red[16] = t;
  }
  // decay mask m_ij (fp32 scratch) and the Gram matrix k k^T
  for (int e = tid; e < C * C; e += NT) {
    const int i = e >> 6, j = e & 63;
    s_m[i * LS + j] = j <= i ? __expf(s_G[i] - s_G[j]) : 0.f;
  }
  mm_abt(s_s, s_k, s_k);
  __syncthreads();
  // part 1 of |H_i|_F^2: sum_{j,l<=i} m_ij m_il gram_jl^2  (8 threads per token, j strided over them)
  {
    const int i = tid >> 3, part = tid & 7;
    float acc = 0.f;
    for (int j = part; j <= i; j += 8) {
      float inner = 0.f;
      for (int l = 0; l <= i; ++l) {
        const float g = s_s[j * LS + l];
        inner += s_m[i * LS + l] * g * g;
      }
      acc += s_m[i * LS + j] * inner;
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (part == 0) s_fro[i] = acc;
  }
  __syncthreads();
  // k Hs -> y ; kHk_j = (k Hs)_j . k_j
  mm_hx(s_y, s_k, s_hs, nullptr, nullptr);
  __syncthreads();
  for (int j = warp; j < C; j += NT / 32) {
    float acc = 0.f;
    for (int d = lane; d < D; d += 32) acc += s_y[j * LY + d] * __bfloat162float(s_k[j * LB + d]);
    acc = warp_sum(acc);
    if (lane == 0) s_khk[j] = acc;
  }
  __syncthreads();
  if (tid < C) {
    const int i = tid;
    float cross = 0.f;
    for (int j = 0; j <= i; ++j) cross += s_m[i * LS + j] * s_khk[j];
    const float eg = s_eg[i];
    const float fro2 = s_fro[i] + eg * eg * s_red[16] + 2.f * eg * cross;
    const float fro = sqrtf(fmaxf(fro2, 0.f));
    const float lam = p.ridge_ratio * fro;
    float denom = 2.f * lam + fro;
    if (denom == 0.f) denom = 1.f;
    s_lam[i] = lam;
    s_step[i] = 2.f / denom;
    const float cc = fro / denom * 0.5f;
    s_c[i] = cc * cc;
    s_om[i] = 2.f;
  }
  __syncthreads();
  // ---- x0 = step q ----
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int e = tid + NT * r, i = e >> 7, d = e & 127;
    xp[r] = 0.f;
    x[r] = s_step[i] * q[r];
    s_x[i * LB + d] = __float2bfloat16(x[r]);
    s_xe[i * LB + d] = __float2bfloat16(x[r] * s_eg[i]);
  }
  __syncthreads();
  for (int it = 0; it < p.num_iter; ++it) {
    const float* om_old = s_om + (it & 1) * C;
    float* om_new = s_om + ((it + 1) & 1) * C;
    // S = x k^T
    mm_abt(s_s, s_x, s_k);
    __syncthreads();
    // P = S o m (bf16 operand)
    for (int e = tid; e < C * C; e += NT) {
      const int i = e >> 6, j = e & 63;
      const float mv = j <= i ? __expf(s_G[i] - s_G[j]) : 0.f;
      s_p[i * LP + j] = __float2bfloat16(s_s[i * LS + j] * mv);
    }
    __syncthreads();
    mm_hx(s_y, s_xe, s_hs, s_p, s_k);
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int e = tid + NT * r, i = e >> 7, d = e & 127;
      const float om = 1.f / (1.f - s_c[i] * om_old[i]);
      const float upd = s_step[i] * om * (s_y[i * LY + d] + s_lam[i] * x[r] - q[r]) + (om - 1.f) * xp[r];
      xp[r] = x[r];
      x[r] = om * x[r] - upd;
      s_x[i * LB + d] = __float2bfloat16(x[r]);
      s_xe[i * LB + d] = __float2bfloat16(x[r] * s_eg[i]);
      if (d == 0) om_new[i] = om;
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int e = tid + NT * r, i = e >> 7, d = e & 127;
    if (t0 + i < p.T) p.x[(((size_t)b * p.T + t0 + i) * p.H + h) * D + d] = x[r];
  }
}

}  // namespace gka_cheb
}  // namespace hmf

using namespace hmf;
using namespace hmf::gka_cheb;

// q, k: [B, T, H, 128] bf16 views (element strides batch / token / head, unit inner stride); gk [B, T, H] fp32
// contiguous or null; hs [B, H, hs_chunks, 128, 128] fp32 contiguous, chunk n < N = ceil(T / 64) is read;
// x [B, T, H, 128] fp32 contiguous.
HMF_API int hmf_gka_cheb_fwd(const void* q, const void* k, const float* gk, const float* hs, float* x, int B, int T, int H,
                             int N, int hs_chunks, long long q_sb, long long q_st, long long q_sh, long long k_sb, long long k_st,
                             long long k_sh, float ridge_ratio, int num_iter, cudaStream_t st) {
  HMF_REQUIRE(q && k && hs && x, "gka_cheb_fwd: null tensor");
  HMF_REQUIRE(N == (T + C - 1) / C && (long long)B * H <= 65535 && num_iter >= 0 && hs_chunks >= N, "gka_cheb_fwd: bad sizes");
  HMF_REQUIRE((reinterpret_cast<uintptr_t>(hs) & 15) == 0, "gka_cheb_fwd: states must be 16-byte aligned");
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(gka_cheb_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  Params p;
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.gk = gk; p.hs = hs; p.x = x;
  p.q_sb = q_sb; p.q_st = q_st; p.q_sh = q_sh; p.k_sb = k_sb; p.k_st = k_st; p.k_sh = k_sh;
  p.B = B; p.T = T; p.H = H; p.N = N; p.hs_chunks = hs_chunks; p.num_iter = num_iter; p.ridge_ratio = ridge_ratio;
  dim3 grid(N, B * H);
  gka_cheb_fwd_kernel<<<grid, NT, SMEM_BYTES, st>>>(p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
