// Gated KalmaNet: chunked Chebyshev ridge solve, forward, on tcgen05 (same math as gka_cheb.cu; that file explains it).
//
// Everything is kept feature-major so that the 128 features are the MMA M dimension and the 64 tokens of the chunk the
// N dimension; thread t of a warp quadrant owns feature row d and keeps its slice of the iterate in registers:
//   S^T[j, i]  = sum_d k[j, d] x[i, d]          A = k  (K-major, rows padded to 128 with zeros), B = x (K-major)
//   T1[d, i]   = sum_d' Hs[d, d'] x[i, d']      A = Hs (K-major),                                  B = x
//   T2[d, i]   = sum_j k[j, d] P[j, i]          A = k  (the same tile read MN-major),              B = P (MN-major)
//   (Hx)^T     = e^{G_i} T1 + T2,   P[j, i] = S^T[j, i] e^{G_i - G_j} [j <= i]
// The operands sit in shared memory in the 128-byte-swizzled layouts the tensor core reads directly (written by the
// threads, no fragment loads), the three accumulators in 192 columns of tensor memory.  One iteration is two round
// trips  MMA -> commit -> mbarrier -> tcgen05.ld;  108 KB of shared memory and 256 TMEM columns per CTA let two chunks
// share an SM, so one chunk's MMAs overlap the other's register math.
#include <math.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace gka_cheb_tc {

using bf16 = __nv_bfloat16;
constexpr int C = 64, D = 128, NT = 256;
constexpr int HS_BLK = D * 128;          // bytes of one K block (64 features) of the Hs tile: 128 rows x 128 B
constexpr int K_BLK = 128 * 128;         // k tile: 128 rows (64 real, 64 zero) x 128 B per block of 64 features
constexpr int X_BLK = C * 128;           // x tile: 64 rows x 128 B per block of 64 features
constexpr int OFF_HS = 0;                           // 32 KB
constexpr int OFF_K = OFF_HS + 2 * HS_BLK;          // 32 KB
constexpr int OFF_X = OFF_K + 2 * K_BLK;            // 16 KB
constexpr int OFF_P = OFF_X + 2 * X_BLK;            //  8 KB  [j][i] bf16, one 128-byte row per j
constexpr int OFF_Q = OFF_P + C * 128;              // 16 KB  q as bf16 [i][d] (plain)
constexpr int OFF_SMALL = OFF_Q + C * D * 2;
constexpr int GR_LD = C + 1;                        // fp32 Gram scratch [64][65] lives in X + P before the loop
constexpr int SMEM_BYTES = OFF_SMALL + 15 * C * 4 + 128;
static_assert(C * GR_LD * 4 <= 2 * X_BLK + C * 128, "Gram scratch must fit into the x and P tiles");
static_assert(SMEM_BYTES <= 113 * 1024, "two CTAs per SM");

struct Params {
  const bf16 *q, *k;
  const float* gk;
  const float* hs;
  float* x;
  long long q_sb, q_st, q_sh, k_sb, k_st, k_sh;
  int B, T, H, N, hs_chunks, num_iter;
  float ridge_ratio;
  unsigned int* status;
};

// element (row, col) of a K-major tile made of blocks of 64 columns: byte address inside the tile
__device__ __forceinline__ uint32_t kmajor_off(int row, int col, int blk_bytes) {
  return (uint32_t)(col >> 6) * blk_bytes + sw128_offset((uint32_t)row, (uint32_t)(col & 63) * 2u);
}

__global__ void __launch_bounds__(NT, 2) gka_cheb_tc_kernel(const Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sHs = smem + OFF_HS;
  uint8_t* sK = smem + OFF_K;
  uint8_t* sX = smem + OFF_X;
  uint8_t* sP = smem + OFF_P;
  bf16* sQ = reinterpret_cast<bf16*>(smem + OFF_Q);
  float* sGr = reinterpret_cast<float*>(smem + OFF_X);      // before the loop only
  float* small = reinterpret_cast<float*>(smem + OFF_SMALL);
  float* s_G = small;
  float* s_eg = small + C;
  float* s_lam = small + 2 * C;
  float* s_step = small + 3 * C;
  float* s_c = small + 4 * C;
  float* s_om = small + 5 * C;       // Chebyshev weight of the previous step
  float* s_coef = small + 6 * C;     // [2][3][C]
  float* s_khk = small + 12 * C;
  float* s_fro = small + 13 * C;
  float* s_red = small + 14 * C;     // [8] warp partials, [8] total
  uint64_t* bar = reinterpret_cast<uint64_t*>(small + 15 * C);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quad = warp & 3, g = warp >> 2;          // TMEM lane quadrant, token half
  const int d = quad * 32 + lane;                    // feature row owned by this thread
  const int i0 = g * 32;                             // first token column owned by this thread
  const int n = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int t0 = n * C;
  const WaitCtx ctx{abort_flag, p.status};

  if (tid == 0) {
    if ((smem_u32(smem) & 1023u) != 0) report_error(p.status, kBadArgument, 0xC1);
    mbar_init(bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  // ---- operand tiles: k (rows 64..127 zero), q, Hs ----
  for (int e = tid; e < C * D; e += NT) {
    const int i = e >> 7, dd = e & 127;
    const bool ok = t0 + i < p.T;
    const bf16 zero = __float2bfloat16(0.f);
    const bf16 kv = ok ? p.k[(size_t)b * p.k_sb + (size_t)(t0 + i) * p.k_st + (size_t)h * p.k_sh + dd] : zero;
    *reinterpret_cast<bf16*>(sK + kmajor_off(i, dd, K_BLK)) = kv;
    *reinterpret_cast<bf16*>(sK + kmajor_off(i + C, dd, K_BLK)) = zero;
    sQ[i * D + dd] = ok ? p.q[(size_t)b * p.q_sb + (size_t)(t0 + i) * p.q_st + (size_t)h * p.q_sh + dd] : zero;
  }
  const float* hs = p.hs + (((size_t)b * p.H + h) * p.hs_chunks + n) * D * D;
  float hsq = 0.f;
  for (int e = tid; e < D * D / 8; e += NT) {            // 8 consecutive columns = one 16-byte chunk of a row
    const int row = e >> 4, col = (e & 15) * 8;
    const float4 v0 = reinterpret_cast<const float4*>(hs)[e * 2], v1 = reinterpret_cast<const float4*>(hs)[e * 2 + 1];
    hsq += v0.x * v0.x + v0.y * v0.y + v0.z * v0.z + v0.w * v0.w + v1.x * v1.x + v1.y * v1.y + v1.z * v1.z + v1.w * v1.w;
    uint4 u;
    u.x = pack_bf16x2(v0.x, v0.y);
    u.y = pack_bf16x2(v0.z, v0.w);
    u.z = pack_bf16x2(v1.x, v1.y);
    u.w = pack_bf16x2(v1.z, v1.w);
    *reinterpret_cast<uint4*>(sHs + kmajor_off(row, col, HS_BLK)) = u;
  }
  hsq = warp_sum(hsq);
  if (lane == 0) s_red[warp] = hsq;
  if (warp == 1) {       // inclusive cumulative log-decay of the chunk (two tokens per lane)
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
  if (tid < C) s_khk[tid] = 0.f;
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tT1 = tmem_base + 64, tT2 = tmem_base + 128;
  const uint32_t lane_bits = (uint32_t)(quad * 32) << 16;
  const uint32_t aHs = smem_u32(sHs), aK = smem_u32(sK), aX = smem_u32(sX), aP = smem_u32(sP);
  constexpr uint32_t idescKK = make_idesc_bf16(128, C, false, false);
  constexpr uint32_t idescMN = make_idesc_bf16(128, C, true, true);
  uint32_t phase = 0;

  // S^T-type and T1-type products against a K-major B tile at address aB with blocks of `b_blk` bytes
  auto issue_pair = [&](uint32_t aB, uint32_t b_blk) {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint64_t bd = make_desc_kmajor_sw128(aB + (kk >> 2) * b_blk + (kk & 3) * 32);
      umma_ss(tS, make_desc_kmajor_sw128(aK + (kk >> 2) * K_BLK + (kk & 3) * 32), bd, idescKK, kk > 0 ? 1u : 0u);
      umma_ss(tT1, make_desc_kmajor_sw128(aHs + (kk >> 2) * HS_BLK + (kk & 3) * 32), bd, idescKK, kk > 0 ? 1u : 0u);
    }
    umma_commit(bar);
  };

  // ---- Frobenius norms: Gram matrix k k^T and k Hs by the same two products with B = k ----
  if (tid == 0) {
    float t = 0.f;
    for (int w = 0; w < NT / 32; ++w) t += s_red[w];
    s_red[8] = t;
    issue_pair(aK, K_BLK);
  }
  bool ok = mbar_wait(bar, phase, ctx, 0xC10);
  phase ^= 1u;
  tc_fence_after();
  {
    uint32_t r[32];
    if (ok && d < C) {       // Gram row j = d, columns i0 .. i0 + 31
      tmem_ld_x32(tS + lane_bits + i0, r);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 32; ++c) sGr[d * GR_LD + i0 + c] = __uint_as_float(r[c]);
    }
    if (ok) {                // (k Hs)^T[d, j]: kHk_j = sum_d (k Hs)[j, d] k[j, d]
      tmem_ld_x32(tT1 + lane_bits + i0, r);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int j = i0 + c;
        const float kv = __bfloat162float(*reinterpret_cast<const bf16*>(sK + kmajor_off(j, d, K_BLK)));
        const float s = warp_sum(__uint_as_float(r[c]) * kv);
        if (lane == 0) atomicAdd(&s_khk[j], s);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  {   // part 1 of |H_i|_F^2 (4 threads per token), then the per-token scalars
    const int i = tid >> 2, part = tid & 3;
    float acc = 0.f;
    for (int j = part; j <= i; j += 4) {
      float inner = 0.f;
      const float mij = __expf(s_G[i] - s_G[j]);
      for (int l = 0; l <= i; ++l) {
        const float gv = sGr[j * GR_LD + l];
        inner += __expf(s_G[i] - s_G[l]) * gv * gv;
      }
      acc += mij * inner;
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if (part == 0) s_fro[i] = acc;
  }
  __syncthreads();
  if (tid < C) {
    const int i = tid;
    float cross = 0.f;
    for (int j = 0; j <= i; ++j) cross += __expf(s_G[i] - s_G[j]) * s_khk[j];
    const float eg = s_eg[i];
    const float fro2 = s_fro[i] + eg * eg * s_red[8] + 2.f * eg * cross;
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

  // ---- iterate: x^T[d, i0 .. i0 + 31] in registers ----
  float x[32], xp[32];
#pragma unroll
  for (int c = 0; c < 32; ++c) {
    const int i = i0 + c;
    xp[c] = 0.f;
    x[c] = s_step[i] * __bfloat162float(sQ[i * D + d]);
    *reinterpret_cast<bf16*>(sX + kmajor_off(i, d, X_BLK)) = __float2bfloat16(x[c]);
  }
  for (int it = 0; it < p.num_iter; ++it) {
    // per-token coefficients of this step, double-buffered by parity (the other buffer may still be read by threads
    // that have not left the previous step): om, step * om, om - 1
    float* coef = s_coef + (it & 1) * 3 * C;
    if (tid < C) {
      const float om = 1.f / (1.f - s_c[tid] * s_om[tid]);
      s_om[tid] = om;
      coef[tid] = om;
      coef[C + tid] = s_step[tid] * om;
      coef[2 * C + tid] = om - 1.f;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      issue_pair(aX, X_BLK);
    }
    ok = mbar_wait(bar, phase, ctx, 0xC20);
    phase ^= 1u;
    tc_fence_after();
    if (ok && d < C) {       // P row j = d: 32 columns = four 16-byte chunks of the row, 16 columns at a time
      const float gj = s_G[d];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[16], w[8];
        tmem_ld_x16(tS + lane_bits + i0 + 16 * half, r);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 16; c += 2) {
          const int i = i0 + 16 * half + c;
          const float m0 = d <= i ? __expf(s_G[i] - gj) : 0.f;
          const float m1 = d <= i + 1 ? __expf(s_G[i + 1] - gj) : 0.f;
          w[c >> 1] = pack_bf16x2(__uint_as_float(r[c]) * m0, __uint_as_float(r[c + 1]) * m1);
        }
#pragma unroll
        for (int q4 = 0; q4 < 2; ++q4)
          *reinterpret_cast<uint4*>(sP + sw128_offset((uint32_t)d, (uint32_t)(i0 * 2 + half * 32 + q4 * 16))) =
              make_uint4(w[q4 * 4], w[q4 * 4 + 1], w[q4 * 4 + 2], w[q4 * 4 + 3]);
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < C / 16; ++kk)
        umma_ss(tT2, make_desc_mnmajor_sw128(aK + kk * 2048, K_BLK), make_desc_mnmajor_sw128(aP + kk * 2048, C * 128),
                idescMN, kk > 0 ? 1u : 0u);
      umma_commit(bar);
    }
    ok = mbar_wait(bar, phase, ctx, 0xC30);
    phase ^= 1u;
    tc_fence_after();
#pragma unroll
    for (int part = 0; part < 4; ++part) {       // 8 token columns at a time keeps the register count under 128
      uint32_t r1[8], r2[8];
      if (ok) {
        tmem_ld_x8(tT1 + lane_bits + i0 + 8 * part, r1);
        tmem_ld_x8(tT2 + lane_bits + i0 + 8 * part, r2);
        tmem_ld_wait();
      }
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        const int c = 8 * part + cc, i = i0 + c;
        const float hx = s_eg[i] * __uint_as_float(r1[cc]) + __uint_as_float(r2[cc]);
        const float upd = coef[C + i] * (hx + s_lam[i] * x[c] - __bfloat162float(sQ[i * D + d])) + coef[2 * C + i] * xp[c];
        xp[c] = x[c];
        x[c] = coef[i] * x[c] - upd;
        *reinterpret_cast<bf16*>(sX + kmajor_off(i, d, X_BLK)) = __float2bfloat16(x[c]);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < 32; ++c) {
    const int i = i0 + c;
    if (t0 + i < p.T) p.x[(((size_t)b * p.T + t0 + i) * p.H + h) * D + d] = x[c];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace gka_cheb_tc
}  // namespace hmf

using namespace hmf;
using namespace hmf::gka_cheb_tc;

// Same contract as hmf_gka_cheb_fwd (gka_cheb.cu).
HMF_API int hmf_gka_cheb_fwd_tc(const void* q, const void* k, const float* gk, const float* hs, float* x, int B, int T, int H,
                                int N, int hs_chunks, long long q_sb, long long q_st, long long q_sh, long long k_sb,
                                long long k_st, long long k_sh, float ridge_ratio, int num_iter, cudaStream_t st) {
  HMF_REQUIRE(q && k && hs && x, "gka_cheb_fwd_tc: null tensor");
  HMF_REQUIRE(N == (T + C - 1) / C && (long long)B * H <= 65535 && num_iter >= 0 && hs_chunks >= N, "gka_cheb_fwd_tc: bad sizes");
  HMF_REQUIRE((reinterpret_cast<uintptr_t>(hs) & 15) == 0, "gka_cheb_fwd_tc: states must be 16-byte aligned");
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(gka_cheb_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  Params p;
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.gk = gk; p.hs = hs; p.x = x;
  p.q_sb = q_sb; p.q_st = q_st; p.q_sh = q_sh; p.k_sb = k_sb; p.k_st = k_st; p.k_sh = k_sh;
  p.B = B; p.T = T; p.H = H; p.N = N; p.hs_chunks = hs_chunks; p.num_iter = num_iter; p.ridge_ratio = ridge_ratio;
  p.status = status_ptr();
  dim3 grid(N, B * H);
  gka_cheb_tc_kernel<<<grid, NT, SMEM_BYTES, st>>>(p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
