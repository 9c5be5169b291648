// Gated delta rule, chunk-parallel preparation (one CTA per 64-token chunk of one head).
//
// From q, k, v, g (log decay), beta it produces the bf16 operand tiles of the scan kernels:
//   wqT [chunk][2][128][64] : w^T and (q e^{G} scale / |q|)^T
//   kPT [chunk][192][64]    : (k e^{g_last - G} / |k|)^T and P = causal((q k^T) . e^{G_i - G_j}) (normalised, scaled)
//   uT  [chunk][128][64]    : u^T
//   glast [chunk]
// with the WY factors  u = T (beta v),  w = T (beta e^{G} k/|k|),  T = (I + tril_strict(beta k k^T . decay))^{-1}.
//
// Tensor-core work is done "feature-major": the 128-wide feature dimension is the MMA M dimension.
//   Gram     : [k ; q] (128 x 128)  x  k^T           -> k k^T | q k^T         (128 x 64)
//   factors  : v^T x (T diag(beta))^T,  k^T x [T diag(beta e^G /|k|) ; diag(e^{gl-G}/|k|)]^T,  q^T x diag(..)^T
// i.e. the row scalings, the triangular solve result and the transposes are all folded into small
// 64x64 B operands written by the threads, so q, k, v are consumed exactly as TMA delivered them.
// The 64x64 unit-lower-triangular inverse is a forward substitution in fp32, one column per thread.
#include <math.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace gdn_prep {

using bf16 = __nv_bfloat16;
constexpr int C = 64;
constexpr int D = 128;
constexpr int KQ_BYTES = 2 * 128 * 128;  // two 64-feature panels of [128 rows x 128 B] (k rows 0-63, q rows 64-127)
constexpr int V_BYTES = 2 * C * 128;     // two panels of [64 rows x 128 B]
constexpr int A_BYTES = C * C * 4;       // fp32 strictly-lower matrix
constexpr int BU_BYTES = C * 128;        // [64 x 64] bf16, K-major swizzled
constexpr int BWK_BYTES = 2 * C * 128;   // [128 x 64]
constexpr int BQ_BYTES = C * 128;
constexpr int OFF_V = KQ_BYTES;
constexpr int OFF_A = OFF_V + V_BYTES;
constexpr int OFF_BU = OFF_A + A_BYTES;
constexpr int OFF_BWK = OFF_BU + BU_BYTES;
constexpr int OFF_BQ = OFF_BWK + BWK_BYTES;
constexpr int OFF_MISC = OFF_BQ + BQ_BYTES;  // G[64], kinv[64], qinv[64], beta[64] fp32 + barriers
constexpr int SMEM = OFF_MISC + 4 * C * 4 + 64;

struct Params {
  const float* g;     // [B, T, H]
  const float* beta;  // [B, T, H]
  bf16* wqT;
  bf16* kPT;
  bf16* uT;
  float* glast;
  int B, T, H, N;
  int k_rep, v_rep;   // query heads per key / value head (1 when k, v are already expanded)
  float scale;
  int l2norm;
  int gla;            // 1: plain gated linear attention (no delta rule): T = I, beta = 1, w = 0
  unsigned int* status;
};

__device__ __forceinline__ float row_sumsq_swizzled(const uint8_t* panel0, int panel_stride, int r) {
  float s = 0.f;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 u = *reinterpret_cast<const uint4*>(panel0 + p * panel_stride + r * 128 + ((c ^ (r & 7)) << 4));
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h2[i]);
        s += f.x * f.x + f.y * f.y;
      }
    }
  }
  return s;
}

__device__ __forceinline__ void store_row_bf16(bf16* dst, const uint32_t (&v)[64]) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint4 w;
    w.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]), __uint_as_float(v[8 * i + 1]));
    w.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
    w.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
    w.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
    d4[i] = w;
  }
}

__global__ void __launch_bounds__(128, 2)
gdn_prep_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sKQ = smem;
  uint8_t* sV = smem + OFF_V;
  float* sA = reinterpret_cast<float*>(smem + OFF_A);
  uint8_t* sBU = smem + OFF_BU;
  uint8_t* sBWK = smem + OFF_BWK;
  uint8_t* sBQ = smem + OFF_BQ;
  float* sG = reinterpret_cast<float*>(smem + OFF_MISC);
  float* sKinv = sG + C;
  float* sQinv = sKinv + C;
  float* sBeta = sQinv + C;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sBeta + C);
  uint64_t* ld_bar = bars;
  uint64_t* mma_bar = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const WaitCtx ctx{abort_flag, p.status};
  const int n = blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int t0 = n * C;
  const long long chunk = (long long)bh * p.N + n;

  if (tid == 0) {
    if ((smem_u32(smem) & 1023u) != 0) report_error(p.status, kBadArgument, 0xC1);
    mbar_init(ld_bar, 1);
    mbar_init(mma_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    mbar_expect_tx(ld_bar, 3 * C * D * 2);
#pragma unroll
    for (int pn = 0; pn < 2; ++pn) {
      tma_load_4d(sKQ + pn * 16384, &tmK, ld_bar, pn * 64, h / p.k_rep, t0, b);
      tma_load_4d(sKQ + pn * 16384 + 8192, &tmQ, ld_bar, pn * 64, h, t0, b);
      tma_load_4d(sV + pn * 8192, &tmV, ld_bar, pn * 64, h / p.v_rep, t0, b);
    }
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  // gates: cumulative sum within the chunk (fp32) and beta
  if (tid < C) {
    const int t = t0 + tid;
    sG[tid] = (t < p.T) ? p.g[((size_t)b * p.T + t) * p.H + h] : 0.f;
    sBeta[tid] = p.gla ? 1.f : ((t < p.T) ? p.beta[((size_t)b * p.T + t) * p.H + h] : 0.f);
  }
  // zero the diagonal B tiles and the k~ half of B_wk while the loads are in flight
  for (int i = tid; i < (BQ_BYTES + BWK_BYTES / 2) / 16; i += 128) {
    uint4* dst = (i < BQ_BYTES / 16) ? reinterpret_cast<uint4*>(sBQ) + i
                                     : reinterpret_cast<uint4*>(sBWK + BWK_BYTES / 2) + (i - BQ_BYTES / 16);
    *dst = make_uint4(0, 0, 0, 0);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tid == 0) {
    float acc = 0.f;
    for (int i = 0; i < C; ++i) {
      acc += sG[i];
      sG[i] = acc;
    }
  }
  mbar_wait(ld_bar, 0, ctx, 0x510);
  // row norms (thread < 64: key row, else query row)
  {
    const int r = tid & 63;
    const uint8_t* base = sKQ + (tid < C ? 0 : 8192);
    const float ss = row_sumsq_swizzled(base, 16384, r);
    const float inv = p.l2norm ? rsqrtf(ss + 1e-6f) : 1.f;
    if (tid < C) sKinv[r] = inv; else sQinv[r] = inv;
  }
  __syncthreads();

  // ---- Gram: [k ; q] x k^T -> TMEM cols [0, 64)
  if (tid == 0) {
    constexpr uint32_t idescG = make_idesc_bf16(128, 64, false, false);
    const uint32_t a = smem_u32(sKQ);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint64_t ad = make_desc_kmajor_sw128(a + (kk / 4) * 16384 + (kk % 4) * 32);
      umma_ss(tmem_base, ad, ad, idescG, kk > 0 ? 1u : 0u);  // B = first 64 rows of the same tile
    }
    umma_commit(mma_bar);
  }
  mbar_wait(mma_bar, 0, ctx, 0x520);
  tc_fence_after();
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
  {
    uint32_t gr[64];
    tmem_ld_x32(tmem_base + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&gr[0]));
    tmem_ld_x32(tmem_base + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&gr[32]));
    tmem_ld_wait();
    const int i = tid & 63;
    const float Gi = sG[i];
    if (tid < C) {
      const float bi = sBeta[i] * sKinv[i];
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const float a = (j < i && !p.gla) ? bi * __uint_as_float(gr[j]) * sKinv[j] * __expf(Gi - sG[j]) : 0.f;
        sA[i * C + j] = a;
      }
    } else {
      const float qi = sQinv[i] * p.scale;
      uint32_t pr[64];
#pragma unroll
      for (int j = 0; j < C; ++j)
        pr[j] = __float_as_uint((j <= i) ? qi * __uint_as_float(gr[j]) * sKinv[j] * __expf(Gi - sG[j]) : 0.f);
      store_row_bf16(p.kPT + ((size_t)chunk * (D + C) + D + i) * C, pr);
    }
  }
  __syncthreads();

  // ---- T = (I + A)^{-1}: thread c owns column c (forward substitution); others fill the diagonal tiles
  if (tid < C) {
    const int c = tid;
    float Tc[C];
#pragma unroll
    for (int i = 0; i < C; ++i) {
      float acc = (i == c) ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) acc = fmaf(-sA[i * C + j], Tc[j], acc);
      Tc[i] = acc;
    }
    const float bc = sBeta[c];
    const float bw = p.gla ? 0.f : bc * __expf(sG[c]) * sKinv[c];
#pragma unroll
    for (int i = 0; i < C; ++i) {
      *reinterpret_cast<bf16*>(sBU + sw128_offset(i, c * 2)) = __float2bfloat16(Tc[i] * bc);
      *reinterpret_cast<bf16*>(sBWK + sw128_offset(i, c * 2)) = __float2bfloat16(Tc[i] * bw);
    }
  } else {
    const int c = tid - C;
    const float gl = sG[C - 1];
    *reinterpret_cast<bf16*>(sBWK + BWK_BYTES / 2 + sw128_offset(c, c * 2)) =
        __float2bfloat16(__expf(gl - sG[c]) * sKinv[c]);
    *reinterpret_cast<bf16*>(sBQ + sw128_offset(c, c * 2)) = __float2bfloat16(p.scale * __expf(sG[c]) * sQinv[c]);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // ---- factor products (A operands MN-major straight from the q, k, v tiles)
  if (tid == 0) {
    constexpr uint32_t idesc64 = make_idesc_bf16(128, 64, true, false);
    constexpr uint32_t idesc128 = make_idesc_bf16(128, 128, true, false);
    const uint32_t aKQ = smem_u32(sKQ), aV = smem_u32(sV);
    const uint32_t bU = smem_u32(sBU), bWK = smem_u32(sBWK), bQ = smem_u32(sBQ);
#pragma unroll
    for (int kk = 0; kk < C / 16; ++kk) {
      umma_ss(tmem_base, make_desc_mnmajor_sw128(aV + kk * 2048, 8192), make_desc_kmajor_sw128(bU + kk * 32), idesc64,
              kk > 0 ? 1u : 0u);
      umma_ss(tmem_base + 64, make_desc_mnmajor_sw128(aKQ + kk * 2048, 16384), make_desc_kmajor_sw128(bWK + kk * 32),
              idesc128, kk > 0 ? 1u : 0u);
      umma_ss(tmem_base + 192, make_desc_mnmajor_sw128(aKQ + 8192 + kk * 2048, 16384),
              make_desc_kmajor_sw128(bQ + kk * 32), idesc64, kk > 0 ? 1u : 0u);
    }
    umma_commit(mma_bar);
    p.glast[chunk] = sG[C - 1];
  }
  mbar_wait(mma_bar, 1, ctx, 0x530);
  tc_fence_after();
  {
    uint32_t r[64];
    // u^T
    tmem_ld_x32(tmem_base + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
    tmem_ld_x32(tmem_base + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
    tmem_ld_wait();
    store_row_bf16(p.uT + ((size_t)chunk * D + tid) * C, r);
    // w^T
    tmem_ld_x32(tmem_base + lane_off + 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
    tmem_ld_x32(tmem_base + lane_off + 96, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
    tmem_ld_wait();
    store_row_bf16(p.wqT + (((size_t)chunk * 2 + 0) * D + tid) * C, r);
    // k~^T
    tmem_ld_x32(tmem_base + lane_off + 128, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
    tmem_ld_x32(tmem_base + lane_off + 160, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
    tmem_ld_wait();
    store_row_bf16(p.kPT + ((size_t)chunk * (D + C) + tid) * C, r);
    // q~^T
    tmem_ld_x32(tmem_base + lane_off + 192, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
    tmem_ld_x32(tmem_base + lane_off + 224, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
    tmem_ld_wait();
    store_row_bf16(p.wqT + (((size_t)chunk * 2 + 1) * D + tid) * C, r);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

static int make_map_bthd(CUtensorMap* m, const void* base, int B, int T, int H, long long sb, long long st,
                         long long sh) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[4] = {2, (uint64_t)sh * 2, (uint64_t)st * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, 1, (uint32_t)C, 1};
  return make_tensor_map(m, base, 0, 4, dims, strides, box, 3);
}

}  // namespace gdn_prep
}  // namespace hmf

// q [B,T,H,128], k [B,T,Hk,128], v [B,T,Hv,128] bf16 with element strides (batch, token, head) and unit
// inner stride; g, beta [B,T,H] fp32 contiguous.  Outputs as described at the top of this file, indexed
// by chunk = (b*H + h)*N + n.
HMF_API int hmf_gdn_prep(const void* q, const void* k, const void* v, const float* g, const float* beta,
                         void* wqT, void* kPT, void* uT, float* glast, int B, int T, int H, int Hk, int Hv,
                         int N, long long q_sb, long long q_st, long long q_sh, long long k_sb, long long k_st,
                         long long k_sh, long long v_sb, long long v_st, long long v_sh, float scale, int l2norm, int gla,
                         cudaStream_t stream) {
  using namespace hmf;
  using namespace hmf::gdn_prep;
  HMF_REQUIRE(q && k && v && g && (beta || gla) && wqT && kPT && uT && glast, "gdn_prep: null tensor");
  HMF_REQUIRE(H % Hk == 0 && H % Hv == 0, "gdn_prep: H=%d must be a multiple of Hk=%d and Hv=%d", H, Hk, Hv);
  HMF_REQUIRE(N * C >= T && N > 0, "gdn_prep: N=%d chunks do not cover T=%d", N, T);
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  if ((rc = make_map_bthd(&tmQ, q, B, T, H, q_sb, q_st, q_sh)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmK, k, B, T, Hk, k_sb, k_st, k_sh)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmV, v, B, T, Hv, v_sb, v_st, v_sh)) != HMF_OK) return rc;
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(gdn_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured = true;
  }
  Params p;
  p.g = g; p.beta = beta; p.wqT = (bf16*)wqT; p.kPT = (bf16*)kPT; p.uT = (bf16*)uT; p.glast = glast;
  p.B = B; p.T = T; p.H = H; p.N = N; p.k_rep = H / Hk; p.v_rep = H / Hv;
  p.scale = scale; p.l2norm = l2norm; p.gla = gla; p.status = status_ptr();
  dim3 grid(N, B * H);
  gdn_prep_kernel<<<grid, 128, SMEM, stream>>>(tmQ, tmK, tmV, p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
