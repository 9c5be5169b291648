// Decode-step kernels for serving (one new token per running request; all memory bound):
//   * paged GQA attention with split-KV partials and a combine pass,
//   * paged KV-cache append (reshape_and_cache),
//   * fused recurrent Gated DeltaNet step on slot-indexed fp32 state (L2 norm, decay, delta update, output),
//   * Mamba2 selective-state update on slot-indexed state,
//   * greedy / temperature sampling helper (argmax over the vocabulary).
// State tensors are indexed through `slots[r]` so continuous batching needs no gather / scatter copies.
#include <float.h>
#include <math.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace decode {

using bf16 = __nv_bfloat16;

// ------------------------------------------------------------------------------------
// KV cache append: k, v [N, Hkv, D] -> cache [num_blocks, block_size, Hkv, D] at slot_mapping[n]
// ------------------------------------------------------------------------------------
__global__ void cache_append_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v,
                                    bf16* __restrict__ kc, bf16* __restrict__ vc,
                                    const long long* __restrict__ slot_mapping, int row_elems, long long k_stride,
                                    long long v_stride) {
  const long long n = blockIdx.x;
  const long long slot = slot_mapping[n];
  if (slot < 0) return;
  for (int i = threadIdx.x * 8; i < row_elems; i += blockDim.x * 8) {
    *reinterpret_cast<uint4*>(kc + slot * row_elems + i) = *reinterpret_cast<const uint4*>(k + n * k_stride + i);
    *reinterpret_cast<uint4*>(vc + slot * row_elems + i) = *reinterpret_cast<const uint4*>(v + n * v_stride + i);
  }
}

// ------------------------------------------------------------------------------------
// Paged attention decode.  grid (R, Hkv, S splits), 128 threads, head dim 128, G = Hq / Hkv <= 8.
// Each CTA walks its share of the request's KV blocks in chunks of CH tokens:
//   scores (thread <-> token), chunk softmax statistics, then P V (thread <-> output dim).
// Partials (m, l, o) per split go to scratch; combine_kernel merges them.
// ------------------------------------------------------------------------------------
constexpr int PD = 128;   // head dim
constexpr int CH = 512;   // tokens per chunk
constexpr int MAXG = 8;

__global__ void __launch_bounds__(128)
paged_attn_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                         const int* __restrict__ block_tables, const int* __restrict__ seq_lens,
                         float* __restrict__ part_o, float* __restrict__ part_ml, int Hq, int Hkv, int block_size,
                         int max_blocks, int window, float scale) {
  const int r = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z, nsp = gridDim.z;
  const int G = Hq / Hkv;
  const int t = threadIdx.x;
  __shared__ float s_q[MAXG][PD];
  __shared__ float s_p[MAXG][CH];
  __shared__ float s_red[MAXG][4];
  const int L = seq_lens[r];
  int lo = window > 0 ? max(0, L - window) : 0;
  // contiguous share of [lo, L) for this split, aligned to chunks
  const int total = L - lo;
  const int per = ((total + nsp - 1) / nsp + CH - 1) / CH * CH;
  const int t_begin = lo + sp * per;
  const int t_end = min(L, t_begin + per);
  for (int g = 0; g < G; ++g) s_q[g][t] = __bfloat162float(q[((size_t)r * Hq + kvh * G + g) * PD + t]) * scale;
  float m_run[MAXG], l_run[MAXG], acc[MAXG];
#pragma unroll
  for (int g = 0; g < MAXG; ++g) { m_run[g] = -INFINITY; l_run[g] = 0.f; acc[g] = 0.f; }
  __syncthreads();
  const int* bt = block_tables + (size_t)r * max_blocks;
  const size_t row = (size_t)Hkv * PD;
  for (int c0 = t_begin; c0 < t_end; c0 += CH) {
    const int cn = min(CH, t_end - c0);
    // scores
    for (int i = t; i < cn; i += 128) {
      const int tok = c0 + i;
      const bf16* kp = kc + ((size_t)bt[tok / block_size] * block_size + tok % block_size) * row + (size_t)kvh * PD;
      float s[MAXG];
#pragma unroll
      for (int g = 0; g < MAXG; ++g) s[g] = 0.f;
#pragma unroll 4
      for (int d8 = 0; d8 < PD / 8; ++d8) {
        const uint4 u = *reinterpret_cast<const uint4*>(kp + d8 * 8);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
#pragma unroll
          for (int g = 0; g < MAXG; ++g)
            if (g < G) s[g] += f.x * s_q[g][d8 * 8 + 2 * j] + f.y * s_q[g][d8 * 8 + 2 * j + 1];
        }
      }
#pragma unroll
      for (int g = 0; g < MAXG; ++g)
        if (g < G) s_p[g][i] = s[g];
    }
    __syncthreads();
    // chunk max per head (warp w reduces heads w, w+4)
    const int warp = t >> 5, lane = t & 31;
    for (int g = warp; g < G; g += 4) {
      float mx = -INFINITY;
      for (int i = lane; i < cn; i += 32) mx = fmaxf(mx, s_p[g][i]);
      mx = warp_max(mx);
      if (lane == 0) s_red[g][0] = mx;
    }
    __syncthreads();
    float alpha[MAXG];
#pragma unroll
    for (int g = 0; g < MAXG; ++g) {
      if (g < G) {
        const float mn = fmaxf(m_run[g], s_red[g][0]);
        alpha[g] = (m_run[g] == -INFINITY) ? 0.f : __expf(m_run[g] - mn);
        m_run[g] = mn;
      }
    }
    for (int g = warp; g < G; g += 4) {
      float sum = 0.f;
      const float mn = m_run[g];
      for (int i = lane; i < cn; i += 32) {
        const float p = __expf(s_p[g][i] - mn);
        s_p[g][i] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      if (lane == 0) s_red[g][1] = sum;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < MAXG; ++g)
      if (g < G) { l_run[g] = l_run[g] * alpha[g] + s_red[g][1]; acc[g] *= alpha[g]; }
    // P V: thread t <-> output dim t
    for (int i = 0; i < cn; ++i) {
      const int tok = c0 + i;
      const float vv = __bfloat162float(
          vc[((size_t)bt[tok / block_size] * block_size + tok % block_size) * row + (size_t)kvh * PD + t]);
#pragma unroll
      for (int g = 0; g < MAXG; ++g)
        if (g < G) acc[g] = fmaf(s_p[g][i], vv, acc[g]);
    }
    __syncthreads();
  }
  for (int g = 0; g < G; ++g) {
    const size_t idx = ((size_t)r * Hq + kvh * G + g) * nsp + sp;
    part_o[idx * PD + t] = acc[g];
    if (t == 0) { part_ml[idx * 2] = m_run[g]; part_ml[idx * 2 + 1] = l_run[g]; }
  }
}

__global__ void __launch_bounds__(128)
paged_attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ o,
                          int nsp) {
  const size_t rh = blockIdx.x;
  const int t = threadIdx.x;
  float m = -INFINITY;
  for (int s = 0; s < nsp; ++s) m = fmaxf(m, part_ml[(rh * nsp + s) * 2]);
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < nsp; ++s) {
    const float ms = part_ml[(rh * nsp + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - m);
    l += part_ml[(rh * nsp + s) * 2 + 1] * w;
    acc += part_o[(rh * nsp + s) * PD + t] * w;
  }
  o[rh * PD + t] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
}

// ------------------------------------------------------------------------------------
// Gated DeltaNet recurrent step.  grid (R, H), 128 threads; thread t owns column t of S [Dk=128, Dv=128].
//   q, k [R, Hq|Hk, 128], v [R, Hv, 128] bf16 (post conv), g, beta [R, H] fp32; state [slots, H, 128, 128] fp32.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
gdn_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                  const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ state,
                  const int* __restrict__ slots, bf16* __restrict__ o, int H, int Hq, int Hk, int Hv, float scale,
                  int l2norm) {
  const int r = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
  __shared__ float s_q[128], s_k[128], s_red[8];
  const int hq = h / (H / Hq), hk = h / (H / Hk), hv = h / (H / Hv);
  float qv = __bfloat162float(q[((size_t)r * Hq + hq) * 128 + t]);
  float kv = __bfloat162float(k[((size_t)r * Hk + hk) * 128 + t]);
  if (l2norm) {
    float sq = warp_sum(qv * qv), sk = warp_sum(kv * kv);
    if ((t & 31) == 0) { s_red[t >> 5] = sq; s_red[4 + (t >> 5)] = sk; }
    __syncthreads();
    sq = s_red[0] + s_red[1] + s_red[2] + s_red[3];
    sk = s_red[4] + s_red[5] + s_red[6] + s_red[7];
    qv *= rsqrtf(sq + 1e-6f);
    kv *= rsqrtf(sk + 1e-6f);
  }
  s_q[t] = qv * scale;
  s_k[t] = kv;
  __syncthreads();
  const float decay = __expf(g[(size_t)r * H + h]);
  const float b = beta[(size_t)r * H + h];
  float* S = state + (((size_t)slots[r] * H + h) * 128) * 128;
  float col[128];
  float pred = 0.f;
#pragma unroll
  for (int d = 0; d < 128; ++d) {
    col[d] = S[(size_t)d * 128 + t] * decay;
    pred = fmaf(col[d], s_k[d], pred);
  }
  const float dv = b * (__bfloat162float(v[((size_t)r * Hv + hv) * 128 + t]) - pred);
  float out = 0.f;
#pragma unroll
  for (int d = 0; d < 128; ++d) {
    col[d] = fmaf(s_k[d], dv, col[d]);
    out = fmaf(col[d], s_q[d], out);
    S[(size_t)d * 128 + t] = col[d];
  }
  o[((size_t)r * H + h) * 128 + t] = __float2bfloat16(out);
}

// ------------------------------------------------------------------------------------
// Mamba2 selective state update.  grid (R, H), P threads (P = head dim <= 128), state [slots, H, P, N] fp32.
//   x [R, Hx, P] bf16 (Hx = H / x_rep), dt [R, H] fp32 (post softplus), A [H], Bm [R, Hb, N], Cm [R, H, N] bf16, D [H].
// ------------------------------------------------------------------------------------
__global__ void ssd_decode_kernel(const bf16* __restrict__ x, const float* __restrict__ dt,
                                  const float* __restrict__ A, const bf16* __restrict__ Bm,
                                  const bf16* __restrict__ Cm, const float* __restrict__ Dp,
                                  float* __restrict__ state, const int* __restrict__ slots, bf16* __restrict__ y,
                                  int H, int Hx, int Hb, int P, int N) {
  const int r = blockIdx.x, h = blockIdx.y, pidx = threadIdx.x;
  extern __shared__ float s_bc[];  // B[N], C[N]
  float* sB = s_bc;
  float* sC = s_bc + N;
  const int hx = h / (H / Hx), hb = h / (H / Hb);
  for (int n = pidx; n < N; n += blockDim.x) {
    sB[n] = __bfloat162float(Bm[((size_t)r * Hb + hb) * N + n]);
    sC[n] = __bfloat162float(Cm[((size_t)r * H + h) * N + n]);
  }
  __syncthreads();
  if (pidx >= P) return;
  const float dtv = dt[(size_t)r * H + h];
  const float a = __expf(dtv * A[h]);
  const float xv = __bfloat162float(x[((size_t)r * Hx + hx) * P + pidx]);
  const float dx = dtv * xv;
  float* S = state + (((size_t)slots[r] * H + h) * P + pidx) * N;
  float acc = 0.f;
  for (int n = 0; n < N; n += 4) {
    float4 s4 = *reinterpret_cast<float4*>(S + n);
    s4.x = fmaf(s4.x, a, dx * sB[n]);
    s4.y = fmaf(s4.y, a, dx * sB[n + 1]);
    s4.z = fmaf(s4.z, a, dx * sB[n + 2]);
    s4.w = fmaf(s4.w, a, dx * sB[n + 3]);
    acc += s4.x * sC[n] + s4.y * sC[n + 1] + s4.z * sC[n + 2] + s4.w * sC[n + 3];
    *reinterpret_cast<float4*>(S + n) = s4;
  }
  y[((size_t)r * H + h) * P + pidx] = __float2bfloat16(acc + (Dp ? Dp[h] * xv : 0.f));
}

// Same update with one warp per state row (N a multiple of 128): lane l holds columns 4l..4l+3 of every
// 128-column group, so a warp reads and writes whole 512-byte rows; 8 warps walk the P rows 4 at a time.
template <int NG>
__global__ void __launch_bounds__(256)
ssd_decode_rows_kernel(const bf16* __restrict__ x, const float* __restrict__ dt, const float* __restrict__ A,
                       const bf16* __restrict__ Bm, const bf16* __restrict__ Cm, const float* __restrict__ Dp,
                       float* __restrict__ state, const int* __restrict__ slots, bf16* __restrict__ y, int H, int Hx,
                       int Hb, int P) {
  constexpr int N = NG * 128;
  const int r = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hx = h / (H / Hx), hb = h / (H / Hb);
  float bv[NG][4], cv[NG][4];
#pragma unroll
  for (int j = 0; j < NG; ++j) {
    const uint2 ub = *reinterpret_cast<const uint2*>(Bm + ((size_t)r * Hb + hb) * N + j * 128 + lane * 4);
    const uint2 uc = *reinterpret_cast<const uint2*>(Cm + ((size_t)r * H + h) * N + j * 128 + lane * 4);
    const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ub.x));
    const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ub.y));
    const float2 c0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uc.x));
    const float2 c1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uc.y));
    bv[j][0] = b0.x; bv[j][1] = b0.y; bv[j][2] = b1.x; bv[j][3] = b1.y;
    cv[j][0] = c0.x; cv[j][1] = c0.y; cv[j][2] = c1.x; cv[j][3] = c1.y;
  }
  const float dtv = dt[(size_t)r * H + h];
  const float a = __expf(dtv * A[h]);
  const float dcoef = Dp ? Dp[h] : 0.f;
  float* S = state + ((size_t)slots[r] * H + h) * P * N;
  constexpr int RU = 4;   // rows in flight per warp
  for (int p0 = warp * RU; p0 < P; p0 += 8 * RU) {
    float4 sv[RU][NG];
    float xv[RU];
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const int pr = min(p0 + u, P - 1);
      xv[u] = __bfloat162float(x[((size_t)r * Hx + hx) * P + pr]);
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

// ------------------------------------------------------------------------------------
// argmax over the vocabulary (greedy sampling): logits [R, V] bf16 or fp32 -> ids [R]
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void argmax_kernel(const T* __restrict__ logits, long long* __restrict__ ids, int V, long long ld) {
  const int r = blockIdx.x;
  float best = -INFINITY;
  int bi = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float f = (float)logits[(size_t)r * ld + i];
    if (f > best) { best = f; bi = i; }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    ids[r] = bi;
  }
}

}  // namespace decode
}  // namespace hmf

using namespace hmf;
using namespace hmf::decode;

HMF_API int hmf_cache_append(const void* k, const void* v, void* kc, void* vc, const long long* slot_mapping,
                             long long n_tokens, int Hkv, int D, long long k_stride, long long v_stride,
                             cudaStream_t st) {
  HMF_REQUIRE((Hkv * D) % 8 == 0 && k_stride % 8 == 0 && v_stride % 8 == 0, "cache_append: rows must be 16-byte multiples");
  if (n_tokens == 0) return HMF_OK;
  cache_append_kernel<<<(unsigned)n_tokens, 128, 0, st>>>((const bf16*)k, (const bf16*)v, (bf16*)kc, (bf16*)vc,
                                                          slot_mapping, Hkv * D, k_stride, v_stride);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// part_o: [R, Hq, splits, 128] fp32, part_ml: [R, Hq, splits, 2] fp32 scratch from the caller.
HMF_API int hmf_paged_attention_decode(const void* q, const void* kc, const void* vc, const int* block_tables,
                                       const int* seq_lens, void* o, float* part_o, float* part_ml, int R, int Hq,
                                       int Hkv, int D, int block_size, int max_blocks, int splits, int window,
                                       float scale, cudaStream_t st) {
  HMF_REQUIRE(D == PD, "paged attention: head dim %d unsupported (128)", D);
  HMF_REQUIRE(Hq % Hkv == 0 && Hq / Hkv <= MAXG, "paged attention: group size %d unsupported (<= %d)", Hq / Hkv, MAXG);
  HMF_REQUIRE(splits >= 1 && splits <= 64, "paged attention: splits=%d out of range", splits);
  if (R == 0) return HMF_OK;
  dim3 grid(R, Hkv, splits);
  paged_attn_decode_kernel<<<grid, 128, 0, st>>>((const bf16*)q, (const bf16*)kc, (const bf16*)vc, block_tables,
                                                 seq_lens, part_o, part_ml, Hq, Hkv, block_size, max_blocks, window,
                                                 scale);
  HMF_CHECK_CUDA(cudaGetLastError());
  paged_attn_combine_kernel<<<R * Hq, 128, 0, st>>>(part_o, part_ml, (bf16*)o, splits);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_gdn_decode(const void* q, const void* k, const void* v, const float* g, const float* beta,
                           float* state, const int* slots, void* o, int R, int H, int Hq, int Hk, int Hv, int Dk,
                           int Dv, float scale, int l2norm, cudaStream_t st) {
  HMF_REQUIRE(Dk == 128 && Dv == 128, "gdn_decode: head dims %d/%d unsupported (128)", Dk, Dv);
  HMF_REQUIRE(H % Hq == 0 && H % Hk == 0 && H % Hv == 0, "gdn_decode: head counts do not divide H=%d", H);
  if (R == 0) return HMF_OK;
  dim3 grid(R, H);
  gdn_decode_kernel<<<grid, 128, 0, st>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, g, beta, state, slots,
                                          (bf16*)o, H, Hq, Hk, Hv, scale, l2norm);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_ssd_decode(const void* x, const float* dt, const float* A, const void* Bm, const void* Cm,
                           const float* Dp, float* state, const int* slots, void* y, int R, int H, int Hx, int Hb,
                           int P, int N, cudaStream_t st) {
  HMF_REQUIRE(P <= 128 && N % 4 == 0 && N <= 256, "ssd_decode: P=%d N=%d unsupported", P, N);
  HMF_REQUIRE(H % Hx == 0 && H % Hb == 0, "ssd_decode: head counts do not divide H=%d", H);
  if (R == 0) return HMF_OK;
  dim3 grid(R, H);
  if (N == 128 || N == 256) {
    if (N == 128)
      ssd_decode_rows_kernel<1><<<grid, 256, 0, st>>>((const bf16*)x, dt, A, (const bf16*)Bm, (const bf16*)Cm, Dp, state,
                                                      slots, (bf16*)y, H, Hx, Hb, P);
    else
      ssd_decode_rows_kernel<2><<<grid, 256, 0, st>>>((const bf16*)x, dt, A, (const bf16*)Bm, (const bf16*)Cm, Dp, state,
                                                      slots, (bf16*)y, H, Hx, Hb, P);
    HMF_CHECK_CUDA(cudaGetLastError());
    return HMF_OK;
  }
  ssd_decode_kernel<<<grid, 128, 2 * N * sizeof(float), st>>>((const bf16*)x, dt, A, (const bf16*)Bm,
                                                              (const bf16*)Cm, Dp, state, slots, (bf16*)y, H, Hx, Hb,
                                                              P, N);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

HMF_API int hmf_argmax(const void* logits, int is_bf16, long long* ids, int R, int V, long long ld, cudaStream_t st) {
  if (R == 0) return HMF_OK;
  if (is_bf16) argmax_kernel<bf16><<<R, 1024, 0, st>>>((const bf16*)logits, ids, V, ld);
  else argmax_kernel<float><<<R, 1024, 0, st>>>((const float*)logits, ids, V, ld);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
