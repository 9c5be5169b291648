// Batched token sampling for the serving engine: temperature, top-k, top-p (nucleus), min-p and an optional
// repetition penalty, one CTA per row of logits, no sort.
//
// For a row with temperature T > 0:  p_i = exp(l_i / T - max) .  The kept set of top-k / top-p / min-p is always
// {i : p_i >= t} for some threshold t, so the three filters reduce to finding thresholds by bisection on t in [0, 1]
// (each step is one pass over the row that counts the survivors or sums their mass):
//   top-k : largest t with   count(p >= t) >= k            (ties at the threshold are all kept)
//   top-p : largest t with   mass(p >= t)  >= top_p * mass(p >= t_k)     (applied after top-k, as in the HF order)
//   min-p : t = min_p (p is relative to the maximum, whose p is 1)
// The sample is drawn by inverse CDF over the survivors in index order with the uniform number the caller passes
// (so the host controls the random stream and a row is reproducible).  T <= 0 is the arg-max.
#include <float.h>
#include <math.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace sampler {

constexpr int THREADS = 1024;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = threadIdx.x < (THREADS >> 5) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    r = warp_sum(r);
    if (threadIdx.x == 0) red[32] = r;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = threadIdx.x < (THREADS >> 5) ? red[threadIdx.x] : -INFINITY;
  if (threadIdx.x < 32) {
    r = warp_max(r);
    if (threadIdx.x == 0) red[32] = r;
  }
  __syncthreads();
  return red[32];
}

template <typename T>
__device__ __forceinline__ float ld(const T* p, long long i);
template <>
__device__ __forceinline__ float ld<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

// params[row] = {temperature, top_p, min_p, uniform}; topk[row] (0 = off)
template <typename T>
__global__ void __launch_bounds__(THREADS, 1)
sample_kernel(const T* __restrict__ logits, long long ld_row, int V, const float4* __restrict__ params,
              const int* __restrict__ topk, long long* __restrict__ out) {
  __shared__ float red[40];
  __shared__ float chunk_mass[THREADS];
  __shared__ int winner;
  const int row = blockIdx.x;
  const T* l = logits + (long long)row * ld_row;
  const float4 pr = params[row];
  const float temp = pr.x;
  const int k = topk ? topk[row] : 0;
  // arg-max (also the T <= 0 answer): lowest index among the maxima
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += THREADS) mx = fmaxf(mx, ld(l, i));
  mx = block_max(mx, red);
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) winner = V;
    __syncthreads();
    int best = V;
    for (int i = threadIdx.x; i < V; i += THREADS)
      if (ld(l, i) == mx) best = min(best, i);
    if (best < V) atomicMin(&winner, best);
    __syncthreads();
    if (threadIdx.x == 0) out[row] = winner < V ? winner : 0;
    return;
  }
  const float inv_t = 1.f / temp;
  auto prob = [&](int i) { return __expf((ld(l, i) - mx) * inv_t); };
  // top-k threshold
  float t_keep = 0.f;
  if (k > 0 && k < V) {
    float lo = 0.f, hi = 1.f;           // invariant: count(p >= lo) >= k
    for (int it = 0; it < 30; ++it) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = threadIdx.x; i < V; i += THREADS) c += prob(i) >= mid ? 1.f : 0.f;
      c = block_sum(c, red);
      if (c >= (float)k) lo = mid; else hi = mid;
    }
    t_keep = lo;
  }
  t_keep = fmaxf(t_keep, pr.z);          // min-p
  if (pr.y > 0.f && pr.y < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += THREADS) { const float p = prob(i); z += p >= t_keep ? p : 0.f; }
    z = block_sum(z, red);
    const float want = pr.y * z;
    float lo = t_keep, hi = 1.f;         // invariant: mass(p >= lo) >= want
    for (int it = 0; it < 30; ++it) {
      const float mid = 0.5f * (lo + hi);
      float m = 0.f;
      for (int i = threadIdx.x; i < V; i += THREADS) { const float p = prob(i); m += p >= mid ? p : 0.f; }
      m = block_sum(m, red);
      if (m >= want) lo = mid; else hi = mid;
    }
    t_keep = lo;
  }
  // inverse CDF over the survivors in index order: thread t owns the contiguous chunk [t*per, (t+1)*per)
  const int per = (V + THREADS - 1) / THREADS;
  const int i0 = threadIdx.x * per, i1 = min(V, i0 + per);
  float mine = 0.f;
  for (int i = i0; i < i1; ++i) { const float p = prob(i); mine += p >= t_keep ? p : 0.f; }
  chunk_mass[threadIdx.x] = mine;
  const float total = block_sum(mine, red);
  if (threadIdx.x == 0) {
    float target = fminf(fmaxf(pr.w, 0.f), 0.99999994f) * total, acc = 0.f;
    int w = 0;
    for (int t = 0; t < THREADS; ++t) {
      if (acc + chunk_mass[t] > target || t == THREADS - 1) { w = t; break; }
      acc += chunk_mass[t];
    }
    // walk back to a chunk that has mass if rounding pushed the target past the last survivor
    while (w > 0 && chunk_mass[w] == 0.f) --w;
    winner = w;
    red[33] = target - acc;
  }
  __syncthreads();
  if (threadIdx.x == winner) {
    float rem = red[33], acc = 0.f;
    int pick = -1, last = -1;
    for (int i = i0; i < i1; ++i) {
      const float p = prob(i);
      if (p >= t_keep) {
        last = i;
        acc += p;
        if (acc > rem) { pick = i; break; }
      }
    }
    out[row] = pick >= 0 ? pick : last;
  }
}

// logits[row, ids[row, j]] /= penalty if positive else *= penalty, for the n_ids[row] first ids of each row
template <typename T>
__global__ void repetition_penalty_kernel(T* __restrict__ logits, long long ld_row, const long long* __restrict__ ids,
                                          int max_ids, const int* __restrict__ n_ids, const float* __restrict__ penalty) {
  const int row = blockIdx.x;
  const float pen = penalty[row];
  if (pen == 1.f) return;
  for (int j = threadIdx.x; j < n_ids[row]; j += blockDim.x) {
    const long long id = ids[(long long)row * max_ids + j];
    // a token that occurs twice must be penalised once: only its first occurrence acts
    bool first = true;
    for (int q = 0; q < j; ++q)
      if (ids[(long long)row * max_ids + q] == id) { first = false; break; }
    if (!first) continue;
    T* p = logits + (long long)row * ld_row + id;
    const float v = ld<T>(p, 0);
    const float r = v > 0.f ? v / pen : v * pen;
    if constexpr (sizeof(T) == 2) *p = __float2bfloat16(r); else *p = r;
  }
}

}  // namespace sampler
}  // namespace hmf

// logits [rows, V] (bf16 if is_bf16 else fp32, row stride ld_row elements); params [rows] float4 = {temperature,
// top_p, min_p, uniform in [0, 1)}; topk [rows] int32 or null; out [rows] int64.
HMF_API int hmf_sample(const void* logits, int is_bf16, long long ld_row, int rows, int V, const void* params,
                       const int* topk, long long* out, cudaStream_t st) {
  using namespace hmf;
  HMF_REQUIRE(logits && params && out && rows > 0 && V > 0, "sample: bad arguments");
  if (is_bf16)
    sampler::sample_kernel<__nv_bfloat16><<<rows, sampler::THREADS, 0, st>>>((const __nv_bfloat16*)logits, ld_row, V,
                                                                            (const float4*)params, topk, out);
  else
    sampler::sample_kernel<float><<<rows, sampler::THREADS, 0, st>>>((const float*)logits, ld_row, V,
                                                                    (const float4*)params, topk, out);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// In place: tokens ids[row, :n_ids[row]] (history of the request) get their logit divided by penalty[row] if positive,
// multiplied otherwise.
HMF_API int hmf_repetition_penalty(void* logits, int is_bf16, long long ld_row, int rows, const long long* ids,
                                   int max_ids, const int* n_ids, const float* penalty, cudaStream_t st) {
  using namespace hmf;
  HMF_REQUIRE(logits && ids && n_ids && penalty && rows > 0, "repetition_penalty: bad arguments");
  if (is_bf16)
    sampler::repetition_penalty_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>((__nv_bfloat16*)logits, ld_row, ids, max_ids, n_ids, penalty);
  else
    sampler::repetition_penalty_kernel<float><<<rows, 256, 0, st>>>((float*)logits, ld_row, ids, max_ids, n_ids, penalty);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
