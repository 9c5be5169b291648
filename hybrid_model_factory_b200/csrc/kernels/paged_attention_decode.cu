// Paged GQA attention for the decode step on tcgen05 ("token-major" formulation).
//
// One CTA handles (request r, KV head, KV split).  A tile is 128 cached tokens:
//   S^T [128 tokens x 16]  = K_tile [128 x 128]   . Q^T [128 x 16]      (A = K tile, K-major, straight from TMA;
//                                                                         B = the G <= 16 query heads of the group)
//   O^T [128 dims  x 16]  += V_tile^T [128 x 128] . P [128 tokens x 16]  (A = V tile, MN-major, straight from TMA;
//                                                                         B = probabilities written by the softmax warps)
// so the tensor core's M dimension is the token / feature axis and the few query heads are N.  K and V
// tiles go from the paged cache to shared memory by TMA (one 64-token x 64-dim box per block half) through a
// 3-stage ring and are never touched by a thread; both accumulators live in tensor memory (48 columns).
// Softmax: thread <-> token row, CTA-wide running reference maximum with lazy rescaling of O^T (only when the
// maximum grows by more than 2^8), partial (m, l, O) per split; `paged_attn_combine` merges the splits.
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5 softmax.
#include <math.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace pad {

using bf16 = __nv_bfloat16;

constexpr int D = 128;        // head dim
constexpr int TT = 128;       // tokens per tile
constexpr int NQ = 16;        // padded number of query heads per KV head (MMA N)
constexpr int NS = 3;         // K/V ring stages
constexpr int PANEL = TT * 128;            // one 64-dim panel of a tile: 128 token rows x 128 B
constexpr int TILE_BYTES = 2 * PANEL;      // 32 KB
constexpr int QP_PANEL = NQ * 128;         // 2 KB: one 64-wide K panel of a 16-row B operand
constexpr int OFF_K = 0;
constexpr int OFF_V = NS * TILE_BYTES;
constexpr int OFF_Q = 2 * NS * TILE_BYTES;
constexpr int OFF_P = OFF_Q + 2 * QP_PANEL;              // 2 buffers x 2 panels
constexpr int OFF_BAR = OFF_P + 2 * 2 * QP_PANEL;
constexpr int OFF_RED = OFF_BAR + 256;                    // [2][4][NQ] floats
constexpr int SMEM_BYTES = OFF_RED + 2 * 4 * NQ * 4 + 1024;
constexpr int TMEM_COLS = 64;
constexpr float RESCALE_THRESHOLD = 8.f;   // log2 units

struct Params {
  const bf16* q;
  const int* block_tables;
  const int* seq_lens;
  float* part_o;
  float* part_ml;
  unsigned int* status;
  int Hq, Hkv, G, block_size, max_blocks, window;
  float scale_log2;
};

__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

constexpr int kMinSplitTiles = 16;     // 2048 cached tokens per KV split at least

__global__ void __launch_bounds__(192, 1)
paged_attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                            const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* k_full = bars + 0;    // [NS]
  uint64_t* v_full = bars + 3;    // [NS]
  uint64_t* kv_empty = bars + 6;  // [NS]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_free = bars + 11;   // [2]
  uint64_t* p_ready = bars + 13;  // [2]
  uint64_t* p_free = bars + 15;   // [2]
  uint64_t* o_done = bars + 17;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_red = reinterpret_cast<float*>(smem + OFF_RED);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};
  const int r = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z, nsp = gridDim.z;
  const int G = p.G;
  const int L = p.seq_lens[r];
  const int lo = p.window > 0 ? max(0, L - p.window) : 0;
  const int tile_first = lo / TT;
  const int tiles_total = (L + TT - 1) / TT - tile_first;
  // a row uses as many of the launch's KV splits as it has pieces of kMinSplitTiles tiles: long rows are cut finer
  // than short ones, so the CTAs of a batch with mixed context lengths carry similar amounts of work
  const int nsp_r = max(1, min(nsp, (tiles_total + kMinSplitTiles - 1) / kMinSplitTiles));
  const int per = (tiles_total + nsp_r - 1) / nsp_r;
  const int t_begin = tile_first + sp * per;
  const int n_tiles = sp < nsp_r ? max(0, min(per, tile_first + tiles_total - t_begin)) : 0;

  if (n_tiles == 0) {   // CTA-uniform: nothing to do for this split
    if (threadIdx.x < G) {
      const size_t idx = ((size_t)r * p.Hq + kvh * G + threadIdx.x) * nsp + sp;
      p.part_ml[idx * 2] = -INFINITY;
      p.part_ml[idx * 2 + 1] = 0.f;
    }
    for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
      const size_t idx = ((size_t)r * p.Hq + kvh * G + i / D) * nsp + sp;
      p.part_o[idx * D + (i % D)] = 0.f;
    }
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_free[b], 128);
      mbar_init(&p_ready[b], 128);
      mbar_init(&p_free[b], 1);
    }
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  // Q^T operand (rows g < G, pre-scaled) and zeroed P buffers
  for (int i = threadIdx.x; i < (2 * QP_PANEL + 4 * QP_PANEL) / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem + OFF_Q)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    const float v = __bfloat162float(p.q[((size_t)r * p.Hq + kvh * G + g) * D + d]) * p.scale_log2;
    *reinterpret_cast<bf16*>(smem + OFF_Q + (d >> 6) * QP_PANEL + sw128_offset(g, (d & 63) * 2)) = __float2bfloat16(v);
  }
  fence_async_smem();
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tO = tmem_base + 32;
  const uint32_t aK = smem_u32(smem + OFF_K), aV = smem_u32(smem + OFF_V);
  const uint32_t aQ = smem_u32(smem + OFF_Q), aP = smem_u32(smem + OFF_P);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const int* bt = p.block_tables + (size_t)r * p.max_blocks;
      for (int i = 0; i < n_tiles; ++i) {
        const int s = i % NS;
        if (i >= NS) mbar_wait(&kv_empty[s], ((i / NS) - 1) & 1, ctx, 0x10 + s);
        const int tok0 = (t_begin + i) * TT;
        int blk[2], off[2];
#pragma unroll
        for (int hfl = 0; hfl < 2; ++hfl) {
          const int tok = tok0 + hfl * 64;
          const int bi = min(tok / p.block_size, p.max_blocks - 1);
          blk[hfl] = bt[bi];
          off[hfl] = tok % p.block_size;
        }
        mbar_expect_tx(&k_full[s], TILE_BYTES);
#pragma unroll
        for (int hfl = 0; hfl < 2; ++hfl)
#pragma unroll
          for (int pn = 0; pn < 2; ++pn)
            tma_load_4d(smem + OFF_K + s * TILE_BYTES + pn * PANEL + hfl * 8192, &tmK, &k_full[s], pn * 64, kvh,
                        off[hfl], blk[hfl]);
        mbar_expect_tx(&v_full[s], TILE_BYTES);
#pragma unroll
        for (int hfl = 0; hfl < 2; ++hfl)
#pragma unroll
          for (int pn = 0; pn < 2; ++pn)
            tma_load_4d(smem + OFF_V + s * TILE_BYTES + pn * PANEL + hfl * 8192, &tmV, &v_full[s], pn * 64, kvh,
                        off[hfl], blk[hfl]);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idescS = make_idesc_bf16(128, NQ, false, false);
      constexpr uint32_t idescO = make_idesc_bf16(128, NQ, true, false);
      auto issue_pv = [&](int j) {
        const int s = j % NS, b = j & 1;
        mbar_wait(&v_full[s], (j / NS) & 1, ctx, 0x20 + s);
        mbar_wait(&p_ready[b], (j >> 1) & 1, ctx, 0x30 + b);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < TT / 16; ++kk)
          umma_ss(tO, make_desc_mnmajor_sw128(aV + s * TILE_BYTES + kk * 2048, PANEL),
                  make_desc_kmajor_sw128(aP + b * 2 * QP_PANEL + (kk >> 2) * QP_PANEL + (kk & 3) * 32), idescO,
                  (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&kv_empty[s]);
        umma_commit(&p_free[b]);
      };
      for (int i = 0; i < n_tiles; ++i) {
        const int s = i % NS, b = i & 1;
        mbar_wait(&k_full[s], (i / NS) & 1, ctx, 0x40 + s);
        if (i >= 2) mbar_wait(&s_free[b], ((i >> 1) - 1) & 1, ctx, 0x50 + b);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_ss(tmem_base + b * NQ, make_desc_kmajor_sw128(aK + s * TILE_BYTES + (kk >> 2) * PANEL + (kk & 3) * 32),
                  make_desc_kmajor_sw128(aQ + (kk >> 2) * QP_PANEL + (kk & 3) * 32), idescS, kk > 0 ? 1u : 0u);
        umma_commit(&s_full[b]);
        if (i > 0) issue_pv(i - 1);
      }
      issue_pv(n_tiles - 1);
      umma_commit(o_done);
    }
  } else {
    // ---------------- softmax warps: thread <-> token row of the tile ----------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_bits = (uint32_t)(quad * 32) << 16;
    const int sw = warp - 2;                 // 0..3, slot in the reduction buffer
    float m_ref[NQ], l_part[NQ];
#pragma unroll
    for (int g = 0; g < NQ; ++g) { m_ref[g] = -INFINITY; l_part[g] = 0.f; }
    for (int i = 0; i < n_tiles; ++i) {
      const int b = i & 1;
      const int tok = (t_begin + i) * TT + row;
      const bool valid = tok >= lo && tok < L;
      mbar_wait(&s_full[b], (i >> 1) & 1, ctx, 0x60 + b);
      tc_fence_after();
      uint32_t sr[16];
      tmem_ld_x16(tmem_base + b * NQ + lane_bits, sr);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_free[b]);
      float sv[NQ];
      float* red = s_red + b * 4 * NQ;
#pragma unroll
      for (int g = 0; g < NQ; ++g) {
        if (g < G) {
          sv[g] = valid ? __uint_as_float(sr[g]) : -INFINITY;
          const float wm = warp_max(sv[g]);
          if (lane == 0) red[sw * NQ + g] = wm;
        }
      }
      named_bar_sync(1, 128);
      bool rescale = false;
      float alpha[NQ];
#pragma unroll
      for (int g = 0; g < NQ; ++g) {
        alpha[g] = 1.f;
        if (g < G) {
          const float mt = fmaxf(fmaxf(red[g], red[NQ + g]), fmaxf(red[2 * NQ + g], red[3 * NQ + g]));
          if (mt > m_ref[g] + RESCALE_THRESHOLD || (m_ref[g] == -INFINITY && mt > -INFINITY)) {
            alpha[g] = (m_ref[g] == -INFINITY) ? 0.f : exp2f(m_ref[g] - mt);
            m_ref[g] = mt;
            rescale = true;
          }
        }
      }
      if (rescale && i > 0) {   // CTA-uniform: every thread saw the same maxima
        mbar_wait(&p_free[(i - 1) & 1], ((i - 1) >> 1) & 1, ctx, 0x70);
        tc_fence_after();
        uint32_t orow[16];
        tmem_ld_x16(tO + lane_bits, orow);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < NQ; ++g)
          if (g < G) orow[g] = __float_as_uint(__uint_as_float(orow[g]) * alpha[g]);
        tmem_st_x16(tO + lane_bits, orow);
        tmem_st_wait();
      }
      if (i >= 2) mbar_wait(&p_free[b], ((i >> 1) - 1) & 1, ctx, 0x78 + b);
      uint8_t* pb = smem + OFF_P + b * 2 * QP_PANEL + (row >> 6) * QP_PANEL;
#pragma unroll
      for (int g = 0; g < NQ; ++g) {
        if (g < G) {
          const float pv = (valid && m_ref[g] > -INFINITY) ? exp2f(sv[g] - m_ref[g]) : 0.f;
          const bf16 pq = __float2bfloat16(pv);
          l_part[g] = l_part[g] * alpha[g] + __bfloat162float(pq);
          *reinterpret_cast<bf16*>(pb + sw128_offset(g, (row & 63) * 2)) = pq;
        }
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&p_ready[b]);
    }
    // ---- epilogue: O^T rows (dims) and the row sums ----
    float* red = s_red;   // [4][NQ]
    named_bar_sync(1, 128);
#pragma unroll
    for (int g = 0; g < NQ; ++g) {
      if (g < G) {
        const float ws = warp_sum(l_part[g]);
        if (lane == 0) red[sw * NQ + g] = ws;
      }
    }
    mbar_wait(o_done, 0, ctx, 0x80);
    tc_fence_after();
    uint32_t orow[16];
    tmem_ld_x16(tO + lane_bits, orow);
    tmem_ld_wait();
    named_bar_sync(1, 128);
#pragma unroll
    for (int g = 0; g < NQ; ++g) {
      if (g < G) {
        const size_t idx = ((size_t)r * p.Hq + kvh * G + g) * nsp + sp;
        p.part_o[idx * D + row] = __uint_as_float(orow[g]);
        if (row == 0) {
          p.part_ml[idx * 2] = m_ref[g] * 0.6931471805599453f;
          p.part_ml[idx * 2 + 1] = red[g] + red[NQ + g] + red[2 * NQ + g] + red[3 * NQ + g];
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

__global__ void __launch_bounds__(128)
paged_attn_combine_tc(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ o,
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
    acc += part_o[(rh * nsp + s) * D + t] * w;
  }
  o[rh * D + t] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
}

}  // namespace pad
}  // namespace hmf

using namespace hmf;
using namespace hmf::pad;

// q [R, Hq, 128] bf16; caches [num_blocks, block_size, Hkv, 128] bf16 (block_size a multiple of 64);
// block_tables [R, max_blocks] int32; seq_lens [R] int32 (including the token just appended);
// part_o [R, Hq, splits, 128] fp32 and part_ml [R, Hq, splits, 2] fp32 are scratch; o [R, Hq, 128] bf16.
HMF_API int hmf_paged_attention_decode_tc(const void* q, const void* kc, const void* vc, const int* block_tables,
                                          const int* seq_lens, void* o, float* part_o, float* part_ml, int R, int Hq,
                                          int Hkv, int Dh, int block_size, int num_blocks, int max_blocks, int splits,
                                          int window, float scale, cudaStream_t st) {
  HMF_REQUIRE(Dh == D, "paged attention (tcgen05): head dim %d unsupported (128)", Dh);
  HMF_REQUIRE(Hq % Hkv == 0 && Hq / Hkv <= NQ, "paged attention (tcgen05): group size %d unsupported (<= %d)",
              Hq / Hkv, NQ);
  HMF_REQUIRE(block_size % 64 == 0 && block_size <= 256, "paged attention (tcgen05): block size %d unsupported",
              block_size);
  HMF_REQUIRE(splits >= 1 && splits <= 64, "paged attention (tcgen05): splits=%d out of range", splits);
  if (R == 0) return HMF_OK;
  CUtensorMap tmK, tmV;
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)block_size, (uint64_t)num_blocks};
  uint64_t strides[4] = {2, (uint64_t)D * 2, (uint64_t)Hkv * D * 2, (uint64_t)block_size * Hkv * D * 2};
  uint32_t box[4] = {64, 1, 64, 1};
  int rc;
  if ((rc = make_tensor_map(&tmK, kc, 0, 4, dims, strides, box, 3)) != HMF_OK) return rc;
  if ((rc = make_tensor_map(&tmV, vc, 0, 4, dims, strides, box, 3)) != HMF_OK) return rc;
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(paged_attn_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        SMEM_BYTES));
    configured = true;
  }
  Params p;
  p.q = (const bf16*)q;
  p.block_tables = block_tables;
  p.seq_lens = seq_lens;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.status = status_ptr();
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.G = Hq / Hkv;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(R, Hkv, splits);
  paged_attn_decode_tc_kernel<<<grid, 192, SMEM_BYTES, st>>>(tmK, tmV, p);
  HMF_CHECK_CUDA(cudaGetLastError());
  paged_attn_combine_tc<<<R * Hq, 128, 0, st>>>(part_o, part_ml, (bf16*)o, splits);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
