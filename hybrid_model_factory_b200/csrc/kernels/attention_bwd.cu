// Flash attention backward for sm_100a (tcgen05 + TMEM + TMA), as three kernels:
//
//   1. delta[b,h,t] = sum_d dO * O                                   (memory bound)
//   2. dQ kernel   : one CTA per 128-row query tile; loops over key tiles of 64:
//                      S = Q K^T, dP = dO V^T  ->  dS = P o (dP - delta) * scale  ->  dQ += dS K
//   3. dK/dV kernel: one CTA per 128-key tile of a KV head; loops over the query heads of the group
//                    and their query tiles of 64:
//                      S^T = K Q^T, dP^T = V dO^T  ->  P^T, dS^T  ->  dV += P^T dO, dK += dS^T Q
//
// Both kernels keep every accumulator in tensor memory, recompute P from the saved log-sum-exp,
// write the bf16 probabilities / score gradients back into tensor memory over S / dP
// (tcgen05.st) and feed them to the next MMA as the TMEM A operand.  No atomics: dQ is owned by
// the query-tile CTA and dK/dV by the key-tile CTA (the GQA group sum happens in the accumulator).
// Masks follow the forward kernel: key visible <=> lo <= q_pos - k_pos < hi.
#include <math.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace attn_bwd {

using bf16 = __nv_bfloat16;
constexpr float kLog2e = 1.4426950408889634f;

struct Params {
  const float* lse;    // [B, Hq, Tq]
  const float* delta;  // [B, Hq, Tq]
  const int* q_pos;    // optional [B, Tq]
  bf16* dq;            // [B, Tq, Hq, D]
  bf16* dk;            // [B, Tk, Hkv, D]
  bf16* dv;            // [B, Tk, Hkv, D]
  int B, Tq, Tk, Hq, Hkv;
  int lo, hi, q_off;
  float scale, scale_log2;
  unsigned int* status;
};

// ------------------------------------------------------------------------------------
// delta = rowsum(dO * O); 16 lanes per row of D <= 128 (D % 8 == 0)
// ------------------------------------------------------------------------------------
// With a gradient on the log-sum-exp output (its derivative w.r.t. the scores is P) the score gradient is
// dS = P o (dP - delta + dlse); it enters here as delta - dlse, so the main kernels are unchanged.
__global__ void delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ d_o, const float* __restrict__ dlse,
                             float* __restrict__ delta, int B, int T, int H, int D) {
  const int lanes = D / 8;  // 8 or 16
  const int rows_per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long row = wid * rows_per_warp + lane / lanes;  // index over (b, t, h)
  const long long total = (long long)B * T * H;
  float s = 0.f;
  if (row < total) {
    const int c = (lane % lanes) * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(o + row * D + c);
    const uint4 g = *reinterpret_cast<const uint4*>(d_o + row * D + c);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(gh[i]);
      s += x.x * y.x + x.y * y.y;
    }
  }
  for (int off = lanes / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (row < total && (lane % lanes) == 0) {
    const long long h = row % H, bt = row / H;
    const long long t = bt % T, b = bt / T;
    const long long idx = (b * H + h) * T + t;
    delta[idx] = dlse != nullptr ? s - dlse[idx] : s;
  }
}

// ------------------------------------------------------------------------------------
// dQ kernel
// ------------------------------------------------------------------------------------
constexpr int BM = 128;  // query rows per CTA
constexpr int BN = 64;   // keys per inner tile

template <int D>
struct SmemDQ {
  static constexpr int NST = 3;                 // K and V rings
  static constexpr int QP = BM * 128;           // one 64-wide panel of Q / dO
  static constexpr int KP = BN * 128;           // one 64-wide panel of K / V
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int KV_BYTES = BN * D * 2;
  static constexpr int OFF_DO = Q_BYTES;
  static constexpr int OFF_K = 2 * Q_BYTES;
  static constexpr int OFF_V = OFF_K + NST * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + NST * KV_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256;
};

template <int N>
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[N]) {
  if constexpr (N == 32) tmem_ld_x32(taddr, r);
  else if constexpr (N == 16) tmem_ld_x16(taddr, r);
  else tmem_ld_x8(taddr, r);
}
template <int N>
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[N]) {
  if constexpr (N == 32) tmem_st_x32(taddr, r);
  else if constexpr (N == 16) tmem_st_x16(taddr, r);
  else tmem_st_x8(taddr, r);
}

constexpr int NWG = 2;                        // softmax warpgroups per CTA: each takes 64 / NWG columns of a tile
constexpr int NSOFT = NWG * 128;              // softmax threads
constexpr int NTHR = 64 + NSOFT;              // + TMA warp + MMA warp
constexpr int WCOLS = 64 / NWG;               // 16 fp32 columns per thread and tile

template <int D>
__global__ void __launch_bounds__(NTHR + 32, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const Params p) {
  // One CTA per SM: S / dP double-buffered in tensor memory so the MMAs of tile j+1 overlap the softmax of tile j;
  // K and V travel through 3-stage rings; NWG softmax warpgroups split the 64 key columns of a tile.
  // Q and dO (reused by every key tile) are copied once into tensor memory as bf16 A operands, so the S and dP
  // MMAs read only the 64-row K / V tile from shared memory (the SS form with a 128-row A operand is bound by
  // shared-memory bandwidth, not by the tensor pipe).
  // Tensor-memory map (512 columns): Q [0,64) dO [64,128) S0 S1 [128,256) dP0 dP1 [256,384) dQ [384,384+D).
  using L = SmemDQ<D>;
  constexpr int NST = L::NST;
  constexpr int TMEM_COLS = 512;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + L::OFF_DO;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* qdo_full = bars + 0;
  uint64_t* k_full = bars + 1;              // [NST]
  uint64_t* k_empty = bars + 1 + NST;       // [NST]
  uint64_t* v_full = bars + 1 + 2 * NST;    // [NST]
  uint64_t* v_empty = bars + 1 + 3 * NST;   // [NST]
  uint64_t* sdp_full = bars + 1 + 4 * NST;  // [2]
  uint64_t* ds_full = bars + 3 + 4 * NST;   // [2]
  uint64_t* dq_done = bars + 5 + 4 * NST;
  uint64_t* a_ready = bars + 6 + 4 * NST;   // Q / dO operands are in tensor memory
  uint64_t* t_free = bars + 7 + 4 * NST;    // [2] dS of a buffer consumed by the dQ MMAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9 + 4 * NST);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};
  const int h = blockIdx.x;
  const int qt = (int)gridDim.y - 1 - (int)blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q0 = qt * BM;
  const int rows_valid = min(BM, p.Tq - q0);

  long long pmin, pmax;
  if (p.q_pos) {
    pmin = p.q_pos[(size_t)b * p.Tq + q0];
    pmax = p.q_pos[(size_t)b * p.Tq + q0 + rows_valid - 1];
  } else {
    pmin = (long long)q0 + p.q_off;
    pmax = (long long)q0 + rows_valid - 1 + p.q_off;
  }
  long long kmin = pmin - (long long)p.hi + 1;
  if (kmin < 0) kmin = 0;
  long long kmax = pmax - (long long)p.lo;
  if (kmax > p.Tk - 1) kmax = p.Tk - 1;
  const int j0 = (int)(kmin / BN);
  const int n_tiles = (kmax >= kmin) ? (int)(kmax / BN) - j0 + 1 : 0;

  if (threadIdx.x == 0) {
    if ((smem_u32(smem) & 1023u) != 0) report_error(p.status, kBadArgument, 0xA1);
    mbar_init(qdo_full, 1);
    for (int s = 0; s < NST; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sdp_full[s], 1);
      mbar_init(&t_free[s], 1);
      mbar_init(&ds_full[s], NSOFT);
    }
    mbar_init(dq_done, 1);
    mbar_init(a_ready, NSOFT);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tQ = tmem_base, tDO = tmem_base + 64;
  auto tS = [&](int s) -> uint32_t { return tmem_base + 128u + (uint32_t)s * 64u; };
  auto tDP = [&](int s) -> uint32_t { return tmem_base + 256u + (uint32_t)s * 64u; };
  const uint32_t tDQ = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(qdo_full, 2 * L::Q_BYTES);
#pragma unroll
      for (int pn = 0; pn < D / 64; ++pn) {
        tma_load_4d(sQ + pn * L::QP, &tmQ, qdo_full, pn * 64, h, q0, b);
        tma_load_4d(sDO + pn * L::QP, &tmDO, qdo_full, pn * 64, h, q0, b);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % NST;
        const int k0 = (j0 + j) * BN;
        if (j >= NST) mbar_wait(&k_empty[s], ((j / NST) - 1) & 1, ctx, 0x110 + s);
        mbar_expect_tx(&k_full[s], L::KV_BYTES);
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn)
          tma_load_4d(sK + s * L::KV_BYTES + pn * L::KP, &tmK, &k_full[s], pn * 64, hkv, k0, b);
        if (j >= NST) mbar_wait(&v_empty[s], ((j / NST) - 1) & 1, ctx, 0x120 + s);
        mbar_expect_tx(&v_full[s], L::KV_BYTES);
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn)
          tma_load_4d(sV + s * L::KV_BYTES + pn * L::KP, &tmV, &v_full[s], pn * 64, hkv, k0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idescS = make_idesc_bf16(BM, BN, false, false);
      auto issue_SdP = [&](int j) {
        const int s = j & 1, ks = j % NST;
        const uint32_t aK = smem_u32(sK + ks * L::KV_BYTES), aV = smem_u32(sV + ks * L::KV_BYTES);
        mbar_wait(&k_full[ks], (j / NST) & 1, ctx, 0x140 + ks);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t bd = make_desc_kmajor_sw128(aK + (kk / 4) * L::KP + (kk % 4) * 32);
          umma_ts(tS(s), tQ + kk * 8, bd, idescS, kk > 0 ? 1u : 0u);
        }
        mbar_wait(&v_full[ks], (j / NST) & 1, ctx, 0x150 + ks);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t bd = make_desc_kmajor_sw128(aV + (kk / 4) * L::KP + (kk % 4) * 32);
          umma_ts(tDP(s), tDO + kk * 8, bd, idescS, kk > 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[ks]);
        umma_commit(&sdp_full[s]);
      };
      // S / dP issuer; the dQ MMAs are issued by a second thread (warp 2 + 4 NWG)
      mbar_wait(a_ready, 0, ctx, 0x130);
      tc_fence_after();
      for (int j = 0; j < n_tiles; ++j) {
        if (j >= 2) mbar_wait(&t_free[j & 1], ((j >> 1) - 1) & 1, ctx, 0x1A0 + (j & 1));
        issue_SdP(j);
      }
    }
  } else if (warp == 2 + 4 * NWG) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idescDQ = make_idesc_bf16(BM, D, false, true);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1, ks = j % NST;
        const uint32_t aK = smem_u32(sK + ks * L::KV_BYTES);
        mbar_wait(&k_full[ks], (j / NST) & 1, ctx, 0x1B0 + ks);
        mbar_wait(&ds_full[s], (j >> 1) & 1, ctx, 0x160 + s);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t bd = make_desc_mnmajor_sw128(aK + kk * 2048, L::KP);
          umma_ts(tDQ, tS(s) + kk * 8, bd, idescDQ, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&k_empty[ks]);
        umma_commit(&t_free[s]);
      }
      umma_commit(dq_done);
    }
  } else {
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;      // warpgroup: key columns [WCOLS part, WCOLS part + WCOLS)
    const int r = quad * 32 + lane;
    const int row = q0 + r;
    const bool row_ok = row < p.Tq;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    long long prow = 0;
    float lse2 = INFINITY, delta = 0.f;
    if (row_ok) {
      prow = p.q_pos ? (long long)p.q_pos[(size_t)b * p.Tq + row] : (long long)row + p.q_off;
      const float l = p.lse[((size_t)b * p.Hq + h) * p.Tq + row];
      lse2 = (l == -INFINITY) ? INFINITY : l * kLog2e;
      delta = p.delta[((size_t)b * p.Hq + h) * p.Tq + row];
    }
    if (n_tiles > 0) {
      // this thread's slice of its Q and dO rows: swizzled shared memory -> packed bf16 pairs in tensor memory
      constexpr int EC = D / NWG;                  // elements per thread and operand (32 or 16)
      mbar_wait(qdo_full, 0, ctx, 0x190);
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint8_t* src = which == 0 ? sQ : sDO;
        uint32_t regs[EC / 2];
#pragma unroll
        for (int c8 = 0; c8 < EC / 8; ++c8) {
          const int col = part * EC + c8 * 8;      // first element of a 16-byte chunk
          const uint4 u = *reinterpret_cast<const uint4*>(src + (col >> 6) * L::QP +
                                                          sw128_offset((uint32_t)r, (uint32_t)(col & 63) * 2));
          regs[c8 * 4 + 0] = u.x; regs[c8 * 4 + 1] = u.y; regs[c8 * 4 + 2] = u.z; regs[c8 * 4 + 3] = u.w;
        }
        const uint32_t dst = (which == 0 ? tQ : tDO) + lane_off + part * (EC / 2);
        tmem_st_n<EC / 2>(dst, regs);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(a_ready);
    }
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      const int k0 = (j0 + j) * BN;
      mbar_wait(&sdp_full[s], (j >> 1) & 1, ctx, 0x170 + s);
      tc_fence_after();
      const bool full_vis = (pmin - (long long)(k0 + BN - 1) >= (long long)p.lo) &&
                            (pmax - (long long)k0 < (long long)p.hi) && (k0 + BN <= p.Tk) &&
                            (rows_valid == BM);
      long long chi = prow - k0 - (long long)p.lo;
      long long clo = prow - k0 - (long long)p.hi;
      const long long cend = (long long)p.Tk - k0 - 1;
      if (chi > cend) chi = cend;
      if (!row_ok) chi = -1;
      const int ichi = (int)max(-1ll, min(chi, 1000ll));
      const int iclo = (int)max(-1ll, min(clo, 1000ll));
      uint32_t sv[WCOLS], dp[WCOLS], pk[WCOLS / 2];
      tmem_ld_n<WCOLS>(tS(s) + lane_off + part * WCOLS, sv);
      tmem_ld_n<WCOLS>(tDP(s) + lane_off + part * WCOLS, dp);
      tmem_ld_wait();
      if (full_vis) {
#pragma unroll
        for (int c = 0; c < WCOLS; c += 2) {
          const float p0 = exp2f(fmaf(__uint_as_float(sv[c]), p.scale_log2, -lse2));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[c + 1]), p.scale_log2, -lse2));
          pk[c >> 1] = pack_bf16x2(p0 * (__uint_as_float(dp[c]) - delta) * p.scale,
                                   p1 * (__uint_as_float(dp[c + 1]) - delta) * p.scale);
        }
      } else {
#pragma unroll
        for (int c = 0; c < WCOLS; c += 2) {
          float d2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int cc = part * WCOLS + c + e;
            const bool vis = (cc <= ichi) && (cc > iclo);
            const float pr = vis ? exp2f(fmaf(__uint_as_float(sv[c + e]), p.scale_log2, -lse2)) : 0.f;
            d2[e] = pr * (__uint_as_float(dp[c + e]) - delta) * p.scale;
          }
          pk[c >> 1] = pack_bf16x2(d2[0], d2[1]);
        }
      }
      // every warpgroup has read its fp32 columns before the packed dS overwrites columns 0..31
      asm volatile("bar.sync 2, %0;" ::"n"(NSOFT) : "memory");
      tmem_st_n<WCOLS / 2>(tS(s) + lane_off + part * (WCOLS / 2), pk);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ds_full[s]);
    }
    if (n_tiles > 0) {
      mbar_wait(dq_done, 0, ctx, 0x180);
      tc_fence_after();
    }
    // warpgroup `part` writes output columns [part * D / NWG, (part + 1) * D / NWG)
    bf16* orow = p.dq + (((size_t)b * p.Tq + row) * p.Hq + h) * D;
    constexpr int OC = D / NWG;       // 32 (D = 128) or 16 (D = 64) columns
    {
      uint32_t o[OC];
      if (n_tiles > 0) {
#pragma unroll
        for (int c32 = 0; c32 < (OC + 31) / 32; ++c32) {
          constexpr int W = OC < 32 ? OC : 32;
          uint32_t (&oo)[W] = *reinterpret_cast<uint32_t (*)[W]>(&o[c32 * 32]);
          tmem_ld_n<W>(tDQ + lane_off + part * OC + c32 * 32, oo);
        }
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < OC; ++i) o[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < OC / 8; ++i) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[8 * i + 0]), __uint_as_float(o[8 * i + 1]));
          w.y = pack_bf16x2(__uint_as_float(o[8 * i + 2]), __uint_as_float(o[8 * i + 3]));
          w.z = pack_bf16x2(__uint_as_float(o[8 * i + 4]), __uint_as_float(o[8 * i + 5]));
          w.w = pack_bf16x2(__uint_as_float(o[8 * i + 6]), __uint_as_float(o[8 * i + 7]));
          reinterpret_cast<uint4*>(orow + part * OC)[i] = w;
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

// ------------------------------------------------------------------------------------
// dK / dV kernel
// ------------------------------------------------------------------------------------
constexpr int KM = 128;  // keys per CTA
constexpr int QN = 64;   // query rows per inner tile

template <int D>
struct SmemDKV {
  static constexpr int KPANEL = KM * 128;
  static constexpr int QPANEL = QN * 128;
  static constexpr int K_BYTES = KM * D * 2;
  static constexpr int Q_BYTES = QN * D * 2;
  static constexpr int OFF_V = K_BYTES;
  static constexpr int NST = 4;                        // [Q | dO] ring: deep enough to hide the TMA latency
  static constexpr int OFF_Q = 2 * K_BYTES;
  static constexpr int STAGE = 2 * Q_BYTES;
  static constexpr int OFF_ROW = OFF_Q + NST * STAGE;  // lse2 / delta / qpos staging: 2 x 3 x 64 x 4
  static constexpr int OFF_BAR = OFF_ROW + 2 * 3 * QN * 4;
  static constexpr int TOTAL = OFF_BAR + 256;
};

// Iterates the (query head of the group, query tile) pairs that can see the key tile [k0, k0+KM).
struct QTileIter {
  int G, nq_tiles, i_lo, i_hi;  // contiguous positions: tiles [i_lo, i_hi]
  __device__ int count() const { return (i_hi >= i_lo) ? G * (i_hi - i_lo + 1) : 0; }
  __device__ void get(int it, int& g, int& i) const {
    const int per = i_hi - i_lo + 1;
    g = it / per;
    i = i_lo + it % per;
  }
};

template <int D>
__global__ void __launch_bounds__(NTHR + 32, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const Params p) {
  using L = SmemDKV<D>;
  constexpr int TMEM_COLS = 512;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sQ = smem + L::OFF_Q;
  float* s_row = reinterpret_cast<float*>(smem + L::OFF_ROW);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  constexpr int NST = L::NST;
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;              // [NST]
  uint64_t* q_empty = bars + 1 + NST;       // [NST]
  uint64_t* st_full = bars + 1 + 2 * NST;   // [2]
  uint64_t* pds_full = bars + 3 + 2 * NST;  // [2]
  uint64_t* acc_done = bars + 5 + 2 * NST;
  uint64_t* t_free = bars + 6 + 2 * NST;    // [2] P^T / dS^T of a buffer consumed by the accumulate MMAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8 + 2 * NST);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};
  const int kt = blockIdx.x;  // ascending: early key tiles (most work under a causal mask) first
  const int hkv = blockIdx.y;
  const int b = blockIdx.z;
  const int k0 = kt * KM;
  const int keys_valid = min(KM, p.Tk - k0);
  const int G = p.Hq / p.Hkv;
  const int nq_tiles = (p.Tq + QN - 1) / QN;

  // query tiles that may see keys [k0, k0+keys_valid): positions in [k0+lo, k0+keys_valid-1+hi-1]
  QTileIter iter;
  iter.G = G;
  iter.nq_tiles = nq_tiles;
  if (p.q_pos) {
    iter.i_lo = 0;  // explicit positions: visit every tile, masks do the rest
    iter.i_hi = nq_tiles - 1;
  } else {
    long long rmin = (long long)k0 + p.lo - p.q_off;
    long long rmax = (long long)k0 + keys_valid - 1 + (long long)p.hi - 1 - p.q_off;
    if (rmin < 0) rmin = 0;
    if (rmax > p.Tq - 1) rmax = p.Tq - 1;
    iter.i_lo = (int)(rmin / QN);
    iter.i_hi = (rmax >= rmin) ? (int)(rmax / QN) : iter.i_lo - 1;
  }
  const int n_it = iter.count();

  if (threadIdx.x == 0) {
    if ((smem_u32(smem) & 1023u) != 0) report_error(p.status, kBadArgument, 0xA2);
    mbar_init(kv_full, 1);
    for (int s = 0; s < NST; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&st_full[s], 1);
      mbar_init(&t_free[s], 1);
      mbar_init(&pds_full[s], NSOFT);
    }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tST = [&](int s) -> uint32_t { return tmem_base + (uint32_t)s * 64u; };
  auto tDPT = [&](int s) -> uint32_t { return tmem_base + 128u + (uint32_t)s * 64u; };
  const uint32_t tDV = tmem_base + 256, tDK = tmem_base + 256 + D;

  if (warp == 0) {
    if (lane == 0 && n_it > 0) {
      mbar_expect_tx(kv_full, 2 * L::K_BYTES);
#pragma unroll
      for (int pn = 0; pn < D / 64; ++pn) {
        tma_load_4d(sK + pn * L::KPANEL, &tmK, kv_full, pn * 64, hkv, k0, b);
        tma_load_4d(sV + pn * L::KPANEL, &tmV, kv_full, pn * 64, hkv, k0, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int s = it % NST;
        int g, i;
        iter.get(it, g, i);
        const int h = hkv * G + g;
        if (it >= NST) mbar_wait(&q_empty[s], ((it / NST) - 1) & 1, ctx, 0x210 + s);
        mbar_expect_tx(&q_full[s], L::STAGE);
        uint8_t* dst = sQ + s * L::STAGE;
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn) {
          tma_load_4d(dst + pn * L::QPANEL, &tmQ, &q_full[s], pn * 64, h, i * QN, b);
          tma_load_4d(dst + L::Q_BYTES + pn * L::QPANEL, &tmDO, &q_full[s], pn * 64, h, i * QN, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idescST = make_idesc_bf16(KM, QN, false, false);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
      auto issue_SdP = [&](int it) {
        const int s = it & 1, qs = it % NST;
        mbar_wait(&q_full[qs], (it / NST) & 1, ctx, 0x220 + qs);
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ + qs * L::STAGE);
        const uint32_t aDO = aQ + L::Q_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t ad = make_desc_kmajor_sw128(aK + (kk / 4) * L::KPANEL + (kk % 4) * 32);
          const uint64_t bd = make_desc_kmajor_sw128(aQ + (kk / 4) * L::QPANEL + (kk % 4) * 32);
          umma_ss(tST(s), ad, bd, idescST, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t ad = make_desc_kmajor_sw128(aV + (kk / 4) * L::KPANEL + (kk % 4) * 32);
          const uint64_t bd = make_desc_kmajor_sw128(aDO + (kk / 4) * L::QPANEL + (kk % 4) * 32);
          umma_ss(tDPT(s), ad, bd, idescST, kk > 0 ? 1u : 0u);
        }
        umma_commit(&st_full[s]);
      };
      // S^T / dP^T issuer; the accumulate MMAs (dV, dK) are issued by a second thread (warp 2 + 4 NWG) so that the
      // two instruction streams do not serialise behind one issuing thread
      mbar_wait(kv_full, 0, ctx, 0x230);
      for (int it = 0; it < n_it; ++it) {
        if (it >= 2) mbar_wait(&t_free[it & 1], ((it >> 1) - 1) & 1, ctx, 0x270 + (it & 1));
        issue_SdP(it);
      }
    }
  } else if (warp == 2 + 4 * NWG) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idescAcc = make_idesc_bf16(KM, D, false, true);
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1, qs = it % NST;
        mbar_wait(&q_full[qs], (it / NST) & 1, ctx, 0x280 + qs);
        mbar_wait(&pds_full[s], (it >> 1) & 1, ctx, 0x240 + s);
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ + qs * L::STAGE);
        const uint32_t aDO = aQ + L::Q_BYTES;
#pragma unroll
        for (int kk = 0; kk < QN / 16; ++kk) {
          const uint64_t bd = make_desc_mnmajor_sw128(aDO + kk * 2048, L::QPANEL);
          umma_ts(tDV, tST(s) + kk * 8, bd, idescAcc, (it > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < QN / 16; ++kk) {
          const uint64_t bd = make_desc_mnmajor_sw128(aQ + kk * 2048, L::QPANEL);
          umma_ts(tDK, tDPT(s) + kk * 8, bd, idescAcc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&q_empty[qs]);
        umma_commit(&t_free[s]);
      }
      umma_commit(acc_done);
    }
  } else {
    // NWG softmax warpgroups: each covers the 128 key rows (TMEM lane quadrant = warp % 4) and WCOLS of the 64
    // query columns of a tile.
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;
    const int r = quad * 32 + lane;  // key row
    const int tid = threadIdx.x - 64;  // 0..NSOFT-1
    const long long kpos = (long long)k0 + r;
    const bool key_ok = r < keys_valid;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    // query position window that sees this key: [kpos + lo, kpos + hi), clamped to int range
    const int vis_lo = (int)min(kpos + (long long)p.lo, 2147483647ll);
    const int vis_hi = (int)min(kpos + (long long)p.hi, 2147483647ll);
    // Per-tile row data (lse, delta, positions of the 64 queries) is staged in shared memory one tile ahead: the
    // global loads of tile it+1 are issued before the work of tile it and stored after it, so their latency is
    // off the critical path.
    auto load_rows = [&](int it, float& v0, int& v1) {
      int g, i;
      iter.get(it, g, i);
      const int h = hkv * G + g;
      const int q0 = i * QN;
      v0 = 0.f;
      v1 = -(1 << 30);
      if (tid < QN) {
        const int qi = q0 + tid;
        v0 = INFINITY;
        if (qi < p.Tq) {
          const float l = p.lse[((size_t)b * p.Hq + h) * p.Tq + qi];
          v0 = (l == -INFINITY) ? INFINITY : l * kLog2e;
          v1 = p.q_pos ? p.q_pos[(size_t)b * p.Tq + qi] : qi + p.q_off;
        }
      } else if (tid < 2 * QN) {
        const int qi = q0 + tid - QN;
        v0 = (qi < p.Tq) ? p.delta[((size_t)b * p.Hq + h) * p.Tq + qi] : 0.f;
      }
    };
    auto store_rows = [&](int it, float v0, int v1) {
      float* b_lse = s_row + (it & 1) * 3 * QN;
      if (tid < QN) {
        b_lse[tid] = v0;
        reinterpret_cast<int*>(b_lse + 2 * QN)[tid] = v1;
      } else if (tid < 2 * QN) {
        b_lse[QN + tid - QN] = v0;
      }
    };
    if (n_it > 0) {
      float v0;
      int v1;
      load_rows(0, v0, v1);
      store_rows(0, v0, v1);
    }
    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      int g, i;
      iter.get(it, g, i);
      const int q0 = i * QN;
      float* st_lse = s_row + s * 3 * QN;
      float* st_del = st_lse + QN;
      int* st_pos = reinterpret_cast<int*>(st_del + QN);
      float nv0 = 0.f;
      int nv1 = 0;
      if (it + 1 < n_it) load_rows(it + 1, nv0, nv1);      // in flight during this tile's work
      // every (key, query) pair of the tile visible?  (CTA-uniform: contiguous positions, full tile)
      const long long pmin = (long long)q0 + p.q_off, pmax = pmin + QN - 1;
      const bool full = p.q_pos == nullptr && keys_valid == KM && q0 + QN <= p.Tq &&
                        pmin - ((long long)k0 + KM - 1) >= (long long)p.lo && pmax - (long long)k0 < (long long)p.hi;
      asm volatile("bar.sync 1, %0;" ::"n"(NSOFT) : "memory");
      mbar_wait(&st_full[s], (it >> 1) & 1, ctx, 0x250 + s);
      tc_fence_after();
      {
        uint32_t sv[WCOLS], dp[WCOLS], pp[WCOLS / 2], pd[WCOLS / 2];
        tmem_ld_n<WCOLS>(tST(s) + lane_off + part * WCOLS, sv);
        tmem_ld_n<WCOLS>(tDPT(s) + lane_off + part * WCOLS, dp);
        tmem_ld_wait();
        if (full) {
#pragma unroll
          for (int c = 0; c < WCOLS; c += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(st_lse + part * WCOLS + c);
            const float4 d4 = *reinterpret_cast<const float4*>(st_del + part * WCOLS + c);
            const float p0 = exp2f(fmaf(__uint_as_float(sv[c + 0]), p.scale_log2, -l4.x));
            const float p1 = exp2f(fmaf(__uint_as_float(sv[c + 1]), p.scale_log2, -l4.y));
            const float p2 = exp2f(fmaf(__uint_as_float(sv[c + 2]), p.scale_log2, -l4.z));
            const float p3 = exp2f(fmaf(__uint_as_float(sv[c + 3]), p.scale_log2, -l4.w));
            pp[(c >> 1) + 0] = pack_bf16x2(p0, p1);
            pp[(c >> 1) + 1] = pack_bf16x2(p2, p3);
            pd[(c >> 1) + 0] = pack_bf16x2(p0 * (__uint_as_float(dp[c + 0]) - d4.x) * p.scale,
                                           p1 * (__uint_as_float(dp[c + 1]) - d4.y) * p.scale);
            pd[(c >> 1) + 1] = pack_bf16x2(p2 * (__uint_as_float(dp[c + 2]) - d4.z) * p.scale,
                                           p3 * (__uint_as_float(dp[c + 3]) - d4.w) * p.scale);
          }
        } else {
#pragma unroll
          for (int c = 0; c < WCOLS; c += 2) {
            float pr[2], ds[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int cc = part * WCOLS + c + e;
              const int pos = st_pos[cc];
              const bool vis = key_ok && pos >= vis_lo && pos < vis_hi;
              pr[e] = vis ? exp2f(fmaf(__uint_as_float(sv[c + e]), p.scale_log2, -st_lse[cc])) : 0.f;
              ds[e] = pr[e] * (__uint_as_float(dp[c + e]) - st_del[cc]) * p.scale;
            }
            pp[c >> 1] = pack_bf16x2(pr[0], pr[1]);
            pd[c >> 1] = pack_bf16x2(ds[0], ds[1]);
          }
        }
        // all 64 S^T / dP^T columns of these rows must have been read (by every warpgroup) before the packed
        // values overwrite columns 0..31
        asm volatile("bar.sync 2, %0;" ::"n"(NSOFT) : "memory");
        tmem_st_n<WCOLS / 2>(tST(s) + lane_off + part * (WCOLS / 2), pp);
        tmem_st_n<WCOLS / 2>(tDPT(s) + lane_off + part * (WCOLS / 2), pd);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&pds_full[s]);
      // the other row buffer was last read before this iteration's second barrier: free to overwrite
      if (it + 1 < n_it) store_rows(it + 1, nv0, nv1);
    }
    if (n_it > 0) {
      mbar_wait(acc_done, 0, ctx, 0x260);
      tc_fence_after();
    }
    {
      // warpgroups 0 .. NWG/2-1 write dV, the others dK; each a contiguous slice of the D columns
      constexpr int PER = NWG / 2;
      constexpr int OC = D / PER;          // columns per warpgroup (64 for D = 128)
      const int which = part / PER, sub = part % PER;
      bf16* base = which == 0 ? p.dv : p.dk;
      const uint32_t tacc = which == 0 ? tDV : tDK;
      bf16* orow = base + (((size_t)b * p.Tk + k0 + r) * p.Hkv + hkv) * D + sub * OC;
#pragma unroll
      for (int ch = 0; ch < OC / 32; ++ch) {
        uint32_t o[32];
        if (n_it > 0) {
          tmem_ld_x32(tacc + lane_off + sub * OC + ch * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (key_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[8 * i + 0]), __uint_as_float(o[8 * i + 1]));
            w.y = pack_bf16x2(__uint_as_float(o[8 * i + 2]), __uint_as_float(o[8 * i + 3]));
            w.z = pack_bf16x2(__uint_as_float(o[8 * i + 4]), __uint_as_float(o[8 * i + 5]));
            w.w = pack_bf16x2(__uint_as_float(o[8 * i + 6]), __uint_as_float(o[8 * i + 7]));
            reinterpret_cast<uint4*>(orow + ch * 32)[i] = w;
          }
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

// ------------------------------------------------------------------------------------
// Fused backward (D = 128): one kernel, five GEMMs per (key tile, query tile) pair
// ------------------------------------------------------------------------------------
// The key-tile owner computes S^T and dP^T once and derives all three gradients from them:
//     dV += P^T dO,   dK += dS^T Q          (accumulated in tensor memory over the whole loop, as above)
//     dQ^T(tile) = K^T dS                    (one fresh [128 d x 64 q] product per pair, added to an fp32 dQ buffer
//                                             in global memory by one tiled TMA reduction per pair)
// The packed P^T and dS^T both go back into the S^T columns (P^T in [0,32), dS^T in [32,64)), so that the whole
// dP^T buffer is free once the softmax threads have read it: the dQ^T product of the same pair is written there.
// dS^T is also stored in shared memory ([key][query], 128-byte swizzle): the MN-major B operand of the dQ^T MMA,
// whose A operand is the K tile read MN-major (M = d).  Four drain warps move each dQ^T tile from tensor memory into
// the shared-memory stage that held the pair's Q / dO (free by then) as a [64 q][128 d] fp32 tile, and one thread
// issues cp.reduce.async.bulk.tensor (.add) for it.  (Per-thread red.global.add.f32, 64 per thread and pair, ran the
// kernel 3x slower: the number of outstanding store requests per SM, not bytes, was the limit.)
// The fp32 buffer must be zero on entry; a small kernel converts it to bf16 afterwards.
// Summation order across key tiles is not fixed: use the two-kernel path above when bit-reproducible gradients
// are required.
constexpr int FTHR = 512;   // warps 0-3: TMA, S/dP MMA, accumulate MMA, spare; 4-11: softmax; 12-15: dQ drain

template <int D>
struct SmemFused {
  static constexpr int KPANEL = KM * 128;
  static constexpr int QPANEL = QN * 128;
  static constexpr int K_BYTES = KM * D * 2;
  static constexpr int Q_BYTES = QN * D * 2;
  static constexpr int OFF_V = K_BYTES;
  static constexpr int NST = 4;
  static constexpr int OFF_Q = 2 * K_BYTES;
  static constexpr int STAGE = 2 * Q_BYTES;
  static constexpr int DS_BYTES = KM * QN * 2;                // 16 KB: dS^T [128 keys][64 queries] bf16
  static constexpr int OFF_DS = OFF_Q + NST * STAGE;
  static constexpr int OFF_ROW = OFF_DS + 2 * DS_BYTES;       // lse2 / delta / qpos staging: 2 x 3 x 64 x 4
  static constexpr int OFF_BAR = OFF_ROW + 2 * 3 * QN * 4;
  static constexpr int TOTAL = OFF_BAR + 256;
};

template <int RegCount>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(RegCount));
}
template <int RegCount>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(RegCount));
}

template <int D>
__global__ void __launch_bounds__(FTHR, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                      const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const __grid_constant__ CUtensorMap tmDQ, const Params p) {
  static_assert(D == 128, "the fused backward is written for head dimension 128");
  using L = SmemFused<D>;
  constexpr int TMEM_COLS = 512;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sDS = smem + L::OFF_DS;
  float* s_row = reinterpret_cast<float*>(smem + L::OFF_ROW);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  constexpr int NST = L::NST;
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;              // [NST]
  uint64_t* q_empty = bars + 1 + NST;       // [NST]
  uint64_t* st_full = bars + 1 + 2 * NST;   // [2] S^T / dP^T written by the MMAs
  uint64_t* pds_full = bars + 3 + 2 * NST;  // [2] P^T / dS^T written by the softmax threads
  uint64_t* dq_full = bars + 5 + 2 * NST;   // [2] dQ^T tile written by the MMAs (all MMAs of the pair are done)
  uint64_t* t_free = bars + 7 + 2 * NST;    // [2] dQ^T tile read by the drain warps: the buffer pair is reusable
  uint64_t* acc_done = bars + 9 + 2 * NST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10 + 2 * NST);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};
  const int kt = blockIdx.x;
  const int hkv = blockIdx.y;
  const int b = blockIdx.z;
  const int k0 = kt * KM;
  const int keys_valid = min(KM, p.Tk - k0);
  const int G = p.Hq / p.Hkv;
  const int nq_tiles = (p.Tq + QN - 1) / QN;

  QTileIter iter;
  iter.G = G;
  iter.nq_tiles = nq_tiles;
  if (p.q_pos) {
    iter.i_lo = 0;
    iter.i_hi = nq_tiles - 1;
  } else {
    long long rmin = (long long)k0 + p.lo - p.q_off;
    long long rmax = (long long)k0 + keys_valid - 1 + (long long)p.hi - 1 - p.q_off;
    if (rmin < 0) rmin = 0;
    if (rmax > p.Tq - 1) rmax = p.Tq - 1;
    iter.i_lo = (int)(rmin / QN);
    iter.i_hi = (rmax >= rmin) ? (int)(rmax / QN) : iter.i_lo - 1;
  }
  const int n_it = iter.count();

  if (threadIdx.x == 0) {
    if ((smem_u32(smem) & 1023u) != 0) report_error(p.status, kBadArgument, 0xA3);
    mbar_init(kv_full, 1);
    for (int s = 0; s < NST; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&st_full[s], 1);
      mbar_init(&dq_full[s], 1);
      mbar_init(&t_free[s], 128);
      mbar_init(&pds_full[s], NSOFT);
    }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tST = [&](int s) -> uint32_t { return tmem_base + (uint32_t)s * 64u; };
  auto tDPT = [&](int s) -> uint32_t { return tmem_base + 128u + (uint32_t)s * 64u; };   // later: dQ^T of the pair
  const uint32_t tDV = tmem_base + 256, tDK = tmem_base + 256 + D;

  const int wg = warp >> 2;
  if (wg == 0) {
    reg_dealloc<48>();
    if (warp == 0) {
      if (lane == 0 && n_it > 0) {
        mbar_expect_tx(kv_full, 2 * L::K_BYTES);
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn) {
          tma_load_4d(sK + pn * L::KPANEL, &tmK, kv_full, pn * 64, hkv, k0, b);
          tma_load_4d(sV + pn * L::KPANEL, &tmV, kv_full, pn * 64, hkv, k0, b);
        }
        for (int it = 0; it < n_it; ++it) {
          const int s = it % NST;
          int g, i;
          iter.get(it, g, i);
          const int h = hkv * G + g;
          if (it >= NST) mbar_wait(&q_empty[s], ((it / NST) - 1) & 1, ctx, 0x310 + s);
          mbar_expect_tx(&q_full[s], L::STAGE);
          uint8_t* dst = sQ + s * L::STAGE;
#pragma unroll
          for (int pn = 0; pn < D / 64; ++pn) {
            tma_load_4d(dst + pn * L::QPANEL, &tmQ, &q_full[s], pn * 64, h, i * QN, b);
            tma_load_4d(dst + L::Q_BYTES + pn * L::QPANEL, &tmDO, &q_full[s], pn * 64, h, i * QN, b);
          }
        }
      }
    } else if (warp == 1) {
      if (lane == 0 && n_it > 0) {
        constexpr uint32_t idescST = make_idesc_bf16(KM, QN, false, false);
        const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
        mbar_wait(kv_full, 0, ctx, 0x330);
        for (int it = 0; it < n_it; ++it) {
          const int s = it & 1, qs = it % NST;
          if (it >= 2) mbar_wait(&t_free[s], ((it >> 1) - 1) & 1, ctx, 0x370 + s);
          mbar_wait(&q_full[qs], (it / NST) & 1, ctx, 0x320 + qs);
          tc_fence_after();
          const uint32_t aQ = smem_u32(sQ + qs * L::STAGE);
          const uint32_t aDO = aQ + L::Q_BYTES;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t ad = make_desc_kmajor_sw128(aK + (kk / 4) * L::KPANEL + (kk % 4) * 32);
            const uint64_t bd = make_desc_kmajor_sw128(aQ + (kk / 4) * L::QPANEL + (kk % 4) * 32);
            umma_ss(tST(s), ad, bd, idescST, kk > 0 ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t ad = make_desc_kmajor_sw128(aV + (kk / 4) * L::KPANEL + (kk % 4) * 32);
            const uint64_t bd = make_desc_kmajor_sw128(aDO + (kk / 4) * L::QPANEL + (kk % 4) * 32);
            umma_ss(tDPT(s), ad, bd, idescST, kk > 0 ? 1u : 0u);
          }
          umma_commit(&st_full[s]);
        }
      }
    } else if (warp == 2) {
      if (lane == 0 && n_it > 0) {
        constexpr uint32_t idescAcc = make_idesc_bf16(KM, D, false, true);     // [128 keys x D], B MN-major
        constexpr uint32_t idescDQ = make_idesc_bf16(D, QN, true, true);       // [D x 64 q], A and B MN-major
        const uint32_t aK = smem_u32(sK);
        for (int it = 0; it < n_it; ++it) {
          const int s = it & 1, qs = it % NST;
          mbar_wait(&q_full[qs], (it / NST) & 1, ctx, 0x380 + qs);
          mbar_wait(&pds_full[s], (it >> 1) & 1, ctx, 0x340 + s);
          tc_fence_after();
          const uint32_t aQ = smem_u32(sQ + qs * L::STAGE);
          const uint32_t aDO = aQ + L::Q_BYTES;
          const uint32_t aDS = smem_u32(sDS + s * L::DS_BYTES);
#pragma unroll
          for (int kk = 0; kk < QN / 16; ++kk) {
            const uint64_t bd = make_desc_mnmajor_sw128(aDO + kk * 2048, L::QPANEL);
            umma_ts(tDV, tST(s) + kk * 8, bd, idescAcc, (it > 0 || kk > 0) ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < QN / 16; ++kk) {
            const uint64_t bd = make_desc_mnmajor_sw128(aQ + kk * 2048, L::QPANEL);
            umma_ts(tDK, tST(s) + 32 + kk * 8, bd, idescAcc, (it > 0 || kk > 0) ? 1u : 0u);
          }
          // dQ^T[d, q] = sum_key K[key, d] dS^T[key, q]: 8 steps of 16 keys (the Q / dO stage is released by the drain
          // warps, which reuse its memory to stage the dQ tile)
#pragma unroll
          for (int kk = 0; kk < KM / 16; ++kk) {
            const uint64_t ad = make_desc_mnmajor_sw128(aK + kk * 2048, L::KPANEL);
            const uint64_t bd = make_desc_mnmajor_sw128(aDS + kk * 2048, L::DS_BYTES);
            umma_ss(tDPT(s), ad, bd, idescDQ, kk > 0 ? 1u : 0u);
          }
          umma_commit(&dq_full[s]);
        }
        umma_commit(acc_done);
      }
    }
  } else if (wg == 3) {
    // dQ drain: lane = d (quadrant * 32 + lane), 64 columns = the query rows of the tile.  The tile goes through the
    // Q / dO ring stage of the same pair (its 32 KB are exactly one [64 q][128 d] fp32 tile, and every MMA that read
    // it has completed once dq_full fires) and leaves as ONE tiled reduction per pair.
    reg_dealloc<96>();
    const int quad = warp & 3;
    const int d = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1, qs = it % NST;
      int g, i;
      iter.get(it, g, i);
      const int h = hkv * G + g;
      const int q0 = i * QN;
      const bool ok = mbar_wait(&dq_full[s], (it >> 1) & 1, ctx, 0x390 + s);
      tc_fence_after();
      uint32_t v0[32], v1[32];
      tmem_ld_x32(tDPT(s) + lane_off, v0);
      tmem_ld_x32(tDPT(s) + lane_off + 32, v1);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_relaxed(&t_free[s]);                // registers hold the tile: the buffer pair may be overwritten
      float* stg = reinterpret_cast<float*>(sQ + qs * L::STAGE);
#pragma unroll
      for (int c = 0; c < 32; ++c) stg[c * D + d] = __uint_as_float(v0[c]);
#pragma unroll
      for (int c = 0; c < 32; ++c) stg[(32 + c) * D + d] = __uint_as_float(v1[c]);
      fence_async_smem();
      asm volatile("bar.sync 3, 128;" ::: "memory");
      if (warp == 12 && lane == 0) {
        if (ok) {
          tma_reduce_add_4d(&tmDQ, stg, 0, h, q0, b);
          tma_store_commit();
          tma_store_wait_read<0>();                   // the stage may be refilled once the reduction has read it
        }
        mbar_arrive(&q_empty[qs]);
      }
    }
  } else {
    reg_alloc<184>();
    const int quad = warp & 3;
    const int part = (warp - 4) >> 2;
    const int r = quad * 32 + lane;  // key row
    const int tid = threadIdx.x - 128;  // 0..NSOFT-1
    const long long kpos = (long long)k0 + r;
    const bool key_ok = r < keys_valid;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const int vis_lo = (int)min(kpos + (long long)p.lo, 2147483647ll);
    const int vis_hi = (int)min(kpos + (long long)p.hi, 2147483647ll);
    auto load_rows = [&](int it, float& v0, int& v1) {
      int g, i;
      iter.get(it, g, i);
      const int h = hkv * G + g;
      const int q0 = i * QN;
      v0 = 0.f;
      v1 = -(1 << 30);
      if (tid < QN) {
        const int qi = q0 + tid;
        v0 = INFINITY;
        if (qi < p.Tq) {
          const float l = p.lse[((size_t)b * p.Hq + h) * p.Tq + qi];
          v0 = (l == -INFINITY) ? INFINITY : l * kLog2e;
          v1 = p.q_pos ? p.q_pos[(size_t)b * p.Tq + qi] : qi + p.q_off;
        }
      } else if (tid < 2 * QN) {
        const int qi = q0 + tid - QN;
        v0 = (qi < p.Tq) ? p.delta[((size_t)b * p.Hq + h) * p.Tq + qi] : 0.f;
      }
    };
    auto store_rows = [&](int it, float v0, int v1) {
      float* b_lse = s_row + (it & 1) * 3 * QN;
      if (tid < QN) {
        b_lse[tid] = v0;
        reinterpret_cast<int*>(b_lse + 2 * QN)[tid] = v1;
      } else if (tid < 2 * QN) {
        b_lse[QN + tid - QN] = v0;
      }
    };
    if (n_it > 0) {
      float v0;
      int v1;
      load_rows(0, v0, v1);
      store_rows(0, v0, v1);
    }
    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      int g, i;
      iter.get(it, g, i);
      const int q0 = i * QN;
      float* st_lse = s_row + s * 3 * QN;
      float* st_del = st_lse + QN;
      int* st_pos = reinterpret_cast<int*>(st_del + QN);
      float nv0 = 0.f;
      int nv1 = 0;
      if (it + 1 < n_it) load_rows(it + 1, nv0, nv1);
      const long long pmin = (long long)q0 + p.q_off, pmax = pmin + QN - 1;
      const bool full = p.q_pos == nullptr && keys_valid == KM && q0 + QN <= p.Tq &&
                        pmin - ((long long)k0 + KM - 1) >= (long long)p.lo && pmax - (long long)k0 < (long long)p.hi;
      asm volatile("bar.sync 1, %0;" ::"n"(NSOFT) : "memory");
      mbar_wait(&st_full[s], (it >> 1) & 1, ctx, 0x350 + s);
      tc_fence_after();
      {
        uint32_t sv[WCOLS], dp[WCOLS], pp[WCOLS / 2], pd[WCOLS / 2];
        tmem_ld_n<WCOLS>(tST(s) + lane_off + part * WCOLS, sv);
        tmem_ld_n<WCOLS>(tDPT(s) + lane_off + part * WCOLS, dp);
        tmem_ld_wait();
        if (full) {
#pragma unroll
          for (int c = 0; c < WCOLS; c += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(st_lse + part * WCOLS + c);
            const float4 d4 = *reinterpret_cast<const float4*>(st_del + part * WCOLS + c);
            const float p0 = exp2f(fmaf(__uint_as_float(sv[c + 0]), p.scale_log2, -l4.x));
            const float p1 = exp2f(fmaf(__uint_as_float(sv[c + 1]), p.scale_log2, -l4.y));
            const float p2 = exp2f(fmaf(__uint_as_float(sv[c + 2]), p.scale_log2, -l4.z));
            const float p3 = exp2f(fmaf(__uint_as_float(sv[c + 3]), p.scale_log2, -l4.w));
            pp[(c >> 1) + 0] = pack_bf16x2(p0, p1);
            pp[(c >> 1) + 1] = pack_bf16x2(p2, p3);
            pd[(c >> 1) + 0] = pack_bf16x2(p0 * (__uint_as_float(dp[c + 0]) - d4.x) * p.scale,
                                           p1 * (__uint_as_float(dp[c + 1]) - d4.y) * p.scale);
            pd[(c >> 1) + 1] = pack_bf16x2(p2 * (__uint_as_float(dp[c + 2]) - d4.z) * p.scale,
                                           p3 * (__uint_as_float(dp[c + 3]) - d4.w) * p.scale);
          }
        } else {
#pragma unroll
          for (int c = 0; c < WCOLS; c += 2) {
            float pr[2], ds[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int cc = part * WCOLS + c + e;
              const int pos = st_pos[cc];
              const bool vis = key_ok && pos >= vis_lo && pos < vis_hi;
              pr[e] = vis ? exp2f(fmaf(__uint_as_float(sv[c + e]), p.scale_log2, -st_lse[cc])) : 0.f;
              ds[e] = pr[e] * (__uint_as_float(dp[c + e]) - st_del[cc]) * p.scale;
            }
            pp[c >> 1] = pack_bf16x2(pr[0], pr[1]);
            pd[c >> 1] = pack_bf16x2(ds[0], ds[1]);
          }
        }
        // dS^T row r, query columns [part * WCOLS, +WCOLS): 64 bytes = 4 swizzled 16-byte chunks of the row
        uint8_t* ds_tile = sDS + s * L::DS_BYTES;
#pragma unroll
        for (int ch = 0; ch < WCOLS / 8; ++ch) {
          uint4 w;
          w.x = pd[4 * ch + 0]; w.y = pd[4 * ch + 1]; w.z = pd[4 * ch + 2]; w.w = pd[4 * ch + 3];
          *reinterpret_cast<uint4*>(ds_tile + sw128_offset((uint32_t)r, (uint32_t)(part * WCOLS * 2 + ch * 16))) = w;
        }
        fence_async_smem();
        // all 64 S^T columns of these rows must have been read (by every warpgroup) before the packed values
        // overwrite them
        asm volatile("bar.sync 2, %0;" ::"n"(NSOFT) : "memory");
        tmem_st_n<WCOLS / 2>(tST(s) + lane_off + part * (WCOLS / 2), pp);
        tmem_st_n<WCOLS / 2>(tST(s) + 32 + lane_off + part * (WCOLS / 2), pd);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&pds_full[s]);
      if (it + 1 < n_it) store_rows(it + 1, nv0, nv1);
    }
    if (n_it > 0) {
      mbar_wait(acc_done, 0, ctx, 0x360);
      tc_fence_after();
    }
    {
      constexpr int PER = NWG / 2;
      constexpr int OC = D / PER;
      const int which = part / PER, sub = part % PER;
      bf16* base = which == 0 ? p.dv : p.dk;
      const uint32_t tacc = which == 0 ? tDV : tDK;
      bf16* orow = base + (((size_t)b * p.Tk + k0 + r) * p.Hkv + hkv) * D + sub * OC;
#pragma unroll
      for (int ch = 0; ch < OC / 32; ++ch) {
        uint32_t o[32];
        if (n_it > 0) {
          tmem_ld_x32(tacc + lane_off + sub * OC + ch * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (key_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[8 * i + 0]), __uint_as_float(o[8 * i + 1]));
            w.y = pack_bf16x2(__uint_as_float(o[8 * i + 2]), __uint_as_float(o[8 * i + 3]));
            w.z = pack_bf16x2(__uint_as_float(o[8 * i + 4]), __uint_as_float(o[8 * i + 5]));
            w.w = pack_bf16x2(__uint_as_float(o[8 * i + 6]), __uint_as_float(o[8 * i + 7]));
            reinterpret_cast<uint4*>(orow + ch * 32)[i] = w;
          }
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

// dq (bf16) = dq_acc (fp32); n elements, n % 8 == 0
__global__ void dq_convert_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, long long n8) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const float4 a = reinterpret_cast<const float4*>(acc)[2 * i];
  const float4 c = reinterpret_cast<const float4*>(acc)[2 * i + 1];
  uint4 w;
  w.x = pack_bf16x2(a.x, a.y); w.y = pack_bf16x2(a.z, a.w);
  w.z = pack_bf16x2(c.x, c.y); w.w = pack_bf16x2(c.z, c.w);
  reinterpret_cast<uint4*>(dq)[i] = w;
}

static int make_map_bthd(CUtensorMap* m, const void* base, int B, int T, int H, int D, long long sb,
                         long long st, long long sh, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[4] = {2, (uint64_t)sh * 2, (uint64_t)st * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_tensor_map(m, base, 0, 4, dims, strides, box, 3);
}

template <int D>
static int launch_all(const void* q, const void* k, const void* v, const void* d_o, const Params& p,
                      const long long* qs, const long long* ks, const long long* vs, cudaStream_t st) {
  CUtensorMap tmQ, tmDO, tmK, tmV;
  int rc;
  const long long os[3] = {(long long)p.Tq * p.Hq * D, (long long)p.Hq * D, D};
  // dQ kernel: Q/dO boxes of 128 rows, K/V boxes of 64 rows
  if ((rc = make_map_bthd(&tmQ, q, p.B, p.Tq, p.Hq, D, qs[0], qs[1], qs[2], BM)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmDO, d_o, p.B, p.Tq, p.Hq, D, os[0], os[1], os[2], BM)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmK, k, p.B, p.Tk, p.Hkv, D, ks[0], ks[1], ks[2], BN)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmV, v, p.B, p.Tk, p.Hkv, D, vs[0], vs[1], vs[2], BN)) != HMF_OK) return rc;
  {
    auto kern = attn_bwd_dq_kernel<D>;
    static bool configured = false;
    if (!configured) {
      HMF_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemDQ<D>::TOTAL));
      configured = true;
    }
    dim3 grid(p.Hq, (p.Tq + BM - 1) / BM, p.B);
    kern<<<grid, NTHR + 32, SmemDQ<D>::TOTAL, st>>>(tmQ, tmDO, tmK, tmV, p);
    HMF_CHECK_CUDA(cudaGetLastError());
  }
  // dK/dV kernel: K/V boxes of 128 rows, Q/dO boxes of 64 rows
  if ((rc = make_map_bthd(&tmQ, q, p.B, p.Tq, p.Hq, D, qs[0], qs[1], qs[2], QN)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmDO, d_o, p.B, p.Tq, p.Hq, D, os[0], os[1], os[2], QN)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmK, k, p.B, p.Tk, p.Hkv, D, ks[0], ks[1], ks[2], KM)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmV, v, p.B, p.Tk, p.Hkv, D, vs[0], vs[1], vs[2], KM)) != HMF_OK) return rc;
  {
    auto kern = attn_bwd_dkv_kernel<D>;
    static bool configured = false;
    if (!configured) {
      HMF_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemDKV<D>::TOTAL));
      configured = true;
    }
    dim3 grid((p.Tk + KM - 1) / KM, p.Hkv, p.B);
    kern<<<grid, NTHR + 32, SmemDKV<D>::TOTAL, st>>>(tmQ, tmDO, tmK, tmV, p);
    HMF_CHECK_CUDA(cudaGetLastError());
  }
  return HMF_OK;
}


static int launch_fused(const void* q, const void* k, const void* v, const void* d_o, const Params& p,
                        const long long* qs, const long long* ks, const long long* vs, float* dq_acc,
                        cudaStream_t st) {
  constexpr int D = 128;
  CUtensorMap tmQ, tmDO, tmK, tmV;
  int rc;
  const long long os[3] = {(long long)p.Tq * p.Hq * D, (long long)p.Hq * D, D};
  if ((rc = make_map_bthd(&tmQ, q, p.B, p.Tq, p.Hq, D, qs[0], qs[1], qs[2], QN)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmDO, d_o, p.B, p.Tq, p.Hq, D, os[0], os[1], os[2], QN)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmK, k, p.B, p.Tk, p.Hkv, D, ks[0], ks[1], ks[2], KM)) != HMF_OK) return rc;
  if ((rc = make_map_bthd(&tmV, v, p.B, p.Tk, p.Hkv, D, vs[0], vs[1], vs[2], KM)) != HMF_OK) return rc;
  CUtensorMap tmDQ;
  {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)p.Hq, (uint64_t)p.Tq, (uint64_t)p.B};
    uint64_t strides[4] = {4, (uint64_t)D * 4, (uint64_t)p.Hq * D * 4, (uint64_t)p.Tq * p.Hq * D * 4};
    uint32_t box[4] = {(uint32_t)D, 1, (uint32_t)QN, 1};
    if ((rc = make_tensor_map(&tmDQ, dq_acc, 1, 4, dims, strides, box, 0)) != HMF_OK) return rc;
  }
  auto kern = attn_bwd_fused_kernel<D>;
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemFused<D>::TOTAL));
    configured = true;
  }
  dim3 grid((p.Tk + KM - 1) / KM, p.Hkv, p.B);
  kern<<<grid, FTHR, SmemFused<D>::TOTAL, st>>>(tmQ, tmDO, tmK, tmV, tmDQ, p);
  HMF_CHECK_CUDA(cudaGetLastError());
  const long long n8 = (long long)p.B * p.Tq * p.Hq * D / 8;
  dq_convert_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(dq_acc, p.dq, n8);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

}  // namespace attn_bwd
}  // namespace hmf

// Gradients of hmf_attention_fwd.  o, d_o, dq: [B,Tq,Hq,D] contiguous; dk, dv: [B,Tk,Hkv,D]
// contiguous; lse from the forward pass; dlse: optional gradient of the lse output [B,Hq,Tq] fp32 (null = none);
// delta: scratch [B,Hq,Tq] fp32 provided by the caller.
HMF_API int hmf_attention_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                              const float* lse, const float* dlse, float* delta, void* dq, void* dk, void* dv,
                              const int* q_pos,
                              int B, int Tq, int Tk, int Hq, int Hkv, int D, long long q_sb, long long q_st,
                              long long q_sh, long long k_sb, long long k_st, long long k_sh, long long v_sb,
                              long long v_st, long long v_sh, int lo, int hi, int q_off, float scale,
                              cudaStream_t stream) {
  using namespace hmf;
  using namespace hmf::attn_bwd;
  HMF_REQUIRE(q && k && v && o && d_o && lse && delta && dq && dk && dv, "attention_bwd: null tensor");
  HMF_REQUIRE(D == 64 || D == 128, "attention_bwd: head dim %d unsupported (64, 128)", D);
  HMF_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "attention_bwd: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  HMF_REQUIRE(lo >= 0 && hi > lo, "attention_bwd: bad window lo=%d hi=%d", lo, hi);
  {
    const long long rows = (long long)B * Tq * Hq;
    const int rpw = 32 / (D / 8);
    const long long warps = (rows + rpw - 1) / rpw;
    const long long blocks = (warps + 7) / 8;
    delta_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const bf16*)o, (const bf16*)d_o, dlse, delta, B, Tq, Hq, D);
    HMF_CHECK_CUDA(cudaGetLastError());
  }
  Params p;
  p.lse = lse; p.delta = delta; p.q_pos = q_pos;
  p.dq = (bf16*)dq; p.dk = (bf16*)dk; p.dv = (bf16*)dv;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv;
  p.lo = lo; p.hi = hi; p.q_off = q_off;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.status = status_ptr();
  const long long qs[3] = {q_sb, q_st, q_sh}, ks[3] = {k_sb, k_st, k_sh}, vs[3] = {v_sb, v_st, v_sh};
  if (D == 64) return launch_all<64>(q, k, v, d_o, p, qs, ks, vs, stream);
  return launch_all<128>(q, k, v, d_o, p, qs, ks, vs, stream);
}

// Single-kernel variant for D = 128 (five GEMMs per tile pair; dQ is summed with fp32 reductions in global memory, so
// the order of that sum, and with it the last bits of dq, may differ from run to run).  Same arguments as
// hmf_attention_bwd plus dq_acc: fp32 scratch [B,Tq,Hq,D] that must be ZERO on entry (it holds dq in fp32 on return).
HMF_API int hmf_attention_bwd_fused(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                    const float* lse, const float* dlse, float* delta, float* dq_acc, void* dq,
                                    void* dk, void* dv, const int* q_pos, int B, int Tq, int Tk, int Hq, int Hkv,
                                    int D, long long q_sb, long long q_st, long long q_sh, long long k_sb,
                                    long long k_st, long long k_sh, long long v_sb, long long v_st, long long v_sh,
                                    int lo, int hi, int q_off, float scale, cudaStream_t stream) {
  using namespace hmf;
  using namespace hmf::attn_bwd;
  HMF_REQUIRE(q && k && v && o && d_o && lse && delta && dq_acc && dq && dk && dv, "attention_bwd_fused: null tensor");
  HMF_REQUIRE(D == 128, "attention_bwd_fused: head dim %d unsupported (128)", D);
  HMF_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "attention_bwd_fused: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  HMF_REQUIRE(lo >= 0 && hi > lo, "attention_bwd_fused: bad window lo=%d hi=%d", lo, hi);
  {
    const long long rows = (long long)B * Tq * Hq;
    const int rpw = 32 / (D / 8);
    const long long warps = (rows + rpw - 1) / rpw;
    const long long blocks = (warps + 7) / 8;
    delta_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const bf16*)o, (const bf16*)d_o, dlse, delta, B, Tq, Hq, D);
    HMF_CHECK_CUDA(cudaGetLastError());
  }
  Params p;
  p.lse = lse; p.delta = delta; p.q_pos = q_pos;
  p.dq = (bf16*)dq; p.dk = (bf16*)dk; p.dv = (bf16*)dv;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv;
  p.lo = lo; p.hi = hi; p.q_off = q_off;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.status = status_ptr();
  const long long qs[3] = {q_sb, q_st, q_sh}, ks[3] = {k_sb, k_st, k_sh}, vs[3] = {v_sb, v_st, v_sh};
  return launch_fused(q, k, v, d_o, p, qs, ks, vs, dq_acc, stream);
}
