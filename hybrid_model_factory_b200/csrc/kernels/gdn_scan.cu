// Gated delta rule: the sequential inter-chunk recurrence (forward and reverse) on tcgen05.
//
// Everything is kept in "feature-major" (transposed) form so that the 128-wide feature dimension
// is the MMA M dimension and the 64 chunk positions are N or K:
//
//   forward, per chunk n with start state S (dk x dv), h := S^T kept in registers (thread <-> dv row)
//     D1 = h (128 x dk) * [w ; q~]^T            -> (w S)^T | (q~ S)^T            (128 x 128)
//     vn^T = u^T - (w S)^T                                                          (128 x 64)
//     D2 = vn^T * [k~^T ; P]^T                   -> dh (128 x dk) | o_intra^T (128 x 64)
//     o^T = (q~ S)^T + o_intra^T ;  h = e^{g_last} h + dh
//   with  w, u the WY factors, q~ = q e^{G} scale, k~ = k e^{g_last - G}, P = (q k^T . decay, causal).
//
// The A operands (h and vn^T in bf16) live in tensor memory, written by tcgen05.st from the
// threads that own the rows; the B operands are per-chunk tiles prepared by the chunk-parallel
// stage and streamed by TMA through a 2-stage ring.  One CTA per (batch, head).
//
// Sequence parallelism is fused here: the kernel can wait (bounded) for its incoming state to be
// written into a local buffer by the previous rank, and pushes its final state straight into the
// next rank's buffer over NVLink, followed by a release flag.
#include <math.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace gdn {

using bf16 = __nv_bfloat16;
constexpr int C = 64;     // chunk length
constexpr int DK = 128;
constexpr int DV = 128;
constexpr int WQ_BYTES = 2 * DK * C * 2;   // [2][128][64] bf16
constexpr int KP_BYTES = (DK + C) * C * 2; // [192][64] bf16
constexpr int U_BYTES = DV * C * 2;        // [128][64] bf16
constexpr int STAGE = WQ_BYTES + KP_BYTES + U_BYTES;  // 73728
constexpr int OTILE = C * DV * 2;                      // 16384
constexpr int SMEM_FWD = 2 * STAGE + 2 * OTILE + 256;
constexpr uint64_t kPeerWaitNs = 4000000000ull;

struct FwdParams {
  const float* glast;  // [BH, N]
  const float* h0;     // [BH, DK, DV] or null
  float* hT;           // [BH, DK, DV] or null
  bf16* o;             // [B, T, H, DV]
  bf16* vnT;           // [BH, N, DV, C] or null
  bf16* h_all;         // [BH, N, DV, DK] or null (chunk-start states, transposed)
  int B, H, T, N;
  // sequence-parallel state exchange (all optional)
  const unsigned int* h0_flag;  // [BH] wait until h0_flag[bh] >= epoch before reading h0
  float* peer_hT;               // next rank's h0 buffer [BH, DK, DV] (peer memory)
  unsigned int* peer_flag;      // next rank's flag
  unsigned int epoch;
  unsigned int* status;
};

__global__ void __launch_bounds__(192, 1)
gdn_scan_fwd_kernel(const __grid_constant__ CUtensorMap tmWQ, const __grid_constant__ CUtensorMap tmKP,
                    const __grid_constant__ CUtensorMap tmU, const FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* otile = smem + 2 * STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * STAGE + 2 * OTILE);
  uint64_t* full = bars + 0;    // [2]
  uint64_t* empty = bars + 2;   // [2]
  uint64_t* h_ready = bars + 4;
  uint64_t* d1_full = bars + 5;
  uint64_t* v_ready = bars + 6;
  uint64_t* d2_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};
  const int bh = blockIdx.x;
  const int b = bh / p.H, hh = bh % p.H;
  const int N = p.N;

  if (threadIdx.x == 0) {
    if ((smem_u32(smem) & 1023u) != 0) report_error(p.status, kBadArgument, 0xB1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(h_ready, 128);
    mbar_init(d1_full, 1);
    mbar_init(v_ready, 128);
    mbar_init(d2_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tAh = tmem_base, tAv = tmem_base + 64, tD1 = tmem_base + 128, tD2 = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      for (int n = 0; n < N; ++n) {
        const int s = n & 1;
        mbar_wait(&empty[s], ((n >> 1) & 1) ^ 1, ctx, 0x310 + s);
        uint8_t* st = smem + s * STAGE;
        const long long chunk = (long long)bh * N + n;
        mbar_expect_tx(&full[s], STAGE);
        tma_load_2d(st, &tmWQ, &full[s], 0, (int)(chunk * 2 * DK));
        tma_load_2d(st + WQ_BYTES, &tmKP, &full[s], 0, (int)(chunk * (DK + C)));
        tma_load_2d(st + WQ_BYTES + KP_BYTES, &tmU, &full[s], 0, (int)(chunk * DV));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc1 = make_idesc_bf16(128, 128, false, true);
      constexpr uint32_t idesc2 = make_idesc_bf16(128, 192, false, false);
      for (int n = 0; n < N; ++n) {
        const int s = n & 1;
        const uint32_t aWQ = smem_u32(smem + s * STAGE);
        const uint32_t aKP = aWQ + WQ_BYTES;
        mbar_wait(&full[s], (n >> 1) & 1, ctx, 0x320 + s);
        mbar_wait(h_ready, n & 1, ctx, 0x330);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk)
          umma_ts(tD1, tAh + kk * 8, make_desc_mnmajor_sw128(aWQ + kk * 2048, DK * 128), idesc1, kk > 0 ? 1u : 0u);
        umma_commit(d1_full);
        mbar_wait(v_ready, n & 1, ctx, 0x340);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < C / 16; ++kk)
          umma_ts(tD2, tAv + kk * 8, make_desc_kmajor_sw128(aKP + kk * 32), idesc2, kk > 0 ? 1u : 0u);
        umma_commit(&empty[s]);
        umma_commit(d2_full);
      }
    }
  } else {
    const int quad = warp & 3;
    const int t = quad * 32 + lane;  // dv row owned by this thread
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    float h[DK];
    if (p.h0 != nullptr) {
      if (p.h0_flag != nullptr) {
        if (t == 0) wait_flag_sys(p.h0_flag + bh, p.epoch, kPeerWaitNs, p.status, 0x350);
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      const float* src = p.h0 + (size_t)bh * DK * DV;
#pragma unroll
      for (int d = 0; d < DK; ++d) h[d] = __ldcv(src + (size_t)d * DV + t);
    } else {
#pragma unroll
      for (int d = 0; d < DK; ++d) h[d] = 0.f;
    }
    for (int n = 0; n < N; ++n) {
      const int s = n & 1;
      const long long chunk = (long long)bh * N + n;
      // (a) publish the state as the bf16 A operand (and save it for the backward pass)
      {
        uint32_t pk[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) pk[i] = pack_bf16x2(h[2 * i], h[2 * i + 1]);
        if (p.h_all != nullptr) {
          uint4* dst = reinterpret_cast<uint4*>(p.h_all + ((size_t)chunk * DV + t) * DK);
#pragma unroll
          for (int i = 0; i < 16; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
        }
        tmem_st_x32(tAh + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
        tmem_st_x32(tAh + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(h_ready);
      }
      // (c) vn^T = u^T - (w S)^T
      mbar_wait(&full[s], (n >> 1) & 1, ctx, 0x360 + s);
      const uint8_t* sU = smem + s * STAGE + WQ_BYTES + KP_BYTES;
      uint32_t uraw[32];
#pragma unroll
      for (int c16 = 0; c16 < 8; ++c16) {
        const uint4 v = *reinterpret_cast<const uint4*>(sU + t * 128 + ((c16 ^ (t & 7)) << 4));
        uraw[4 * c16] = v.x; uraw[4 * c16 + 1] = v.y; uraw[4 * c16 + 2] = v.z; uraw[4 * c16 + 3] = v.w;
      }
      mbar_wait(d1_full, n & 1, ctx, 0x370);
      tc_fence_after();
      {
        uint32_t wh[64], pk[32];
        tmem_ld_x32(tD1 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&wh[0]));
        tmem_ld_x32(tD1 + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&wh[32]));
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const __nv_bfloat162 u2 = *reinterpret_cast<const __nv_bfloat162*>(&uraw[i]);
          const float2 uf = __bfloat1622float2(u2);
          pk[i] = pack_bf16x2(uf.x - __uint_as_float(wh[2 * i]), uf.y - __uint_as_float(wh[2 * i + 1]));
        }
        tmem_st_x32(tAv + lane_off, pk);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(v_ready);
        if (p.vnT != nullptr) {
          uint4* dst = reinterpret_cast<uint4*>(p.vnT + ((size_t)chunk * DV + t) * C);
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
        }
      }
      // (e) output and state update
      mbar_wait(d2_full, n & 1, ctx, 0x380);
      tc_fence_after();
      bf16* ot = reinterpret_cast<bf16*>(otile + s * OTILE);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t qh[32], oi[32];
        tmem_ld_x32(tD1 + lane_off + 64 + half * 32, qh);
        tmem_ld_x32(tD2 + lane_off + 128 + half * 32, oi);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          ot[(half * 32 + i) * DV + t] = __float2bfloat16(__uint_as_float(qh[i]) + __uint_as_float(oi[i]));
      }
      const float decay = __expf(p.glast[chunk]);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t dh[32];
        tmem_ld_x32(tD2 + lane_off + ch * 32, dh);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) h[ch * 32 + i] = fmaf(h[ch * 32 + i], decay, __uint_as_float(dh[i]));
      }
      tc_fence_before();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      // cooperative store of the [64 x 128] output tile: rows of 256 bytes
      {
        const int t0 = n * C;
#pragma unroll
        for (int pass = 0; pass < 8; ++pass) {
          const int row = pass * 8 + (t >> 4);
          const int c16 = t & 15;
          if (t0 + row < p.T) {
            const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(ot) + row * 256 + c16 * 16);
            bf16* dst = p.o + (((size_t)b * p.T + t0 + row) * p.H + hh) * DV;
            reinterpret_cast<uint4*>(dst)[c16] = v;
          }
        }
      }
    }
    // final state (fp32, [DK, DV]) to the local output and, under sequence parallelism, to the next rank
    if (p.hT != nullptr) {
      float* dst = p.hT + (size_t)bh * DK * DV;
#pragma unroll
      for (int d = 0; d < DK; ++d) dst[(size_t)d * DV + t] = h[d];
    }
    if (p.peer_hT != nullptr) {
      float* dst = p.peer_hT + (size_t)bh * DK * DV;
#pragma unroll
      for (int d = 0; d < DK; ++d) dst[(size_t)d * DV + t] = h[d];
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      // one flag word per (batch, head): the receiving CTA of the same index waits for this epoch
      if (t == 0 && p.peer_flag != nullptr) st_release_sys(p.peer_flag + bh, p.epoch);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------
// Reverse scan (backward).  Per chunk n, with dS' the gradient of the state after the chunk
// (thread <-> dv row of dS'^T, fp32 registers):
//   dvn^T = dO^T P + dS'^T k~^T                         (128 x 64)   -> saved (this is du^T)
//   dS^T  = dO^T q~ + e^{g_last} dS'^T - dvn^T w        (128 x dk)
// dS'^T of every chunk is saved in bf16 for the chunk-parallel stage.
// ------------------------------------------------------------------------------------
constexpr int DO_BYTES = C * DV * 2;  // two 64-wide panels of [64 pos x 128 B]
constexpr int SMEM_BWD = 2 * STAGE + 256;

struct BwdParams {
  const float* glast;  // [BH, N]
  const float* dhT;    // [BH, DK, DV] gradient of the final state, or null
  float* dh0;          // [BH, DK, DV] gradient of the initial state, or null
  bf16* dvnT;          // [BH, N, DV, C]
  bf16* dS_all;        // [BH, N, DV, DK]  dS'^T per chunk (gradient of the chunk's final state)
  int B, H, T, N;
  const unsigned int* dhT_flag;  // [BH] wait (sequence parallel) before reading dhT
  float* peer_dh0;               // previous rank's dhT buffer
  unsigned int* peer_flag;
  unsigned int epoch;
  unsigned int* status;
};

__global__ void __launch_bounds__(192, 1)
gdn_scan_bwd_kernel(const __grid_constant__ CUtensorMap tmWQ, const __grid_constant__ CUtensorMap tmKP,
                    const __grid_constant__ CUtensorMap tmDO, const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * STAGE);
  uint64_t* full = bars + 0;
  uint64_t* empty = bars + 2;
  uint64_t* s_ready = bars + 4;   // dS' published (128 arrivals)
  uint64_t* da_full = bars + 5;   // dvn^T accumulator complete
  uint64_t* dv_ready = bars + 6;  // dvn^T bf16 published (128 arrivals)
  uint64_t* dc_full = bars + 7;   // dS^T accumulator complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};
  const int bh = blockIdx.x;
  const int b = bh / p.H, hh = bh % p.H;
  const int N = p.N;

  if (threadIdx.x == 0) {
    if ((smem_u32(smem) & 1023u) != 0) report_error(p.status, kBadArgument, 0xB2);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(s_ready, 128);
    mbar_init(da_full, 1);
    mbar_init(dv_ready, 128);
    mbar_init(dc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tAs = tmem_base, tAd = tmem_base + 64, tDA = tmem_base + 128, tDC = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      for (int it = 0; it < N; ++it) {
        const int n = N - 1 - it;
        const int s = it & 1;
        mbar_wait(&empty[s], ((it >> 1) & 1) ^ 1, ctx, 0x410 + s);
        uint8_t* st = smem + s * STAGE;
        const long long chunk = (long long)bh * N + n;
        mbar_expect_tx(&full[s], STAGE);
        tma_load_2d(st, &tmWQ, &full[s], 0, (int)(chunk * 2 * DK));
        tma_load_2d(st + WQ_BYTES, &tmKP, &full[s], 0, (int)(chunk * (DK + C)));
        tma_load_4d(st + WQ_BYTES + KP_BYTES, &tmDO, &full[s], 0, hh, n * C, b);
        tma_load_4d(st + WQ_BYTES + KP_BYTES + DO_BYTES / 2, &tmDO, &full[s], 64, hh, n * C, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idescA = make_idesc_bf16(128, 64, true, true);    // dO^T (MN) x P (MN)
      constexpr uint32_t idescB = make_idesc_bf16(128, 64, false, true);   // dS'^T (TMEM) x k~^T (MN)
      constexpr uint32_t idescC = make_idesc_bf16(128, 128, true, false);  // dO^T (MN) x q~^T (K)
      constexpr uint32_t idescD = make_idesc_bf16(128, 128, false, false) | (1u << 13);  // -(dvn^T) x w^T (K)
      for (int it = 0; it < N; ++it) {
        const int s = it & 1;
        const uint32_t aWQ = smem_u32(smem + s * STAGE);
        const uint32_t aKP = aWQ + WQ_BYTES;
        const uint32_t aDO = aKP + KP_BYTES;
        mbar_wait(&full[s], (it >> 1) & 1, ctx, 0x420 + s);
        tc_fence_after();
        // state-independent parts first
#pragma unroll
        for (int kk = 0; kk < C / 16; ++kk)
          umma_ss(tDA, make_desc_mnmajor_sw128(aDO + kk * 2048, DO_BYTES / 2),
                  make_desc_mnmajor_sw128(aKP + DK * 128 + kk * 2048, C * 128), idescA, kk > 0 ? 1u : 0u);
        // s_ready also tells that the threads have finished reading the previous dS^T accumulator
        mbar_wait(s_ready, it & 1, ctx, 0x430);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk)
          umma_ts(tDA, tAs + kk * 8, make_desc_mnmajor_sw128(aKP + kk * 2048, DK * 128), idescB, 1u);
        umma_commit(da_full);
#pragma unroll
        for (int kk = 0; kk < C / 16; ++kk)
          umma_ss(tDC, make_desc_mnmajor_sw128(aDO + kk * 2048, DO_BYTES / 2),
                  make_desc_kmajor_sw128(aWQ + DK * 128 + kk * 32), idescC, kk > 0 ? 1u : 0u);
        mbar_wait(dv_ready, it & 1, ctx, 0x440);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < C / 16; ++kk)
          umma_ts(tDC, tAd + kk * 8, make_desc_kmajor_sw128(aWQ + kk * 32), idescD, 1u);
        umma_commit(&empty[s]);
        umma_commit(dc_full);
      }
    }
  } else {
    const int quad = warp & 3;
    const int t = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    float ds[DK];
    if (p.dhT != nullptr) {
      if (p.dhT_flag != nullptr) {
        if (t == 0) wait_flag_sys(p.dhT_flag + bh, p.epoch, kPeerWaitNs, p.status, 0x450);
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      const float* src = p.dhT + (size_t)bh * DK * DV;
#pragma unroll
      for (int d = 0; d < DK; ++d) ds[d] = __ldcv(src + (size_t)d * DV + t);
    } else {
#pragma unroll
      for (int d = 0; d < DK; ++d) ds[d] = 0.f;
    }
    for (int it = 0; it < N; ++it) {
      const int n = N - 1 - it;
      const long long chunk = (long long)bh * N + n;
      {
        uint32_t pk[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) pk[i] = pack_bf16x2(ds[2 * i], ds[2 * i + 1]);
        uint4* dst = reinterpret_cast<uint4*>(p.dS_all + ((size_t)chunk * DV + t) * DK);
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
        tmem_st_x32(tAs + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
        tmem_st_x32(tAs + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(s_ready);
      }
      mbar_wait(da_full, it & 1, ctx, 0x460);
      tc_fence_after();
      {
        uint32_t dv[64], pk[32];
        tmem_ld_x32(tDA + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&dv[0]));
        tmem_ld_x32(tDA + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&dv[32]));
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) pk[i] = pack_bf16x2(__uint_as_float(dv[2 * i]), __uint_as_float(dv[2 * i + 1]));
        tmem_st_x32(tAd + lane_off, pk);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(dv_ready);
        uint4* dst = reinterpret_cast<uint4*>(p.dvnT + ((size_t)chunk * DV + t) * C);
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
      }
      mbar_wait(dc_full, it & 1, ctx, 0x470);
      tc_fence_after();
      const float decay = __expf(p.glast[chunk]);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t dc[32];
        tmem_ld_x32(tDC + lane_off + ch * 32, dc);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) ds[ch * 32 + i] = fmaf(ds[ch * 32 + i], decay, __uint_as_float(dc[i]));
      }
      tc_fence_before();
    }
    if (p.dh0 != nullptr) {
      float* dst = p.dh0 + (size_t)bh * DK * DV;
#pragma unroll
      for (int d = 0; d < DK; ++d) dst[(size_t)d * DV + t] = ds[d];
    }
    if (p.peer_dh0 != nullptr) {
      float* dst = p.peer_dh0 + (size_t)bh * DK * DV;
#pragma unroll
      for (int d = 0; d < DK; ++d) dst[(size_t)d * DV + t] = ds[d];
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (t == 0 && p.peer_flag != nullptr) st_release_sys(p.peer_flag + bh, p.epoch);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Gated linear attention only (no delta rule): a sequence cut into P segments can be scanned segment-parallel, because
// the state transition of a segment is a scalar decay per head.  Given every segment's final state from a zero start
// (`seg_state` [P, H, E]) and its per-chunk log-decays (`glast` [P, H, n_seg]), this writes the true incoming state of
// every segment (`s_in` [P, H, E]) and the state after the last one (`s_out` [H, E]).
__global__ void gla_segment_prefix_kernel(const float* __restrict__ seg_state, const float* __restrict__ glast,
                                          const float* __restrict__ h0, float* __restrict__ s_in,
                                          float* __restrict__ s_out, int P, int n_seg, int E, long long st_p,
                                          long long st_h, long long gl_p, long long gl_h, long long in_p, long long in_h,
                                          long long out_h) {
  const int h = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  float s = h0 != nullptr ? h0[(size_t)h * E + e] : 0.f;
  for (int p = 0; p < P; ++p) {
    s_in[(size_t)p * in_p + (size_t)h * in_h + e] = s;
    float ld = 0.f;
    for (int n = 0; n < n_seg; ++n) ld += glast[(size_t)p * gl_p + (size_t)h * gl_h + n];
    s = __expf(ld) * s + seg_state[(size_t)p * st_p + (size_t)h * st_h + e];
  }
  s_out[(size_t)h * out_h + e] = s;
}

}  // namespace gdn
}  // namespace hmf

using namespace hmf;
using namespace hmf::gdn;

// Forward scan.  Per-chunk operand tiles (bf16, contiguous):
//   wqT [BH, N, 2, 128, 64]  (w^T, then (q e^{G} scale)^T)      kPT [BH, N, 192, 64]  ((k e^{g_last-G})^T, then P)
//   uT  [BH, N, 128, 64]     glast [BH, N] fp32                 h0 / hT [BH, 128, 128] fp32 (dk, dv)
// Outputs: o [B, T, H, 128] bf16; optional vnT [BH, N, 128, 64], h_all [BH, N, 128(dv), 128(dk)] bf16.
// Sequence-parallel hooks: h0_flag[BH] (wait for >= epoch), peer_hT / peer_flag (push to the next rank).
HMF_API int hmf_gdn_scan_fwd(const void* wqT, const void* kPT, const void* uT, const float* glast,
                             const float* h0, float* hT, void* o, void* vnT, void* h_all, int B, int H, int T,
                             int N, const unsigned int* h0_flag, float* peer_hT, unsigned int* peer_flag,
                             unsigned int epoch, cudaStream_t stream) {
  HMF_REQUIRE(wqT && kPT && uT && glast && o, "gdn_scan_fwd: null tensor");
  HMF_REQUIRE(B > 0 && H > 0 && N > 0 && T > 0 && T <= N * C, "gdn_scan_fwd: bad sizes B=%d H=%d T=%d N=%d", B, H, T, N);
  const long long BH = (long long)B * H;
  HMF_REQUIRE(BH * N * 2 * DK < 2147483647ll, "gdn_scan_fwd: problem too large for 32-bit tile coordinates");
  CUtensorMap tmWQ, tmKP, tmU;
  int rc;
  if ((rc = make_map_2d_bf16(&tmWQ, wqT, BH * N * 2 * DK, C, C, 2 * DK, C)) != HMF_OK) return rc;
  if ((rc = make_map_2d_bf16(&tmKP, kPT, BH * N * (DK + C), C, C, DK + C, C)) != HMF_OK) return rc;
  if ((rc = make_map_2d_bf16(&tmU, uT, BH * N * DV, C, C, DV, C)) != HMF_OK) return rc;
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(gdn_scan_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_FWD));
    configured = true;
  }
  FwdParams p;
  p.glast = glast; p.h0 = h0; p.hT = hT; p.o = (bf16*)o; p.vnT = (bf16*)vnT; p.h_all = (bf16*)h_all;
  p.B = B; p.H = H; p.T = T; p.N = N;
  p.h0_flag = h0_flag; p.peer_hT = peer_hT; p.peer_flag = peer_flag; p.epoch = epoch;
  p.status = status_ptr();
  gdn_scan_fwd_kernel<<<(unsigned)BH, 192, SMEM_FWD, stream>>>(tmWQ, tmKP, tmU, p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// Reverse scan.  d_o [B, T, H, 128] bf16 contiguous; outputs dvnT [BH, N, 128, 64], dS_all [BH, N, 128(dv), 128(dk)].
HMF_API int hmf_gdn_scan_bwd(const void* wqT, const void* kPT, const void* d_o, const float* glast,
                             const float* dhT, float* dh0, void* dvnT, void* dS_all, int B, int H, int T, int N,
                             const unsigned int* dhT_flag, float* peer_dh0, unsigned int* peer_flag,
                             unsigned int epoch, cudaStream_t stream) {
  HMF_REQUIRE(wqT && kPT && d_o && glast && dvnT && dS_all, "gdn_scan_bwd: null tensor");
  HMF_REQUIRE(B > 0 && H > 0 && N > 0 && T > 0 && T <= N * C, "gdn_scan_bwd: bad sizes");
  const long long BH = (long long)B * H;
  HMF_REQUIRE(BH * N * 2 * DK < 2147483647ll, "gdn_scan_bwd: problem too large for 32-bit tile coordinates");
  CUtensorMap tmWQ, tmKP, tmDO;
  int rc;
  if ((rc = make_map_2d_bf16(&tmWQ, wqT, BH * N * 2 * DK, C, C, 2 * DK, C)) != HMF_OK) return rc;
  if ((rc = make_map_2d_bf16(&tmKP, kPT, BH * N * (DK + C), C, C, DK + C, C)) != HMF_OK) return rc;
  {
    uint64_t dims[4] = {(uint64_t)DV, (uint64_t)H, (uint64_t)T, (uint64_t)B};
    uint64_t strides[4] = {2, (uint64_t)DV * 2, (uint64_t)H * DV * 2, (uint64_t)T * H * DV * 2};
    uint32_t box[4] = {64, 1, (uint32_t)C, 1};
    if ((rc = make_tensor_map(&tmDO, d_o, 0, 4, dims, strides, box, 3)) != HMF_OK) return rc;
  }
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(gdn_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BWD));
    configured = true;
  }
  BwdParams p;
  p.glast = glast; p.dhT = dhT; p.dh0 = dh0; p.dvnT = (bf16*)dvnT; p.dS_all = (bf16*)dS_all;
  p.B = B; p.H = H; p.T = T; p.N = N;
  p.dhT_flag = dhT_flag; p.peer_dh0 = peer_dh0; p.peer_flag = peer_flag; p.epoch = epoch;
  p.status = status_ptr();
  gdn_scan_bwd_kernel<<<(unsigned)BH, 192, SMEM_BWD, stream>>>(tmWQ, tmKP, tmDO, p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// Segment s of head h: state contribution seg_state[s * st_p + h * st_h + e] (e < E), log-decays
// glast[s * gl_p + h * gl_h + n] (n < n_seg); h0 [H, E] or null.  Writes the incoming state of every segment to
// s_in[s * in_p + h * in_h + e] and the state after the last one to s_out[h * out_h + e].  All fp32.
HMF_API int hmf_gla_segment_prefix(const float* seg_state, const float* glast, const float* h0, float* s_in, float* s_out,
                                   int P, int H, int n_seg, int E, long long st_p, long long st_h, long long gl_p,
                                   long long gl_h, long long in_p, long long in_h, long long out_h, cudaStream_t stream) {
  HMF_REQUIRE(seg_state && glast && s_in && s_out && P > 0 && H > 0 && n_seg > 0 && E > 0, "gla_segment_prefix: bad arguments");
  HMF_REQUIRE(H <= 65535, "gla_segment_prefix: too many heads");
  dim3 grid((E + 255) / 256, H);
  gla_segment_prefix_kernel<<<grid, 256, 0, stream>>>(seg_state, glast, h0, s_in, s_out, P, n_seg, E, st_p, st_h, gl_p, gl_h,
                                                      in_p, in_h, out_h);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
