// Flash attention forward for sm_100a: tcgen05 tensor cores, accumulators in tensor memory,
// operands staged by TMA.  GQA, causal / sliding-window / hollow-window masks expressed as
//     key visible  <=>  lo <= q_pos - k_pos < hi ,
// bottom-right aligned causal for Tq < Tk via q_off, optional explicit query positions (query-
// sparse attention), log-sum-exp output.
//
// One CTA handles one 128-row query tile of one (batch, head); two CTAs are resident per SM so
// that one CTA's softmax overlaps the other's tensor-core work.
//   warp 0    : TMA loads (Q once; K and V tiles of 64 keys through 2-stage rings)
//   warp 1    : tcgen05.mma issue.  S_j = Q K_j^T (SS, 128x64xD) into a double-buffered S region;
//               O += P_j V_j (TS: P read from tensor memory, V MN-major in shared memory)
//   warps 2-5 : softmax, one query row per thread (no shuffles): tcgen05.ld S, mask, running max with
//               lazy rescaling of O (only when the max grows by more than 2^8), exp2, bf16 P stored back
//               over S by tcgen05.st; final O / l and LSE written straight to global memory.
// Tensor-memory map (256 columns; 512 at D = 256): S0 [0,64) S1 [64,128) O [128,128+D).  P_j aliases the first
// 32 columns of S_j.  At D = 256 (Qwen3-Next gated attention) the tiles take 192 KB, so one CTA runs per SM.
#include <float.h>
#include <math.h>

#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace attn {

constexpr int BM = 128;
constexpr int BN = 64;
constexpr int NTHREADS = 192;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct FwdParams {
  __nv_bfloat16* o;  // [B, Tq, Hq, D] contiguous
  float* lse;        // [B, Hq, Tq]
  const int* q_pos;  // optional [B, Tq]
  int B, Tq, Tk, Hq, Hkv;
  int lo, hi, q_off;
  float scale_log2;
  unsigned int* status;
  // context parallelism: keys / values live in 2*SP zig-zag chunks spread over the ranks' symmetric buffers.
  // src_maps = [K map of chunk 0 .. n_chunks-1 | V map of chunk 0 .. n_chunks-1] in global memory (each over
  // [B, chunk_len, Hkv, D] of the owner's buffer); src_flags[r] >= epoch once rank r has published its K/V.
  const CUtensorMap* src_maps;
  const unsigned int* src_flags;
  int n_chunks, chunk_len;
  unsigned int epoch;
};

constexpr uint64_t kPeerWaitNs = 2000000000ull;

template <int D>
struct Smem {
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int KV_BYTES = BN * D * 2;
  static constexpr int Q_PANEL = BM * 128;
  static constexpr int KV_PANEL = BN * 128;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + 2 * KV_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(NTHREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  using L = Smem<D>;
  constexpr int TMEM_COLS = (128 + D) <= 256 ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;   // [2]
  uint64_t* p_full = bars + 11;  // [2]
  uint64_t* o_done = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};
  const int h = blockIdx.x;
  const int qt = (int)gridDim.y - 1 - (int)blockIdx.y;  // longest tiles first
  const int b = blockIdx.z;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q0 = qt * BM;
  const int rows_valid = min(BM, p.Tq - q0);

  // key-tile range visible to this query tile
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
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
    }
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tS = [&](int s) -> uint32_t { return tmem_base + (uint32_t)s * 64u; };
  const uint32_t tO = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int pn = 0; pn < D / 64; ++pn) tma_load_4d(sQ + pn * L::Q_PANEL, &tmQ, q_full, pn * 64, h, q0, b);
      unsigned int waited = 0u;   // owners whose publication flag has been seen
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        int k0 = (j0 + j) * BN;
        const CUtensorMap* km = &tmK;
        const CUtensorMap* vm = &tmV;
        if (p.src_maps != nullptr) {
          // remote tile: plain (non-multicast) TMA from the owner's memory over NVLink
          const int c = k0 / p.chunk_len;
          const int sp = p.n_chunks >> 1;
          const int owner = c < sp ? c : p.n_chunks - 1 - c;
          if (!((waited >> owner) & 1u)) {
            wait_flag_sys(p.src_flags + owner, p.epoch, kPeerWaitNs, p.status, 0xA0 + owner);
            waited |= 1u << owner;
          }
          km = p.src_maps + c;
          vm = p.src_maps + p.n_chunks + c;
          k0 -= c * p.chunk_len;
        }
        mbar_wait(&k_empty[s], par, ctx, 0x10 + s);
        mbar_expect_tx(&k_full[s], L::KV_BYTES);
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn)
          tma_load_4d(sK + s * L::KV_BYTES + pn * L::KV_PANEL, km, &k_full[s], pn * 64, hkv, k0, b);
        mbar_wait(&v_empty[s], par, ctx, 0x20 + s);
        mbar_expect_tx(&v_full[s], L::KV_BYTES);
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn)
          tma_load_4d(sV + s * L::KV_BYTES + pn * L::KV_PANEL, vm, &v_full[s], pn * 64, hkv, k0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idescS = make_idesc_bf16(BM, BN, false, false);
      constexpr uint32_t idescPV = make_idesc_bf16(BM, D, false, true);
      const uint32_t aQ = smem_u32(sQ);
      auto issue_S = [&](int j) {
        const int s = j & 1;
        mbar_wait(&k_full[s], (j >> 1) & 1, ctx, 0x30 + s);
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + s * L::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t ad = make_desc_kmajor_sw128(aQ + (kk / 4) * L::Q_PANEL + (kk % 4) * 32);
          const uint64_t bd = make_desc_kmajor_sw128(aK + (kk / 4) * L::KV_PANEL + (kk % 4) * 32);
          umma_ss(tS(s), ad, bd, idescS, kk > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[s]);
      };
      mbar_wait(q_full, 0, ctx, 0x40);
      issue_S(0);
      if (n_tiles > 1) issue_S(1);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        const uint32_t par = (j >> 1) & 1;
        mbar_wait(&v_full[s], par, ctx, 0x50 + s);
        mbar_wait(&p_full[s], par, ctx, 0x60 + s);
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + s * L::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t bd = make_desc_mnmajor_sw128(aV + kk * 2048, L::KV_PANEL);
          umma_ts(tO, tS(s) + kk * 8, bd, idescPV, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[s]);
        umma_commit(o_done);
        if (j + 2 < n_tiles) issue_S(j + 2);
      }
    }
  } else {
    // ---------------- softmax: thread <-> query row ----------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int row = q0 + r;
    const bool row_ok = row < p.Tq;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    long long prow = 0;
    if (row_ok) prow = p.q_pos ? (long long)p.q_pos[(size_t)b * p.Tq + row] : (long long)row + p.q_off;
    float m_stale = -INFINITY, l = 0.f;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      const int k0 = (j0 + j) * BN;
      mbar_wait(&s_full[s], (j >> 1) & 1, ctx, 0x70 + s);
      tc_fence_after();
      uint32_t sr[64];
      tmem_ld_x32(tS(s) + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
      tmem_ld_x32(tS(s) + lane_off + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
      tmem_ld_wait();
      const bool full_vis = (pmin - (long long)(k0 + BN - 1) >= (long long)p.lo) &&
                            (pmax - (long long)k0 < (long long)p.hi) && (k0 + BN <= p.Tk);
      float mx = -INFINITY;
      if (!full_vis) {
        long long chi = prow - k0 - (long long)p.lo;  // visible: c <= chi
        long long clo = prow - k0 - (long long)p.hi;  // visible: c >  clo
        const long long cend = (long long)p.Tk - k0 - 1;
        if (chi > cend) chi = cend;
        if (!row_ok) chi = -1;
        const int ichi = (int)max(-1ll, min(chi, 1000ll));
        const int iclo = (int)max(-1ll, min(clo, 1000ll));
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const bool vis = (c <= ichi) && (c > iclo);
          const float v = vis ? __uint_as_float(sr[c]) : -INFINITY;
          sr[c] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) mx = fmaxf(mx, __uint_as_float(sr[c]));
      }
      const float m_new = mx * p.scale_log2;
      const bool grow = m_new > m_stale + kRescaleThreshold;  // false when m_new == -inf
      if (__any_sync(0xffffffffu, grow)) {
        const float m_next = fmaxf(m_stale, m_new);
        const float alpha = (m_stale == -INFINITY) ? 0.f : exp2f(m_stale - m_next);
        if (j > 0) {
          mbar_wait(o_done, (j - 1) & 1, ctx, 0x80);
          tc_fence_after();
#pragma unroll
          for (int ch = 0; ch < D / 32; ++ch) {
            uint32_t o[32];
            tmem_ld_x32(tO + lane_off + ch * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(tO + lane_off + ch * 32, o);
          }
          tmem_st_wait();
        }
        l *= alpha;
        m_stale = m_next;
      }
      const float offs = (m_stale == -INFINITY) ? 0.f : m_stale;
      float rs = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = exp2f(fmaf(__uint_as_float(sr[c]), p.scale_log2, -offs));
        const float p1 = exp2f(fmaf(__uint_as_float(sr[c + 1]), p.scale_log2, -offs));
        rs += p0 + p1;
        pk[c >> 1] = pack_bf16x2(p0, p1);
      }
      l += rs;
      tmem_st_x32(tS(s) + lane_off, pk);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[s]);
    }
    // ---------------- epilogue ----------------
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (n_tiles > 0) {
      mbar_wait(o_done, (n_tiles - 1) & 1, ctx, 0x90);
      tc_fence_after();
    }
    __nv_bfloat16* orow = p.o + (((size_t)b * p.Tq + row) * p.Hq + h) * D;
#pragma unroll
    for (int ch = 0; ch < D / 32; ++ch) {
      uint32_t o[32];
      if (n_tiles > 0) {
        tmem_ld_x32(tO + lane_off + ch * 32, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
          w.y = pack_bf16x2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
          w.z = pack_bf16x2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
          w.w = pack_bf16x2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
          reinterpret_cast<uint4*>(orow + ch * 32)[i] = w;
        }
      }
    }
    if (row_ok && p.lse)
      p.lse[((size_t)b * p.Hq + h) * p.Tq + row] =
          l > 0.f ? (m_stale * 0.6931471805599453f + __logf(l)) : -INFINITY;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

static int make_map_bthd(CUtensorMap* m, const void* base, int B, int T, int H, int D, long long sb,
                         long long st, long long sh, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[4] = {2, (uint64_t)sh * 2, (uint64_t)st * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_tensor_map(m, base, 0, 4, dims, strides, box, 3);
}

template <int D>
static int launch(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const FwdParams& p,
                  cudaStream_t st) {
  auto kern = attn_fwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<D>::TOTAL));
    configured = true;
  }
  dim3 grid(p.Hq, (p.Tq + BM - 1) / BM, p.B);
  kern<<<grid, NTHREADS, Smem<D>::TOTAL, st>>>(tmQ, tmK, tmV, p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

}  // namespace attn
}  // namespace hmf

// q [B,Tq,Hq,D], k/v [B,Tk,Hkv,D] bf16 with element strides (batch, token, head) and unit inner
// stride; o [B,Tq,Hq,D] contiguous bf16; lse [B,Hq,Tq] fp32 (may be null).
// Mask: key j visible to query i  <=>  lo <= pos_i - j < hi,  pos_i = q_pos ? q_pos[b,i] : i + q_off.
// q_pos rows must be ascending within a batch entry.  scale multiplies q k^T.
HMF_API int hmf_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                              const int* q_pos, int B, int Tq, int Tk, int Hq, int Hkv, int D,
                              long long q_sb, long long q_st, long long q_sh, long long k_sb, long long k_st,
                              long long k_sh, long long v_sb, long long v_st, long long v_sh, int lo, int hi,
                              int q_off, float scale, cudaStream_t stream) {
  using namespace hmf;
  using namespace hmf::attn;
  HMF_REQUIRE(q && k && v && o, "attention: null tensor");
  HMF_REQUIRE(D == 64 || D == 128 || D == 256, "attention: head dim %d unsupported (64, 128, 256)", D);
  HMF_REQUIRE(Hkv > 0 && Hq % Hkv == 0, "attention: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  HMF_REQUIRE(B > 0 && Tq > 0 && Tk > 0, "attention: empty problem");
  HMF_REQUIRE(lo >= 0 && hi > lo, "attention: bad window lo=%d hi=%d", lo, hi);
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_map_bthd(&tmQ, q, B, Tq, Hq, D, q_sb, q_st, q_sh, BM);
  if (rc != HMF_OK) return rc;
  rc = make_map_bthd(&tmK, k, B, Tk, Hkv, D, k_sb, k_st, k_sh, BN);
  if (rc != HMF_OK) return rc;
  rc = make_map_bthd(&tmV, v, B, Tk, Hkv, D, v_sb, v_st, v_sh, BN);
  if (rc != HMF_OK) return rc;
  FwdParams p;
  p.o = (__nv_bfloat16*)o;
  p.lse = lse;
  p.q_pos = q_pos;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv;
  p.lo = lo; p.hi = hi; p.q_off = q_off;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_ptr();
  p.src_maps = nullptr; p.src_flags = nullptr; p.n_chunks = 0; p.chunk_len = 0; p.epoch = 0;
  if (D == 64) return launch<64>(tmQ, tmK, tmV, p, stream);
  if (D == 256) return launch<256>(tmQ, tmK, tmV, p, stream);   // one CTA per SM: 192 KB of tiles, 384 TMEM columns
  return launch<128>(tmQ, tmK, tmV, p, stream);
}

namespace hmf {
namespace attn {
__global__ void peer_signal_kernel(unsigned int* const* flags, int n, int index, unsigned int value) {
  if ((int)threadIdx.x < n) {
    __threadfence_system();
    st_release_sys(flags[threadIdx.x] + index, value);
  }
}
}  // namespace attn
}  // namespace hmf

// Raises flag[index] = value on every rank of `flag_ptrs` (device array of n addresses, one per rank, as mapped
// into this process).  Work queued before on the stream (the copies into the symmetric K/V buffers) is complete
// and visible to the peers when they see the flag.
HMF_API int hmf_peer_signal(const void* flag_ptrs_dev, int n, int index, unsigned int value, cudaStream_t stream) {
  using namespace hmf;
  HMF_REQUIRE(n >= 1 && n <= 32, "peer_signal: %d ranks unsupported", n);
  hmf::attn::peer_signal_kernel<<<1, 32, 0, stream>>>((unsigned int* const*)flag_ptrs_dev, n, index, value);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// Context-parallel forward: queries are local ([B, Tq, Hq, D]); keys / values of global chunk c
// (c = 0 .. n_vis-1, chunk_len tokens each) are read from kv_ptrs[c] / kv_ptrs[n_chunks + c] (host array of
// device addresses of [B, chunk_len, Hkv, D] blocks with batch stride kv_sb elements, in the owners' symmetric
// buffers).  maps_dev: 2 * n_chunks * 128 bytes of device scratch (64-byte aligned) that stays untouched until the
// kernel has finished.  flags_local[r] >= epoch signals that rank r's buffers are complete.
HMF_API int hmf_attention_fwd_cp(const void* q, const unsigned long long* kv_ptrs, void* maps_dev,
                                 const unsigned int* flags_local, unsigned int epoch, void* o, float* lse, int B,
                                 int Tq, int chunk_len, int n_chunks, int n_vis, int Hq, int Hkv, int D,
                                 long long q_sb, long long q_st, long long q_sh, long long kv_sb, int lo, int hi,
                                 int q_off, float scale, cudaStream_t stream) {
  using namespace hmf;
  using namespace hmf::attn;
  HMF_REQUIRE(q && kv_ptrs && maps_dev && flags_local && o, "attention_cp: null argument");
  HMF_REQUIRE(D == 64 || D == 128, "attention_cp: head dim %d unsupported (64, 128)", D);
  HMF_REQUIRE(n_chunks >= 2 && n_chunks <= 64 && n_chunks % 2 == 0 && n_vis >= 1 && n_vis <= n_chunks,
              "attention_cp: bad chunk counts %d / %d", n_vis, n_chunks);
  HMF_REQUIRE(chunk_len % BN == 0, "attention_cp: chunk length %d must be a multiple of %d", chunk_len, BN);
  HMF_REQUIRE(((uintptr_t)maps_dev & 63) == 0, "attention_cp: descriptor scratch must be 64-byte aligned");
  CUtensorMap tmQ;
  int rc = make_map_bthd(&tmQ, q, B, Tq, Hq, D, q_sb, q_st, q_sh, BM);
  if (rc != HMF_OK) return rc;
  CUtensorMap host_maps[128];
  for (int i = 0; i < 2 * n_chunks; ++i) {
    const int c = i % n_chunks;
    const unsigned long long base = kv_ptrs[c < n_vis ? i : (i / n_chunks) * n_chunks];   // unused chunks alias chunk 0
    rc = make_map_bthd(&host_maps[i], reinterpret_cast<const void*>(base), B, chunk_len, Hkv, D, kv_sb,
                       (long long)Hkv * D, D, BN);
    if (rc != HMF_OK) return rc;
  }
  HMF_CHECK_CUDA(cudaMemcpyAsync(maps_dev, host_maps, sizeof(CUtensorMap) * 2 * n_chunks, cudaMemcpyHostToDevice, stream));
  FwdParams p;
  p.o = (__nv_bfloat16*)o;
  p.lse = lse;
  p.q_pos = nullptr;
  p.B = B; p.Tq = Tq; p.Tk = n_vis * chunk_len; p.Hq = Hq; p.Hkv = Hkv;
  p.lo = lo; p.hi = hi; p.q_off = q_off;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_ptr();
  p.src_maps = reinterpret_cast<const CUtensorMap*>(maps_dev);
  p.src_flags = flags_local;
  p.n_chunks = n_chunks; p.chunk_len = chunk_len; p.epoch = epoch;
  if (D == 64) return launch<64>(tmQ, host_maps[0], host_maps[n_chunks], p, stream);
  return launch<128>(tmQ, host_maps[0], host_maps[n_chunks], p, stream);
}
