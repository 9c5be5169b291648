// bf16 GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a.
//
//   C[M,N] = op(A) * op(B)^T (+ bias), fp32 accumulation in tensor memory; same operand contract as gemm_bf16.cu.
//
// Two CTAs on the two SMs of one TPC work on one 256 x 256 output tile.  Each CTA loads its own 128 rows of A and its
// own 128 of the 256 columns of B, so a k-block costs every SM 32 KB of shared-memory fill and 32 KB of operand reads
// instead of 48 + 48 KB with a 128 x 256 tile per CTA: the MMA of the pair reads B from both shared memories.  The
// leader CTA (even cluster rank) issues the MMAs for both; each CTA keeps the accumulator of its own 128 rows in its
// own tensor memory and writes them out itself.
//
//   warp 0   : TMA producer of this CTA (6-stage ring; plain per-CTA loads, completion bytes reported to the leader's
//              mbarrier; no cluster multicast)
//   warp 1   : tensor-memory allocation in both CTAs; in the leader: MMA issuer (tcgen05.mma.cta_group::2 256x256x16)
//   warps 2-5: epilogue of this CTA's rows (tcgen05.ld -> registers -> global), accumulators double-buffered so the
//              epilogue of tile i overlaps the main loop of tile i+1
//
// Barriers: full[s] lives in the leader (1 arrival + the bytes of both CTAs); empty[s] and tfull[a] are signalled in
// both CTAs by a multicast tcgen05.commit; tempty[a] lives in the leader and collects the 4 + 4 epilogue warps.
#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace gemm2 {

constexpr int BM = 128;            // rows per CTA (256 per pair)
constexpr int BN = 256;            // columns per pair; each CTA loads BN / 2 of them
constexpr int BNH = BN / 2;
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;    // 16 KB
constexpr int B_BYTES = BNH * BK * 2;   // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int PANEL_BYTES = BK * 128;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;         // tile order: 8 x 256 rows by ~9 x 256 columns in flight (see gemm_bf16.cu)

enum OutMode : int { kOutBf16 = 0, kOutF32 = 1, kOutF32Accumulate = 2 };

struct Params {
  void* C;
  const float* bias;
  int M, N, K;
  long long ldc;
  int out_mode;
  unsigned int* status;
  const float* scale_a;   // fp8 form: per-row scales of A [M] and of B [N]; C = (A_q B_q^T) * scale_a[m] * scale_b[n]
  const float* scale_b;
  int fmt_a, fmt_b;       // fp8 form: 0 = e4m3, 1 = e5m2
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(tiles_m - first_m, GROUP_M);
  const int r = tile - g * per_group;
  m0 = (first_m + r % gsz) * (2 * BM);
  n0 = (r / gsz) * BN;
}

// FP8 = true: both operands are 8-bit floats, K-major, 128 elements (one 128-byte swizzled row) per k-block, and the
// epilogue applies the row scales of the two operands (row-wise scaled float8 training).
template <bool A_MN, bool B_MN, bool FP8 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared memory starts at the same offset in both CTAs, so the aligned tile area does too
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                      // [STAGES]  used in the leader
  uint64_t* empty = bars + STAGES;            // [STAGES]  one per CTA
  uint64_t* tfull = bars + 2 * STAGES;        // [2]       one per CTA
  uint64_t* tempty = bars + 2 * STAGES + 2;   // [2]       used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();    // 0 = leader of the pair
  const bool leader = rank == 0;
  const WaitCtx ctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);               // 4 epilogue warps of each CTA
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  // both CTAs have initialised their barriers before either sends anything to the other
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  constexpr int BKE = FP8 ? 2 * BK : BK;      // elements per k-block (a 128-byte row either way)
  const int num_kb = (p.K + BKE - 1) / BKE;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs) {
        int m0, n0;
        tile_coords(tile, tiles_m, tiles_n, m0, n0);
        m0 += rank * BM;                      // this CTA's rows of A
        const int nb = n0 + rank * BNH;       // this CTA's columns of B
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&empty[s], ph ^ 1, ctx, 0x500 + s);
          uint8_t* sA = smem + s * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          if (leader) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);   // bytes of both CTAs land on the leader's barrier
          if (!A_MN) {
            tma_load_2d_pair(sA, &tmA, &full[s], kb * BKE, m0);
          } else {
#pragma unroll
            for (int pn = 0; pn < BM / 64; ++pn)
              tma_load_2d_pair(sA + pn * PANEL_BYTES, &tmA, &full[s], m0 + pn * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sB, &tmB, &full[s], kb * BKE, nb);
          } else {
#pragma unroll
            for (int pn = 0; pn < BNH / 64; ++pn)
              tma_load_2d_pair(sB + pn * PANEL_BYTES, &tmB, &full[s], nb + pn * 64, kb * BK);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      const uint32_t idesc = FP8 ? make_idesc_f8(2 * BM, BN, p.fmt_a, p.fmt_b) : make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
        const int a = it & 1;
        mbar_wait(&tempty[a], ((it >> 1) & 1) ^ 1, ctx, 0x600 + a);
        tc_fence_after();
        const uint32_t d = tmem_base + a * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&full[s], ph, ctx, 0x700 + s);
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = A_MN ? make_desc_mnmajor_sw128(sA + k * 2048, PANEL_BYTES)
                                     : make_desc_kmajor_sw128(sA + k * 32);
            const uint64_t bd = B_MN ? make_desc_mnmajor_sw128(sB + k * 2048, PANEL_BYTES)
                                     : make_desc_kmajor_sw128(sB + k * 32);
            if (FP8) umma_ss_pair_f8(d, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_ss_pair(d, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[s]);        // both CTAs may refill the stage
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        umma_commit_pair(&tfull[a]);          // both CTAs' epilogues may read their accumulators
      }
    }
  } else {
    const int q = warp & 3;
    int it = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
      const int a = it & 1;
      int m0, n0;
      tile_coords(tile, tiles_m, tiles_n, m0, n0);
      const int row = m0 + rank * BM + q * 32 + lane;
      const float sa = (FP8 && row < p.M) ? p.scale_a[row] : 1.f;
      mbar_wait(&tfull[a], (it >> 1) & 1, ctx, 0x800 + a);
      tc_fence_after();
      const uint32_t tbase = tmem_base + a * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(tbase + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (FP8) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= sa * (col0 + j < p.N ? p.scale_b[col0 + j] : 0.f);
          }
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) v[j] += p.bias[col0 + j];
          }
          const bool full_vec = (col0 + 32 <= p.N);
          if (p.out_mode == kOutBf16) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0;
            if (full_vec && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 w;
                w.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
                w.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
                w.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
                w.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
                reinterpret_cast<uint4*>(out)[j] = w;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) out[j] = __float2bfloat16(v[j]);
            }
          } else {
            float* out = reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col0;
            const bool acc = p.out_mode == kOutF32Accumulate;
            if (full_vec && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 w = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                if (acc) {
                  const float4 o = reinterpret_cast<float4*>(out)[j];
                  w.x += o.x; w.y += o.y; w.z += o.z; w.w += o.w;
                }
                reinterpret_cast<float4*>(out)[j] = w;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) out[j] = acc ? out[j] + v[j] : v[j];
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tempty[a]);     // the leader's MMA thread waits for both CTAs
    }
  }

  // neither CTA may leave (or free tensor memory) while the other can still signal its barriers or run MMAs on it
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, bool FP8 = false>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p, cudaStream_t stream) {
  auto kern = gemm_bf16_2cta_kernel<A_MN, B_MN, FP8>;
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN);
  int pairs = sm_count() / 2;
  if (tiles < pairs) pairs = tiles;
  if (pairs < 1) pairs = 1;
  kern<<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

}  // namespace gemm2
}  // namespace hmf

// Same contract as hmf_gemm_bf16 (see gemm_bf16.cu), on CTA pairs.
HMF_API int hmf_gemm_bf16_2cta(const void* A, const void* B, void* C, const float* bias, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major,
                               int out_mode, cudaStream_t stream) {
  using namespace hmf;
  using namespace hmf::gemm2;
  HMF_REQUIRE(A && B && C, "gemm: null operand");
  HMF_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem %d x %d x %d", M, N, K);
  HMF_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "gemm: lda=%lld ldb=%lld must be multiples of 8", lda, ldb);
  HMF_REQUIRE(out_mode >= 0 && out_mode <= 2, "gemm: out_mode %d", out_mode);
  CUtensorMap tmA, tmB;
  int rc;
  rc = !a_mn_major ? make_map_2d_bf16(&tmA, A, M, K, lda, BM, BK) : make_map_2d_bf16(&tmA, A, K, M, lda, BK, 64);
  if (rc != HMF_OK) return rc;
  rc = !b_mn_major ? make_map_2d_bf16(&tmB, B, N, K, ldb, BNH, BK) : make_map_2d_bf16(&tmB, B, K, N, ldb, BK, 64);
  if (rc != HMF_OK) return rc;
  Params p{C, bias, M, N, K, ldc, out_mode, status_ptr(), nullptr, nullptr, 0, 0};
  if (!a_mn_major && !b_mn_major) return launch<false, false>(tmA, tmB, p, stream);
  if (!a_mn_major && b_mn_major) return launch<false, true>(tmA, tmB, p, stream);
  if (a_mn_major && !b_mn_major) return launch<true, false>(tmA, tmB, p, stream);
  return launch<true, true>(tmA, tmB, p, stream);
}


// Row-wise scaled float8 GEMM: C[M,N] = (A_q[M,K] . B_q[N,K]^T) * scale_a[m] * scale_b[n] (+ bias), A_q / B_q 8-bit
// floats (fmt 0 = e4m3, 1 = e5m2) stored K-major with row strides lda / ldb in bytes = elements, fp32 accumulation.
// Requirements: 16-byte aligned pointers, lda / ldb multiples of 16.
HMF_API int hmf_gemm_fp8_2cta(const void* A, const void* B, void* C, const float* scale_a, const float* scale_b,
                              const float* bias, int M, int N, int K, long long lda, long long ldb, long long ldc,
                              int fmt_a, int fmt_b, int out_mode, cudaStream_t stream) {
  using namespace hmf;
  using namespace hmf::gemm2;
  HMF_REQUIRE(A && B && C && scale_a && scale_b, "fp8 gemm: null operand");
  HMF_REQUIRE(M > 0 && N > 0 && K > 0, "fp8 gemm: empty problem %d x %d x %d", M, N, K);
  HMF_REQUIRE(lda % 16 == 0 && ldb % 16 == 0, "fp8 gemm: lda=%lld ldb=%lld must be multiples of 16", lda, ldb);
  HMF_REQUIRE(fmt_a >= 0 && fmt_a <= 1 && fmt_b >= 0 && fmt_b <= 1, "fp8 gemm: formats must be 0 (e4m3) or 1 (e5m2)");
  HMF_REQUIRE(out_mode >= 0 && out_mode <= 1, "fp8 gemm: out_mode %d", out_mode);
  CUtensorMap tmA, tmB;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t strides[2] = {1, (uint64_t)lda};
    uint32_t box[2] = {2 * BK, BM};
    if ((rc = make_tensor_map(&tmA, A, 2, 2, dims, strides, box, 3)) != HMF_OK) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t strides[2] = {1, (uint64_t)ldb};
    uint32_t box[2] = {2 * BK, BNH};
    if ((rc = make_tensor_map(&tmB, B, 2, 2, dims, strides, box, 3)) != HMF_OK) return rc;
  }
  Params p{C, bias, M, N, K, ldc, out_mode, status_ptr(), scale_a, scale_b, fmt_a, fmt_b};
  return launch<false, false, true>(tmA, tmB, p, stream);
}
