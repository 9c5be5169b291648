// Persistent warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] = op(A) * op(B)^T (+ bias) , fp32 accumulation in tensor memory.
//
// Operand storage (row-major in global memory):
//   A K-major : A[M,K]   (activations in a forward linear)
//   A MN-major: A[K,M]   (dY^T in a weight gradient, read without a transpose pass)
//   B K-major : B[N,K]   (nn.Linear weight in forward)
//   B MN-major: B[K,N]   (weight in the input gradient, X in the weight gradient)
//
// Structure per CTA (one per SM, persistent over output tiles of 128x256):
//   warp 0   : TMA producer  (cp.async.bulk.tensor, 128B swizzle, 4-stage ring)
//   warp 1   : MMA issuer    (tcgen05.mma 128x256x16, one thread), owns the TMEM allocation
//   warps 2-5: epilogue      (tcgen05.ld -> registers -> global), double-buffered accumulators
//                             so the epilogue of tile i overlaps the main loop of tile i+1.
#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int PANEL_BYTES = BK * 128;  // one 64-wide MN panel of an MN-major operand
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;

enum OutMode : int { kOutBf16 = 0, kOutF32 = 1, kOutF32Accumulate = 2 };

// Grouped forms (mixture-of-experts layers; rows sorted by expert, every group padded to whole 128-row tiles):
//   GMODE 1, grouped rows:        C[rows of group g] = A[rows of group g] . op(B_g)^T.  `mtile_group[m_tile]` names the
//            group of every 128-row tile (-1: tile unused, skipped by every role); B holds the groups stacked
//            ([G*N, K] K-major or [G*K, N] MN-major).
//   GMODE 2, grouped contraction: C_g[M, N] = A[k range of g, M]^T . B[k range of g, N] (weight gradients of all
//            experts in one launch); `k_offsets[g] .. k_offsets[g+1]` (multiples of 64) is the row range of group g in
//            the MN-major A and B, C holds the groups stacked ([G*M, N]).  An empty group writes zeros.
struct Params {
  void* C;
  const float* bias;  // [N] or null
  int M, N, K;
  long long ldc;
  int out_mode;
  unsigned int* status;
  const int* mtile_group;   // GMODE 1
  const int* k_offsets;     // GMODE 2
  int groups;
};

// Tile order: groups of GROUP_M row tiles are walked column by column, so the CTAs that run at the same time
// (consecutive tile ids) cover a block of about 16 x 9 tiles and share 16 A panels and 9 B panels through L2,
// instead of one B panel and 148 A panels (measured before the change: 7.6x the algorithmic DRAM reads at 8192^3).
constexpr int GROUP_M = 16;
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(tiles_m - first_m, GROUP_M);
  const int r = tile - g * per_group;
  m0 = (first_m + r % gsz) * BM;
  n0 = (r / gsz) * BN;
}

// Work item `tile` of the persistent loop -> output tile origin, group and contraction range.  Returns false for a
// tile that no role touches.
template <int GMODE>
__device__ __forceinline__ bool tile_work(const Params& p, int tile, int tiles_m, int tiles_n, int& m0, int& n0,
                                          int& group, int& k_first, int& num_kb) {
  group = 0;
  k_first = 0;
  num_kb = (p.K + BK - 1) / BK;
  if (GMODE == 2) {
    const int per = tiles_m * tiles_n;
    group = tile / per;
    tile_coords(tile - group * per, tiles_m, tiles_n, m0, n0);
    k_first = p.k_offsets[group];
    num_kb = (p.k_offsets[group + 1] - k_first) / BK;
    return true;
  }
  tile_coords(tile, tiles_m, tiles_n, m0, n0);
  if (GMODE == 1) {
    group = p.mtile_group[m0 / BM];
    return group >= 0;
  }
  return true;
}

template <bool A_MN, bool B_MN, int GMODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES]
  uint64_t* empty = bars + STAGES;          // [STAGES]
  uint64_t* tfull = bars + 2 * STAGES;      // [2]
  uint64_t* tempty = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n * (GMODE == 2 ? p.groups : 1);

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int m0, n0, group, k_first, num_kb;
        if (!tile_work<GMODE>(p, tile, tiles_m, tiles_n, m0, n0, group, k_first, num_kb)) continue;
        // stacked B of the grouped-rows form: group g starts at row g*N (K-major) or g*K (MN-major)
        const int b_row0 = GMODE == 1 ? group * (B_MN ? p.K : p.N) : 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&empty[s], ph ^ 1, ctx, 0x100 + s);
          uint8_t* sA = smem + s * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          const int k0 = k_first + kb * BK;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(sA, &tmA, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int pn = 0; pn < BM / 64; ++pn)
              tma_load_2d(sA + pn * PANEL_BYTES, &tmA, &full[s], m0 + pn * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(sB, &tmB, &full[s], k0, b_row0 + n0);
          } else {
#pragma unroll
            for (int pn = 0; pn < BN / 64; ++pn)
              tma_load_2d(sB + pn * PANEL_BYTES, &tmB, &full[s], n0 + pn * 64, b_row0 + k0);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int m0, n0, group, k_first, num_kb;
        if (!tile_work<GMODE>(p, tile, tiles_m, tiles_n, m0, n0, group, k_first, num_kb) || num_kb == 0) continue;
        const int a = it & 1;
        mbar_wait(&tempty[a], ((it >> 1) & 1) ^ 1, ctx, 0x200 + a);
        tc_fence_after();
        const uint32_t d = tmem_base + a * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&full[s], ph, ctx, 0x300 + s);
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = A_MN ? make_desc_mnmajor_sw128(sA + k * 2048, PANEL_BYTES)
                                     : make_desc_kmajor_sw128(sA + k * 32);
            const uint64_t bd = B_MN ? make_desc_mnmajor_sw128(sB + k * 2048, PANEL_BYTES)
                                     : make_desc_kmajor_sw128(sB + k * 32);
            umma_ss(d, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        umma_commit(&tfull[a]);
        ++it;
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quadrant this warp can reach
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int m0, n0, group, k_first, num_kb;
      if (!tile_work<GMODE>(p, tile, tiles_m, tiles_n, m0, n0, group, k_first, num_kb)) continue;
      const int a = it & 1;
      const int row = m0 + q * 32 + lane;
      const long long crow = (GMODE == 2 ? (long long)group * p.M : 0) + row;   // row of the stacked output
      const bool have_acc = num_kb > 0;          // an empty group of the grouped-contraction form: zeros, no MMA ran
      if (have_acc) {
        mbar_wait(&tfull[a], (it >> 1) & 1, ctx, 0x400 + a);
        tc_fence_after();
      }
      const uint32_t tbase = tmem_base + a * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        if (have_acc) {
          tmem_ld_x32(tbase + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) v[j] += p.bias[col0 + j];
          }
          const bool full_vec = (col0 + 32 <= p.N);
          if (p.out_mode == kOutBf16) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)crow * p.ldc + col0;
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
            float* out = reinterpret_cast<float*>(p.C) + (size_t)crow * p.ldc + col0;
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
      if (have_acc) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[a]);
        ++it;
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

template <bool A_MN, bool B_MN, int GMODE = 0>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p,
                  cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, GMODE>;
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  const long long tiles = (long long)((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * (GMODE == 2 ? p.groups : 1);
  int grid = tiles < sm_count() ? (int)tiles : sm_count();
  if (grid < 1) grid = 1;
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

}  // namespace gemm
}  // namespace hmf

// C = op(A) op(B)^T (+bias).  lda/ldb/ldc are row strides (elements) of the stored matrices.
//   a_mn_major = 0: A stored [M,K];  1: A stored [K,M]
//   b_mn_major = 0: B stored [N,K];  1: B stored [K,N]
//   out_mode   = 0: bf16 C;  1: fp32 C;  2: fp32 C += result
// Requirements: pointers 16-byte aligned, lda/ldb multiples of 8 elements.
HMF_API int hmf_gemm_bf16(const void* A, const void* B, void* C, const float* bias, int M, int N,
                          int K, long long lda, long long ldb, long long ldc, int a_mn_major,
                          int b_mn_major, int out_mode, cudaStream_t stream) {
  using namespace hmf;
  using namespace hmf::gemm;
  HMF_REQUIRE(A && B && C, "gemm: null operand");
  HMF_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem %d x %d x %d", M, N, K);
  HMF_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "gemm: lda=%lld ldb=%lld must be multiples of 8", lda, ldb);
  HMF_REQUIRE(out_mode >= 0 && out_mode <= 2, "gemm: out_mode %d", out_mode);
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn_major) {
    rc = make_map_2d_bf16(&tmA, A, M, K, lda, BM, BK);
  } else {
    rc = make_map_2d_bf16(&tmA, A, K, M, lda, BK, 64);
  }
  if (rc != HMF_OK) return rc;
  if (!b_mn_major) {
    rc = make_map_2d_bf16(&tmB, B, N, K, ldb, BN, BK);
  } else {
    rc = make_map_2d_bf16(&tmB, B, K, N, ldb, BK, 64);
  }
  if (rc != HMF_OK) return rc;
  Params p{C, bias, M, N, K, ldc, out_mode, status_ptr(), nullptr, nullptr, 1};
  if (!a_mn_major && !b_mn_major) return launch<false, false>(tmA, tmB, p, stream);
  if (!a_mn_major && b_mn_major) return launch<false, true>(tmA, tmB, p, stream);
  if (a_mn_major && !b_mn_major) return launch<true, false>(tmA, tmB, p, stream);
  return launch<true, true>(tmA, tmB, p, stream);
}


// Grouped rows: C[R, N] = A[R, K] . op(B_g)^T where g = mtile_group[row / 128] (device int32 [ceil(R / 128)], -1 = tile
// not used: its rows of C are left untouched).  B holds `groups` matrices stacked: [groups*N, K] (b_mn_major = 0,
// the layout of stacked nn.Linear weights) or [groups*K, N] (b_mn_major = 1: input gradients).  bf16 in and out.
HMF_API int hmf_grouped_gemm_bf16(const void* A, const void* B, void* C, const int* mtile_group, int R, int N, int K,
                                  int groups, long long lda, long long ldb, long long ldc, int b_mn_major,
                                  cudaStream_t stream) {
  using namespace hmf;
  using namespace hmf::gemm;
  HMF_REQUIRE(A && B && C && mtile_group, "grouped gemm: null operand");
  HMF_REQUIRE(R > 0 && N > 0 && K > 0 && groups > 0, "grouped gemm: empty problem %d x %d x %d (%d groups)", R, N, K, groups);
  HMF_REQUIRE(R % BM == 0, "grouped gemm: %d rows are not whole 128-row tiles", R);
  HMF_REQUIRE(lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0, "grouped gemm: strides must be multiples of 8");
  HMF_REQUIRE(!b_mn_major || K % BK == 0, "grouped gemm: MN-major B needs K %% 64 == 0 (K = %d)", K);
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = make_map_2d_bf16(&tmA, A, R, K, lda, BM, BK)) != HMF_OK) return rc;
  rc = b_mn_major ? make_map_2d_bf16(&tmB, B, (uint64_t)groups * K, N, ldb, BK, 64)
                  : make_map_2d_bf16(&tmB, B, (uint64_t)groups * N, K, ldb, BN, BK);
  if (rc != HMF_OK) return rc;
  Params p{C, nullptr, R, N, K, ldc, kOutBf16, status_ptr(), mtile_group, nullptr, groups};
  return b_mn_major ? launch<false, true, 1>(tmA, tmB, p, stream) : launch<false, false, 1>(tmA, tmB, p, stream);
}

// Grouped contraction (weight gradients of every group in one launch): C_g[M, N] = A[k_g .. k_{g+1}, M]^T .
// B[k_g .. k_{g+1}, N] with k_offsets (device int32 [groups + 1], multiples of 64).  A stored [Rtot, M], B stored
// [Rtot, N], C stored [groups*M, N] bf16 (a group without rows gets zeros).
HMF_API int hmf_grouped_gemm_wgrad_bf16(const void* A, const void* B, void* C, const int* k_offsets, int Rtot, int M,
                                        int N, int groups, long long lda, long long ldb, long long ldc,
                                        cudaStream_t stream) {
  using namespace hmf;
  using namespace hmf::gemm;
  HMF_REQUIRE(A && B && C && k_offsets, "grouped wgrad: null operand");
  HMF_REQUIRE(Rtot > 0 && M > 0 && N > 0 && groups > 0, "grouped wgrad: empty problem");
  HMF_REQUIRE(lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0, "grouped wgrad: strides must be multiples of 8");
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = make_map_2d_bf16(&tmA, A, Rtot, M, lda, BK, 64)) != HMF_OK) return rc;
  if ((rc = make_map_2d_bf16(&tmB, B, Rtot, N, ldb, BK, 64)) != HMF_OK) return rc;
  Params p{C, nullptr, M, N, Rtot, ldc, kOutBf16, status_ptr(), nullptr, k_offsets, groups};
  return launch<true, true, 2>(tmA, tmB, p, stream);
}
