// Grouped expert GEMM for mixture-of-experts layers, fused with the expert-parallel all-to-all.
//
// Work is described by *segments*: `rows` consecutive rows of some source buffer that all go through expert
// `expert`.  C_seg = A_seg [rows, K] . W[expert] [N, K]^T.  One persistent kernel walks all (segment, 128-row block,
// 256-column block) tiles (tile table in device memory, built by `moe_build_tables_kernel` without a host round trip).
//
//   * dispatch fused into GEMM 1: the A tiles of a segment are fetched by TMA straight from the *source rank's*
//     send buffer in symmetric memory (one tensor map per source rank, plain non-multicast TMA over NVLink) after that
//     rank's publication flag has been seen (bounded wait);
//   * combine fused into GEMM 2: the epilogue stores each output row straight into the *destination rank's* receive
//     buffer (peer stores); a flag raised after the kernel tells the owner that its rows are complete.
// With one rank (or local buffers) the same kernel is the plain grouped GEMM of a local MoE layer.
//
// Structure per CTA: warp 0 TMA producer (4-stage ring), warp 1 tcgen05.mma issuer (128x256x16, double-buffered TMEM
// accumulators), warps 2-5 epilogue with row masks (rows of a block that belong to the next segment are computed
// but not stored).
#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace moe {

using bf16 = __nv_bfloat16;
constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int MAX_RANKS = 8;
constexpr uint64_t kPeerWaitNs = 2000000000ull;

// Segment / tile tables (device memory, int32 each):
//   seg[6 * s + {0..5}] = src buffer index, first row in the source, rows, expert, destination index, first row there
//   mtile[2 * t + {0, 1}] = segment, 128-row block inside the segment;  counts[0] = number of m-tiles
struct Params {
  const CUtensorMap* a_maps;        // [n_src] in global memory
  const int* seg;
  const int* mtile;
  const int* counts;
  bf16* out[MAX_RANKS + 1];         // destination buffers (peer addresses as mapped here; last = local)
  const unsigned int* src_flags;    // optional: src_flags[r] >= epoch once source r is published
  unsigned int epoch;
  int N, K;
  long long ldc;
  unsigned int* status;
};

__global__ void __launch_bounds__(192, 1)
moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles_n = p.N / BN + (p.N % BN != 0);
  const int num_tiles = p.counts[0] * tiles_n;
  const int num_kb = p.K / BK;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      unsigned int waited = 0u;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int mt = tile / tiles_n, n0 = (tile % tiles_n) * BN;
        const int sg = p.mtile[2 * mt], mb = p.mtile[2 * mt + 1];
        const int src = p.seg[6 * sg], row0 = p.seg[6 * sg + 1] + mb * BM, expert = p.seg[6 * sg + 3];
        if (p.src_flags != nullptr && !((waited >> src) & 1u)) {
          wait_flag_sys(p.src_flags + src, p.epoch, kPeerWaitNs, p.status, 0xB0 + src);
          waited |= 1u << src;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&empty[s], ph ^ 1, ctx, 0x100 + s);
          uint8_t* sA = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          tma_load_2d(sA, p.a_maps + src, &full[s], kb * BK, row0);
          tma_load_3d(sA + A_BYTES, &tmB, &full[s], kb * BK, n0, expert);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, false, false);
      int s = 0, it = 0;
      uint32_t ph = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
        const int a = it & 1;
        mbar_wait(&tempty[a], ((it >> 1) & 1) ^ 1, ctx, 0x200 + a);
        tc_fence_after();
        const uint32_t d = tmem_base + a * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&full[s], ph, ctx, 0x300 + s);
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * STAGE_BYTES), sB = sA + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_ss(d, make_desc_kmajor_sw128(sA + k * 32), make_desc_kmajor_sw128(sB + k * 32), idesc,
                    (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        umma_commit(&tfull[a]);
      }
    }
  } else {
    const int q = warp & 3;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int a = it & 1;
      const int mt = tile / tiles_n, n0 = (tile % tiles_n) * BN;
      const int sg = p.mtile[2 * mt], mb = p.mtile[2 * mt + 1];
      const int rows = p.seg[6 * sg + 2], dst = p.seg[6 * sg + 4], out0 = p.seg[6 * sg + 5];
      const int row = mb * BM + q * 32 + lane;              // row inside the segment
      mbar_wait(&tfull[a], (it >> 1) & 1, ctx, 0x400 + a);
      tc_fence_after();
      const uint32_t tbase = tmem_base + a * BN + ((uint32_t)(q * 32) << 16);
      bf16* orow = p.out[dst] + (size_t)(out0 + row) * p.ldc + n0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(tbase + c * 32, r);
        tmem_ld_wait();
        if (row < rows && n0 + c * 32 < p.N) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            w.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            w.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            w.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            reinterpret_cast<uint4*>(orow + c * 32)[j] = w;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[a]);
    }
    __threadfence_system();       // rows pushed to peers are visible before the completion flag that follows the kernel
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Builds the segment and tile tables of both GEMMs of an expert-parallel MoE layer on this rank.
//   cnt_ptrs[r]: rank r's published count table int32 [world, E_local] (rows r sends to (dest, local expert)),
//                as mapped here; rows in r's send buffer are ordered by (dest, expert).
// Outputs: seg1 / seg2 [6 * world * E_local], mtile [2 * max_mtiles] (shared by both GEMMs), counts[0] = m-tiles,
//          counts[1] = rows received in total, counts[2] = overflow flag (received rows beyond `capacity` are dropped).
__global__ void moe_build_tables_kernel(const int* const* cnt_ptrs, const unsigned int* flags, unsigned int epoch,
                                        int world, int me, int e_local, int capacity, int max_mtiles, int* seg1,
                                        int* seg2, int* mtile, int* counts, unsigned int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int nseg = 0, nmt = 0, loc = 0, overflow = 0;
  for (int r = 0; r < world; ++r) {
    if (flags != nullptr) wait_flag_sys(flags + r, epoch, kPeerWaitNs, status, 0xC0 + r);
    const volatile int* c = cnt_ptrs[r];
    int off = 0;                                   // first row of block (me, 0) in r's send buffer
    for (int d = 0; d < me; ++d)
      for (int e = 0; e < e_local; ++e) off += c[d * e_local + e];
    for (int e = 0; e < e_local; ++e) {
      int rows = c[me * e_local + e];
      if (loc + rows > capacity) { rows = max(0, capacity - loc); overflow = 1; }
      if (rows > 0) {
        int* s1 = seg1 + 6 * nseg;
        int* s2 = seg2 + 6 * nseg;
        s1[0] = r; s1[1] = off; s1[2] = rows; s1[3] = e; s1[4] = MAX_RANKS; s1[5] = loc;     // pull from r, write local
        s2[0] = 0; s2[1] = loc; s2[2] = rows; s2[3] = e; s2[4] = r; s2[5] = off;             // read local, push to r
        for (int mb = 0; mb * BM < rows && nmt < max_mtiles; ++mb) {
          mtile[2 * nmt] = nseg;
          mtile[2 * nmt + 1] = mb;
          ++nmt;
        }
        ++nseg;
      }
      off += c[me * e_local + e];
      loc += rows;
    }
  }
  counts[0] = nmt;
  counts[1] = loc;
  counts[2] = overflow;
}

__global__ void peer_wait_kernel(const unsigned int* flags, int n, unsigned int epoch, unsigned int* status) {
  if ((int)threadIdx.x < n) wait_flag_sys(flags + threadIdx.x, epoch, kPeerWaitNs, status, 0xD0 + threadIdx.x);
}

}  // namespace moe
}  // namespace hmf

using namespace hmf;
using namespace hmf::moe;

HMF_API int hmf_moe_build_tables(const void* cnt_ptrs_dev, const unsigned int* flags, unsigned int epoch, int world,
                                 int me, int e_local, int capacity, int max_mtiles, int* seg1, int* seg2, int* mtile,
                                 int* counts, cudaStream_t st) {
  HMF_REQUIRE(world >= 1 && world <= MAX_RANKS && me >= 0 && me < world, "moe tables: bad rank %d / world %d", me, world);
  moe_build_tables_kernel<<<1, 32, 0, st>>>((const int* const*)cnt_ptrs_dev, flags, epoch, world, me, e_local, capacity,
                                            max_mtiles, seg1, seg2, mtile, counts, status_ptr());
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// Waits (bounded) on the device until flags[0..n) >= epoch; later work on the stream runs after it.
HMF_API int hmf_peer_wait(const unsigned int* flags, int n, unsigned int epoch, cudaStream_t st) {
  HMF_REQUIRE(n >= 1 && n <= 32, "peer_wait: %d flags unsupported", n);
  peer_wait_kernel<<<1, 32, 0, st>>>(flags, n, epoch, status_ptr());
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// a_ptrs: n_src device addresses of row-major [a_rows, K] bf16 buffers (peer buffers as mapped here);
// maps_dev: n_src * 128 bytes of 64-byte aligned device scratch, untouched until the kernel has finished;
// w: [E_local, N, K] bf16; out_ptrs: MAX_RANKS + 1 addresses (slot MAX_RANKS = local buffer); row stride ldc.
HMF_API int hmf_moe_grouped_gemm(const unsigned long long* a_ptrs, int n_src, long long a_rows, void* maps_dev,
                                 const void* w, int e_local, int N, int K, const unsigned long long* out_ptrs,
                                 long long ldc, const int* seg, const int* mtile, const int* counts,
                                 const unsigned int* src_flags, unsigned int epoch, int sm_count, cudaStream_t st) {
  HMF_REQUIRE(n_src >= 1 && n_src <= MAX_RANKS, "moe gemm: %d sources unsupported", n_src);
  HMF_REQUIRE(K % BK == 0 && N % 32 == 0 && ldc % 8 == 0, "moe gemm: K=%d must be a multiple of 64, N=%d of 32", K, N);
  HMF_REQUIRE(((uintptr_t)maps_dev & 63) == 0, "moe gemm: descriptor scratch must be 64-byte aligned");
  CUtensorMap host_maps[MAX_RANKS];
  int rc;
  for (int r = 0; r < n_src; ++r)
    if ((rc = make_map_2d_bf16(&host_maps[r], reinterpret_cast<const void*>(a_ptrs[r]), a_rows, K, K, BM, BK)) != HMF_OK)
      return rc;
  HMF_CHECK_CUDA(cudaMemcpyAsync(maps_dev, host_maps, sizeof(CUtensorMap) * n_src, cudaMemcpyHostToDevice, st));
  CUtensorMap tmB;
  {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)e_local};
    uint64_t strides[3] = {2, (uint64_t)K * 2, (uint64_t)N * K * 2};
    uint32_t box[3] = {BK, BN, 1};
    if ((rc = make_tensor_map(&tmB, w, 0, 3, dims, strides, box, 3)) != HMF_OK) return rc;
  }
  static bool configured = false;
  if (!configured) {
    HMF_CHECK_CUDA(cudaFuncSetAttribute(moe_grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  Params p;
  p.a_maps = reinterpret_cast<const CUtensorMap*>(maps_dev);
  p.seg = seg; p.mtile = mtile; p.counts = counts;
  for (int i = 0; i <= MAX_RANKS; ++i) p.out[i] = reinterpret_cast<bf16*>(out_ptrs[i]);
  p.src_flags = src_flags; p.epoch = epoch;
  p.N = N; p.K = K; p.ldc = ldc;
  p.status = status_ptr();
  moe_grouped_gemm_kernel<<<sm_count > 0 ? sm_count : 148, 192, SMEM_BYTES, st>>>(tmB, p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}
