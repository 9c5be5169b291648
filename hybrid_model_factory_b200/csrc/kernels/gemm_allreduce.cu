// Row-parallel GEMM fused with its tensor-parallel all-reduce over peer memory (decode-sized M).
//
//   y[M, N] = sum over ranks r of  x_r[M, Ks] . W_r[N, Ks]^T          (Ks = K / world, M <= 256)
//
// One kernel per rank, one CTA per (128 output columns, K split); the K splits of a tile exist only to put more SMs
// on the weight stream (a row-parallel shard has few 128-column tiles) and are summed in the same reduction:
//   1. swap-AB tcgen05 GEMM: D^T[128 cols x Mpad] = W_tile[128 x Ks] . x^T   (A = weight rows and B = activations,
//      both K-major, TMA -> shared memory ring -> tcgen05.mma, accumulator in tensor memory);
//   2. the partial tile goes (bf16) to this rank's slot of a symmetric buffer; a release store raises the
//      tile's flag on every peer;
//   3. the CTA waits (bounded) for the same tile's flag from every rank, loads the W partials over NVLink with
//      plain peer loads, adds them in rank order (every rank gets bit-identical results) and stores y.
// The transfer of a tile overlaps the GEMM of the other tiles; no separate collective kernel is launched.
//
// Two more forms share the kernel:
//   * reduce-scatter (mode 1): the 128-column tiles are owned in contiguous blocks of N / (128 world) tiles per rank; a
//     CTA raises its tile's flag on the owner only, and only the owner's CTA reduces, into y_shard [M, N / world];
//   * all-gather -> GEMM (x_maps != null): the activations are sharded over the ranks along K ([M, Ks] each, in
//     symmetric buffers); the TMA producer fetches every k-block of x from its owner's buffer (plain, non-multicast
//     TMA over NVLink) after that rank's publication flag has been seen, so y = concat_r(x_r) . W^T needs no separate
//     all-gather.  There is no cross-rank sum in this form (the reduction runs over this rank's own partial).
//
//   * NVLS (mc_part != null): in the reduction step one multimem.ld_reduce through the NVSwitch multicast mapping of
//     the partial buffers replaces the `world` peer loads per 16 bytes (the sum happens inside the switch).
//
// Epochs come from device memory (`sync[0]`, advanced by the last CTA of each launch), so the kernel can be
// replayed from a CUDA graph.  Partials are double-buffered by epoch parity: a rank can only be one launch
// ahead of the slowest peer because it needs that peer's flags to finish a launch.
#include "../common/host.h"
#include "../common/sm100.cuh"

namespace hmf {
namespace gar {

using bf16 = __nv_bfloat16;

constexpr int BN = 128;          // output columns (weight rows) per CTA = MMA M
constexpr int BK = 64;           // K per stage (one 128-byte swizzle atom)
constexpr int MAX_STAGES = 8;
constexpr int A_BYTES = BN * BK * 2;             // 16 KB
constexpr int MAX_M = 256;
// Shared memory per CTA: `stages` x (A tile 16 KB + B tile Mpad x 128 B rounded up to 1 KB) + barriers.  The ring is
// sized by the launch: few activation rows leave room for a deeper ring AND a second CTA on the SM, whose prologue
// and epilogue then overlap the other CTA's weight stream.
constexpr int BAR_BYTES = 256;
__host__ __device__ inline int b_stage_bytes(int Mpad) { return (Mpad * BK * 2 + 1023) / 1024 * 1024; }
constexpr int MAX_WORLD = 8;
constexpr int MAX_SPLIT = 4;
constexpr int FLAGS_PER_TILE = MAX_WORLD * MAX_SPLIT;
constexpr uint64_t kPeerWaitNs = 2000000000ull;

struct Params {
  bf16* y;                          // [M, N] local result
  bf16* part[MAX_WORLD];            // every rank's partial buffers [2][splits][M * N] as mapped here
  unsigned int* flags[MAX_WORLD];   // every rank's flag array [max_tiles][MAX_WORLD * MAX_SPLIT]
  unsigned int* sync;               // local: [0] epoch of the last finished launch, [1] CTA ticket
  unsigned int* status;
  long long part_stride;            // elements between the two parity buffers
  int M, N, Ks, Mpad, rank, world, tmem_cols, splits;
  int mode;                         // 0 all-reduce, 1 reduce-scatter
  int ldy, tiles_per_rank;          // reduce-scatter: row stride of y_shard, tiles owned by each rank
  const CUtensorMap* x_maps;        // all-gather form: [ag_world] maps of the ranks' x shards (global memory)
  const unsigned int* x_flags;      // x_flags[r] >= x_epoch once rank r has published its shard
  unsigned int x_epoch;
  int ag_world, ag_ks;              // ranks and K per rank of the gathered activations
  const bf16* mc_part;              // NVLS form: the partial buffers through their NVSwitch multicast mapping (or null)
  const bf16* bias;                 // [N] added to the result (or null)
  int direct;                       // one rank, one K split: the accumulator goes straight to y (no partial, no flags)
  int stages, b_bytes;              // depth of the shared-memory ring, bytes of one B stage
  int part_f32;                     // single-GPU K splits: the partials stay fp32 (the buffers hold half as many)
  int cluster_split;                // single-GPU K splits as one thread-block cluster: partials meet in shared memory
};

// One load that returns the sum over every rank's copy of 8 bf16 values (reduced inside NVSwitch, fp32 accumulation).
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const bf16* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}

// NVLS variant of the tile reduction: the cross-rank sum is one multimem.ld_reduce per 16 bytes instead of `world`
// peer loads; the K splits (separate partial buffers) are added here.
__device__ __forceinline__ void reduce_tile_nvls(const Params& p, int et, int chunks, int ksp, int n0, unsigned parity,
                                                 size_t split_elems, int y_col0) {
  for (int c = et; c < chunks; c += 128) {
    const int m = ksp + (c / (BN / 8)) * p.splits, cc = (c % (BN / 8)) * 8;
    const size_t off = (size_t)m * p.N + n0 + cc;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int sp = 0; sp < p.splits; ++sp) {
      const uint4 u = multimem_ld_reduce_bf16x8(p.mc_part + (size_t)parity * p.part_stride + off + (size_t)sp * split_elems);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h2[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(p.y + (size_t)m * p.ldy + (n0 - y_col0) + cc) = o;
  }
}

// Single-GPU K splits: fp32 partials of this GPU, summed in split order (no rounding before the final conversion).
__device__ __forceinline__ void reduce_tile_f32(const Params& p, int et, int chunks, int ksp, int n0, unsigned parity,
                                                size_t split_elems) {
  const float* base = reinterpret_cast<const float*>(p.part[0]) + (size_t)parity * (p.part_stride / 2);
  for (int c = et; c < chunks; c += 128) {
    const int m = ksp + (c / (BN / 8)) * p.splits, cc = (c % (BN / 8)) * 8;
    const size_t off = (size_t)m * p.N + n0 + cc;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = p.bias != nullptr ? __bfloat162float(p.bias[n0 + cc + j]) : 0.f;
    for (int sp = 0; sp < p.splits; ++sp) {
      const float* src = base + off + (size_t)sp * split_elems;
      float4 a, b;
      asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w) : "l"(src));
      asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(b.x), "=f"(b.y), "=f"(b.z), "=f"(b.w) : "l"(src + 4));
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(p.y + (size_t)m * p.ldy + n0 + cc) = o;
  }
}

// Rank-ordered sum of every (rank, split) partial of one tile.  Remote loads take microseconds, so they go out in
// batches before the first use: 8 partials of CU chunks at a time.  The sums are still taken in (rank, split) order,
// so every rank gets the same bits.
template <int CU>
__device__ __forceinline__ void reduce_tile(const Params& p, int et, int chunks, int ksp, int n0, unsigned parity,
                                            size_t split_elems, int y_col0) {
  const int total = p.world * p.splits;
  for (int c0 = et; c0 < chunks; c0 += 128 * CU) {
    float acc[CU][8];
    size_t off[CU], yoff[CU];
#pragma unroll
    for (int q = 0; q < CU; ++q) {
      const int c = c0 + q * 128;
      const int m = ksp + (c / (BN / 8)) * p.splits, cc = (c % (BN / 8)) * 8;
      off[q] = (size_t)m * p.N + n0 + cc;
      yoff[q] = (size_t)m * p.ldy + (n0 - y_col0) + cc;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[q][j] = 0.f;
    }
    for (int rs0 = 0; rs0 < total; rs0 += 8) {
      uint4 u[CU][8];
#pragma unroll
      for (int q = 0; q < CU; ++q) {
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          const int rs = rs0 + b;
          if (rs < total && c0 + q * 128 < chunks) {
            const bf16* src = p.part[rs / p.splits] + (size_t)parity * p.part_stride + off[q] +
                              (size_t)(rs % p.splits) * split_elems;
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(u[q][b].x), "=r"(u[q][b].y), "=r"(u[q][b].z), "=r"(u[q][b].w)
                         : "l"(src));
          } else {
            u[q][b] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
#pragma unroll
      for (int q = 0; q < CU; ++q) {
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u[q][b]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h2[j]);
            acc[q][2 * j] += f.x;
            acc[q][2 * j + 1] += f.y;
          }
        }
      }
    }
#pragma unroll
    for (int q = 0; q < CU; ++q) {
      if (c0 + q * 128 < chunks) {
        if (p.bias != nullptr) {
          const int cc = ((c0 + q * 128) % (BN / 8)) * 8;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[q][j] += __bfloat162float(p.bias[n0 + cc + j]);
        }
        uint4 o;
        o.x = pack_bf16x2(acc[q][0], acc[q][1]);
        o.y = pack_bf16x2(acc[q][2], acc[q][3]);
        o.z = pack_bf16x2(acc[q][4], acc[q][5]);
        o.w = pack_bf16x2(acc[q][6], acc[q][7]);
        *reinterpret_cast<uint4*>(p.y + yoff[q]) = o;
      }
    }
  }
}

// PAIR: two CTAs per SM (the single-GPU skinny GEMM: short ring, small reduction); otherwise one CTA per SM with
// the full register budget for the batched remote loads of the cross-rank reduction.
template <bool PAIR>
__global__ void __launch_bounds__(192, PAIR ? 2 : 1)
gemm_allreduce_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int STAGES = p.stages, B_BYTES = p.b_bytes;
  const int OFF_A = 0, OFF_B = STAGES * A_BYTES, OFF_BAR = OFF_B + STAGES * B_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* full = bars;                 // [MAX_STAGES]
  uint64_t* empty = bars + MAX_STAGES;   // [MAX_STAGES]
  uint64_t* acc_done = bars + 2 * MAX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};
  const int tile = blockIdx.x / p.splits, ksp = blockIdx.x % p.splits;
  const int n0 = tile * BN;
  const int k_steps = p.Ks / p.splits / BK;
  const int kb0 = ksp * k_steps;
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(p.sync) + 1u;
  const int parity = (int)(epoch & 1u);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t bytes = A_BYTES + (uint32_t)p.Mpad * BK * 2;
      unsigned int x_seen = 0u;
      for (int i = 0; i < k_steps; ++i) {
        const int s = i % STAGES;
        if (i >= STAGES) mbar_wait(&empty[s], ((i / STAGES) - 1) & 1, ctx, 0x10 + s);
        mbar_expect_tx(&full[s], bytes);
        tma_load_2d(smem + OFF_A + s * A_BYTES, &tmW, &full[s], (kb0 + i) * BK, n0);
        if (p.x_maps == nullptr) {
          tma_load_2d(smem + OFF_B + s * B_BYTES, &tmX, &full[s], (kb0 + i) * BK, 0);
        } else {
          const int kg = (kb0 + i) * BK;                 // column of the gathered activations
          const int src = kg / p.ag_ks;
          if (!((x_seen >> src) & 1u)) {
            wait_flag_sys(p.x_flags + src, p.x_epoch, kPeerWaitNs, p.status, 0x50 + src);
            x_seen |= 1u << src;
          }
          tma_load_2d(smem + OFF_B + s * B_BYTES, p.x_maps + src, &full[s], kg - src * p.ag_ks, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BN, p.Mpad, false, false);
      for (int i = 0; i < k_steps; ++i) {
        const int s = i % STAGES;
        mbar_wait(&full[s], (i / STAGES) & 1, ctx, 0x20 + s);
        tc_fence_after();
        const uint32_t a = smem_u32(smem + OFF_A + s * A_BYTES), b = smem_u32(smem + OFF_B + s * B_BYTES);
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk)
          umma_ss(tmem_base, make_desc_kmajor_sw128(a + kk * 32), make_desc_kmajor_sw128(b + kk * 32), idesc,
                  (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&empty[s]);
      }
      umma_commit(acc_done);
    }
  } else {
    // ---------------- epilogue: partial store, flags, cross-rank reduction ----------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;                 // output column n0 + row
    const int et = threadIdx.x - 64;                  // 0..127
    const uint32_t lane_bits = (uint32_t)(quad * 32) << 16;
    const size_t split_elems = (size_t)p.M * p.N;
    bf16* mine = p.part[p.rank] + (size_t)parity * p.part_stride + (size_t)ksp * split_elems;
    mbar_wait(acc_done, 0, ctx, 0x30);
    tc_fence_after();
    if (p.cluster_split) {
      // the K splits of a tile are the CTAs of one cluster: the fp32 partial goes to this CTA's shared memory (the
      // ring is idle once the accumulator is complete) and is summed below, after a cluster barrier, through
      // distributed shared memory -- no global scratch, no flags, no polling
      float* stg = reinterpret_cast<float*>(smem);
      for (int m0 = 0; m0 < p.Mpad; m0 += 16) {
        uint32_t v[16];
        tmem_ld_x16(tmem_base + lane_bits + m0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) stg[(m0 + j) * BN + row] = __uint_as_float(v[j]);
      }
    } else if (p.direct) {
      // single-GPU skinny GEMM: thread = output column, a warp writes 32 consecutive columns of one row per store
      const float bv = p.bias != nullptr ? __bfloat162float(p.bias[n0 + row]) : 0.f;
      for (int m0 = 0; m0 < p.Mpad; m0 += 16) {
        uint32_t v[16];
        tmem_ld_x16(tmem_base + lane_bits + m0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (m0 + j < p.M) p.y[(size_t)(m0 + j) * p.ldy + n0 + row] = __float2bfloat16(__uint_as_float(v[j]) + bv);
      }
    } else {
    float* mine_f = reinterpret_cast<float*>(p.part[p.rank]) + (size_t)parity * (p.part_stride / 2) +
                    (size_t)ksp * split_elems;
    for (int m0 = 0; m0 < p.Mpad; m0 += 16) {
      uint32_t v[16];
      tmem_ld_x16(tmem_base + lane_bits + m0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (m0 + j < p.M) {
          if (p.part_f32) mine_f[(size_t)(m0 + j) * p.N + n0 + row] = __uint_as_float(v[j]);
          else mine[(size_t)(m0 + j) * p.N + n0 + row] = __float2bfloat16(__uint_as_float(v[j]));
        }
    }
    // the CTA barrier orders every thread's partial stores before the (cumulative) system-scope release stores
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int owner = p.mode == 1 ? tile / p.tiles_per_rank : -1;     // reduce-scatter: the rank that owns the tile
    if (et < p.world && (owner < 0 || et == owner))
      st_release_sys(p.flags[et] + (size_t)tile * FLAGS_PER_TILE + p.rank * p.splits + ksp, epoch);
    const bool reduce_here = owner < 0 || owner == p.rank;
    if (reduce_here && et < p.world * p.splits)
      wait_flag_sys(p.flags[p.rank] + (size_t)tile * FLAGS_PER_TILE + et, epoch, kPeerWaitNs, p.status, 0x40 + et);
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // this CTA reduces the rows m = ksp, ksp + splits, ... of the tile: rows x 16 chunks of 8 columns, summed over
    // every (rank, split) partial in a fixed order
    const int rows = (p.M - ksp + p.splits - 1) / p.splits;
    const int chunks = rows * (BN / 8);
    // few chunks per thread (many K splits): two at a time; a whole 64-row tile per CTA (8 ranks, no splits): four, so
    // the tile takes two rounds of remote latency instead of four
    const int y_col0 = p.mode == 1 ? p.rank * p.tiles_per_rank * BN : 0;
    if (reduce_here && p.part_f32) {
      reduce_tile_f32(p, et, chunks, ksp, n0, parity, split_elems);
    } else if (reduce_here && p.mc_part != nullptr) {
      reduce_tile_nvls(p, et, chunks, ksp, n0, parity, split_elems, y_col0);
    } else if (reduce_here) {
      if (!PAIR && chunks > 256) reduce_tile<4>(p, et, chunks, ksp, n0, parity, split_elems, y_col0);
      else reduce_tile<PAIR ? 1 : 2>(p, et, chunks, ksp, n0, parity, split_elems, y_col0);
    }
    }  // !direct
  }

  if (p.cluster_split) {
    tc_fence_before();
    __syncthreads();
    cluster_arrive();                 // release: every CTA's partial is in its shared memory
    cluster_wait();
    if (warp >= 2) {
      // CTA `ksp` sums the rows ksp, ksp + splits, ...; thread = output column, so every remote read is one
      // contiguous 128-byte line per warp
      const int col = (warp & 3) * 32 + lane;
      const uint32_t local = smem_u32(smem);
      const float bv = p.bias != nullptr ? __bfloat162float(p.bias[n0 + col]) : 0.f;
      uint32_t remote[MAX_SPLIT];
      for (int sp = 0; sp < p.splits; ++sp)
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[sp]) : "r"(local), "r"(sp));
      for (int m = ksp; m < p.M; m += p.splits) {
        float acc = bv;
        for (int sp = 0; sp < p.splits; ++sp) {
          float v;
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote[sp] + (uint32_t)(m * BN + col) * 4u));
          acc += v;
        }
        p.y[(size_t)m * p.ldy + n0 + col] = __float2bfloat16(acc);
      }
    }
    cluster_arrive();                 // nobody leaves while a peer may still read its shared memory
    cluster_wait();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  // the last CTA of the launch publishes the epoch for the next launch
  if (threadIdx.x == 0 && !p.direct && !p.cluster_split) {
    __threadfence();
    const unsigned int ticket = atomicAdd(p.sync + 1, 1u);
    if (ticket == gridDim.x - 1) {
      p.sync[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(p.sync) = epoch;
    }
  }
}

}  // namespace gar
}  // namespace hmf

using namespace hmf;
using namespace hmf::gar;

static int launch_tp(const void* x, const void* w, void* y, int M, int N, int Ks, long long ldx, long long ldw,
                     const unsigned long long* part_ptrs, const unsigned long long* flag_ptrs, unsigned int* sync,
                     long long part_stride, int max_tiles, int rank, int world, int splits, int mode,
                     const unsigned long long* x_ptrs, void* maps_dev, const unsigned int* x_flags,
                     unsigned int x_epoch, int ag_world, const void* mc_part, cudaStream_t st, int x_epoch_flags = 0,
                     const void* bias = nullptr, bool allow_direct = false) {
  const int Ktot = x_ptrs ? Ks * ag_world : Ks;
  HMF_REQUIRE(splits >= 1 && splits <= MAX_SPLIT && Ktot % (splits * BK) == 0,
              "tp gemm: %d K splits do not divide K=%d into multiples of 64", splits, Ktot);
  HMF_REQUIRE(M >= 1 && M <= MAX_M, "tp gemm: M=%d out of range (1..%d)", M, MAX_M);
  HMF_REQUIRE(N % BN == 0 && Ks % BK == 0 && Ks > 0, "tp gemm: N=%d must be a multiple of 128, Ks=%d of 64", N, Ks);
  HMF_REQUIRE(world >= 1 && world <= MAX_WORLD && rank >= 0 && rank < world, "tp gemm: bad rank %d / world %d", rank, world);
  // only the plain single-GPU GEMM skips the partial / flag protocol; the tensor-parallel entry points keep it on one
  // rank too (that is how the protocol is tested without peers)
  const bool direct = allow_direct && world == 1 && splits == 1 && mode == 0 && x_ptrs == nullptr && mc_part == nullptr;
  HMF_REQUIRE(direct || N / BN <= max_tiles, "tp gemm: %d tiles exceed the flag array (%d)", N / BN, max_tiles);
  const bool part_f32 = allow_direct && !direct && world == 1 && mode == 0 && x_ptrs == nullptr && mc_part == nullptr;
  HMF_REQUIRE(direct || (long long)M * N * splits * (part_f32 ? 2 : 1) <= part_stride,
              "tp gemm: partial buffer too small");
  HMF_REQUIRE(bias == nullptr || mc_part == nullptr, "tp gemm: no bias in the NVLS form");
  HMF_REQUIRE(mode == 0 || (N / BN) % world == 0, "tp gemm: reduce-scatter needs N / 128 = %d tiles divisible by %d ranks",
              N / BN, world);
  CUtensorMap tmW, tmX;
  int rc;
  const int Mpad = (M + 15) / 16 * 16;
  if ((rc = make_map_2d_bf16(&tmW, w, N, Ktot, ldw, BN, BK)) != HMF_OK) return rc;
  Params p;
  p.x_maps = nullptr; p.x_flags = nullptr; p.x_epoch = 0; p.ag_world = 1; p.ag_ks = Ks;
  if (x_ptrs == nullptr) {
    if ((rc = make_map_2d_bf16(&tmX, x, M, Ks, ldx, Mpad, BK)) != HMF_OK) return rc;
  } else {
    HMF_REQUIRE(maps_dev && x_flags && ag_world >= 1 && ag_world <= MAX_WORLD, "tp gemm: bad all-gather arguments");
    HMF_REQUIRE(((uintptr_t)maps_dev & 63) == 0, "tp gemm: descriptor scratch must be 64-byte aligned");
    CUtensorMap host_maps[MAX_WORLD];
    for (int r = 0; r < ag_world; ++r)
      if ((rc = make_map_2d_bf16(&host_maps[r], reinterpret_cast<const void*>(x_ptrs[r]), M, Ks, ldx, Mpad, BK)) != HMF_OK)
        return rc;
    if (!(x_epoch_flags & 1))
      HMF_CHECK_CUDA(cudaMemcpyAsync(maps_dev, host_maps, sizeof(CUtensorMap) * ag_world, cudaMemcpyHostToDevice, st));
    tmX = host_maps[0];
    p.x_maps = reinterpret_cast<const CUtensorMap*>(maps_dev);
    p.x_flags = x_flags; p.x_epoch = x_epoch; p.ag_world = ag_world;
  }
  // ring depth: as many stages as fit in half an SM's shared memory (two CTAs per SM), at least 3; a launch with many
  // activation rows takes the whole SM with 4 stages
  const int bst = b_stage_bytes(Mpad);
  int stages = (100 * 1024 - BAR_BYTES - 1024) / (A_BYTES + bst);
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  const bool pair = world == 1 && x_ptrs == nullptr && stages >= 3;
  if (!pair) stages = 4;
  const int smem_bytes = stages * (A_BYTES + bst) + BAR_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    const int most = 4 * (A_BYTES + b_stage_bytes(MAX_M)) + BAR_BYTES + 1024;
    HMF_CHECK_CUDA(cudaFuncSetAttribute(gemm_allreduce_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
    HMF_CHECK_CUDA(cudaFuncSetAttribute(gemm_allreduce_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
    configured = true;
  }
  p.y = (bf16*)y;
  for (int r = 0; r < MAX_WORLD; ++r) {
    p.part[r] = r < world ? reinterpret_cast<bf16*>(part_ptrs[r]) : nullptr;
    p.flags[r] = r < world ? reinterpret_cast<unsigned int*>(flag_ptrs[r]) : nullptr;
  }
  p.sync = sync;
  p.status = status_ptr();
  p.part_stride = part_stride;
  p.M = M; p.N = N; p.Ks = Ktot; p.Mpad = Mpad; p.rank = rank; p.world = world; p.splits = splits;
  p.mode = mode;
  p.mc_part = (const bf16*)mc_part;
  p.bias = (const bf16*)bias;
  p.direct = direct ? 1 : 0;
  p.stages = stages;
  p.part_f32 = part_f32 ? 1 : 0;
  // the cluster form needs the fp32 tile (Mpad x 128 x 4 bytes) to fit in the ring of the two-CTAs-per-SM variant
  const bool cluster_split = part_f32 && pair && splits > 1 && Mpad * BN * 4 <= stages * (A_BYTES + bst);
  p.cluster_split = cluster_split ? 1 : 0;
  p.b_bytes = bst;
  p.tiles_per_rank = mode == 1 ? (N / BN) / world : N / BN;
  p.ldy = mode == 1 ? N / world : N;
  int cols = 32;
  while (cols < Mpad) cols *= 2;
  p.tmem_cols = cols;
  if (cluster_split) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N / BN) * splits);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;        // consecutive CTAs = the K splits of one tile
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    HMF_CHECK_CUDA(cudaLaunchKernelEx(&cfg, gemm_allreduce_kernel<true>, tmW, tmX, p));
  } else if (pair) gemm_allreduce_kernel<true><<<(N / BN) * splits, 192, smem_bytes, st>>>(tmW, tmX, p);
  else gemm_allreduce_kernel<false><<<(N / BN) * splits, 192, smem_bytes, st>>>(tmW, tmX, p);
  HMF_CHECK_CUDA(cudaGetLastError());
  return HMF_OK;
}

// x [M, Ks] bf16 (row stride ldx), w [N, Ks] bf16 (row stride ldw), y [M, N] bf16.
// part_ptrs / flag_ptrs: `world` device addresses (this process' mappings of every rank's buffers);
// sync: two zero-initialised uint32 on this device, shared by every launch that uses the same buffers.
// flag arrays hold max_tiles * 32 words; partial buffers 2 * part_stride elements with part_stride >= splits * M * N.
HMF_API int hmf_gemm_allreduce(const void* x, const void* w, void* y, int M, int N, int Ks, long long ldx,
                               long long ldw, const unsigned long long* part_ptrs,
                               const unsigned long long* flag_ptrs, unsigned int* sync, long long part_stride,
                               int max_tiles, int rank, int world, int splits, cudaStream_t st) {
  return launch_tp(x, w, y, M, N, Ks, ldx, ldw, part_ptrs, flag_ptrs, sync, part_stride, max_tiles, rank, world, splits,
                   0, nullptr, nullptr, nullptr, 0, 1, nullptr, st);
}

// The all-reduce (mode 0) and reduce-scatter (mode 1) forms with the cross-rank sum done inside NVSwitch:
// mc_part is the multicast address of the partial buffers (the same offset as part_ptrs[r] in every rank's buffer).
HMF_API int hmf_gemm_reduce_nvls(const void* x, const void* w, void* y, int M, int N, int Ks, long long ldx,
                                 long long ldw, const unsigned long long* part_ptrs,
                                 const unsigned long long* flag_ptrs, unsigned int* sync, long long part_stride,
                                 int max_tiles, int rank, int world, int splits, int mode, const void* mc_part,
                                 cudaStream_t st) {
  HMF_REQUIRE(mc_part != nullptr && (mode == 0 || mode == 1), "gemm_reduce_nvls: bad arguments");
  return launch_tp(x, w, y, M, N, Ks, ldx, ldw, part_ptrs, flag_ptrs, sync, part_stride, max_tiles, rank, world, splits,
                   mode, nullptr, nullptr, nullptr, 0, 1, mc_part, st);
}

// Single-GPU skinny GEMM (decode-sized M <= 256): y [M, N] = x [M, K] . w [N, K]^T + bias, the swap-AB kernel above on
// one rank.  splits == 1: the accumulator is stored straight to y.  splits > 1 (few 128-column tiles: K is split over
// more SMs to stream the weight): the splits are summed through the LOCAL partial / flag buffers as in the
// multi-rank forms; the grid must then fit on the device at once (the caller keeps tiles * splits <= the SM count).
HMF_API int hmf_gemm_skinny(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, long long ldx,
                            long long ldw, const unsigned long long* part_ptrs, const unsigned long long* flag_ptrs,
                            unsigned int* sync, long long part_stride, int max_tiles, int splits, cudaStream_t st) {
  return launch_tp(x, w, y, M, N, K, ldx, ldw, part_ptrs, flag_ptrs, sync, part_stride, max_tiles, 0, 1, splits, 0,
                   nullptr, nullptr, nullptr, 0, 1, nullptr, st, 0, bias, true);
}

// Row-parallel GEMM fused with a reduce-scatter over the output columns: y_shard [M, N / world] holds columns
// [rank * N / world, (rank + 1) * N / world) of sum_r x_r W_r^T.  Other arguments as hmf_gemm_allreduce.
HMF_API int hmf_gemm_reduce_scatter(const void* x, const void* w, void* y_shard, int M, int N, int Ks, long long ldx,
                                    long long ldw, const unsigned long long* part_ptrs,
                                    const unsigned long long* flag_ptrs, unsigned int* sync, long long part_stride,
                                    int max_tiles, int rank, int world, int splits, cudaStream_t st) {
  return launch_tp(x, w, y_shard, M, N, Ks, ldx, ldw, part_ptrs, flag_ptrs, sync, part_stride, max_tiles, rank, world,
                   splits, 1, nullptr, nullptr, nullptr, 0, 1, nullptr, st);
}

// All-gather fused into a column-parallel GEMM: y [M, N] = concat_r(x_r) [M, ag_world * Ks] . w [N, ag_world * Ks]^T,
// where x_r [M, Ks] (row stride ldx) is rank r's shard at x_ptrs[r] (this process' mapping of the symmetric buffers)
// and x_flags[r] >= x_epoch (local flags) says that shard is complete.  maps_dev: ag_world * 128 bytes of 64-byte
// aligned device scratch, untouched until the kernel has finished.  part / flag / sync buffers: LOCAL ones (world 1).
// maps_ready != 0: maps_dev already holds the descriptors of exactly these shard addresses and sizes (a caller
// that reuses its buffers can skip the host-to-device copy of the descriptors on every call after the first).
HMF_API int hmf_allgather_gemm(const unsigned long long* x_ptrs, void* maps_dev, const unsigned int* x_flags,
                               unsigned int x_epoch, int ag_world, const void* w, void* y, int M, int N, int Ks,
                               long long ldx, long long ldw, const unsigned long long* part_ptrs,
                               const unsigned long long* flag_ptrs, unsigned int* sync, long long part_stride,
                               int max_tiles, int splits, int maps_ready, cudaStream_t st) {
  HMF_REQUIRE(x_ptrs != nullptr, "allgather_gemm: null shard table");
  return launch_tp(nullptr, w, y, M, N, Ks, ldx, ldw, part_ptrs, flag_ptrs, sync, part_stride, max_tiles, 0, 1, splits,
                   0, x_ptrs, maps_dev, x_flags, x_epoch, ag_world, nullptr, st, maps_ready ? 1 : 0);
}
