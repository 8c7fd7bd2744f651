// All-gather fused into a tensor-parallel GEMM for sm_100a:
//
//   C[M, N_loc] = A_full[M, K] * B_loc[N_loc, K]^T,   A_full = the row shards of all ranks
//
// Every rank owns M / W consecutive rows of A (its tokens under sequence parallelism) inside a
// buffer of the full [M, K] shape that the peers have mapped.  ONE kernel does both jobs:
//   * four gather warps per CTA pull the peers' shards over NVLink (16-byte peer loads, ring order
//     starting at the next rank) into this rank's copy of the buffer, 16 rows at a time, taking
//     work items from an atomic counter, and publish a per-m-tile ready count;
//   * the usual TMA -> tcgen05.mma -> TMEM pipeline multiplies the rank's own rows first and the
//     remote m-tiles in the order they arrive, its producer waiting (bounded) on the ready count.
// A remote row crosses NVLink once, however many output tiles reuse it, and the transfer overlaps
// the multiplication of the tiles that are already here.  The arithmetic per output element is
// det_gemm's (one fp32 accumulator, ascending k), so the result is bitwise the GEMM of the
// gathered matrix.  The reference gathers with NCCL and then calls its GEMM
// (rl_engine/backends/cuda/ffn/ffn.py:601-603).
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

constexpr int ABM = 128, ABN = 256, ABK = 64;
constexpr int kAgThreads = 320;  // warp0 TMA, warp1 MMA, warps2-5 epilogue, warps6-9 gather
constexpr int kAgStageA = ABM * ABK * 2, kAgStageB = ABN * ABK * 2, kAgStage = kAgStageA + kAgStageB;
constexpr int kAgStages = 4;
constexpr int kAgSmem = kAgStages * kAgStage + 1024 + 256;
constexpr int kSubRows = 16;                 // rows per gather work item
constexpr int kSubPerTile = ABM / kSubRows;  // 8 items make one m-tile ready

struct AgGemmParams {
  int M, N, K;
  int m_tiles, n_tiles;
  int world, rank;
  int rows_per_rank;            // M / world (multiple of 128)
  const unsigned char* a_peer[8];  // every rank's [M, K] buffer as mapped here (own buffer at `rank`)
  unsigned char* a_local;       // = a_peer[rank]
  __nv_bfloat16* C;
  long long ldc;
  int* ready;                   // [m_tiles] items landed per m-tile (zeroed before the launch)
  int* work;                    // next gather work item (zeroed before the launch)
  int* status;
};

// m-tiles in processing order: own shard first, then the peers' shards in ring order.
__device__ __forceinline__ int ag_mtile(const AgGemmParams& p, int ord) {
  const int per = p.rows_per_rank / ABM;
  const int shard = (p.rank + ord / per) % p.world;
  return shard * per + ord % per;
}

// Tile t -> (position of its m-tile in processing order, n-tile).  Groups of kAgGroupM m-tiles
// sweep all n-tiles with the m-tile varying fastest, so the CTAs that run at the same time share a
// few B tiles and the group's A rows stay in L2 while B streams through once per group.
constexpr int kAgGroupM = 8;
__device__ __forceinline__ void ag_tile_coords(const AgGemmParams& p, int t, int& ord, int& nt) {
  const int per_group = kAgGroupM * p.n_tiles;
  const int g = t / per_group;
  const int first = g * kAgGroupM;
  const int gsize = min(p.m_tiles - first, kAgGroupM);
  const int r = t - g * per_group;
  ord = first + r % gsize;
  nt = r / gsize;
}

__global__ void __launch_bounds__(kAgThreads, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const AgGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kAgStages * kAgStage);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kAgStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* item_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kAgStages);
  const uint32_t accf0 = smem_u32(bars + 2 * kAgStages), acce0 = smem_u32(bars + 2 * kAgStages + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kAgStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(accf0 + 8 * a, 1);
      mbar_init(acce0 + 8 * a, 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total = p.m_tiles * p.n_tiles;
  const uint32_t smem_base = smem_u32(smem);
  const int kbs = p.K / ABK;
  const int own_tiles = p.rows_per_rank / ABM;

  // Producer and MMA warps: all 32 lanes walk the loops (warp-uniform state), one elected lane
  // issues, waits are warp votes.
  if (warp == 0) {
    {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total; t += gridDim.x) {
        int ord, nt;
        ag_tile_coords(p, t, ord, nt);
        const int mt = ag_mtile(p, ord);
        if (ord >= own_tiles) {
          // remote rows: wait until all of the m-tile's gather items have landed
          const uint64_t t0 = globaltimer_ns();
          uint32_t spins = 0;
          int v;
          while (true) {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.ready + mt) : "memory");
            if (v >= kSubPerTile) break;
            if ((++spins & 63) == 0 && (*abort_flag || globaltimer_ns() - t0 > RLK_WAIT_LIMIT_NS)) {
              *abort_flag = 1;
              if (p.status) atomicCAS(p.status, 0, 501);
              break;
            }
          }
          if (__any_sync(0xffffffffu, *abort_flag != 0)) break;
          asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy stores -> TMA reads
        }
        for (int kb = 0; kb < kbs; ++kb, ++it) {
          const uint32_t s = it % kAgStages, ph = (it / kAgStages) & 1;
          if (!mbar_wait_warp(empty0 + 8 * s, ph ^ 1, abort_flag, p.status, 502)) break;
          const uint32_t fb = full0 + 8 * s;
          const uint32_t sa = smem_base + s * kAgStage;
          if (!elect_one()) continue;
          mbar_expect_tx(fb, kAgStage);
          tma_load_2d(sa, &tmA, kb * ABK, mt * ABM, fb);
          tma_load_2d(sa + kAgStageA, &tmB, kb * ABK, nt * ABN, fb);
        }
        if (__any_sync(0xffffffffu, *abort_flag != 0)) break;
      }
    }
  } else if (warp == 1) {
    {
      constexpr uint32_t idesc = umma_idesc_bf16(ABM, ABN, 0, 0);
      uint32_t it = 0, u = 0;
      for (int t = blockIdx.x; t < total && !__any_sync(0xffffffffu, *abort_flag != 0); t += gridDim.x, ++u) {
        const uint32_t a = u & 1;
        if (!mbar_wait_warp(acce0 + 8 * a, ((u >> 1) & 1) ^ 1, abort_flag, p.status, 503)) break;
        tc_fence_after();
        for (int kb = 0; kb < kbs; ++kb, ++it) {
          const uint32_t s = it % kAgStages, ph = (it / kAgStages) & 1;
          if (!mbar_wait_warp(full0 + 8 * s, ph, abort_flag, p.status, 504)) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * kAgStage, sb = sa + kAgStageA;
          if (!elect_one()) continue;
#pragma unroll
          for (int k = 0; k < ABK / 16; ++k)
            umma_bf16_ss(tmem_base + a * ABN, umma_desc_sw128(sa + k * 32, 16, 1024),
                         umma_desc_sw128(sb + k * 32, 16, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(empty0 + 8 * s);
        }
        if (elect_one()) umma_commit(accf0 + 8 * a);
      }
    }
  } else if (warp < 6) {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t u = 0;
    for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x, ++u) {
      int ord, nt;
      ag_tile_coords(p, t, ord, nt);
      const int row = ag_mtile(p, ord) * ABM + r;
      const uint32_t a = u & 1;
      if (!mbar_wait(accf0 + 8 * a, (u >> 1) & 1, abort_flag, p.status, 505)) break;
      tc_fence_after();
      __nv_bfloat16* dst = p.C + static_cast<long long>(row) * p.ldc + nt * ABN;
#pragma unroll 1
      for (int col0 = 0; col0 < ABN; col0 += 32) {
        uint32_t x[32];
        tmem_ld32(tmem_base + lane_off + a * ABN + col0, x);
        tmem_ld_wait();
        if (row < p.M) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (nt * ABN + col0 + j < p.N) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(x[j]), __uint_as_float(x[j + 1]));
              o.y = pack_bf16x2(__uint_as_float(x[j + 2]), __uint_as_float(x[j + 3]));
              o.z = pack_bf16x2(__uint_as_float(x[j + 4]), __uint_as_float(x[j + 5]));
              o.w = pack_bf16x2(__uint_as_float(x[j + 6]), __uint_as_float(x[j + 7]));
              *reinterpret_cast<uint4*>(dst + col0 + j) = o;
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(acce0 + 8 * a);
    }
  } else {
    // ------------------------------------------------------------------ gather warps (128 threads)
    const int gt = threadIdx.x - 192;
    const int remote_tiles = p.m_tiles - own_tiles;
    const int n_items = remote_tiles * kSubPerTile;
    const long long row_bytes = static_cast<long long>(p.K) * 2;
    const long long item_vecs = kSubRows * row_bytes / 16;   // 16-byte pieces per item (rows are contiguous)
    while (true) {
      if (gt == 0) *item_slot = atomicAdd(p.work, 1);
      asm volatile("bar.sync 2, 128;" ::: "memory");
      const int item = *item_slot;
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (item >= n_items) break;
      const int ord = own_tiles + item / kSubPerTile;
      const int mt = ag_mtile(p, ord);
      const int shard = mt / own_tiles;
      const long long off = (static_cast<long long>(mt) * ABM + (item % kSubPerTile) * kSubRows) * row_bytes;
      const uint4* src = reinterpret_cast<const uint4*>(p.a_peer[shard] + off);
      uint4* dst = reinterpret_cast<uint4*>(p.a_local + off);
      for (long long v0 = gt; v0 < item_vecs; v0 += 128 * 8) {
        uint4 q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const long long v = v0 + 128 * j;
          if (v < item_vecs)
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(q[j].x), "=r"(q[j].y), "=r"(q[j].z), "=r"(q[j].w) : "l"(src + v) : "memory");
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const long long v = v0 + 128 * j;
          if (v < item_vecs) dst[v] = q[j];
        }
      }
      __threadfence();
      asm volatile("fence.proxy.async;" ::: "memory");
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (gt == 0) atomicAdd(p.ready + mt, 1);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace rlk
using namespace rlk;

// Number of ints of zero-initialisable scratch rlk_ag_gemm needs for an M-row problem.
RLK_API long long rlk_ag_gemm_scratch_ints(int M) { return (M + ABM - 1) / ABM + 1; }

// a_ptrs[r]: rank r's [M, K] bf16 buffer (contiguous rows) as mapped in this process; rank r's own
// rows [r * M / world, (r + 1) * M / world) of its buffer are valid on entry, and on exit this
// rank's buffer holds all of A.  B: [N, K] with pitch ldb; C: [M, N] with pitch ldc.  `scratch`:
// rlk_ag_gemm_scratch_ints(M) ints, cleared here.  The caller brackets the call with barriers of
// the group: one before (every shard is written), one after (nobody overwrites a shard that a
// peer may still be reading).
RLK_API int rlk_ag_gemm(void* const* a_ptrs, int world, int rank, int M, int N, int K, const void* B,
                        long long ldb, void* C, long long ldc, int* scratch, void* stream) {
  RLK_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world, "ag_gemm: bad rank geometry");
  RLK_REQUIRE(M > 0 && M % (world * ABM) == 0, "ag_gemm: M must be a multiple of world * 128");
  RLK_REQUIRE(K % ABK == 0 && N % 8 == 0, "ag_gemm: K %% 64 and N %% 8 must be 0");
  AgGemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.m_tiles = M / ABM;
  p.n_tiles = (N + ABN - 1) / ABN;
  p.world = world; p.rank = rank;
  p.rows_per_rank = M / world;
  for (int i = 0; i < 8; ++i) p.a_peer[i] = static_cast<const unsigned char*>(a_ptrs[i < world ? i : 0]);
  p.a_local = static_cast<unsigned char*>(a_ptrs[rank]);
  p.C = static_cast<__nv_bfloat16*>(C);
  p.ldc = ldc;
  p.ready = scratch;
  p.work = scratch + p.m_tiles;
  p.status = device_status_word();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RLK_CHECK_CUDA(cudaMemsetAsync(scratch, 0, sizeof(int) * (p.m_tiles + 1), s));
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = make_tmap_2d_sw128(&tmA, p.a_local, M, K, K, ABM, 64, 2))) return rc;
  if ((rc = make_tmap_2d_sw128(&tmB, B, N, K, ldb, ABN, 64, 2))) return rc;
  static bool attr_set[64] = {false};
  int dev = 0;
  RLK_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    RLK_CHECK_CUDA(cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAgSmem));
    attr_set[dev & 63] = true;
  }
  const int tiles = p.m_tiles * p.n_tiles;
  // every CTA gathers, so all of them must be resident at once: at most one per SM
  const int grid = tiles < sm_count() ? tiles : sm_count();
  ag_gemm_kernel<<<grid, kAgThreads, kAgSmem, s>>>(tmA, tmB, p);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
