// Batch-invariant bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM.
//
//   C[M,N] = A[M,K] * B[N,K]^T        (A and B may each be K-major or MN-major in memory)
//
// Numerical contract (what makes it deterministic, batch-invariant and TP-invariant):
//   * every output element is one fp32 TMEM accumulator fed by UMMA K=16 steps in ascending k;
//     no split-K, no atomics, one CTA owns a whole output tile;
//   * the arithmetic of a row never depends on the other rows of its tile, so padding M to the
//     128-row tile (TMA zero fill) makes every batch size run the same per-row program;
//   * optional canonical K chunks (`nchunks` = 1,2,4,8, equal sizes): each chunk is accumulated
//     in its own fp32 accumulator, rounded to bf16 once, and the chunks are combined by a
//     balanced binary tree with a bf16 rounding at every node.  A rank that owns 8/TP canonical
//     chunks therefore produces exactly the sub-tree that the fixed-order collective continues,
//     and TP=1 reproduces the bits of TP=2/4/8.
// The same tree is restated for the CPU in rl_kernel_b200/reference/gemm/det_gemm.py.
//
// Covers the reference's det_gemm_fwd / fwd_rhs_transposed / da / db entry points
// (csrc/cuda/gemm/det_gemm_kernel.cu:527-602) with one kernel template.
#include "rlk/host.h"
#include "rlk/logp_contract.cuh"
#include "rlk/no_alloc.h"
#include "rlk/ptx.cuh"
#include "rlk/symm.h"

#include <mutex>

namespace rlk {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;  // warp0 TMA, warp1 MMA, warps2-5 epilogue
// Tiles of 128 columns and more get a second set of epilogue warps (warps 6-9): two warps share a
// TMEM lane quadrant and each drains half of the tile's columns, which keeps the epilogue of the
// chunk-tree variants (one accumulator drain per canonical K chunk) off the critical path.
constexpr int kGemmThreadsWide = 320;
template <int BN> constexpr int gemm_threads() { return BN >= 128 ? kGemmThreadsWide : kGemmThreads; }

struct GemmParams {
  int M, N, K;
  int nchunks;          // canonical K chunks (power of two)
  int kb_per_chunk;     // 64-wide k blocks per chunk
  int m_tiles, n_tiles;
  void* C;              // bf16 or fp32, row-major
  long long ldc;
  int out_fp32;         // 1: C is fp32
  int accumulate;       // 1: C += result (read-modify-write in fp32, rounded to C's dtype)
  int* status;
  uint4* tree_scratch;      // tile_n 256 with chunks: per-CTA tree stack [grid][3][128][32] uint4 (L2 resident)
  int a_box_rows;           // rows of A that TMA brings per tile (128, or fewer when M < 128)
  int stage_a_bytes;        // shared-memory bytes reserved for the A tile of one stage
  int stages;               // depth of the shared-memory ring
  int tma_store;            // 1: plain bf16 tiles of 128+ columns leave through shared memory and TMA stores
                            //    (two 128 x 64 staging slabs behind the barriers, one per set of epilogue warps)
  int kslabs;               // 64-wide k blocks per ring stage (1, 2 or 4).  More than one: both operands are
                            //   K-major and a stage is brought by ONE 3-D TMA box per operand ([slab][row][64]),
                            //   so the two single-lane roles pay their per-stage waits once per 128 or 256 k
  // Fused gate/up + SwiGLU (192-wide tiles only, act_blk > 0): B holds gate and up rows interleaved
  // in blocks of act_blk rows ([g_0 | u_0 | g_1 | u_1 ...]); a tile multiplies by 96 gate rows and
  // the 96 matching up rows, and the epilogue writes silu(bf16(gate)) * bf16(up) -- the bits of
  // the separate SwiGLU kernel on the bf16 gate/up tensor -- to C [M, act_I].
  int act_blk, act_I;
  int tree_l0_smem;         // tile_n 256 with chunks: level 0 of the tree stack lives in shared memory
                            //   behind the barriers (kTreeL0Pitch bytes per tile row)
  int b_static;             // 1: B was complete before the previous kernel of the stream started (a
                            //    weight): its first tiles are fetched before the dependency wait
  int split_chunks;         // > 1: every canonical chunk is its own tile and writes its bf16 leaf
  long long split_stride;   //      to C + chunk * split_stride (elements); nchunks is 1 then
  // fused LM-head epilogue (tile_n == 128, nchunks == 1): per-(row, tile) softmax statistics
  float2* stats;            // null = plain GEMM
  long long stats_stride;   // float2 elements per row of `stats`
  int stats_tile0;          // global tile index of this shard's first tile
  const long long* targets; // [M] global target ids, may be null
  long long vocab_start;    // global id of column 0
  float* tgt_logit;         // [M]
  float inv_temp;
  const float* min_keep;    // [M] or null: a scaled logit below its row's value is outside the support (-inf)
  // vocab-parallel exchange fused into the same epilogue (stats_world > 1): every statistic and
  // the owner's target logit are also stored into the other tensor-parallel ranks' buffers
  // (peer stores over NVLink), so after one barrier every rank holds all tiles of every row.
  int stats_world, stats_rank;
  float2* stats_peer[8];
  float* tgt_peer[8];
  // fused all-reduce epilogue (ar_world > 1): C points into this rank's symmetric frame; after a
  // tile's partial is stored there the epilogue warps shake hands with the same tile on every
  // peer, pull the peers' partials over NVLink, finish the balanced tree and write ar_out.
  int ar_world, ar_rank;
  unsigned char* ar_frame[8];
  unsigned long long* ar_flags[8];
  unsigned long long ar_seq;
  const unsigned long long* ar_epoch;
  int ar_use_epoch;
  __nv_bfloat16* ar_out;
  long long ar_ld_out;
  // reduce-scatter form of the fused epilogue (rs_row1 > rs_row0): this rank finishes only the tiles of rows
  // [rs_row0, rs_row1) -- a whole number of 128-row tiles -- and ar_out is biased so that row rs_row0 lands on the
  // caller's row 0.  Every rank still publishes all its partial tiles; the peers pull the ones they own.
  int rs_row0, rs_row1;
#ifdef RLK_GEMM_TRACE
  // profiling build only: clock64 stamps of CTA 0's two single-thread roles, [5][kTraceLen]
  // (producer: after the empty wait, after the TMA issue; MMA thread: after the full wait, after
  // the MMA issue, after the commit)
  long long* trace;
#endif
};
#ifdef RLK_GEMM_TRACE
constexpr int kTraceLen = 512;
#define RLK_TRACE_T(row, idx) do { if (p.trace && blockIdx.x == 0 && threadIdx.x == 64 && (idx) < kTraceLen) p.trace[(row) * kTraceLen + (idx)] = clock64(); } while (0)
#define RLK_TRACE(row, idx) do { if (p.trace && blockIdx.x == 0 && (idx) < kTraceLen) p.trace[(row) * kTraceLen + (idx)] = clock64(); } while (0)
#else
#define RLK_TRACE(row, idx) do { } while (0)
#define RLK_TRACE_T(row, idx) do { } while (0)
#endif

__device__ __forceinline__ uint4 ar_ld_peer_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Weak 16-byte load that bypasses L1 (the peers' partial tiles: their visibility is established by
// the acquire on the tile's flag plus the CTA barrier; strong .sys loads would complete one after
// the other within a thread -- measured 2.7 us each over NVLink -- instead of overlapping).
__device__ __forceinline__ uint4 ar_ld_peer_weak_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ar_tree_node(const uint4 a, const uint4 b) {
  uint4 o;
  o.x = pack_bf16x2(__fadd_rn(bf16_lo(a.x), bf16_lo(b.x)), __fadd_rn(bf16_hi(a.x), bf16_hi(b.x)));
  o.y = pack_bf16x2(__fadd_rn(bf16_lo(a.y), bf16_lo(b.y)), __fadd_rn(bf16_hi(a.y), bf16_hi(b.y)));
  o.z = pack_bf16x2(__fadd_rn(bf16_lo(a.z), bf16_lo(b.z)), __fadd_rn(bf16_hi(a.z), bf16_hi(b.z)));
  o.w = pack_bf16x2(__fadd_rn(bf16_lo(a.w), bf16_lo(b.w)), __fadd_rn(bf16_hi(a.w), bf16_hi(b.w)));
  return o;
}

// Pulls one 128 x BN tile's partials from the W ranks' frames (this rank's own from local memory,
// the others over NVLink with 16-byte loads, NB pieces per thread in flight so that a tile costs
// one or two round trips), combines them with the balanced tree and writes the result.
template <int BN, int W, int NB>
__device__ __forceinline__ void ar_pull_tile(const GemmParams& p, int m0, int n0, int et) {
  constexpr int kPerRow = BN / 8;                         // 16-byte pieces per tile row
  const unsigned char* frames[W];
#pragma unroll
  for (int r = 0; r < W; ++r) frames[r] = p.ar_frame[r];
  const int M = p.M, N = p.N;
  const long long ldc = p.ldc;
  unsigned char* out = reinterpret_cast<unsigned char*>(p.ar_out);
  for (int base = et; base < BM * kPerRow; base += 256 * NB) {
    // every piece of every rank is requested before the first one is used: a thread pays one
    // NVLink round trip and one local one per batch, not one per piece
    uint4 v[NB][W];
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      const int idx = base + u * 256;
      const int rr = idx / kPerRow, cc = (idx % kPerRow) * 8;
      if (idx < BM * kPerRow && m0 + rr < M && n0 + cc < N) {
        const long long off = (static_cast<long long>(m0 + rr) * ldc + n0 + cc) * 2;
#pragma unroll
        for (int r = 0; r < W; ++r) v[u][r] = ar_ld_peer_weak_v4(frames[r] + off);
      }
    }
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      const int idx = base + u * 256;
      const int rr = idx / kPerRow, cc = (idx % kPerRow) * 8;
      if (!(idx < BM * kPerRow && m0 + rr < M && n0 + cc < N)) continue;
      const long long off = (static_cast<long long>(m0 + rr) * ldc + n0 + cc) * 2;
#pragma unroll
      for (int n = W; n > 1; n >>= 1)
#pragma unroll
        for (int j = 0; j < n / 2; ++j) v[u][j] = ar_tree_node(v[u][2 * j], v[u][2 * j + 1]);
      // (the frame is laid out with the caller's output pitch: the byte offsets coincide)
      *reinterpret_cast<uint4*>(out + off) = v[u][0];
    }
  }
}

// Waits (bounded) until every peer has published its partial of tile t, then reduces the tile.
// Called by all 256 epilogue threads; returns false when a wait gave up.
template <int BN>
__device__ __noinline__ bool ar_finish_tile(const GemmParams& p, int t, int m0, int n0, int et,
                                               unsigned long long seq, volatile int* abort_flag) {
  // reduce-scatter: a tile outside this rank's rows is somebody else's to finish (same answer in all 256 threads,
  // so the barrier below is skipped by all of them or by none)
  if (p.rs_row1 > p.rs_row0 && (m0 >= p.rs_row1 || m0 + BM <= p.rs_row0)) return true;
  if (et < p.ar_world && et != p.ar_rank) {
    const unsigned long long* f = p.ar_flags[p.ar_rank] + et * kMaxSlices + t;
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    unsigned long long v;
    while (true) {
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(f) : "memory");
      if (v >= seq) break;
      if ((++it & 63) == 0 && (*abort_flag || globaltimer_ns() - t0 > RLK_WAIT_LIMIT_NS)) {
        *abort_flag = 1;
        if (p.status) atomicCAS(p.status, 0, 105);
        break;
      }
    }
  }
  asm volatile("bar.sync 2, 256;" ::: "memory");
  RLK_TRACE_T(3, (t - blockIdx.x) / gridDim.x);            // peers' flags seen
  if (*abort_flag) return false;
  if (p.ar_world == 2) ar_pull_tile<BN, 2, 8>(p, m0, n0, et);
  else if (p.ar_world == 4) ar_pull_tile<BN, 4, 4>(p, m0, n0, et);
  else ar_pull_tile<BN, 8, 2>(p, m0, n0, et);
  return true;
}

constexpr int kMaxStages = 16;
constexpr int kTreeL0Pitch = 528;   // 512 bytes of packed bf16 per row + 16: 16-byte accesses of a warp spread over all banks

template <int BN>
struct GemmSmem {
  static constexpr int kStageA = BM * BK * 2;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (BN >= 192) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int kBarBytes = 512;           // room for the barriers of kMaxStages stages
  static constexpr int kBytes = 227 * 1024;       // the launch may use up to all of an SM's shared memory
};

__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int& mt, int& nt) {
  constexpr int GROUP_M = 16;
  const int per_group = GROUP_M * n_tiles;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gsize = min(m_tiles - first_m, GROUP_M);
  const int r = t - g * per_group;
  mt = first_m + (r % gsize);
  nt = r / gsize;
}

// Fused gate/up + SwiGLU tiles: first gate row of tile nt (its up rows start act_blk rows later).
__device__ __forceinline__ int act_gate_row(int nt, int act_blk) {
  const int c0 = nt * 96;
  return (c0 / act_blk) * 2 * act_blk + c0 % act_blk;
}

// AR: the instantiation with the fused all-reduce / reduce-scatter epilogue.  It is a template parameter rather than
// a run-time branch because the tile reduction is a real function call whose registers (batched peer loads) would
// otherwise count against every instantiation and cost the small-M kernels their second resident CTA.
template <int BN, bool A_MN, bool B_MN, bool AR = false>
__global__ void __launch_bounds__(gemm_threads<BN>(), 1)
det_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const __grid_constant__ GemmParams p) {
  using S = GemmSmem<BN>;
  const uint32_t kStages = static_cast<uint32_t>(p.stages);   // ring depth chosen by the host (<= kMaxStages)
  // TMEM columns: two accumulators (+ three packed-bf16 tree levels when chunked, BN==128 only)
  constexpr uint32_t kAcc = (BN == 192) ? 256 : BN;   // column stride between the two accumulators
  constexpr uint32_t kTmemCols = (BN == 128 || BN == 192) ? 512 : (2 * BN < 32 ? 32 : 2 * BN);
  constexpr uint32_t kStackCol = 2 * BN;  // first column of the tree stack (BN == 128)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t kslabs = static_cast<uint32_t>(p.kslabs);
  const uint32_t a_region = kslabs * static_cast<uint32_t>(p.stage_a_bytes);           // A slabs of a stage, then its B slabs
  const uint32_t stage_bytes = a_region + kslabs * S::kStageB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * stage_bytes);
  // bars: full[kStages], empty[kStages], acc_full[2], acc_empty[2], then tmem ptr + abort flag
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kStages);
  const uint32_t accf0 = smem_u32(bars + 2 * kStages);
  const uint32_t acce0 = smem_u32(bars + 2 * kStages + 2);

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(accf0 + 8 * a, 1);
      mbar_init(acce0 + 8 * a, gemm_threads<BN>() - 64);   // every epilogue thread arrives
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.m_tiles * p.n_tiles * p.split_chunks;
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the loop (its state is warp-uniform, so it can live in uniform
    // registers, which is where the TMA and barrier instructions take their operands from); one
    // elected lane issues.
    {
      uint32_t it = 0, pre = 0;
      uint32_t ps = 0, pph = 0, psa = smem_base;   // ring slot, its phase, its shared-memory address
      const uint32_t stage_tx = kslabs * ((A_MN ? S::kStageA : static_cast<uint32_t>(p.a_box_rows) * BK * 2) + S::kStageB);
      if (p.b_static && static_cast<int>(blockIdx.x) < total_tiles) {
        // weights do not depend on the previous kernel: start streaming the first tile's B blocks
        // while that kernel is still running
        int mt, nt;
        tile_coords(blockIdx.x / p.split_chunks, p.m_tiles, p.n_tiles, mt, nt);
        const uint32_t kbs = static_cast<uint32_t>(p.nchunks * p.kb_per_chunk) / kslabs;   // ring stages of a tile
        const int kb0 = (blockIdx.x % p.split_chunks) * p.kb_per_chunk;
        pre = kbs < kStages ? kbs : kStages;
        for (uint32_t kb = 0; kb < pre; ++kb) {
          const uint32_t fb = full0 + 8 * kb;
          const uint32_t sb = smem_base + kb * stage_bytes + a_region;
          const int k0 = (kb0 + static_cast<int>(kb * kslabs)) * BK;
          if (!elect_one()) continue;
          mbar_expect_tx(fb, stage_tx);
          if (BN == 192 && p.act_blk > 0) {
            const int gr = act_gate_row(nt, p.act_blk);
            for (uint32_t sl = 0; sl < kslabs; ++sl) {
              tma_load_2d(sb + sl * S::kStageB, &tmB, k0 + sl * BK, gr, fb);
              tma_load_2d(sb + sl * S::kStageB + 96 * 128, &tmB, k0 + sl * BK, gr + p.act_blk, fb);
            }
          } else if (!B_MN) {
            if (kslabs > 1) tma_load_3d(sb, &tmB, 0, nt * BN, k0 / BK, fb);
            else tma_load_2d(sb, &tmB, k0, nt * BN, fb);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * 8192, &tmB, nt * BN + 64 * i, k0, fb);
          }
        }
      }
      griddep_sync();
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        int mt, nt;
        const int chunk = t % p.split_chunks;
        tile_coords(t / p.split_chunks, p.m_tiles, p.n_tiles, mt, nt);
        const int m0 = mt * BM, n0 = nt * BN;
        const int kbs = p.nchunks * p.kb_per_chunk / static_cast<int>(kslabs);   // ring stages of this tile
        const int kb0 = chunk * p.kb_per_chunk;
        const int k_step = BK * static_cast<int>(kslabs);
        int k0 = kb0 * BK;
        for (int kb = 0; kb < kbs; ++kb, ++it, k0 += k_step) {
          const uint32_t fb = full0 + 8 * ps;
          const bool fresh = it >= pre;   // else: armed, and B requested, before the dependency wait
          if (fresh && !mbar_wait_warp(empty0 + 8 * ps, pph ^ 1, abort_flag, p.status, 101)) break;
          RLK_TRACE(0, it);
          const uint32_t sa = psa;
          const uint32_t sb = sa + a_region;
          // ring position of the next stage (no divisions in this loop)
          if (++ps == kStages) { ps = 0; pph ^= 1; psa = smem_base; } else { psa += stage_bytes; }
          if (!elect_one()) continue;
          if (fresh) mbar_expect_tx(fb, stage_tx);
          if (!A_MN) {
            if (kslabs > 1) tma_load_3d(sa, &tmA, 0, m0, k0 / BK, fb);
            else tma_load_2d(sa, &tmA, k0, m0, fb);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * 8192, &tmA, m0 + 64 * i, k0, fb);
          }
          if (!fresh) continue;
          if (BN == 192 && p.act_blk > 0) {
            const int gr = act_gate_row(nt, p.act_blk);
            for (uint32_t sl = 0; sl < kslabs; ++sl) {
              tma_load_2d(sb + sl * S::kStageB, &tmB, k0 + sl * BK, gr, fb);
              tma_load_2d(sb + sl * S::kStageB + 96 * 128, &tmB, k0 + sl * BK, gr + p.act_blk, fb);
            }
          } else if (!B_MN) {
            if (kslabs > 1) tma_load_3d(sb, &tmB, 0, n0, k0 / BK, fb);
            else tma_load_2d(sb, &tmB, k0, n0, fb);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * 8192, &tmB, n0 + 64 * i, k0, fb);
          }
          RLK_TRACE(1, it);
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // (whole warp in the loop, one elected lane issues: see the producer)
    {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      // One thread issues every MMA, so each instruction of this loop is on the critical path of a
      // small tile.  The shared-memory descriptors differ only in their 14-bit start-address field
      // (address / 16, bits 0-13; shared memory ends below 2^18, so adding never carries out of
      // it): build them once and step the low word per k step and per ring slot.
      const uint64_t da_base = A_MN ? umma_desc_sw128(smem_base, 8192, 1024) : umma_desc_sw128(smem_base, 16, 1024);
      const uint64_t db_base = B_MN ? umma_desc_sw128(smem_base + a_region, 8192, 1024)
                                    : umma_desc_sw128(smem_base + a_region, 16, 1024);
      const uint32_t da_hi = static_cast<uint32_t>(da_base >> 32), db_hi = static_cast<uint32_t>(db_base >> 32);
      const uint32_t da_lo0 = static_cast<uint32_t>(da_base), db_lo0 = static_cast<uint32_t>(db_base);
      constexpr uint32_t ka_step = (A_MN ? 2048u : 32u) >> 4, kb_step = (B_MN ? 2048u : 32u) >> 4;
      const uint32_t slot_step = stage_bytes >> 4;
      const uint32_t a_slab_step = static_cast<uint32_t>(p.stage_a_bytes) >> 4, b_slab_step = S::kStageB >> 4;
      const int stages_per_chunk = p.kb_per_chunk / static_cast<int>(kslabs);
      uint32_t s = 0, ph = 0, da_lo = da_lo0, db_lo = db_lo0, u = 0;
#ifdef RLK_GEMM_TRACE
      int tr = 0;
#endif
      auto desc64 = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        for (int c = 0; c < p.nchunks; ++c, ++u) {
          const uint32_t a = u & 1;
          if (!mbar_wait_warp(acce0 + 8 * a, ((u >> 1) & 1) ^ 1, abort_flag, p.status, 102)) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + a * kAcc;
          for (int kb = 0; kb < stages_per_chunk; ++kb) {
            // (no tcgen05 fence here: the operands come from TMA, whose completion the barrier
            // itself orders; the fence after the accumulator wait above covers the epilogue's loads)
            if (!mbar_wait_warp(full0 + 8 * s, ph, abort_flag, p.status, 103)) break;
            RLK_TRACE(2, tr);
            if (elect_one()) {
              umma_bf16_ss(d_tmem, desc64(da_lo, da_hi), desc64(db_lo, db_hi), idesc, kb != 0 ? 1u : 0u);
#pragma unroll
              for (uint32_t k = 1; k < BK / UMMA_K; ++k)
                umma_bf16_ss(d_tmem, desc64(da_lo + k * ka_step, da_hi), desc64(db_lo + k * kb_step, db_hi), idesc, 1u);
              for (uint32_t sl = 1; sl < kslabs; ++sl) {      // further k slabs of this stage (K-major operands only)
                const uint32_t al = da_lo + sl * a_slab_step, bl = db_lo + sl * b_slab_step;
#pragma unroll
                for (uint32_t k = 0; k < BK / UMMA_K; ++k)
                  umma_bf16_ss(d_tmem, desc64(al + k * ka_step, da_hi), desc64(bl + k * kb_step, db_hi), idesc, 1u);
              }
              RLK_TRACE(3, tr);
              umma_commit(empty0 + 8 * s);  // frees the smem stage when these MMAs retire
              RLK_TRACE(4, tr);
            }
#ifdef RLK_GEMM_TRACE
            ++tr;
#endif
            if (++s == kStages) { s = 0; ph ^= 1; da_lo = da_lo0; db_lo = db_lo0; }
            else { da_lo += slot_step; db_lo += slot_step; }
          }
          if (elect_one()) umma_commit(accf0 + 8 * a);  // accumulator of this chunk complete
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 or 8 warps)
    const int quad = warp & 3;                  // TMEM lane quadrant this warp may access
    const int half = (warp - 2) >> 2;           // 0: warps 2-5; 1: warps 6-9 (tiles of >= 128 columns only)
    constexpr int kColsPerWarp = BN >= 128 ? BN / 2 : BN;
    const int row_in_tile = quad * 32 + lane;   // one thread owns one output row
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t u = 0;
    int ar_prev_t = -1, ar_prev_m0 = 0, ar_prev_n0 = 0;     // fused all-reduce: the tile whose reduction is still due
    griddep_sync();            // C, the statistics and the tree scratch may still be in use by the previous kernel
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      int mt, nt;
      tile_coords(t / p.split_chunks, p.m_tiles, p.n_tiles, mt, nt);
      const int row = mt * BM + row_in_tile;
      const int n0 = nt * BN;
      const long long c_off = static_cast<long long>(t % p.split_chunks) * p.split_stride;
      for (int c = 0; c < p.nchunks; ++c, ++u) {
        const uint32_t a = u & 1;
        if (!mbar_wait(accf0 + 8 * a, (u >> 1) & 1, abort_flag, p.status, 104)) break;
        tc_fence_after();
        if (c == 0) RLK_TRACE_T(4, (t - blockIdx.x) / gridDim.x);   // first accumulator of the tile ready
        const bool last = (c == p.nchunks - 1);
        if ((BN == 128 || BN == 256) && p.stats != nullptr) {
          // 128-wide tiles: the first set of epilogue warps walks the tile's one vocabulary tile;
          // 256-wide tiles: each set walks its own 128 columns = its own vocabulary tile
          constexpr int kVT = BN / 128;                       // vocabulary tiles per GEMM tile
          const int cbase = (BN == 256) ? half * 128 : 0;     // first column of this thread's vocabulary tile
          if ((BN == 256 || half == 0) && n0 + cbase < p.N) {
          // fused selected-logp statistics: logit = bf16(acc); z = logit * inv_temp
          // (one thread walks all 128 columns of its row: the statistics have a fixed order)
          const long long tgt_col = (p.targets && row < p.M) ? p.targets[row] - p.vocab_start - n0 - cbase : -1;
          const float keep_from = (p.min_keep && row < p.M) ? p.min_keep[row] : -INFINITY;   // restricted sampling support
          float m = -INFINITY;
#pragma unroll 1
          for (int col0 = 0; col0 < 128; col0 += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_base + lane_off + a * kAcc + cbase + col0, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + cbase + col0 + j < p.N) {
                const float zj = logp_scale(round_bf16(__uint_as_float(r[j])), p.inv_temp);
                if (zj >= keep_from) m = fmaxf(m, zj);
              }
          }
          TileSum ts;
#pragma unroll 1
          for (int col0 = 0; col0 < 128; col0 += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_base + lane_off + a * kAcc + cbase + col0, r);
            tmem_ld_wait();
            float z[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float zj = logp_scale(round_bf16(__uint_as_float(r[j])), p.inv_temp);
              z[j] = (n0 + cbase + col0 + j < p.N && zj >= keep_from) ? zj : -INFINITY;
            }
            if (m > -INFINITY) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) ts.add4(z[j], z[j + 1], z[j + 2], z[j + 3], m);
            }
            if (tgt_col >= col0 && tgt_col < col0 + 32) {
              float zt = 0.f;
#pragma unroll
              for (int j = 0; j < 32; ++j) if (tgt_col - col0 == j) zt = z[j];
              if (n0 + cbase + tgt_col < p.N) {
                p.tgt_logit[row] = zt;
                for (int pr = 0; pr < p.stats_world; ++pr)
                  if (pr != p.stats_rank) p.tgt_peer[pr][row] = zt;
              }
            }
            if (p.C != nullptr && row < p.M) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + n0 + cbase + col0;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (n0 + cbase + col0 + j < p.N) {
                  uint4 v;
                  v.x = pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                  v.y = pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                  v.z = pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                  v.w = pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                  *reinterpret_cast<uint4*>(dst + j) = v;
                }
              }
            }
          }
          if (row < p.M) {
            const float2 st2 = make_float2(m, ts.total());
            const long long si = row * p.stats_stride + p.stats_tile0 + nt * kVT + (BN == 256 ? half : 0);
            p.stats[si] = st2;
            for (int pr = 0; pr < p.stats_world; ++pr)
              if (pr != p.stats_rank) p.stats_peer[pr][si] = st2;
          }
          }
        } else if (BN == 192 && p.act_blk > 0) {
          // fused SwiGLU: accumulator columns [0, 96) are gate, [96, 192) the matching up columns;
          // each set of epilogue warps takes 48 of the 96 output columns
          // (the tensor-memory loads are warp-wide instructions: every lane runs them, rows past M
          // only skip the stores)
          const int c0 = nt * 96 + half * 48;                     // first activation column of this thread
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + c0;
#pragma unroll 1
          for (int pc = 0; pc < 3; ++pc) {
            uint32_t g[16], u2[16];
            tmem_ld16(tmem_base + lane_off + a * kAcc + half * 48 + pc * 16, g);
            tmem_ld16(tmem_base + lane_off + a * kAcc + 96 + half * 48 + pc * 16, u2);
            tmem_ld_wait();
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float g0 = round_bf16(__uint_as_float(g[2 * j])), g1 = round_bf16(__uint_as_float(g[2 * j + 1]));
              const float u0 = round_bf16(__uint_as_float(u2[2 * j])), u1 = round_bf16(__uint_as_float(u2[2 * j + 1]));
              o[j] = pack_bf16x2((g0 / (1.f + __expf(-g0))) * u0, (g1 / (1.f + __expf(-g1))) * u1);
            }
            if (row < p.M) {
              *reinterpret_cast<uint4*>(dst + pc * 16) = make_uint4(o[0], o[1], o[2], o[3]);
              *reinterpret_cast<uint4*>(dst + pc * 16 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
            }
          }
        } else if (BN == 256 && p.nchunks > 1) {
          // chunk tree with 128x256 tiles: both accumulators fill TMEM, so the tree stack cannot live
          // there.  Level 0 (four of the seven pushes and pops of a tile) sits in shared memory, in
          // the space a fourth pipeline stage would take; levels 1 and 2 in a per-CTA global buffer
          // (L2 resident).  A row's entries of a slice are only ever touched by the one thread that
          // owns that row and slice.  (Level 0 in registers was tried: 64 more live registers spill
          // under the 168-register cap.)
          int nmerge = 0;
          while ((c >> nmerge) & 1) ++nmerge;                       // levels to fold into this chunk
          uint4* sbase = p.tree_scratch + (static_cast<size_t>(blockIdx.x) * 3 * BM + row_in_tile) * 32;
          constexpr size_t kLevel = static_cast<size_t>(BM) * 32;   // uint4 per level
          const int sl0 = half * 4;   // this warp's four 32-column slices
          uint4* l0row = reinterpret_cast<uint4*>(smem + kStages * stage_bytes + S::kBarBytes +
                                                  row_in_tile * kTreeL0Pitch);
#pragma unroll
          for (int si = 0; si < 4; ++si) {
            const int sl = sl0 + si;
            // stack entries of this slice: issued before the TMEM load so that both are in flight
            uint4 cur[3][4];
#pragma unroll
            for (int lv = 0; lv < 3; ++lv)
              if (lv < nmerge)
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  cur[lv][q] = (lv == 0 && p.tree_l0_smem) ? l0row[sl * 4 + q] : sbase[lv * kLevel + sl * 4 + q];
            uint32_t r[32];
            tmem_ld32(tmem_base + lane_off + a * kAcc + sl * 32, r);
            tmem_ld_wait();
            uint32_t v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
              v[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
#pragma unroll
            for (int lv = 0; lv < 3; ++lv) {
              if (lv < nmerge) {
                const uint32_t sv[16] = {cur[lv][0].x, cur[lv][0].y, cur[lv][0].z, cur[lv][0].w,
                                         cur[lv][1].x, cur[lv][1].y, cur[lv][1].z, cur[lv][1].w,
                                         cur[lv][2].x, cur[lv][2].y, cur[lv][2].z, cur[lv][2].w,
                                         cur[lv][3].x, cur[lv][3].y, cur[lv][3].z, cur[lv][3].w};
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  v[j] = pack_bf16x2(__fadd_rn(bf16_lo(sv[j]), bf16_lo(v[j])), __fadd_rn(bf16_hi(sv[j]), bf16_hi(v[j])));
              }
            }
            const int col0 = sl * 32;
            if (!last) {
              uint4* dst4 = (nmerge == 0 && p.tree_l0_smem) ? l0row + sl * 4 : sbase + nmerge * kLevel + sl * 4;
#pragma unroll
              for (int q = 0; q < 4; ++q)
                dst4[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else if (row < p.M) {
              if (p.out_fp32) {
                float* dst = reinterpret_cast<float*>(p.C) + c_off + static_cast<long long>(row) * p.ldc + n0 + col0;
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                  if (n0 + col0 + 2 * j < p.N) {
                    float4 o = make_float4(bf16_lo(v[j]), bf16_hi(v[j]), bf16_lo(v[j + 1]), bf16_hi(v[j + 1]));
                    if (p.accumulate) {
                      const float4 q4 = *reinterpret_cast<const float4*>(dst + 2 * j);
                      o.x += q4.x; o.y += q4.y; o.z += q4.z; o.w += q4.w;
                    }
                    *reinterpret_cast<float4*>(dst + 2 * j) = o;
                  }
                }
              } else {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + static_cast<long long>(row) * p.ldc + n0 + col0;
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                  if (n0 + col0 + 2 * j < p.N) {
                    uint4 o = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    if (p.accumulate) {
                      const uint4 q4 = *reinterpret_cast<const uint4*>(dst + 2 * j);
                      o.x = pack_bf16x2(bf16_lo(o.x) + bf16_lo(q4.x), bf16_hi(o.x) + bf16_hi(q4.x));
                      o.y = pack_bf16x2(bf16_lo(o.y) + bf16_lo(q4.y), bf16_hi(o.y) + bf16_hi(q4.y));
                      o.z = pack_bf16x2(bf16_lo(o.z) + bf16_lo(q4.z), bf16_hi(o.z) + bf16_hi(q4.z));
                      o.w = pack_bf16x2(bf16_lo(o.w) + bf16_lo(q4.w), bf16_hi(o.w) + bf16_hi(q4.w));
                    }
                    *reinterpret_cast<uint4*>(dst + 2 * j) = o;
                  }
                }
              }
            }
          }
        } else if ((BN == 128 || BN == 256) && p.tma_store) {
          // Plain bf16 tile: accumulator -> registers -> swizzled staging slab -> one TMA store per
          // 128 x 64 block.  (Row-per-thread global stores, 16 bytes each to 32 different rows per
          // instruction, fill the SM's memory-instruction queue and hold up the MMA warp's issue for
          // the length of the epilogue: measured 596 against 519 cycles per k block at 128 x 256.)
          // Each set of four epilogue warps owns one slab and a named barrier of its 128 threads.
          uint8_t* slab = smem + kStages * stage_bytes + 1024 + half * (BM * 128);
          const uint32_t slab_u32 = smem_u32(slab);
          const bool store_leader = (warp == 2 + 4 * half) && lane == 0;
          const int bar_id = 3 + half;
#pragma unroll 1
          for (int g0 = 0; g0 < kColsPerWarp; g0 += 64) {
            const int col0 = half * kColsPerWarp + g0;
            uint32_t r0[32], r1[32];
            tmem_ld32(tmem_base + lane_off + a * kAcc + col0, r0);
            tmem_ld32(tmem_base + lane_off + a * kAcc + col0 + 32, r1);
            if (store_leader) tma_store_wait_read();          // the slab's previous store has been read out
            tmem_ld_wait();
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r0[8 * q]), __uint_as_float(r0[8 * q + 1]));
              v.y = pack_bf16x2(__uint_as_float(r0[8 * q + 2]), __uint_as_float(r0[8 * q + 3]));
              v.z = pack_bf16x2(__uint_as_float(r0[8 * q + 4]), __uint_as_float(r0[8 * q + 5]));
              v.w = pack_bf16x2(__uint_as_float(r0[8 * q + 6]), __uint_as_float(r0[8 * q + 7]));
              *reinterpret_cast<uint4*>(slab + sw128_offset(row_in_tile, q)) = v;
              v.x = pack_bf16x2(__uint_as_float(r1[8 * q]), __uint_as_float(r1[8 * q + 1]));
              v.y = pack_bf16x2(__uint_as_float(r1[8 * q + 2]), __uint_as_float(r1[8 * q + 3]));
              v.z = pack_bf16x2(__uint_as_float(r1[8 * q + 4]), __uint_as_float(r1[8 * q + 5]));
              v.w = pack_bf16x2(__uint_as_float(r1[8 * q + 6]), __uint_as_float(r1[8 * q + 7]));
              *reinterpret_cast<uint4*>(slab + sw128_offset(row_in_tile, 4 + q)) = v;
            }
            fence_proxy_async_smem();                          // generic-proxy writes -> the TMA store's reads
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
            if (store_leader && n0 + col0 < p.N) {
              tma_store_2d(&tmC, slab_u32, n0 + col0, mt * BM);
              tma_store_commit();
            }
          }
        } else
#pragma unroll 1
        for (int col0 = half * kColsPerWarp; col0 < (half + 1) * kColsPerWarp; col0 += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_off + a * kAcc + col0, r);
          tmem_ld_wait();
          if (p.nchunks == 1) {
            if (row < p.M) {
              if (p.out_fp32) {
                float* dst = reinterpret_cast<float*>(p.C) + c_off + static_cast<long long>(row) * p.ldc + n0 + col0;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  if (n0 + col0 + j < p.N) {
                    float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                           __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                    if (p.accumulate) {
                      const float4 o = *reinterpret_cast<const float4*>(dst + j);
                      v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                    }
                    *reinterpret_cast<float4*>(dst + j) = v;
                  }
                }
              } else {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off +
                                     static_cast<long long>(row) * p.ldc + n0 + col0;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  if (n0 + col0 + j < p.N) {
                    uint4 v;
                    if (p.accumulate) {
                      const uint4 o = *reinterpret_cast<const uint4*>(dst + j);
                      v.x = pack_bf16x2(__uint_as_float(r[j]) + bf16_lo(o.x), __uint_as_float(r[j + 1]) + bf16_hi(o.x));
                      v.y = pack_bf16x2(__uint_as_float(r[j + 2]) + bf16_lo(o.y), __uint_as_float(r[j + 3]) + bf16_hi(o.y));
                      v.z = pack_bf16x2(__uint_as_float(r[j + 4]) + bf16_lo(o.z), __uint_as_float(r[j + 5]) + bf16_hi(o.z));
                      v.w = pack_bf16x2(__uint_as_float(r[j + 6]) + bf16_lo(o.w), __uint_as_float(r[j + 7]) + bf16_hi(o.w));
                    } else {
                      v.x = pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                      v.y = pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                      v.z = pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                      v.w = pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                    }
                    *reinterpret_cast<uint4*>(dst + j) = v;
                  }
                }
              }
            }
          } else if (BN == 128) {
            // canonical chunk tree: leaf = bf16(fp32 accumulator); node = bf16(fp32(a)+fp32(b)).
            uint32_t v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
              v[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            int cc = c, level = 0;
            while (cc & 1) {
              uint32_t sv[16];
              if (BN == 128) {
                tmem_ld16(tmem_base + lane_off + kStackCol + level * 64 + (col0 >> 1), sv);
                tmem_ld_wait();
              } else {
                // tile_n 256: both accumulators fill TMEM, the stack lives in a per-CTA global buffer
                // that only this thread ever touches for its row (and that stays in L2)
                const uint4* sp = p.tree_scratch + ((static_cast<size_t>(blockIdx.x) * 3 + level) * BM + row_in_tile) * (BN / 8) + (col0 >> 3);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 t4 = sp[q];
                  sv[4 * q] = t4.x; sv[4 * q + 1] = t4.y; sv[4 * q + 2] = t4.z; sv[4 * q + 3] = t4.w;
                }
              }
#pragma unroll
              for (int j = 0; j < 16; ++j)
                v[j] = pack_bf16x2(__fadd_rn(bf16_lo(sv[j]), bf16_lo(v[j])),
                                   __fadd_rn(bf16_hi(sv[j]), bf16_hi(v[j])));
              cc >>= 1;
              ++level;
            }
            if (!last) {
              if (BN == 128) {
                tmem_st16(tmem_base + lane_off + kStackCol + level * 64 + (col0 >> 1), v);
              } else {
                uint4* sp = p.tree_scratch + ((static_cast<size_t>(blockIdx.x) * 3 + level) * BM + row_in_tile) * (BN / 8) + (col0 >> 3);
#pragma unroll
                for (int q = 0; q < 4; ++q) sp[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
              }
            } else if (row < p.M) {
              if (p.out_fp32) {
                float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + n0 + col0;
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                  if (n0 + col0 + 2 * j < p.N) {
                    float4 o = make_float4(bf16_lo(v[j]), bf16_hi(v[j]), bf16_lo(v[j + 1]), bf16_hi(v[j + 1]));
                    if (p.accumulate) {
                      const float4 q = *reinterpret_cast<const float4*>(dst + 2 * j);
                      o.x += q.x; o.y += q.y; o.z += q.z; o.w += q.w;
                    }
                    *reinterpret_cast<float4*>(dst + 2 * j) = o;
                  }
                }
              } else {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) +
                                     static_cast<long long>(row) * p.ldc + n0 + col0;
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                  if (n0 + col0 + 2 * j < p.N) {
                    uint4 o = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    if (p.accumulate) {
                      const uint4 q = *reinterpret_cast<const uint4*>(dst + 2 * j);
                      o.x = pack_bf16x2(bf16_lo(o.x) + bf16_lo(q.x), bf16_hi(o.x) + bf16_hi(q.x));
                      o.y = pack_bf16x2(bf16_lo(o.y) + bf16_lo(q.y), bf16_hi(o.y) + bf16_hi(q.y));
                      o.z = pack_bf16x2(bf16_lo(o.z) + bf16_lo(q.z), bf16_hi(o.z) + bf16_hi(q.z));
                      o.w = pack_bf16x2(bf16_lo(o.w) + bf16_lo(q.w), bf16_hi(o.w) + bf16_hi(q.w));
                    }
                    *reinterpret_cast<uint4*>(dst + 2 * j) = o;
                  }
                }
              }
            }
          }
        }
        if (p.nchunks > 1 && BN == 128) tmem_st_wait();
        tc_fence_before();
        mbar_arrive(acce0 + 8 * a);
      }
      if constexpr (AR) {
        // ---- fused all-reduce, one tile behind the accumulator drain.  This tile's partial is in the
        // frame: make it visible and tell the peers; then finish the PREVIOUS tile, whose peers have
        // had a whole tile's time to answer, so the flag round trip is off the critical path.
        const int et = threadIdx.x - 64;  // 0..255 among the epilogue threads (tiles of 128 columns)
        const unsigned long long seq = p.ar_use_epoch ? p.ar_seq + p.ar_epoch[0] * p.ar_epoch[1] : p.ar_seq;
        RLK_TRACE_T(0, (t - blockIdx.x) / gridDim.x);      // drained
        // (no fence per thread: the barrier orders the 256 threads' stores before the flag threads'
        // st.release.sys, and a release is cumulative over what its thread has observed)
        asm volatile("bar.sync 2, 256;" ::: "memory");
        RLK_TRACE_T(1, (t - blockIdx.x) / gridDim.x);      // fenced
        if (et < p.ar_world && et != p.ar_rank)
          asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.ar_flags[et] + p.ar_rank * kMaxSlices + t), "l"(seq) : "memory");
        if (ar_prev_t >= 0 && !ar_finish_tile<BN>(p, ar_prev_t, ar_prev_m0, ar_prev_n0, et, seq, abort_flag)) break;
        RLK_TRACE_T(2, (t - blockIdx.x) / gridDim.x);      // previous tile reduced
        ar_prev_t = t; ar_prev_m0 = mt * BM; ar_prev_n0 = n0;
      }
    }
    if constexpr (AR) if (ar_prev_t >= 0 && !*abort_flag) {
      const unsigned long long seq = p.ar_use_epoch ? p.ar_seq + p.ar_epoch[0] * p.ar_epoch[1] : p.ar_seq;
      ar_finish_tile<BN>(p, ar_prev_t, ar_prev_m0, ar_prev_n0, static_cast<int>(threadIdx.x) - 64, seq, abort_flag);
    }
    if ((BN == 128 || BN == 256) && p.tma_store && lane == 0 && (warp == 2 || warp == 6)) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Ring depth / CTAs per SM of the small-M (decode) launches; 0 = the built-in choice.
static int g_small_m_stages = 0, g_small_m_ctas = 0, g_small_m_kslabs = 0;
static int g_tma_store = 1;
#ifdef RLK_GEMM_TRACE
static long long* g_trace_ptr = nullptr;
#endif

template <int BN, bool A_MN, bool B_MN, bool AR = false>
static int launch_gemm(const void* A, const void* B, const GemmParams& p0, long long lda,
                       long long ldb, cudaStream_t stream) {
  GemmParams p = p0;
  CUtensorMap tmA, tmB;
  int rc;
  if (p.split_chunks < 1) p.split_chunks = 1;
  p.b_static = static_b_operand();
  p.a_box_rows = BM;
  if (!A_MN && p.M < BM) p.a_box_rows = (p.M + 7) / 8 * 8;  // rows beyond are never stored: skip loading them
  // The UMMA still addresses 128 A rows; with a short A box the rows past it alias the B tile /
  // next stage (finite garbage feeding accumulator rows nobody stores), and the stage shrinks so
  // two CTAs fit on an SM -- more loads in flight for the bandwidth-bound small-M case.
  p.stage_a_bytes = A_MN ? GemmSmem<BN>::kStageA : (p.a_box_rows * BK * 2 + 1023) / 1024 * 1024;   // per k slab
  // k slabs per ring stage.  Few rows (decode): the tile is paced by the per-stage waits and issues
  // of its producer and MMA warps, so a stage carries 128 k; full tiles are bound by the tensor
  // pipe and keep one slab per stage.
  p.kslabs = 1;
  if (!A_MN && !B_MN && p.M < BM && p.K % BK == 0) {
    int want = g_small_m_kslabs > 0 ? g_small_m_kslabs : 2;
    while (want > 1 && (p.kb_per_chunk % want != 0 || p.kb_per_chunk / want < 2)) want >>= 1;
    p.kslabs = want;
  }
  const int stage_bytes = p.kslabs * (p.stage_a_bytes + GemmSmem<BN>::kStageB);
  const int slack = GemmSmem<BN>::kStageA - p.stage_a_bytes;   // reads past the last stage stay in bounds
  // Ring depth.  Full tiles: the per-width default.  Few rows (measured at 64 rows, K = 4096 and
  // 12288, L2 flushed): when one wave of CTAs covers all tiles (QKV, gate/up) one CTA per SM with a
  // deep ring is fastest (N = 6144: 21.5 us with 6 stages of 128 k against 29.7 us with 4 stages of
  // 64 k); with several short tiles per SM (the chunked row-parallel projections) two CTAs per SM
  // with 3 stages each, so that one CTA issues while the other is between tiles.
  p.stages = GemmSmem<BN>::kStages;
  if (!A_MN && p.M < BM) {
    const long long n_tiles_all = static_cast<long long>((p.N + BN - 1) / BN) * (p.split_chunks < 1 ? 1 : p.split_chunks);
    const bool one_wave = n_tiles_all <= sm_count();
    p.stages = g_small_m_stages > 0 ? g_small_m_stages : (p.kslabs > 1 ? (one_wave ? 6 : 3) : 4);
    const int fit = (GemmSmem<BN>::kBytes - 1024 - GemmSmem<BN>::kBarBytes - slack) / stage_bytes;
    if (p.stages > fit) p.stages = fit;
  }
  int smem_bytes = p.stages * stage_bytes + 1024 + GemmSmem<BN>::kBarBytes + slack;
  // plain bf16 tiles of full-size launches leave through staging slabs and TMA stores
  p.tma_store = ((BN == 128 || BN == 256) && p.M >= BM && p.nchunks == 1 && p.split_chunks == 1 && !p.out_fp32 && !p.accumulate &&
                 p.stats == nullptr && p.act_blk == 0 && p.ar_world <= 1 && p.C != nullptr && g_tma_store) ? 1 : 0;
  if (p.tma_store) {
    smem_bytes = p.stages * stage_bytes + 1024 + 1024 + 2 * BM * 128;      // ring, alignment, barriers, two slabs
    if (smem_bytes > GemmSmem<BN>::kBytes) p.tma_store = 0, smem_bytes = p.stages * stage_bytes + 1024 + GemmSmem<BN>::kBarBytes + slack;
  }
  p.tree_l0_smem = 0;
  if (BN == 256 && p.nchunks > 1 && p.tree_scratch != nullptr) {
    // three stages instead of four; the freed space holds level 0 of the tree stack
    p.stages = 3;
    p.tree_l0_smem = 1;
    smem_bytes = p.stages * stage_bytes + 1024 + GemmSmem<BN>::kBarBytes + slack + BM * kTreeL0Pitch;
  }
  // (with several slabs per stage a K-major operand [rows, K] is addressed as [K / 64][rows][64])
  if (!A_MN && p.kslabs > 1) rc = make_tmap_3d_sw128_box(&tmA, A, p.K / BK, p.M, 64, lda, 64, p.kslabs, p.a_box_rows, 64, 2);
  else if (!A_MN) rc = make_tmap_2d_sw128(&tmA, A, p.M, p.K, lda, p.a_box_rows, 64, 2);
  else rc = make_tmap_2d_sw128(&tmA, A, p.K, p.M, lda, BK, 64, 2);
  if (rc) return rc;
  if (BN == 192 && p.act_blk > 0) rc = make_tmap_2d_sw128(&tmB, B, p.N, p.K, ldb, 96, 64, 2);
  else if (!B_MN && p.kslabs > 1) rc = make_tmap_3d_sw128_box(&tmB, B, p.K / BK, p.N, 64, ldb, 64, p.kslabs, BN, 64, 2);
  else if (!B_MN) rc = make_tmap_2d_sw128(&tmB, B, p.N, p.K, ldb, BN, 64, 2);
  else rc = make_tmap_2d_sw128(&tmB, B, p.K, p.N, ldb, BK, 64, 2);
  if (rc) return rc;
  CUtensorMap tmC = tmA;                                  // placeholder when the tile is stored directly
  if (p.tma_store) {
    rc = make_tmap_2d_sw128(&tmC, p.C, p.M, p.N, p.ldc, BM, 64, 2);
    if (rc) return rc;
  }
  p.m_tiles = (p.M + BM - 1) / BM;
  p.n_tiles = (p.N + BN - 1) / BN;
  if (BN == 192 && p.act_blk > 0) p.n_tiles = p.act_I / 96;
  const int tiles = p.m_tiles * p.n_tiles * p.split_chunks;
  int ctas_per_sm = (GemmSmem<BN>::kBytes + 1024) / (smem_bytes + 1024);   // shared memory
  const int tmem_fit = 512 / ((BN == 128 || BN == 192) ? 512 : (2 * BN < 32 ? 32 : 2 * BN));   // tensor memory columns
  if (ctas_per_sm > tmem_fit) ctas_per_sm = tmem_fit;
  if (ctas_per_sm > 2) ctas_per_sm = 2;
  if (!A_MN && p.M < BM && g_small_m_ctas > 0 && ctas_per_sm > g_small_m_ctas) ctas_per_sm = g_small_m_ctas;
  if (ctas_per_sm < 1) ctas_per_sm = 1;
#ifdef RLK_GEMM_TRACE
  p.trace = g_trace_ptr;
#endif
  const int grid = tiles < sm_count() * ctas_per_sm ? tiles : sm_count() * ctas_per_sm;
  auto kfn = det_gemm_kernel<BN, A_MN, B_MN, AR>;
  RLK_REQUIRE((p.ar_world > 1) == AR, "det_gemm: all-reduce parameters and the kernel's epilogue do not match");
  static bool attr_set[64] = {false};
  static std::mutex attr_mu;
  int dev = 0;
  RLK_CHECK_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(attr_mu);
    if (!attr_set[dev & 63]) {
      RLK_CHECK_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          GemmSmem<BN>::kBytes));
      attr_set[dev & 63] = true;
    }
  }
  RLK_CHECK_CUDA(launch_pdl(kfn, dim3(grid), dim3(gemm_threads<BN>()), smem_bytes, stream, tmA, tmB, tmC, p));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// out[i] = balanced tree over the nchunks bf16 leaves leaf[c][i], node = bf16(fp32(a) + fp32(b)).
__global__ void __launch_bounds__(256)
chunk_tree_kernel(const __nv_bfloat16* __restrict__ leaves, long long chunk_stride,
                  __nv_bfloat16* __restrict__ out, int M, int N, long long ld, int nchunks) {
  griddep_sync();
  const int per_row = N / 8;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(M) * per_row) return;
  const long long off = (idx / per_row) * ld + (idx % per_row) * 8;
  uint4 v[8];
  for (int c = 0; c < nchunks; ++c) v[c] = *reinterpret_cast<const uint4*>(leaves + c * chunk_stride + off);
  for (int n = nchunks; n > 1; n >>= 1) {
    for (int i = 0; i < n / 2; ++i) {
      const uint4 a = v[2 * i], b = v[2 * i + 1];
      v[i].x = pack_bf16x2(__fadd_rn(bf16_lo(a.x), bf16_lo(b.x)), __fadd_rn(bf16_hi(a.x), bf16_hi(b.x)));
      v[i].y = pack_bf16x2(__fadd_rn(bf16_lo(a.y), bf16_lo(b.y)), __fadd_rn(bf16_hi(a.y), bf16_hi(b.y)));
      v[i].z = pack_bf16x2(__fadd_rn(bf16_lo(a.z), bf16_lo(b.z)), __fadd_rn(bf16_hi(a.z), bf16_hi(b.z)));
      v[i].w = pack_bf16x2(__fadd_rn(bf16_lo(a.w), bf16_lo(b.w)), __fadd_rn(bf16_hi(a.w), bf16_hi(b.w)));
    }
  }
  *reinterpret_cast<uint4*>(out + off) = v[0];
}

}  // namespace rlk

// Benchmark knob: ring depth and CTAs per SM of the launches with fewer than 128 rows (0 = built-in).
RLK_API int rlk_gemm_small_m_tuning(int stages, int ctas_per_sm) {
  RLK_REQUIRE(stages >= 0 && stages <= rlk::kMaxStages && ctas_per_sm >= 0 && ctas_per_sm <= 2, "gemm tuning out of range");
  rlk::g_small_m_stages = stages;
  rlk::g_small_m_ctas = ctas_per_sm;
  return RLK_OK;
}
// Benchmark knob: 1 = full-size plain bf16 tiles leave through TMA stores (default), 0 = direct stores.
RLK_API int rlk_gemm_tma_store(int on) {
  const int old = rlk::g_tma_store;
  rlk::g_tma_store = on ? 1 : 0;
  return old;
}
// Benchmark knob: 64-wide k blocks per ring stage of those launches (1, 2 or 4; 0 = built-in).
RLK_API int rlk_gemm_small_m_kslabs(int kslabs) {
  RLK_REQUIRE(kslabs == 0 || kslabs == 1 || kslabs == 2 || kslabs == 4, "kslabs must be 0, 1, 2 or 4");
  rlk::g_small_m_kslabs = kslabs;
  return RLK_OK;
}
#ifdef RLK_GEMM_TRACE
RLK_API int rlk_gemm_set_trace(void* ptr) { rlk::g_trace_ptr = static_cast<long long*>(ptr); return RLK_OK; }
#endif

// Per-device scratch of the tile_n 256 chunk tree: one stack of 3 levels per CTA of a full grid.
static uint4* tree_scratch_for_device() {
  static uint4* ptr[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!ptr[dev]) {
    void* p = nullptr;
    const size_t bytes = static_cast<size_t>(2 * rlk::sm_count()) * 3 * 128 * 32 * sizeof(uint4);
    if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
    ptr[dev] = static_cast<uint4*>(p);
  }
  return ptr[dev];
}

// act[M, I] = silu(bf16(X Wg^T)) * bf16(X Wu^T) for a packed gate/up weight Wgu [2 I, K] whose rows
// come in blocks of `blk`: [g_0 | u_0 | g_1 | u_1 | ...] (blk = I: plain [gate | up]).  One kernel:
// 192-wide tiles of 96 gate + 96 up columns, SwiGLU in the epilogue; the gate/up tensor is never
// written.  Bits equal rlk_det_gemm followed by rlk_swiglu_fwd.  I and blk must be multiples of 96.
RLK_API int rlk_det_gemm_swiglu(const void* X, const void* Wgu, void* act, int M, int I, int K,
                                long long ldx, long long ldw, long long ld_act, int blk, void* stream) {
  using namespace rlk;
  RLK_REQUIRE(M > 0 && I > 0 && K > 0 && K % 8 == 0, "det_gemm_swiglu: bad shape");
  RLK_REQUIRE(blk > 0 && I % blk == 0 && blk % 96 == 0, "det_gemm_swiglu: the gate/up block must be a multiple of 96 columns");
  RLK_REQUIRE((reinterpret_cast<uintptr_t>(act) & 15) == 0 && (ld_act * 2) % 16 == 0, "det_gemm_swiglu: act must be 16-byte aligned");
  GemmParams p{};
  p.M = M; p.N = 2 * I; p.K = K;
  p.nchunks = 1;
  p.kb_per_chunk = (K + 63) / 64;
  p.C = act; p.ldc = ld_act;
  p.status = device_status_word();
  p.act_blk = blk;
  p.act_I = I;
  return launch_gemm<192, false, false>(X, Wgu, p, ldx, ldw, static_cast<cudaStream_t>(stream));
}

// C[M,N] = A * B^T.
//  a_mn = 0: A is [M,K] row-major (lda >= K);  a_mn = 1: A is stored [K,M] row-major (lda >= M).
//  b_mn = 0: B is [N,K] row-major (ldb >= K);  b_mn = 1: B is stored [K,N] row-major (ldb >= N).
//  nchunks: canonical K chunks (1,2,4,8); K/nchunks must be a multiple of 64 when nchunks > 1.
//  tile_n: 0 = pick from the shape; else one of 32, 64, 128, 256 (chunked GEMMs: 128 or 256).
//  out_fp32 / accumulate: C dtype and C += result.
RLK_API int rlk_det_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                         long long ldb, long long ldc, int a_mn, int b_mn, int nchunks,
                         int tile_n, int out_fp32, int accumulate, void* stream) {
  using namespace rlk;
  RLK_REQUIRE(M > 0 && N > 0 && K > 0, "det_gemm: empty shape");
  RLK_REQUIRE(N % 8 == 0, "det_gemm: N must be a multiple of 8 (got %d)", N);
  RLK_REQUIRE(K % 8 == 0, "det_gemm: K must be a multiple of 8 (got %d)", K);
  RLK_REQUIRE(nchunks == 1 || nchunks == 2 || nchunks == 4 || nchunks == 8,
              "det_gemm: nchunks must be 1, 2, 4 or 8");
  RLK_REQUIRE(nchunks == 1 || (K % (nchunks * 64) == 0),
              "det_gemm: K/nchunks must be a multiple of 64 (K=%d, nchunks=%d)", K, nchunks);
  RLK_REQUIRE((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * (out_fp32 ? 4 : 2)) % 16 == 0,
              "det_gemm: C must be 16-byte aligned with a 16-byte multiple pitch");
  if (a_mn) RLK_REQUIRE(M % 8 == 0, "det_gemm: MN-major A needs M %% 8 == 0");
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.nchunks = nchunks;
  p.kb_per_chunk = nchunks == 1 ? (K + 63) / 64 : K / nchunks / 64;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.status = device_status_word();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int bn = tile_n;
  if (nchunks > 1) {
    // many tiles: 128x256 tiles (full tensor-core rate) with the tree stack in an L2-resident
    // scratch; few tiles: 128x128 tiles with the stack in TMEM
    const long long tiles256 = static_cast<long long>((M + 127) / 128) * ((N + 255) / 256);
    // (measured, 12288 x 4096 outputs, 8 chunks: chunks of 512 k run at 891 TFLOP/s on 128-wide
    // tiles against 868 on 256-wide ones; chunks of 768 k at 867 against 997)
    bn = (tile_n == 256 || (tile_n == 0 && tiles256 >= sm_count() && K / nchunks >= 768)) ? 256 : 128;
    if (a_mn) bn = 128;
    if (bn == 256) {
      p.tree_scratch = tree_scratch_for_device();
      if (!p.tree_scratch) return set_error(RLK_ERR_CUDA, "det_gemm: cannot allocate the tree scratch");
    }
  }
  if (bn == 0) {
    const int m_tiles = (M + 127) / 128;
    const int sms = sm_count();
    bn = 256;
    // widest tile that still gives about two thirds of the SMs a tile: at decode sizes a wider
    // tile re-reads the activation rows fewer times, which matters more than idle SMs
    // (measured, M = 64, K = 4096: N = 24576 57 us at 256 vs 62 us at 128; N = 6144 equal at 32 / 64)
    while (bn > 32 && (long long)m_tiles * ((N + bn - 1) / bn) < sms * 5 / 8) bn >>= 1;
    if (b_mn || a_mn) bn = bn < 128 ? 128 : bn;
    // one row of tiles (decode): a 256-wide tile takes in its k blocks at the SM's ingest rate, so
    // 192-wide tiles on more SMs finish sooner when they still fit in one wave
    // (N = 24576: 128 tiles instead of 96)
    if (bn == 256 && m_tiles == 1 && !a_mn && !b_mn && N % 192 == 0 && N / 192 <= sms && N / 192 > (N + 255) / 256)
      bn = 192;
  }
#define RLK_GEMM_CASE(BN_, AM_, BM_)                                       \
  if (bn == BN_ && a_mn == AM_ && b_mn == BM_)                             \
    return launch_gemm<BN_, (AM_ != 0), (BM_ != 0)>(A, B, p, lda, ldb, s);
  RLK_GEMM_CASE(256, 0, 0)
  RLK_GEMM_CASE(192, 0, 0)
  RLK_GEMM_CASE(128, 0, 0)
  RLK_GEMM_CASE(64, 0, 0)
  RLK_GEMM_CASE(32, 0, 0)
  RLK_GEMM_CASE(256, 0, 1)
  RLK_GEMM_CASE(128, 0, 1)
  RLK_GEMM_CASE(256, 1, 1)
  RLK_GEMM_CASE(128, 1, 1)
  RLK_GEMM_CASE(256, 1, 0)
  RLK_GEMM_CASE(128, 1, 0)
#undef RLK_GEMM_CASE
  return set_error(RLK_ERR_UNSUPPORTED, "det_gemm: no kernel for tile_n=%d a_mn=%d b_mn=%d", bn,
                   a_mn, b_mn);
}

// Small-M form of the chunked GEMM (decode): every canonical K chunk becomes its own set of CTAs
// (nchunks times more parallelism), each writes its rounded bf16 leaf into `scratch`
// ([nchunks][M][ldc] bf16), and a second kernel combines the leaves with the same balanced tree
// the single-kernel form applies in its epilogue: identical bits, far better occupancy when
// M <= a few hundred rows.  A and B are K-major.
RLK_API long long rlk_det_gemm_split_scratch_elems(int M, long long ldc, int nchunks) {
  return static_cast<long long>(nchunks) * M * ldc;
}

// C == nullptr: only the leaves are produced (scratch [nchunks][M][ldc]); the caller folds the tree
// into its next kernel (rlk_rmsnorm_fwd_leaves).
RLK_API int rlk_det_gemm_split(const void* A, const void* B, void* C, void* scratch, int M, int N,
                               int K, long long lda, long long ldb, long long ldc, int nchunks,
                               int tile_n, void* stream) {
  using namespace rlk;
  RLK_REQUIRE(M > 0 && N > 0 && K > 0 && N % 8 == 0 && K % 8 == 0, "det_gemm_split: bad shape");
  RLK_REQUIRE(nchunks == 2 || nchunks == 4 || nchunks == 8, "det_gemm_split: nchunks must be 2, 4 or 8");
  RLK_REQUIRE(K % (nchunks * 64) == 0, "det_gemm_split: K/nchunks must be a multiple of 64");
  RLK_REQUIRE(A != nullptr && B != nullptr, "det_gemm_split: A and B must not be null");
  RLK_REQUIRE(ldc >= N, "det_gemm_split: ldc (%lld) must be at least N (%d)", ldc, N);
  RLK_REQUIRE((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0 &&
                  scratch != nullptr && (ldc * 2) % 16 == 0, "det_gemm_split: C and scratch must be 16-byte aligned");
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.nchunks = 1;
  p.kb_per_chunk = K / nchunks / 64;
  p.C = scratch; p.ldc = ldc;
  p.status = device_status_word();
  p.split_chunks = nchunks;
  p.split_stride = static_cast<long long>(M) * ldc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc;
  if (tile_n == 32) rc = launch_gemm<32, false, false>(A, B, p, lda, ldb, s);
  else if (tile_n == 128) rc = launch_gemm<128, false, false>(A, B, p, lda, ldb, s);
  else rc = launch_gemm<64, false, false>(A, B, p, lda, ldb, s);
  if (rc) return rc;
  if (C == nullptr) return RLK_OK;
  const long long n = static_cast<long long>(M) * (N / 8);
  RLK_CHECK_CUDA(launch_pdl(chunk_tree_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s,
                            static_cast<const __nv_bfloat16*>(scratch), p.split_stride, static_cast<__nv_bfloat16*>(C), M, N, ldc, nchunks));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// 1: the fused all-reduce / reduce-scatter entries may use 128 x 256 tiles (0 keeps them on 128 x 128).  Every rank
// of a group must use the same value (the tile numbering is part of the flag protocol).
static int g_ar_wide_tiles = 1;
RLK_API int rlk_det_gemm_ar_set_wide_tiles(int on) { g_ar_wide_tiles = on ? 1 : 0; return RLK_OK; }

// GEMM + fixed-order all-reduce in ONE kernel (row-parallel projections: o_proj, FFN down):
// out = all_reduce_tree_over_ranks( A_local @ B_local^T with nchunks canonical K chunks ).
// `state` is the rlk_symm_create handle of the tensor-parallel group; every rank calls this with
// the same shapes on its own stream.  The partial result lives only in the symmetric frame; the
// transfer of a tile overlaps the MMA of the following tiles.  M * ld_out * 2 bytes must fit the
// frame and the number of 128 x tile_n tiles must not exceed the flag slots.
RLK_API int rlk_det_gemm_ar(void* state, const void* A, const void* B, void* out, int M, int N, int K,
                            long long lda, long long ldb, long long ld_out, int nchunks, void* stream) {
  using namespace rlk;
  SymmState* st = static_cast<SymmState*>(state);
  RLK_REQUIRE(st != nullptr && st->w.world > 1, "det_gemm_ar: needs a symmetric-memory group of 2+ ranks");
  RLK_REQUIRE(M > 0 && N > 0 && K > 0 && N % 8 == 0 && K % 8 == 0, "det_gemm_ar: bad shape");
  RLK_REQUIRE(nchunks == 1 || nchunks == 2 || nchunks == 4 || nchunks == 8, "det_gemm_ar: nchunks must be 1, 2, 4 or 8");
  RLK_REQUIRE(nchunks == 1 || K % (nchunks * 64) == 0, "det_gemm_ar: K/nchunks must be a multiple of 64");
  RLK_REQUIRE(2ll * M * ld_out <= st->w.frame_bytes, "det_gemm_ar: %lld bytes exceed the frame capacity %lld",
              2ll * M * ld_out, st->w.frame_bytes);
  const long long tiles = static_cast<long long>((M + 127) / 128) * ((N + 127) / 128);
  RLK_REQUIRE(tiles < kMaxSlices - 1, "det_gemm_ar: %lld tiles exceed the flag slots", tiles);
  RLK_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15) == 0 && (ld_out * 2) % 16 == 0, "det_gemm_ar: out must be 16-byte aligned");
  st->seq += 1;
  const int frame = static_cast<int>(st->seq & 1);
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.nchunks = nchunks;
  p.kb_per_chunk = nchunks == 1 ? (K + 63) / 64 : K / nchunks / 64;
  p.C = st->peers[st->w.rank] + kFlagBytes + frame * st->w.frame_bytes;
  p.ldc = ld_out;
  p.status = device_status_word();
  p.ar_world = st->w.world;
  p.ar_rank = st->w.rank;
  for (int r = 0; r < st->w.world; ++r) {
    p.ar_frame[r] = st->peers[r] + kFlagBytes + frame * st->w.frame_bytes;
    p.ar_flags[r] = reinterpret_cast<unsigned long long*>(st->peers[r]);
  }
  p.ar_seq = st->seq;
  p.ar_epoch = st->dev_epoch;
  p.ar_use_epoch = st->w.use_epoch;
  p.ar_out = static_cast<__nv_bfloat16*>(out);
  p.ar_ld_out = ld_out;
  // many tiles: 128 x 256 tiles (the faster chunk-tree kernel, tree stack in the L2-resident scratch), as rlk_det_gemm
  // picks them; few tiles: 128 x 128.  All ranks see the same shape, so they number the tiles alike.
  const long long tiles256 = static_cast<long long>((M + 127) / 128) * ((N + 255) / 256);
  if (g_ar_wide_tiles && tiles256 >= sm_count() && (nchunks == 1 || K / nchunks >= 768)) {
    if (nchunks > 1) {
      p.tree_scratch = tree_scratch_for_device();
      if (!p.tree_scratch) return set_error(RLK_ERR_CUDA, "det_gemm_ar: cannot allocate the tree scratch");
    }
    return launch_gemm<256, false, false, true>(A, B, p, lda, ldb, static_cast<cudaStream_t>(stream));
  }
  return launch_gemm<128, false, false, true>(A, B, p, lda, ldb, static_cast<cudaStream_t>(stream));
}

// GEMM + fixed-order reduce-scatter over token rows in ONE kernel (sequence-parallel row-parallel projections):
// out [M / world, N] = rows [rank * M / world, (rank + 1) * M / world) of the tree-all-reduce of the ranks' partial
// products.  Same protocol, frames and tree as rlk_det_gemm_ar -- the bits of a row are those the all-reduce form
// gives -- but a rank pulls and reduces only the tiles of its own rows, so each partial tile crosses NVLink once
// instead of world - 1 times.  M must be a multiple of 128 * world (whole tiles per rank).
RLK_API int rlk_det_gemm_rs(void* state, const void* A, const void* B, void* out, int M, int N, int K,
                            long long lda, long long ldb, long long ld_out, int nchunks, void* stream) {
  using namespace rlk;
  SymmState* st = static_cast<SymmState*>(state);
  RLK_REQUIRE(st != nullptr && st->w.world > 1, "det_gemm_rs: needs a symmetric-memory group of 2+ ranks");
  RLK_REQUIRE(M > 0 && N > 0 && K > 0 && N % 8 == 0 && K % 8 == 0, "det_gemm_rs: bad shape");
  RLK_REQUIRE(M % (128 * st->w.world) == 0, "det_gemm_rs: M (%d) must be a multiple of 128 x world (%d)", M, st->w.world);
  RLK_REQUIRE(nchunks == 1 || nchunks == 2 || nchunks == 4 || nchunks == 8, "det_gemm_rs: nchunks must be 1, 2, 4 or 8");
  RLK_REQUIRE(nchunks == 1 || K % (nchunks * 64) == 0, "det_gemm_rs: K/nchunks must be a multiple of 64");
  RLK_REQUIRE(ld_out >= N, "det_gemm_rs: ld_out (%lld) must be at least N (%d)", ld_out, N);
  RLK_REQUIRE(2ll * M * ld_out <= st->w.frame_bytes, "det_gemm_rs: %lld bytes exceed the frame capacity %lld",
              2ll * M * ld_out, st->w.frame_bytes);
  const long long tiles = static_cast<long long>((M + 127) / 128) * ((N + 127) / 128);
  RLK_REQUIRE(tiles < kMaxSlices - 1, "det_gemm_rs: %lld tiles exceed the flag slots", tiles);
  RLK_REQUIRE(A && B && out && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (ld_out * 2) % 16 == 0,
              "det_gemm_rs: out must be 16-byte aligned");
  st->seq += 1;
  const int frame = static_cast<int>(st->seq & 1);
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.nchunks = nchunks;
  p.kb_per_chunk = nchunks == 1 ? (K + 63) / 64 : K / nchunks / 64;
  p.C = st->peers[st->w.rank] + kFlagBytes + frame * st->w.frame_bytes;
  p.ldc = ld_out;
  p.status = device_status_word();
  p.ar_world = st->w.world;
  p.ar_rank = st->w.rank;
  for (int r = 0; r < st->w.world; ++r) {
    p.ar_frame[r] = st->peers[r] + kFlagBytes + frame * st->w.frame_bytes;
    p.ar_flags[r] = reinterpret_cast<unsigned long long*>(st->peers[r]);
  }
  p.ar_seq = st->seq;
  p.ar_epoch = st->dev_epoch;
  p.ar_use_epoch = st->w.use_epoch;
  const int rows = M / st->w.world;
  p.rs_row0 = st->w.rank * rows;
  p.rs_row1 = p.rs_row0 + rows;
  // only rows [rs_row0, rs_row1) are ever written: bias the base so that they land on the caller's rows 0..rows-1
  p.ar_out = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uintptr_t>(out) - static_cast<uintptr_t>(2ll * p.rs_row0 * ld_out));
  p.ar_ld_out = ld_out;
  // many tiles: 128 x 256 tiles (the faster chunk-tree kernel, tree stack in the L2-resident scratch), as rlk_det_gemm
  // picks them; few tiles: 128 x 128.  All ranks see the same shape, so they number the tiles alike.
  const long long tiles256 = static_cast<long long>((M + 127) / 128) * ((N + 255) / 256);
  if (g_ar_wide_tiles && tiles256 >= sm_count() && (nchunks == 1 || K / nchunks >= 768)) {
    if (nchunks > 1) {
      p.tree_scratch = tree_scratch_for_device();
      if (!p.tree_scratch) return set_error(RLK_ERR_CUDA, "det_gemm_ar: cannot allocate the tree scratch");
    }
    return launch_gemm<256, false, false, true>(A, B, p, lda, ldb, static_cast<cudaStream_t>(stream));
  }
  return launch_gemm<128, false, false, true>(A, B, p, lda, ldb, static_cast<cudaStream_t>(stream));
}

// ---- the variant that allocates nothing (see rlk/no_alloc.h for the contract) ----------------
// The partial results of the chunks live in this array, which is part of the library image.  Its
// name is a host-side stand-in in host code, not a device address: the address the kernels get is
// looked up once per device below.
static __device__ __align__(256) unsigned char g_split_static_scratch[RLK_STATIC_SCRATCH_BYTES];

RLK_API int rlk_det_gemm_split_static(const void* A, const void* B, void* C, int M, int N, int K,
                                      long long lda, long long ldb, long long ldc, int nchunks,
                                      int tile_n, void* stream) {
  using namespace rlk;
  RLK_REQUIRE(M > 0 && N > 0 && K > 0 && N % 8 == 0 && K % 8 == 0, "det_gemm_split_static: bad shape");
  RLK_REQUIRE(nchunks == 2 || nchunks == 4 || nchunks == 8, "det_gemm_split_static: nchunks must be 2, 4 or 8");
  RLK_REQUIRE(K % (nchunks * 64) == 0, "det_gemm_split_static: K/nchunks must be a multiple of 64");
  // unlike rlk_det_gemm_split there is no leaves-only mode: the partials never leave the library
  RLK_REQUIRE(A != nullptr && B != nullptr && C != nullptr, "det_gemm_split_static: A, B and C must not be null");
  RLK_REQUIRE(ldc >= N, "det_gemm_split_static: ldc (%lld) must be at least N (%d)", ldc, N);
  RLK_REQUIRE((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * 2) % 16 == 0,
              "det_gemm_split_static: C must be 16-byte aligned with a 16-byte multiple pitch");
  const long long need = 2ll * nchunks * M * ldc;
  RLK_REQUIRE(need <= RLK_STATIC_SCRATCH_BYTES,
              "det_gemm_split_static: nchunks*M*ldc*2 = %lld bytes exceeds the built-in scratch of %lld bytes; "
              "use rlk_det_gemm_split with your own scratch", need, (long long)RLK_STATIC_SCRATCH_BYTES);
  // once per device, with that device current: the device address of the built-in array
  static unsigned char* dev_ptr[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  RLK_CHECK_CUDA(cudaGetDevice(&dev));
  RLK_REQUIRE(dev >= 0 && dev < 64, "det_gemm_split_static: device index out of range");
  unsigned char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!dev_ptr[dev]) {
      void* ptr = nullptr;
      RLK_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_split_static_scratch));
      dev_ptr[dev] = static_cast<unsigned char*>(ptr);
    }
    scratch = dev_ptr[dev];
  }
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.nchunks = 1;
  p.kb_per_chunk = K / nchunks / 64;
  p.C = scratch; p.ldc = ldc;
  p.status = nullptr;  // no status word: nothing may be allocated here
  p.split_chunks = nchunks;
  p.split_stride = static_cast<long long>(M) * ldc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc;
  if (tile_n == 32) rc = launch_gemm<32, false, false>(A, B, p, lda, ldb, s);
  else if (tile_n == 128) rc = launch_gemm<128, false, false>(A, B, p, lda, ldb, s);
  else rc = launch_gemm<64, false, false>(A, B, p, lda, ldb, s);
  if (rc) return rc;
  const long long n = static_cast<long long>(M) * (N / 8);
  RLK_CHECK_CUDA(launch_pdl(chunk_tree_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s,
                            reinterpret_cast<const __nv_bfloat16*>(scratch), p.split_stride, static_cast<__nv_bfloat16*>(C), M, N, ldc, nchunks));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// Fused vocab-(parallel) LM head: logits tile = H[M,K] * W[N,K]^T is reduced in the GEMM epilogue
// to per-(row, 128-id tile) softmax statistics (see rlk/logp_contract.cuh) without writing the
// [M,N] logits, unless `logits_out` is given.  W holds global vocab ids [vocab_start,
// vocab_start+N); stats rows are float2[stats_stride] indexed by GLOBAL tile id.
// Follow with rlk_logp_merge (after gathering the tiles of the other shards, if any).
static int lmhead_stats_impl(const void* H, const void* W, int M, int N, int K, long long ldh,
                             long long ldw, const long long* targets, long long vocab_start,
                             float inv_temp, const float* min_keep, void* stats, long long stats_stride, float* tgt_logit,
                             void* logits_out, long long ld_logits, void* const* stats_ptrs,
                             void* const* tgt_ptrs, int world, int rank, void* stream) {
  using namespace rlk;
  // the stats epilogue masks ids >= N and the weight rows beyond N read as zero through the tensor map, so N is free
  // unless the logits are also written (their rows then need a 16-byte pitch)
  RLK_REQUIRE(M > 0 && N > 0 && K > 0 && K % 8 == 0 && (N % 8 == 0 || logits_out == nullptr),
              "lmhead_logp_stats: bad shape");
  RLK_REQUIRE(vocab_start % kVocabTile == 0, "lmhead_logp_stats: vocab_start must be a multiple of 128");
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.nchunks = 1;
  p.kb_per_chunk = (K + 63) / 64;
  p.C = logits_out; p.ldc = ld_logits; p.out_fp32 = 0; p.accumulate = 0;
  p.status = device_status_word();
  p.stats = static_cast<float2*>(stats);
  p.stats_stride = stats_stride;
  p.stats_tile0 = static_cast<int>(vocab_start / kVocabTile);
  p.targets = targets;
  p.vocab_start = vocab_start;
  p.tgt_logit = tgt_logit;
  p.inv_temp = inv_temp;
  p.min_keep = min_keep;
  p.stats_world = world > 1 ? world : 0;
  p.stats_rank = rank;
  for (int i = 0; i < 8; ++i) {
    p.stats_peer[i] = world > 1 ? static_cast<float2*>(stats_ptrs[i < world ? i : 0]) : nullptr;
    p.tgt_peer[i] = world > 1 ? static_cast<float*>(tgt_ptrs[i < world ? i : 0]) : nullptr;
  }
  // enough 256-wide tiles for every SM: full tensor-core rate, each set of epilogue warps reduces
  // its own vocabulary tile; otherwise 128-wide tiles (more of them)
  const long long tiles256 = static_cast<long long>((M + 127) / 128) * ((N + 255) / 256);
  if (tiles256 >= 2 * sm_count())
    return launch_gemm<256, false, false>(H, W, p, ldh, ldw, static_cast<cudaStream_t>(stream));
  return launch_gemm<128, false, false>(H, W, p, ldh, ldw, static_cast<cudaStream_t>(stream));
}

RLK_API int rlk_lmhead_logp_stats(const void* H, const void* W, int M, int N, int K, long long ldh,
                                  long long ldw, const long long* targets, long long vocab_start,
                                  float inv_temp, void* stats, long long stats_stride,
                                  float* tgt_logit, void* logits_out, long long ld_logits,
                                  void* stream) {
  return lmhead_stats_impl(H, W, M, N, K, ldh, ldw, targets, vocab_start, inv_temp, nullptr, stats, stats_stride,
                           tgt_logit, logits_out, ld_logits, nullptr, nullptr, 1, 0, stream);
}

// The same with a restricted sampling support: min_keep[row] is the smallest scaled logit
// (logit * inv_temp) that top-k / top-p kept for that row at rollout time; smaller logits count as
// -inf in the statistics and in the target logit, exactly as if the logits had been masked first.
RLK_API int rlk_lmhead_logp_stats_keep(const void* H, const void* W, int M, int N, int K, long long ldh,
                                       long long ldw, const long long* targets, long long vocab_start,
                                       float inv_temp, const float* min_keep, void* stats, long long stats_stride,
                                       float* tgt_logit, void* logits_out, long long ld_logits, void* stream) {
  return lmhead_stats_impl(H, W, M, N, K, ldh, ldw, targets, vocab_start, inv_temp, min_keep, stats, stats_stride,
                           tgt_logit, logits_out, ld_logits, nullptr, nullptr, 1, 0, stream);
}

// Vocab-parallel form: stats_ptrs[r] / tgt_ptrs[r] are rank r's stats and target-logit buffers as
// mapped in this process (this rank's own at index `rank`), all with the same geometry.  The
// epilogue stores every statistic of this shard into all `world` buffers; after a barrier of the
// group each rank can run rlk_logp_merge on complete rows.  Tiles no shard owns (vocab padding)
// must hold (-inf, 0) beforehand.
RLK_API int rlk_lmhead_logp_stats_vp(const void* H, const void* W, int M, int N, int K, long long ldh,
                                     long long ldw, const long long* targets, long long vocab_start,
                                     float inv_temp, void* const* stats_ptrs, long long stats_stride,
                                     void* const* tgt_ptrs, int world, int rank, void* stream) {
  RLK_REQUIRE(world >= 2 && world <= 8 && rank >= 0 && rank < world, "lmhead_logp_stats_vp: world must be 2..8");
  return lmhead_stats_impl(H, W, M, N, K, ldh, ldw, targets, vocab_start, inv_temp, nullptr, stats_ptrs[rank],
                           stats_stride, static_cast<float*>(tgt_ptrs[rank]), nullptr, 0, stats_ptrs, tgt_ptrs,
                           world, rank, stream);
}

RLK_API int rlk_lmhead_logp_stats_vp_keep(const void* H, const void* W, int M, int N, int K, long long ldh,
                                          long long ldw, const long long* targets, long long vocab_start,
                                          float inv_temp, const float* min_keep, void* const* stats_ptrs,
                                          long long stats_stride, void* const* tgt_ptrs, int world, int rank,
                                          void* stream) {
  RLK_REQUIRE(world >= 2 && world <= 8 && rank >= 0 && rank < world, "lmhead_logp_stats_vp: world must be 2..8");
  return lmhead_stats_impl(H, W, M, N, K, ldh, ldw, targets, vocab_start, inv_temp, min_keep, stats_ptrs[rank],
                           stats_stride, static_cast<float*>(tgt_ptrs[rank]), nullptr, 0, stats_ptrs, tgt_ptrs,
                           world, rank, stream);
}
