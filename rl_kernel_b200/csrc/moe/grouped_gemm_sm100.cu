// Grouped (per-expert) bf16 GEMM for sm_100a driven by a device-resident tile list.
//
// A mixture-of-experts layer multiplies a data-dependent number of rows with every expert's
// weights.  The routing kernels (moe_routing.cu) lay the rows of each expert out back to back,
// padded to the 128-row tile, and write one GroupTile per output tile; this kernel is a persistent
// TMA -> tcgen05.mma -> TMEM pipeline that walks that list.  The host never learns the counts, so a
// whole layer can be enqueued (or graph-captured) without a synchronisation.
//
// All operands are plain 2-D tensors: the weights of all experts are stacked along rows, so the
// expert only shows up as a row offset inside the tile record.  The three operand layouts cover
//   forward          C[rows, N]   = A[rows, K] * W[e][N, K]^T          (A K-major, B K-major)
//   input gradient   dA[rows, K]  = dC[rows, N] * W[e][N, K]           (A K-major, B MN-major)
//   weight gradient  dW[e][N, K] += dC_e[rows, N]^T * A_e[rows, K]     (A MN-major, B MN-major,
//                                                                      contraction over the rows)
// Numerical contract: one fp32 TMEM accumulator per output element, k ascending, no split-K, no
// atomics; a row's result does not depend on which other rows share its tile, so the outputs of
// a token are independent of how many tokens every expert received.
//
// The reference has no grouped GEMM (its MoE packages are empty placeholders,
// rl_engine/ops/moe/__init__.py); this is the expert-GEMM part of its roadmap.
#include "rlk/host.h"
#include "rlk/moe.h"
#include "rlk/ptx.cuh"

namespace rlk {

constexpr int GBM = 128, GBN = 256, GBK = 64;
constexpr int kGroupedThreads = 192;  // warp0 TMA, warp1 MMA, warps2-5 epilogue
constexpr int kGStageA = GBM * GBK * 2;
constexpr int kGStageB = GBN * GBK * 2;
constexpr int kGStage = kGStageA + kGStageB;
constexpr int kGStages = 4;
constexpr int kGSmemBytes = kGStages * kGStage + 1024 + 256;

struct GroupedParams {
  const GroupTile* tiles;
  const int* n_tiles;     // device scalar
  __nv_bfloat16* C;
  long long ldc;
  int accumulate;         // C += result (fp32 add, rounded to bf16)
  int* status;
};

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGroupedThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kGStages * kGStage);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kGStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kGStages);
  const uint32_t accf0 = smem_u32(bars + 2 * kGStages), acce0 = smem_u32(bars + 2 * kGStages + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGStages; ++s) {
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
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total = *p.n_tiles;
  const uint32_t smem_base = smem_u32(smem);

  // Producer and MMA warps: all 32 lanes walk the loops (warp-uniform state), one elected lane
  // issues, waits are warp votes.
  if (warp == 0) {
    {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total; t += gridDim.x) {
        const GroupTile g = p.tiles[t];
        for (int kb = 0; kb < g.kblocks; ++kb, ++it) {
          const uint32_t s = it % kGStages, ph = (it / kGStages) & 1;
          if (!mbar_wait_warp(empty0 + 8 * s, ph ^ 1, abort_flag, p.status, 401)) break;
          const uint32_t fb = full0 + 8 * s;
          const uint32_t sa = smem_base + s * kGStage, sb = sa + kGStageA;
          if (!elect_one()) continue;
          mbar_expect_tx(fb, kGStage);
          if (!A_MN) {
            tma_load_2d(sa, &tmA, g.ka0 + kb * GBK, g.a_m0, fb);
          } else {
#pragma unroll
            for (int i = 0; i < GBM / 64; ++i) tma_load_2d(sa + i * 8192, &tmA, g.a_m0 + 64 * i, g.ka0 + kb * GBK, fb);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmB, g.kb0 + kb * GBK, g.b_n0, fb);
          } else {
#pragma unroll
            for (int i = 0; i < GBN / 64; ++i) tma_load_2d(sb + i * 8192, &tmB, g.b_n0 + 64 * i, g.kb0 + kb * GBK, fb);
          }
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    {
      constexpr uint32_t idesc = umma_idesc_bf16(GBM, GBN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0, u = 0;
      for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x, ++u) {
        const int kblocks = p.tiles[t].kblocks;
        const uint32_t a = u & 1;
        if (!mbar_wait_warp(acce0 + 8 * a, ((u >> 1) & 1) ^ 1, abort_flag, p.status, 402)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * GBN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % kGStages, ph = (it / kGStages) & 1;
          if (!mbar_wait_warp(full0 + 8 * s, ph, abort_flag, p.status, 403)) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * kGStage, sb = sa + kGStageA;
          if (!elect_one()) continue;
#pragma unroll
          for (int k = 0; k < GBK / 16; ++k) {
            const uint64_t da = A_MN ? umma_desc_sw128(sa + k * 2048, 8192, 1024)
                                     : umma_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_desc_sw128(sb + k * 2048, 8192, 1024)
                                     : umma_desc_sw128(sb + k * 32, 16, 1024);
            umma_bf16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * s);
        }
        if (elect_one()) umma_commit(accf0 + 8 * a);
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t u = 0;
    for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x, ++u) {
      const GroupTile g = p.tiles[t];
      const uint32_t a = u & 1;
      if (!mbar_wait(accf0 + 8 * a, (u >> 1) & 1, abort_flag, p.status, 404)) break;
      tc_fence_after();
      __nv_bfloat16* dst = p.C + static_cast<long long>(g.c_row + r) * p.ldc + g.c_col;
#pragma unroll 1
      for (int col0 = 0; col0 < GBN; col0 += 32) {
        uint32_t x[32];
        tmem_ld32(tmem_base + lane_off + a * GBN + col0, x);
        tmem_ld_wait();
        if (r < g.rows_valid && g.kblocks > 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(x[j]), __uint_as_float(x[j + 1]));
            o.y = pack_bf16x2(__uint_as_float(x[j + 2]), __uint_as_float(x[j + 3]));
            o.z = pack_bf16x2(__uint_as_float(x[j + 4]), __uint_as_float(x[j + 5]));
            o.w = pack_bf16x2(__uint_as_float(x[j + 6]), __uint_as_float(x[j + 7]));
            if (p.accumulate) {
              const uint4 q = *reinterpret_cast<const uint4*>(dst + col0 + j);
              o.x = pack_bf16x2(bf16_lo(o.x) + bf16_lo(q.x), bf16_hi(o.x) + bf16_hi(q.x));
              o.y = pack_bf16x2(bf16_lo(o.y) + bf16_lo(q.y), bf16_hi(o.y) + bf16_hi(q.y));
              o.z = pack_bf16x2(bf16_lo(o.z) + bf16_lo(q.z), bf16_hi(o.z) + bf16_hi(q.z));
              o.w = pack_bf16x2(bf16_lo(o.w) + bf16_lo(q.w), bf16_hi(o.w) + bf16_hi(q.w));
            }
            *reinterpret_cast<uint4*>(dst + col0 + j) = o;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(acce0 + 8 * a);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <bool A_MN, bool B_MN>
static int launch_grouped(const void* A, long long a_rows, long long a_cols, long long lda, const void* B,
                          long long b_rows, long long b_cols, long long ldb, const GroupedParams& p,
                          int max_tiles, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc;
  // K-major operand [rows = MN, cols = K]: box 64 (k) x tile rows.  MN-major operand
  // [rows = K, cols = MN]: box 64 (mn) x 64 (k), one box per 64 MN elements.
  if ((rc = make_tmap_2d_sw128(&tmA, A, a_rows, a_cols, lda, A_MN ? GBK : GBM, 64, 2))) return rc;
  if ((rc = make_tmap_2d_sw128(&tmB, B, b_rows, b_cols, ldb, B_MN ? GBK : GBN, 64, 2))) return rc;
  auto kfn = grouped_gemm_kernel<A_MN, B_MN>;
  static bool attr_set[64] = {false};
  int dev = 0;
  RLK_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    RLK_CHECK_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, kGSmemBytes));
    attr_set[dev & 63] = true;
  }
  const int grid = max_tiles < sm_count() ? max_tiles : sm_count();
  kfn<<<grid, kGroupedThreads, kGSmemBytes, stream>>>(tmA, tmB, p);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

}  // namespace rlk
using namespace rlk;

// A: [a_rows, a_cols] bf16 with pitch lda; B: [b_rows, b_cols] with pitch ldb; C bf16 with pitch
// ldc.  `tiles` / `n_tiles` are device memory (rlk::GroupTile records and their count, at most
// max_tiles).  a_mn / b_mn: the operand's rows are the contraction dimension.  Output tiles are
// 128 x 256; every tile's 256 columns and, for K-major A, its 128 A rows must exist in the tensors
// (the routing kernels pad each expert's rows to 128).
RLK_API int rlk_grouped_gemm(const void* A, long long a_rows, long long a_cols, long long lda,
                             const void* B, long long b_rows, long long b_cols, long long ldb,
                             void* C, long long ldc, const void* tiles, const int* n_tiles,
                             int max_tiles, int a_mn, int b_mn, int accumulate, void* stream) {
  RLK_REQUIRE(max_tiles > 0, "grouped_gemm: max_tiles must be positive");
  RLK_REQUIRE((ldc * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0, "grouped_gemm: C must be 16-byte aligned");
  GroupedParams p{static_cast<const GroupTile*>(tiles), n_tiles, static_cast<__nv_bfloat16*>(C), ldc,
                  accumulate, device_status_word()};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch_grouped<false, false>(A, a_rows, a_cols, lda, B, b_rows, b_cols, ldb, p, max_tiles, s);
  if (!a_mn && b_mn) return launch_grouped<false, true>(A, a_rows, a_cols, lda, B, b_rows, b_cols, ldb, p, max_tiles, s);
  if (a_mn && b_mn) return launch_grouped<true, true>(A, a_rows, a_cols, lda, B, b_rows, b_cols, ldb, p, max_tiles, s);
  RLK_REQUIRE(false, "grouped_gemm: A MN-major with B K-major is not instantiated");
  return RLK_OK;
}
