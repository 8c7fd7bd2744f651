// Deterministic attention backward for sm_100a (head_dim 128, bf16), three kernels:
//
//   attn_bwd_delta : delta[row, head] = sum_d dO * O                        (fp32 scratch)
//   attn_bwd_dq    : one CTA per query tile, KV blocks in ascending order,
//                    dQ accumulated in TMEM across blocks
//   attn_bwd_dkv   : one CTA per (128-key block, KV head), the query heads of the GQA group and
//                    the query tiles that see the block in ascending order, dK and dV accumulated
//                    in TMEM
// Both main kernels recompute S = Q K^T and P = exp(S*scale - lse) with tcgen05 and never use
// atomics or split accumulation, so gradients are bitwise reproducible run to run and do not
// depend on the batch size.  (The reference relies on FA4's deterministic backward,
// rl_engine/backends/cuda/attention/flash_attn.py:343-353, or the materialising kernels of
// csrc/cuda/attention/deterministic_attention.cu:385-561.)
#include "rlk/attn_common.cuh"
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

constexpr int kBwdThreads = 576;  // TMA warp, UMMA warp, 16 compute warps (4 threads per row)
constexpr int kTile = 128 * 128 * 2;
constexpr int kHalf = 128 * 64 * 2;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float bwd_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------------------------ delta
__global__ void __launch_bounds__(256)
attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ O, long long ldo, const __nv_bfloat16* __restrict__ dO,
                      long long lddo, float* __restrict__ delta, int T, int Hq) {
  const long long gw = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(T) * Hq) return;
  const long long t = gw / Hq;
  const int h = static_cast<int>(gw % Hq);
  const uint2 a = *reinterpret_cast<const uint2*>(O + t * ldo + h * 128 + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dO + t * lddo + h * 128 + lane * 4);
  float s = bf16_lo(a.x) * bf16_lo(b.x);
  s = fmaf(bf16_hi(a.x), bf16_hi(b.x), s);
  s = fmaf(bf16_lo(a.y), bf16_lo(b.y), s);
  s = fmaf(bf16_hi(a.y), bf16_hi(b.y), s);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) delta[gw] = s;
}

// ------------------------------------------------------------------------------------ dQ
struct AttnDqParams {
  const AttnTile* tiles;
  int n_tiles;
  const float* lse;    // same indexing as forward (tile.lse_off + r * tile.lse_stride)
  const float* delta;  // same indexing
  __nv_bfloat16* dQ;
  long long lddq;
  float scale, scale_log2;
  CpLayout cp;         // context parallel: which rank's K/V holds canonical block b
  CpStage stage;       // remote K/V blocks are copied once into local memory (rows = 0: off)
  int* status;
};

struct DqSmem {
  static constexpr int kQ = 0;
  static constexpr int kDO = kQ + kTile;
  static constexpr int kK = kDO + kTile;
  static constexpr int kV = kK + 2 * kTile;
  static constexpr int kDS = kV + 2 * kTile;
  static constexpr int kBars = kDS + kTile;
  static constexpr int kBytes = kBars + 256 + 1024;
};

template <int NSRC>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ KvMaps<NSRC> kv, const __grid_constant__ KvMaps<1> staged,
                   const AttnDqParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DqSmem::kBars);
  enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, SDP_FULL = 9, DS_FULL = 10,
         DS_EMPTY = 11, ACC_FULL = 12, NBARS = 13 };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const AttnTile t = p.tiles[blockIdx.x];
  const bool use_stage = NSRC > 1 && p.stage.rows > 0;
  volatile int* stage_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);
  if (t.n_rows <= 0) {
    if (use_stage && warp >= 2) cp_stage_gather(p.stage, threadIdx.x - 64, kBwdThreads - 64, 3, stage_slot);
    return;
  }
  int max_kv = t.pos0 + (t.n_rows - 1) * t.pos_step + 1;
  if (max_kv > t.kv_cap) max_kv = t.kv_cap;
  const int nblk = (max_kv + kAttnBlock - 1) / kAttnBlock;

  if (threadIdx.x == 0) {
    mbar_init(BAR(Q_FULL), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(BAR(K_FULL + s), 1);
      mbar_init(BAR(K_EMPTY + s), 1);
      mbar_init(BAR(V_FULL + s), 1);
      mbar_init(BAR(V_EMPTY + s), 1);
    }
    mbar_init(BAR(SDP_FULL), 1);
    mbar_init(BAR(DS_FULL), 512);
    mbar_init(BAR(DS_EMPTY), 1);
    mbar_init(BAR(ACC_FULL), 1);
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
  const uint32_t sQ = smem_u32(smem + DqSmem::kQ), sDO = smem_u32(smem + DqSmem::kDO);
  const uint32_t sK = smem_u32(smem + DqSmem::kK), sV = smem_u32(smem + DqSmem::kV);
  const uint32_t sDS = smem_u32(smem + DqSmem::kDS);
  constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DQ = 256;

  // Producer and MMA warps: all 32 lanes walk the loops (warp-uniform state lives in uniform
  // registers, where the TMA / MMA / barrier instructions take their operands from), one elected
  // lane issues, waits are warp votes.
  if (warp == 0) {
    {
      if (elect_one()) {
        mbar_expect_tx(BAR(Q_FULL), 2 * kTile);
        tma_load_2d(sQ, &tmQ, t.q_col0, t.q_row0, BAR(Q_FULL));
        tma_load_2d(sQ + kHalf, &tmQ, t.q_col0 + 64, t.q_row0, BAR(Q_FULL));
        tma_load_2d(sDO, &tmDO, t.q_col0, t.q_row0, BAR(Q_FULL));
        tma_load_2d(sDO + kHalf, &tmDO, t.q_col0 + 64, t.q_row0, BAR(Q_FULL));
      }
      for (int b = 0; b < nblk; ++b) {
        const int s = b & 1;
        const uint32_t ph = (b >> 1) & 1;
        int src, lb;
        cp_locate_block(p.cp, b, src, lb);   // plain TMA loads, possibly from a peer's memory
        if (NSRC == 1) src = 0;
        int row = t.kv_row0 + lb * kAttnBlock;
        const CUtensorMap* mk = &kv.k[src];
        const CUtensorMap* mv = &kv.v[src];
        if (use_stage && src != p.stage.rank) {
          if (!__all_sync(0xffffffffu, cp_stage_wait(p.stage, src, row / kAttnBlock, abort_flag, p.status, 320))) break;
          row += src * p.stage.rows;
          mk = &staged.k[0];
          mv = &staged.v[0];
        }
        if (!mbar_wait_warp(BAR(K_EMPTY + s), ph ^ 1, abort_flag, p.status, 301)) break;
        if (elect_one()) {
          mbar_expect_tx(BAR(K_FULL + s), kTile);
          tma_load_2d(sK + s * kTile, mk, t.kv_col0, row, BAR(K_FULL + s));
          tma_load_2d(sK + s * kTile + kHalf, mk, t.kv_col0 + 64, row, BAR(K_FULL + s));
        }
        if (!mbar_wait_warp(BAR(V_EMPTY + s), ph ^ 1, abort_flag, p.status, 302)) break;
        if (elect_one()) {
          mbar_expect_tx(BAR(V_FULL + s), kTile);
          tma_load_2d(sV + s * kTile, mv, t.kv_col0, row, BAR(V_FULL + s));
          tma_load_2d(sV + s * kTile + kHalf, mv, t.kv_col0 + 64, row, BAR(V_FULL + s));
        }
      }
    }
  } else if (warp == 1) {
    {
      constexpr uint32_t idesc_kk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_kmn = umma_idesc_bf16(128, 128, 0, 1);
      bool ok = mbar_wait_warp(BAR(Q_FULL), 0, abort_flag, p.status, 303);
      for (int b = 0; ok && b < nblk; ++b) {
        const int s = b & 1;
        const uint32_t ph = (b >> 1) & 1;
        if (!mbar_wait_warp(BAR(K_FULL + s), ph, abort_flag, p.status, 304)) break;
        if (!mbar_wait_warp(BAR(V_FULL + s), ph, abort_flag, p.status, 305)) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = (k >> 2) * kHalf + (k & 3) * 32;
            umma_bf16_ss(tmem_base + TM_S, umma_desc_sw128(sQ + off, 16, 1024),
                         umma_desc_sw128(sK + s * kTile + off, 16, 1024), idesc_kk, k != 0);
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = (k >> 2) * kHalf + (k & 3) * 32;
            umma_bf16_ss(tmem_base + TM_DP, umma_desc_sw128(sDO + off, 16, 1024),
                         umma_desc_sw128(sV + s * kTile + off, 16, 1024), idesc_kk, k != 0);
          }
          umma_commit(BAR(SDP_FULL));
          umma_commit(BAR(V_EMPTY + s));
        }
        if (!mbar_wait_warp(BAR(DS_FULL), b & 1, abort_flag, p.status, 306)) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t aoff = (k >> 2) * kHalf + (k & 3) * 32;
            umma_bf16_ss(tmem_base + TM_DQ, umma_desc_sw128(sDS + aoff, 16, 1024),
                         umma_desc_sw128(sK + s * kTile + k * 2048, kHalf, 1024), idesc_kmn,
                         (b | k) != 0);
          }
          umma_commit(BAR(K_EMPTY + s));
          umma_commit(BAR(DS_EMPTY));
        }
      }
      if (elect_one()) umma_commit(BAR(ACC_FULL));
    }
  } else {
    // warp -> (quad, split): quad = TMEM lane quadrant, split = which 32 of the 128 columns
    const int quad = warp & 3;
    const int split = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    int kv_len = t.pos0 + r * t.pos_step + 1;
    if (kv_len > t.kv_cap) kv_len = t.kv_cap;
    if (r >= t.n_rows) kv_len = 0;
    float lse2 = 0.f, dlt = 0.f;
    if (r < t.n_rows) {
      const long long li = t.lse_off + static_cast<long long>(r) * t.lse_stride;
      lse2 = p.lse[li] * kLog2e;
      dlt = p.delta[li];
    }
    uint8_t* ds_base = smem + DqSmem::kDS;
    if (use_stage) cp_stage_gather(p.stage, threadIdx.x - 64, kBwdThreads - 64, 3, stage_slot);
    for (int b = 0; b < nblk; ++b) {
      if (!mbar_wait(BAR(SDP_FULL), b & 1, abort_flag, p.status, 307)) break;
      // the previous block's dQ MMA must have finished reading the dS tile
      if (b > 0 && !mbar_wait(BAR(DS_EMPTY), (b - 1) & 1, abort_flag, p.status, 308)) break;
      tc_fence_after();
      const int nvis = kv_len - b * kAttnBlock - split * 32;
      uint32_t sx[32], dx[32];
      tmem_ld32(tmem_base + lane_off + TM_S + split * 32, sx);
      tmem_ld32(tmem_base + lane_off + TM_DP + split * 32, dx);
      tmem_ld_wait();
      uint32_t pk[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        float d0 = 0.f, d1 = 0.f;
        if (j < nvis) {
          const float pr = bwd_exp2(fmaf(__uint_as_float(sx[j]), p.scale_log2, -lse2));
          d0 = pr * (__uint_as_float(dx[j]) - dlt) * p.scale;
        }
        if (j + 1 < nvis) {
          const float pr = bwd_exp2(fmaf(__uint_as_float(sx[j + 1]), p.scale_log2, -lse2));
          d1 = pr * (__uint_as_float(dx[j + 1]) - dlt) * p.scale;
        }
        pk[j >> 1] = pack_bf16x2(d0, d1);
      }
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4)
        *reinterpret_cast<uint4*>(ds_base + (split >> 1) * kHalf + sw128_offset(r, (split & 1) * 4 + q4)) =
            make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(BAR(DS_FULL));
    }
    if (mbar_wait(BAR(ACC_FULL), 0, abort_flag, p.status, 309)) {
      tc_fence_after();
      __nv_bfloat16* dst = p.dQ + static_cast<long long>(t.q_row0 + r) * p.lddq + t.q_col0 + split * 32;
      uint32_t x[32];
      if (nblk > 0) {
        tmem_ld32(tmem_base + lane_off + TM_DQ + split * 32, x);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] = 0u;
      }
      if (r < t.n_rows) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(x[j]), __uint_as_float(x[j + 1]));
          v.y = pack_bf16x2(__uint_as_float(x[j + 2]), __uint_as_float(x[j + 3]));
          v.z = pack_bf16x2(__uint_as_float(x[j + 4]), __uint_as_float(x[j + 5]));
          v.w = pack_bf16x2(__uint_as_float(x[j + 6]), __uint_as_float(x[j + 7]));
          *reinterpret_cast<uint4*>(dst + j) = v;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------ dK / dV
struct AttnKvTile {
  int kv_row;      // y coordinate of the first key of this 128-key block in K / V / dK / dV
  int kv_col0;     // x coordinate of the KV head
  int key0;        // position (key index within the sequence) of the first key of the block
  int n_keys;      // valid keys in the block (1..128)
  int q_row0;      // y coordinate in Q / dO of the sequence's first query row
  int q_pos0;      // position of that first query row
  int n_q;         // query rows of the sequence
  int q_col0;      // x coordinate of the first query head of the GQA group
  int group;       // query heads per KV head
  int lse_off;     // lse index of (query row 0, first head of the group)
  int lse_stride;  // index step between consecutive query rows
  int lse_head_stride;  // index step between consecutive heads
};

struct AttnDkvParams {
  const AttnKvTile* tiles;
  int n_tiles;
  const float* lse[8];    // per context-parallel rank (index 0 only when not context parallel)
  const float* delta[8];
  CpLayout cp;            // which rank holds query tile qt of a sequence, and where
  CpStage stage;          // remote Q / dO tiles are copied once into local memory (rows = 0: off)
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  long long lddkv;
  float scale, scale_log2;
  int* status;
};

struct DkvSmem {
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTile;
  static constexpr int kQ = kV + kTile;
  static constexpr int kDO = kQ + kTile;
  static constexpr int kP = kDO + kTile;
  static constexpr int kDS = kP + kTile;
  static constexpr int kBars = kDS + kTile;
  static constexpr int kBytes = kBars + 256 + 1024;
};

// Context parallel (NSRC > 1): the key block is local; the query tiles that see it are spread over
// the ranks.  Q and dO tiles arrive through the owning rank's tensor maps (qdo.k = Q, qdo.v = dO)
// and lse / delta through plain peer loads, in the same ascending query-tile order as on one GPU.
template <int NSRC>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ KvMaps<NSRC> qdo, const __grid_constant__ KvMaps<1> staged,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const AttnDkvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DkvSmem::kBars);
  enum { KV_FULL = 0, Q_FULL = 1, Q_EMPTY = 2, SDP_FULL = 3, PDS_FULL = 4, ACC_FULL = 5, NBARS = 6 };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const AttnKvTile t = p.tiles[blockIdx.x];
  const bool use_stage = NSRC > 1 && p.stage.rows > 0;
  volatile int* stage_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);
  if (t.n_keys <= 0) {
    if (use_stage && warp >= 2) cp_stage_gather(p.stage, threadIdx.x - 64, kBwdThreads - 64, 3, stage_slot);
    return;
  }
  // first query row that can see key0, rounded down to the sequence's 128-row tile grid
  int i0 = t.key0 - t.q_pos0;
  if (i0 < 0) i0 = 0;
  const int qt0 = i0 / 128;
  const int qt1 = (t.n_q + 127) / 128;
  const int n_qt = qt1 > qt0 ? qt1 - qt0 : 0;
  const int n_iter = n_qt * t.group;

  if (threadIdx.x == 0) {
    mbar_init(BAR(KV_FULL), 1);
    mbar_init(BAR(Q_FULL), 1);
    mbar_init(BAR(Q_EMPTY), 1);
    mbar_init(BAR(SDP_FULL), 1);
    mbar_init(BAR(PDS_FULL), 512);
    mbar_init(BAR(ACC_FULL), 1);
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
  const uint32_t sK = smem_u32(smem + DkvSmem::kK), sV = smem_u32(smem + DkvSmem::kV);
  const uint32_t sQ = smem_u32(smem + DkvSmem::kQ), sDO = smem_u32(smem + DkvSmem::kDO);
  const uint32_t sP = smem_u32(smem + DkvSmem::kP), sDS = smem_u32(smem + DkvSmem::kDS);
  constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DK = 256, TM_DV = 384;

  if (warp == 0) {     // (all lanes walk the loops, one elected lane issues: see the dQ kernel)
    {
      if (elect_one()) {
        mbar_expect_tx(BAR(KV_FULL), 2 * kTile);
        tma_load_2d(sK, &tmK, t.kv_col0, t.kv_row, BAR(KV_FULL));
        tma_load_2d(sK + kHalf, &tmK, t.kv_col0 + 64, t.kv_row, BAR(KV_FULL));
        tma_load_2d(sV, &tmV, t.kv_col0, t.kv_row, BAR(KV_FULL));
        tma_load_2d(sV + kHalf, &tmV, t.kv_col0 + 64, t.kv_row, BAR(KV_FULL));
      }
      for (int it = 0; it < n_iter; ++it) {
        const int g = it / n_qt, qt = qt0 + it % n_qt;
        if (!mbar_wait_warp(BAR(Q_EMPTY), (it & 1) ^ 1, abort_flag, p.status, 311)) break;
        int src, lb;
        cp_locate_block(p.cp, qt, src, lb);
        if (NSRC == 1) src = 0;
        int row = t.q_row0 + lb * 128;
        const int col = t.q_col0 + g * 128;
        const CUtensorMap* mq = &qdo.k[src];
        const CUtensorMap* md = &qdo.v[src];
        if (use_stage && src != p.stage.rank) {
          if (!__all_sync(0xffffffffu, cp_stage_wait(p.stage, src, row / 128, abort_flag, p.status, 321))) break;
          row += src * p.stage.rows;
          mq = &staged.k[0];
          md = &staged.v[0];
        }
        if (elect_one()) {
          mbar_expect_tx(BAR(Q_FULL), 2 * kTile);
          tma_load_2d(sQ, mq, col, row, BAR(Q_FULL));
          tma_load_2d(sQ + kHalf, mq, col + 64, row, BAR(Q_FULL));
          tma_load_2d(sDO, md, col, row, BAR(Q_FULL));
          tma_load_2d(sDO + kHalf, md, col + 64, row, BAR(Q_FULL));
        }
      }
    }
  } else if (warp == 1) {
    {
      constexpr uint32_t idesc_kk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_mm = umma_idesc_bf16(128, 128, 1, 1);
      bool ok = mbar_wait_warp(BAR(KV_FULL), 0, abort_flag, p.status, 312);
      for (int it = 0; ok && it < n_iter; ++it) {
        if (!mbar_wait_warp(BAR(Q_FULL), it & 1, abort_flag, p.status, 313)) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {  // S[q][key] = Q K^T
            const uint32_t off = (k >> 2) * kHalf + (k & 3) * 32;
            umma_bf16_ss(tmem_base + TM_S, umma_desc_sw128(sQ + off, 16, 1024),
                         umma_desc_sw128(sK + off, 16, 1024), idesc_kk, k != 0);
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {  // dP[q][key] = dO V^T
            const uint32_t off = (k >> 2) * kHalf + (k & 3) * 32;
            umma_bf16_ss(tmem_base + TM_DP, umma_desc_sw128(sDO + off, 16, 1024),
                         umma_desc_sw128(sV + off, 16, 1024), idesc_kk, k != 0);
          }
          umma_commit(BAR(SDP_FULL));
        }
        if (!mbar_wait_warp(BAR(PDS_FULL), it & 1, abort_flag, p.status, 314)) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {  // dV[key][d] += P^T dO   (contraction over the 128 query rows)
            umma_bf16_ss(tmem_base + TM_DV, umma_desc_sw128(sP + k * 2048, kHalf, 1024),
                         umma_desc_sw128(sDO + k * 2048, kHalf, 1024), idesc_mm, (it | k) != 0);
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {  // dK[key][d] += dS^T Q
            umma_bf16_ss(tmem_base + TM_DK, umma_desc_sw128(sDS + k * 2048, kHalf, 1024),
                         umma_desc_sw128(sQ + k * 2048, kHalf, 1024), idesc_mm, (it | k) != 0);
          }
          umma_commit(BAR(Q_EMPTY));
        }
      }
      if (elect_one()) umma_commit(BAR(ACC_FULL));
    }
  } else {
    const int quad = warp & 3;
    const int split = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    uint8_t* p_base = smem + DkvSmem::kP;
    uint8_t* ds_base = smem + DkvSmem::kDS;
    if (use_stage) cp_stage_gather(p.stage, threadIdx.x - 64, kBwdThreads - 64, 3, stage_slot);
    for (int it = 0; it < n_iter; ++it) {
      const int g = it / n_qt, qt = qt0 + it % n_qt;
      const int qi = qt * 128 + r;  // query row index within the sequence
      float lse2 = 0.f, dlt = 0.f;
      int nvis = 0;  // keys of this block visible to this query row
      if (qi < t.n_q) {
        int src, lb;
        cp_locate_block(p.cp, qt, src, lb);
        if (NSRC == 1) src = 0;
        const long long li = t.lse_off + static_cast<long long>(lb * 128 + r) * t.lse_stride +
                             static_cast<long long>(g) * t.lse_head_stride;
        lse2 = p.lse[src][li] * kLog2e;
        dlt = p.delta[src][li];
        nvis = t.q_pos0 + qi + 1 - t.key0;
        if (nvis > t.n_keys) nvis = t.n_keys;
      }
      nvis -= split * 32;           // among this thread's 32 keys
      if (!mbar_wait(BAR(SDP_FULL), it & 1, abort_flag, p.status, 315)) break;
      // P / dS tiles of the previous iteration must have been consumed (Q_EMPTY commit covers them)
      if (it > 0 && !mbar_wait(BAR(Q_EMPTY), (it - 1) & 1, abort_flag, p.status, 316)) break;
      tc_fence_after();
      uint32_t sx[32], dx[32];
      tmem_ld32(tmem_base + lane_off + TM_S + split * 32, sx);
      tmem_ld32(tmem_base + lane_off + TM_DP + split * 32, dx);
      tmem_ld_wait();
      uint32_t pp[16], pd[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        float p0 = 0.f, p1 = 0.f, d0 = 0.f, d1 = 0.f;
        if (j < nvis) {
          p0 = bwd_exp2(fmaf(__uint_as_float(sx[j]), p.scale_log2, -lse2));
          d0 = p0 * (__uint_as_float(dx[j]) - dlt) * p.scale;
        }
        if (j + 1 < nvis) {
          p1 = bwd_exp2(fmaf(__uint_as_float(sx[j + 1]), p.scale_log2, -lse2));
          d1 = p1 * (__uint_as_float(dx[j + 1]) - dlt) * p.scale;
        }
        pp[j >> 1] = pack_bf16x2(p0, p1);
        pd[j >> 1] = pack_bf16x2(d0, d1);
      }
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint32_t off = (split >> 1) * kHalf + sw128_offset(r, (split & 1) * 4 + q4);
        *reinterpret_cast<uint4*>(p_base + off) = make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2], pp[4 * q4 + 3]);
        *reinterpret_cast<uint4*>(ds_base + off) = make_uint4(pd[4 * q4], pd[4 * q4 + 1], pd[4 * q4 + 2], pd[4 * q4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(BAR(PDS_FULL));
    }
    if (mbar_wait(BAR(ACC_FULL), 0, abort_flag, p.status, 317)) {
      tc_fence_after();
      // thread (r, split) owns key r of the block and head dims [32 split, 32 split + 32)
      __nv_bfloat16* dk = p.dK + static_cast<long long>(t.kv_row + r) * p.lddkv + t.kv_col0 + split * 32;
      __nv_bfloat16* dv = p.dV + static_cast<long long>(t.kv_row + r) * p.lddkv + t.kv_col0 + split * 32;
      uint32_t xk[32], xv[32];
      if (n_iter > 0) {
        tmem_ld32(tmem_base + lane_off + TM_DK + split * 32, xk);
        tmem_ld32(tmem_base + lane_off + TM_DV + split * 32, xv);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) { xk[j] = 0u; xv[j] = 0u; }
      }
      if (r < t.n_keys) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 a, b;
          a.x = pack_bf16x2(__uint_as_float(xk[j]), __uint_as_float(xk[j + 1]));
          a.y = pack_bf16x2(__uint_as_float(xk[j + 2]), __uint_as_float(xk[j + 3]));
          a.z = pack_bf16x2(__uint_as_float(xk[j + 4]), __uint_as_float(xk[j + 5]));
          a.w = pack_bf16x2(__uint_as_float(xk[j + 6]), __uint_as_float(xk[j + 7]));
          b.x = pack_bf16x2(__uint_as_float(xv[j]), __uint_as_float(xv[j + 1]));
          b.y = pack_bf16x2(__uint_as_float(xv[j + 2]), __uint_as_float(xv[j + 3]));
          b.z = pack_bf16x2(__uint_as_float(xv[j + 4]), __uint_as_float(xv[j + 5]));
          b.w = pack_bf16x2(__uint_as_float(xv[j + 6]), __uint_as_float(xv[j + 7]));
          *reinterpret_cast<uint4*>(dk + j) = a;
          *reinterpret_cast<uint4*>(dv + j) = b;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename K>
static int set_smem_attr(K kfn, int bytes, bool* flags) {
  int dev = 0;
  RLK_CHECK_CUDA(cudaGetDevice(&dev));
  if (!flags[dev & 63]) {
    RLK_CHECK_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    flags[dev & 63] = true;
  }
  return RLK_OK;
}

}  // namespace rlk
using namespace rlk;

// delta[t * Hq + h] = sum_d O[t,h,d] * dO[t,h,d]
RLK_API int rlk_attn_bwd_delta(const void* O, long long ldo, const void* dO, long long lddo,
                               float* delta, int T, int Hq, void* stream) {
  RLK_REQUIRE(T > 0 && Hq > 0, "attn_bwd_delta: empty");
  const long long warps = static_cast<long long>(T) * Hq;
  attn_bwd_delta_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)O, ldo, (const __nv_bfloat16*)dO, lddo, delta, T, Hq);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// Geometry as in rlk_attn_fwd; lse and delta use the forward's lse indexing.  n_src in 2..8
// (context parallel): k_ptrs[s] / v_ptrs[s] is rank s's K / V buffer mapped into this process,
// cp_blocks_per_chunk / cp_zigzag describe the layout (rlk::CpLayout).
RLK_API int rlk_attn_bwd_dq(const void* Q, const void* dO, long long q_rows, long long q_cols,
                            long long ldq, long long lddo, const void* const* k_ptrs,
                            const void* const* v_ptrs, int n_src, long long kv_rows, long long kv_cols,
                            long long ldkv, const float* lse, const float* delta, void* dQ,
                            long long lddq, const void* tiles, int n_tiles, float scale,
                            int cp_blocks_per_chunk, int cp_zigzag, void* stage_k, void* stage_v,
                            int* stage_flags, int stage_rows, int cp_rank, void* stream) {
  RLK_REQUIRE(n_tiles > 0, "attn_bwd_dq: no tiles");
  RLK_REQUIRE(n_src == 1 || (n_src >= 2 && n_src <= 8), "attn_bwd_dq: n_src must be 1..8");
  RLK_REQUIRE(n_src == 1 || cp_blocks_per_chunk > 0, "attn_bwd_dq: cp_blocks_per_chunk must be positive");
  CUtensorMap tmQ, tmDO;
  int rc;
  if ((rc = make_tmap_2d_sw128(&tmQ, Q, q_rows, q_cols, ldq, 128, 64, 2))) return rc;
  if ((rc = make_tmap_2d_sw128(&tmDO, dO, q_rows, q_cols, lddo, 128, 64, 2))) return rc;
  AttnDqParams p{};
  p.tiles = static_cast<const AttnTile*>(tiles);
  p.n_tiles = n_tiles;
  p.lse = lse;
  p.delta = delta;
  p.dQ = static_cast<__nv_bfloat16*>(dQ);
  p.lddq = lddq;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.cp = CpLayout{n_src > 1 ? n_src : 1, cp_blocks_per_chunk, cp_zigzag};
  p.status = device_status_word();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_src == 1) {
    KvMaps<1> kv;
    if ((rc = make_tmap_2d_sw128(&kv.k[0], k_ptrs[0], kv_rows, kv_cols, ldkv, 128, 64, 2))) return rc;
    if ((rc = make_tmap_2d_sw128(&kv.v[0], v_ptrs[0], kv_rows, kv_cols, ldkv, 128, 64, 2))) return rc;
    static bool flags[64] = {false};
    if ((rc = set_smem_attr(attn_bwd_dq_kernel<1>, DqSmem::kBytes, flags))) return rc;
    attn_bwd_dq_kernel<1><<<n_tiles, kBwdThreads, DqSmem::kBytes, st>>>(tmQ, tmDO, kv, kv, p);
  } else {
    KvMaps<8> kv;
    for (int i = 0; i < 8; ++i) {
      const int j = i < n_src ? i : 0;
      if ((rc = make_tmap_2d_sw128(&kv.k[i], k_ptrs[j], kv_rows, kv_cols, ldkv, 128, 64, 2))) return rc;
      if ((rc = make_tmap_2d_sw128(&kv.v[i], v_ptrs[j], kv_rows, kv_cols, ldkv, 128, 64, 2))) return rc;
    }
    KvMaps<1> staged;
    staged.k[0] = kv.k[0];
    staged.v[0] = kv.v[0];
    if (stage_rows > 0) {
      RLK_REQUIRE(stage_k && stage_v && stage_flags && stage_rows % 128 == 0 && stage_rows <= kv_rows &&
                  ldkv == kv_cols && cp_rank >= 0 && cp_rank < n_src, "attn_bwd_dq: bad staging arguments");
      CpStage& sg = p.stage;
      for (int i = 0; i < 8; ++i) {
        sg.src_a[i] = static_cast<const unsigned char*>(k_ptrs[i < n_src ? i : 0]);
        sg.src_b[i] = static_cast<const unsigned char*>(v_ptrs[i < n_src ? i : 0]);
      }
      sg.dst_a = static_cast<unsigned char*>(stage_k);
      sg.dst_b = static_cast<unsigned char*>(stage_v);
      sg.flags = stage_flags;
      sg.rows = stage_rows;
      sg.row_bytes_a = sg.row_bytes_b = static_cast<int>(kv_cols * 2);
      sg.ranks = n_src;
      sg.rank = cp_rank;
      const long long total = static_cast<long long>(n_src) * stage_rows;
      if ((rc = make_tmap_2d_sw128(&staged.k[0], stage_k, total, kv_cols, kv_cols, 128, 64, 2))) return rc;
      if ((rc = make_tmap_2d_sw128(&staged.v[0], stage_v, total, kv_cols, kv_cols, 128, 64, 2))) return rc;
      RLK_CHECK_CUDA(cudaMemsetAsync(stage_flags, 0, sizeof(int) * (n_src * (stage_rows / 128) * 2 + 1), st));
    }
    static bool flags[64] = {false};
    if ((rc = set_smem_attr(attn_bwd_dq_kernel<8>, DqSmem::kBytes, flags))) return rc;
    attn_bwd_dq_kernel<8><<<n_tiles, kBwdThreads, DqSmem::kBytes, st>>>(tmQ, tmDO, kv, staged, p);
  }
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// `tiles` is a device array of rlk::AttnKvTile (12 ints each).  n_src in 2..8 (context parallel):
// q_ptrs / do_ptrs / lse_ptrs / delta_ptrs hold one pointer per rank (this rank's own at its own
// index), all with the same shape and pitch; the tiles give key positions in the whole sequence
// (key0), n_q = the whole sequence length and q_row0 / lse_off for the sequence's first LOCAL row.
RLK_API int rlk_attn_bwd_dkv(const void* const* q_ptrs, const void* const* do_ptrs, int n_src,
                             long long q_rows, long long q_cols, long long ldq, long long lddo,
                             const void* K, const void* V, long long kv_rows, long long kv_cols,
                             long long ldkv, const float* const* lse_ptrs,
                             const float* const* delta_ptrs, void* dK, void* dV, long long lddkv,
                             const void* tiles, int n_tiles, float scale, int cp_blocks_per_chunk,
                             int cp_zigzag, void* stage_q, void* stage_do, int* stage_flags,
                             int stage_rows, int cp_rank, void* stream) {
  RLK_REQUIRE(n_tiles > 0, "attn_bwd_dkv: no tiles");
  RLK_REQUIRE(n_src == 1 || (n_src >= 2 && n_src <= 8), "attn_bwd_dkv: n_src must be 1..8");
  RLK_REQUIRE(n_src == 1 || cp_blocks_per_chunk > 0, "attn_bwd_dkv: cp_blocks_per_chunk must be positive");
  CUtensorMap tmK, tmV;
  int rc;
  if ((rc = make_tmap_2d_sw128(&tmK, K, kv_rows, kv_cols, ldkv, 128, 64, 2))) return rc;
  if ((rc = make_tmap_2d_sw128(&tmV, V, kv_rows, kv_cols, ldkv, 128, 64, 2))) return rc;
  AttnDkvParams p{};
  p.tiles = static_cast<const AttnKvTile*>(tiles);
  p.n_tiles = n_tiles;
  for (int i = 0; i < 8; ++i) {
    const int j = i < n_src ? i : 0;
    p.lse[i] = lse_ptrs[j];
    p.delta[i] = delta_ptrs[j];
  }
  p.cp = CpLayout{n_src > 1 ? n_src : 1, cp_blocks_per_chunk, cp_zigzag};
  p.dK = static_cast<__nv_bfloat16*>(dK);
  p.dV = static_cast<__nv_bfloat16*>(dV);
  p.lddkv = lddkv;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.status = device_status_word();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_src == 1) {
    KvMaps<1> qdo;
    if ((rc = make_tmap_2d_sw128(&qdo.k[0], q_ptrs[0], q_rows, q_cols, ldq, 128, 64, 2))) return rc;
    if ((rc = make_tmap_2d_sw128(&qdo.v[0], do_ptrs[0], q_rows, q_cols, lddo, 128, 64, 2))) return rc;
    static bool flags[64] = {false};
    if ((rc = set_smem_attr(attn_bwd_dkv_kernel<1>, DkvSmem::kBytes, flags))) return rc;
    attn_bwd_dkv_kernel<1><<<n_tiles, kBwdThreads, DkvSmem::kBytes, st>>>(qdo, qdo, tmK, tmV, p);
  } else {
    KvMaps<8> qdo;
    for (int i = 0; i < 8; ++i) {
      const int j = i < n_src ? i : 0;
      if ((rc = make_tmap_2d_sw128(&qdo.k[i], q_ptrs[j], q_rows, q_cols, ldq, 128, 64, 2))) return rc;
      if ((rc = make_tmap_2d_sw128(&qdo.v[i], do_ptrs[j], q_rows, q_cols, lddo, 128, 64, 2))) return rc;
    }
    KvMaps<1> staged;
    staged.k[0] = qdo.k[0];
    staged.v[0] = qdo.v[0];
    if (stage_rows > 0) {
      RLK_REQUIRE(stage_q && stage_do && stage_flags && stage_rows % 128 == 0 && stage_rows <= q_rows &&
                  ldq == q_cols && lddo == q_cols && cp_rank >= 0 && cp_rank < n_src,
                  "attn_bwd_dkv: bad staging arguments");
      CpStage& sg = p.stage;
      for (int i = 0; i < 8; ++i) {
        sg.src_a[i] = static_cast<const unsigned char*>(q_ptrs[i < n_src ? i : 0]);
        sg.src_b[i] = static_cast<const unsigned char*>(do_ptrs[i < n_src ? i : 0]);
      }
      sg.dst_a = static_cast<unsigned char*>(stage_q);
      sg.dst_b = static_cast<unsigned char*>(stage_do);
      sg.flags = stage_flags;
      sg.rows = stage_rows;
      sg.row_bytes_a = sg.row_bytes_b = static_cast<int>(q_cols * 2);
      sg.ranks = n_src;
      sg.rank = cp_rank;
      const long long total = static_cast<long long>(n_src) * stage_rows;
      if ((rc = make_tmap_2d_sw128(&staged.k[0], stage_q, total, q_cols, q_cols, 128, 64, 2))) return rc;
      if ((rc = make_tmap_2d_sw128(&staged.v[0], stage_do, total, q_cols, q_cols, 128, 64, 2))) return rc;
      RLK_CHECK_CUDA(cudaMemsetAsync(stage_flags, 0, sizeof(int) * (n_src * (stage_rows / 128) * 2 + 1), st));
    }
    static bool flags[64] = {false};
    if ((rc = set_smem_attr(attn_bwd_dkv_kernel<8>, DkvSmem::kBytes, flags))) return rc;
    attn_bwd_dkv_kernel<8><<<n_tiles, kBwdThreads, DkvSmem::kBytes, st>>>(qdo, staged, tmK, tmV, p);
  }
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
