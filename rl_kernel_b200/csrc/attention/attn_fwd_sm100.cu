// Deterministic causal GQA attention forward for sm_100a (head_dim 128, bf16).
//
// One CTA per work tile (see rlk/attn_common.cuh): 128 query rows x one KV head's keys.
//   warp 0   : TMA producer  (Q once, then K and V blocks through 2-stage rings)
//   warp 1   : UMMA issuer   (S = Q K^T into TMEM, O_blk = P V into TMEM)
//   warps 2-17: softmax + accumulation, four threads per query row (each owns 32 of the 128 keys
//              of a block and 32 of the 128 output dims; only the block maximum and the final row
//              sum are exchanged, through shared memory).  A row's arithmetic never depends on
//              what else is in the tile.
// Keys are consumed in canonical 128-key blocks in ascending order with an online softmax;
// no split-KV, no atomics.  P is rounded to bf16 before P V (as every flash kernel does); the
// row sum uses the unrounded fp32 probabilities, added in a fixed order.
//
// With NSRC > 1 the K/V blocks of a tile live on several GPUs (context parallel): block b is
// read straight from its owner's memory with a plain (non-multicast) TMA load through that
// peer's tensor map, so the KV exchange happens inside the kernel and the per-row arithmetic
// is identical to the single-GPU run.
//
// Replaces the external FA4 call (rl_engine/backends/cuda/attention/flash_attn.py:343-353), the
// materialising kernels in csrc/cuda/attention/deterministic_attention.cu and the AG -> full
// attention -> scatter scheme of rl_engine/backends/cuda/attention/cp_comm.py:444-566.
#include "rlk/attn_common.cuh"
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

constexpr int kAttnThreads = 576;  // TMA warp, UMMA warp, 16 softmax warps
constexpr int kSplit = 4;           // threads (column slices) per query row
constexpr int kTileBytes = 128 * 128 * 2;  // one 128x128 bf16 operand tile (two 64-wide boxes)
constexpr int kHalfBytes = 128 * 64 * 2;

struct AttnFwdParams {
  const AttnTile* tiles;
  int n_tiles;
  __nv_bfloat16* O;
  long long ldo;      // elements between consecutive rows of O
  float* lse;         // may be null
  float scale_log2;   // softmax scale * log2(e)
  float scale;        // softmax scale
  int cp_blocks_per_chunk;  // NSRC > 1: 128-key blocks per contiguous chunk of the sequence
  int cp_ranks;             // NSRC > 1: number of ranks holding the sequence
  int cp_zigzag;            // NSRC > 1: 1 = rank c holds chunks c and 2*cp-1-c; 0 = chunk c on rank c
  int q_rows_box;           // 128 (training / prefill) or 8 (decode: at most 8 query rows per tile)
  const int* page_table;    // paged KV cache: see cp_locate; null = contiguous KV
  CpStage stage;            // context parallel: remote K/V blocks are copied here once (rows = 0: off)
  // Resumable rows (shared-prefix decode).  tile_ext[4 * tile] = {first block, mode, state row, 0}:
  // mode 1 tiles stop after their last block and write every row's running (max, partial sums,
  // unnormalised output) to `state` instead of O; mode 2 tiles start at `first block` from that
  // state.  A row's program is the same sequence of block updates either way, so the bits equal
  // an uninterrupted run.  State row of tile row r: state_row + (r / q_rows_per_seq) * q_seq_rows
  // + r % q_rows_per_seq, kAttnStateFloats floats each.
  const int* tile_ext;
  float* state;
  int q_rows_per_seq;       // rows of one sequence inside a tile (the GQA group size)
  int q_seq_rows;           // rows between consecutive sequences in Q (query heads per sequence)
  int q3d;                  // 1: Q comes through a 3-D map {128, q_seq_rows, sequences}: a tile's rows are
                            //    q_rows_per_seq rows of each of q_rows_box / q_rows_per_seq consecutive sequences
  int* status;
};

constexpr int kAttnStateFloats = 136;   // per row: max, 3 unused, 4 partial sums, 128 outputs

// Shared memory: [Q (| Q) | P | K ring | V ring | barriers | exchange].  Full tiles: Q and P are
// 32 KB each and the rings have 2 stages.  Decode tiles (<= 32 query rows): two Q buffers and P of
// at most 8 KB each -- the UMMA still reads 128 "rows" from those addresses, the ones past the
// tile's rows are whatever follows in shared memory and only feed accumulator rows nobody reads --
// and the freed space makes the rings 3 stages deep, which keeps enough K/V bytes in flight to
// stream the cache at memory speed.
template <bool DEC>
struct AttnFwdSmem {
  static constexpr int kBars = 6 * kTileBytes + (DEC ? 24576 : 0);
  static constexpr int kXch = kBars + 256;             // row-wise exchange of partial maxima / sums
  static constexpr int kBytes = kXch + 8192 + 1024;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Which tensor map and which local row holds canonical block b of a sequence.
// Paged KV (tile.reserved = 1 + index of the sequence's first entry in page_table): canonical block
// b of the sequence lives in page (entry & 0xffffff) -- 128 rows starting at row 128 * page -- of
// the K/V buffer of rank (entry >> 24), so a sequence's pages may sit anywhere and, with several
// source maps, on other GPUs (prefill / decode context parallelism over a distributed page pool).
__device__ __forceinline__ void cp_locate(const AttnFwdParams& p, const AttnTile& t, int b,
                                          int& src, int& row) {
  if (p.page_table != nullptr && t.reserved > 0) {
    const int e = p.page_table[t.reserved - 1 + b];
    src = e >> 24;
    row = (e & 0xffffff) * kAttnBlock;
    return;
  }
  if (p.cp_ranks <= 1) {
    src = t.kv_src;
    row = t.kv_row0 + b * kAttnBlock;
    return;
  }
  int lb;
  cp_locate_block(CpLayout{p.cp_ranks, p.cp_blocks_per_chunk, p.cp_zigzag}, b, src, lb);
  row = t.kv_row0 + lb * kAttnBlock;
}

// DEC: decode tiles (at most 32 query rows; small Q / P buffers, three-stage rings, persistent CTAs
// that walk several tiles, resumable rows).  Full tiles compile without any of that, which keeps
// the softmax loop's registers where they were.
template <int NSRC, bool DEC>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ KvMaps<NSRC> kv,
                const __grid_constant__ KvMaps<1> staged, const AttnFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttnFwdSmem<DEC>::kBars);
  // barrier indices
  enum { Q_FULL = 0, Q_EMPTY = 2, K_FULL = 4, K_EMPTY = 7, V_FULL = 10, V_EMPTY = 13, S_FULL = 16, S_EMPTY = 18,
         P_FULL = 20, O_FULL = 21, XCH = 22, ST_FULL = 26, ST_EMPTY = 28, NBARS = 30 };
  constexpr bool decode = DEC;
  constexpr int nstage = decode ? 3 : 2;
  const uint32_t q_half = static_cast<uint32_t>(p.q_rows_box) * 128u;  // bytes of one 64-column half of Q / P
  const uint32_t off_p = (decode ? 4 : 2) * q_half;   // decode: two Q buffers, then P
  const uint32_t off_k = off_p + 2 * q_half;
  const uint32_t off_v = off_k + nstage * kTileBytes;
  constexpr int n_active = (decode ? 32 : 128) * kSplit;  // softmax threads that take part
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* stage_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Decode: barriers and tensor memory are set up before the dependency wait, so this part
  // overlaps the tail of the previous kernel of the stream; nothing before the wait touches global
  // memory.  Full tiles wait first and fetch their one tile descriptor right away, so that its
  // latency hides behind the set-up instead.
  AttnTile tile0{};
  if (!DEC) {
    griddep_sync();
    tile0 = p.tiles[blockIdx.x];
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(BAR(Q_FULL + s), 1);
      mbar_init(BAR(Q_EMPTY + s), 1);
    }
    for (int s = 0; s < 3; ++s) {
      mbar_init(BAR(K_FULL + s), 1);
      mbar_init(BAR(K_EMPTY + s), 1);
      mbar_init(BAR(V_FULL + s), 1);
      mbar_init(BAR(V_EMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(BAR(S_FULL + s), 1);
      mbar_init(BAR(S_EMPTY + s), n_active);
    }
    mbar_init(BAR(P_FULL), n_active);
    for (int q = 0; q < 4; ++q) mbar_init(BAR(XCH + q), 32 * kSplit);
    for (int s = 0; s < 2; ++s) {
      mbar_init(BAR(ST_FULL + s), 1);
      mbar_init(BAR(ST_EMPTY + s), n_active);
    }
    mbar_init(BAR(O_FULL), 1);
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
  if (DEC) griddep_sync();

  // A CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  (decode launches are persistent: one
  // CTA per SM; the loads of the next tile start while the current one is still in its softmax
  // and epilogue, which hides the per-tile start-up).  Barrier phases therefore follow running
  // counters -- blocks, S buffers, tiles -- that every role advances in the same way.
  const bool use_stage = NSRC > 1 && p.stage.rows > 0;
  constexpr int nq = decode ? 2 : 1;             // Q buffers (decode tiles are small enough for two)
  // full tiles: exactly one tile per CTA (the loops below then run once and fold away)
  const int tile_step = decode ? static_cast<int>(gridDim.x) : 0x40000000;
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sP = sQ + off_p;
  const uint32_t sK = sQ + off_k;
  const uint32_t sV = sQ + off_v;
  constexpr uint32_t TM_S = 0;     // two S buffers: columns [0,128) and [128,256)
  constexpr uint32_t TM_O = 256;   // O_blk: columns [256,384)

  struct TileInfo { AttnTile t; int nblk, b0, st_mode, st_row; bool st_smem; };
  // Resuming tiles whose rows are consecutive in the state array get their saved state copied into
  // shared memory by the producer (two slots in the space between the V ring and the barriers, free
  // when the tiles have few rows), so its latency is off the softmax warps' path.
  const uint32_t sp_off = off_v + nstage * kTileBytes;
  const int sp_room = decode ? (24576 - 6 * static_cast<int>(q_half)) / 2 : 0;     // bytes per slot
  auto read_tile = [&](int idx) {
    TileInfo ti;
    ti.t = DEC ? p.tiles[idx] : tile0;
    int max_kv = ti.t.pos0 + (ti.t.n_rows - 1) * ti.t.pos_step + 1;
    if (max_kv > ti.t.kv_cap) max_kv = ti.t.kv_cap;
    ti.nblk = ti.t.n_rows > 0 ? (max_kv + kAttnBlock - 1) / kAttnBlock : 0;
    // blocks [b0, nblk) are processed
    ti.b0 = 0; ti.st_mode = 0; ti.st_row = 0;
    if (decode && p.tile_ext != nullptr) {
      ti.b0 = p.tile_ext[4 * idx];
      ti.st_mode = p.tile_ext[4 * idx + 1];
      ti.st_row = p.tile_ext[4 * idx + 2];
      if (ti.b0 > ti.nblk) ti.b0 = ti.nblk;
    }
    ti.st_smem = decode && ti.st_mode == 2 && p.q_rows_per_seq > 0 && ti.t.n_rows <= p.q_rows_per_seq &&
                 ti.t.n_rows * kAttnStateFloats * 4 <= sp_room;
    return ti;
  };

  // The producer and MMA warps walk their loops with all 32 lanes (the loop state is warp-uniform
  // and stays in uniform registers, where the TMA / MMA / barrier instructions take their operands
  // from); one elected lane issues.  Waits are warp votes, so a timeout leaves no lane behind.
  if (warp == 0) {
    {
      uint32_t kc = 0, tc = 0;       // blocks and tiles issued so far
      uint32_t stc = 0;              // saved-state copies issued so far
      bool ok = true;
      for (int idx = blockIdx.x; ok && idx < p.n_tiles; idx += tile_step) {
        const TileInfo ti = read_tile(idx);
        const AttnTile& t = ti.t;
        if (t.n_rows <= 0) continue;
        const uint32_t qs = tc % nq, qph = (tc / nq) & 1;
        ++tc;
        if (!mbar_wait_warp(BAR(Q_EMPTY + qs), qph ^ 1, abort_flag, p.status, 213)) break;
        const uint32_t q_dst = sQ + qs * 2 * q_half;
        if (elect_one()) {
          mbar_expect_tx(BAR(Q_FULL + qs), 2 * q_half);
          if (p.q3d) {
            const int y = t.q_row0 % p.q_seq_rows, z = t.q_row0 / p.q_seq_rows;
            tma_load_3d(q_dst, &tmQ, t.q_col0, y, z, BAR(Q_FULL + qs));
            tma_load_3d(q_dst + q_half, &tmQ, t.q_col0 + 64, y, z, BAR(Q_FULL + qs));
          } else {
            tma_load_2d(q_dst, &tmQ, t.q_col0, t.q_row0, BAR(Q_FULL + qs));
            tma_load_2d(q_dst + q_half, &tmQ, t.q_col0 + 64, t.q_row0, BAR(Q_FULL + qs));
          }
        }
        if (ti.st_smem) {
          const uint32_t ss = stc & 1, sph = (stc >> 1) & 1;
          ++stc;
          if (!mbar_wait_warp(BAR(ST_EMPTY + ss), sph ^ 1, abort_flag, p.status, 214)) break;
          const uint32_t nbytes = static_cast<uint32_t>(t.n_rows) * kAttnStateFloats * 4;
          if (elect_one()) {
            mbar_expect_tx(BAR(ST_FULL + ss), nbytes);
            bulk_load_1d(sQ + sp_off + ss * sp_room, p.state + static_cast<long long>(ti.st_row) * kAttnStateFloats,
                         nbytes, BAR(ST_FULL + ss));
          }
        }
        for (int b = ti.b0; b < ti.nblk; ++b, ++kc) {
          const int s = kc % nstage;
          const uint32_t ph = (kc / nstage) & 1;
          int src, row;
          cp_locate(p, t, b, src, row);
          if (NSRC == 1) src = 0;
          const CUtensorMap* mk = &kv.k[src];
          const CUtensorMap* mv = &kv.v[src];
          if (use_stage && src != p.stage.rank) {
            // remote block: read the local copy once it has landed
            if (!__all_sync(0xffffffffu, cp_stage_wait(p.stage, src, row / kAttnBlock, abort_flag, p.status, 212))) { ok = false; break; }
            row += src * p.stage.rows;
            mk = &staged.k[0];
            mv = &staged.v[0];
          }
          if (!mbar_wait_warp(BAR(K_EMPTY + s), ph ^ 1, abort_flag, p.status, 201)) { ok = false; break; }
          if (elect_one()) {
            mbar_expect_tx(BAR(K_FULL + s), kTileBytes);
            tma_load_2d(sK + s * kTileBytes, mk, t.kv_col0, row, BAR(K_FULL + s));
            tma_load_2d(sK + s * kTileBytes + kHalfBytes, mk, t.kv_col0 + 64, row, BAR(K_FULL + s));
          }
          if (!mbar_wait_warp(BAR(V_EMPTY + s), ph ^ 1, abort_flag, p.status, 202)) { ok = false; break; }
          if (elect_one()) {
            mbar_expect_tx(BAR(V_FULL + s), kTileBytes);
            tma_load_2d(sV + s * kTileBytes, mv, t.kv_col0, row, BAR(V_FULL + s));
            tma_load_2d(sV + s * kTileBytes + kHalfBytes, mv, t.kv_col0 + 64, row, BAR(V_FULL + s));
          }
        }
      }
    }
  } else if (warp == 1) {
    {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);  // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, 128, 0, 1);  // P (K-major) x V (MN-major)
      uint32_t sc = 0;        // S products issued so far (K ring slot, S buffer)
      uint32_t pc = 0;        // P*V products issued so far (V ring slot, P / O phases)
      uint32_t tc = 0;
      uint32_t q_cur = sQ;
      auto issue_s = [&]() -> bool {
        const int s = sc % nstage;              // K/V ring slot
        const uint32_t ph = (sc / nstage) & 1;
        const int sb = sc & 1;                  // S accumulator buffer
        const uint32_t phs = (sc >> 1) & 1;
        ++sc;
        if (!mbar_wait_warp(BAR(K_FULL + s), ph, abort_flag, p.status, 203)) return false;
        if (!mbar_wait_warp(BAR(S_EMPTY + sb), phs ^ 1, abort_flag, p.status, 204)) return false;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t offq = (k >> 2) * q_half + (k & 3) * 32;
            const uint32_t offk = (k >> 2) * kHalfBytes + (k & 3) * 32;
            umma_bf16_ss(tmem_base + TM_S + sb * 128, umma_desc_sw128(q_cur + offq, 16, 1024),
                         umma_desc_sw128(sK + s * kTileBytes + offk, 16, 1024), idesc_s, k != 0);
          }
          umma_commit(BAR(S_FULL + sb));
          umma_commit(BAR(K_EMPTY + s));
        }
        return true;
      };
      bool ok = true;
      for (int idx = blockIdx.x; ok && idx < p.n_tiles; idx += tile_step) {
        const TileInfo ti = read_tile(idx);
        if (ti.t.n_rows <= 0) continue;
        const int nb = ti.nblk - ti.b0;
        const uint32_t qs = tc % nq, qph = (tc / nq) & 1;
        ++tc;
        q_cur = sQ + qs * 2 * q_half;
        ok = mbar_wait_warp(BAR(Q_FULL + qs), qph, abort_flag, p.status, 205);
        if (ok && nb > 0) ok = issue_s();
        for (int b = 0; ok && b < nb; ++b) {
          if (b + 1 < nb) ok = issue_s();
          if (!ok) break;
          if (b + 1 >= nb && elect_one()) umma_commit(BAR(Q_EMPTY + qs));   // every S product of this tile has been issued
          const int s = pc % nstage;
          const uint32_t ph = (pc / nstage) & 1;
          const uint32_t pph = pc & 1;
          ++pc;
          if (!mbar_wait_warp(BAR(V_FULL + s), ph, abort_flag, p.status, 206)) { ok = false; break; }
          if (!mbar_wait_warp(BAR(P_FULL), pph, abort_flag, p.status, 207)) { ok = false; break; }
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint32_t aoff = (k >> 2) * q_half + (k & 3) * 32;
              umma_bf16_ss(tmem_base + TM_O, umma_desc_sw128(sP + aoff, 16, 1024),
                           umma_desc_sw128(sV + s * kTileBytes + k * 2048, kHalfBytes, 1024), idesc_o,
                           k != 0);
            }
            umma_commit(BAR(O_FULL));
            umma_commit(BAR(V_EMPTY + s));
          }
        }
        if (ok && nb <= 0 && elect_one()) umma_commit(BAR(Q_EMPTY + qs));
      }
    }
  } else if (!decode || (warp & 3) == 0) {
    // ---------------------------------------------------------------- softmax / accumulate
    // Sixteen warps: warp -> (quad, split).  quad = warp % 4 is the TMEM lane quadrant the hardware
    // lets the warp touch, split = (warp - 2) / 4 selects which 32 of the 128 S columns (keys) and
    // which 32 of the 128 O columns (head dims) the thread owns.  The four threads of a row
    // exchange their partial maxima through shared memory; everything else is private.
    // (decode tiles have at most 32 rows: only the quad-0 warps take part)
    const int quad = warp & 3;
    const int split = (warp - 2) >> 2;
    const int r = quad * 32 + lane;  // this thread's query row within the tile
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    uint8_t* p_row = smem + off_p;
    float* xch = reinterpret_cast<float*>(smem + AttnFwdSmem<DEC>::kXch);  // [2][128][4] maxima, then [2][128][4] sums
    uint32_t bc = 0;     // blocks done so far (S buffer, P / O phases, maxima slot)
    uint32_t xc = 0;     // exchange rounds done so far (one per block, one per tile)
    uint32_t stc = 0;    // saved-state copies consumed so far
    bool alive = true;
    // context parallel with staging: the compute warps first help copy the remote K/V blocks
    // (the CTAs that start first do all of it; later ones find the work counter exhausted);
    // a CTA whose tile is empty helps too -- its threads do nothing else
    if (use_stage && !decode) cp_stage_gather(p.stage, threadIdx.x - 64, kAttnThreads - 64, 3, stage_slot);

    for (int idx = blockIdx.x; alive && idx < p.n_tiles; idx += tile_step) {
      const TileInfo ti = read_tile(idx);
      const AttnTile& t = ti.t;
      if (t.n_rows <= 0) continue;
      const int nb = ti.nblk - ti.b0;
      int kv_len = t.pos0 + r * t.pos_step + 1;
      if (kv_len > t.kv_cap) kv_len = t.kv_cap;
      if (r >= t.n_rows) kv_len = 0;
      float m_run = -INFINITY, l_part = 0.f;
      float o[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = 0.f;
      float* st_ptr = nullptr;     // this row's saved state (resumable rows)
      if (ti.st_smem) {
        const uint32_t ss = stc & 1, sph = (stc >> 1) & 1;
        ++stc;
        if (!mbar_wait(BAR(ST_FULL + ss), sph, abort_flag, p.status, 215)) { alive = false; break; }
        if (r < t.n_rows) {
          const float* sp = reinterpret_cast<const float*>(smem + sp_off + ss * sp_room) + r * kAttnStateFloats;
          m_run = sp[0];
          l_part = sp[4 + split];
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 v = *reinterpret_cast<const float4*>(sp + 8 + split * 32 + j);
            o[j] = v.x; o[j + 1] = v.y; o[j + 2] = v.z; o[j + 3] = v.w;
          }
        }
        mbar_arrive(BAR(ST_EMPTY + ss));
      } else if (ti.st_mode != 0 && r < t.n_rows) {
        const int rps = p.q_rows_per_seq > 0 ? p.q_rows_per_seq : 1;
        st_ptr = p.state + static_cast<long long>(ti.st_row + (r / rps) * p.q_seq_rows + r % rps) * kAttnStateFloats;
        if (ti.st_mode == 2) {
          m_run = st_ptr[0];
          l_part = st_ptr[4 + split];
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 v = *reinterpret_cast<const float4*>(st_ptr + 8 + split * 32 + j);
            o[j] = v.x; o[j + 1] = v.y; o[j + 2] = v.z; o[j + 3] = v.w;
          }
        }
      }
      float alpha_prev = 0.f;

      for (int b = 0; b < nb; ++b, ++bc, ++xc) {    // b counts from the tile's first block b0
        const int s = bc & 1;
        const uint32_t ph = (bc >> 1) & 1;
        if (!mbar_wait(BAR(S_FULL + s), ph, abort_flag, p.status, 208)) { alive = false; break; }
        tc_fence_after();
        const int nvis = kv_len - (ti.b0 + b) * kAttnBlock - split * 32;  // visible keys among this thread's 32
        uint32_t x[32];
        tmem_ld32(tmem_base + lane_off + TM_S + s * 128 + split * 32, x);
        tmem_ld_wait();
        float m_part = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < nvis) m_part = fmaxf(m_part, __uint_as_float(x[j]));
        xch[(xc & 1) * 512 + r * 4 + split] = m_part;
        mbar_arrive(BAR(XCH + quad));
        if (!mbar_wait(BAR(XCH + quad), xc & 1, abort_flag, p.status, 210)) { alive = false; break; }
        const float4 mm = *reinterpret_cast<const float4*>(xch + (xc & 1) * 512 + r * 4);
        const float m_blk = fmaxf(fmaxf(mm.x, mm.y), fmaxf(mm.z, mm.w));
        const float m_new = fmaxf(m_run, m_blk);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = fast_exp2((m_run - m_use) * p.scale_log2);  // m_run = -inf -> 0
        const float neg_ms = -m_use * p.scale_log2;
        float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float e0 = (j + 0 < nvis) ? fast_exp2(fmaf(__uint_as_float(x[j + 0]), p.scale_log2, neg_ms)) : 0.f;
          const float e1 = (j + 1 < nvis) ? fast_exp2(fmaf(__uint_as_float(x[j + 1]), p.scale_log2, neg_ms)) : 0.f;
          const float e2 = (j + 2 < nvis) ? fast_exp2(fmaf(__uint_as_float(x[j + 2]), p.scale_log2, neg_ms)) : 0.f;
          const float e3 = (j + 3 < nvis) ? fast_exp2(fmaf(__uint_as_float(x[j + 3]), p.scale_log2, neg_ms)) : 0.f;
          sum0 += e0; sum1 += e1; sum2 += e2; sum3 += e3;
          pk[j / 2] = pack_bf16x2(e0, e1);
          pk[j / 2 + 1] = pack_bf16x2(e2, e3);
        }
        // The previous block's P*V product is collected only now, after this block's exponentials
        // are already in registers: the MMA of block b-1 runs while block b's scores are reduced.
        // (It must be collected before P is overwritten and before the next P*V reuses the O columns.)
        if (b > 0) {
          if (!mbar_wait(BAR(O_FULL), (bc - 1) & 1, abort_flag, p.status, 209)) { alive = false; break; }
          tc_fence_after();
          uint32_t xo[32];
          tmem_ld32(tmem_base + lane_off + TM_O + split * 32, xo);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = fmaf(o[j], alpha_prev, __uint_as_float(xo[j]));
        }
        // this thread's 32 keys = 4 chunks of 16 bytes; keys [64h, 64h+64) live in half h of the P tile
        if (r < p.q_rows_box) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            *reinterpret_cast<uint4*>(p_row + (split >> 1) * q_half + sw128_offset(r, (split & 1) * 4 + q4)) =
                make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
        }
        fence_proxy_async_smem();  // make the generic-proxy P writes visible to the UMMA
        tc_fence_before();
        mbar_arrive(BAR(S_EMPTY + s));
        mbar_arrive(BAR(P_FULL));
        l_part = l_part * alpha + ((sum0 + sum1) + (sum2 + sum3));
        m_run = m_new;
        alpha_prev = alpha;
      }
      if (!alive) break;
      if (nb > 0) {
        if (mbar_wait(BAR(O_FULL), (bc - 1) & 1, abort_flag, p.status, 209)) {
          tc_fence_after();
          uint32_t xo[32];
          tmem_ld32(tmem_base + lane_off + TM_O + split * 32, xo);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = fmaf(o[j], alpha_prev, __uint_as_float(xo[j]));
        } else {
          alive = false;
          break;
        }
      }
      // ---------------------------------------------------------------- epilogue
      // row sum = (l0 + l1) + (l2 + l3) over the four column slices
      float* lx = xch + 1024 + (xc & 1) * 512;   // two slots: a row's threads may be one round apart
      lx[r * 4 + split] = l_part;
      mbar_arrive(BAR(XCH + quad));
      const bool synced = mbar_wait(BAR(XCH + quad), xc & 1, abort_flag, p.status, 211);
      ++xc;
      if (!synced) { alive = false; break; }
      if (ti.st_mode == 1) {
        // resumable rows: hand the running state on instead of normalising
        if (st_ptr != nullptr) {
          if (split == 0) st_ptr[0] = m_run;
          st_ptr[4 + split] = l_part;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(st_ptr + 8 + split * 32 + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
        }
      } else if (r < t.n_rows) {
        const float4 ll = *reinterpret_cast<const float4*>(lx + r * 4);
        const float l_run = (ll.x + ll.y) + (ll.z + ll.w);
        const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* dst = p.O + static_cast<long long>(t.q_row0 + r) * p.ldo + t.q_col0 + split * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 v;
          v.x = pack_bf16x2(o[j] * inv_l, o[j + 1] * inv_l);
          v.y = pack_bf16x2(o[j + 2] * inv_l, o[j + 3] * inv_l);
          v.z = pack_bf16x2(o[j + 4] * inv_l, o[j + 5] * inv_l);
          v.w = pack_bf16x2(o[j + 6] * inv_l, o[j + 7] * inv_l);
          *reinterpret_cast<uint4*>(dst + j) = v;
        }
        if (p.lse && split == 0) {
          const float lse = (l_run > 0.f) ? fmaf(m_run, p.scale, logf(l_run)) : -INFINITY;
          p.lse[t.lse_off + static_cast<long long>(r) * t.lse_stride] = lse;
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

template <int NSRC, bool DEC>
static int launch_attn_fwd(const CUtensorMap& tmQ, const KvMaps<NSRC>& kv, const KvMaps<1>& staged,
                           const AttnFwdParams& p, cudaStream_t stream) {
  auto kfn = attn_fwd_kernel<NSRC, DEC>;
  static bool attr_set[64] = {false};
  int dev = 0;
  RLK_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    RLK_CHECK_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        AttnFwdSmem<DEC>::kBytes));
    attr_set[dev & 63] = true;
  }
  // decode tiles are short and alike: one persistent CTA per SM walks them, so that a tile's loads
  // overlap the previous tile's tail; full tiles keep one CTA each (the hardware hands them out as
  // CTAs finish, which balances causal tiles of different lengths)
  const int grid = (DEC && p.n_tiles > sm_count()) ? sm_count() : p.n_tiles;
  RLK_CHECK_CUDA(launch_pdl(kfn, dim3(grid), dim3(kAttnThreads), AttnFwdSmem<DEC>::kBytes, stream, tmQ, kv, staged, p));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

}  // namespace rlk

// Q: [q_rows, q_cols] bf16 row-major with pitch ldq; K and V: [kv_rows, kv_cols] with pitch ldkv.
// `tiles` is a device array of n_tiles rlk::AttnTile.  O has Q's geometry with pitch ldo.
// decode_rows != 0 promises that every tile has n_rows <= 8 (single-token decode with GQA packing)
// and selects the small-Q layout; the per-row arithmetic is unchanged.
// page_table (device int32, may be null): tiles with reserved > 0 read their KV blocks through it
// (see cp_locate); entries must name source ranks < n_src.
// stage_rows > 0 (context parallel only): the first stage_rows rows of every peer's K / V are
// copied once into stage_k / stage_v ([n_src * stage_rows, kv_cols]) by the kernel itself and
// remote blocks are read from there; stage_flags holds n_src * stage_rows / 128 * 2 + 1 ints.
// n_src == 1: k_ptrs/v_ptrs hold one pointer each.  n_src in 2..8 (context parallel): pointer s
// is rank s's K / V buffer (same shape and pitch on every rank), mapped into this process.
RLK_API int rlk_attn_fwd(const void* Q, long long q_rows, long long q_cols, long long ldq,
                         const void* const* k_ptrs, const void* const* v_ptrs, int n_src,
                         long long kv_rows, long long kv_cols, long long ldkv, void* O,
                         long long ldo, float* lse, const void* tiles, int n_tiles, float scale,
                         int cp_blocks_per_chunk, int cp_zigzag, int decode_rows,
                         const int* page_table, void* stage_k, void* stage_v, int* stage_flags,
                         int stage_rows, int cp_rank, const int* tile_ext, float* state,
                         int q_rows_per_seq, int q_seq_rows, int q_group, void* stream) {
  using namespace rlk;
  RLK_REQUIRE(n_tiles > 0, "attn_fwd: no tiles");
  RLK_REQUIRE(n_src == 1 || (n_src >= 2 && n_src <= 8), "attn_fwd: n_src must be 1..8");
  RLK_REQUIRE(q_cols % 128 == 0 && kv_cols % 128 == 0, "attn_fwd: head_dim must be 128");
  RLK_REQUIRE((reinterpret_cast<uintptr_t>(O) & 15) == 0 && (ldo * 2) % 16 == 0,
              "attn_fwd: O must be 16-byte aligned");
  AttnFwdParams p{};
  p.tiles = static_cast<const AttnTile*>(tiles);
  p.n_tiles = n_tiles;
  p.O = static_cast<__nv_bfloat16*>(O);
  p.ldo = ldo;
  p.lse = lse;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.cp_blocks_per_chunk = cp_blocks_per_chunk;
  p.cp_ranks = n_src > 1 ? n_src : 1;
  p.cp_zigzag = cp_zigzag;
  p.status = device_status_word();
  p.page_table = page_table;
  p.q_rows_box = decode_rows ? 8 : 128;
  p.tile_ext = tile_ext;
  p.state = state;
  p.q_rows_per_seq = q_rows_per_seq;
  p.q_seq_rows = q_seq_rows;
  RLK_REQUIRE(tile_ext == nullptr || (decode_rows && state != nullptr && n_src == 1 && q_seq_rows > 0),
              "attn_fwd: resumable rows are decode tiles with a state buffer, one KV source and the row geometry");
  CUtensorMap tmQ;
  int rc;
  if (q_group > 0) {
    // a tile's rows: q_rows_per_seq rows of each of q_group consecutive sequences
    RLK_REQUIRE(decode_rows && q_rows_per_seq > 0 && q_seq_rows > 0 && q_rows_per_seq * q_group <= 32 &&
                    (q_rows_per_seq * q_group) % 8 == 0 && q_rows % q_seq_rows == 0 && q_cols == 128,
                "attn_fwd: grouped query tiles hold 8 to 32 rows of 128 columns");
    p.q_rows_box = q_rows_per_seq * q_group;
    p.q3d = 1;
    rc = make_tmap_3d_sw128_box(&tmQ, Q, q_rows / q_seq_rows, q_seq_rows, q_cols, ldq, ldq * q_seq_rows,
                                q_group, q_rows_per_seq, 64, 2);
  } else {
    rc = make_tmap_2d_sw128(&tmQ, Q, q_rows, q_cols, ldq, p.q_rows_box, 64, 2);
  }
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n_src == 1) {
    KvMaps<1> kv;
    if ((rc = make_tmap_2d_sw128(&kv.k[0], k_ptrs[0], kv_rows, kv_cols, ldkv, 128, 64, 2))) return rc;
    if ((rc = make_tmap_2d_sw128(&kv.v[0], v_ptrs[0], kv_rows, kv_cols, ldkv, 128, 64, 2))) return rc;
    return decode_rows ? launch_attn_fwd<1, true>(tmQ, kv, kv, p, s) : launch_attn_fwd<1, false>(tmQ, kv, kv, p, s);
  }
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
    // remote K/V blocks are copied once into [n_src * stage_rows, kv_cols] buffers of this GPU
    RLK_REQUIRE(stage_k && stage_v && stage_flags, "attn_fwd: staging buffers missing");
    RLK_REQUIRE(stage_rows % 128 == 0 && stage_rows <= kv_rows && ldkv == kv_cols && page_table == nullptr,
                "attn_fwd: staging needs 128-row multiples, contiguous K/V rows and no page table");
    RLK_REQUIRE(cp_rank >= 0 && cp_rank < n_src, "attn_fwd: bad cp_rank");
    CpStage& st = p.stage;
    for (int i = 0; i < 8; ++i) {
      st.src_a[i] = static_cast<const unsigned char*>(k_ptrs[i < n_src ? i : 0]);
      st.src_b[i] = static_cast<const unsigned char*>(v_ptrs[i < n_src ? i : 0]);
    }
    st.dst_a = static_cast<unsigned char*>(stage_k);
    st.dst_b = static_cast<unsigned char*>(stage_v);
    st.flags = stage_flags;
    st.rows = stage_rows;
    st.row_bytes_a = st.row_bytes_b = static_cast<int>(kv_cols * 2);
    st.ranks = n_src;
    st.rank = cp_rank;
    const long long total = static_cast<long long>(n_src) * stage_rows;
    if ((rc = make_tmap_2d_sw128(&staged.k[0], stage_k, total, kv_cols, kv_cols, 128, 64, 2))) return rc;
    if ((rc = make_tmap_2d_sw128(&staged.v[0], stage_v, total, kv_cols, kv_cols, 128, 64, 2))) return rc;
    RLK_CHECK_CUDA(cudaMemsetAsync(stage_flags, 0, sizeof(int) * (n_src * (stage_rows / 128) * 2 + 1), s));
  }
  return decode_rows ? launch_attn_fwd<8, true>(tmQ, kv, staged, p, s) : launch_attn_fwd<8, false>(tmQ, kv, staged, p, s);
}
