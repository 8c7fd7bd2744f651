// Work-item description shared by the attention forward and backward kernels.
//
// Attention runs over "tiles" of up to 128 query rows that all read keys from one contiguous
// run of rows of the K/V tensors (one sequence, one KV head).  Training (packed varlen),
// prefill, single-token decode against a KV cache (the 4 query heads of a GQA group become 4
// rows of one tile) and context-parallel shards are all expressed as lists of such tiles, so
// every mode executes the same per-row program:
//   * keys are consumed in canonical blocks of 128, block b = keys [128 b, 128 b + 128) counted
//     from the first key of the sequence, in ascending b;
//   * row r sees keys j < kv_len(r) = min(kv_cap, pos0 + r * pos_step + 1);
//   * a block that is completely masked for a row leaves that row's state bit-for-bit unchanged.
// That is what makes selected-token log-probs of rollout (decode) and training (full sequence)
// bitwise equal, for every batch size and query tiling.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace rlk {

struct AttnTile {
  int q_row0;    // first query row: y coordinate in the Q / O / dO tensor maps
  int q_col0;    // x coordinate of the head in Q / O (elements)
  int n_rows;    // valid query rows in this tile (1..128); 0 = empty tile
  int kv_row0;   // y coordinate of key 0 of the sequence in the K / V tensor maps
  int kv_col0;   // x coordinate of the KV head in K / V (elements)
  int pos0;      // position (key index) of query row 0
  int pos_step;  // 1: consecutive rows are consecutive positions; 0: all rows share pos0
  int kv_cap;    // number of keys that exist (kv_len never exceeds it)
  int lse_off;   // lse[lse_off + r * lse_stride] receives row r's log-sum-exp
  int lse_stride;
  int kv_src;    // index into the K/V tensor-map table (context parallel: owning rank); 0 otherwise
  int reserved;
};

constexpr int kAttnBlock = 128;  // canonical KV block and query tile
constexpr int kHeadDim = 128;

// One tensor map per context-parallel rank for a pair of operands that are fetched together
// (K and V in the forward and dQ kernels, Q and dO in the dK/dV kernel).
template <int NSRC>
struct KvMaps {
  CUtensorMap k[NSRC];
  CUtensorMap v[NSRC];
};

// How the 128-token blocks of one sequence are spread over context-parallel ranks.  Every rank
// stores its blocks of a sequence back to back, so "local block i" is row 128*i after the
// sequence's first local row.  contiguous: the sequence is cut into `ranks` chunks of
// `blocks_per_chunk` blocks, chunk c on rank c.  zigzag: 2*ranks chunks, rank c holds chunks c and
// 2*ranks-1-c (in that order), which balances causal work.
struct CpLayout {
  int ranks;             // <= 1: not context parallel
  int blocks_per_chunk;
  int zigzag;
};

__host__ __device__ __forceinline__ void cp_locate_block(const CpLayout& c, int b, int& src, int& local_block) {
  if (c.ranks <= 1) {
    src = 0;
    local_block = b;
    return;
  }
  const int chunk = b / c.blocks_per_chunk;
  const int within = b - chunk * c.blocks_per_chunk;
  int local_chunk = 0;
  if (c.zigzag) {
    if (chunk < c.ranks) {
      src = chunk;
    } else {
      src = 2 * c.ranks - 1 - chunk;
      local_chunk = 1;
    }
  } else {
    src = chunk;
  }
  local_block = local_chunk * c.blocks_per_chunk + within;
}

}  // namespace rlk
