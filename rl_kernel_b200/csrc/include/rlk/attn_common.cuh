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

}  // namespace rlk
