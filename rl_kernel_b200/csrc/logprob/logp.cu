// Selected-token log-prob from materialised bf16 logits, the ordered merge of per-tile
// statistics, and the logits-gradient kernel.  See rlk/logp_contract.cuh for the contract.
//
// Kernels:
//   logits_tile_stats : one thread per (row, 128-id tile) -> (max, sumexp), + target logit
//   logp_merge        : one thread per row, tiles in ascending order -> logp, lse
//   dlogits           : in place  logits <- g * (onehot(target) - softmax(z)) * inv_temp
// Counterparts in the reference: csrc/cuda/logprob/deterministic_logp_kernel.cu:451-612
// (tile_stats / backward) and csrc/cuda/logprob/fused_logp_kernel.cu:606-648 (ordered merge).
#include <climits>

#include "rlk/host.h"
#include "rlk/logp_contract.cuh"
#include "rlk/ptx.cuh"

namespace rlk {

// One thread owns one 128-id vocabulary tile of one row (its statistics have a fixed order), but the 256 bytes of a
// tile are fetched by the whole warp: a warp's 32 tiles are 8 KB of contiguous logits, read as 16 fully coalesced
// 512-byte requests into shared memory (tile pitch 272 bytes: the 16-byte reads of a quarter warp then fall into eight
// different bank groups) and consumed by their owners from there.  Grid: (rows, groups of 128 tiles).
constexpr int kTilePitch = 272;
__global__ void __launch_bounds__(128)
logits_tile_stats_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                         float2* __restrict__ stats, long long stats_row_stride, float* __restrict__ tgt_logit,
                         int rows, int n_local, long long vocab_start, int tile_start, int n_tiles_local,
                         float inv_temp, const long long* __restrict__ row_indices, const float* __restrict__ min_keep) {
  __shared__ __align__(16) unsigned char stage[4][32 * kTilePitch];
  griddep_sync();
  const int row = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lt0 = (blockIdx.y * 4 + warp) * 32;          // first tile of this warp
  if (lt0 >= n_tiles_local) return;
  // indexed form: output row `row` scores logits row row_indices[row] (the launch geometry
  // depends only on the number of scored rows and the vocabulary, never on the index values)
  const long long src_row = row_indices ? row_indices[row] : row;
  const __nv_bfloat16* wsrc = logits + src_row * ld + static_cast<long long>(lt0) * kVocabTile;
  unsigned char* st = stage[warp];
  uint4 piece[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {                          // all 16 requests in flight before the first store
    const int p = i * 32 + lane;                          // 16-byte piece of the warp's 8 KB
    piece[i] = make_uint4(0, 0, 0, 0);
    if (lt0 * kVocabTile + p * 8 < n_local) piece[i] = *reinterpret_cast<const uint4*>(wsrc + p * 8);   // n_local % 8 == 0
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int p = i * 32 + lane;
    *reinterpret_cast<uint4*>(st + (p >> 4) * kTilePitch + (p & 15) * 16) = piece[i];
  }
  __syncwarp();
  const int lt = lt0 + lane;
  if (lt >= n_tiles_local) return;
  const int col0 = lt * kVocabTile;
  // restricted sampling support: scaled logits below the row's threshold count as -inf
  const float keep_from = min_keep ? min_keep[row] : -INFINITY;
  float z[128];
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    const bool in = col0 + c * 8 < n_local;
    const uint4 v = *reinterpret_cast<const uint4*>(st + lane * kTilePitch + c * 16);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float z0 = logp_scale(bf16_lo(u[k]), inv_temp), z1 = logp_scale(bf16_hi(u[k]), inv_temp);
      z[c * 8 + 2 * k] = (in && z0 >= keep_from) ? z0 : -INFINITY;
      z[c * 8 + 2 * k + 1] = (in && z1 >= keep_from) ? z1 : -INFINITY;
    }
  }
  float m, s;
  tile_stats_128(z, m, s);
  stats[row * stats_row_stride + tile_start + lt] = make_float2(m, s);
  if (targets) {
    const long long tl = targets[row] - vocab_start - col0;
    if (tl >= 0 && tl < kVocabTile && col0 + tl < n_local) {
      const float zt = logp_scale(__bfloat162float(logits[src_row * ld + col0 + tl]), inv_temp);
      tgt_logit[row] = zt >= keep_from ? zt : -INFINITY;
    }
  }
}

// One warp per row.  The maximum is order-free; the sum keeps the contract's order exactly: the 32
// lanes compute exp(m_t - M) for 32 consecutive tiles in parallel, then lane 0 folds them into S
// with S = fma(s_t, e_t, S) in ascending t (values handed over by shuffles).
__global__ void __launch_bounds__(128)
logp_merge_kernel(const float2* __restrict__ stats, long long stats_row_stride, int n_tiles,
                  const float* __restrict__ tgt_logit, float* __restrict__ logp, float* __restrict__ lse,
                  int rows) {
  griddep_sync();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float2* st = stats + row * stats_row_stride;
  float M = -INFINITY;
  for (int t = lane; t < n_tiles; t += 32) M = fmaxf(M, st[t].x);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  float S = 0.f;
  for (int t0 = 0; t0 < n_tiles; t0 += 32) {
    const int t = t0 + lane;
    float y = 0.f, e = 0.f;
    if (t < n_tiles) {
      const float2 v = st[t];
      if (v.x > -INFINITY) { y = v.y; e = logp_exp(__fsub_rn(v.x, M)); }
    }
    // (unrolled: the shuffles of all 32 tiles are in flight at once and only the fma chain is
    // serial; tiles past the end carry y = e = 0 and are skipped like empty ones)
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float yj = __shfl_sync(0xffffffffu, y, j), ej = __shfl_sync(0xffffffffu, e, j);
      if (ej != 0.f || yj != 0.f) S = fmaf(yj, ej, S);
    }
  }
  if (lane == 0) {
    const float l = __fadd_rn(M, logf(S));
    if (lse) lse[row] = l;
    if (logp) logp[row] = fminf(__fsub_rn(tgt_logit[row], l), 0.f);
  }
}

// logits[row, j] <- (g[row] * inv_temp) * ( [j == target] - exp(z_j - lse[row]) )   (bf16, in place)
__global__ void __launch_bounds__(256)
dlogits_kernel(__nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ targets,
               const float* __restrict__ lse, const float* __restrict__ g, int rows, int n_local,
               long long vocab_start, float inv_temp, const float* __restrict__ g_lse,
               const float* __restrict__ min_keep) {
  const int per_row = n_local / 8;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(rows) * per_row) return;
  const int row = static_cast<int>(idx / per_row), c = static_cast<int>(idx % per_row) * 8;
  const float gr = g[row] * inv_temp, l = lse[row];
  const float gl = g_lse ? g_lse[row] * inv_temp : 0.f;   // d(loss)/d(lse): adds g_lse * p
  const float keep_from = min_keep ? min_keep[row] : -INFINITY;   // outside the support: p = 0, no gradient
  const long long tl = targets[row] - vocab_start - c;
  uint4* ptr = reinterpret_cast<uint4*>(logits + row * ld + c);
  const uint4 v = *ptr;
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float z0 = bf16_lo(u[k]) * inv_temp, z1 = bf16_hi(u[k]) * inv_temp;
    const float p0 = z0 >= keep_from ? logp_exp(z0 - l) : 0.f, p1 = z1 >= keep_from ? logp_exp(z1 - l) : 0.f;
    float d0 = gr * ((tl == 2 * k ? 1.f : 0.f) - p0), d1 = gr * ((tl == 2 * k + 1 ? 1.f : 0.f) - p1);
    if (g_lse) { d0 = fmaf(gl, p0, d0); d1 = fmaf(gl, p1, d1); }
    o[k] = pack_bf16x2(d0, d1);
  }
  *ptr = make_uint4(o[0], o[1], o[2], o[3]);
}

// Restricted-support statistics from a compact id list instead of a mask or a threshold: row r keeps
// only the (up to 64) global ids replay_ids[r, 0..K).  One warp per row sorts the ids that fall into
// this shard, drops duplicates, and walks them tile by tile in ascending order: per touched tile
// m = max z and the four chains (position mod 4) summed in ascending position, s = (c0+c1)+(c2+c3)
// -- the masked-out positions of the dense kernel add exp(-inf) = +0 to their chain, which changes
// nothing, so these are the bits logits_tile_stats would give for logits masked to the same ids.
// Output: stats_compact[r, 0..K) = the touched tiles' (m, s) in ascending tile order, then
// (-inf, 0) fillers, which logp_merge skips exactly as it skips untouched tiles of the dense list.
// (counterpart: linear_logp_top_p_local_bf16_forward_kernel,
// csrc/cuda/logprob/fused_linear_logp_sm90.cu:741-884, which lane-assigns ids for its 256-lane order.)
constexpr int kReplayMax = 64;

__global__ void __launch_bounds__(128)
replay_tile_stats_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                         const long long* __restrict__ replay_ids, int K, float2* __restrict__ stats_compact,
                         float* __restrict__ tgt_logit, int rows, int n_local, long long vocab_start, float inv_temp,
                         const long long* __restrict__ row_indices) {
  griddep_sync();
  __shared__ int s_col[4][kReplayMax];
  __shared__ float s_z[4][kReplayMax];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + w;
  if (row >= rows) return;                                   // whole warps leave together
  const long long src_row = row_indices ? row_indices[row] : row;
  const __nv_bfloat16* src = logits + src_row * ld;
  // 1. local columns of this row's ids (INT_MAX: not in this shard / past K)
  int col[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int i = lane + 32 * h;
    col[h] = INT_MAX;
    if (i < K) {
      const long long c = replay_ids[static_cast<long long>(row) * K + i] - vocab_start;
      if (c >= 0 && c < n_local) col[h] = static_cast<int>(c);
    }
    s_col[w][i] = col[h];
  }
  __syncwarp();
  // 2. drop duplicates (keep the first occurrence), then rank = number of smaller distinct ids
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int i = lane + 32 * h;
    bool dup = false;
    for (int j = 0; j < i; ++j) dup = dup || (s_col[w][j] == col[h]);
    if (dup) col[h] = INT_MAX;
  }
  __syncwarp();
#pragma unroll
  for (int h = 0; h < 2; ++h) s_col[w][lane + 32 * h] = col[h];
  __syncwarp();
  int rank[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    int r = 0;
    for (int j = 0; j < kReplayMax; ++j) r += (s_col[w][j] < col[h]) ? 1 : 0;
    rank[h] = col[h] == INT_MAX ? -1 : r;
  }
  __syncwarp();
#pragma unroll
  for (int h = 0; h < 2; ++h) s_col[w][lane + 32 * h] = INT_MAX;
  __syncwarp();
  int n_valid = 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (rank[h] >= 0) {
      s_col[w][rank[h]] = col[h];
      s_z[w][rank[h]] = logp_scale(__bfloat162float(src[col[h]]), inv_temp);
    }
    n_valid += __popc(__ballot_sync(0xffffffffu, rank[h] >= 0));
  }
  __syncwarp();
  // 3. every lane walks the sorted list the same way (warp-uniform, a few hundred instructions)
  float2* out = stats_compact + static_cast<long long>(row) * K;
  const long long tcol = targets ? targets[row] - vocab_start : -1;
  float zt = -INFINITY;
  bool own_target = targets && tcol >= 0 && tcol < n_local;
  int n_out = 0;
  for (int i = 0; i < n_valid;) {
    const int tile = s_col[w][i] / kVocabTile;
    int e = i;
    float m = -INFINITY;
    while (e < n_valid && s_col[w][e] / kVocabTile == tile) { m = fmaxf(m, s_z[w][e]); ++e; }
    float c4[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = i; j < e; ++j) {                          // ascending position within each chain
      const int ch = s_col[w][j] & 3;
      c4[ch] = __fadd_rn(c4[ch], logp_exp(__fsub_rn(s_z[w][j], m)));
      if (s_col[w][j] == tcol) zt = s_z[w][j];
    }
    if (lane == 0) out[n_out] = make_float2(m, __fadd_rn(__fadd_rn(c4[0], c4[1]), __fadd_rn(c4[2], c4[3])));
    ++n_out;
    i = e;
  }
  for (int i = n_out + lane; i < K; i += 32) out[i] = make_float2(-INFINITY, 0.f);
  if (lane == 0 && own_target) tgt_logit[row] = zt;        // -inf when the target is not in the replay set
}

}  // namespace rlk
using namespace rlk;

// stats: float2 [rows][stats_row_stride]; this call fills tiles [tile_start, tile_start + n_tiles_local)
// from a local logits shard [rows, n_local] whose first column is global vocab id `vocab_start`
// (a multiple of 128). tgt_logit[row] is written only by the shard that owns the target.
RLK_API int rlk_logits_tile_stats_keep(const void* logits, long long ld, const long long* targets,
                                       void* stats, long long stats_row_stride, float* tgt_logit, int rows,
                                       int n_local, long long vocab_start, float inv_temp,
                                       const long long* row_indices, const float* min_keep, void* stream) {
  RLK_REQUIRE(rows > 0 && n_local > 0 && n_local % 8 == 0 && ld % 8 == 0, "tile_stats: bad shape");
  RLK_REQUIRE(vocab_start % kVocabTile == 0, "tile_stats: vocab_start must be a multiple of 128");
  const int n_tiles_local = (n_local + kVocabTile - 1) / kVocabTile;
  RLK_CHECK_CUDA(launch_pdl(logits_tile_stats_kernel, dim3(static_cast<unsigned>(rows), static_cast<unsigned>((n_tiles_local + 127) / 128)), dim3(128), 0,
                            static_cast<cudaStream_t>(stream), (const __nv_bfloat16*)logits, ld, targets,
                            (float2*)stats, stats_row_stride, tgt_logit, rows, n_local, vocab_start,
                            static_cast<int>(vocab_start / kVocabTile), n_tiles_local, inv_temp, row_indices, min_keep));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_logits_tile_stats_indexed(const void* logits, long long ld, const long long* targets,
                                          void* stats, long long stats_row_stride, float* tgt_logit, int rows,
                                          int n_local, long long vocab_start, float inv_temp,
                                          const long long* row_indices, void* stream) {
  return rlk_logits_tile_stats_keep(logits, ld, targets, stats, stats_row_stride, tgt_logit, rows, n_local,
                                    vocab_start, inv_temp, row_indices, nullptr, stream);
}

// replay_ids int64 [rows, K] (K <= 64, global ids, duplicates and ids of other shards allowed);
// stats_compact float2 [rows, K]; tgt_logit[row] is written only by the shard that owns the target
// (-inf if the target is not among the row's ids).  Merge with rlk_logp_merge(stats_compact, K, K, ...),
// or gather the shards' lists in rank order first.
RLK_API int rlk_replay_tile_stats(const void* logits, long long ld, const long long* targets,
                                  const long long* replay_ids, int K, void* stats_compact, float* tgt_logit,
                                  int rows, int n_local, long long vocab_start, float inv_temp,
                                  const long long* row_indices, void* stream) {
  RLK_REQUIRE(rows > 0 && n_local > 0 && ld >= n_local, "replay_tile_stats: bad shape");
  RLK_REQUIRE(K > 0 && K <= kReplayMax, "replay_tile_stats: K must be 1..64");
  RLK_REQUIRE(vocab_start % kVocabTile == 0, "replay_tile_stats: vocab_start must be a multiple of 128");
  RLK_REQUIRE(logits && replay_ids && stats_compact, "replay_tile_stats: null pointer");
  RLK_CHECK_CUDA(launch_pdl(replay_tile_stats_kernel, dim3((rows + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(stream),
                            (const __nv_bfloat16*)logits, ld, targets, replay_ids, K, (float2*)stats_compact, tgt_logit,
                            rows, n_local, vocab_start, inv_temp, row_indices));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_logits_tile_stats(const void* logits, long long ld, const long long* targets,
                                  void* stats, long long stats_row_stride, float* tgt_logit, int rows,
                                  int n_local, long long vocab_start, float inv_temp, void* stream) {
  return rlk_logits_tile_stats_indexed(logits, ld, targets, stats, stats_row_stride, tgt_logit, rows, n_local,
                                       vocab_start, inv_temp, nullptr, stream);
}

RLK_API int rlk_logp_merge(const void* stats, long long stats_row_stride, int n_tiles,
                           const float* tgt_logit, float* logp, float* lse, int rows, void* stream) {
  RLK_REQUIRE(rows > 0 && n_tiles > 0, "logp_merge: bad shape");
  RLK_CHECK_CUDA(launch_pdl(logp_merge_kernel, dim3((rows + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(stream),
                            (const float2*)stats, stats_row_stride, n_tiles, tgt_logit, logp, lse, rows));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// In place: logits <- g_logp * (onehot(target) - p) + g_lse * p, p = softmax(logits * inv_temp),
// both scaled by inv_temp (g_lse may be null: the log-sum-exp does not enter the loss).
RLK_API int rlk_dlogits_keep(void* logits, long long ld, const long long* targets, const float* lse,
                             const float* g, const float* g_lse, const float* min_keep, int rows, int n_local,
                             long long vocab_start, float inv_temp, void* stream) {
  RLK_REQUIRE(rows > 0 && n_local % 8 == 0 && ld % 8 == 0, "dlogits: bad shape");
  const long long n = static_cast<long long>(rows) * (n_local / 8);
  dlogits_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (__nv_bfloat16*)logits, ld, targets, lse, g, rows, n_local, vocab_start, inv_temp, g_lse, min_keep);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_dlogits_lse(void* logits, long long ld, const long long* targets, const float* lse,
                            const float* g, const float* g_lse, int rows, int n_local, long long vocab_start,
                            float inv_temp, void* stream) {
  return rlk_dlogits_keep(logits, ld, targets, lse, g, g_lse, nullptr, rows, n_local, vocab_start, inv_temp, stream);
}

RLK_API int rlk_dlogits(void* logits, long long ld, const long long* targets, const float* lse,
                        const float* g, int rows, int n_local, long long vocab_start, float inv_temp,
                        void* stream) {
  return rlk_dlogits_lse(logits, ld, targets, lse, g, nullptr, rows, n_local, vocab_start, inv_temp, stream);
}
