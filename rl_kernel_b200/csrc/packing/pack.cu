// Varlen packing: rows of a padded [B * S, row_bytes] tensor are compacted into [T, row_bytes]
// (and scattered back) by an index list, with 16-byte vector copies.  The index list is the
// row-major order of the kept positions (cu_seqlens order), so packing never reorders tokens.
// (parity: NativePackOp, rl_engine/reference/packing/pack.py:95; the reference packs with torch
// boolean indexing.)
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

// dst[t] = src[idx[t]] (gather = pack) or dst[idx[t]] = src[t] (scatter = unpack); one warp per row.
template <bool SCATTER>
__global__ void __launch_bounds__(256)
move_rows_kernel(const unsigned char* __restrict__ src, long long src_pitch, const long long* __restrict__ idx,
                 unsigned char* __restrict__ dst, long long dst_pitch, int n, int row_bytes, long long idx_limit) {
  griddep_sync();
  const int lane = threadIdx.x & 31;
  for (long long t = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); t < n;
       t += static_cast<long long>(gridDim.x) * 8) {
    const long long j = idx[t];
    if (j < 0 || j >= idx_limit) continue;            // defensive: an index outside the other tensor is skipped
    const unsigned char* s = src + (SCATTER ? t : j) * src_pitch;
    unsigned char* d = dst + (SCATTER ? j : t) * dst_pitch;
    // four 16-byte loads per lane in flight before the first store (2 KB of the row per warp and round trip)
    int b = lane * 16;
    for (; b + 1536 < row_bytes; b += 2048) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const uint4*>(s + b + u * 512);
#pragma unroll
      for (int u = 0; u < 4; ++u) *reinterpret_cast<uint4*>(d + b + u * 512) = v[u];
    }
    for (; b < row_bytes; b += 512) *reinterpret_cast<uint4*>(d + b) = *reinterpret_cast<const uint4*>(s + b);
  }
}

}  // namespace rlk
using namespace rlk;

// scatter = 0: dst[t] = src[idx[t]], t < n (idx values < idx_limit = rows of src).
// scatter = 1: dst[idx[t]] = src[t], t < n (idx values < idx_limit = rows of dst; rows of dst that no
// index names keep what the caller put there, e.g. a fill value).
RLK_API int rlk_move_rows(const void* src, long long src_pitch, const long long* idx, void* dst, long long dst_pitch,
                          int n, int row_bytes, long long idx_limit, int scatter, void* stream) {
  RLK_REQUIRE(n >= 0 && row_bytes > 0 && row_bytes % 16 == 0, "move_rows: row_bytes must be a positive multiple of 16");
  RLK_REQUIRE(src_pitch % 16 == 0 && dst_pitch % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(dst) & 15) == 0, "move_rows: 16-byte aligned rows required");
  if (n == 0) return RLK_OK;
  const int grid = (n + 7) / 8 < 8 * sm_count() ? (n + 7) / 8 : 8 * sm_count();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (scatter)
    RLK_CHECK_CUDA(launch_pdl(move_rows_kernel<true>, dim3(grid), dim3(256), 0, s, (const unsigned char*)src, src_pitch, idx,
                              (unsigned char*)dst, dst_pitch, n, row_bytes, idx_limit));
  else
    RLK_CHECK_CUDA(launch_pdl(move_rows_kernel<false>, dim3(grid), dim3(256), 0, s, (const unsigned char*)src, src_pitch, idx,
                              (unsigned char*)dst, dst_pitch, n, row_bytes, idx_limit));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
