// Embedding gather and its deterministic weight gradient.
//
// Backward: token positions are sorted by id on the host side of the op (stable sort), so all
// occurrences of one id are adjacent and in ascending token order.  One CTA per distinct id
// walks its run sequentially and adds the rows in fp32 — fixed order, no atomics — then adds
// the run total to the weight-gradient row.  (Reference: csrc/cuda/embedding/
// embedding_lm_head_sm90.cu:66-114 and _deterministic_embedding_grad_weight in
// rl_engine/backends/cuda/embedding/embedding.py:22.)
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

__global__ void __launch_bounds__(128)
embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                     __nv_bfloat16* __restrict__ out, int T, int H, long long vocab_start,
                     long long vocab_rows) {
  griddep_sync();
  const int t = blockIdx.x;
  const long long id = ids[t] - vocab_start;
  const bool mine = id >= 0 && id < vocab_rows;
  const uint4* src = reinterpret_cast<const uint4*>(w + (mine ? id : 0) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H);
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = mine ? src[c] : make_uint4(0, 0, 0, 0);
}

// sorted_ids[i] ascending, order[i] = original token index of sorted position i.
__global__ void __launch_bounds__(128)
embedding_bwd_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ order,
                     const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dw, int T,
                     int H, long long vocab_start, long long vocab_rows) {
  const int i = blockIdx.x;
  const long long id = sorted_ids[i];
  if (i > 0 && sorted_ids[i - 1] == id) return;  // not the start of a run
  const long long row = id - vocab_start;
  if (row < 0 || row >= vocab_rows) return;
  int end = i + 1;
  while (end < T && sorted_ids[end] == id) ++end;
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = i; j < end; ++j) {
      const uint4 v = *reinterpret_cast<const uint4*>(dy + order[j] * H + c * 8);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] += bf16_lo(u[k]);
        acc[2 * k + 1] += bf16_hi(u[k]);
      }
    }
    uint4* d = reinterpret_cast<uint4*>(dw + row * H + c * 8);
    const uint4 o = *d;
    *d = make_uint4(pack_bf16x2(bf16_lo(o.x) + acc[0], bf16_hi(o.x) + acc[1]),
                    pack_bf16x2(bf16_lo(o.y) + acc[2], bf16_hi(o.y) + acc[3]),
                    pack_bf16x2(bf16_lo(o.z) + acc[4], bf16_hi(o.z) + acc[5]),
                    pack_bf16x2(bf16_lo(o.w) + acc[6], bf16_hi(o.w) + acc[7]));
  }
}

}  // namespace rlk
using namespace rlk;

// out[t] = w[ids[t] - vocab_start] if that row is in [0, vocab_rows) else 0 (vocab-parallel shard).
RLK_API int rlk_embedding_fwd(const long long* ids, const void* w, void* out, int T, int H,
                              long long vocab_start, long long vocab_rows, void* stream) {
  RLK_REQUIRE(T > 0 && H % 8 == 0, "embedding: H must be a multiple of 8");
  RLK_CHECK_CUDA(launch_pdl(embedding_fwd_kernel, dim3(T), dim3(128), 0, static_cast<cudaStream_t>(stream), ids,
                            (const __nv_bfloat16*)w, (__nv_bfloat16*)out, T, H, vocab_start, vocab_rows));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// dw[id] += sum of dy rows whose token has that id, in ascending token order.
RLK_API int rlk_embedding_bwd(const long long* sorted_ids, const long long* order, const void* dy,
                              void* dw, int T, int H, long long vocab_start, long long vocab_rows,
                              void* stream) {
  RLK_REQUIRE(T > 0 && H % 8 == 0, "embedding_bwd: H must be a multiple of 8");
  embedding_bwd_kernel<<<T, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      sorted_ids, order, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dw, T, H, vocab_start, vocab_rows);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
