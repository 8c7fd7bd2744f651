// The selected-token log-prob contract, shared by the fused LM-head epilogue and the
// from-logits kernels so both produce the same bits.
//
//   * logits are bf16 (the rounded fp32 accumulator); z = fp32(logit) * inv_temperature;
//   * the vocabulary is cut into canonical tiles of 128 consecutive GLOBAL vocab ids
//     (tile t = ids [128 t, 128 t + 128)); columns at or beyond the real vocab size count as -inf;
//   * per (row, tile):  m = max z ;  s = sum_j exp(z_j - m), the 128 terms added as four
//     interleaved sequential chains (j mod 4) that are combined as (c0 + c1) + (c2 + c3);
//   * per row: M = max_t m_t ; S = sum_t s_t * exp(m_t - M) added sequentially in ascending t;
//     lse = M + log(S) ; logp = min(z_target - lse, 0).
// Tiles never straddle a tensor-parallel vocab shard when the padded vocab is a multiple of
// 128 * TP, so TP = 1, 2, 4, 8 merge the very same list of tile statistics.
// (The reference's equivalent is the 64-tile contract of
// rl_engine/reference/logprob/vocab_parallel_logp.py:4-36.)
#pragma once
#include <cuda_runtime.h>
#include <math.h>

namespace rlk {

constexpr int kVocabTile = 128;

__device__ __forceinline__ float logp_exp(float x) { return __expf(x); }
// z = fp32(bf16 logit) * inv_temperature with an explicit, never-fused multiply.
__device__ __forceinline__ float logp_scale(float logit, float inv_temp) { return __fmul_rn(logit, inv_temp); }

// z[0..127] already scaled and masked (-inf for invalid columns).
__device__ __forceinline__ void tile_stats_128(const float (&z)[128], float& m_out, float& s_out) {
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < 128; ++j) m = fmaxf(m, z[j]);
  float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
  if (m > -INFINITY) {
#pragma unroll
    for (int j = 0; j < 128; j += 4) {
      c0 = __fadd_rn(c0, logp_exp(__fsub_rn(z[j], m)));
      c1 = __fadd_rn(c1, logp_exp(__fsub_rn(z[j + 1], m)));
      c2 = __fadd_rn(c2, logp_exp(__fsub_rn(z[j + 2], m)));
      c3 = __fadd_rn(c3, logp_exp(__fsub_rn(z[j + 3], m)));
    }
  }
  m_out = m;
  s_out = __fadd_rn(__fadd_rn(c0, c1), __fadd_rn(c2, c3));
}

// Streaming form used where the 128 values arrive in four 32-wide pieces (TMEM chunks):
// call max over all pieces first, then tile_sum_piece for pieces 0..3 in order.
struct TileSum {
  float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
  __device__ __forceinline__ void add4(float z0, float z1, float z2, float z3, float m) {
    c0 = __fadd_rn(c0, logp_exp(__fsub_rn(z0, m)));
    c1 = __fadd_rn(c1, logp_exp(__fsub_rn(z1, m)));
    c2 = __fadd_rn(c2, logp_exp(__fsub_rn(z2, m)));
    c3 = __fadd_rn(c3, logp_exp(__fsub_rn(z3, m)));
  }
  __device__ __forceinline__ float total() const {
    return __fadd_rn(__fadd_rn(c0, c1), __fadd_rn(c2, c3));
  }
};

}  // namespace rlk
