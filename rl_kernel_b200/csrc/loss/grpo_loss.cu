// GRPO / PPO clipped-ratio surrogate with the k3 reference-KL penalty, from per-token log-probs.
//
// Per token (mask = 1):  ratio = exp(logp - old);  surr = -min(ratio*A, clip(ratio,1-e,1+e)*A)
//                        d = ref - logp;           kl  = exp(d) - d - 1              (k3)
// Outputs per token: loss term, kl term, ratio, and dloss/dlogp (already divided by the
// normaliser), plus deterministic sums: one warp per sequence adds its tokens lane-strided in
// ascending order and folds the 32 lanes with the xor butterfly; a last kernel adds the
// per-sequence totals in ascending sequence order (sequence-major fixed sums as in the
// reference's DistributedGRPOLossOp, rl_engine/reference/loss/distributed_grpo_loss.py:177-299).
// Math follows rl_engine/reference/loss/grpo_loss.py:101-129 and ratio_kl.py:55-75.
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

struct GrpoParams {
  const float* logp; const float* old_logp; const float* ref_logp;  // [B, L]
  const float* adv;          // [B] per-sequence advantage
  const unsigned char* mask; // [B, L]
  float* loss_tok; float* kl_tok; float* ratio_tok; float* dlogp;   // [B, L], any may be null
  float* seq_sums;           // [B, 4]: policy-loss sum, kl sum, token count, clipped count
  int B, L;
  float clip_lo, clip_hi, beta;
  float inv_norm;            // 1 / normaliser applied to dlogp (e.g. 1 / total active tokens)
};

__global__ void __launch_bounds__(256) grpo_token_kernel(const GrpoParams p) {
  const int seq = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (seq >= p.B) return;
  const float A = p.adv[seq];
  float s_pol = 0.f, s_kl = 0.f, s_cnt = 0.f, s_clip = 0.f;
  for (int j = lane; j < p.L; j += 32) {
    const long long i = static_cast<long long>(seq) * p.L + j;
    const bool on = p.mask[i] != 0;
    float pol = 0.f, kl = 0.f, ratio = 0.f, g = 0.f;
    if (on) {
      const float lp = p.logp[i];
      ratio = __expf(lp - p.old_logp[i]);
      const float unclipped = ratio * A;
      const float rc = fminf(fmaxf(ratio, p.clip_lo), p.clip_hi);
      const float clipped = rc * A;
      pol = -fminf(unclipped, clipped);
      const bool use_unclipped = unclipped <= clipped;
      float dpol = use_unclipped ? -A * ratio : ((rc == ratio) ? -A * ratio : 0.f);
      if (p.ref_logp) {
        const float d = p.ref_logp[i] - lp;
        const float e = __expf(d);
        kl = e - d - 1.f;
        g = dpol + p.beta * (1.f - e);
      } else {
        g = dpol;
      }
      s_pol += pol; s_kl += kl; s_cnt += 1.f;
      s_clip += (rc != ratio) ? 1.f : 0.f;
    }
    if (p.loss_tok) p.loss_tok[i] = pol + p.beta * kl;
    if (p.kl_tok) p.kl_tok[i] = kl;
    if (p.ratio_tok) p.ratio_tok[i] = ratio;
    if (p.dlogp) p.dlogp[i] = g * p.inv_norm;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s_pol += __shfl_xor_sync(0xffffffffu, s_pol, o);
    s_kl += __shfl_xor_sync(0xffffffffu, s_kl, o);
    s_cnt += __shfl_xor_sync(0xffffffffu, s_cnt, o);
    s_clip += __shfl_xor_sync(0xffffffffu, s_clip, o);
  }
  if (lane == 0 && p.seq_sums) {
    p.seq_sums[seq * 4 + 0] = s_pol;
    p.seq_sums[seq * 4 + 1] = s_kl;
    p.seq_sums[seq * 4 + 2] = s_cnt;
    p.seq_sums[seq * 4 + 3] = s_clip;
  }
}

// totals[0..3] = ascending-sequence sums of seq_sums columns; totals[4] = loss = (pol + beta*kl)/cnt
__global__ void grpo_total_kernel(const float* __restrict__ seq_sums, int B, float beta, float* totals) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  float t[4] = {0.f, 0.f, 0.f, 0.f};
  for (int b = 0; b < B; ++b)
    for (int k = 0; k < 4; ++k) t[k] += seq_sums[b * 4 + k];
  for (int k = 0; k < 4; ++k) totals[k] = t[k];
  const float cnt = fmaxf(t[2], 1.f);
  totals[4] = (t[0] + beta * t[1]) / cnt;
  totals[5] = t[0] / cnt;
  totals[6] = t[1] / cnt;
  totals[7] = t[3] / cnt;
}

// Group-relative advantages: rewards [G, n] -> (r - mean) / max(std, eps), two-pass variance.
__global__ void group_adv_kernel(const float* __restrict__ rewards, float* __restrict__ adv, int groups,
                                 int n, float eps) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  const float* r = rewards + static_cast<long long>(g) * n;
  float mean = 0.f;
  for (int i = 0; i < n; ++i) mean += r[i];
  mean /= static_cast<float>(n);
  float var = 0.f;
  for (int i = 0; i < n; ++i) { const float d = r[i] - mean; var = fmaf(d, d, var); }
  var /= static_cast<float>(n);
  const float sd = fmaxf(sqrtf(var), eps);
  for (int i = 0; i < n; ++i) adv[static_cast<long long>(g) * n + i] = (r[i] - mean) / sd;
}

}  // namespace rlk
using namespace rlk;

RLK_API int rlk_grpo_loss(const float* logp, const float* old_logp, const float* ref_logp,
                          const float* adv, const unsigned char* mask, float* loss_tok,
                          float* kl_tok, float* ratio_tok, float* dlogp, float* seq_sums,
                          float* totals, int B, int L, float clip_eps_lo, float clip_eps_hi,
                          float beta, float inv_norm, void* stream) {
  RLK_REQUIRE(B > 0 && L > 0, "grpo_loss: empty batch");
  RLK_REQUIRE(seq_sums != nullptr, "grpo_loss: seq_sums scratch [B,4] is required");
  GrpoParams p{logp, old_logp, ref_logp, adv, mask, loss_tok, kl_tok, ratio_tok, dlogp, seq_sums,
               B, L, 1.f - clip_eps_lo, 1.f + clip_eps_hi, beta, inv_norm};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  grpo_token_kernel<<<(B + 7) / 8, 256, 0, s>>>(p);
  RLK_CHECK_CUDA(cudaGetLastError());
  if (totals) {
    grpo_total_kernel<<<1, 32, 0, s>>>(seq_sums, B, beta, totals);
    RLK_CHECK_CUDA(cudaGetLastError());
  }
  return RLK_OK;
}

RLK_API int rlk_group_advantages(const float* rewards, float* adv, int groups, int n, float eps,
                                 void* stream) {
  RLK_REQUIRE(groups > 0 && n > 0, "group_advantages: empty");
  group_adv_kernel<<<(groups + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(rewards, adv, groups, n, eps);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
