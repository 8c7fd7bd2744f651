// RMSNorm forward / backward (optionally fused with the residual add) and the fused
// per-head QK-RMSNorm + NeoX RoPE used on attention inputs.
//
// Reduction contract (depends on the row width only, never on the number of rows):
//   forward: 128 threads own one row; thread t reads the 16-byte chunks t, t+128, ... and adds their
//   squares to a private fp32 sum in ascending element order; each warp folds its 32 sums with the
//   xor butterfly 16,8,4,2,1 and the four warp sums are combined as (w0+w1)+(w2+w3).
//   y = bf16( x * rstd * w ) with all factors fp32 ("multiply in fp32, round once").
//   (backward and the 128-wide head norm use one warp per row with the same butterfly.)
// Weight gradients are reduced in two fixed stages: each CTA sums its 32 rows in ascending order
// (in registers) into a partial row of a scratch buffer, then a second kernel adds the partial
// rows in ascending order.
//
// Covers csrc/cuda/norm/rmsnorm.cu:81-244 and csrc/cuda/rope/rope_sm90.cu:24-102 of the
// reference, plus the QK-norm preprocessing of rl_engine/ops/attention/preprocess.py:180-345.
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

__device__ __forceinline__ float warp_sum_xor(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int kNormWarps = 8;

// y = rmsnorm(x [+ res]) * w ; optionally writes the summed residual stream and rstd.
// One CTA of 128 threads per row: thread t owns the 16-byte chunks t, t+128, ... (kept in
// registers between the two passes when the row has at most 8 chunks per thread).
constexpr int kRowThreads = 128;
constexpr int kMaxChunks = 8;

// NCH > 1: `x` holds NCH canonical K-chunk partial results (leaves) of a row-parallel GEMM,
// chunk_stride elements apart; the balanced bf16 tree over them (the GEMM's own chunk tree:
// node = bf16(fp32 a + fp32 b)) is evaluated while loading, so the separate tree pass and its
// round trip through memory disappear.
template <bool HAS_RES, int NCH>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int rows,
                   int H, float eps, long long chunk_stride) {
  griddep_sync();
  __shared__ float swarp[4];
  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * H);
  const uint4* rr = HAS_RES ? reinterpret_cast<const uint4*>(res + static_cast<long long>(row) * H) : nullptr;
  uint4* ro = HAS_RES ? reinterpret_cast<uint4*>(res_out + static_cast<long long>(row) * H) : nullptr;
  const int nchunk = H / 8;
  uint4 keep[kMaxChunks];
  float ss = 0.f;
  auto load_chunk = [&](int c) -> uint4 {
    uint4 v = xr[c];
    if (NCH > 1) {
      uint4 leaf[NCH > 1 ? NCH : 1];
      leaf[0] = v;
#pragma unroll
      for (int k = 1; k < NCH; ++k)
        leaf[k] = *reinterpret_cast<const uint4*>(x + k * chunk_stride + static_cast<long long>(row) * H + c * 8);
#pragma unroll
      for (int n = NCH; n > 1; n >>= 1)
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
          const uint4 a = leaf[2 * i], b = leaf[2 * i + 1];
          leaf[i].x = pack_bf16x2(__fadd_rn(bf16_lo(a.x), bf16_lo(b.x)), __fadd_rn(bf16_hi(a.x), bf16_hi(b.x)));
          leaf[i].y = pack_bf16x2(__fadd_rn(bf16_lo(a.y), bf16_lo(b.y)), __fadd_rn(bf16_hi(a.y), bf16_hi(b.y)));
          leaf[i].z = pack_bf16x2(__fadd_rn(bf16_lo(a.z), bf16_lo(b.z)), __fadd_rn(bf16_hi(a.z), bf16_hi(b.z)));
          leaf[i].w = pack_bf16x2(__fadd_rn(bf16_lo(a.w), bf16_lo(b.w)), __fadd_rn(bf16_hi(a.w), bf16_hi(b.w)));
        }
      v = leaf[0];
    }
    if (HAS_RES) {
      const uint4 q = rr[c];
      v.x = pack_bf16x2(bf16_lo(v.x) + bf16_lo(q.x), bf16_hi(v.x) + bf16_hi(q.x));
      v.y = pack_bf16x2(bf16_lo(v.y) + bf16_lo(q.y), bf16_hi(v.y) + bf16_hi(q.y));
      v.z = pack_bf16x2(bf16_lo(v.z) + bf16_lo(q.z), bf16_hi(v.z) + bf16_hi(q.z));
      v.w = pack_bf16x2(bf16_lo(v.w) + bf16_lo(q.w), bf16_hi(v.w) + bf16_hi(q.w));
      ro[c] = v;
    }
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = bf16_lo(u[i]), b = bf16_hi(u[i]);
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
    return v;
  };
#pragma unroll
  for (int i = 0; i < kMaxChunks; ++i) {
    const int c = tid + i * kRowThreads;
    if (c < nchunk) keep[i] = load_chunk(c);
  }
  for (int c = tid + kMaxChunks * kRowThreads; c < nchunk; c += kRowThreads) load_chunk(c);
  ss = warp_sum_xor(ss);
  if ((tid & 31) == 0) swarp[tid >> 5] = ss;
  __syncthreads();
  ss = (swarp[0] + swarp[1]) + (swarp[2] + swarp[3]);
  const float rstd = rsqrtf(ss / static_cast<float>(H) + eps);
  if (rstd_out && tid == 0) rstd_out[row] = rstd;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<long long>(row) * H);
  const uint4* src = HAS_RES ? reinterpret_cast<const uint4*>(ro) : xr;
  auto store_chunk = [&](int c, const uint4 v) {
    const uint4 g = wr[c];
    uint4 o;
    o.x = pack_bf16x2(bf16_lo(v.x) * rstd * bf16_lo(g.x), bf16_hi(v.x) * rstd * bf16_hi(g.x));
    o.y = pack_bf16x2(bf16_lo(v.y) * rstd * bf16_lo(g.y), bf16_hi(v.y) * rstd * bf16_hi(g.y));
    o.z = pack_bf16x2(bf16_lo(v.z) * rstd * bf16_lo(g.z), bf16_hi(v.z) * rstd * bf16_hi(g.z));
    o.w = pack_bf16x2(bf16_lo(v.w) * rstd * bf16_lo(g.w), bf16_hi(v.w) * rstd * bf16_hi(g.w));
    yr[c] = o;
  };
#pragma unroll
  for (int i = 0; i < kMaxChunks; ++i) {
    const int c = tid + i * kRowThreads;
    if (c < nchunk) store_chunk(c, keep[i]);
  }
  for (int c = tid + kMaxChunks * kRowThreads; c < nchunk; c += kRowThreads) store_chunk(c, src[c]);
}

// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) [+ dres];  partial dw[cta] = sum_rows dy * xhat.
// One CTA of 128 threads walks `rows_per_cta` consecutive rows; thread t owns the 16-byte chunks
// t, t+128, ... of every row, so its slice of the weight gradient accumulates in registers in
// ascending row order -- no shared-memory traffic, fixed order.
constexpr int kBwdRowsPerCta = 32;

__global__ void __launch_bounds__(kRowThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ dres,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int rows, int H,
                   float eps) {
  __shared__ float red[2][4];
  const int tid = threadIdx.x;
  const int nchunk = H / 8;
  const int r0 = blockIdx.x * kBwdRowsPerCta;
  const int r1 = min(rows, r0 + kBwdRowsPerCta);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float dwacc[kMaxChunks][8];
#pragma unroll
  for (int i = 0; i < kMaxChunks; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  for (int row = r0; row < r1; ++row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + static_cast<long long>(row) * H);
    uint4 xv[kMaxChunks], gv[kMaxChunks], wv[kMaxChunks];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
      const int c = tid + i * kRowThreads;
      if (c < nchunk) {
        xv[i] = xr[c]; gv[i] = gr[c]; wv[i] = wr[c];
        const uint32_t u[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float a = bf16_lo(u[k]), b = bf16_hi(u[k]);
          ss = fmaf(a, a, ss);
          ss = fmaf(b, b, ss);
        }
      }
    }
    ss = warp_sum_xor(ss);
    if ((tid & 31) == 0) red[0][tid >> 5] = ss;
    __syncthreads();
    ss = (red[0][0] + red[0][1]) + (red[0][2] + red[0][3]);
    const float rstd = rsqrtf(ss / static_cast<float>(H) + eps);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
      const int c = tid + i * kRowThreads;
      if (c < nchunk) {
        const uint32_t xu[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w}, gu[4] = {gv[i].x, gv[i].y, gv[i].z, gv[i].w},
                       wu[4] = {wv[i].x, wv[i].y, wv[i].z, wv[i].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          dot = fmaf(bf16_lo(wu[k]) * bf16_lo(gu[k]), bf16_lo(xu[k]) * rstd, dot);
          dot = fmaf(bf16_hi(wu[k]) * bf16_hi(gu[k]), bf16_hi(xu[k]) * rstd, dot);
        }
      }
    }
    dot = warp_sum_xor(dot);
    if ((tid & 31) == 0) red[1][tid >> 5] = dot;
    __syncthreads();
    dot = ((red[1][0] + red[1][1]) + (red[1][2] + red[1][3])) / static_cast<float>(H);
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<long long>(row) * H);
    const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + static_cast<long long>(row) * H) : nullptr;
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
      const int c = tid + i * kRowThreads;
      if (c < nchunk) {
        uint4 dr = make_uint4(0, 0, 0, 0);
        if (drr) dr = drr[c];
        const uint32_t xu[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w}, gu[4] = {gv[i].x, gv[i].y, gv[i].z, gv[i].w},
                       wu[4] = {wv[i].x, wv[i].y, wv[i].z, wv[i].w}, du[4] = {dr.x, dr.y, dr.z, dr.w};
        uint32_t ov[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float xh0 = bf16_lo(xu[k]) * rstd, xh1 = bf16_hi(xu[k]) * rstd;
          const float g0 = bf16_lo(gu[k]), g1 = bf16_hi(gu[k]);
          ov[k] = pack_bf16x2(rstd * (bf16_lo(wu[k]) * g0 - xh0 * dot) + bf16_lo(du[k]),
                              rstd * (bf16_hi(wu[k]) * g1 - xh1 * dot) + bf16_hi(du[k]));
          dwacc[i][2 * k] += g0 * xh0;
          dwacc[i][2 * k + 1] += g1 * xh1;
        }
        dxr[c] = make_uint4(ov[0], ov[1], ov[2], ov[3]);
      }
    }
    __syncthreads();   // red[] is reused by the next row
  }
  float* out = dw_partial + static_cast<long long>(blockIdx.x) * H;
#pragma unroll
  for (int i = 0; i < kMaxChunks; ++i) {
    const int c = tid + i * kRowThreads;
    if (c < nchunk) {
      *reinterpret_cast<float4*>(out + c * 8) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      *reinterpret_cast<float4*>(out + c * 8 + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// out[i] (+)= sum over partial rows in ascending order; output bf16 or fp32.
__global__ void reduce_partials_kernel(const float* __restrict__ partial, int nparts, int H,
                                       __nv_bfloat16* out_bf16, float* out_f32, int accumulate) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= H) return;
  float s = 0.f;
  for (int k = 0; k < nparts; ++k) s += partial[static_cast<long long>(k) * H + i];
  if (out_f32) out_f32[i] = accumulate ? out_f32[i] + s : s;
  if (out_bf16) out_bf16[i] = __float2bfloat16_rn(accumulate ? __bfloat162float(out_bf16[i]) + s : s);
}

// ------------------------------------------------------------------ QK-norm + RoPE (head_dim 128)
// One warp per (token, head). Lane l owns elements 2l, 2l+1 and their rotate-half partners
// 64+2l, 64+2l+1.  The fused QKV activation is GQA-group-major: for every KV head g the columns
// hold [G query heads of the group | key head g | value head g], G = Hq / Hkv.  A tensor-parallel
// rank owns whole groups, so the layout (and every reduction over it) is the same for any TP.
// Destination rows: q -> q_out[t], k/v -> k_out/v_out[kv_slot ? kv_slot[t] : t].
struct QkRopeParams {
  const __nv_bfloat16* qkv; long long ld_qkv;
  const __nv_bfloat16* q_w; const __nv_bfloat16* k_w;
  const float* cos_tab; const float* sin_tab;   // [max_pos][64]
  const int* pos;                               // [T]
  const int* kv_slot;                           // [T] or null
  __nv_bfloat16* q_out; long long ld_q;
  __nv_bfloat16* k_out; __nv_bfloat16* v_out; long long ld_kv;
  int T, Hq, Hkv; float eps;
  float* q_rstd; float* k_rstd;                 // optional [T,Hq] / [T,Hkv] (saved for backward)
};

__global__ void __launch_bounds__(256) qk_norm_rope_fwd_kernel(const QkRopeParams p) {
  griddep_sync();
  const int lane = threadIdx.x & 31;
  const int gw = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int heads = p.Hq + 2 * p.Hkv;
  if (gw >= p.T * heads) return;
  const int t = gw / heads, hh = gw - t * heads;
  const int G = p.Hq / p.Hkv;
  const int grp = hh / (G + 2), jj = hh - grp * (G + 2);
  // logical head index in the "all q | all k | all v" numbering used below
  const int h = jj < G ? grp * G + jj : (jj == G ? p.Hq + grp : p.Hq + p.Hkv + grp);
  const __nv_bfloat16* src = p.qkv + static_cast<long long>(t) * p.ld_qkv + hh * 128;
  const uint32_t lo = *reinterpret_cast<const uint32_t*>(src + 2 * lane);
  const uint32_t hi = *reinterpret_cast<const uint32_t*>(src + 64 + 2 * lane);
  if (h >= p.Hq + p.Hkv) {  // value head: plain copy into the cache / output
    const long long dr = p.kv_slot ? p.kv_slot[t] : t;
    if (dr < 0) return;
    __nv_bfloat16* dst = p.v_out + dr * p.ld_kv + (h - p.Hq - p.Hkv) * 128;
    *reinterpret_cast<uint32_t*>(dst + 2 * lane) = lo;
    *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = hi;
    return;
  }
  const bool is_q = h < p.Hq;
  const float a0 = bf16_lo(lo), a1 = bf16_hi(lo), b0 = bf16_lo(hi), b1 = bf16_hi(hi);
  float ss = fmaf(a0, a0, 0.f);
  ss = fmaf(a1, a1, ss);
  ss = fmaf(b0, b0, ss);
  ss = fmaf(b1, b1, ss);
  ss = warp_sum_xor(ss);
  const float rstd = rsqrtf(ss * (1.f / 128.f) + p.eps);
  const __nv_bfloat16* w = is_q ? p.q_w : p.k_w;
  const uint32_t wlo = *reinterpret_cast<const uint32_t*>(w + 2 * lane);
  const uint32_t whi = *reinterpret_cast<const uint32_t*>(w + 64 + 2 * lane);
  const float n_a0 = a0 * rstd * bf16_lo(wlo), n_a1 = a1 * rstd * bf16_hi(wlo);
  const float n_b0 = b0 * rstd * bf16_lo(whi), n_b1 = b1 * rstd * bf16_hi(whi);
  const int ps = p.pos[t];
  const float2 c = *reinterpret_cast<const float2*>(p.cos_tab + static_cast<long long>(ps) * 64 + 2 * lane);
  const float2 s = *reinterpret_cast<const float2*>(p.sin_tab + static_cast<long long>(ps) * 64 + 2 * lane);
  const float o_a0 = n_a0 * c.x - n_b0 * s.x, o_a1 = n_a1 * c.y - n_b1 * s.y;
  const float o_b0 = n_b0 * c.x + n_a0 * s.x, o_b1 = n_b1 * c.y + n_a1 * s.y;
  __nv_bfloat16* dst;
  if (is_q) {
    dst = p.q_out + static_cast<long long>(t) * p.ld_q + h * 128;
    if (p.q_rstd && lane == 0) p.q_rstd[static_cast<long long>(t) * p.Hq + h] = rstd;
  } else {
    const long long dr = p.kv_slot ? p.kv_slot[t] : t;
    if (p.k_rstd && lane == 0) p.k_rstd[static_cast<long long>(t) * p.Hkv + (h - p.Hq)] = rstd;
    if (dr < 0) return;
    dst = p.k_out + dr * p.ld_kv + (h - p.Hq) * 128;
  }
  *reinterpret_cast<uint32_t*>(dst + 2 * lane) = pack_bf16x2(o_a0, o_a1);
  *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = pack_bf16x2(o_b0, o_b1);
}

// Backward of the fused op: rotate the incoming gradient back, then RMSNorm backward over the
// 128-wide head.  Writes d(qkv) [T, ld_qkv] (values: copy of dv) and per-CTA partial weight
// gradients for q_norm / k_norm: partial[cta][0..127] (q), partial[cta][128..255] (k).
struct QkRopeBwdParams {
  const __nv_bfloat16* qkv; long long ld_qkv;   // forward input (pre-norm)
  const __nv_bfloat16* q_w; const __nv_bfloat16* k_w;
  const float* cos_tab; const float* sin_tab; const int* pos;
  const __nv_bfloat16* dq; long long ld_dq;
  const __nv_bfloat16* dk; const __nv_bfloat16* dv; long long ld_dkv;
  __nv_bfloat16* dqkv; long long ld_dqkv;
  float* partial;  // [gridDim.x][256], or [gridDim.x][Hkv][256] with per_group
  int T, Hq, Hkv; float eps; int tokens_per_cta;
  int per_group;   // 1: one partial row per KV group (its G query heads and its key head): the sums do
                   //    not depend on how many groups a tensor-parallel rank holds
};

__global__ void __launch_bounds__(256) qk_norm_rope_bwd_kernel(const QkRopeBwdParams p) {
  __shared__ float sw[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = lane; i < 256; i += 32) sw[warp][i] = 0.f;
  __syncwarp();
  const int heads = p.Hq + 2 * p.Hkv;
  const int t0 = blockIdx.x * p.tokens_per_cta;
  const int t1 = min(p.T, t0 + p.tokens_per_cta);
  const int G = p.Hq / p.Hkv;
  // per_group: the CTA walks the KV groups one after the other and every group's items go to the
  // warps in the same way whatever the number of groups; else one pass over all heads
  const int n_pass = p.per_group ? p.Hkv : 1;
  const int heads_pass = p.per_group ? G + 2 : heads;
  const int items = (t1 - t0) * heads_pass;
  for (int pass = 0; pass < n_pass; ++pass) {
  if (pass > 0) {
    __syncthreads();
    for (int i = lane; i < 256; i += 32) sw[warp][i] = 0.f;
    __syncwarp();
  }
  for (int it = warp; it < items; it += 8) {
    const int t = t0 + it / heads_pass, hh = pass * heads_pass + it % heads_pass;
    const int grp = hh / (G + 2), jj = hh - grp * (G + 2);
    const int h = jj < G ? grp * G + jj : (jj == G ? p.Hq + grp : p.Hq + p.Hkv + grp);
    __nv_bfloat16* dst = p.dqkv + static_cast<long long>(t) * p.ld_dqkv + hh * 128;
    if (h >= p.Hq + p.Hkv) {
      const __nv_bfloat16* g = p.dv + static_cast<long long>(t) * p.ld_dkv + (h - p.Hq - p.Hkv) * 128;
      *reinterpret_cast<uint32_t*>(dst + 2 * lane) = *reinterpret_cast<const uint32_t*>(g + 2 * lane);
      *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = *reinterpret_cast<const uint32_t*>(g + 64 + 2 * lane);
      continue;
    }
    const bool is_q = h < p.Hq;
    const __nv_bfloat16* g = is_q ? p.dq + static_cast<long long>(t) * p.ld_dq + h * 128
                                  : p.dk + static_cast<long long>(t) * p.ld_dkv + (h - p.Hq) * 128;
    const uint32_t glo = *reinterpret_cast<const uint32_t*>(g + 2 * lane);
    const uint32_t ghi = *reinterpret_cast<const uint32_t*>(g + 64 + 2 * lane);
    const int ps = p.pos[t];
    const float2 c = *reinterpret_cast<const float2*>(p.cos_tab + static_cast<long long>(ps) * 64 + 2 * lane);
    const float2 s = *reinterpret_cast<const float2*>(p.sin_tab + static_cast<long long>(ps) * 64 + 2 * lane);
    // transpose of the rotation
    const float ga0 = bf16_lo(glo), ga1 = bf16_hi(glo), gb0 = bf16_lo(ghi), gb1 = bf16_hi(ghi);
    const float dn_a0 = ga0 * c.x + gb0 * s.x, dn_a1 = ga1 * c.y + gb1 * s.y;
    const float dn_b0 = gb0 * c.x - ga0 * s.x, dn_b1 = gb1 * c.y - ga1 * s.y;
    const __nv_bfloat16* src = p.qkv + static_cast<long long>(t) * p.ld_qkv + hh * 128;
    const uint32_t lo = *reinterpret_cast<const uint32_t*>(src + 2 * lane);
    const uint32_t hi = *reinterpret_cast<const uint32_t*>(src + 64 + 2 * lane);
    const float a0 = bf16_lo(lo), a1 = bf16_hi(lo), b0 = bf16_lo(hi), b1 = bf16_hi(hi);
    float ss = fmaf(a0, a0, 0.f);
    ss = fmaf(a1, a1, ss);
    ss = fmaf(b0, b0, ss);
    ss = fmaf(b1, b1, ss);
    ss = warp_sum_xor(ss);
    const float rstd = rsqrtf(ss * (1.f / 128.f) + p.eps);
    const __nv_bfloat16* w = is_q ? p.q_w : p.k_w;
    const uint32_t wlo = *reinterpret_cast<const uint32_t*>(w + 2 * lane);
    const uint32_t whi = *reinterpret_cast<const uint32_t*>(w + 64 + 2 * lane);
    const float xa0 = a0 * rstd, xa1 = a1 * rstd, xb0 = b0 * rstd, xb1 = b1 * rstd;
    const float wa0 = bf16_lo(wlo), wa1 = bf16_hi(wlo), wb0 = bf16_lo(whi), wb1 = bf16_hi(whi);
    float dot = (wa0 * dn_a0) * xa0;
    dot = fmaf(wa1 * dn_a1, xa1, dot);
    dot = fmaf(wb0 * dn_b0, xb0, dot);
    dot = fmaf(wb1 * dn_b1, xb1, dot);
    dot = warp_sum_xor(dot) * (1.f / 128.f);
    *reinterpret_cast<uint32_t*>(dst + 2 * lane) =
        pack_bf16x2(rstd * (wa0 * dn_a0 - xa0 * dot), rstd * (wa1 * dn_a1 - xa1 * dot));
    *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) =
        pack_bf16x2(rstd * (wb0 * dn_b0 - xb0 * dot), rstd * (wb1 * dn_b1 - xb1 * dot));
    float* acc = &sw[warp][is_q ? 0 : 128];
    acc[2 * lane] += dn_a0 * xa0;
    acc[2 * lane + 1] += dn_a1 * xa1;
    acc[64 + 2 * lane] += dn_b0 * xb0;
    acc[64 + 2 * lane + 1] += dn_b1 * xb1;
  }
  __syncthreads();
  {
    const int i = threadIdx.x;  // 256 threads, 256 partial entries
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += sw[k][i];
    p.partial[(static_cast<long long>(blockIdx.x) * n_pass + pass) * 256 + i] = s;
  }
  }
}

// Canonical q_norm / k_norm weight gradients: per KV group, the per-CTA partials are summed in
// ascending CTA order (fp32) and rounded to bf16 -- a leaf; the leaves of the `ngroups` groups this
// rank holds are combined by a balanced tree with a bf16 rounding at every node.  A tensor-parallel
// rank therefore produces exactly the sub-tree that the fixed-order all-reduce continues, and one
// rank holding all groups reproduces the bits of 2, 4 or 8 ranks.  out[256] = [q_norm | k_norm];
// accumulate: out = bf16(float(out) + node).
__global__ void __launch_bounds__(256) qk_dw_group_tree_kernel(const float* __restrict__ partial, int ncta, int ngroups,
                                                               __nv_bfloat16* out, int accumulate) {
  const int i = threadIdx.x;
  float leaf[8];
  for (int g = 0; g < ngroups; ++g) {
    float s = 0.f;
    for (int c = 0; c < ncta; ++c) s += partial[(static_cast<long long>(c) * ngroups + g) * 256 + i];
    leaf[g] = round_bf16(s);
  }
  for (int n = ngroups; n > 1; n >>= 1)
    for (int j = 0; j < n / 2; ++j) leaf[j] = round_bf16(__fadd_rn(leaf[2 * j], leaf[2 * j + 1]));
  out[i] = __float2bfloat16_rn(accumulate ? __fadd_rn(__bfloat162float(out[i]), leaf[0]) : leaf[0]);
}

}  // namespace rlk

using namespace rlk;

RLK_API int rlk_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out,
                            float* rstd_out, int rows, int H, float eps, void* stream) {
  RLK_REQUIRE(rows > 0 && H > 0 && H % 8 == 0, "rmsnorm: H must be a positive multiple of 8");
  RLK_REQUIRE(!res || res_out, "rmsnorm: residual input needs res_out");
  const int grid = rows;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (res)
    RLK_CHECK_CUDA(launch_pdl(rmsnorm_fwd_kernel<true, 1>, dim3(grid), dim3(kRowThreads), 0, s,
                              (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,
                              (__nv_bfloat16*)y, (__nv_bfloat16*)res_out, rstd_out, rows, H, eps, 0ll));
  else
    RLK_CHECK_CUDA(launch_pdl(rmsnorm_fwd_kernel<false, 1>, dim3(grid), dim3(kRowThreads), 0, s,
                              (const __nv_bfloat16*)x, (const __nv_bfloat16*)nullptr, (const __nv_bfloat16*)w,
                              (__nv_bfloat16*)y, (__nv_bfloat16*)nullptr, rstd_out, rows, H, eps, 0ll));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// y = rmsnorm(tree(leaves) + res) * w where `leaves` holds nchunks (2, 4 or 8) partial results of a
// row-parallel GEMM, each [rows, H] and chunk_stride elements apart (rlk_det_gemm_split_leaves);
// res_out receives tree(leaves) + res.  Bitwise the result of the tree pass followed by
// rlk_rmsnorm_fwd.
RLK_API int rlk_rmsnorm_fwd_leaves(const void* leaves, long long chunk_stride, int nchunks, const void* res,
                                   const void* w, void* y, void* res_out, int rows, int H, float eps,
                                   void* stream) {
  RLK_REQUIRE(rows > 0 && H > 0 && H % 8 == 0, "rmsnorm_fwd_leaves: H must be a positive multiple of 8");
  RLK_REQUIRE(res && res_out, "rmsnorm_fwd_leaves: residual input and output are required");
  RLK_REQUIRE(nchunks == 2 || nchunks == 4 || nchunks == 8, "rmsnorm_fwd_leaves: nchunks must be 2, 4 or 8");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define RLK_RMS_LEAVES(N_)                                                                                    \
  RLK_CHECK_CUDA(launch_pdl(rmsnorm_fwd_kernel<true, N_>, dim3(rows), dim3(kRowThreads), 0, s,               \
                            (const __nv_bfloat16*)leaves, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, \
                            (__nv_bfloat16*)y, (__nv_bfloat16*)res_out, (float*)nullptr, rows, H, eps, chunk_stride))
  if (nchunks == 2) RLK_RMS_LEAVES(2);
  else if (nchunks == 4) RLK_RMS_LEAVES(4);
  else RLK_RMS_LEAVES(8);
#undef RLK_RMS_LEAVES
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// Number of fp32 elements of scratch that rlk_rmsnorm_bwd needs for `rows` x `H`.
RLK_API long long rlk_rmsnorm_bwd_scratch_elems(int rows, int H) {
  return static_cast<long long>((rows + kBwdRowsPerCta - 1) / kBwdRowsPerCta) * H;
}

// dx = d/dx [ rmsnorm(x) * w ] (+ dres); dw (bf16 or fp32, optionally accumulated) in fixed order.
RLK_API int rlk_rmsnorm_bwd(const void* x, const void* w, const void* dy, const void* dres,
                            void* dx, float* scratch, void* dw_bf16, float* dw_f32,
                            int accumulate_dw, int rows, int H, float eps, void* stream) {
  RLK_REQUIRE(rows > 0 && H > 0 && H % 8 == 0 && H <= kRowThreads * kMaxChunks * 8,
              "rmsnorm_bwd: H must be a multiple of 8, <= 8192");
  const int grid = (rows + kBwdRowsPerCta - 1) / kBwdRowsPerCta;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  rmsnorm_bwd_kernel<<<grid, kRowThreads, 0, s>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy,
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, scratch, rows, H, eps);
  RLK_CHECK_CUDA(cudaGetLastError());
  reduce_partials_kernel<<<(H + 255) / 256, 256, 0, s>>>(scratch, grid, H, (__nv_bfloat16*)dw_bf16,
                                                         dw_f32, accumulate_dw);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_qk_norm_rope_fwd(const void* qkv, long long ld_qkv, const void* q_w, const void* k_w,
                                 const float* cos_tab, const float* sin_tab, const int* pos,
                                 const int* kv_slot, void* q_out, long long ld_q, void* k_out,
                                 void* v_out, long long ld_kv, int T, int Hq, int Hkv, float eps,
                                 float* q_rstd, float* k_rstd, void* stream) {
  RLK_REQUIRE(T > 0 && Hq > 0 && Hkv > 0, "qk_norm_rope: empty shape");
  QkRopeParams p{(const __nv_bfloat16*)qkv, ld_qkv, (const __nv_bfloat16*)q_w,
                 (const __nv_bfloat16*)k_w, cos_tab, sin_tab, pos, kv_slot,
                 (__nv_bfloat16*)q_out, ld_q, (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, ld_kv,
                 T, Hq, Hkv, eps, q_rstd, k_rstd};
  const long long warps = static_cast<long long>(T) * (Hq + 2 * Hkv);
  RLK_CHECK_CUDA(launch_pdl(qk_norm_rope_fwd_kernel, dim3(static_cast<unsigned>((warps + 7) / 8)), dim3(256), 0,
                            static_cast<cudaStream_t>(stream), p));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API long long rlk_qk_norm_rope_bwd_scratch_elems(int T) {
  return static_cast<long long>((T + 15) / 16 + 1) * 256 * 8;    // room for one partial row per KV group (<= 8)
}

// Same backward with canonical weight gradients (see qk_dw_group_tree_kernel): dqk_bf16[256] =
// [d q_norm | d k_norm] of the Hkv KV groups this rank holds (a power of two, at most 8).
// accumulate_dw = 1 adds into dqk_bf16 (single rank); a tensor-parallel caller passes 0, all-reduces
// the 256 values over the ranks (fixed tree) and accumulates afterwards.
RLK_API int rlk_qk_norm_rope_bwd_canonical(const void* qkv, long long ld_qkv, const void* q_w, const void* k_w,
                                           const float* cos_tab, const float* sin_tab, const int* pos,
                                           const void* dq, long long ld_dq, const void* dk, const void* dv,
                                           long long ld_dkv, void* dqkv, long long ld_dqkv, float* scratch,
                                           void* dqk_bf16, int accumulate_dw, int T, int Hq, int Hkv, float eps,
                                           void* stream) {
  RLK_REQUIRE(T > 0, "qk_norm_rope_bwd: empty shape");
  RLK_REQUIRE(Hkv == 1 || Hkv == 2 || Hkv == 4 || Hkv == 8, "qk_norm_rope_bwd_canonical: 1, 2, 4 or 8 KV groups per rank (got %d)", Hkv);
  const int tokens_per_cta = 16;
  const int grid = (T + tokens_per_cta - 1) / tokens_per_cta;
  QkRopeBwdParams p{(const __nv_bfloat16*)qkv, ld_qkv, (const __nv_bfloat16*)q_w,
                    (const __nv_bfloat16*)k_w, cos_tab, sin_tab, pos, (const __nv_bfloat16*)dq,
                    ld_dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)dv, ld_dkv,
                    (__nv_bfloat16*)dqkv, ld_dqkv, scratch, T, Hq, Hkv, eps, tokens_per_cta, 1};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  qk_norm_rope_bwd_kernel<<<grid, 256, 0, s>>>(p);
  RLK_CHECK_CUDA(cudaGetLastError());
  qk_dw_group_tree_kernel<<<1, 256, 0, s>>>(scratch, grid, Hkv, (__nv_bfloat16*)dqk_bf16, accumulate_dw);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_qk_norm_rope_bwd(const void* qkv, long long ld_qkv, const void* q_w, const void* k_w,
                                 const float* cos_tab, const float* sin_tab, const int* pos,
                                 const void* dq, long long ld_dq, const void* dk, const void* dv,
                                 long long ld_dkv, void* dqkv, long long ld_dqkv, float* scratch,
                                 void* dqw_bf16, void* dkw_bf16, int accumulate_dw, int T, int Hq,
                                 int Hkv, float eps, void* stream) {
  RLK_REQUIRE(T > 0, "qk_norm_rope_bwd: empty shape");
  const int tokens_per_cta = 16;
  const int grid = (T + tokens_per_cta - 1) / tokens_per_cta;
  QkRopeBwdParams p{(const __nv_bfloat16*)qkv, ld_qkv, (const __nv_bfloat16*)q_w,
                    (const __nv_bfloat16*)k_w, cos_tab, sin_tab, pos, (const __nv_bfloat16*)dq,
                    ld_dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)dv, ld_dkv,
                    (__nv_bfloat16*)dqkv, ld_dqkv, scratch, T, Hq, Hkv, eps, tokens_per_cta, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  qk_norm_rope_bwd_kernel<<<grid, 256, 0, s>>>(p);
  RLK_CHECK_CUDA(cudaGetLastError());
  // partial rows are [grid][256]: first 128 columns = q_norm grad, last 128 = k_norm grad
  reduce_partials_kernel<<<1, 256, 0, s>>>(scratch, grid, 256, nullptr, scratch + static_cast<long long>(grid) * 256, 0);
  RLK_CHECK_CUDA(cudaGetLastError());
  // tiny epilogue: convert the reduced fp32 row into the two bf16 weight gradients
  reduce_partials_kernel<<<1, 128, 0, s>>>(scratch + static_cast<long long>(grid) * 256, 1, 128,
                                           (__nv_bfloat16*)dqw_bf16, nullptr, accumulate_dw);
  reduce_partials_kernel<<<1, 128, 0, s>>>(scratch + static_cast<long long>(grid) * 256 + 128, 1, 128,
                                           (__nv_bfloat16*)dkw_bf16, nullptr, accumulate_dw);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
