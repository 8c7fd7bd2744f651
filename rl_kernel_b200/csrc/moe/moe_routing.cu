// Mixture-of-experts routing for sm_100a: softmax top-k router (forward and backward), the
// deterministic dispatch plan, and the expert all-to-all as plain peer stores (dispatch) and peer
// loads (combine) over NVLink from inside the kernels.
//
// Contract (what makes the layer reproducible and independent of batch and expert-parallel size):
//   * router: fp32 softmax over all experts, top-k by probability with ties going to the lower
//     expert id, weights renormalised over the selected experts; a token's selected experts are
//     kept in ascending expert id and every per-token sum runs in that order;
//   * dispatch: expert e's rows are ordered by (source rank, token index, k) -- a pure function
//     of the routing, obtained from integer counts (order-free) and a stable ranking;
//   * expert GEMMs never mix rows (grouped_gemm_sm100.cu), so where a row sits does not matter;
//   * combine: out[t] = bf16(fma(w_K-1, y_K-1, ... fma(w_0, y_0, base[t]))), experts ascending.
// The reference only reserves the package names for this (rl_engine/ops/moe/__init__.py and
// docs/blog/2026-08-09-dsv4-flash-moe-consistency-roadmap.md:120-134 list it as roadmap).
#include "rlk/host.h"
#include "rlk/moe.h"
#include "rlk/ptx.cuh"

namespace rlk {

__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// ------------------------------------------------------------------------------------ router
template <int PER>  // experts per lane; E = 32 * PER
__global__ void __launch_bounds__(256)
moe_router_topk_kernel(const float* __restrict__ logits, int T, int K, int* __restrict__ idx,
                       float* __restrict__ w, float* __restrict__ probs, int* __restrict__ counts) {
  constexpr int E = 32 * PER;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= T) return;
  float p[PER];
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    p[j] = logits[static_cast<long long>(t) * E + lane * PER + j];
    m = fmaxf(m, p[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    p[j] = expf(p[j] - m);
    s = __fadd_rn(s, p[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    p[j] = __fdiv_rn(p[j], s);
    if (probs) probs[static_cast<long long>(t) * E + lane * PER + j] = p[j];
  }
  uint32_t sel = 0;
  for (int k = 0; k < K; ++k) {
    float v = -1.f;
    int bi = E;
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (!((sel >> j) & 1) && p[j] > v) { v = p[j]; bi = lane * PER + j; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > v || (ov == v && oi < bi)) { v = ov; bi = oi; }
    }
    if (bi / PER == lane) sel |= 1u << (bi % PER);
  }
  float ssel = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j)
    if ((sel >> j) & 1) ssel = __fadd_rn(ssel, p[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ssel = __fadd_rn(ssel, __shfl_xor_sync(0xffffffffu, ssel, o));
  const int c = __popc(sel);
  int incl = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  const int prefix = incl - c;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    if ((sel >> j) & 1) {
      const int r = prefix + __popc(sel & ((1u << j) - 1u));
      const int e = lane * PER + j;
      idx[static_cast<long long>(t) * K + r] = e;
      w[static_cast<long long>(t) * K + r] = __fdiv_rn(p[j], ssel);
      if (counts) atomicAdd(&counts[e], 1);  // integer: exact in any order
    }
  }
}

// dlogits[t, idx_k] = w_k * (dw_k - sum_k' dw_k' w_k'), zero elsewhere (the renormalised top-k
// softmax is the softmax restricted to the selected experts).
__global__ void __launch_bounds__(256)
moe_router_bwd_kernel(const int* __restrict__ idx, const float* __restrict__ w, const float* __restrict__ dw,
                      int T, int K, int E, __nv_bfloat16* __restrict__ dlogits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= T) return;
  __nv_bfloat16* row = dlogits + static_cast<long long>(t) * E;
  for (int e = lane; e < E; e += 32) row[e] = __float2bfloat16_rn(0.f);
  __syncwarp();
  float c = 0.f;
  for (int k = 0; k < K; ++k) c = fmaf(dw[static_cast<long long>(t) * K + k], w[static_cast<long long>(t) * K + k], c);
  if (lane < K) {
    const long long j = static_cast<long long>(t) * K + lane;
    row[idx[j]] = __float2bfloat16_rn(w[j] * (dw[j] - c));
  }
}

// ------------------------------------------------------------------------------------ plan
// counts_all[s][e]: tokens rank s routes to expert e.  Expert e lives on rank e / E_loc; its rows
// there start at base[e] (experts of a rank back to back, each padded to 128 rows) and are ordered
// by source rank.  loc[el] = {base, total, padded, 0} for this rank's experts.
__global__ void __launch_bounds__(256)
moe_plan_kernel(const int* __restrict__ counts_all, int W, int rank, int E, int E_loc,
                int* __restrict__ send_row0, int* __restrict__ loc, int* __restrict__ rows_used) {
  __shared__ int padded_s[256];
  const int e = threadIdx.x;
  int total = 0, before = 0;
  if (e < E) {
    for (int s = 0; s < W; ++s) {
      const int c = counts_all[s * E + e];
      if (s < rank) before += c;
      total += c;
    }
    padded_s[e] = (total + 127) / 128 * 128;
  }
  __syncthreads();
  if (e < E) {
    const int owner = e / E_loc;
    int base = 0;
    for (int q = owner * E_loc; q < e; ++q) base += padded_s[q];
    send_row0[e] = base + before;
    if (owner == rank) {
      int* l = loc + (e - rank * E_loc) * 4;
      l[0] = base; l[1] = total; l[2] = padded_s[e]; l[3] = 0;
    }
  }
  if (e == 0) {
    int r = 0;
    for (int q = rank * E_loc; q < (rank + 1) * E_loc; ++q) r += padded_s[q];
    *rows_used = r;
  }
}

// kind 0: C[rows, n_cols] = A[rows, k_dim] x expert weights (rows = this rank's received rows);
//         b_mn = 0: B is [E_loc * n_cols, k_dim]; b_mn = 1: B is [E_loc * k_dim, n_cols].
// kind 1: dW[el] [m_out, n_cols] (+)= A_el^T B_el, contraction over expert el's rows.
__global__ void __launch_bounds__(128)
moe_tiles_kernel(const int* __restrict__ loc, int E_loc, int kind, int n_cols, int k_dim, int b_mn,
                 int m_out, GroupTile* __restrict__ tiles, int* __restrict__ n_tiles, int max_tiles) {
  __shared__ int off_s[129];
  const int el = threadIdx.x;
  const int nb_n = n_cols / 256;
  int mine = 0;
  if (el < E_loc) {
    const int padded = loc[el * 4 + 2];
    mine = kind == 0 ? (padded / 128) * nb_n : (padded > 0 ? (m_out / 128) * nb_n : 0);
  }
  off_s[el + 1] = mine;
  __syncthreads();
  if (el == 0) {
    off_s[0] = 0;
    for (int q = 0; q < E_loc; ++q) off_s[q + 1] += off_s[q];
    *n_tiles = off_s[E_loc] < max_tiles ? off_s[E_loc] : max_tiles;
  }
  __syncthreads();
  if (el >= E_loc) return;
  const int base = loc[el * 4 + 0], padded = loc[el * 4 + 2];
  int o = off_s[el];
  const int n_mb = kind == 0 ? padded / 128 : m_out / 128;
  for (int nb = 0; nb < nb_n; ++nb) {
    for (int mb = 0; mb < n_mb && mine > 0; ++mb, ++o) {
      if (o >= max_tiles) return;
      GroupTile g;
      if (kind == 0) {
        g.a_m0 = base + mb * 128;
        g.b_n0 = b_mn ? nb * 256 : el * n_cols + nb * 256;
        g.ka0 = 0;
        g.kb0 = b_mn ? el * k_dim : 0;
        g.kblocks = k_dim / 64;
        g.c_row = g.a_m0;
      } else {
        g.a_m0 = mb * 128;
        g.b_n0 = nb * 256;
        g.ka0 = base;
        g.kb0 = base;
        g.kblocks = padded / 64;
        g.c_row = el * m_out + mb * 128;
      }
      g.c_col = nb * 256;
      g.rows_valid = 128;
      tiles[o] = g;
    }
  }
}

// slot_row[j] = row in the owner's buffer of routed copy j = t * K + k: this rank's rows of expert
// e keep the order of j (stable ranking: CTA e counts the earlier copies routed to e).
__global__ void __launch_bounds__(256)
moe_slots_kernel(const int* __restrict__ idx, int n, const int* __restrict__ send_row0,
                 int* __restrict__ slot_row) {
  __shared__ int wcount[8];
  const int e = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = send_row0[e];
  int running = 0;
  for (int b = 0; b < n; b += 256) {
    const int j = b + threadIdx.x;
    const bool hit = j < n && idx[j] == e;
    const uint32_t bal = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) wcount[warp] = __popc(bal);
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (q < warp) before += wcount[q];
      all += wcount[q];
    }
    if (hit) slot_row[j] = row0 + running + before + __popc(bal & ((1u << lane) - 1u));
    running += all;
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------ all-to-all
// Push: routed copy j of token t = j / K goes to row slot_row[j] of the buffer of the rank that
// owns expert idx[j]; optional per-copy scale (the backward pushes w_j * dOut[t]).
__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const float* __restrict__ scale,
                    const int* __restrict__ idx, const int* __restrict__ slot_row, int n, int K, int E_loc,
                    int H, const PeerPtrs dst, long long ld_dst) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x * 8 + warp;
  if (j < n) {
    const int t = j / K;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * ldx);
    uint4* d = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(dst.p[idx[j] / E_loc]) +
                                        static_cast<long long>(slot_row[j]) * ld_dst);
    const float sc = scale ? scale[j] : 1.f;
    for (int v = lane; v < H / 8; v += 32) {
      uint4 q = src[v];
      if (scale) {
        q.x = pack_bf16x2(bf16_lo(q.x) * sc, bf16_hi(q.x) * sc);
        q.y = pack_bf16x2(bf16_lo(q.y) * sc, bf16_hi(q.y) * sc);
        q.z = pack_bf16x2(bf16_lo(q.z) * sc, bf16_hi(q.z) * sc);
        q.w = pack_bf16x2(bf16_lo(q.w) * sc, bf16_hi(q.w) * sc);
      }
      d[v] = q;
    }
  }
  __threadfence_system();
}

// Pull: out[t] = bf16(base[t] + sum_k w_k * Y[row_k]) accumulated with fma in ascending k (= ascending
// expert id), Y read from the owner's buffer.  w == null: unit weights (the backward's gather of dX).
__global__ void __launch_bounds__(128)
moe_combine_kernel(const __nv_bfloat16* __restrict__ base, long long ld_base, const float* __restrict__ w,
                   const int* __restrict__ idx, const int* __restrict__ slot_row, int T, int K, int E_loc,
                   int H, const PeerPtrs src, long long ld_src, __nv_bfloat16* __restrict__ out, long long ldo) {
  const int t = blockIdx.x;
  if (t >= T) return;
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
    float acc[8];
    if (base) {
      const uint4 b = *reinterpret_cast<const uint4*>(base + static_cast<long long>(t) * ld_base + v * 8);
      acc[0] = bf16_lo(b.x); acc[1] = bf16_hi(b.x); acc[2] = bf16_lo(b.y); acc[3] = bf16_hi(b.y);
      acc[4] = bf16_lo(b.z); acc[5] = bf16_hi(b.z); acc[6] = bf16_lo(b.w); acc[7] = bf16_hi(b.w);
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    }
    for (int k = 0; k < K; ++k) {
      const long long j = static_cast<long long>(t) * K + k;
      const __nv_bfloat16* y = static_cast<const __nv_bfloat16*>(src.p[idx[j] / E_loc]) +
                               static_cast<long long>(slot_row[j]) * ld_src + v * 8;
      const uint4 q = ld_sys_v4(y);
      const float wk = w ? w[j] : 1.f;
      acc[0] = fmaf(wk, bf16_lo(q.x), acc[0]); acc[1] = fmaf(wk, bf16_hi(q.x), acc[1]);
      acc[2] = fmaf(wk, bf16_lo(q.y), acc[2]); acc[3] = fmaf(wk, bf16_hi(q.y), acc[3]);
      acc[4] = fmaf(wk, bf16_lo(q.z), acc[4]); acc[5] = fmaf(wk, bf16_hi(q.z), acc[5]);
      acc[6] = fmaf(wk, bf16_lo(q.w), acc[6]); acc[7] = fmaf(wk, bf16_hi(q.w), acc[7]);
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * ldo + v * 8) = o;
  }
}

// dw[j] = <dOut[t], Y[row_j]> (gradient of the combine with respect to the routing weight).
__global__ void __launch_bounds__(256)
moe_combine_dw_kernel(const __nv_bfloat16* __restrict__ dout, long long ldd, const int* __restrict__ idx,
                      const int* __restrict__ slot_row, int n, int K, int E_loc, int H, const PeerPtrs src,
                      long long ld_src, float* __restrict__ dw) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x * 8 + warp;
  if (j >= n) return;
  const int t = j / K;
  const __nv_bfloat16* y = static_cast<const __nv_bfloat16*>(src.p[idx[j] / E_loc]) +
                           static_cast<long long>(slot_row[j]) * ld_src;
  const __nv_bfloat16* g = dout + static_cast<long long>(t) * ldd;
  float s = 0.f;
  for (int v = lane; v < H / 8; v += 32) {
    const uint4 a = ld_sys_v4(y + v * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(g + v * 8);
    s = fmaf(bf16_lo(a.x), bf16_lo(b.x), s); s = fmaf(bf16_hi(a.x), bf16_hi(b.x), s);
    s = fmaf(bf16_lo(a.y), bf16_lo(b.y), s); s = fmaf(bf16_hi(a.y), bf16_hi(b.y), s);
    s = fmaf(bf16_lo(a.z), bf16_lo(b.z), s); s = fmaf(bf16_hi(a.z), bf16_hi(b.z), s);
    s = fmaf(bf16_lo(a.w), bf16_lo(b.w), s); s = fmaf(bf16_hi(a.w), bf16_hi(b.w), s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
  if (lane == 0) dw[j] = s;
}

// Rows [base + total, base + padded) of every local expert are set to zero so that they add
// nothing to a weight gradient (which contracts over the rows).
__global__ void __launch_bounds__(256)
moe_zero_pad_kernel(const int* __restrict__ loc, __nv_bfloat16* __restrict__ buf, long long ld, int cols) {
  const int el = blockIdx.x;
  const int r0 = loc[el * 4 + 0] + loc[el * 4 + 1], r1 = loc[el * 4 + 0] + loc[el * 4 + 2];
  const int per_row = cols / 8;
  for (long long i = threadIdx.x; i < static_cast<long long>(r1 - r0) * per_row; i += blockDim.x) {
    const long long r = r0 + i / per_row;
    *reinterpret_cast<uint4*>(buf + r * ld + (i % per_row) * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
}

static PeerPtrs make_peers(void* const* ptrs, int n) {
  PeerPtrs pp;
  for (int i = 0; i < 8; ++i) pp.p[i] = ptrs[i < n ? i : 0];
  return pp;
}

}  // namespace rlk
using namespace rlk;

// logits fp32 [T, E] (E = 32, 64, 128 or 256) -> idx int32 [T, K] (ascending expert ids), w fp32
// [T, K], optionally probs fp32 [T, E] and counts int32 [E] += tokens per expert.
RLK_API int rlk_moe_router_topk(const float* logits, int T, int E, int K, int* idx, float* w, float* probs,
                                int* counts, void* stream) {
  RLK_REQUIRE(T > 0 && K >= 1 && K <= 32 && K <= E, "moe_router_topk: bad sizes");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = (T + 7) / 8;
  switch (E) {
    case 32: moe_router_topk_kernel<1><<<grid, 256, 0, s>>>(logits, T, K, idx, w, probs, counts); break;
    case 64: moe_router_topk_kernel<2><<<grid, 256, 0, s>>>(logits, T, K, idx, w, probs, counts); break;
    case 128: moe_router_topk_kernel<4><<<grid, 256, 0, s>>>(logits, T, K, idx, w, probs, counts); break;
    case 256: moe_router_topk_kernel<8><<<grid, 256, 0, s>>>(logits, T, K, idx, w, probs, counts); break;
    default: RLK_REQUIRE(false, "moe_router_topk: E must be 32, 64, 128 or 256 (got %d)", E);
  }
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_moe_router_bwd(const int* idx, const float* w, const float* dw, int T, int K, int E,
                               void* dlogits, void* stream) {
  RLK_REQUIRE(T > 0 && K <= 32, "moe_router_bwd: bad sizes");
  moe_router_bwd_kernel<<<(T + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      idx, w, dw, T, K, E, static_cast<__nv_bfloat16*>(dlogits));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// counts_all int32 [W, E] -> send_row0 int32 [E], loc int32 [E / W, 4], rows_used int32 [1].
RLK_API int rlk_moe_plan(const int* counts_all, int W, int rank, int E, int* send_row0, int* loc,
                         int* rows_used, void* stream) {
  RLK_REQUIRE(E <= 256 && W >= 1 && E % W == 0 && rank >= 0 && rank < W, "moe_plan: bad geometry");
  moe_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts_all, W, rank, E, E / W, send_row0,
                                                                   loc, rows_used);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_moe_tiles(const int* loc, int E_loc, int kind, int n_cols, int k_dim, int b_mn, int m_out,
                          void* tiles, int* n_tiles, int max_tiles, void* stream) {
  RLK_REQUIRE(E_loc >= 1 && E_loc <= 128, "moe_tiles: at most 128 local experts");
  RLK_REQUIRE(n_cols % 256 == 0 && k_dim % 64 == 0 && (kind == 0 || m_out % 128 == 0),
              "moe_tiles: n_cols %% 256, k_dim %% 64 and m_out %% 128 must be 0");
  moe_tiles_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      loc, E_loc, kind, n_cols, k_dim, b_mn, m_out, static_cast<GroupTile*>(tiles), n_tiles, max_tiles);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_moe_slots(const int* idx, int n, int E, const int* send_row0, int* slot_row, void* stream) {
  RLK_REQUIRE(n > 0 && E > 0, "moe_slots: empty");
  moe_slots_kernel<<<E, 256, 0, static_cast<cudaStream_t>(stream)>>>(idx, n, send_row0, slot_row);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_moe_dispatch(const void* x, long long ldx, const float* scale, const int* idx,
                             const int* slot_row, int n, int K, int E_loc, int H, void* const* dst_ptrs,
                             int n_ranks, long long ld_dst, void* stream) {
  RLK_REQUIRE(n > 0 && H % 8 == 0 && n_ranks >= 1 && n_ranks <= 8, "moe_dispatch: bad sizes");
  moe_dispatch_kernel<<<(n + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, scale, idx, slot_row, n, K, E_loc, H,
      make_peers(dst_ptrs, n_ranks), ld_dst);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_moe_combine(const void* base, long long ld_base, const float* w, const int* idx,
                            const int* slot_row, int T, int K, int E_loc, int H, void* const* src_ptrs,
                            int n_ranks, long long ld_src, void* out, long long ldo, void* stream) {
  RLK_REQUIRE(T > 0 && H % 8 == 0 && n_ranks >= 1 && n_ranks <= 8, "moe_combine: bad sizes");
  moe_combine_kernel<<<T, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(base), ld_base, w, idx, slot_row, T, K, E_loc, H,
      make_peers(src_ptrs, n_ranks), ld_src, static_cast<__nv_bfloat16*>(out), ldo);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_moe_combine_dw(const void* dout, long long ldd, const int* idx, const int* slot_row, int n,
                               int K, int E_loc, int H, void* const* src_ptrs, int n_ranks, long long ld_src,
                               float* dw, void* stream) {
  RLK_REQUIRE(n > 0 && H % 8 == 0 && n_ranks >= 1 && n_ranks <= 8, "moe_combine_dw: bad sizes");
  moe_combine_dw_kernel<<<(n + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dout), ldd, idx, slot_row, n, K, E_loc, H,
      make_peers(src_ptrs, n_ranks), ld_src, dw);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_moe_zero_pad(const int* loc, int E_loc, void* buf, long long ld, int cols, void* stream) {
  RLK_REQUIRE(E_loc >= 1 && cols % 8 == 0, "moe_zero_pad: bad sizes");
  moe_zero_pad_kernel<<<E_loc, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      loc, static_cast<__nv_bfloat16*>(buf), ld, cols);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
