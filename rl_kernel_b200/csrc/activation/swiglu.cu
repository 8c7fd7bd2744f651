// Packed SwiGLU forward / backward.  The column-parallel FFN GEMM writes gate and up interleaved
// in blocks of `blk` columns: [g_0 | u_0 | g_1 | u_1 | ...] where g_c / u_c are columns
// [c*blk, (c+1)*blk) of gate / up (blk = I gives the plain [gate | up] layout; the model uses
// blk = I/8, one block per canonical tensor-parallel shard, so any TP degree sees the same
// layout).  out[:, c*blk + j] = silu(g_c[j]) * u_c[j].
// fp32 math, expf, one rounding at the store (same materialisation boundary as the reference's
// csrc/cuda/activation/activation.cu:32-135).  Eight elements per thread, 16-byte accesses.
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }

// Which 16-byte piece (row r, first column c) this thread owns.  The grid is (row blocks, 256-piece column chunks):
// a row with at least 256 pieces gets one block row per row, a narrower one shares a block with its neighbours, so
// no thread pays a 64-bit division to find its row.  (swiglu_grid() is the host side of the same rule.)
__device__ __forceinline__ bool swiglu_piece(int rows, int I, int& r, int& c) {
  const int per_row = I / 8;
  int piece;
  if (per_row >= 256) {
    r = blockIdx.x;
    piece = blockIdx.y * 256 + threadIdx.x;
  } else {
    const int rpb = 256 / per_row, lr = threadIdx.x / per_row;
    if (lr >= rpb) return false;
    r = blockIdx.x * rpb + lr;
    piece = threadIdx.x - lr * per_row;
  }
  c = piece * 8;
  return r < rows && piece < per_row;
}

__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, long long ld_gu, __nv_bfloat16* __restrict__ out,
                  long long ld_out, int rows, int I, int blk, const int* __restrict__ rows_limit) {
  griddep_sync();
  int r, c;
  if (!swiglu_piece(rows, I, r, c)) return;
  if (rows_limit && r >= *rows_limit) return;  // row count known only on the device (MoE)
  const long long gc = static_cast<long long>(c / blk) * 2 * blk + (c % blk);  // column of gate[c]
  const uint4 g = *reinterpret_cast<const uint4*>(gu + r * ld_gu + gc);
  const uint4 u = *reinterpret_cast<const uint4*>(gu + r * ld_gu + gc + blk);
  const uint32_t gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    o[i] = pack_bf16x2(silu_f(bf16_lo(gv[i])) * bf16_lo(uv[i]), silu_f(bf16_hi(gv[i])) * bf16_hi(uv[i]));
  *reinterpret_cast<uint4*>(out + r * ld_out + c) = make_uint4(o[0], o[1], o[2], o[3]);
}

// d(gate) = dout * up * silu'(gate), d(up) = dout * silu(gate); written packed like the input.
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, long long ld_gu, const __nv_bfloat16* __restrict__ dout,
                  long long ld_dout, __nv_bfloat16* __restrict__ dgu, long long ld_dgu, int rows, int I, int blk,
                  const int* __restrict__ rows_limit) {
  int r, c;
  if (!swiglu_piece(rows, I, r, c)) return;
  if (rows_limit && r >= *rows_limit) return;
  const long long gc = static_cast<long long>(c / blk) * 2 * blk + (c % blk);  // column of gate[c]
  const uint4 g = *reinterpret_cast<const uint4*>(gu + r * ld_gu + gc);
  const uint4 u = *reinterpret_cast<const uint4*>(gu + r * ld_gu + gc + blk);
  const uint4 d = *reinterpret_cast<const uint4*>(dout + r * ld_dout + c);
  const uint32_t gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w}, dv[4] = {d.x, d.y, d.z, d.w};
  uint32_t og[4], ou[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float dgl[2], dul[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float gg = h ? bf16_hi(gv[i]) : bf16_lo(gv[i]);
      const float uu = h ? bf16_hi(uv[i]) : bf16_lo(uv[i]);
      const float dd = h ? bf16_hi(dv[i]) : bf16_lo(dv[i]);
      const float sig = 1.f / (1.f + __expf(-gg));
      const float sl = gg * sig;
      dul[h] = dd * sl;
      dgl[h] = dd * uu * (sig * (1.f + gg * (1.f - sig)));
    }
    og[i] = pack_bf16x2(dgl[0], dgl[1]);
    ou[i] = pack_bf16x2(dul[0], dul[1]);
  }
  *reinterpret_cast<uint4*>(dgu + r * ld_dgu + gc) = make_uint4(og[0], og[1], og[2], og[3]);
  *reinterpret_cast<uint4*>(dgu + r * ld_dgu + gc + blk) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
}

// The same two operations on gate and up held in two tensors (the public ``swiglu(gate, up)``): no packed copy is
// made first.  Identical per-element arithmetic to the packed kernels.
__global__ void __launch_bounds__(256)
swiglu_split_fwd_kernel(const __nv_bfloat16* __restrict__ gate, long long ld_g, const __nv_bfloat16* __restrict__ up,
                        long long ld_u, __nv_bfloat16* __restrict__ out, long long ld_out, int rows, int I) {
  griddep_sync();
  int r, c;
  if (!swiglu_piece(rows, I, r, c)) return;
  const uint4 g = *reinterpret_cast<const uint4*>(gate + r * ld_g + c);
  const uint4 u = *reinterpret_cast<const uint4*>(up + r * ld_u + c);
  const uint32_t gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    o[i] = pack_bf16x2(silu_f(bf16_lo(gv[i])) * bf16_lo(uv[i]), silu_f(bf16_hi(gv[i])) * bf16_hi(uv[i]));
  *reinterpret_cast<uint4*>(out + r * ld_out + c) = make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void __launch_bounds__(256)
swiglu_split_bwd_kernel(const __nv_bfloat16* __restrict__ gate, long long ld_g, const __nv_bfloat16* __restrict__ up,
                        long long ld_u, const __nv_bfloat16* __restrict__ dout, long long ld_dout,
                        __nv_bfloat16* __restrict__ dgate, long long ld_dg, __nv_bfloat16* __restrict__ dup, long long ld_du,
                        int rows, int I) {
  int r, c;
  if (!swiglu_piece(rows, I, r, c)) return;
  const uint4 g = *reinterpret_cast<const uint4*>(gate + r * ld_g + c);
  const uint4 u = *reinterpret_cast<const uint4*>(up + r * ld_u + c);
  const uint4 d = *reinterpret_cast<const uint4*>(dout + r * ld_dout + c);
  const uint32_t gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w}, dv[4] = {d.x, d.y, d.z, d.w};
  uint32_t og[4], ou[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float dgl[2], dul[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float gg = h ? bf16_hi(gv[i]) : bf16_lo(gv[i]);
      const float uu = h ? bf16_hi(uv[i]) : bf16_lo(uv[i]);
      const float dd = h ? bf16_hi(dv[i]) : bf16_lo(dv[i]);
      const float sig = 1.f / (1.f + __expf(-gg));
      const float sl = gg * sig;
      dul[h] = dd * sl;
      dgl[h] = dd * uu * (sig * (1.f + gg * (1.f - sig)));
    }
    og[i] = pack_bf16x2(dgl[0], dgl[1]);
    ou[i] = pack_bf16x2(dul[0], dul[1]);
  }
  *reinterpret_cast<uint4*>(dgate + r * ld_dg + c) = make_uint4(og[0], og[1], og[2], og[3]);
  *reinterpret_cast<uint4*>(dup + r * ld_du + c) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
}

}  // namespace rlk
using namespace rlk;

static dim3 swiglu_grid(int rows, int I) {
  const int per_row = I / 8;
  if (per_row >= 256) return dim3(static_cast<unsigned>(rows), static_cast<unsigned>((per_row + 255) / 256));
  const int rpb = 256 / per_row;
  return dim3(static_cast<unsigned>((rows + rpb - 1) / rpb), 1);
}

// rows_limit (device int, may be null): rows at or beyond *rows_limit are skipped.
RLK_API int rlk_swiglu_fwd_dyn(const void* gu, long long ld_gu, void* out, long long ld_out, int rows,
                               int I, int blk, const int* rows_limit, void* stream) {
  RLK_REQUIRE(rows > 0 && I > 0 && I % 8 == 0 && ld_gu % 8 == 0 && ld_out % 8 == 0,
              "swiglu: I and pitches must be multiples of 8");
  RLK_REQUIRE(blk > 0 && blk % 8 == 0 && I % blk == 0, "swiglu: blk must divide I and be a multiple of 8");
  RLK_CHECK_CUDA(launch_pdl(swiglu_fwd_kernel, swiglu_grid(rows, I), dim3(256), 0,
                            static_cast<cudaStream_t>(stream), (const __nv_bfloat16*)gu, ld_gu, (__nv_bfloat16*)out,
                            ld_out, rows, I, blk, rows_limit));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_swiglu_fwd(const void* gu, long long ld_gu, void* out, long long ld_out, int rows,
                           int I, int blk, void* stream) {
  return rlk_swiglu_fwd_dyn(gu, ld_gu, out, ld_out, rows, I, blk, nullptr, stream);
}

RLK_API int rlk_swiglu_bwd_dyn(const void* gu, long long ld_gu, const void* dout, long long ld_dout,
                               void* dgu, long long ld_dgu, int rows, int I, int blk, const int* rows_limit,
                               void* stream) {
  RLK_REQUIRE(rows > 0 && I > 0 && I % 8 == 0 && ld_gu % 8 == 0 && ld_dout % 8 == 0 && ld_dgu % 8 == 0,
              "swiglu_bwd: I and pitches must be multiples of 8");
  RLK_REQUIRE(blk > 0 && blk % 8 == 0 && I % blk == 0, "swiglu_bwd: blk must divide I and be a multiple of 8");
  swiglu_bwd_kernel<<<swiglu_grid(rows, I), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)gu, ld_gu, (const __nv_bfloat16*)dout, ld_dout, (__nv_bfloat16*)dgu, ld_dgu, rows, I, blk, rows_limit);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_swiglu_bwd(const void* gu, long long ld_gu, const void* dout, long long ld_dout,
                           void* dgu, long long ld_dgu, int rows, int I, int blk, void* stream) {
  return rlk_swiglu_bwd_dyn(gu, ld_gu, dout, ld_dout, dgu, ld_dgu, rows, I, blk, nullptr, stream);
}

// gate / up / out (and their gradients) as separate [rows, I] tensors with their own pitches (elements, multiples of 8).
RLK_API int rlk_swiglu_split_fwd(const void* gate, long long ld_g, const void* up, long long ld_u, void* out,
                                 long long ld_out, int rows, int I, void* stream) {
  RLK_REQUIRE(rows > 0 && I > 0 && I % 8 == 0 && ld_g % 8 == 0 && ld_u % 8 == 0 && ld_out % 8 == 0,
              "swiglu_split: I and pitches must be multiples of 8");
  RLK_REQUIRE(gate && up && out, "swiglu_split: null pointer");
  RLK_CHECK_CUDA(launch_pdl(swiglu_split_fwd_kernel, swiglu_grid(rows, I), dim3(256), 0, static_cast<cudaStream_t>(stream),
                            (const __nv_bfloat16*)gate, ld_g, (const __nv_bfloat16*)up, ld_u, (__nv_bfloat16*)out, ld_out,
                            rows, I));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_swiglu_split_bwd(const void* gate, long long ld_g, const void* up, long long ld_u, const void* dout,
                                 long long ld_dout, void* dgate, long long ld_dg, void* dup, long long ld_du, int rows,
                                 int I, void* stream) {
  RLK_REQUIRE(rows > 0 && I > 0 && I % 8 == 0 && ld_g % 8 == 0 && ld_u % 8 == 0 && ld_dout % 8 == 0 && ld_dg % 8 == 0 &&
                  ld_du % 8 == 0, "swiglu_split_bwd: I and pitches must be multiples of 8");
  RLK_REQUIRE(gate && up && dout && dgate && dup, "swiglu_split_bwd: null pointer");
  swiglu_split_bwd_kernel<<<swiglu_grid(rows, I), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)gate, ld_g, (const __nv_bfloat16*)up, ld_u, (const __nv_bfloat16*)dout, ld_dout,
      (__nv_bfloat16*)dgate, ld_dg, (__nv_bfloat16*)dup, ld_du, rows, I);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
