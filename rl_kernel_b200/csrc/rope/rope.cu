// Stand-alone NeoX (rotate-half) RoPE over x [rows, heads, D] with one position per row, from the
// same fp32 cos/sin tables [max_pos, D/2] that the fused QK-norm + RoPE kernel reads, so a model
// that applies the two steps separately rounds from the same angles.  ``inverse`` rotates by the
// negative angle, which is the backward of the forward (the rotation is orthogonal).  fp32 math,
// one rounding to the output type.  (parity: RoPESM90Op, rl_engine/backends/cuda/rope/rope.py:83
// and csrc/cuda/rope/rope.cu; the reference recomputes angles from theta per element.)
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

template <typename T>
__global__ void __launch_bounds__(256)
rope_kernel(const T* __restrict__ x, long long x_pitch, const int* __restrict__ pos, const float* __restrict__ cos_t,
            const float* __restrict__ sin_t, T* __restrict__ y, long long y_pitch, long long rows, int heads, int D,
            int max_pos, int inverse) {
  griddep_sync();
  const int half = D >> 1;
  const long long per_row = static_cast<long long>(heads) * half;
  const long long total = rows * per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / per_row;
    const int rem = static_cast<int>(i - r * per_row);
    const int h = rem / half, j = rem - h * half;
    int p = pos[r];
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);     // a position outside the table is clamped, never read past it
    const float c = cos_t[static_cast<long long>(p) * half + j];
    const float s = inverse ? -sin_t[static_cast<long long>(p) * half + j] : sin_t[static_cast<long long>(p) * half + j];
    const T* xr = x + r * x_pitch + static_cast<long long>(h) * D;
    T* yr = y + r * y_pitch + static_cast<long long>(h) * D;
    const float a = static_cast<float>(xr[j]), b = static_cast<float>(xr[j + half]);
    // explicit single-rounding multiplies and adds (no FMA contraction): the same bits as the
    // PyTorch expression a*c - b*s evaluated in fp32
    yr[j] = static_cast<T>(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
    yr[j + half] = static_cast<T>(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s)));
  }
}

// Vector form: one thread owns 16 bytes of a head's first half and the matching 16 bytes of its second half
// (V = 8 bf16 or 4 fp32 pairs), reads the pairs' cos / sin as 16-byte pieces of the table row and writes both
// halves with 16-byte stores.  A block walks whole rows (several at once when a row has fewer than 256 pieces),
// so no 64-bit division is paid per element.  Needs D/2 % V == 0 and 16-byte aligned rows.
template <typename T>
__global__ void __launch_bounds__(256)
rope_vec_kernel(const T* __restrict__ x, long long x_pitch, const int* __restrict__ pos, const float* __restrict__ cos_t,
                const float* __restrict__ sin_t, T* __restrict__ y, long long y_pitch, long long rows, int heads, int D,
                int max_pos, int inverse, int per_row, int rows_per_block) {
  constexpr int V = 16 / sizeof(T);
  griddep_sync();
  const int half = D >> 1;
  const int per_half = half / V;                                  // 16-byte pieces per half head
  const int lr = threadIdx.x / per_row, piece0 = threadIdx.x - lr * per_row;
  const int step = rows_per_block > 1 ? per_row : 256;            // several rows per block: one piece per thread
  if (lr >= rows_per_block) return;
  for (long long r = static_cast<long long>(blockIdx.x) * rows_per_block + lr; r < rows;
       r += static_cast<long long>(gridDim.x) * rows_per_block) {
    int p = pos[r];
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);             // a position outside the table is clamped
    const float* cr = cos_t + static_cast<long long>(p) * half;
    const float* sr = sin_t + static_cast<long long>(p) * half;
    for (int piece = piece0; piece < per_row; piece += step) {
      const int h = piece / per_half, j = (piece - h * per_half) * V;
      const T* xr = x + r * x_pitch + static_cast<long long>(h) * D + j;
      T* yr = y + r * y_pitch + static_cast<long long>(h) * D + j;
      const uint4 ua = *reinterpret_cast<const uint4*>(xr);
      const uint4 ub = *reinterpret_cast<const uint4*>(xr + half);
      float c[V], s[V], a[V], b[V];
#pragma unroll
      for (int q = 0; q < V / 4; ++q) {
        const float4 cq = __ldg(reinterpret_cast<const float4*>(cr + j) + q);
        const float4 sq = __ldg(reinterpret_cast<const float4*>(sr + j) + q);
        c[4 * q] = cq.x; c[4 * q + 1] = cq.y; c[4 * q + 2] = cq.z; c[4 * q + 3] = cq.w;
        s[4 * q] = sq.x; s[4 * q + 1] = sq.y; s[4 * q + 2] = sq.z; s[4 * q + 3] = sq.w;
      }
      const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w}, wb[4] = {ub.x, ub.y, ub.z, ub.w};
      if constexpr (sizeof(T) == 2) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          a[2 * q] = bf16_lo(wa[q]); a[2 * q + 1] = bf16_hi(wa[q]);
          b[2 * q] = bf16_lo(wb[q]); b[2 * q + 1] = bf16_hi(wb[q]);
        }
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) { a[q] = __uint_as_float(wa[q]); b[q] = __uint_as_float(wb[q]); }
      }
      float o1[V], o2[V];
#pragma unroll
      for (int q = 0; q < V; ++q) {
        const float sq = inverse ? -s[q] : s[q];
        // explicit single-rounding multiplies and adds (no FMA contraction), as in the scalar form
        o1[q] = __fsub_rn(__fmul_rn(a[q], c[q]), __fmul_rn(b[q], sq));
        o2[q] = __fadd_rn(__fmul_rn(b[q], c[q]), __fmul_rn(a[q], sq));
      }
      uint4 r1, r2;
      if constexpr (sizeof(T) == 2) {
        r1 = make_uint4(pack_bf16x2(o1[0], o1[1]), pack_bf16x2(o1[2], o1[3]), pack_bf16x2(o1[4], o1[5]), pack_bf16x2(o1[6], o1[7]));
        r2 = make_uint4(pack_bf16x2(o2[0], o2[1]), pack_bf16x2(o2[2], o2[3]), pack_bf16x2(o2[4], o2[5]), pack_bf16x2(o2[6], o2[7]));
      } else {
        r1 = make_uint4(__float_as_uint(o1[0]), __float_as_uint(o1[1]), __float_as_uint(o1[2]), __float_as_uint(o1[3]));
        r2 = make_uint4(__float_as_uint(o2[0]), __float_as_uint(o2[1]), __float_as_uint(o2[2]), __float_as_uint(o2[3]));
      }
      *reinterpret_cast<uint4*>(yr) = r1;
      *reinterpret_cast<uint4*>(yr + half) = r2;
    }
  }
}

}  // namespace rlk
using namespace rlk;

// dtype: 0 = bf16, 1 = fp32.  Pitches are in elements.  x and y may alias (each thread reads its
// pair before it writes it).
RLK_API int rlk_rope(const void* x, long long x_pitch, const int* pos, const float* cos_t, const float* sin_t, void* y,
                     long long y_pitch, long long rows, int heads, int D, int max_pos, int inverse, int dtype,
                     void* stream) {
  RLK_REQUIRE(x && y && pos && cos_t && sin_t, "rope: null pointer");
  RLK_REQUIRE(rows >= 0 && heads > 0 && D > 0 && D % 2 == 0 && max_pos > 0, "rope: bad shape");
  RLK_REQUIRE(x_pitch >= static_cast<long long>(heads) * D && y_pitch >= static_cast<long long>(heads) * D, "rope: pitch < heads*D");
  RLK_REQUIRE(dtype == 0 || dtype == 1, "rope: dtype must be 0 (bf16) or 1 (fp32)");
  if (rows == 0) return RLK_OK;
  const long long total = rows * heads * (D / 2);
  const long long want = (total + 255) / 256;
  const int grid = static_cast<int>(want < 8LL * sm_count() ? want : 8LL * sm_count());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // 16-byte pieces when the layout allows it (every model shape does); the scalar kernel takes the rest
  const int V = dtype == 0 ? 8 : 4;
  const long long esz = dtype == 0 ? 2 : 4;
  const bool vec = (D / 2) % V == 0 && (x_pitch * esz) % 16 == 0 && (y_pitch * esz) % 16 == 0 &&
                   (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(cos_t) & 15) == 0 && (reinterpret_cast<uintptr_t>(sin_t) & 15) == 0;
  if (vec) {
    const int per_row = heads * (D / 2 / V);
    const int rpb = per_row >= 256 ? 1 : 256 / per_row;
    const long long blocks = (rows + rpb - 1) / rpb;
    const int vgrid = static_cast<int>(blocks < 16LL * sm_count() ? blocks : 16LL * sm_count());
    if (dtype == 0)
      RLK_CHECK_CUDA(launch_pdl(rope_vec_kernel<__nv_bfloat16>, dim3(vgrid), dim3(256), 0, s, (const __nv_bfloat16*)x, x_pitch,
                                pos, cos_t, sin_t, (__nv_bfloat16*)y, y_pitch, rows, heads, D, max_pos, inverse, per_row, rpb));
    else
      RLK_CHECK_CUDA(launch_pdl(rope_vec_kernel<float>, dim3(vgrid), dim3(256), 0, s, (const float*)x, x_pitch, pos, cos_t,
                                sin_t, (float*)y, y_pitch, rows, heads, D, max_pos, inverse, per_row, rpb));
    RLK_CHECK_CUDA(cudaGetLastError());
    return RLK_OK;
  }
  if (dtype == 0)
    RLK_CHECK_CUDA(launch_pdl(rope_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, (const __nv_bfloat16*)x, x_pitch, pos,
                              cos_t, sin_t, (__nv_bfloat16*)y, y_pitch, rows, heads, D, max_pos, inverse));
  else
    RLK_CHECK_CUDA(launch_pdl(rope_kernel<float>, dim3(grid), dim3(256), 0, s, (const float*)x, x_pitch, pos, cos_t, sin_t,
                              (float*)y, y_pitch, rows, heads, D, max_pos, inverse));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
