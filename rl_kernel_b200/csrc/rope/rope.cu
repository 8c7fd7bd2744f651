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
  if (dtype == 0)
    RLK_CHECK_CUDA(launch_pdl(rope_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, (const __nv_bfloat16*)x, x_pitch, pos,
                              cos_t, sin_t, (__nv_bfloat16*)y, y_pitch, rows, heads, D, max_pos, inverse));
  else
    RLK_CHECK_CUDA(launch_pdl(rope_kernel<float>, dim3(grid), dim3(256), 0, s, (const float*)x, x_pitch, pos, cos_t, sin_t,
                              (float*)y, y_pitch, rows, heads, D, max_pos, inverse));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
