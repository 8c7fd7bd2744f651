// Fused AdamW over a flat parameter shard: bf16 gradient in, fp32 master / m / v state updated,
// bf16 working copy written, all in one pass (16 bytes per element of state traffic is the floor).
// Also the exact, partition-independent sum of squares used for gradient clipping (integer
// per-exponent bins, the same idea as rl_engine/ops/norm/reproducible.py:17-57).
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

struct AdamParams {
  float* master; float* m; float* v; const __nv_bfloat16* grad; __nv_bfloat16* param;
  long long n;
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;  // bc = 1 - beta^t
  const float* grad_scale;  // device scalar multiplied into the gradient (clip factor), or null
};

__global__ void __launch_bounds__(256) adamw_kernel(const AdamParams p) {
  const long long i0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i0 >= p.n) return;
  const float gs = p.grad_scale ? *p.grad_scale : 1.f;
  if (i0 + 8 <= p.n) {
    const uint4 g = *reinterpret_cast<const uint4*>(p.grad + i0);
    const uint32_t gu[4] = {g.x, g.y, g.z, g.w};
    float w[8], mm[8], vv[8];
    *reinterpret_cast<float4*>(w) = *reinterpret_cast<const float4*>(p.master + i0);
    *reinterpret_cast<float4*>(w + 4) = *reinterpret_cast<const float4*>(p.master + i0 + 4);
    *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(p.m + i0);
    *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(p.m + i0 + 4);
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(p.v + i0);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(p.v + i0 + 4);
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = ((k & 1) ? bf16_hi(gu[k >> 1]) : bf16_lo(gu[k >> 1])) * gs;
      mm[k] = p.beta1 * mm[k] + (1.f - p.beta1) * gk;
      vv[k] = p.beta2 * vv[k] + (1.f - p.beta2) * gk * gk;
      const float mh = mm[k] / p.bc1, vh = vv[k] / p.bc2;
      w[k] = w[k] - p.lr * (mh / (sqrtf(vh) + p.eps) + p.weight_decay * w[k]);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = pack_bf16x2(w[2 * k], w[2 * k + 1]);
    *reinterpret_cast<float4*>(p.master + i0) = *reinterpret_cast<float4*>(w);
    *reinterpret_cast<float4*>(p.master + i0 + 4) = *reinterpret_cast<float4*>(w + 4);
    *reinterpret_cast<float4*>(p.m + i0) = *reinterpret_cast<float4*>(mm);
    *reinterpret_cast<float4*>(p.m + i0 + 4) = *reinterpret_cast<float4*>(mm + 4);
    *reinterpret_cast<float4*>(p.v + i0) = *reinterpret_cast<float4*>(vv);
    *reinterpret_cast<float4*>(p.v + i0 + 4) = *reinterpret_cast<float4*>(vv + 4);
    *reinterpret_cast<uint4*>(p.param + i0) = make_uint4(o[0], o[1], o[2], o[3]);
  } else {
    for (long long i = i0; i < p.n; ++i) {
      const float gk = __bfloat162float(p.grad[i]) * gs;
      const float m1 = p.beta1 * p.m[i] + (1.f - p.beta1) * gk;
      const float v1 = p.beta2 * p.v[i] + (1.f - p.beta2) * gk * gk;
      const float w1 = p.master[i] - p.lr * ((m1 / p.bc1) / (sqrtf(v1 / p.bc2) + p.eps) + p.weight_decay * p.master[i]);
      p.m[i] = m1; p.v[i] = v1; p.master[i] = w1;
      p.param[i] = __float2bfloat16_rn(w1);
    }
  }
}

// Exact sum of squares.  A finite bf16 value is mant * 2^ex with mant < 2^8, so its square is an
// integer sq < 2^16 times 2^(2 ex).  Squares are summed as integers into one 64-bit bin per
// biased exponent (256 bins); integer addition is associative, so the bins -- and the norm
// computed from them in a fixed order -- do not depend on how the gradient is split over
// threads, blocks or ranks.  bins[255] counts non-finite inputs.
//
// Each warp keeps a private 256 x uint32 histogram in shared memory (native 32-bit shared atomics;
// lanes that hit the same bin are serialised by the hardware, nothing spins) and spills it to the
// 64-bit global bins before any bin could overflow: at most 64 iterations x 8 values x 32 lanes
// squares of < 2^16 each lie between two spills.
__device__ __forceinline__ void sumsq_add(uint32_t* hist, uint32_t h) {
  const uint32_t e = (h >> 7) & 0xff;
  uint32_t mant = h & 0x7f;
  if (e == 0xff) { atomicAdd(&hist[255], 1u); return; }
  if (e != 0) mant |= 0x80;
  if (mant != 0) atomicAdd(&hist[e], mant * mant);
}

__global__ void __launch_bounds__(256)
sumsq_bins_kernel(const __nv_bfloat16* __restrict__ g, long long n, unsigned long long* bins) {
  __shared__ uint32_t sh[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* hist = sh[warp];
#pragma unroll
  for (int k = 0; k < 8; ++k) hist[lane + 32 * k] = 0u;
  __syncwarp();
  auto spill = [&]() {
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t v = hist[lane + 32 * k];
      if (v) {
        atomicAdd(&bins[lane + 32 * k], static_cast<unsigned long long>(v));
        hist[lane + 32 * k] = 0u;
      }
    }
    __syncwarp();
  };
  // elements before the first 16-byte boundary and after the last full vector: one thread
  const uintptr_t addr = reinterpret_cast<uintptr_t>(g);
  long long head = ((16 - (addr & 15)) & 15) / 2;
  if (head > n) head = n;
  const long long nvec = (n - head) / 8;
  const long long tail0 = head + nvec * 8;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const unsigned short* u = reinterpret_cast<const unsigned short*>(g);
    for (long long i = 0; i < head; ++i) sumsq_add(hist, u[i]);
    for (long long i = tail0; i < n; ++i) sumsq_add(hist, u[i]);
  }
  const uint4* v4 = reinterpret_cast<const uint4*>(g + head);
  int since = 0;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  // the loop bounds are warp-uniform, so the whole warp reaches every spill together
  for (long long base = static_cast<long long>(blockIdx.x) * blockDim.x + warp * 32; base < nvec; base += stride) {
    const long long i = base + lane;
    if (i < nvec) {
      const uint4 x = v4[i];
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        sumsq_add(hist, w[k] & 0xffffu);
        sumsq_add(hist, w[k] >> 16);
      }
    }
    if (++since == 64) {
      since = 0;
      spill();
    }
  }
  spill();
}

// fp32 inputs: a finite value is m * 2^(e - 150) with an integer m < 2^24, so m^2 < 2^48 is split
// into three 16-bit limbs and every (exponent, limb) pair gets its own integer bin (768 bins):
// bins[3 e + l] += limb_l(m^2).  Still exact and order-free; the caller folds the limbs back with
// weights 2^(16 l) * 2^(2 (max(e, 1) - 150)).  bins[3 * 255] counts non-finite inputs.
__global__ void __launch_bounds__(256)
sumsq_bins_f32_kernel(const float* __restrict__ g, long long n, unsigned long long* bins) {
  __shared__ uint32_t sh[4][768];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* hist = sh[warp >> 1];   // two warps share one histogram (shared atomics make that safe)
  for (int k = threadIdx.x; k < 4 * 768; k += 256) (&sh[0][0])[k] = 0u;
  __syncthreads();
  auto add = [&](uint32_t u) {
    const uint32_t e = (u >> 23) & 0xff;
    if (e == 0xff) { atomicAdd(&hist[3 * 255], 1u); return; }
    unsigned long long m = u & 0x7fffffu;
    if (e != 0) m |= 0x800000u;
    if (m == 0) return;
    const unsigned long long sq = m * m;
    atomicAdd(&hist[3 * e], static_cast<uint32_t>(sq & 0xffffu));
    atomicAdd(&hist[3 * e + 1], static_cast<uint32_t>((sq >> 16) & 0xffffu));
    atomicAdd(&hist[3 * e + 2], static_cast<uint32_t>(sq >> 32));
  };
  auto spill = [&]() {
    __syncthreads();
    for (int k = threadIdx.x; k < 4 * 768; k += 256) {
      const uint32_t v = (&sh[0][0])[k];
      if (v) {
        atomicAdd(&bins[k % 768], static_cast<unsigned long long>(v));
        (&sh[0][0])[k] = 0u;
      }
    }
    __syncthreads();
  };
  const uint32_t* u = reinterpret_cast<const uint32_t*>(g);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  int since = 0;
  // block-uniform trip count: every thread of the block reaches every spill
  for (long long base = static_cast<long long>(blockIdx.x) * blockDim.x; base < n; base += stride) {
    const long long i = base + threadIdx.x;
    if (i < n) add(u[i]);
    if (++since == 512) {    // 512 iterations x 64 lanes x limbs < 2^16 stays below 2^31 per bin
      since = 0;
      spill();
    }
  }
  spill();
}

}  // namespace rlk
using namespace rlk;

RLK_API int rlk_adamw(float* master, float* m, float* v, const void* grad, void* param, long long n,
                      float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                      const float* grad_scale, void* stream) {
  RLK_REQUIRE(n > 0 && step >= 1, "adamw: n > 0 and step >= 1 required");
  RLK_REQUIRE(((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) |
                reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(grad) |
                reinterpret_cast<uintptr_t>(param)) & 15) == 0, "adamw: buffers must be 16-byte aligned");
  AdamParams p{master, m, v, (const __nv_bfloat16*)grad, (__nv_bfloat16*)param, n, lr, beta1, beta2, eps,
               weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step), grad_scale};
  const long long threads = (n + 7) / 8;
  adamw_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// bins: 256 x uint64, zeroed by the caller.  bins[e] += sum of mant^2 over elements with biased
// exponent e (e = 0 holds subnormals with exponent 1's scale); bins[255] += count of inf/nan.
// sum of squares = sum_e bins[e] * 2^(2 * (max(e,1) - 127 - 7)).
RLK_API int rlk_sumsq_bins(const void* grad, long long n, unsigned long long* bins, void* stream) {
  RLK_REQUIRE(n > 0, "sumsq_bins: empty");
  long long blocks = (n + 256 * 64 - 1) / (256 * 64);
  if (blocks > 148 * 8) blocks = 148 * 8;
  sumsq_bins_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)grad, n, bins);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// fp32 form: bins is 768 x uint64 (zeroed by the caller), bins[3 e + l] += limb l (16 bits) of the
// squared 24-bit significand of every element with biased exponent e; bins[765] counts inf / nan.
// sum of squares = sum_{e,l} bins[3 e + l] * 2^(16 l) * 2^(2 * (max(e,1) - 150)).
RLK_API int rlk_sumsq_bins_f32(const float* grad, long long n, unsigned long long* bins, void* stream) {
  RLK_REQUIRE(n > 0, "sumsq_bins_f32: empty");
  long long blocks = (n + 256 * 32 - 1) / (256 * 32);
  if (blocks > 148 * 8) blocks = 148 * 8;
  sumsq_bins_f32_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(grad, n, bins);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
