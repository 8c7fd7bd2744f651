// Issue-rate microbenchmark for tcgen05.mma (one CTA, one issuing thread, operands are zeros in
// shared memory, no global traffic).  It answers three questions that shape the kernels here:
//   mode 0: cycles per MMA of a chain into one accumulator, as a function of the tile width N
//           (measured on B200: 129 cycles at N = 256 and 65 at N = 128, the tensor pipe's own time;
//           about 54 at N <= 64 when eight MMAs are issued back to back and 92-99 in a loop of
//           four -- below N = 128 the issuing thread, not the tensor pipe, sets the pace);
//           alternating over several accumulators changes nothing: a dependent chain runs at full rate;
//   mode 1: plus one tcgen05.commit per four MMAs (about 60-85 cycles per commit);
//   mode 2: plus a wait for that commit (the round trip MMA -> commit -> mbarrier -> waiting thread).
// UNI = true runs the loop warp-uniformly with the MMAs under an elected lane.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I rl_kernel_b200/csrc/include \
//        -o mma_issue_rate rl_kernel_b200/benchmarks/native/mma_issue_rate.cu -lcuda && ./mma_issue_rate
#include <cstdio>
#include <cuda_runtime.h>
#include <cuda.h>
#include "rlk/ptx.cuh"
using namespace rlk;

template <int M, int N, bool UNI>
__global__ void __launch_bounds__(128, 1) chain_kernel(int n_mma, int n_acc, int per_commit, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t bar, bar2;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  fence_proxy_async_smem();
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); mbar_init(smem_u32(&bar2), 1); abort_flag = 0; mbar_fence_init(); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_slot), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const bool leader = UNI ? elect_one() : true;
  if (UNI ? (threadIdx.x >> 5) == 1 : threadIdx.x == 32) {
    constexpr uint32_t idesc = umma_idesc_bf16(M, N, 0, 0);
    const uint32_t sa = smem_u32(smem), sb = sa + 16384;
    uint32_t ph = 0;
    for (int rep = 0; rep < 3; ++rep) {
      const long long t0 = clock64();
      const uint64_t da0 = umma_desc_sw128(sa, 16, 1024), db0 = umma_desc_sw128(sb, 16, 1024);
      const uint32_t nm = n_acc - 1;   // n_acc is a power of two
      uint32_t ph2 = (rep * (n_mma / 4)) & 1;   // bar2 gets one arrival per group of 4
      for (int i = 0; i < n_mma; i += 4) {
        if (leader) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t a = (i + j) & nm;
            umma_bf16_ss(tmem_base + a * N, da0 + 2 * (j & 3), db0 + 2 * (j & 3), idesc, i >= n_acc ? 1u : 0u);
          }
          if (per_commit >= 1) umma_commit(smem_u32(&bar2));
        }
        if (per_commit >= 2) { mbar_wait(smem_u32(&bar2), ph2, &abort_flag, nullptr, 2); }
        ph2 ^= 1;
      }
      if (leader) umma_commit(smem_u32(&bar));
      const long long t1 = clock64();
      mbar_wait(smem_u32(&bar), ph, &abort_flag, nullptr, 1);
      ph ^= 1;
      const long long t2 = clock64();
      if (rep == 2 && (threadIdx.x & 31) == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int M, int N, bool UNI = false>
void run(int n_mma, int n_acc, int mode = 0) {
  long long* d; cudaMalloc(&d, 16);
  auto k = chain_kernel<M, N, UNI>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  k<<<1, 128, 52 * 1024>>>(n_mma, n_acc, mode, d);
  long long h[2] = {0, 0};
  cudaError_t e = cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
  printf("uni=%d mode=%d M=%d N=%3d acc=%d mmas=%d: issue %lld cyc, total %lld cyc, %.1f cyc/mma (%s)\n", int(UNI), mode, M, N, n_acc, n_mma, h[0], h[1],
         double(h[1]) / n_mma, cudaGetErrorString(e));
  cudaFree(d);
}

int main() {
  for (int mode = 0; mode < 3; ++mode) {
    run<128, 64>(256, 1, mode); run<128, 256>(256, 1, mode);
    run<128, 64, true>(256, 1, mode); run<128, 256, true>(256, 1, mode);
  }
  return 0;
}
