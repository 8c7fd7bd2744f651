// Train -> rollout weight synchronisation as ONE kernel: every source rank pushes the blocks of
// its parameter shard straight into the rollout engines' parameter buffers on the peer GPUs
// (NVLink stores through peer pointers), re-laying them out on the way.  A transfer is a list of
// 2-D block copies {src offset/pitch -> dst offset/pitch, rows x row_bytes, destination mask};
// resharding between tensor-parallel degrees (column / row slices of a matrix) and the
// broadcast to several replicas are both just such lists, so "broadcast + repack" needs no
// staging buffer and no second pass.  After the copies the kernel publishes the new weight
// version into a flag word of every destination (st.release.sys) which the consumer polls with a
// bounded wait before its first kernel of the new version.
// Also here: plain CUDA-IPC export/import of device allocations for cross-process bridges.
// (The reference moves weights through CUDA-VMM aliases, shared memory or a disk export:
// rl_engine/integrations/common/weights.py:985-2371.)
#include "rlk/host.h"
#include "rlk/ptx.cuh"

#include <cstring>

namespace rlk {

struct CopyDesc {
  long long src_off, dst_off;     // bytes
  long long src_pitch, dst_pitch; // bytes between rows
  int rows, row_bytes;            // row_bytes multiple of 16
  unsigned int dst_mask;          // bit r set: copy to destination r
  int pad;
};

struct PushTargets {
  unsigned char* base[8];
  unsigned long long* version_flag[8];  // may be null
};

__global__ void __launch_bounds__(256)
weight_push_kernel(const unsigned char* __restrict__ src, const CopyDesc* __restrict__ descs, int ndesc,
                   const PushTargets tg, int ntargets, unsigned long long version, unsigned int* done_counter) {
  for (int d = blockIdx.y; d < ndesc; d += gridDim.y) {
    const CopyDesc c = descs[d];
    const int per_row = c.row_bytes / 16;
    const long long total = static_cast<long long>(c.rows) * per_row;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long r = i / per_row, q = i % per_row;
      const uint4 v = *reinterpret_cast<const uint4*>(src + c.src_off + r * c.src_pitch + q * 16);
#pragma unroll
      for (int t = 0; t < 8; ++t)
        if (t < ntargets && (c.dst_mask >> t) & 1u)
          *reinterpret_cast<uint4*>(tg.base[t] + c.dst_off + r * c.dst_pitch + q * 16) = v;
    }
  }
  // last CTA to finish publishes the version to every destination
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int total_ctas = gridDim.x * gridDim.y;
    if (atomicAdd(done_counter, 1u) == total_ctas - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int t = 0; t < ntargets; ++t)
        if (tg.version_flag[t])
          asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(tg.version_flag[t]), "l"(version) : "memory");
    }
  }
}

// Bounded wait until *flag >= version; writes 1 to *ok on success, 0 (and a status code) on timeout.
__global__ void version_wait_kernel(const unsigned long long* flag, unsigned long long version, int* ok, int* status) {
  const uint64_t t0 = globaltimer_ns();
  unsigned long long v;
  uint32_t it = 0;
  while (true) {
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
    if (v >= version) { *ok = 1; return; }
    if ((++it & 63) == 0 && globaltimer_ns() - t0 > RLK_WAIT_LIMIT_NS) {
      *ok = 0;
      if (status) atomicCAS(status, 0, 501);
      return;
    }
  }
}

}  // namespace rlk
using namespace rlk;

// descs: device array of ndesc CopyDesc (48 bytes each). dst_bases/version_flags: host arrays of
// ntargets device pointers (flags may be null). counter: device uint32, zero before the first use.
RLK_API int rlk_weight_push(const void* src, const void* descs, int ndesc, const void* const* dst_bases,
                            void* const* version_flags, int ntargets, unsigned long long version,
                            void* counter, void* stream) {
  RLK_REQUIRE(ndesc > 0 && ntargets >= 1 && ntargets <= 8, "weight_push: need 1..8 targets and at least one block");
  PushTargets tg{};
  for (int t = 0; t < ntargets; ++t) {
    tg.base[t] = static_cast<unsigned char*>(const_cast<void*>(dst_bases[t]));
    tg.version_flag[t] = version_flags ? static_cast<unsigned long long*>(version_flags[t]) : nullptr;
  }
  dim3 grid(64, ndesc < 64 ? ndesc : 64);
  weight_push_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char*>(src), static_cast<const CopyDesc*>(descs), ndesc, tg, ntargets, version,
      static_cast<unsigned int*>(counter));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_version_wait(const void* flag, unsigned long long version, int* ok_device, void* stream) {
  version_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned long long*>(flag), version, ok_device, device_status_word());
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// ---- CUDA IPC helpers (cudaMalloc'ed memory only; torch's expandable segments cannot be exported)
RLK_API int rlk_ipc_alloc(long long bytes, void** ptr_out, void* handle_out) {
  RLK_REQUIRE(bytes > 0, "ipc_alloc: empty");
  void* p = nullptr;
  RLK_CHECK_CUDA(cudaMalloc(&p, bytes));
  RLK_CHECK_CUDA(cudaMemset(p, 0, bytes));
  cudaIpcMemHandle_t h;
  RLK_CHECK_CUDA(cudaIpcGetMemHandle(&h, p));
  memcpy(handle_out, &h, sizeof(h));
  *ptr_out = p;
  return RLK_OK;
}
RLK_API int rlk_ipc_open(const void* handle, void** ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  RLK_CHECK_CUDA(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
  return RLK_OK;
}
RLK_API int rlk_ipc_close(void* ptr) {
  RLK_CHECK_CUDA(cudaIpcCloseMemHandle(ptr));
  return RLK_OK;
}
RLK_API int rlk_ipc_free(void* ptr) {
  RLK_CHECK_CUDA(cudaFree(ptr));
  return RLK_OK;
}
