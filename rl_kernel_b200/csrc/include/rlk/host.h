// Host-side helpers shared by every translation unit of librlk_b200: error codes, the
// per-device status word that bounded device waits report into, and TMA tensor-map
// creation through the driver entry point (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define RLK_API extern "C" __attribute__((visibility("default")))

enum RlkError : int {
  RLK_OK = 0,
  RLK_ERR_BAD_ARG = 1,      // shape / alignment rejected on the host, nothing launched
  RLK_ERR_CUDA = 2,         // a CUDA runtime / driver call failed (see rlk_last_error)
  RLK_ERR_UNSUPPORTED = 3,  // valid request this build has no kernel for
  RLK_ERR_TIMEOUT = 4,      // a bounded device wait gave up (read by rlk_status_poll)
};

namespace rlk {

// Records a message retrievable through rlk_last_error(); returns `code` for one-line use.
int set_error(int code, const char* fmt, ...);

#define RLK_CHECK_CUDA(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess)                                                                \
      return ::rlk::set_error(RLK_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,               \
                              cudaGetErrorString(_e), __FILE__, __LINE__);                \
  } while (0)

#define RLK_REQUIRE(cond, ...)                                                            \
  do {                                                                                    \
    if (!(cond)) return ::rlk::set_error(RLK_ERR_BAD_ARG, __VA_ARGS__);                   \
  } while (0)

// Device pointer to this device's status word (int, zero = healthy). Allocated once per
// device on first use; kernels atomicCAS a non-zero code into it when a wait times out.
int* device_status_word();

// 2-D bf16 (or any 2-byte element) row-major tensor map with 128-byte swizzle.
//  rows x cols elements, row pitch `ld` elements; box = box_rows x 64 elements (128 bytes).
int make_tmap_2d_sw128(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                       uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols, int elem_bytes);

// 3-D variant: [batch][rows][cols] with explicit strides (elements) for rows and batch.
int make_tmap_3d_sw128(CUtensorMap* out, const void* base, uint64_t batch, uint64_t rows,
                       uint64_t cols, uint64_t row_stride_elems, uint64_t batch_stride_elems,
                       uint32_t box_rows, uint32_t box_cols, int elem_bytes);
// Same with a box that spans box_batch consecutive batch entries (they land one after the other in
// shared memory, box_rows rows of 128 bytes each).
int make_tmap_3d_sw128_box(CUtensorMap* out, const void* base, uint64_t batch, uint64_t rows,
                           uint64_t cols, uint64_t row_stride_elems, uint64_t batch_stride_elems,
                           uint32_t box_batch, uint32_t box_rows, uint32_t box_cols, int elem_bytes);

int sm_count();

// 1 when kernels that start with griddep_sync() are launched with programmatic stream
// serialization (rlk_set_pdl); their launch latency then overlaps the previous kernel's execution.
int pdl_enabled();
// 1 while the calling thread has declared the B operands of its GEMMs static (rlk_set_static_b).
int static_b_operand();

#ifdef __CUDACC__
// Launch for kernels whose first statement is griddep_sync() (rlk/ptx.cuh).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

}  // namespace rlk
