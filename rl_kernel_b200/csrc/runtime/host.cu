// Host runtime shared by all kernels: last-error text, per-device status word, tensor maps.
#include "rlk/host.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace rlk {

static thread_local char g_err[1024] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static constexpr int kMaxDevices = 64;
static int* g_status[kMaxDevices] = {nullptr};
static int g_sms[kMaxDevices] = {0};
static std::mutex g_mu;

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[dev] = p;
  }
  return g_status[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (!g_sms[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sms[dev] = n > 0 ? n : 148;
  }
  return g_sms[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static CUtensorMapDataType dtype_for(int elem_bytes) {
  switch (elem_bytes) {
    case 2: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case 4: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

int make_tmap_2d_sw128(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                       uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols, int elem_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(RLK_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  RLK_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base must be 16-byte aligned");
  RLK_REQUIRE((ld_elems * elem_bytes) % 16 == 0, "TMA row pitch must be a multiple of 16 bytes");
  RLK_REQUIRE(box_cols * elem_bytes == 128, "128-byte swizzle needs a 128-byte inner box");
  RLK_REQUIRE(box_rows >= 1 && box_rows <= 256, "TMA box rows out of range");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype_for(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(RLK_ERR_CUDA, "cuTensorMapEncodeTiled(2d) failed with %d", (int)r);
  return RLK_OK;
}

int make_tmap_3d_sw128(CUtensorMap* out, const void* base, uint64_t batch, uint64_t rows,
                       uint64_t cols, uint64_t row_stride_elems, uint64_t batch_stride_elems,
                       uint32_t box_rows, uint32_t box_cols, int elem_bytes) {
  return make_tmap_3d_sw128_box(out, base, batch, rows, cols, row_stride_elems, batch_stride_elems, 1,
                                box_rows, box_cols, elem_bytes);
}

int make_tmap_3d_sw128_box(CUtensorMap* out, const void* base, uint64_t batch, uint64_t rows,
                           uint64_t cols, uint64_t row_stride_elems, uint64_t batch_stride_elems,
                           uint32_t box_batch, uint32_t box_rows, uint32_t box_cols, int elem_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(RLK_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  RLK_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base must be 16-byte aligned");
  RLK_REQUIRE((row_stride_elems * elem_bytes) % 16 == 0 &&
                  (batch_stride_elems * elem_bytes) % 16 == 0,
              "TMA strides must be multiples of 16 bytes");
  RLK_REQUIRE(box_cols * elem_bytes == 128, "128-byte swizzle needs a 128-byte inner box");
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {row_stride_elems * static_cast<uint64_t>(elem_bytes),
                           batch_stride_elems * static_cast<uint64_t>(elem_bytes)};
  RLK_REQUIRE(box_batch >= 1 && box_batch <= 256 && box_rows >= 1 && box_rows <= 256, "TMA box out of range");
  cuuint32_t box[3] = {box_cols, box_rows, box_batch};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dtype_for(elem_bytes), 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(RLK_ERR_CUDA, "cuTensorMapEncodeTiled(3d) failed with %d", (int)r);
  return RLK_OK;
}

static int g_pdl = 1;
int pdl_enabled() { return g_pdl; }
static thread_local int g_static_b = 0;
int static_b_operand() { return g_static_b && g_pdl; }

}  // namespace rlk

// Programmatic dependent launch for the library's kernel chains: 1 = on (default), 0 = off.
RLK_API int rlk_set_pdl(int on) {
  const int old = rlk::g_pdl;
  rlk::g_pdl = on ? 1 : 0;
  return old;
}

// While on (per host thread), det_gemm launches may fetch their B operand before the previous
// kernel of the stream has finished.  The caller promises that B (a weight) was complete before
// that previous kernel was launched; A and C keep the full dependency.  Returns the old setting.
RLK_API int rlk_set_static_b(int on) {
  const int old = rlk::g_static_b;
  rlk::g_static_b = on ? 1 : 0;
  return old;
}

RLK_API const char* rlk_last_error() { return rlk::g_err; }

// Reads and clears this device's status word on `stream` (synchronises that stream).
RLK_API int rlk_status_poll(void* stream, int* out_code) {
  int* w = rlk::device_status_word();
  if (!w) return rlk::set_error(RLK_ERR_CUDA, "status word unavailable");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int v = 0;
  RLK_CHECK_CUDA(cudaMemcpyAsync(&v, w, sizeof(int), cudaMemcpyDeviceToHost, s));
  RLK_CHECK_CUDA(cudaStreamSynchronize(s));
  if (v != 0) RLK_CHECK_CUDA(cudaMemsetAsync(w, 0, sizeof(int), s));
  *out_code = v;
  return RLK_OK;
}

RLK_API int rlk_abi_version() { return 1; }

