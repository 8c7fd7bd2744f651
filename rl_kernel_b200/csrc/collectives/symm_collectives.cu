// Symmetric-memory runtime and fixed-order collectives over NVLink peer access (single node).
//
// Every rank allocates one "window" with cudaMalloc, exports it with a CUDA IPC handle and maps the
// windows of its peers; a window is [flag area | frame 0 | frame 1].  Collectives are ONE kernel
// per call, launched by every rank on its own stream:
//   * the payload is processed in slices; CTA b of every rank owns slices b, b+grid, ... in the same
//     order on every rank, so a CTA only ever waits for the same-numbered slice of its peers;
//   * a CTA copies its slice into the local frame, publishes `seq` into flag[me][slice] of every
//     peer (st.release.sys), waits until its own flag[peer][slice] words reach `seq`
//     (ld.acquire.sys, BOUNDED: after the limit it records a status code and skips the slice),
//     then reads the peers' slices with plain peer loads and combines them;
//   * sums use the balanced tree ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7)) in fp32 with a rounding to the
//     tensor dtype at every node -- the continuation of det_gemm's canonical K-chunk tree, so
//     TP = 1, 2, 4, 8 give identical bits.  Nothing here uses multimem reductions for sums: the
//     in-switch order and precision are not this contract.
//   * two frames alternate between calls; stream order plus the per-slice handshake make a frame
//     safe to reuse two calls later.
// No NCCL, no multicast TMA; only ld/st to peer pointers.  The design replaces the reference's
// CUDA-IPC collective (csrc/cuda/collectives/deterministic_collective.cu:109-1949), whose device
// waits are unbounded.
#include "rlk/host.h"
#include "rlk/ptx.cuh"
#include "rlk/symm.h"

#include <cstring>

namespace rlk {

constexpr int kMinSliceBytes = 32768;                   // payload bytes per slice (grows with the payload)
constexpr int kCollThreads = 256;

__device__ __forceinline__ unsigned long long effective_seq(const SymmWorld& w, unsigned long long base) {
  return w.use_epoch ? base + w.epoch[0] * w.epoch[1] : base;
}

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long* flag_ptr(unsigned char* win, int src, int slice) {
  return reinterpret_cast<unsigned long long*>(win) + src * kMaxSlices + slice;
}
__device__ __forceinline__ unsigned char* frame_ptr(unsigned char* win, long long frame_bytes, int f) {
  return win + kFlagBytes + f * frame_bytes;
}

// Publish "my slice is in my frame" to every peer and wait for theirs. Returns false on timeout.
__device__ __forceinline__ bool slice_handshake(const SymmWorld& w, int slice, unsigned long long seq,
                                                int* status, int code) {
  __shared__ int ok_flag;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < w.world) {
    const int peer = threadIdx.x;
    if (peer != w.rank) st_release_sys_u64(flag_ptr(w.win[peer], w.rank, slice), seq);
  }
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < w.world && threadIdx.x != w.rank) {
    const unsigned long long* f = flag_ptr(w.win[w.rank], threadIdx.x, slice);
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    while (ld_acquire_sys_u64(f) < seq) {
      if ((++it & 63) == 0 && globaltimer_ns() - t0 > RLK_WAIT_LIMIT_NS) {
        ok_flag = 0;
        if (status) atomicCAS(status, 0, code);
        break;
      }
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

template <int DT>  // 0 = bf16, 1 = fp32
__device__ __forceinline__ uint4 tree_node(const uint4 a, const uint4 b) {
  uint4 o;
  if (DT == 0) {
    o.x = pack_bf16x2(__fadd_rn(bf16_lo(a.x), bf16_lo(b.x)), __fadd_rn(bf16_hi(a.x), bf16_hi(b.x)));
    o.y = pack_bf16x2(__fadd_rn(bf16_lo(a.y), bf16_lo(b.y)), __fadd_rn(bf16_hi(a.y), bf16_hi(b.y)));
    o.z = pack_bf16x2(__fadd_rn(bf16_lo(a.z), bf16_lo(b.z)), __fadd_rn(bf16_hi(a.z), bf16_hi(b.z)));
    o.w = pack_bf16x2(__fadd_rn(bf16_lo(a.w), bf16_lo(b.w)), __fadd_rn(bf16_hi(a.w), bf16_hi(b.w)));
  } else {
    o.x = __float_as_uint(__fadd_rn(__uint_as_float(a.x), __uint_as_float(b.x)));
    o.y = __float_as_uint(__fadd_rn(__uint_as_float(a.y), __uint_as_float(b.y)));
    o.z = __float_as_uint(__fadd_rn(__uint_as_float(a.z), __uint_as_float(b.z)));
    o.w = __float_as_uint(__fadd_rn(__uint_as_float(a.w), __uint_as_float(b.w)));
  }
  return o;
}

// One-shot all-reduce: every rank reduces every slice itself (lowest latency; used for all sizes
// the engine needs -- activations of a decode step or a training micro-batch).
// staged != 0: the payload already sits in the local frame (a GEMM wrote it there).
template <int DT>
__device__ __forceinline__ void all_reduce_kernel_body(const SymmWorld w, const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                  long long nbytes, int slice_bytes, int frame, unsigned long long base_seq, int staged, int* status, int bx, int gx) {
  const unsigned long long seq = effective_seq(w, base_seq);
  const int nslices = static_cast<int>((nbytes + slice_bytes - 1) / slice_bytes);
  unsigned char* mine = frame_ptr(w.win[w.rank], w.frame_bytes, frame);
  for (int s = bx; s < nslices; s += gx) {
    const long long off = static_cast<long long>(s) * slice_bytes;
    const int n16 = static_cast<int>(min(static_cast<long long>(slice_bytes), nbytes - off) / 16);
    if (!staged)
      for (int i = threadIdx.x; i < n16; i += blockDim.x)
        reinterpret_cast<uint4*>(mine + off)[i] = reinterpret_cast<const uint4*>(src + off)[i];
    if (!slice_handshake(w, s, seq, status, 401)) continue;
    for (int i = threadIdx.x; i < n16; i += blockDim.x) {
      uint4 v[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < w.world)
          v[r] = (r == w.rank) ? reinterpret_cast<const uint4*>(mine + off)[i]
                               : ld_peer_v4(frame_ptr(w.win[r], w.frame_bytes, frame) + off + 16ll * i);
#pragma unroll
      for (int n = kMaxRanks; n > 1; n >>= 1)
        if (n <= w.world)
#pragma unroll
          for (int j = 0; j < n / 2; ++j) v[j] = tree_node<DT>(v[2 * j], v[2 * j + 1]);
      reinterpret_cast<uint4*>(dst + off)[i] = v[0];
    }
  }
}

template <int DT>
__global__ void __launch_bounds__(kCollThreads)
all_reduce_kernel(const SymmWorld w, const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                  long long nbytes, int slice_bytes, int frame, unsigned long long base_seq, int staged, int* status) {
  all_reduce_kernel_body<DT>(w, src, dst, nbytes, slice_bytes, frame, base_seq, staged, status, blockIdx.x, gridDim.x);
}

// Publish / wait for a single flag word of one slice (thread 0 of the CTA does the memory ops).
__device__ __forceinline__ void slice_publish(const SymmWorld& w, int slice, unsigned long long seq) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < w.world && threadIdx.x != w.rank)
    st_release_sys_u64(flag_ptr(w.win[threadIdx.x], w.rank, slice), seq);
}
// Wait until flag[src][slice] of this rank's window reaches seq, for every src with bit set in mask.
__device__ __forceinline__ bool slice_wait(const SymmWorld& w, int slice, unsigned long long seq, unsigned mask,
                                           int* status, int code) {
  __shared__ int ok2;
  if (threadIdx.x == 0) ok2 = 1;
  __syncthreads();
  if (threadIdx.x < w.world && ((mask >> threadIdx.x) & 1u)) {
    const unsigned long long* f = flag_ptr(w.win[w.rank], threadIdx.x, slice);
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    while (ld_acquire_sys_u64(f) < seq) {
      if ((++it & 63) == 0 && globaltimer_ns() - t0 > RLK_WAIT_LIMIT_NS) {
        ok2 = 0;
        if (status) atomicCAS(status, 0, code);
        break;
      }
    }
  }
  __syncthreads();
  return ok2 != 0;
}

// Two-shot all-reduce for large payloads: slice s is reduced by its owner (rank s % world) alone --
// it reads the other ranks' partials of that slice, runs the same balanced tree as the one-shot
// kernel, keeps the result in its own frame -- and the other ranks then copy the finished slice.
// Every rank moves 2 (W-1)/W of the payload over NVLink instead of (W-1) times the payload, and
// every element still sees exactly the tree ((r0+r1)+(r2+r3))+..., so the bits equal the one-shot
// kernel's.  Uses two flag values: seq_a = "my partial of this slice is in my frame",
// seq_b = "the reduced slice is in the owner's frame".
template <int DT, int W>
__device__ __forceinline__ void all_reduce_2shot_kernel_body(const SymmWorld w, const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                        long long nbytes, int slice_bytes, int frame, unsigned long long base_seq, int* status, int bx, int gx) {
  const unsigned long long seq_a = effective_seq(w, base_seq), seq_b = seq_a + 1;
  const int nslices = static_cast<int>((nbytes + slice_bytes - 1) / slice_bytes);
  unsigned char* mine = frame_ptr(w.win[w.rank], w.frame_bytes, frame);
  constexpr int U = 16 / W;   // independent 16-byte loads in flight per thread and rank
  // ---- phase 1: stage my partial of every slice this CTA handles
  for (int s = bx; s < nslices; s += gx) {
    const long long off = static_cast<long long>(s) * slice_bytes;
    const int n16 = static_cast<int>(min(static_cast<long long>(slice_bytes), nbytes - off) / 16);
    if (s % W != w.rank)   // the owner reads its own partial straight from src
      for (int i = threadIdx.x; i < n16; i += blockDim.x)
        reinterpret_cast<uint4*>(mine + off)[i] = reinterpret_cast<const uint4*>(src + off)[i];
    slice_publish(w, s, seq_a);
  }
  // ---- phase 2: reduce the slices I own
  for (int s = bx; s < nslices; s += gx) {
    if (s % W != w.rank) continue;
    const long long off = static_cast<long long>(s) * slice_bytes;
    const int n16 = static_cast<int>(min(static_cast<long long>(slice_bytes), nbytes - off) / 16);
    if (slice_wait(w, s, seq_a, ((1u << W) - 1u) & ~(1u << w.rank), status, 404)) {
      for (int i0 = threadIdx.x; i0 < n16; i0 += blockDim.x * U) {
        uint4 v[U][W];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = i0 + u * blockDim.x;
          if (i < n16) {
#pragma unroll
            for (int r = 0; r < W; ++r)
              v[u][r] = (r == w.rank) ? reinterpret_cast<const uint4*>(src + off)[i]
                                      : ld_peer_v4(frame_ptr(w.win[r], w.frame_bytes, frame) + off + 16ll * i);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = i0 + u * blockDim.x;
          if (i < n16) {
#pragma unroll
            for (int n = W; n > 1; n >>= 1)
#pragma unroll
              for (int j = 0; j < n / 2; ++j) v[u][j] = tree_node<DT>(v[u][2 * j], v[u][2 * j + 1]);
            reinterpret_cast<uint4*>(mine + off)[i] = v[u][0];
            reinterpret_cast<uint4*>(dst + off)[i] = v[u][0];
          }
        }
      }
    }
    slice_publish(w, s, seq_b);
  }
  // ---- phase 3: fetch the slices the others reduced
  for (int s = bx; s < nslices; s += gx) {
    const int owner = s % W;
    if (owner == w.rank) continue;
    const long long off = static_cast<long long>(s) * slice_bytes;
    const int n16 = static_cast<int>(min(static_cast<long long>(slice_bytes), nbytes - off) / 16);
    if (!slice_wait(w, s, seq_b, 1u << owner, status, 405)) continue;
    const unsigned char* pf = frame_ptr(w.win[owner], w.frame_bytes, frame) + off;
    for (int i0 = threadIdx.x; i0 < n16; i0 += blockDim.x * 8) {
      uint4 q[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < n16) q[u] = ld_peer_v4(pf + 16ll * i);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < n16) reinterpret_cast<uint4*>(dst + off)[i] = q[u];
      }
    }
  }
}

template <int DT, int W>
__global__ void __launch_bounds__(kCollThreads)
all_reduce_2shot_kernel(const SymmWorld w, const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                        long long nbytes, int slice_bytes, int frame, unsigned long long base_seq, int* status) {
  all_reduce_2shot_kernel_body<DT, W>(w, src, dst, nbytes, slice_bytes, frame, base_seq, status, blockIdx.x, gridDim.x);
}

// Reduce-scatter: the payload is `world` equal ranges; rank r ends with the balanced-tree sum of
// range r (dst holds per_rank bytes).  Every rank stages the ranges it does not own in its frame,
// the owner of a range pulls the peers' copies slice by slice -- half of the two-shot all-reduce.
template <int DT, int W>
__device__ __forceinline__ void reduce_scatter_kernel_body(const SymmWorld w, const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                      long long per_rank, int slice_bytes, int frame, unsigned long long base_seq, int* status, int bx, int gx) {
  const unsigned long long seq = effective_seq(w, base_seq);
  const int spr = static_cast<int>((per_rank + slice_bytes - 1) / slice_bytes);   // slices per range
  const int nslices = spr * W;
  unsigned char* mine = frame_ptr(w.win[w.rank], w.frame_bytes, frame);
  constexpr int U = 16 / W;
  for (int s = bx; s < nslices; s += gx) {
    const int owner = s / spr;
    const long long in_range = static_cast<long long>(s % spr) * slice_bytes;
    const long long off = owner * per_rank + in_range;
    const int n16 = static_cast<int>(min(static_cast<long long>(slice_bytes), per_rank - in_range) / 16);
    if (owner != w.rank)
      for (int i = threadIdx.x; i < n16; i += blockDim.x)
        reinterpret_cast<uint4*>(mine + off)[i] = reinterpret_cast<const uint4*>(src + off)[i];
    slice_publish(w, s, seq);
  }
  for (int i = 0; i < spr; ++i) {
    const int s = w.rank * spr + i;
    if (s % gx != bx) continue;
    const long long in_range = static_cast<long long>(i) * slice_bytes;
    const long long off = w.rank * per_rank + in_range;
    const int n16 = static_cast<int>(min(static_cast<long long>(slice_bytes), per_rank - in_range) / 16);
    if (!slice_wait(w, s, seq, ((1u << W) - 1u) & ~(1u << w.rank), status, 406)) continue;
    for (int i0 = threadIdx.x; i0 < n16; i0 += blockDim.x * U) {
      uint4 v[U][W];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = i0 + u * blockDim.x;
        if (k < n16) {
#pragma unroll
          for (int r = 0; r < W; ++r)
            v[u][r] = (r == w.rank) ? reinterpret_cast<const uint4*>(src + off)[k]
                                    : ld_peer_v4(frame_ptr(w.win[r], w.frame_bytes, frame) + off + 16ll * k);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = i0 + u * blockDim.x;
        if (k < n16) {
#pragma unroll
          for (int n = W; n > 1; n >>= 1)
#pragma unroll
            for (int j = 0; j < n / 2; ++j) v[u][j] = tree_node<DT>(v[u][2 * j], v[u][2 * j + 1]);
          reinterpret_cast<uint4*>(dst + in_range)[k] = v[u][0];
        }
      }
    }
  }
}

template <int DT, int W>
__global__ void __launch_bounds__(kCollThreads)
reduce_scatter_kernel(const SymmWorld w, const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                      long long per_rank, int slice_bytes, int frame, unsigned long long base_seq, int* status) {
  reduce_scatter_kernel_body<DT, W>(w, src, dst, per_rank, slice_bytes, frame, base_seq, status, blockIdx.x, gridDim.x);
}

// All-gather: dst[r] = rank r's payload (rank order).  Every CTA first stages and publishes all of
// its slices, then pulls the peers' copies with eight 16-byte loads in flight per thread, so the
// NVLink round trip is paid once per batch of loads instead of once per load.
__device__ __forceinline__ void all_gather_kernel_body(const SymmWorld w, const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                  long long nbytes, int slice_bytes, int frame, unsigned long long base_seq, int* status, int bx, int gx) {
  const unsigned long long seq = effective_seq(w, base_seq);
  const int nslices = static_cast<int>((nbytes + slice_bytes - 1) / slice_bytes);
  unsigned char* mine = frame_ptr(w.win[w.rank], w.frame_bytes, frame);
  for (int s = bx; s < nslices; s += gx) {
    const long long off = static_cast<long long>(s) * slice_bytes;
    const int n16 = static_cast<int>(min(static_cast<long long>(slice_bytes), nbytes - off) / 16);
    for (int i = threadIdx.x; i < n16; i += blockDim.x) {
      const uint4 v = reinterpret_cast<const uint4*>(src + off)[i];
      reinterpret_cast<uint4*>(mine + off)[i] = v;
      reinterpret_cast<uint4*>(dst + w.rank * nbytes + off)[i] = v;
    }
    slice_publish(w, s, seq);
  }
  const unsigned others = ((1u << w.world) - 1u) & ~(1u << w.rank);
  for (int s = bx; s < nslices; s += gx) {
    const long long off = static_cast<long long>(s) * slice_bytes;
    const int n16 = static_cast<int>(min(static_cast<long long>(slice_bytes), nbytes - off) / 16);
    if (!slice_wait(w, s, seq, others, status, 402)) continue;
    for (int r = 0; r < w.world; ++r) {
      if (r == w.rank) continue;
      const unsigned char* pf = frame_ptr(w.win[r], w.frame_bytes, frame) + off;
      unsigned char* out = dst + r * nbytes + off;
      for (int i0 = threadIdx.x; i0 < n16; i0 += blockDim.x * 8) {
        uint4 q[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * blockDim.x;
          if (i < n16) q[u] = ld_peer_v4(pf + 16ll * i);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * blockDim.x;
          if (i < n16) reinterpret_cast<uint4*>(out)[i] = q[u];
        }
      }
    }
  }
}

__global__ void __launch_bounds__(kCollThreads)
all_gather_kernel(const SymmWorld w, const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                  long long nbytes, int slice_bytes, int frame, unsigned long long base_seq, int* status) {
  all_gather_kernel_body(w, src, dst, nbytes, slice_bytes, frame, base_seq, status, blockIdx.x, gridDim.x);
}

// Single-GPU emulation of a W-rank group for testing the W = 4 and W = 8 code paths without W
// GPUs: all ranks' windows live on this device and ONE cooperative kernel runs every rank's CTAs
// (blockIdx.y = rank), so the CTAs that wait on one another are guaranteed to be resident together.
// mode: 0 one-shot all-reduce, 1 two-shot all-reduce, 2 reduce-scatter, 3 all-gather.
struct EmulArgs {
  SymmWorld w[kMaxRanks];
  const unsigned char* src[kMaxRanks];
  unsigned char* dst[kMaxRanks];
};

template <int DT, int W>
__global__ void __launch_bounds__(kCollThreads)
emulate_kernel(const EmulArgs a, int mode, long long nbytes, int slice_bytes, int* status) {
  const int r = blockIdx.y;
  if (mode == 0) all_reduce_kernel_body<DT>(a.w[r], a.src[r], a.dst[r], nbytes, slice_bytes, 1, 1ull, 0, status, blockIdx.x, gridDim.x);
  else if (mode == 1) all_reduce_2shot_kernel_body<DT, W>(a.w[r], a.src[r], a.dst[r], nbytes, slice_bytes, 1, 1ull, status, blockIdx.x, gridDim.x);
  else if (mode == 2) reduce_scatter_kernel_body<DT, W>(a.w[r], a.src[r], a.dst[r], nbytes / W, slice_bytes, 1, 1ull, status, blockIdx.x, gridDim.x);
  else all_gather_kernel_body(a.w[r], a.src[r], a.dst[r], nbytes, slice_bytes, 1, 1ull, status, blockIdx.x, gridDim.x);
}

// Bounded barrier across ranks: everyone publishes seq in slice 0 of a dedicated flag row.
__global__ void barrier_kernel(const SymmWorld w, unsigned long long base_seq, int* status) {
  slice_handshake(w, kMaxSlices - 1, effective_seq(w, base_seq), status, 403);
}

__global__ void epoch_bump_kernel(unsigned long long* epoch) { epoch[0] += 1; }

}  // namespace rlk
using namespace rlk;

RLK_API long long rlk_symm_window_bytes(long long frame_bytes) { return kFlagBytes + 2 * frame_bytes; }
RLK_API int rlk_symm_ipc_handle_bytes() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

// Allocates this rank's window (zeroed) and writes its IPC handle into handle_out.
RLK_API int rlk_symm_alloc(long long frame_bytes, void** window_out, void* handle_out) {
  RLK_REQUIRE(frame_bytes > 0 && frame_bytes % 256 == 0, "symm_alloc: frame_bytes must be a positive multiple of 256");
  void* p = nullptr;
  RLK_CHECK_CUDA(cudaMalloc(&p, rlk_symm_window_bytes(frame_bytes)));
  RLK_CHECK_CUDA(cudaMemset(p, 0, rlk_symm_window_bytes(frame_bytes)));
  RLK_CHECK_CUDA(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  RLK_CHECK_CUDA(cudaIpcGetMemHandle(&h, p));
  memcpy(handle_out, &h, sizeof(h));
  *window_out = p;
  return RLK_OK;
}

// handles: world * handle_bytes, rank order. Returns an opaque state pointer in state_out.
RLK_API int rlk_symm_create(void* local_window, const void* handles, int world, int rank,
                            long long frame_bytes, void** state_out) {
  RLK_REQUIRE(world >= 1 && world <= kMaxRanks && (world & (world - 1)) == 0, "symm_create: world must be 1, 2, 4 or 8");
  RLK_REQUIRE(rank >= 0 && rank < world, "symm_create: bad rank");
  SymmState* st = new SymmState();
  memset(st, 0, sizeof(*st));
  RLK_CHECK_CUDA(cudaGetDevice(&st->device));
  st->local = static_cast<unsigned char*>(local_window);
  st->w.world = world;
  st->w.rank = rank;
  st->w.frame_bytes = frame_bytes;
  for (int r = 0; r < world; ++r) {
    if (r == rank) {
      st->peers[r] = st->local;
    } else {
      cudaIpcMemHandle_t h;
      memcpy(&h, static_cast<const unsigned char*>(handles) + r * sizeof(h), sizeof(h));
      void* p = nullptr;
      cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        delete st;
        return set_error(RLK_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d) failed: %s", r, cudaGetErrorString(e));
      }
      st->peers[r] = static_cast<unsigned char*>(p);
    }
    st->w.win[r] = st->peers[r];
  }
  st->seq = 0;
  RLK_CHECK_CUDA(cudaMalloc(&st->dev_epoch, 16));
  RLK_CHECK_CUDA(cudaMemset(st->dev_epoch, 0, 16));
  st->w.epoch = st->dev_epoch;
  st->w.use_epoch = 0;
  *state_out = st;
  return RLK_OK;
}

RLK_API int rlk_symm_destroy(void* state, int free_local) {
  SymmState* st = static_cast<SymmState*>(state);
  if (!st) return RLK_OK;
  for (int r = 0; r < st->w.world; ++r)
    if (r != st->w.rank && st->peers[r]) cudaIpcCloseMemHandle(st->peers[r]);
  if (free_local && st->local) cudaFree(st->local);
  if (st->dev_epoch) cudaFree(st->dev_epoch);
  delete st;
  return RLK_OK;
}

// Device pointer of frame f of rank r's window as mapped in this process.
RLK_API void* rlk_symm_frame_ptr(void* state, int r, int f) {
  SymmState* st = static_cast<SymmState*>(state);
  return st->peers[r] + kFlagBytes + f * st->w.frame_bytes;
}
RLK_API int rlk_symm_next_frame(void* state) {
  return static_cast<int>((static_cast<SymmState*>(state)->seq + 1) & 1);
}

static int slice_bytes_for(long long nbytes) {
  long long sb = kMinSliceBytes;
  while ((nbytes + sb - 1) / sb > 1024) sb *= 2;
  return static_cast<int>(sb);
}
constexpr long long kTwoShotMinBytes = 4ll << 20;
static int coll_grid_large(long long nbytes) {
  const long long sl = (nbytes + slice_bytes_for(nbytes) - 1) / slice_bytes_for(nbytes);
  const int cap = 2 * sm_count();      // two CTAs per SM keep enough peer loads in flight
  return static_cast<int>(sl < cap ? sl : cap);
}
static int coll_grid(long long nbytes) {
  const long long s = (nbytes + slice_bytes_for(nbytes) - 1) / slice_bytes_for(nbytes);
  const int cap = nbytes > (8 << 20) ? 128 : 64;  // small payloads: leave SMs to overlapping compute
  return static_cast<int>(s < cap ? (s < 1 ? 1 : s) : cap);
}

// dtype: 0 = bf16, 1 = fp32. staged: src is ignored, the payload is already in the frame returned
// by rlk_symm_next_frame() (written there by the producing kernel on the same stream).
RLK_API int rlk_symm_all_reduce(void* state, const void* src, void* dst, long long nbytes, int dtype,
                                int staged, void* stream) {
  SymmState* st = static_cast<SymmState*>(state);
  RLK_REQUIRE(nbytes > 0 && nbytes % 16 == 0, "all_reduce: byte count must be a positive multiple of 16");
  RLK_REQUIRE(nbytes <= st->w.frame_bytes, "all_reduce: %lld bytes exceed the frame capacity %lld", nbytes, st->w.frame_bytes);
  RLK_REQUIRE(dtype == 0 || dtype == 1, "all_reduce: dtype must be 0 (bf16) or 1 (fp32)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned char* sp = static_cast<const unsigned char*>(src);
  unsigned char* dp = static_cast<unsigned char*>(dst);
  if (!staged && nbytes >= kTwoShotMinBytes && st->w.world > 1) {
    // large payload: reduce-scatter + all-gather over the same tree.  Three sequence numbers are
    // consumed (two are used as flag values) so that consecutive calls keep alternating frames.
    st->seq += 1;
    const int frame2 = static_cast<int>(st->seq & 1);
    const unsigned long long base = st->seq;
    st->seq += 2;
    const int sb = slice_bytes_for(nbytes);
    const int grid = coll_grid_large(nbytes);
    int* stw = device_status_word();
#define RLK_LAUNCH_2SHOT(DT, WW) all_reduce_2shot_kernel<DT, WW><<<grid, kCollThreads, 0, s>>>(st->w, sp, dp, nbytes, sb, frame2, base, stw)
    if (dtype == 0) {
      if (st->w.world == 2) RLK_LAUNCH_2SHOT(0, 2); else if (st->w.world == 4) RLK_LAUNCH_2SHOT(0, 4); else RLK_LAUNCH_2SHOT(0, 8);
    } else {
      if (st->w.world == 2) RLK_LAUNCH_2SHOT(1, 2); else if (st->w.world == 4) RLK_LAUNCH_2SHOT(1, 4); else RLK_LAUNCH_2SHOT(1, 8);
    }
#undef RLK_LAUNCH_2SHOT
    RLK_CHECK_CUDA(cudaGetLastError());
    return RLK_OK;
  }
  st->seq += 1;
  const int frame = static_cast<int>(st->seq & 1);
  if (dtype == 0)
    all_reduce_kernel<0><<<coll_grid(nbytes), kCollThreads, 0, s>>>(st->w, sp, dp, nbytes, slice_bytes_for(nbytes), frame, st->seq, staged, device_status_word());
  else
    all_reduce_kernel<1><<<coll_grid(nbytes), kCollThreads, 0, s>>>(st->w, sp, dp, nbytes, slice_bytes_for(nbytes), frame, st->seq, staged, device_status_word());
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// src: world * per_rank bytes (range r belongs to rank r); dst: per_rank bytes.
RLK_API int rlk_symm_reduce_scatter(void* state, const void* src, void* dst, long long per_rank, int dtype,
                                    void* stream) {
  SymmState* st = static_cast<SymmState*>(state);
  const int W = st->w.world;
  RLK_REQUIRE(per_rank > 0 && per_rank % 16 == 0, "reduce_scatter: bytes per rank must be a positive multiple of 16");
  RLK_REQUIRE(per_rank * W <= st->w.frame_bytes, "reduce_scatter: %lld bytes exceed the frame capacity %lld", per_rank * W, st->w.frame_bytes);
  RLK_REQUIRE(dtype == 0 || dtype == 1, "reduce_scatter: dtype must be 0 (bf16) or 1 (fp32)");
  RLK_REQUIRE(W == 2 || W == 4 || W == 8, "reduce_scatter: world must be 2, 4 or 8");
  st->seq += 1;
  const int frame = static_cast<int>(st->seq & 1);
  const unsigned long long base = st->seq;
  long long sb = kMinSliceBytes;
  while (((per_rank + sb - 1) / sb) * W > kMaxSlices - 1) sb *= 2;
  const long long nsl = ((per_rank + sb - 1) / sb) * W;
  const int cap = per_rank * W >= kTwoShotMinBytes ? 2 * sm_count() : 64;
  const int grid = static_cast<int>(nsl < cap ? nsl : cap);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned char* sp = static_cast<const unsigned char*>(src);
  unsigned char* dp = static_cast<unsigned char*>(dst);
  int* stw = device_status_word();
#define RLK_LAUNCH_RS(DT, WW) reduce_scatter_kernel<DT, WW><<<grid, kCollThreads, 0, s>>>(st->w, sp, dp, per_rank, static_cast<int>(sb), frame, base, stw)
  if (dtype == 0) {
    if (W == 2) RLK_LAUNCH_RS(0, 2); else if (W == 4) RLK_LAUNCH_RS(0, 4); else RLK_LAUNCH_RS(0, 8);
  } else {
    if (W == 2) RLK_LAUNCH_RS(1, 2); else if (W == 4) RLK_LAUNCH_RS(1, 4); else RLK_LAUNCH_RS(1, 8);
  }
#undef RLK_LAUNCH_RS
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_symm_all_gather(void* state, const void* src, void* dst, long long nbytes, void* stream) {
  SymmState* st = static_cast<SymmState*>(state);
  RLK_REQUIRE(nbytes > 0 && nbytes % 16 == 0, "all_gather: byte count must be a positive multiple of 16");
  RLK_REQUIRE(nbytes <= st->w.frame_bytes, "all_gather: %lld bytes exceed the frame capacity %lld", nbytes, st->w.frame_bytes);
  st->seq += 1;
  const int frame = static_cast<int>(st->seq & 1);
  all_gather_kernel<<<nbytes >= kTwoShotMinBytes ? coll_grid_large(nbytes) : coll_grid(nbytes), kCollThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      st->w, static_cast<const unsigned char*>(src), static_cast<unsigned char*>(dst), nbytes,
      slice_bytes_for(nbytes), frame, st->seq, device_status_word());
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API int rlk_symm_barrier(void* state, void* stream) {
  SymmState* st = static_cast<SymmState*>(state);
  st->seq += 1;
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(st->w, st->seq, device_status_word());
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// ---- CUDA-graph protocol (all ranks must do the same):
//   rlk_symm_graph_begin(state, capture_stream)      first thing inside the capture
//   ... collectives on the capture stream ...
//   n = rlk_symm_graph_end(state, capture_stream)    last thing inside the capture
//   rlk_symm_graph_commit(state)                     after the capture has ended, before a replay
//   rlk_symm_graph_replayed(state, k)                after k replays were enqueued
RLK_API int rlk_symm_graph_begin(void* state, void* stream) {
  SymmState* st = static_cast<SymmState*>(state);
  RLK_REQUIRE(!st->capturing, "symm_graph_begin: a capture is already open");
  st->capturing = 1;
  st->w.use_epoch = 1;
  st->capture_begin_seq = st->seq;
  epoch_bump_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(st->dev_epoch);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

RLK_API long long rlk_symm_graph_end(void* state, void* stream) {
  SymmState* st = static_cast<SymmState*>(state);
  if (!st->capturing) return -1;
  if ((st->seq - st->capture_begin_seq) & 1) rlk_symm_barrier(state, stream);  // keep the stride even
  st->graph_stride = st->seq - st->capture_begin_seq;
  st->capturing = 0;
  st->w.use_epoch = 0;
  return static_cast<long long>(st->graph_stride);
}

RLK_API int rlk_symm_graph_commit(void* state) {
  SymmState* st = static_cast<SymmState*>(state);
  const unsigned long long vals[2] = {0ull, st->graph_stride};
  RLK_CHECK_CUDA(cudaMemcpy(st->dev_epoch, vals, 16, cudaMemcpyHostToDevice));
  return RLK_OK;
}

RLK_API int rlk_symm_graph_replayed(void* state, long long times) {
  SymmState* st = static_cast<SymmState*>(state);
  st->seq += static_cast<unsigned long long>(times) * st->graph_stride;
  return RLK_OK;
}

// Sequence-number access for recovery after a timed-out collective: the ranks agree on the
// maximum over the host (torch.distributed) and continue from there.
RLK_API long long rlk_symm_get_seq(void* state) { return static_cast<long long>(static_cast<SymmState*>(state)->seq); }
RLK_API int rlk_symm_set_seq(void* state, long long seq) {
  static_cast<SymmState*>(state)->seq = static_cast<unsigned long long>(seq);
  return RLK_OK;
}

// Test entry: runs `mode` for a group of `world` emulated ranks on the current device.  srcs / dsts
// hold one device pointer per rank (all-reduce: nbytes each; reduce-scatter: dst nbytes / world;
// all-gather: dst world * nbytes).  Allocates and frees its own windows; synchronises the stream.
RLK_API int rlk_symm_emulate(int world, int mode, long long nbytes, int dtype, void* const* srcs,
                             void* const* dsts, void* stream) {
  RLK_REQUIRE(world == 2 || world == 4 || world == 8, "symm_emulate: world must be 2, 4 or 8");
  RLK_REQUIRE(mode >= 0 && mode <= 3 && nbytes > 0 && nbytes % (16 * world) == 0, "symm_emulate: bad arguments");
  RLK_REQUIRE(dtype == 0 || dtype == 1, "symm_emulate: dtype must be 0 (bf16) or 1 (fp32)");
  const long long frame_bytes = (nbytes + 255) / 256 * 256;
  EmulArgs a{};
  unsigned char* wins[kMaxRanks] = {nullptr};
  for (int r = 0; r < world; ++r) {
    RLK_CHECK_CUDA(cudaMalloc(&wins[r], rlk_symm_window_bytes(frame_bytes)));
    RLK_CHECK_CUDA(cudaMemset(wins[r], 0, kFlagBytes));
  }
  for (int r = 0; r < world; ++r) {
    for (int q = 0; q < kMaxRanks; ++q) a.w[r].win[q] = wins[q < world ? q : 0];
    a.w[r].world = world;
    a.w[r].rank = r;
    a.w[r].frame_bytes = frame_bytes;
    a.w[r].epoch = nullptr;
    a.w[r].use_epoch = 0;
    a.src[r] = static_cast<const unsigned char*>(srcs[r]);
    a.dst[r] = static_cast<unsigned char*>(dsts[r]);
  }
  long long payload = mode == 2 ? nbytes / world : nbytes;
  long long sb = kMinSliceBytes;
  while (((payload + sb - 1) / sb) * (mode == 2 ? world : 1) > 1024) sb *= 2;
  const long long nsl = ((payload + sb - 1) / sb) * (mode == 2 ? world : 1);
  // every CTA of every rank must be resident at once: a small grid per rank
  int gx = static_cast<int>(nsl < 8 ? nsl : 8);
  int slice = static_cast<int>(sb);
  int* stw = device_status_word();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  void* args[] = {&a, &mode, &nbytes, &slice, &stw};
  const void* fn = nullptr;
#define RLK_EMUL(DT, WW) fn = reinterpret_cast<const void*>(&emulate_kernel<DT, WW>)
  if (dtype == 0) { if (world == 2) RLK_EMUL(0, 2); else if (world == 4) RLK_EMUL(0, 4); else RLK_EMUL(0, 8); }
  else { if (world == 2) RLK_EMUL(1, 2); else if (world == 4) RLK_EMUL(1, 4); else RLK_EMUL(1, 8); }
#undef RLK_EMUL
  cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(gx, world), dim3(kCollThreads), args, 0, st);
  cudaError_t e2 = cudaStreamSynchronize(st);
  for (int r = 0; r < world; ++r) cudaFree(wins[r]);
  RLK_CHECK_CUDA(e);
  RLK_CHECK_CUDA(e2);
  return RLK_OK;
}
