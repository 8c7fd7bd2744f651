// Work-item description shared by the attention forward and backward kernels.
//
// Attention runs over "tiles" of up to 128 query rows that all read keys from one contiguous
// run of rows of the K/V tensors (one sequence, one KV head).  Training (packed varlen),
// prefill, single-token decode against a KV cache (the 4 query heads of a GQA group become 4
// rows of one tile) and context-parallel shards are all expressed as lists of such tiles, so
// every mode executes the same per-row program:
//   * keys are consumed in canonical blocks of 128, block b = keys [128 b, 128 b + 128) counted
//     from the first key of the sequence, in ascending b;
//   * row r sees keys j < kv_len(r) = min(kv_cap, pos0 + r * pos_step + 1);
//   * a block that is completely masked for a row leaves that row's state bit-for-bit unchanged.
// That is what makes selected-token log-probs of rollout (decode) and training (full sequence)
// bitwise equal, for every batch size and query tiling.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#ifdef __CUDACC__
#include "rlk/ptx.cuh"
#endif

namespace rlk {

struct AttnTile {
  int q_row0;    // first query row: y coordinate in the Q / O / dO tensor maps
  int q_col0;    // x coordinate of the head in Q / O (elements)
  int n_rows;    // valid query rows in this tile (1..128); 0 = empty tile
  int kv_row0;   // y coordinate of key 0 of the sequence in the K / V tensor maps
  int kv_col0;   // x coordinate of the KV head in K / V (elements)
  int pos0;      // position (key index) of query row 0
  int pos_step;  // 1: consecutive rows are consecutive positions; 0: all rows share pos0
  int kv_cap;    // number of keys that exist (kv_len never exceeds it)
  int lse_off;   // lse[lse_off + r * lse_stride] receives row r's log-sum-exp
  int lse_stride;
  int kv_src;    // index into the K/V tensor-map table (context parallel: owning rank); 0 otherwise
  int reserved;
};

constexpr int kAttnBlock = 128;  // canonical KV block and query tile
constexpr int kHeadDim = 128;

// One tensor map per context-parallel rank for a pair of operands that are fetched together
// (K and V in the forward and dQ kernels, Q and dO in the dK/dV kernel).
template <int NSRC>
struct KvMaps {
  CUtensorMap k[NSRC];
  CUtensorMap v[NSRC];
};

// How the 128-token blocks of one sequence are spread over context-parallel ranks.  Every rank
// stores its blocks of a sequence back to back, so "local block i" is row 128*i after the
// sequence's first local row.  contiguous: the sequence is cut into `ranks` chunks of
// `blocks_per_chunk` blocks, chunk c on rank c.  zigzag: 2*ranks chunks, rank c holds chunks c and
// 2*ranks-1-c (in that order), which balances causal work.
struct CpLayout {
  int ranks;             // <= 1: not context parallel
  int blocks_per_chunk;
  int zigzag;
};

__host__ __device__ __forceinline__ void cp_locate_block(const CpLayout& c, int b, int& src, int& local_block) {
  if (c.ranks <= 1) {
    src = 0;
    local_block = b;
    return;
  }
  const int chunk = b / c.blocks_per_chunk;
  const int within = b - chunk * c.blocks_per_chunk;
  int local_chunk = 0;
  if (c.zigzag) {
    if (chunk < c.ranks) {
      src = chunk;
    } else {
      src = 2 * c.ranks - 1 - chunk;
      local_chunk = 1;
    }
  } else {
    src = chunk;
  }
  local_block = local_chunk * c.blocks_per_chunk + within;
}

// ---------------------------------------------------------------------------------------------
// Context-parallel staging.  A remote K/V (or Q/dO) block is needed by many work items of a rank;
// fetching it over NVLink every time makes the kernel NVLink-bound at long sequences.  With
// staging, the compute warps of the CTAs that start first copy every remote 128-row block ONCE
// into this GPU's memory (work items from an atomic counter, 16-byte peer loads, eight in flight per
// thread) and publish a ready flag per block; the TMA producers of all CTAs then read remote blocks
// from the local copy after a bounded wait on that flag.  Two operands ("a" and "b": K and V, or Q
// and dO) are staged side by side.  flags: [ranks * blocks * 2] ready words followed by the work
// counter, all zero at launch.
struct CpStage {
  const unsigned char* src_a[8];   // every rank's operand a (this rank's own at its index), row-major, same pitch
  const unsigned char* src_b[8];
  unsigned char* dst_a;            // local staging [ranks * rows, row_bytes]
  unsigned char* dst_b;
  int* flags;
  int rows;                        // rows staged per rank (multiple of 128); 0 = staging off
  int row_bytes_a, row_bytes_b;
  int ranks, rank;
};

#ifdef __CUDACC__
// Called by `nthreads` threads of a CTA (thread index tid, named barrier `bar_id`, one int of shared
// scratch).  Returns when no work items are left.
__device__ __forceinline__ void cp_stage_gather(const CpStage& st, int tid, int nthreads, int bar_id,
                                                volatile int* slot) {
  if (st.rows <= 0 || st.ranks <= 1) return;
  const int nb = st.rows / 128;
  const int n_items = (st.ranks - 1) * nb * 2;
  int* work = st.flags + st.ranks * nb * 2;
  while (true) {
    if (tid == 0) *slot = atomicAdd(work, 1);
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
    const int item = *slot;
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
    if (item >= n_items) break;
    const int which = item & 1;
    const int blk = (item >> 1) % nb;
    const int src = (st.rank + 1 + (item >> 1) / nb) % st.ranks;   // ring order: next rank first
    const long long row_bytes = which ? st.row_bytes_b : st.row_bytes_a;
    const unsigned char* from = (which ? st.src_b[src] : st.src_a[src]) + static_cast<long long>(blk) * 128 * row_bytes;
    unsigned char* to = (which ? st.dst_b : st.dst_a) +
                        (static_cast<long long>(src) * st.rows + static_cast<long long>(blk) * 128) * row_bytes;
    const long long n16 = 128 * row_bytes / 16;
    for (long long v0 = tid; v0 < n16; v0 += static_cast<long long>(nthreads) * 8) {
      uint4 q[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const long long v = v0 + static_cast<long long>(u) * nthreads;
        if (v < n16)
          asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(q[u].x), "=r"(q[u].y), "=r"(q[u].z), "=r"(q[u].w)
                       : "l"(reinterpret_cast<const uint4*>(from) + v) : "memory");
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const long long v = v0 + static_cast<long long>(u) * nthreads;
        if (v < n16) reinterpret_cast<uint4*>(to)[v] = q[u];
      }
    }
    __threadfence();
    asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy stores, later read by TMA
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
    if (tid == 0) {
      int* f = st.flags + (src * nb + blk) * 2 + which;
      asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(f), "r"(1) : "memory");
    }
  }
}

// Producer side: wait (bounded) until both operands of remote block `blk` of rank `src` are staged.
__device__ __forceinline__ bool cp_stage_wait(const CpStage& st, int src, int blk, volatile int* abort_flag,
                                              int* status, int code) {
  const int nb = st.rows / 128;
  const int* f = st.flags + (src * nb + blk) * 2;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    int a, b;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(a) : "l"(f) : "memory");
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(b) : "l"(f + 1) : "memory");
    if (a > 0 && b > 0) break;
    if ((++spins & 63) == 0 && (*abort_flag || globaltimer_ns() - t0 > RLK_WAIT_LIMIT_NS)) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
  asm volatile("fence.proxy.async;" ::: "memory");
  return true;
}
#endif

}  // namespace rlk
