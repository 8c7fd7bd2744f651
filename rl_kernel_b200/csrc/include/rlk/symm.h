// Layout of a symmetric-memory window and the host-side state of a collective group, shared by
// the stand-alone collectives (collectives/symm_collectives.cu) and the kernels that fuse a
// collective into their epilogue (gemm/det_gemm_sm100.cu).
#pragma once
#include <stdint.h>

namespace rlk {

constexpr int kMaxRanks = 8;
constexpr int kMaxSlices = 8192;                        // flag slots per source rank
constexpr int kFlagBytes = kMaxRanks * kMaxSlices * 8;  // u64 flag[src_rank][slot]

struct SymmWorld {
  unsigned char* win[kMaxRanks];  // window base of every rank (own entry = local pointer)
  int world, rank;
  long long frame_bytes;
  // CUDA-graph support: a captured kernel's sequence number is base + epoch * stride, where epoch
  // (device word 0) is bumped once per replay and stride (device word 1) is the EVEN number of
  // collective calls in the graph, so the frame parity of every captured call is fixed.
  const unsigned long long* epoch;
  int use_epoch;
};

struct SymmState {
  SymmWorld w;
  unsigned char* local;
  unsigned char* peers[kMaxRanks];
  unsigned long long seq;
  int device;
  unsigned long long* dev_epoch;       // [epoch, stride]
  int capturing;
  unsigned long long capture_begin_seq;
  unsigned long long graph_stride;
};

}  // namespace rlk
