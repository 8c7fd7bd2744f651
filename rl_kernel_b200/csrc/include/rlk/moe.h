// Records shared by the mixture-of-experts routing kernels and the grouped GEMM.
#pragma once

namespace rlk {

// One 128 x 256 output tile of a grouped GEMM.  Coordinates are element indices into the 2-D
// operand tensors; the expert only appears as an offset.
struct GroupTile {
  int a_m0;        // first MN index of the tile in A (row for K-major A, column for MN-major A)
  int b_n0;        // first MN index of the tile in B
  int ka0;         // first K index in A
  int kb0;         // first K index in B
  int kblocks;     // number of 64-wide K blocks (0: nothing to do, C is left untouched)
  int c_row;       // first output row
  int c_col;       // first output column
  int rows_valid;  // rows of the tile that are stored (1..128)
};

// Device pointers of the same buffer on every expert-parallel rank (index = rank; this rank's own
// pointer at its own index).  Unused entries repeat entry 0.
struct PeerPtrs {
  void* p[8];
};

}  // namespace rlk
