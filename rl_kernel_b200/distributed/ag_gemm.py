"""All-gather -> GEMM as one kernel (sequence-parallel activations into a column-parallel weight).

Each tensor-parallel rank writes its M / W rows of the activation into its slice of a peer-mapped
[M, K] buffer; ``AllGatherGemm`` then launches csrc/gemm/ag_gemm_sm100.cu, whose gather warps pull
the other slices over NVLink while the tensor-core pipeline already multiplies the rows that are
present.  Output bits equal ``det_gemm`` on the gathered matrix.  (Reference: NCCL all-gather of
the tokens followed by the GEMM, rl_engine/backends/cuda/ffn/ffn.py:601-603.)
"""
from __future__ import annotations

import ctypes

import torch

from rl_kernel_b200.backends import extension as ext
from rl_kernel_b200.backends import native as nv
from rl_kernel_b200.distributed.cp_attention import PeerMappedBuffers


class AllGatherGemm:
    def __init__(self, collective, device: torch.device, M: int, K: int):
        self.coll, self.device, self.M, self.K = collective, device, M, K
        self.world, self.rank = collective.world, collective.rank
        if M % (self.world * 128) or K % 64:
            raise ValueError("M must be a multiple of world * 128 and K a multiple of 64")
        self.rows = M // self.world
        self.bufs = PeerMappedBuffers(collective.group, device, {"a": ((M, K), torch.bfloat16)})
        lib = ext.load()
        lib.rlk_ag_gemm_scratch_ints.restype = ctypes.c_longlong
        self.scratch = torch.zeros(int(lib.rlk_ag_gemm_scratch_ints(ctypes.c_int(M))), dtype=torch.int32, device=device)

    @property
    def local_shard(self) -> torch.Tensor:
        """[M / W, K] view the producer of this rank's rows writes into."""
        return self.bufs.local("a")[self.rank * self.rows:(self.rank + 1) * self.rows]

    @property
    def gathered(self) -> torch.Tensor:
        """[M, K]: complete after ``__call__`` (needed again by the backward's weight gradient)."""
        return self.bufs.local("a")

    def __call__(self, b: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[M, N] = gathered A @ b[N, K]^T."""
        lib = ext.load()
        ptrs = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in self.bufs["a"]])
        self.coll.barrier()                       # every rank's shard is written
        ext.check(lib.rlk_ag_gemm(ptrs, ctypes.c_int(self.world), ctypes.c_int(self.rank), ctypes.c_int(self.M),
                                  ctypes.c_int(b.shape[0]), ctypes.c_int(self.K), ext.ptr(b),
                                  ctypes.c_longlong(b.stride(0)), ext.ptr(out), ctypes.c_longlong(out.stride(0)),
                                  ext.ptr(self.scratch), ext.stream_ptr(self.device)), "ag_gemm")
        nv._count()
        self.coll.barrier()                       # shards may be overwritten again
        return out
