"""Context-parallel causal attention with the KV exchange inside the kernel.

Every CP rank keeps the K/V of its own sequence positions in a buffer that its peers have mapped
(CUDA IPC over NVLink).  The attention kernel of a rank walks the canonical 128-key blocks of a
query tile in ascending order and loads each block straight from the rank that owns it with a
plain (non-multicast) TMA load through that peer's tensor map (csrc/attention/attn_fwd_sm100.cu,
NSRC = 8).  Nothing is gathered beforehand and no partial results are merged afterwards: a query
row executes exactly the single-GPU program, so the output is bitwise equal to CP = 1 for every CP
degree and layout.  (The reference all-gathers Q/K/V, lets every rank compute the whole sequence
and scatters rank 0's result: rl_engine/backends/cuda/attention/cp_comm.py:444-566.)

Layouts: ``contiguous`` (rank c owns positions [c*S/cp, (c+1)*S/cp)) and ``zigzag`` (2*cp chunks,
rank c owns chunks c and 2*cp-1-c: balanced causal work, Megatron's layout).
"""
from __future__ import annotations

import ctypes
import math

import torch

from rl_kernel_b200.backends import extension as ext
from rl_kernel_b200.backends import native as nv
from rl_kernel_b200.distributed.transports.symm import _DevicePtrView


def cp_positions(seq_len: int, cp: int, rank: int, layout: str) -> torch.Tensor:
    """Global positions of the tokens rank ``rank`` holds, in its local order."""
    if cp == 1:
        return torch.arange(seq_len)
    if layout == "contiguous":
        c = seq_len // cp
        return torch.arange(rank * c, (rank + 1) * c)
    c = seq_len // (2 * cp)
    return torch.cat([torch.arange(rank * c, (rank + 1) * c), torch.arange((2 * cp - 1 - rank) * c, (2 * cp - rank) * c)])


class CPAttention:
    def __init__(self, collective, device: torch.device, *, num_q_heads: int, num_kv_heads: int, head_dim: int = 128,
                 max_local_tokens: int, layout: str = "zigzag"):
        if layout not in ("zigzag", "contiguous"):
            raise ValueError(layout)
        if head_dim != 128:
            raise ValueError("head_dim must be 128")
        self.coll, self.device, self.layout = collective, device, layout
        self.cp, self.rank = collective.world, collective.rank
        self.hq, self.hkv, self.d = num_q_heads, num_kv_heads, head_dim
        self.max_tokens = max_local_tokens
        self.scale = 1.0 / math.sqrt(head_dim)
        lib = ext.load()
        nbytes = max_local_tokens * num_kv_heads * head_dim * 2
        self._bufs = []
        handles = []
        for _ in range(2):                                   # K and V
            h = ctypes.create_string_buffer(lib.rlk_symm_ipc_handle_bytes())
            p = ctypes.c_void_p(0)
            with torch.cuda.device(device):
                ext.check(lib.rlk_ipc_alloc(ctypes.c_longlong(nbytes), ctypes.byref(p), h), "ipc_alloc")
            self._bufs.append(p.value)
            handles.append(bytes(h.raw))
        import torch.distributed as dist

        gathered = [None] * self.cp
        dist.all_gather_object(gathered, handles, group=collective.group)
        self._peer_ptrs = [[], []]
        for r in range(self.cp):
            for i in range(2):
                if r == self.rank:
                    self._peer_ptrs[i].append(self._bufs[i])
                else:
                    p = ctypes.c_void_p(0)
                    with torch.cuda.device(device):
                        ext.check(lib.rlk_ipc_open(gathered[r][i], ctypes.byref(p)), "ipc_open")
                    self._peer_ptrs[i].append(p.value)
        shape = (max_local_tokens, num_kv_heads * head_dim)
        view = lambda p: torch.as_tensor(_DevicePtrView(p, nbytes), device=device).view(torch.bfloat16).view(shape)  # noqa: E731
        self.k_bufs = [view(p) for p in self._peer_ptrs[0]]
        self.v_bufs = [view(p) for p in self._peer_ptrs[1]]
        self._tiles: dict = {}

    def _tiles_for(self, nseq: int, seq_len: int) -> torch.Tensor:
        key = (nseq, seq_len)
        if key in self._tiles:
            return self._tiles[key]
        cp, g = self.cp, self.hq // self.hkv
        nchunks = cp if self.layout == "contiguous" else 2 * cp
        chunk = seq_len // nchunks
        if seq_len % nchunks or chunk % 128:
            raise ValueError(f"sequence length {seq_len} must split into {nchunks} chunks of a multiple of 128")
        s_local = seq_len // cp
        my_chunks = [self.rank] if self.layout == "contiguous" else [self.rank, 2 * cp - 1 - self.rank]
        rows = []
        for b in range(nseq):
            for li, ch in enumerate(my_chunks):
                for qt in range(chunk // 128 - 1, -1, -1):
                    for h in range(self.hq):
                        row0 = b * s_local + li * chunk + qt * 128
                        rows.append([row0, h * self.d, 128, b * s_local, (h // g) * self.d, ch * chunk + qt * 128, 1,
                                     seq_len, row0 * self.hq + h, self.hq, 0, 0])
        rows.sort(key=lambda r: -r[5])                      # longest (latest positions) first
        t = torch.tensor(rows, dtype=torch.int32, device=self.device).contiguous()
        self._tiles[key] = (t, chunk // 128)
        return self._tiles[key]

    @torch.no_grad()
    def forward(self, q_local: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor, nseq: int, seq_len: int):
        """q_local [nseq * S/cp, Hq*D], k/v_local [nseq * S/cp, Hkv*D] in this rank's local order
        (``cp_positions``).  Returns (out [same as q_local], lse [tokens, Hq])."""
        T = q_local.shape[0]
        if T > self.max_tokens:
            raise ValueError("more local tokens than the buffers were sized for")
        self.k_bufs[self.rank][:T].copy_(k_local)
        self.v_bufs[self.rank][:T].copy_(v_local)
        self.coll.barrier()                                  # every rank's K/V is in place and visible
        tiles, bpc = self._tiles_for(nseq, seq_len)
        out = torch.empty_like(q_local)
        lse = torch.empty(T, self.hq, device=self.device, dtype=torch.float32)
        nv.attn_fwd(q_local, self.k_bufs, self.v_bufs, out, lse, tiles, self.scale, cp_blocks_per_chunk=bpc,
                    cp_zigzag=self.layout == "zigzag")
        self.coll.barrier()                                  # nobody overwrites K/V while a peer still reads
        return out, lse
