"""Context-parallel causal attention, forward and backward, with the exchange inside the kernels.

Every CP rank keeps the tensors its peers need (K, V for the forward and the dQ kernel; Q, dO, lse
and delta for the dK/dV kernel) in buffers that the peers have mapped (CUDA IPC over NVLink).  A
kernel walks the canonical 128-token blocks of its work item in ascending order.  Remote blocks
reach it in one of two ways, both inside the same kernel launch (csrc/attention/attn_fwd_sm100.cu,
attn_bwd_sm100.cu, NSRC = 8): with ``stage_remote`` (default) the compute warps of the CTAs that
start first copy every remote block once into a local staging buffer (16-byte peer loads, work
items from an atomic counter, a ready flag per block) and the TMA producers read the local copy
after a bounded wait on the flag -- a block crosses NVLink once however many tiles use it; without
it every tile loads the block straight from its owner with a plain (non-multicast) TMA load through
that peer's tensor map.  Nothing is merged or reduce-scattered afterwards: every query row (forward, dQ) and
every key row (dK, dV) executes exactly the single-GPU program, so outputs and gradients are bitwise
equal to CP = 1 for every CP degree and layout.  (The reference all-gathers Q/K/V, lets every rank
compute the whole sequence and scatters rank 0's result, and reduce-scatters dK/dV:
rl_engine/backends/cuda/attention/cp_comm.py:444-566.)

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


def cp_tiles(cp: int, rank: int, layout: str, nseq: int, seq_len: int, hq: int, hkv: int, d: int, device):
    """Work items of one context-parallel rank: (forward/dQ tiles, dK/dV tiles, blocks per chunk) for
    ``nseq`` sequences of global length ``seq_len`` whose local tokens are stored sequence after
    sequence.  Positions are global, rows are local."""
    g = hq // hkv
    nchunks = cp if layout == "contiguous" else 2 * cp
    chunk = seq_len // nchunks
    if seq_len % nchunks or chunk % 128:
        raise ValueError(f"sequence length {seq_len} must split into {nchunks} chunks of a multiple of 128")
    my_chunks = [rank] if layout == "contiguous" else [rank, 2 * cp - 1 - rank]
    s_local = seq_len // cp
    bpc = chunk // 128
    fw, kv = [], []
    for b in range(nseq):
        for li, ch in enumerate(my_chunks):
            for t in range(bpc):
                row0 = b * s_local + li * chunk + t * 128
                gpos = ch * chunk + t * 128
                for h in range(hq):
                    fw.append([row0, h * d, 128, b * s_local, (h // g) * d, gpos, 1,
                               seq_len, row0 * hq + h, hq, 0, 0])
                for hk in range(hkv):
                    kv.append([row0, hk * d, gpos, 128, b * s_local, 0, seq_len, hk * g * d, g,
                               (b * s_local) * hq + hk * g, hq, 1])
    fw.sort(key=lambda r: -r[5])                      # most keys first
    kv.sort(key=lambda r: r[2])                       # most query tiles first
    return (torch.tensor(fw, dtype=torch.int32, device=device).contiguous(),
            torch.tensor(kv, dtype=torch.int32, device=device).contiguous(), bpc)


class PeerMappedBuffers:
    """Named device buffers of identical shape on every rank of a group, each rank's copy mapped
    into every other rank's address space.  ``self[name][r]`` is rank r's tensor as seen from here."""

    def __init__(self, group, device: torch.device, specs: dict[str, tuple[tuple[int, ...], torch.dtype]]):
        import torch.distributed as dist

        self.device = device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        lib = ext.load()
        offs, total = {}, 0
        for name, (shape, dtype) in specs.items():
            nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
            offs[name] = (total, nbytes, shape, dtype)
            total += (nbytes + 1023) // 1024 * 1024
        handle = ctypes.create_string_buffer(lib.rlk_symm_ipc_handle_bytes())
        base = ctypes.c_void_p(0)
        with torch.cuda.device(device):
            ext.check(lib.rlk_ipc_alloc(ctypes.c_longlong(total), ctypes.byref(base), handle), "ipc_alloc")
        gathered = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle.raw), group=group)
        self._bases = []
        for r in range(self.world):
            if r == self.rank:
                self._bases.append(base.value)
            else:
                p = ctypes.c_void_p(0)
                with torch.cuda.device(device):
                    ext.check(lib.rlk_ipc_open(gathered[r], ctypes.byref(p)), "ipc_open")
                self._bases.append(p.value)
        self.nbytes = total
        self._t: dict[str, list[torch.Tensor]] = {}
        for name, (off, nbytes, shape, dtype) in offs.items():
            self._t[name] = [torch.as_tensor(_DevicePtrView(b + off, nbytes), device=device).view(dtype).view(shape)
                             for b in self._bases]

    def __getitem__(self, name: str) -> list[torch.Tensor]:
        return self._t[name]

    def local(self, name: str) -> torch.Tensor:
        return self._t[name][self.rank]


class CPAttention:
    def __init__(self, collective, device: torch.device, *, num_q_heads: int, num_kv_heads: int, head_dim: int = 128,
                 max_local_tokens: int, layout: str = "zigzag", with_backward: bool = True,
                 stage_remote: bool = True):
        if layout not in ("zigzag", "contiguous"):
            raise ValueError(layout)
        if head_dim != 128:
            raise ValueError("head_dim must be 128")
        self.coll, self.device, self.layout = collective, device, layout
        self.cp, self.rank = collective.world, collective.rank
        self.hq, self.hkv, self.d = num_q_heads, num_kv_heads, head_dim
        self.max_tokens = max_local_tokens
        self.scale = 1.0 / math.sqrt(head_dim)
        T, bf16, f32 = max_local_tokens, torch.bfloat16, torch.float32
        specs = {"k": ((T, num_kv_heads * head_dim), bf16), "v": ((T, num_kv_heads * head_dim), bf16)}
        if with_backward:
            specs.update({"q": ((T, num_q_heads * head_dim), bf16), "do": ((T, num_q_heads * head_dim), bf16),
                          "lse": ((T, num_q_heads), f32), "delta": ((T, num_q_heads), f32)})
        self.bufs = PeerMappedBuffers(collective.group, device, specs)
        self.k_bufs, self.v_bufs = self.bufs["k"], self.bufs["v"]
        self._tiles: dict = {}
        # Local copies of the peers' blocks: the kernels fill them themselves, once per call, so a
        # remote block crosses NVLink once instead of once per tile that needs it.
        self.stage_remote = stage_remote
        if stage_remote:
            R = (T + 127) // 128 * 128
            z = lambda cols: torch.zeros(self.cp * R, cols, dtype=bf16, device=device)  # noqa: E731
            self._st_k, self._st_v = z(num_kv_heads * head_dim), z(num_kv_heads * head_dim)
            self._st_flags = torch.zeros(self.cp * (R // 128) * 2 + 1, dtype=torch.int32, device=device)
            if with_backward:
                self._st_q, self._st_do = z(num_q_heads * head_dim), z(num_q_heads * head_dim)
                self._st_flags2 = torch.zeros_like(self._st_flags)

    # ------------------------------------------------------------------ geometry
    def local_positions(self, seq_len: int) -> torch.Tensor:
        return cp_positions(seq_len, self.cp, self.rank, self.layout)

    def tiles_for(self, nseq: int, seq_len: int):
        """(forward/dQ tiles, dK/dV tiles, blocks per chunk) for ``nseq`` sequences of global length
        ``seq_len`` whose local tokens are stored sequence after sequence."""
        key = (nseq, seq_len)
        if key not in self._tiles:
            self._tiles[key] = cp_tiles(self.cp, self.rank, self.layout, nseq, seq_len, self.hq, self.hkv, self.d,
                                        self.device)
        return self._tiles[key]

    def _stage_kv(self, T: int):
        if not self.stage_remote:
            return None
        return (self._st_k, self._st_v, self._st_flags, (T + 127) // 128 * 128, self.rank)

    # ------------------------------------------------------------------ in-place API (engine)
    def forward_inplace(self, q_local: torch.Tensor, out: torch.Tensor, lse: torch.Tensor | None, nseq: int,
                        seq_len: int) -> None:
        """K and V of this rank's tokens are already in ``bufs.local('k'|'v')[:T]``."""
        tiles, _, bpc = self.tiles_for(nseq, seq_len)
        self.coll.barrier()                                  # every rank's K/V is in place and visible
        nv.attn_fwd(q_local, self.k_bufs, self.v_bufs, out, lse, tiles, self.scale, cp_blocks_per_chunk=bpc,
                    cp_zigzag=self.layout == "zigzag", stage=self._stage_kv(q_local.shape[0]))
        self.coll.barrier()                                  # nobody overwrites K/V while a peer still reads

    def backward_inplace(self, dq: torch.Tensor, dk: torch.Tensor, dv: torch.Tensor, nseq: int, seq_len: int) -> None:
        """Q, dO, lse, delta, K, V of this rank's tokens are in the peer-mapped buffers (first T rows)."""
        T = dq.shape[0]
        b = self.bufs
        tiles, kvtiles, bpc = self.tiles_for(nseq, seq_len)
        zz = self.layout == "zigzag"
        self.coll.barrier()
        nv.attn_bwd_dq(b.local("q")[:T], b.local("do")[:T], self.k_bufs, self.v_bufs, b.local("lse"),
                       b.local("delta"), dq, tiles, self.scale, cp_blocks_per_chunk=bpc, cp_zigzag=zz,
                       stage=self._stage_kv(T))
        st_q = None
        if self.stage_remote:
            st_q = (self._st_q, self._st_do, self._st_flags2, (T + 127) // 128 * 128, self.rank)
        nv.attn_bwd_dkv(b["q"], b["do"], b.local("k"), b.local("v"), b["lse"], b["delta"], dk, dv, kvtiles,
                        self.scale, cp_blocks_per_chunk=bpc, cp_zigzag=zz, stage=st_q)
        self.coll.barrier()

    # ------------------------------------------------------------------ copying API
    @torch.no_grad()
    def forward(self, q_local: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor, nseq: int, seq_len: int):
        """q_local [nseq * S/cp, Hq*D], k/v_local [nseq * S/cp, Hkv*D] in this rank's local order
        (``cp_positions``).  Returns (out [same as q_local], lse [tokens, Hq])."""
        T = q_local.shape[0]
        if T > self.max_tokens:
            raise ValueError("more local tokens than the buffers were sized for")
        self.k_bufs[self.rank][:T].copy_(k_local)
        self.v_bufs[self.rank][:T].copy_(v_local)
        out = torch.empty_like(q_local)
        lse = torch.empty(T, self.hq, device=self.device, dtype=torch.float32)
        self.forward_inplace(q_local, out, lse, nseq, seq_len)
        return out, lse

    @torch.no_grad()
    def backward(self, q_local, k_local, v_local, out, lse, dout, nseq: int, seq_len: int):
        """Gradients (dq, dk, dv) of this rank's tokens; all tensors in the local order."""
        T = q_local.shape[0]
        b = self.bufs
        b.local("k")[:T].copy_(k_local)
        b.local("v")[:T].copy_(v_local)
        b.local("q")[:T].copy_(q_local)
        b.local("do")[:T].copy_(dout)
        b.local("lse")[:T].copy_(lse)
        nv.attn_bwd_delta(out, b.local("do")[:T], b.local("delta"), T, self.hq)
        dq = torch.empty_like(q_local)
        dk = torch.empty_like(k_local)
        dv = torch.empty_like(v_local)
        self.backward_inplace(dq, dk, dv, nseq, seq_len)
        return dq, dk, dv
