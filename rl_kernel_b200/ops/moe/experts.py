"""Routed mixture-of-experts FFN on the sm_100a kernels, with expert parallelism over NVLink.

One layer =  router GEMM -> softmax top-k -> plan (integer counts, stable ranking) -> dispatch
(peer stores straight into the owning rank's buffer) -> grouped gate/up GEMM -> SwiGLU -> grouped
down GEMM -> combine (peer loads, per-token fma chain in ascending expert id).  Nothing on this path
synchronises with the host: the routing counts stay on the device and the grouped GEMMs read their
tile lists from device memory (csrc/moe/moe_routing.cu, csrc/moe/grouped_gemm_sm100.cu).

The expert all-to-all is not a collective call: ``dispatch`` and ``combine`` are ordinary kernels
that address the peers' buffers (CUDA IPC mappings), separated by two barriers of the symmetric
memory collective per layer.  With one rank the same code runs with itself as the only peer.

The reference reserves ``rl_engine/ops/moe`` for this and ships no implementation.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from rl_kernel_b200.backends import native as nv

BF16 = torch.bfloat16


@dataclass
class MoEWeights:
    """Parameters (and optionally gradients) of one layer's routed experts held by this rank."""
    router: torch.Tensor          # [E, H]
    w1: torch.Tensor              # [E_loc * 2I, H]   rows of expert e: [gate (I) | up (I)]
    w2: torch.Tensor              # [E_loc * H, I]
    g_router: torch.Tensor | None = None
    g_w1: torch.Tensor | None = None
    g_w2: torch.Tensor | None = None


class MoEBuffers:
    """Activation buffers and routing state of one expert-parallel group; shared by all layers.

    Capacity is the worst case (every routed copy of every rank lands here), so no token is ever
    dropped and no size has to travel to the host."""

    def __init__(self, device: torch.device, *, hidden: int, inter: int, num_experts: int, top_k: int,
                 max_tokens: int, collective=None, with_backward: bool = True):
        self.dev, self.H, self.I, self.E, self.K = device, hidden, inter, num_experts, top_k
        self.coll = collective if collective is not None and collective.world > 1 else None
        self.W = self.coll.world if self.coll else 1
        self.rank = self.coll.rank if self.coll else 0
        if num_experts % self.W or num_experts // self.W > 128:
            raise ValueError("experts must split evenly over the ranks, at most 128 per rank")
        if hidden % 256 or inter % 256 or (2 * inter) % 256:
            raise ValueError("hidden and intermediate sizes must be multiples of 256")
        self.E_loc = num_experts // self.W
        self.T = max_tokens
        self.cap = self.W * max_tokens * top_k + self.E_loc * 128
        cap, H, I = self.cap, hidden, inter
        peer = {"xr": ((cap, H), BF16), "y": ((cap, H), BF16)}
        if with_backward:
            peer.update({"dy": ((cap, H), BF16), "dxr": ((cap, H), BF16)})
        if self.coll:
            from rl_kernel_b200.distributed.cp_attention import PeerMappedBuffers

            self._pm = PeerMappedBuffers(self.coll.group, device, peer)
            self.peer = {n: self._pm[n] for n in peer}
        else:
            self.peer = {n: [torch.zeros(s, dtype=d, device=device)] for n, (s, d) in peer.items()}
        z = lambda *s, dt=BF16: torch.zeros(*s, dtype=dt, device=device)  # noqa: E731
        self.gu, self.act = z(cap, 2 * I), z(cap, I)
        if with_backward:
            self.dgu, self.dact = z(cap, 2 * I), z(cap, I)
            self.dw = z(max_tokens, top_k, dt=torch.float32)
            self.dlogits = z(max_tokens, num_experts)
        i32 = torch.int32
        self.logits = z(max_tokens, num_experts, dt=torch.float32)
        self.idx, self.w = z(max_tokens, top_k, dt=i32), z(max_tokens, top_k, dt=torch.float32)
        self.counts, self.send_row0 = z(num_experts, dt=i32), z(num_experts, dt=i32)
        self.loc, self.rows_used = z(self.E_loc, 4, dt=i32), z(1, dt=i32)
        self.slot_row = z(max_tokens * top_k, dt=i32)
        mb = cap // 128
        shapes = {"gu": (0, 2 * I, H, False, 0), "dn": (0, H, I, False, 0)}
        if with_backward:
            shapes.update({"dact": (0, I, H, True, 0), "dxr": (0, H, 2 * I, True, 0),
                           "dw2": (1, I, 0, True, H), "dw1": (1, H, 0, True, 2 * I)})
        self._tile_cfg = shapes
        self.tiles, self.n_tiles = {}, {}
        for name, (kind, n_cols, k_dim, b_mn, m_out) in shapes.items():
            mx = mb * (n_cols // 256) if kind == 0 else self.E_loc * (m_out // 128) * (n_cols // 256)
            self.tiles[name], self.n_tiles[name] = z(mx, 8, dt=i32), z(1, dt=i32)

    def local(self, name: str) -> torch.Tensor:
        return self.peer[name][self.rank]

    def barrier(self) -> None:
        if self.coll:
            self.coll.barrier()


class MoEExperts:
    """Forward / backward of the routed-expert part of an MoE layer over ``MoEBuffers``."""

    def __init__(self, bufs: MoEBuffers):
        self.b = bufs

    def _view(self, T: int) -> None:
        """The first T rows of the per-token state (the buffers are sized for the largest call)."""
        b = self.b
        self.idx, self.w, self.logits = b.idx[:T], b.w[:T], b.logits[:T]
        self.slot_row = b.slot_row[: T * b.K]
        if hasattr(b, "dw"):
            self.dw, self.dlogits = b.dw[:T], b.dlogits[:T]

    # ------------------------------------------------------------------ routing
    def route(self, x: torch.Tensor, wts: MoEWeights) -> None:
        b = self.b
        T = x.shape[0]
        if T > b.T:
            raise ValueError(f"the buffers were sized for {b.T} tokens per rank, got {T}")
        self._view(T)
        nv.det_gemm(x, wts.router, self.logits, M=T, N=b.E, K=b.H)
        b.counts.zero_()
        nv.moe_router_topk(self.logits, self.idx, self.w, None, b.counts)
        counts_all = b.coll.all_gather(b.counts) if b.coll else b.counts.unsqueeze(0)
        nv.moe_plan(counts_all.contiguous(), b.rank, b.send_row0, b.loc, b.rows_used)
        nv.moe_slots(self.idx, b.E, b.send_row0, self.slot_row)
        for name, (kind, n_cols, k_dim, b_mn, m_out) in b._tile_cfg.items():
            nv.moe_tiles(b.loc, kind, n_cols, k_dim, b_mn, m_out, b.tiles[name], b.n_tiles[name])

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, wts: MoEWeights, out: torch.Tensor, base: torch.Tensor | None = None,
                *, routed: bool = False) -> torch.Tensor:
        """out[t] = base[t] + sum_k w[t,k] * expert_{idx[t,k]}(x[t]).  ``routed``: ``route`` already ran
        for this ``x`` (the backward re-runs the experts without routing again)."""
        b = self.b
        if not routed:
            self.route(x, wts)
        nv.moe_dispatch(x, None, self.idx, self.slot_row, b.E_loc, b.peer["xr"])
        b.barrier()                                   # every rank's rows have landed
        nv.moe_zero_pad(b.loc, b.local("xr"))
        nv.grouped_gemm(b.local("xr"), wts.w1, b.gu, b.tiles["gu"], b.n_tiles["gu"])
        nv.swiglu_fwd(b.gu, b.act, b.I, b.I, rows_limit=b.rows_used)
        nv.grouped_gemm(b.act, wts.w2, b.local("y"), b.tiles["dn"], b.n_tiles["dn"])
        b.barrier()                                   # every rank's expert outputs are complete
        nv.moe_combine(base, self.w, self.idx, self.slot_row, b.E_loc, b.peer["y"], out)
        return out

    # ------------------------------------------------------------------ backward
    def backward(self, x: torch.Tensor, dout: torch.Tensor, wts: MoEWeights, dx: torch.Tensor,
                 dx_base: torch.Tensor | None = None) -> torch.Tensor:
        """Gradients of ``forward`` given that its buffers (routing, xr, gu, act, y) are still in place:
        dx[t] = dx_base[t] + d(router path) + sum_k dXr[row(t,k)]; expert and router weight gradients
        are accumulated into ``wts.g_*``."""
        b = self.b
        T = x.shape[0]
        # routing-weight gradient and the scaled copies of dOut for the experts
        nv.moe_combine_dw(dout, self.idx, self.slot_row, b.E_loc, b.peer["y"], self.dw)
        nv.moe_dispatch(dout, self.w, self.idx, self.slot_row, b.E_loc, b.peer["dy"])
        b.barrier()
        dy = b.local("dy")
        nv.moe_zero_pad(b.loc, dy)
        nv.grouped_gemm(dy, wts.w2, b.dact, b.tiles["dact"], b.n_tiles["dact"], b_mn=True)
        nv.grouped_gemm(dy, b.act, wts.g_w2, b.tiles["dw2"], b.n_tiles["dw2"], a_mn=True, b_mn=True,
                        accumulate=True)
        nv.swiglu_bwd(b.gu, b.dact, b.dgu, b.I, b.I, rows_limit=b.rows_used)
        nv.grouped_gemm(b.dgu, wts.w1, b.local("dxr"), b.tiles["dxr"], b.n_tiles["dxr"], b_mn=True)
        nv.grouped_gemm(b.dgu, b.local("xr"), wts.g_w1, b.tiles["dw1"], b.n_tiles["dw1"], a_mn=True, b_mn=True,
                        accumulate=True)
        # router: dlogits -> dx (through the router weights) and the router weight gradient
        nv.moe_router_bwd(self.idx, self.w, self.dw, self.dlogits)
        dxr_router = dx                                # reuse the output as the fma chain's start
        nv.det_gemm(self.dlogits, wts.router, dxr_router, M=T, N=b.H, K=b.E, b_mn=True)
        nv.det_gemm(self.dlogits, x, wts.g_router, M=b.E, N=b.H, K=T, a_mn=True, b_mn=True, accumulate=True)
        if dx_base is not None:
            dx.add_(dx_base)
        b.barrier()                                   # every rank's dXr is complete
        nv.moe_combine(dx, None, self.idx, self.slot_row, b.E_loc, b.peer["dxr"], dx)
        return dx
