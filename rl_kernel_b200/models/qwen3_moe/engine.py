"""Qwen3-MoE on the sm_100a kernels: the dense engine's attention block, a shared SwiGLU expert and
the routed experts of ``rl_kernel_b200.ops.moe`` with expert parallelism over NVLink.

Parallel layout: every rank of the expert-parallel group is also a data-parallel replica for
everything that is not an expert (embeddings, attention, norms, router, shared expert): it runs its
own sequences, its tokens visit the experts of all ranks through the dispatch / combine kernels, and
the gradients of the replicated parameters are summed over the group with the fixed-tree all-reduce
after the backward.  Expert weights and their gradients stay local.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.models.qwen3.engine import BF16, PackedParams, ParallelContext, Qwen3Engine, _Slot
from rl_kernel_b200.models.qwen3_moe.spec import Qwen3MoeSpec
from rl_kernel_b200.ops.moe import MoEBuffers, MoEExperts, MoEWeights


class MoEPackedParams(PackedParams):
    """Flat parameter buffer: replicated parameters first (one contiguous range to all-reduce),
    this rank's routed experts last."""

    def __init__(self, spec: Qwen3MoeSpec, ep_rank: int, ep_size: int, device: torch.device,
                 with_grad: bool = False):
        if spec.num_experts % ep_size:
            raise ValueError("num_experts must be a multiple of the expert-parallel size")
        self.ep_rank, self.ep_size = ep_rank, ep_size
        self.e_local = spec.num_experts // ep_size
        self._moe_spec = spec
        super().__init__(spec, 0, 1, device, with_grad)
        first = self.slots["l0.w1"].offset
        self.replicated_numel = first

    def _mlp_slots(self, l: int) -> list[_Slot]:
        h = self.spec.hidden_size
        return super()._mlp_slots(l) + [_Slot(f"l{l}.router", (self._moe_spec.num_experts, h))]

    def _trailing_slots(self) -> list[_Slot]:
        s, h = self._moe_spec, self._moe_spec.hidden_size
        out = []
        for l in range(s.num_hidden_layers):
            out += [_Slot(f"l{l}.w1", (self.e_local * 2 * s.moe_intermediate_size, h)),
                    _Slot(f"l{l}.w2", (self.e_local * h, s.moe_intermediate_size))]
        return out

    def init_synthetic_(self, seed: int = 0, std: float = 0.02) -> "MoEPackedParams":
        """Replicated parameters are the same on every rank; expert e of layer l is drawn from a
        generator keyed by (seed, l, e), so any expert-parallel size holds the same model."""
        s = self._moe_spec
        gen = torch.Generator(device=self.device).manual_seed(seed * 1000)
        for name, slot in self.slots.items():
            if name.endswith((".w1", ".w2")):
                continue
            if len(slot.shape) == 1:
                self.w[name].fill_(1.0)
            else:
                w = self.w[name]
                step = max(1, (1 << 26) // max(1, w.shape[1]))
                for r0 in range(0, w.shape[0], step):
                    blk = w[r0:r0 + step]
                    blk.copy_(torch.randn(blk.shape, generator=gen, device=self.device, dtype=torch.float32).mul_(std))
        for name in ("embed", "lm_head"):
            if self.v_real_local < self.v_local:
                self.w[name][self.v_real_local:].zero_()
        i2, h, inter = 2 * s.moe_intermediate_size, s.hidden_size, s.moe_intermediate_size
        for l in range(s.num_hidden_layers):
            for el in range(self.e_local):
                e = self.ep_rank * self.e_local + el
                g = torch.Generator(device=self.device).manual_seed((seed * 1000 + l + 1) * 4096 + e)
                self.w[f"l{l}.w1"][el * i2:(el + 1) * i2].copy_(
                    torch.randn(i2, h, generator=g, device=self.device, dtype=torch.float32).mul_(std))
                self.w[f"l{l}.w2"][el * h:(el + 1) * h].copy_(
                    torch.randn(h, inter, generator=g, device=self.device, dtype=torch.float32).mul_(std))
        return self

    def load(self, weights):  # pragma: no cover - no public checkpoint of this roadmap family exists
        raise NotImplementedError("the MoE roadmap stack is initialised synthetically")


class Qwen3MoeEngine(Qwen3Engine):
    def __init__(self, spec: Qwen3MoeSpec, params: MoEPackedParams, ctx: ParallelContext | None = None, *,
                 ep_collective=None, max_tokens: int, max_positions: int = 4096, with_backward: bool = True):
        super().__init__(spec, params, ctx, max_positions=max_positions)
        if self.ctx.tp_size != 1:
            raise ValueError("the MoE engine uses expert + data parallelism, not tensor parallelism")
        self.ep = ep_collective if ep_collective is not None and ep_collective.world > 1 else None
        self.moe = MoEExperts(MoEBuffers(self.dev, hidden=spec.hidden_size, inter=spec.moe_intermediate_size,
                                         num_experts=spec.num_experts, top_k=spec.num_experts_per_tok,
                                         max_tokens=max_tokens, collective=self.ep, with_backward=with_backward))

    def _moe_weights(self, l: int) -> MoEWeights:
        w, g = self.p.w, self.p.g
        return MoEWeights(w[f"l{l}.router"], w[f"l{l}.w1"], w[f"l{l}.w2"], g.get(f"l{l}.router"),
                          g.get(f"l{l}.w1"), g.get(f"l{l}.w2"))

    supports_stored_activations = False     # the expert buffers are shared by all layers: recompute
    fold_tree_into_norm = False             # the shared expert's output feeds the combine, not a norm

    def _mlp_fwd(self, l, h2, T, tag, keep, store_tag=None):
        shared = super()._mlp_fwd(l, h2, T, tag, keep)
        out = self.ws.get(f"{tag}.moe_out", (T, self.spec.hidden_size))
        self.moe.forward(h2, self._moe_weights(l), out, base=shared)
        return out

    def _mlp_bwd(self, l, ds, keep, T, cp_geom=None):
        # the expert buffers still hold this layer's recomputed forward
        dshared = super()._mlp_bwd(l, ds, keep, T, cp_geom)
        dx = self.ws.get("b.moe_dx", (T, self.spec.hidden_size))
        self.moe.backward(keep["h2"], ds, self._moe_weights(l), dx, dx_base=dshared)
        return dx

    def sync_replicated_grads(self) -> None:
        """Sum the gradients of everything that is not a routed expert over the data-parallel
        (= expert-parallel) group, in the collective's fixed order."""
        if self.ep is not None:
            self.ep.all_reduce_(self.p.grad[: self.p.replicated_numel])
