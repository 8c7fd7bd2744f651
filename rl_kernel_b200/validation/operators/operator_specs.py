"""Operator specs of the validation harness (parity: rl_engine/validation/operators/operator_specs.py:18-370).

An ``OperatorSpec`` names an operator, its class, the fp32 gold and the candidates per backend, and
points at an *adapter*: the code that lays the logical tokens of a batch out physically for one
configuration (packed / chunked / singleton / permuted / padded), runs the operator object on that
layout and returns the outputs keyed by logical token.  Adapters are what make operators of very
different shapes (row-wise, per-sequence, per-batch) comparable token by token.

Candidates: ``b200`` (the sm_100a kernels; needs CUDA tensors) and ``pytorch`` (the reference
operators, any device).  ``gold`` is always fp32 PyTorch math written out here, independent of both.
"""
from __future__ import annotations

import argparse
import importlib
import math
from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from rl_kernel_b200.config.workload import LogicalBatch, PaddedBatch, PhysicalLayout
from rl_kernel_b200.validation.operators import operator_inputs as oi

Key = tuple[str, int]


@dataclass(frozen=True)
class OperatorSpec:
    name: str
    op_class: str                                   # reduction | elementwise | attention | gather | logprob | layout | loss | sampling
    gold_path: str
    gold_method: str
    candidate_paths: dict[str, str]
    grad_input_names: tuple[str, ...] = ()
    adapter: str = "token_rows"                     # name of the adapter in ADAPTERS
    output_dtype: str = "input"                     # input | float32
    tolerance_key: str | None = None
    params: dict = field(default_factory=dict)


def _load_object(path: str) -> Any:
    module_path, object_name = path.rsplit(".", 1)
    return getattr(importlib.import_module(module_path), object_name)


# ------------------------------------------------------------------------------------ small operator objects
class GtestPackOp:
    """pack -> unpack round trip: the operator under test is the pair; its output is the restored padded tensor."""

    def __init__(self, impl=None):
        from rl_kernel_b200.reference.packing.pack import NativePackOp

        self.impl = impl or NativePackOp()

    def forward(self, x, mask):
        packed, _ = self.impl.pack(x, mask)
        return self.impl.unpack(packed, mask, fill=0.0)

    forward_fp32 = __call__ = forward


class GtestDevicePackOp(GtestPackOp):
    def __init__(self):
        from rl_kernel_b200.ops.packing import PackOp

        super().__init__(PackOp())


class GtestPrefixSharedAttentionOp:
    """fp32 gold of prefix-shared attention: q [bs, G, Lq, Hq, D] against shared k, v [bs, Lkv, Hkv, D], no mask."""

    def forward_fp32(self, q, k, v):
        g = q.shape[3] // k.shape[2]
        kk, vv = k.float().repeat_interleave(g, 2), v.float().repeat_interleave(g, 2)
        s = torch.einsum("bgqhd,bkhd->bgqhk", q.float(), kk) / math.sqrt(q.shape[-1])
        return torch.einsum("bgqhk,bkhd->bgqhd", torch.softmax(s, -1), vv)

    def forward(self, q, k, v):
        return self.forward_fp32(q, k, v).to(q.dtype)

    __call__ = forward


class _DeviceDetGemm:
    """``op(x, w)`` = x @ w^T with a [N, K] weight on the deterministic GEMM (differentiable)."""

    def __call__(self, x, w):
        from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_linear

        return det_gemm_linear(x, w)


class _ReferenceDetGemm:
    def __call__(self, x, w):
        from rl_kernel_b200.reference.gemm.det_gemm import det_gemm_reference

        return det_gemm_reference(x, w)


class _RowOp:
    """Wraps plain functions of this package as operator objects."""

    def __init__(self, fn: Callable):
        self.fn = fn

    def __call__(self, *a, **k):
        return self.fn(*a, **k)


def _dev_rms():
    from rl_kernel_b200.ops.norm import rms_norm

    return _RowOp(lambda x, w: rms_norm(x, w, oi.DEFAULT_RMS_EPS))


def _dev_rope():
    from rl_kernel_b200.ops.rope import rope

    return _RowOp(lambda x, pos: rope(x, pos, theta=oi.DEFAULT_ROPE_THETA))


def _dev_swiglu():
    from rl_kernel_b200.ops.activation import swiglu

    return _RowOp(swiglu)


def _dev_embedding():
    from rl_kernel_b200.ops.embedding.canonical_embedding import embedding

    return _RowOp(lambda ids, w: embedding(ids, w))


def _dev_linear_logp():
    from rl_kernel_b200.ops.logprob import linear_logp

    return _RowOp(lambda h, w, t: linear_logp(h, w, t))


def _dev_logp():
    from rl_kernel_b200.ops.logprob import logp_from_logits

    return _RowOp(lambda lg, t: logp_from_logits(lg, t))


def _dev_attention():
    from rl_kernel_b200.ops.attention.attention import causal_attention

    return _RowOp(causal_attention)


def _dev_loss():
    from rl_kernel_b200.ops.loss import grpo_loss

    return _RowOp(grpo_loss)


def _dev_sampler():
    from rl_kernel_b200.ops.sampling.api import sample

    return _RowOp(sample)


FACTORIES = {"rms_norm": _dev_rms, "qk_norm": _dev_rms, "rope": _dev_rope, "swiglu": _dev_swiglu, "embedding": _dev_embedding,
             "linear_logp": _dev_linear_logp, "batch_invariant_logp": _dev_logp, "logp": _dev_logp, "attention": _dev_attention,
             "kv_cache_attention": _dev_attention, "grpo_loss": _dev_loss, "sampling": _dev_sampler,
             "det_gemm": _DeviceDetGemm, "lm_head": _DeviceDetGemm, "matmul": _DeviceDetGemm}
"""Operator name -> callable building the candidate object.  The ops entry points of this package dispatch on the
device of their inputs: the sm_100a kernels for CUDA tensors, the PyTorch references for CPU tensors, so one factory
serves both candidates (``b200`` requires device='cuda' and fails loudly if the library is missing)."""


# ------------------------------------------------------------------------------------ gold formulas (fp32)
def _gold_rms(x, w):
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + oi.DEFAULT_RMS_EPS) * w.float()


def _gold_rope(x, pos):
    D = x.shape[-1]
    inv = 1.0 / (oi.DEFAULT_ROPE_THETA ** (torch.arange(0, D, 2, dtype=torch.float64, device=x.device) / D))
    ang = pos.double().unsqueeze(-1) * inv
    c, s = ang.cos().float().unsqueeze(-2), ang.sin().float().unsqueeze(-2)
    a, b = x.float()[..., : D // 2], x.float()[..., D // 2:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def _gold_swiglu(gate, up):
    return torch.nn.functional.silu(gate.float()) * up.float()


def _gold_gemm(x, w):
    return x.float() @ w.float().t()


def _gold_linear_logp(h, w, t):
    return torch.log_softmax((h.float() @ w.float().t()).bfloat16().float() if h.dtype == torch.bfloat16
                             else h.float() @ w.float().t(), -1).gather(1, t[:, None])[:, 0]


def _gold_logp(lg, t):
    return torch.log_softmax(lg.float(), -1).gather(1, t[:, None])[:, 0]


def _gold_attention_seq(q, k, v, q_pos0: int = 0):
    """One sequence: q [n, Hq, D] at positions q_pos0.., k/v [m, Hkv, D]."""
    g = q.shape[1] // k.shape[1]
    kk, vv = k.float().repeat_interleave(g, 1), v.float().repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk) / math.sqrt(q.shape[-1])
    qp = torch.arange(q.shape[0], device=q.device)[:, None] + q_pos0
    s = s.masked_fill(torch.arange(k.shape[0], device=q.device)[None, :] > qp, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv)


GOLD = {"rms_norm": _gold_rms, "qk_norm": _gold_rms, "rope": _gold_rope, "swiglu": _gold_swiglu, "det_gemm": _gold_gemm,
        "lm_head": _gold_gemm, "matmul": _gold_gemm, "linear_logp": _gold_linear_logp, "batch_invariant_logp": _gold_logp,
        "logp": _gold_logp, "embedding": lambda ids, w: w.float()[ids]}


# ------------------------------------------------------------------------------------ the table
def _spec(name, op_class, gold, b200, ref, grads=(), adapter="token_rows", out="input", tol=None, **params):
    return OperatorSpec(name, op_class, gold, "forward_fp32", {"b200": b200, "pytorch": ref}, tuple(grads), adapter, out, tol,
                        params)


OP_SPECS: dict[str, OperatorSpec] = {
    "rms_norm": _spec("rms_norm", "reduction", "rl_engine.reference.norm.rms_norm.NativeRMSNormOp",
                      "rl_engine.backends.cuda.norm.rmsnorm.RMSNormCudaOp", "rl_engine.reference.norm.rms_norm.NativeRMSNormOp",
                      ("x", "weight"), width=1024),
    "qk_norm": _spec("qk_norm", "reduction", "rl_engine.reference.norm.rms_norm.NativeRMSNormOp",
                     "rl_engine.backends.cuda.norm.rmsnorm.RMSNormCudaOp", "rl_engine.reference.norm.rms_norm.NativeRMSNormOp",
                     ("x", "weight"), width=128, heads=6),
    "rope": _spec("rope", "elementwise", "rl_engine.reference.rope.rope.NativeRoPEOp", "rl_engine.backends.cuda.rope.rope.RoPESM100Op",
                  "rl_engine.reference.rope.rope.NativeRoPEOp", ("x",), adapter="token_rows_pos", width=128, heads=4),
    "swiglu": _spec("swiglu", "elementwise", "rl_engine.reference.activation.swiglu.NativeSwiGLUOp",
                    "rl_engine.backends.cuda.activation.swiglu.SwiGLUCudaOp", "rl_engine.reference.activation.swiglu.NativeSwiGLUOp",
                    ("gate", "up"), adapter="token_rows_pair", width=768),
    "silu": _spec("silu", "elementwise", "rl_engine.backends.cuda.activation.swiglu.SiLUCudaOp",
                  "rl_engine.backends.cuda.activation.swiglu.SiLUCudaOp", "rl_engine.backends.cuda.activation.swiglu.SiLUCudaOp",
                  ("x",), width=768),
    "det_gemm": _spec("det_gemm", "reduction", "rl_engine.reference.gemm.det_gemm.NativeGemmOp",
                      "rl_engine.backends.cuda.gemm.det_gemm.DetGemmOp", "rl_engine.reference.gemm.det_gemm.NativeGemmOp",
                      ("x", "weight"), adapter="token_rows_weight", width=512, out_features=384),
    "matmul": _spec("matmul", "reduction", "rl_engine.reference.gemm.det_gemm.NativeGemmOp",
                    "rl_engine.backends.cuda.gemm.det_gemm.DetGemmOp", "rl_engine.reference.gemm.det_gemm.NativeGemmOp",
                    ("x", "weight"), adapter="token_rows_weight", tol="det_gemm", width=256, out_features=256),
    "lm_head": _spec("lm_head", "reduction", "rl_engine.reference.embedding.lm_head.NativeLMHeadOp",
                     "rl_engine.backends.cuda.embedding.lm_head.SM100LMHeadOp", "rl_engine.reference.embedding.lm_head.NativeLMHeadOp",
                     ("x", "weight"), adapter="token_rows_weight", tol="det_gemm", width=256, out_features=2048),
    "embedding": _spec("embedding", "gather", "rl_engine.reference.embedding.embedding.NativeEmbeddingOp",
                       "rl_engine.backends.cuda.embedding.embedding.SM100EmbeddingOp",
                       "rl_engine.reference.embedding.embedding.NativeEmbeddingOp", ("weight",), adapter="token_ids", width=256,
                       vocab=4096),
    "linear_logp": _spec("linear_logp", "logprob", "rl_engine.reference.logprob.linear_logp.NativeLinearLogpOp",
                         "rl_engine.backends.cuda.logprob.linear_logp.FusedLinearLogpSM100Op",
                         "rl_engine.reference.logprob.linear_logp.NativeLinearLogpOp", ("x", "weight"), adapter="token_logp_linear",
                         out="float32", width=256, vocab=2048),
    "batch_invariant_logp": _spec("batch_invariant_logp", "logprob",
                                  "rl_engine.reference.logprob.batch_invariant_logp.NativeBatchInvariantLogpOp",
                                  "rl_engine.backends.cuda.logprob.batch_invariant_logp.BatchInvariantLogpSM100Op",
                                  "rl_engine.reference.logprob.batch_invariant_logp.NativeBatchInvariantLogpOp", ("x",),
                                  adapter="token_logp_logits", out="float32", tol="linear_logp", vocab=2048),
    "logp": _spec("logp", "logprob", "rl_engine.reference.logprob.logp.NativeLogpOp", "rl_engine.backends.cuda.logprob.logp.FusedLogpSM100Op",
                  "rl_engine.reference.logprob.logp.NativeLogpOp", ("x",), adapter="token_logp_logits", out="float32",
                  tol="linear_logp", vocab=1024),
    "attention": _spec("attention", "attention", "rl_engine.reference.attention.standard_attn.NativeAttentionOp",
                       "rl_engine.backends.cuda.attention.deterministic_attn.DeterministicAttentionOp",
                       "rl_engine.reference.attention.standard_attn.NativeAttentionOp", ("q", "k", "v"), adapter="attention",
                       hq=4, hkv=2),
    "kv_cache_attention": _spec("kv_cache_attention", "attention", "rl_engine.reference.attention.kv_cache.NativeKVCacheAttnOp",
                                "rl_engine.ops.attention.paged.paged_attention_block_table",
                                "rl_engine.reference.attention.kv_cache.NativeKVCacheAttnOp", (), adapter="attention_chunked",
                                tol="attention", hq=4, hkv=2),
    "prefix_shared_attention": _spec("prefix_shared_attention", "attention",
                                     "rl_engine.validation.operators.operator_specs.GtestPrefixSharedAttentionOp",
                                     "rl_engine.backends.cuda.attention.prefix_shared_attn.PrefixSharedAttentionOp",
                                     "rl_engine.validation.operators.operator_specs.GtestPrefixSharedAttentionOp", (),
                                     adapter="prefix_shared", tol="attention", hq=4, hkv=2),
    "pack": _spec("pack", "layout", "rl_engine.validation.operators.operator_specs.GtestPackOp",
                  "rl_engine.validation.operators.operator_specs.GtestDevicePackOp",
                  "rl_engine.validation.operators.operator_specs.GtestPackOp", (), adapter="pack", width=256),
    "grpo_loss": _spec("grpo_loss", "loss", "rl_engine.reference.loss.grpo_loss.NativeGRPOLossOp", "rl_engine.ops.loss.GRPOLossOp",
                       "rl_engine.reference.loss.grpo_loss.NativeGRPOLossOp", ("logp",), adapter="loss", out="float32"),
    "sampling": _spec("sampling", "sampling", "rl_engine.reference.sampling.policy.sample_from_logits",
                      "rl_engine.ops.sampling.api.sample", "rl_engine.reference.sampling.policy.sample_from_logits", (),
                      adapter="sampling", out="int64", vocab=1024),
}


def operator_names() -> tuple[str, ...]:
    return tuple(OP_SPECS)


# ------------------------------------------------------------------------------------ adapters
# An adapter has ``prepare(spec, batch, device, dtype, seed) -> state`` (the logical inputs: one tensor per logical token
# or per sample, plus shared parameters) and ``run(spec, state, layout, grads) -> dict[key] -> tensor`` which lays the
# inputs out as ``layout`` says, calls the candidate and maps results back.  ``gold(spec, state)`` evaluates the fp32
# formula in logical order.  With ``grads`` (a dict) the adapter also runs backward with d(out) = state["gout"] and
# stores token gradients keyed by logical token and parameter gradients as tensors.

def _rows(layout, table: dict[Key, torch.Tensor], filler: torch.Tensor) -> tuple[torch.Tensor, list[Key | None]]:
    """Physical rows of ``layout`` from a per-token table; padding slots get ``filler`` (values that must not matter)."""
    if isinstance(layout, PaddedBatch):
        keys = [k for row in layout.restore_map for k in row]
    else:
        keys = list(layout.restore_map)
    return torch.stack([table[k] if k is not None else filler for k in keys]), keys


def _back(keys, out: torch.Tensor) -> dict[Key, torch.Tensor]:
    return {k: out[i] for i, k in enumerate(keys) if k is not None}


class _TokenRows:
    """Row-wise operators: out[row] depends on that row (and shared parameters) only."""
    inputs = ("x",)

    def prepare(self, spec, batch, device, dtype, seed):
        p = spec.params
        width = p.get("width", 256) * p.get("heads", 1)
        st = {"x": oi.token_table(batch, width, device, dtype, seed), "gout": None}
        st["weight"] = oi.shared_weight(spec, device, dtype, seed)
        st["filler"] = oi.filler_row(width, device, dtype, seed)
        return st

    def call(self, spec, op, st, x, keys, layout):
        if spec.name == "qk_norm":
            h = spec.params["heads"]
            return op(x.view(x.shape[0], h, -1), st["weight"]).reshape(x.shape[0], -1)
        if spec.name == "silu":
            return op(x)
        return op(x, st["weight"])

    def gold(self, spec, st, batch):
        keys = list(batch.logical_keys())
        x = torch.stack([st["x"][k] for k in keys])
        if spec.name == "silu":
            y = torch.nn.functional.silu(x.float())
        elif spec.name == "qk_norm":
            h = spec.params["heads"]
            y = _gold_rms(x.view(x.shape[0], h, -1), st["weight"]).reshape(x.shape[0], -1)
        else:
            y = GOLD[spec.name](x, st["weight"])
        return _back(keys, y)

    def run(self, spec, op, st, layout, grads=None):
        x, keys = _rows(layout, st["x"], st["filler"])
        w = st.get("weight")
        if grads is not None:
            x = x.detach().clone().requires_grad_(True)
            if w is not None and "weight" in spec.grad_input_names:
                st = {**st, "weight": w.detach().clone().requires_grad_(True)}
        out = self.call(spec, op, st, x, keys, layout)
        if grads is not None:
            go = oi.grad_rows(keys, out, st["seed"], st["batch"])
            out.backward(go)
            grads["x"] = _back(keys, x.grad)
            if w is not None and "weight" in spec.grad_input_names and st["weight"].grad is not None:
                grads["weight"] = st["weight"].grad.detach()
        return _back(keys, out.detach())


class _TokenRowsPos(_TokenRows):
    def call(self, spec, op, st, x, keys, layout):
        h = spec.params["heads"]
        pos = torch.tensor([k[1] if k is not None else 0 for k in keys], device=x.device)
        # rows are tokens: heads lead, so that the token axis is the sequence axis next to D
        return op(x.view(x.shape[0], h, -1).transpose(0, 1), pos).transpose(0, 1).reshape(x.shape[0], -1)

    def gold(self, spec, st, batch):
        keys = list(batch.logical_keys())
        x = torch.stack([st["x"][k] for k in keys])
        h = spec.params["heads"]
        pos = torch.tensor([k[1] for k in keys], device=x.device)
        return _back(keys, _gold_rope(x.view(x.shape[0], h, -1), pos).reshape(x.shape[0], -1))


class _TokenRowsPair(_TokenRows):
    def prepare(self, spec, batch, device, dtype, seed):
        st = super().prepare(spec, batch, device, dtype, seed)
        st["up"] = oi.token_table(batch, spec.params["width"], device, dtype, seed + 101)
        return st

    def run(self, spec, op, st, layout, grads=None):
        g, keys = _rows(layout, st["x"], st["filler"])
        u, _ = _rows(layout, st["up"], st["filler"])
        if grads is not None:
            g, u = g.detach().clone().requires_grad_(True), u.detach().clone().requires_grad_(True)
        out = op(g, u)
        if grads is not None:
            out.backward(oi.grad_rows(keys, out, st["seed"], st["batch"]))
            grads["gate"], grads["up"] = _back(keys, g.grad), _back(keys, u.grad)
        return _back(keys, out.detach())

    def gold(self, spec, st, batch):
        keys = list(batch.logical_keys())
        return _back(keys, _gold_swiglu(torch.stack([st["x"][k] for k in keys]), torch.stack([st["up"][k] for k in keys])))


class _TokenRowsWeight(_TokenRows):
    pass                                            # x @ weight^T: the base class already passes the shared weight


class _TokenIds(_TokenRows):
    def prepare(self, spec, batch, device, dtype, seed):
        p = spec.params
        ids = {(t.sample_id, t.token_position): torch.tensor(t.token_id % p["vocab"], device=device)
               for s in batch.samples for t in s.tokens()}
        return {"x": ids, "weight": oi.randn((p["vocab"], p["width"]), device, dtype, seed + 5), "filler": torch.tensor(0, device=device)}

    def run(self, spec, op, st, layout, grads=None):
        ids, keys = _rows(layout, st["x"], st["filler"])
        w = st["weight"].detach().clone().requires_grad_(True) if grads is not None else st["weight"]
        out = op(ids, w)
        if grads is not None:
            go = oi.grad_rows(keys, out, st["seed"], st["batch"])
            go = go * torch.tensor([k is not None for k in keys], device=go.device, dtype=go.dtype).unsqueeze(-1)
            out.backward(go)
            grads["weight"] = w.grad.detach()
        return _back(keys, out.detach())

    def gold(self, spec, st, batch):
        keys = list(batch.logical_keys())
        return _back(keys, st["weight"].float()[torch.stack([st["x"][k] for k in keys])])


class _TokenLogpLinear(_TokenRows):
    def prepare(self, spec, batch, device, dtype, seed):
        st = super().prepare(spec, batch, device, dtype, seed)
        st["weight"] = oi.randn((spec.params["vocab"], spec.params["width"]), device, dtype, seed + 9, scale=0.15)
        st["targets"] = {(t.sample_id, t.token_position): torch.tensor((t.token_id * 7 + t.token_position) % spec.params["vocab"],
                                                                         device=device) for s in batch.samples for t in s.tokens()}
        return st

    def call(self, spec, op, st, x, keys, layout):
        tg = torch.stack([st["targets"][k] if k is not None else torch.tensor(0, device=x.device) for k in keys])
        return op(x, st["weight"], tg)

    def gold(self, spec, st, batch):
        keys = list(batch.logical_keys())
        x = torch.stack([st["x"][k] for k in keys])
        return _back(keys, _gold_linear_logp(x, st["weight"], torch.stack([st["targets"][k] for k in keys])))


class _TokenLogpLogits(_TokenLogpLinear):
    def prepare(self, spec, batch, device, dtype, seed):
        V = spec.params["vocab"]
        st = {"x": oi.token_table(batch, V, device, dtype, seed, scale=3.0), "weight": None,
              "filler": oi.filler_row(V, device, dtype, seed)}
        st["targets"] = {(t.sample_id, t.token_position): torch.tensor((t.token_id * 7 + t.token_position) % V, device=device)
                         for s in batch.samples for t in s.tokens()}
        return st

    def call(self, spec, op, st, x, keys, layout):
        tg = torch.stack([st["targets"][k] if k is not None else torch.tensor(0, device=x.device) for k in keys])
        return op(x, tg)

    def gold(self, spec, st, batch):
        keys = list(batch.logical_keys())
        return _back(keys, _gold_logp(torch.stack([st["x"][k] for k in keys]), torch.stack([st["targets"][k] for k in keys])))


class _Attention:
    """Causal self-attention per sample; q/k/v per logical token."""

    def prepare(self, spec, batch, device, dtype, seed):
        hq, hkv, d = spec.params["hq"], spec.params["hkv"], 128
        return {"q": oi.token_table(batch, hq * d, device, dtype, seed), "k": oi.token_table(batch, hkv * d, device, dtype, seed + 1),
                "v": oi.token_table(batch, hkv * d, device, dtype, seed + 2), "geom": (hq, hkv, d)}

    def _packed(self, st, layout, batch):
        """Tokens of ``layout`` grouped into whole samples in physical sample order -> packed tensors + cu_seqlens."""
        if isinstance(layout, PaddedBatch):
            order = [(sid, [k for k in row if k is not None]) for sid, row in zip(layout.sample_ids, layout.restore_map)]
        else:
            order, seen = [], {}
            for k in layout.restore_map:
                if k[0] not in seen:
                    seen[k[0]] = []
                    order.append((k[0], seen[k[0]]))
                seen[k[0]].append(k)
        keys = [k for _, ks in order for k in sorted(ks, key=lambda kk: kk[1])]
        cu = [0]
        for _, ks in order:
            cu.append(cu[-1] + len(ks))
        return keys, cu

    def run(self, spec, op, st, layout, grads=None):
        hq, hkv, d = st["geom"]
        keys, cu = self._packed(st, layout, st["batch"])
        q = torch.stack([st["q"][k] for k in keys]).view(-1, hq, d)
        k = torch.stack([st["k"][kk] for kk in keys]).view(-1, hkv, d)
        v = torch.stack([st["v"][kk] for kk in keys]).view(-1, hkv, d)
        if grads is not None:
            q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
        out = op(q, k, v, cu)
        if grads is not None:
            out.backward(oi.grad_rows(keys, out.reshape(len(keys), -1), st["seed"], st["batch"]).view_as(out))
            for name, t in (("q", q), ("k", k), ("v", v)):
                grads[name] = _back(keys, t.grad.reshape(len(keys), -1))
        return _back(keys, out.detach().reshape(len(keys), -1))

    def gold(self, spec, st, batch):
        hq, hkv, d = st["geom"]
        out = {}
        for s in batch.samples:
            ks = [(s.sample_id, p) for p in range(s.seq_len)]
            q = torch.stack([st["q"][k] for k in ks]).view(-1, hq, d)
            k = torch.stack([st["k"][kk] for kk in ks]).view(-1, hkv, d)
            v = torch.stack([st["v"][kk] for kk in ks]).view(-1, hkv, d)
            out.update(_back(ks, _gold_attention_seq(q, k, v).reshape(len(ks), -1)))
        return out


class _AttentionChunked(_Attention):
    """Chunked prefill / decode over a block KV cache: every chunk of a sample attends to the cache filled so far.
    Layouts that are not chunked run each sample as a single chunk."""

    def run(self, spec, op, st, layout, grads=None):
        from rl_kernel_b200.ops.attention.paged import PAGE, paged_attention_block_table, write_kv_slots

        hq, hkv, d = st["geom"]
        batch = st["batch"]
        dev = next(iter(st["q"].values())).device
        dtype = next(iter(st["q"].values())).dtype
        if isinstance(layout, PhysicalLayout) and layout.layout_kind == "chunked":
            segs = list(zip(layout.segment_sample_ids, layout.segment_position_starts, layout.segment_lengths))
        else:
            sids = layout.sample_ids if isinstance(layout, PaddedBatch) else list(dict.fromkeys(k[0] for k in layout.restore_map))
            segs = [(sid, 0, batch.sample(sid).seq_len) for sid in sids]
        pages_of, nxt = {}, 0
        for sid in dict.fromkeys(s[0] for s in segs):
            need = (batch.sample(sid).seq_len + PAGE - 1) // PAGE
            pages_of[sid] = list(range(nxt, nxt + need))
            nxt += need
        kv = torch.zeros(2, nxt, PAGE, hkv, d, device=dev, dtype=dtype)
        kp, vp = kv[0].view(-1, hkv * d), kv[1].view(-1, hkv * d)
        out = {}
        for sid, start, n in segs:                                  # chunks of a sample arrive in ascending order
            ks = [(sid, p) for p in range(start, start + n)]
            q = torch.stack([st["q"][k] for k in ks]).view(n, hq, d)
            slots = torch.tensor([pages_of[sid][p // PAGE] * PAGE + p % PAGE for p in range(start, start + n)], device=dev)
            write_kv_slots(kp, vp, torch.stack([st["k"][k] for k in ks]), torch.stack([st["v"][k] for k in ks]), slots)
            table = torch.tensor([pages_of[sid]], dtype=torch.int32, device=dev)
            o = paged_attention_block_table(q, kp, vp, table, [start + n], [0, n], num_kv_heads=hkv)
            out.update(_back(ks, o.reshape(n, -1)))
        return out


class _PrefixShared:
    """G candidates of one prompt attend to the prompt's K/V; logical token = (sample, position) of a candidate row."""

    def prepare(self, spec, batch, device, dtype, seed):
        hq, hkv, d = spec.params["hq"], spec.params["hkv"], 128
        return {"q": oi.token_table(batch, hq * d, device, dtype, seed), "geom": (hq, hkv, d),
                "k": oi.randn((40, hkv, d), device, dtype, seed + 3), "v": oi.randn((40, hkv, d), device, dtype, seed + 4)}

    def run(self, spec, op, st, layout, grads=None):
        hq, hkv, d = st["geom"]
        keys = [k for k in ([kk for row in layout.restore_map for kk in row] if isinstance(layout, PaddedBatch) else layout.restore_map)
                if k is not None]
        q = torch.stack([st["q"][k] for k in keys]).view(1, len(keys), 1, hq, d)        # every row is one "candidate"
        o = op(q, st["k"][None], st["v"][None])
        return _back(keys, o.reshape(len(keys), -1))

    def gold(self, spec, st, batch):
        hq, hkv, d = st["geom"]
        keys = list(batch.logical_keys())
        q = torch.stack([st["q"][k] for k in keys]).view(1, len(keys), 1, hq, d)
        return _back(keys, GtestPrefixSharedAttentionOp().forward_fp32(q, st["k"][None], st["v"][None]).reshape(len(keys), -1))


class _Pack:
    def prepare(self, spec, batch, device, dtype, seed):
        return {"x": oi.token_table(batch, spec.params["width"], device, dtype, seed),
                "filler": oi.filler_row(spec.params["width"], device, dtype, seed)}

    def run(self, spec, op, st, layout, grads=None):
        from rl_kernel_b200.config.workload import apply_padding

        padded = layout if isinstance(layout, PaddedBatch) else apply_padding(
            LogicalBatch(st["batch"].workload_id, st["batch"].seed,
                         tuple(st["batch"].sample(sid) for sid in dict.fromkeys(k[0] for k in layout.restore_map))), pad_side="right")
        rows, keys = _rows(padded, st["x"], st["filler"])
        B, L = len(padded.restore_map), padded.padded_len
        mask = torch.tensor(padded.physical_attention_mask, dtype=torch.bool, device=rows.device)
        out = op(rows.view(B, L, -1), mask)
        return _back(keys, out.reshape(B * L, -1))

    def gold(self, spec, st, batch):
        return {k: st["x"][k].float() for k in batch.logical_keys()}


class _Loss:
    """GRPO loss terms: the per-token quantity compared is d(loss)/d(logp) and the three scalars must agree between a
    batched run and the sum of singleton runs with the same global denominator."""

    def prepare(self, spec, batch, device, dtype, seed):
        f32 = torch.float32
        lp = oi.token_table(batch, 1, device, f32, seed, scale=0.3)
        return {"logp": {k: -v.abs() for k, v in lp.items()},
                "old": {k: -v.abs() for k, v in oi.token_table(batch, 1, device, f32, seed + 1, scale=0.3).items()},
                "ref": {k: -v.abs() for k, v in oi.token_table(batch, 1, device, f32, seed + 2, scale=0.3).items()},
                "adv": {s.sample_id: torch.tensor(1.0 if i % 2 == 0 else -0.7, device=device) for i, s in enumerate(
                    sorted(batch.samples, key=lambda s: s.sample_id))}}

    def run(self, spec, op, st, layout, grads=None):
        from rl_kernel_b200.config.workload import apply_padding

        batch = st["batch"]
        sids = layout.sample_ids if isinstance(layout, PaddedBatch) else list(dict.fromkeys(k[0] for k in layout.restore_map))
        sub = LogicalBatch(batch.workload_id, batch.seed, tuple(batch.sample(s) for s in sids))
        padded = layout if isinstance(layout, PaddedBatch) else apply_padding(sub, pad_side="right")
        B, L = len(sids), padded.padded_len
        dev = next(iter(st["logp"].values())).device
        z = torch.zeros(1, device=dev)
        pick = lambda tab: torch.stack([tab[k] if k is not None else z for row in padded.restore_map for k in row]).view(B, L)  # noqa: E731
        mask = torch.tensor(padded.physical_loss_mask, dtype=torch.bool, device=dev)
        lp = pick(st["logp"]).detach().clone().requires_grad_(True)
        adv = torch.stack([st["adv"][s] for s in sids])
        # every run divides by the fixture's global active-token count (the chain's loss denominator), so that runs over
        # subsets of the batch are commensurable term by term
        loss, _pol, _kl = op(lp, pick(st["old"]), pick(st["ref"]), adv, mask, clip_eps=0.2, beta=0.01,
                             denominator=float(batch.active_token_count()))
        loss.backward()
        keys = [k for row in padded.restore_map for k in row]
        return _back(keys, lp.grad.reshape(B * L, 1))

    def gold(self, spec, st, batch):
        out = {}
        n = float(batch.active_token_count())
        for s in batch.samples:
            for p in range(s.seq_len):
                k = (s.sample_id, p)
                if p < s.prompt_len:
                    out[k] = torch.zeros(1, device=st["logp"][k].device)
                    continue
                lp = st["logp"][k].double().requires_grad_(True)
                ratio = torch.exp(lp - st["old"][k].double())
                a = st["adv"][s.sample_id].double()
                pol = -torch.minimum(ratio * a, torch.clamp(ratio, 0.8, 1.2) * a)
                d = st["ref"][k].double() - lp
                (pol + 0.01 * (torch.exp(d) - d - 1)).sum().div(n).backward()
                out[k] = lp.grad.float()
        return out


class _Sampling:
    """Keyed sampling: the draw of a token position depends on its key (sample, position), never on its row."""

    def prepare(self, spec, batch, device, dtype, seed):
        V = spec.params["vocab"]
        order = {sid: i for i, sid in enumerate(sorted(batch.sample_ids))}
        return {"x": oi.token_table(batch, V, device, dtype, seed, scale=2.0), "filler": oi.filler_row(V, device, dtype, seed),
                "key": {k: torch.tensor(order[k[0]] * 65536 + k[1], device=device) for k in batch.logical_keys()}}

    def run(self, spec, op, st, layout, grads=None):
        x, keys = _rows(layout, st["x"], st["filler"])
        rk = torch.stack([st["key"][k] if k is not None else torch.tensor(2 ** 40, device=x.device) for k in keys]).long()
        if x.is_cuda:
            ids = op(x, temperature=0.9, seed=77, row_keys=rk)
        else:
            # the PyTorch sampler has no per-row keys: draw every row from its own generator
            ids = torch.stack([op(x[i:i + 1], temperature=0.9, generator=torch.Generator().manual_seed(int(rk[i]) % (2 ** 31)))[0]
                               for i in range(x.shape[0])])
        return _back(keys, ids.view(-1, 1))

    def gold(self, spec, st, batch):
        return {}                                                  # a sample has no fp32 gold; only invariance is judged


ADAPTERS = {"token_rows": _TokenRows(), "token_rows_pos": _TokenRowsPos(), "token_rows_pair": _TokenRowsPair(),
            "token_rows_weight": _TokenRowsWeight(), "token_ids": _TokenIds(), "token_logp_linear": _TokenLogpLinear(),
            "token_logp_logits": _TokenLogpLogits(), "attention": _Attention(), "attention_chunked": _AttentionChunked(),
            "prefix_shared": _PrefixShared(), "pack": _Pack(), "loss": _Loss(), "sampling": _Sampling()}


@dataclass
class CandidateSpec:
    op_name: str
    candidate: str
    device: str
    dtype: torch.dtype
    path: str
    op: Any


def make_candidate(args: argparse.Namespace | None = None, *, op_name: str | None = None, candidate: str = "auto",
                   device: str | None = None, dtype: torch.dtype | None = None) -> CandidateSpec:
    """Candidate from CLI-style ``args`` (``op``, ``candidate``, ``device``, ``dtype``) or keywords.  ``auto`` = ``b200``
    on a CUDA device, ``pytorch`` otherwise."""
    if args is not None:
        op_name = op_name or args.op
        candidate = getattr(args, "candidate", candidate)
        device = device or getattr(args, "device", None)
        dtype = dtype or getattr(args, "dtype", None)
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    if isinstance(dtype, str):
        dtype = getattr(torch, dtype)
    dtype = dtype or (torch.bfloat16 if device.startswith("cuda") else torch.float32)
    spec = OP_SPECS[op_name]
    if candidate == "auto":
        candidate = "b200" if device.startswith("cuda") else "pytorch"
    if candidate == "b200" and not device.startswith("cuda"):
        raise ValueError("the b200 candidate runs on CUDA tensors only")
    if candidate not in spec.candidate_paths:
        raise KeyError(f"operator {op_name} has no candidate {candidate!r}; choose from {sorted(spec.candidate_paths)}")
    op = FACTORIES[op_name]() if op_name in FACTORIES else _load_object(_local(spec.candidate_paths[candidate]))()
    return CandidateSpec(op_name, candidate, device, dtype, spec.candidate_paths[candidate], op)


def _local(path: str) -> str:
    """Spec paths are spelled with the public package name; load them from this package."""
    return "rl_kernel_b200." + path[len("rl_engine."):] if path.startswith("rl_engine.") else path


def make_operator_case(op_name: str, *, batch: LogicalBatch, device: str, dtype: torch.dtype, seed: int = 0):
    """(spec, adapter, prepared state) of one operator on one logical batch."""
    spec = OP_SPECS[op_name]
    adapter = ADAPTERS[spec.adapter]
    st = adapter.prepare(spec, batch, torch.device(device), dtype, seed)
    st["batch"], st["seed"] = batch, seed
    return spec, adapter, st


__all__ = ["ADAPTERS", "CandidateSpec", "FACTORIES", "GOLD", "GtestDevicePackOp", "GtestPackOp", "GtestPrefixSharedAttentionOp",
           "OP_SPECS", "OperatorSpec", "make_candidate", "make_operator_case", "operator_names"]
