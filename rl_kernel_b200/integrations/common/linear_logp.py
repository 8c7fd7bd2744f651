"""The strict "hidden states (or LM-head logits) -> selected-token log-probs" boundary that the
framework bindings share (parity: LinearLogpWrapper and the rollout context helpers,
rl_engine/integrations/common/linear_logp.py:216-1178).

One object serves both engines of an RL step so that rollout and training log-probs are those of the same program:

* ``wrapper(hidden, lm_head_weight, target_ids, ...)``: the fused LM head (tcgen05 GEMM whose epilogue emits the
  128-id tile statistics; no [T, V] logits).  With a tensor-parallel group the shards' tile statistics and the owner's
  target logit are gathered in rank order and merged in ascending tile order on every rank -- no floating-point
  all-reduce -- so the result does not depend on the TP degree.  Differentiable in ``hidden`` and the weight.
* ``from_local_logits``: the same contract on logits a rollout engine has already computed (no second GEMM).
* ``from_local_logits_top_p`` / ``from_local_logits_sparse_nucleus`` / ``from_replicated_logits_sparse_nucleus``:
  the restricted sampling support of top-k / top-p replayed from the id list the sampler kept (compact kernel for up
  to 64 ids per row, masked full pass beyond that), optionally with the entropy of the restricted distribution.
* ``publish_ / take_ / clear_rollout_linear_logp_context``: the hand-over of (hidden, LM head) from a model's
  ``compute_logits`` to the sampler that scores the sampled ids right after it.

CUDA bf16 operands run the native kernels; anything else runs the PyTorch definition of the same tile contract
(CPU tests, gloo ranks).  ``RL_KERNEL_ALIGNMENT_DIAGNOSTICS=1`` with ``RL_KERNEL_ALIGNMENT_DIAGNOSTICS_DIR`` writes
one bounded record per call (ids, selected logits, results, row checksums) for offline comparison of two engines.
"""
from __future__ import annotations

import hashlib
import os
import pathlib
import threading
from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any

import torch

from rl_kernel_b200.contracts.operators.logprob import LogprobContract, VocabShardingSpec

TILE = 128
COMPACT_REPLAY_WIDTH = 64          # widest id list the compact replay kernel takes
CONTRACT_VERSION = "b200-det-gemm-tile-logp-v1"


# ------------------------------------------------------------------------------------- diagnostics
_DIAG_LOCK = threading.Lock()
_DIAG_CALLS = 0


def _alignment_diagnostics_enabled() -> bool:
    return os.getenv("RL_KERNEL_ALIGNMENT_DIAGNOSTICS", "").strip().lower() in {"1", "true", "yes", "on"}


def _diagnostic_rank() -> int:
    try:
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            return int(torch.distributed.get_rank())
    except (RuntimeError, ValueError):
        pass
    try:
        return int(os.getenv("RANK", "0"))
    except ValueError:
        return 0


def alignment_tensor_summary(value: torch.Tensor) -> dict[str, Any]:
    """Shape, dtype, ends, fp32 checksums and a digest of the raw bytes of ``value`` (the digest is what two
    engines compare first: equal digests end the search)."""
    t = value.detach()
    flat = t.reshape(-1)
    out: dict[str, Any] = {"shape": list(t.shape), "dtype": str(t.dtype).removeprefix("torch."), "device": str(t.device),
                           "first16": flat[:16].float().cpu().tolist(), "last16": flat[-16:].float().cpu().tolist()}
    if t.numel():
        f = t.float()
        out.update(sum_fp32=float(f.sum()), abs_sum_fp32=float(f.abs().sum()), min_fp32=float(f.min()), max_fp32=float(f.max()),
                   sha256=hashlib.sha256(t.contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest())
    return out


def _record_alignment_diagnostics(*, target: str, target_ids: torch.Tensor, result: torch.Tensor, lse: torch.Tensor | None,
                                  vocab_start_index: int, local_logits: torch.Tensor | None = None,
                                  hidden: torch.Tensor | None = None, lm_head_weight: torch.Tensor | None = None) -> None:
    """Cold unless explicitly enabled: device-to-host copies and reductions for debugging only."""
    if not _alignment_diagnostics_enabled():
        return
    root = os.getenv("RL_KERNEL_ALIGNMENT_DIAGNOSTICS_DIR", "").strip()
    if not root:
        return
    global _DIAG_CALLS
    with _DIAG_LOCK:
        call_index = _DIAG_CALLS
        _DIAG_CALLS += 1
    payload: dict[str, Any] = {
        "schema_version": "rl_kernel_b200.linear_logp_alignment_diagnostic.v1", "target": target, "rank": _diagnostic_rank(),
        "pid": os.getpid(), "call_index": call_index, "vocab_start_index": int(vocab_start_index),
        "target_ids": target_ids.detach().to("cpu", torch.int64), "result": result.detach().float().cpu(),
        "lse": None if lse is None else lse.detach().float().cpu()}
    if local_logits is not None:
        lg = local_logits.detach()
        local = target_ids.detach().long() - int(vocab_start_index)
        own = (local >= 0) & (local < lg.shape[1])
        sel = lg.gather(1, local.clamp(0, max(lg.shape[1] - 1, 0)).reshape(-1, 1)).reshape(-1).float()
        payload.update(selected_local_logits=torch.where(own, sel, torch.full_like(sel, float("nan"))).cpu(),
                       row_sum_fp32=lg.float().sum(1).cpu(), row_abs_sum_fp32=lg.float().abs().sum(1).cpu(),
                       logits_head=lg[:, :8].cpu(), logits_tail=lg[:, -8:].cpu(), logits_summary=alignment_tensor_summary(lg))
    if hidden is not None:
        payload.update(hidden=hidden.detach().cpu(), hidden_summary=alignment_tensor_summary(hidden))
    if lm_head_weight is not None:
        w = lm_head_weight.detach()
        payload.update(lm_head_weight_head=w[:8].cpu(), lm_head_weight_tail=w[-8:].cpu(),
                       lm_head_weight_summary=alignment_tensor_summary(w))
    out_dir = pathlib.Path(root)
    out_dir.mkdir(parents=True, exist_ok=True)
    torch.save(payload, out_dir / f"{target}-pid{os.getpid()}-rank{_diagnostic_rank():05d}-call{call_index:08d}.pt")


# ------------------------------------------------------------------------------------- rollout hand-over
@dataclass(frozen=True)
class RolloutLinearLogpContext:
    """The exact hidden rows and LM-head shard behind the logits the next sampler call will sample from."""
    hidden: torch.Tensor
    lm_head_weight: torch.Tensor
    lm_head_bias: torch.Tensor | None
    tp_group: Any
    vocab_start_index: int
    global_vocab_size: int
    real_vocab_size: int


_ROLLOUT_CONTEXT: RolloutLinearLogpContext | None = None


def publish_rollout_linear_logp_context(hidden: torch.Tensor, lm_head_weight: torch.Tensor, lm_head_bias: torch.Tensor | None, *,
                                        tp_group: Any, vocab_start_index: int, global_vocab_size: int,
                                        real_vocab_size: int) -> None:
    """Called by the patched ``compute_logits``: one context for the sampler invocation that follows."""
    global _ROLLOUT_CONTEXT
    if hidden.ndim != 2:
        raise ValueError(f"rollout linear_logp hidden must be [tokens, hidden], got {tuple(hidden.shape)}")
    if lm_head_weight.ndim != 2:
        raise ValueError("rollout linear_logp LM-head weight must be [vocab_local, hidden]")
    if hidden.device != lm_head_weight.device:
        raise ValueError("rollout linear_logp hidden and LM-head must share a device")
    if hidden.shape[1] != lm_head_weight.shape[1]:
        raise ValueError("rollout linear_logp hidden and LM-head hidden widths must match")
    if lm_head_bias is not None and (lm_head_bias.ndim != 1 or lm_head_bias.shape[0] != lm_head_weight.shape[0]
                                     or lm_head_bias.device != hidden.device):
        raise ValueError("rollout linear_logp bias must match the complete local LM-head shard")
    if int(global_vocab_size) <= 0 or int(real_vocab_size) <= 0:
        raise ValueError("rollout linear_logp vocab sizes must be positive")
    if int(real_vocab_size) > int(global_vocab_size):
        raise ValueError("rollout linear_logp real vocab cannot exceed padded global vocab")
    _ROLLOUT_CONTEXT = RolloutLinearLogpContext(hidden, lm_head_weight, lm_head_bias, tp_group, int(vocab_start_index),
                                                int(global_vocab_size), int(real_vocab_size))


def clear_rollout_linear_logp_context() -> None:
    """Logits were computed but nothing will be sampled from them (e.g. a prompt-logprob pass)."""
    global _ROLLOUT_CONTEXT
    _ROLLOUT_CONTEXT = None


def take_rollout_linear_logp_context() -> RolloutLinearLogpContext:
    """Consume the context of the matching ``compute_logits`` call; a sampler without one is an error."""
    global _ROLLOUT_CONTEXT
    ctx, _ROLLOUT_CONTEXT = _ROLLOUT_CONTEXT, None
    if ctx is None:
        raise RuntimeError("strict rollout linear_logp sampler has no matching hidden/LM-head context")
    return ctx


# ------------------------------------------------------------------------------------- transport over a TP group
class _Transport:
    """Rank-ordered all-gather over whatever the caller calls its tensor-parallel group: ``None`` (one rank), an
    object with ``world`` / ``rank`` / ``all_gather`` (the deterministic collectives of this package) or a
    ``torch.distributed`` process group."""

    def __init__(self, tp_group: Any):
        self.group, self.collective = tp_group, None
        if tp_group is None:
            self.rank, self.world = 0, 1
        elif hasattr(tp_group, "all_gather") and hasattr(tp_group, "world"):
            self.collective, self.rank, self.world = tp_group, int(tp_group.rank), int(tp_group.world)
        else:
            import torch.distributed as dist

            if not (dist.is_available() and dist.is_initialized()):
                raise RuntimeError("strict TP linear_logp requires initialized torch.distributed")
            self.rank, self.world = int(dist.get_rank(group=tp_group)), int(dist.get_world_size(group=tp_group))

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[...] -> [world, ...] in rank order, bits unchanged."""
        if self.world == 1:
            return t.unsqueeze(0)
        if self.collective is not None:
            return self.collective.all_gather(t)
        import torch.distributed as dist

        t = t.contiguous()
        out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        if t.is_cuda:
            dist.all_gather_into_tensor(out, t, group=self.group)
        else:
            dist.all_gather(list(out.unbind(0)), t, group=self.group)
        return out

    def tree_sum(self, t: torch.Tensor) -> torch.Tensor:
        """Fixed balanced-tree sum over the ranks (rounded to ``t.dtype`` at every node)."""
        if self.world == 1:
            return t
        if self.collective is not None and hasattr(self.collective, "all_reduce"):
            return self.collective.all_reduce(t)
        from rl_kernel_b200.distributed.algorithms.collectives import balanced_tree_sum

        return balanced_tree_sum(list(self.all_gather(t).unbind(0)), t.dtype)


# ------------------------------------------------------------------------------------- the tile contract on one shard
def _native(*tensors: torch.Tensor) -> bool:
    from rl_kernel_b200.ops._dispatch import use_native

    return all(t.dtype == torch.bfloat16 for t in tensors) and use_native(*tensors)


def _shard_stats_from_hidden(hidden, weight, targets, *, vocab_start: int, inv_temp: float, min_keep):
    """(stats [n, tiles of this shard, 2], target z [n] -- zero unless this shard owns the target)."""
    n, nt = hidden.shape[0], (weight.shape[0] + TILE - 1) // TILE
    if _native(hidden, weight):
        from rl_kernel_b200.backends import native as nv

        # the kernel addresses tile slots by global tile number: give it a row of vocab_start / 128 + nt slots and keep
        # this shard's part
        tz = torch.zeros(n, device=hidden.device, dtype=torch.float32)
        full = torch.zeros(n, vocab_start // TILE + nt, 2, device=hidden.device, dtype=torch.float32)
        nv.lmhead_logp_stats(hidden.contiguous(), weight.contiguous(), targets.contiguous(), full, tz, vocab_start=vocab_start,
                             inv_temp=inv_temp, min_keep=None if min_keep is None else min_keep.float().contiguous())
        return full[:, vocab_start // TILE:].contiguous(), tz
    from rl_kernel_b200.reference.logprob.tile_logp import NativeLinearLogpOp

    op = NativeLinearLogpOp(1.0)
    op.inv_temp = inv_temp
    st, tz, _ = op(hidden, weight, targets, vocab_start=vocab_start, n_tiles_total=vocab_start // TILE + nt, return_stats=True,
                   min_keep=min_keep)
    return st[:, vocab_start // TILE:].contiguous(), tz


def _shard_stats_from_logits(logits, targets, *, vocab_start: int, inv_temp: float, min_keep, keep_mask=None):
    n, nt = logits.shape[0], (logits.shape[1] + TILE - 1) // TILE
    if keep_mask is None and logits.shape[1] % 8 == 0 and _native(logits):
        from rl_kernel_b200.backends import native as nv

        full = torch.zeros(n, vocab_start // TILE + nt, 2, device=logits.device, dtype=torch.float32)
        tz = torch.zeros(n, device=logits.device, dtype=torch.float32)
        nv.logits_tile_stats(logits.contiguous(), targets.contiguous(), full, tz, vocab_start=vocab_start, inv_temp=inv_temp,
                             min_keep=None if min_keep is None else min_keep.float().contiguous())
        return full[:, vocab_start // TILE:].contiguous(), tz
    from rl_kernel_b200.reference.logprob.tile_logp import _restrict, _target_z, tile_stats_reference

    lg = _restrict(logits, inv_temp, min_keep, keep_mask)
    st = tile_stats_reference(lg, vocab_start=vocab_start, inv_temp=inv_temp, n_tiles_total=vocab_start // TILE + nt)
    tz, _ = _target_z(lg, targets, vocab_start, inv_temp)
    return st[:, vocab_start // TILE:].contiguous(), tz


def _merge(stats: torch.Tensor, tz: torch.Tensor):
    """Ordered merge of a row's tile statistics -> (logp, lse)."""
    if stats.is_cuda:
        from rl_kernel_b200.backends import native as nv
        from rl_kernel_b200.ops._dispatch import use_native

        if use_native(stats):
            lp, lse = torch.empty_like(tz), torch.empty_like(tz)
            nv.logp_merge(stats.contiguous(), tz.contiguous(), lp, lse)
            return lp, lse
    from rl_kernel_b200.reference.logprob.tile_logp import merge_tile_stats

    return merge_tile_stats(stats, tz)


def _pad_tiles(stats: torch.Tensor, n_tiles: int) -> torch.Tensor:
    """A shard whose tail is vocabulary padding has fewer real tiles: empty tiles (-inf, 0) fill its list to the
    shard's width so that every rank contributes the same number of slots."""
    if stats.shape[1] >= n_tiles:
        return stats
    pad = stats.new_zeros(stats.shape[0], n_tiles - stats.shape[1], 2)
    pad[..., 0] = float("-inf")
    return torch.cat([stats, pad], dim=1)


def _gathered_merge(tr: _Transport, stats: torch.Tensor, tz: torch.Tensor, shard_tiles: int | None = None):
    if tr.world > 1:
        if shard_tiles is not None:
            stats = _pad_tiles(stats, shard_tiles)
        stats = tr.all_gather(stats).permute(1, 0, 2, 3).reshape(stats.shape[0], -1, 2).contiguous()   # rank-major = tile order
        tz = tr.all_gather(tz).sum(0)                      # exactly one shard holds a non-zero entry per row
    return _merge(stats, tz)


class _TPLinearLogpFn(torch.autograd.Function):
    """Vocabulary-parallel fused LM-head log-prob over a ``torch.distributed`` group, with gradients: the backward
    recomputes this shard's logits in row chunks, forms d(logits) from the saved log-sum-exp, and sums the hidden
    gradient over the shards with the fixed balanced tree."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, wrapper_state):
        tr, vocab_start, inv_temp, min_keep, shard_tiles = wrapper_state
        with torch.no_grad():
            st, tz = _shard_stats_from_hidden(hidden, weight, targets, vocab_start=vocab_start, inv_temp=inv_temp, min_keep=min_keep)
            lp, lse = _gathered_merge(tr, st, tz, shard_tiles)
        ctx.save_for_backward(hidden, weight, targets, lse)
        ctx.state = wrapper_state
        ctx.mark_non_differentiable(lse)
        return lp, lse

    @staticmethod
    def backward(ctx, g, _g_lse):
        from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_da, det_gemm_db, det_gemm_fwd

        hidden, weight, targets, lse = ctx.saved_tensors
        tr, vocab_start, inv_temp, min_keep, _ = ctx.state
        V = weight.shape[0]
        Vp = (V + 7) // 8 * 8                                     # the GEMMs want multiples of 8: zero rows, masked below
        wp = weight if Vp == V else torch.cat([weight, weight.new_zeros(Vp - V, weight.shape[1])])
        dh = torch.zeros_like(hidden)
        dw = torch.zeros(Vp, weight.shape[1], device=weight.device, dtype=torch.float32)
        local = targets.long() - vocab_start
        own = (local >= 0) & (local < V)
        for a in range(0, hidden.shape[0], 2048):
            b = min(hidden.shape[0], a + 2048)
            z = det_gemm_fwd(hidden[a:b].contiguous(), wp).float() * inv_temp       # this shard's scaled logits
            z[:, V:] = float("-inf")
            if min_keep is not None:
                z = z.masked_fill(z < min_keep[a:b].float().reshape(-1, 1), float("-inf"))
            gg = g[a:b].float().reshape(-1, 1)
            dz = -torch.exp(z - lse[a:b].reshape(-1, 1)) * gg
            rows = torch.nonzero(own[a:b]).reshape(-1)
            dz[rows, local[a:b][rows]] += gg.reshape(-1)[rows]
            dl = (dz * inv_temp).to(hidden.dtype)
            dh[a:b] = det_gemm_da(dl, wp).to(hidden.dtype)
            dw += det_gemm_db(dl, hidden[a:b].contiguous()).float()
        return tr.tree_sum(dh), dw[:V].to(weight.dtype), None, None


# ------------------------------------------------------------------------------------- the wrapper
class LinearLogpWrapper:
    """See the module docstring.  Constructor arguments are defaults for the per-call keywords, so a worker can
    bind temperature / vocabulary geometry once (``LinearLogpWrapper(temperature, real_vocab, tp_group, vocab_start,
    padded_vocab)``) or pass them per call as the reference's wrapper does."""

    backend_id = "rl_kernel_b200.linear_logp.bitwise.v1"

    def __init__(self, temperature: float | None = None, real_vocab: int | None = None, tp_group: Any = None,
                 vocab_start: int = 0, padded_vocab: int | None = None):
        self.temperature, self.real_vocab = temperature, real_vocab
        self.tp_group, self.vocab_start, self.padded_vocab = tp_group, int(vocab_start), padded_vocab
        self._last_provenance: dict[str, Any] = {}
        self.contract: LogprobContract | None = None
        self._checked = False

    # ---- introspection
    @property
    def provenance(self) -> Mapping[str, Any]:
        return dict(self._last_provenance)

    def contract_for(self, num_tokens: int, mask=None, *, tp_group: Any = None, real_vocab_size: int | None = None,
                     padded_vocab_size: int | None = None, temperature: float | None = None) -> LogprobContract:
        tr = _Transport(tp_group if tp_group is not None else self.tp_group)
        real = real_vocab_size or self.real_vocab or padded_vocab_size or self.padded_vocab or TILE
        padded = padded_vocab_size or self.padded_vocab or (real + TILE * tr.world - 1) // (TILE * tr.world) * (TILE * tr.world)
        vocab = VocabShardingSpec(tp_size=tr.world, real_vocab=real, padded_vocab=padded)
        return LogprobContract.for_tokens(num_tokens, real_vocab_size=vocab.real_vocab, padded_vocab_size=vocab.padded_vocab,
                                          tp_rank=tr.rank, tp_world_size=tr.world,
                                          temperature=float(temperature or self.temperature or 1.0), active_mask=mask)

    # ---- argument checks shared by the entry points
    @staticmethod
    def _tp_coordinates(tp_group: Any) -> tuple[int, int]:
        tr = _Transport(tp_group)
        return tr.rank, tr.world

    @staticmethod
    def _temperature_rows(temperature: float | torch.Tensor | None, rows: int) -> list[tuple[float, torch.Tensor | None]]:
        """[(temperature, row index tensor or None for all rows)]: one entry per distinct value.  Rows are independent
        in every kernel here, so scoring the rows of each temperature separately gives the bits of one call."""
        if temperature is None:
            return [(1.0, None)]
        if isinstance(temperature, torch.Tensor):
            v = temperature.detach().float().reshape(-1)
            if v.numel() not in (1, rows):
                raise ValueError(f"temperature must be scalar or one value per row, got {v.numel()}")
            if not bool((v > 0).all()):
                raise ValueError("temperature must be positive")
            if v.numel() == 1 or bool((v == v[0]).all()):
                return [(float(v[0]), None)]
            return [(float(u), torch.nonzero(v == u).reshape(-1)) for u in torch.unique(v)]
        t = float(temperature)
        if not t > 0:
            raise ValueError(f"temperature must be positive, got {t}")
        return [(t, None)]

    @staticmethod
    def _validate_targets(target_ids: torch.Tensor, *, rows: int, real_vocab_size: int) -> None:
        if target_ids.ndim != 1 or target_ids.numel() != rows:
            raise ValueError(f"linear_logp target_ids must be [rows]={rows}, got {tuple(target_ids.shape)}")
        if target_ids.is_floating_point() or target_ids.is_complex():
            raise TypeError("linear_logp target_ids must use an integer dtype")
        if target_ids.numel():
            t = target_ids.long()
            valid = ((t >= 0) & (t < real_vocab_size)).all()
            if valid.is_cuda:
                torch._assert_async(valid, f"linear_logp target_ids must be in [0, {real_vocab_size})")
            elif not bool(valid):
                raise ValueError(f"linear_logp target_ids must be in [0, {real_vocab_size}), got invalid ids")

    def _geometry(self, local_vocab: int, *, tp_group: Any, vocab_start_index: int | None, global_vocab_size: int | None,
                  real_vocab_size: int | None, what: str) -> tuple[_Transport, int, int, int]:
        """(transport, vocab_start, global vocabulary, real vocabulary) after the shard checks."""
        group = tp_group if tp_group is not None else self.tp_group
        tr = _Transport(group)
        start = self.vocab_start if vocab_start_index is None else int(vocab_start_index)
        glob = global_vocab_size if global_vocab_size is not None else (self.padded_vocab if group is self.tp_group else None)
        glob = local_vocab * tr.world if glob is None else int(glob)
        if glob <= 0:
            raise ValueError("linear_logp global_vocab_size must be positive")
        if tr.world > 1 or start != 0:
            if group is None:
                raise ValueError("TP linear_logp requires an explicit TP process group")
            if glob != local_vocab * tr.world:
                raise ValueError(f"{what} requires complete equal shards: local={local_vocab}, world={tr.world}, global={glob}")
            if start != tr.rank * local_vocab:
                raise ValueError(f"{what} vocab_start_index does not match the rank-local shard: got {start}, "
                                 f"expected {tr.rank * local_vocab}")
            if tr.world > 1 and local_vocab % TILE:
                raise ValueError(f"{what}: a vocabulary shard must be whole {TILE}-id tiles (got {local_vocab} ids); pad the LM head")
        elif glob != local_vocab:
            raise ValueError("non-TP linear_logp must use the complete local vocab at offset zero")
        real = real_vocab_size if real_vocab_size is not None else (self.real_vocab if self.real_vocab is not None else glob)
        real = int(real)
        if not 0 < real <= glob:
            raise ValueError(f"linear_logp real_vocab_size must be in [1, {glob}], got {real}")
        return tr, start, glob, real

    def _note(self, **kw: Any) -> None:
        self._last_provenance = {
            "module": "logp", "actual_backend": self.backend_id, "deterministic_linear_logp": True, "contract_version": CONTRACT_VERSION,
            "arithmetic_contract": {"batch_invariant": True, "fixed_k_reduction": True, "vocab_tile_width": TILE,
                                    "summary_merge_order": "ascending_tile", "vocab_reduction_axis": "TP",
                                    "cp_is_merge_axis": False, "output_dtype": "fp32"},
            **kw}

    # ---- hidden states -> log-probs
    def __call__(self, hidden: torch.Tensor, lm_head_weight: torch.Tensor, target_ids: torch.Tensor,
                 bias: torch.Tensor | None = None, *, mask: torch.Tensor | None = None, tp_group: Any = None,
                 vocab_start_index: int | None = None, global_vocab_size: int | None = None, real_vocab_size: int | None = None,
                 target: str = "training", temperature: float | torch.Tensor | None = None,
                 min_keep: torch.Tensor | None = None, return_lse: bool = False):
        shp = target_ids.shape
        h = hidden.reshape(-1, hidden.shape[-1])
        tg = target_ids.reshape(-1)
        if h.ndim != 2 or lm_head_weight.ndim != 2:
            raise ValueError("linear_logp expects hidden [tokens, hidden] and an LM-head shard [vocab_local, hidden]")
        if lm_head_weight.device != h.device or tg.device != h.device:
            raise ValueError("linear_logp hidden, LM-head and target_ids must share a device")
        if h.shape[1] != lm_head_weight.shape[1]:
            raise ValueError("linear_logp hidden width must match LM-head width")
        if bias is not None and (bias.ndim != 1 or bias.shape[0] != lm_head_weight.shape[0] or bias.device != h.device):
            raise ValueError("linear_logp bias must match the complete local LM-head shard")
        tr, start, glob, real = self._geometry(lm_head_weight.shape[0], tp_group=tp_group, vocab_start_index=vocab_start_index,
                                               global_vocab_size=global_vocab_size, real_vocab_size=real_vocab_size,
                                               what="TP linear_logp")
        self._validate_targets(tg, rows=h.shape[0], real_vocab_size=real)
        if not self._checked and self.tp_group is not None and tr.collective is None:
            self.contract = self.contract_for(tg.numel(), mask, tp_group=tr.group, real_vocab_size=real, padded_vocab_size=glob,
                                              temperature=None if isinstance(temperature, torch.Tensor) else temperature)
            self.contract.preflight(tr.group)
            self._checked = True
        temperature = self.temperature if temperature is None else temperature
        mk = None if min_keep is None else min_keep.reshape(-1)
        real_rows = max(0, min(lm_head_weight.shape[0], real - start))      # rows of this shard that are real ids
        w = lm_head_weight[:real_rows]
        lp = torch.empty(h.shape[0], device=h.device, dtype=torch.float32)
        lse = torch.empty(h.shape[0], device=h.device, dtype=torch.float32)
        pieces = self._temperature_rows(temperature, h.shape[0])
        path = ""
        for t, rows in pieces:
            hh, tt = (h, tg) if rows is None else (h[rows], tg[rows])
            kk = mk if (mk is None or rows is None) else mk[rows]
            if bias is not None:
                # a biased head: the logits are materialised once (GEMM, bias, rounding) and scored from there
                from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_fwd

                logits = (det_gemm_fwd(hh.contiguous(), w.contiguous()).float() + bias[:real_rows].float()).to(hh.dtype)
                p_lp, p_lse = self._logits_piece(tr, logits, tt, start, t, kk, None)
                path = "materialised_logits_with_bias"
            elif tr.world == 1:
                p_lp, p_lse = self._single_rank_piece(hh, w, tt, t, kk, need_lse=return_lse)
                path = "fused_lm_head"
            elif tr.collective is not None and kk is None and not return_lse and self._native_vp_ok(hh, lm_head_weight, glob):
                from rl_kernel_b200.ops.distributed.vocab_parallel_logp import VocabParallelLinearLogpOp

                op = VocabParallelLinearLogpOp(real_vocab=real, padded_vocab=glob, collective=tr.collective, temperature=t)
                p_lp, p_lse = op(hh, lm_head_weight, tt), None
                path = "fused_lm_head_vocab_parallel_peer_memory"
            else:
                p_lp, p_lse = _TPLinearLogpFn.apply(hh.contiguous(), w.contiguous(), tt.contiguous(),
                                                    (tr, start, 1.0 / t, kk, lm_head_weight.shape[0] // TILE))
                path = "fused_lm_head_vocab_parallel_gather"
            if rows is None:
                lp, lse = p_lp, p_lse
            else:
                lp = lp.index_copy(0, rows, p_lp)
                if p_lse is not None:
                    lse = lse.index_copy(0, rows, p_lse)
        if return_lse and lse is None:
            raise RuntimeError("this path does not expose the log-sum-exp; call without return_lse")
        _record_alignment_diagnostics(target=target, target_ids=tg, result=lp, lse=lse if isinstance(lse, torch.Tensor) else None,
                                      vocab_start_index=start, hidden=h, lm_head_weight=lm_head_weight)
        self._note(target=target, strict_entrypoint=path, runtime_platform="cuda" if h.is_cuda else "cpu-reference",
                   native_kernels=bool(h.is_cuda and h.dtype == torch.bfloat16), hidden_shape=list(h.shape),
                   hidden_dtype=str(h.dtype).removeprefix("torch."), lm_head_weight_shape=list(lm_head_weight.shape),
                   target_shape=list(shp), tp_group_present=tr.world > 1, tp_rank=tr.rank, tp_world_size=tr.world,
                   vocab_start_index=start, global_vocab_size=glob, real_vocab_size=real,
                   temperature=None if temperature is None else ("per_row" if len(pieces) > 1 else pieces[0][0]),
                   restricted_support=mk is not None, logits_materialized=bias is not None)
        lp = lp.view(shp)
        if mask is not None:
            lp = lp.masked_fill(~mask.bool(), 0.0)
        return (lp, lse.view(shp)) if return_lse else lp

    @staticmethod
    def _native_vp_ok(h: torch.Tensor, weight: torch.Tensor, padded: int) -> bool:
        return h.is_cuda and h.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and padded % (8 * TILE) == 0

    @staticmethod
    def _single_rank_piece(h, w, tg, temperature: float, min_keep, *, need_lse: bool):
        if need_lse:
            return _TPLinearLogpFn.apply(h.contiguous(), w.contiguous(), tg.contiguous(), (_Transport(None), 0, 1.0 / temperature, min_keep, None))
        from rl_kernel_b200.ops.logprob import linear_logp

        return linear_logp(h, w, tg, temperature, min_keep=min_keep), None

    @staticmethod
    def _logits_piece(tr: _Transport, logits, tg, start: int, temperature: float, min_keep, keep_mask):
        if tr.world == 1 and keep_mask is None and logits.requires_grad:
            from rl_kernel_b200.ops.logprob import logp_from_logits

            return logp_from_logits(logits, tg, temperature, min_keep=min_keep), None
        st, tz = _shard_stats_from_logits(logits.detach(), tg, vocab_start=start, inv_temp=1.0 / temperature, min_keep=min_keep,
                                          keep_mask=keep_mask)
        return _gathered_merge(tr, st, tz, None if tr.world == 1 else -(-(logits.shape[1] + 0) // TILE))

    # ---- logits a rollout engine already holds -> log-probs
    def from_local_logits(self, local_logits: torch.Tensor, target_ids: torch.Tensor, *, tp_group: Any = None,
                          vocab_start_index: int = 0, global_vocab_size: int | None = None, real_vocab_size: int | None = None,
                          target: str = "rollout", temperature: float | torch.Tensor | None = None, return_lse: bool = False,
                          min_keep: torch.Tensor | None = None, diagnostics_hidden: torch.Tensor | None = None,
                          diagnostics_lm_head_weight: torch.Tensor | None = None):
        """Score LM-head logits [T, V_local] without a second GEMM.  Columns at or beyond ``real_vocab_size`` (padding)
        take no part in the softmax."""
        if local_logits.ndim != 2 or local_logits.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            raise TypeError("strict reused LM-head logits must be 2-D bf16/fp16/fp32")
        if target_ids.device != local_logits.device:
            raise ValueError("linear_logp target_ids must share the logits device")
        tr, start, glob, real = self._geometry(local_logits.shape[1], tp_group=tp_group, vocab_start_index=vocab_start_index,
                                               global_vocab_size=global_vocab_size, real_vocab_size=real_vocab_size,
                                               what="reused rollout LM-head logits")
        tg = target_ids.reshape(-1)
        self._validate_targets(tg, rows=local_logits.shape[0], real_vocab_size=real)
        real_cols = max(0, min(local_logits.shape[1], real - start))
        lg = local_logits[:, :real_cols]
        rows_n = lg.shape[0]
        lp = torch.empty(rows_n, device=lg.device, dtype=torch.float32)
        lse = torch.empty(rows_n, device=lg.device, dtype=torch.float32)
        mk = None if min_keep is None else min_keep.reshape(-1)
        pieces = self._temperature_rows(self.temperature if temperature is None else temperature, rows_n)
        for t, rows in pieces:
            ll, tt = (lg, tg) if rows is None else (lg[rows], tg[rows])
            kk = mk if (mk is None or rows is None) else mk[rows]
            st, tz = _shard_stats_from_logits(ll, tt, vocab_start=start, inv_temp=1.0 / t, min_keep=kk)
            p_lp, p_lse = _gathered_merge(tr, st, tz, local_logits.shape[1] // TILE if tr.world > 1 else None)
            if rows is None:
                lp, lse = p_lp, p_lse
            else:
                lp, lse = lp.index_copy(0, rows, p_lp), lse.index_copy(0, rows, p_lse)
        _record_alignment_diagnostics(target=target, target_ids=tg, result=lp, lse=lse, vocab_start_index=start, local_logits=local_logits,
                                      hidden=diagnostics_hidden, lm_head_weight=diagnostics_lm_head_weight)
        self._note(target=target, strict_entrypoint="reused_local_logits", runtime_platform="cuda" if lg.is_cuda else "cpu-reference",
                   logits_shape=list(local_logits.shape), logits_dtype=str(local_logits.dtype).removeprefix("torch."),
                   tp_group_present=tr.world > 1, tp_rank=tr.rank, tp_world_size=tr.world, vocab_start_index=start,
                   global_vocab_size=glob, real_vocab_size=real, restricted_support=mk is not None, logits_materialized=True,
                   temperature="per_row" if len(pieces) > 1 else pieces[0][0])
        return (lp, lse) if return_lse else lp

    # ---- restricted support given as id lists
    def from_local_logits_sparse_nucleus(self, local_logits: torch.Tensor, target_ids: torch.Tensor, nucleus_ids: torch.Tensor, *,
                                         tp_group: Any = None, vocab_start_index: int = 0, global_vocab_size: int | None = None,
                                         real_vocab_size: int | None = None, temperature: float | torch.Tensor | None = None,
                                         target: str = "rollout", valid: torch.Tensor | None = None, return_entropy: bool = False):
        """Log-prob of ``target_ids`` under the softmax restricted to ``nucleus_ids`` [T, K] (global ids; entries with
        ``valid`` False, or negative ids, are padding).  Every target must be among its row's ids.  Bit-equal to scoring
        logits masked to -inf outside the ids."""
        if local_logits.ndim != 2 or nucleus_ids.ndim != 2:
            raise ValueError("sparse top-p replay expects [T,V_local] logits and [T,K] IDs")
        if nucleus_ids.shape[0] != local_logits.shape[0]:
            raise ValueError("sparse top-p nucleus rows must match local logits")
        if nucleus_ids.device != local_logits.device:
            raise ValueError("sparse top-p nucleus IDs must share the logits device")
        tr, start, glob, real = self._geometry(local_logits.shape[1], tp_group=tp_group, vocab_start_index=vocab_start_index,
                                               global_vocab_size=global_vocab_size, real_vocab_size=real_vocab_size,
                                               what="sparse top-p replay")
        tg = target_ids.reshape(-1).long()
        self._validate_targets(tg, rows=local_logits.shape[0], real_vocab_size=real)
        ids = nucleus_ids.long()
        ok = (ids >= 0) & (ids < real) if valid is None else (valid.bool() & (ids >= 0) & (ids < real))
        present = (ok & (ids == tg.reshape(-1, 1))).any(1).all()
        if present.is_cuda:
            torch._assert_async(present, "strict sparse top-p nucleus does not contain every target token")
        elif not bool(present):
            raise ValueError("strict sparse top-p nucleus does not contain every target token")
        # padding entries repeat the row's target: duplicates do not change a support
        ids = torch.where(ok, ids, tg.reshape(-1, 1).expand_as(ids))
        pieces = self._temperature_rows(self.temperature if temperature is None else temperature, local_logits.shape[0])
        lp = torch.empty(local_logits.shape[0], device=local_logits.device, dtype=torch.float32)
        lse = torch.empty_like(lp)
        compact = ids.shape[1] <= COMPACT_REPLAY_WIDTH and not (torch.is_grad_enabled() and local_logits.requires_grad)
        for t, rows in pieces:
            ll, tt, ii = (local_logits, tg, ids) if rows is None else (local_logits[rows], tg[rows], ids[rows])
            if compact and ll.dtype == torch.bfloat16:
                from rl_kernel_b200.ops.logprob import replay_logp_from_logits

                p_lp, p_lse = replay_logp_from_logits(ll, tt, ii, t, vocab_start=start, return_lse=True,
                                                      collective=tr if tr.world > 1 else None)
            else:
                loc = ii - start
                own = (loc >= 0) & (loc < ll.shape[1])
                keep = torch.zeros(ll.shape, dtype=torch.bool, device=ll.device)
                r = torch.arange(ll.shape[0], device=ll.device).reshape(-1, 1).expand_as(loc)
                keep[r[own], loc[own]] = True
                if tr.world == 1 and ll.requires_grad and torch.is_grad_enabled():
                    from rl_kernel_b200.ops.logprob import logp_from_logits

                    p_lp = logp_from_logits(ll.masked_fill(~keep, float("-inf")), tt, t)
                    p_lse = torch.zeros_like(p_lp)
                else:
                    st, tz = _shard_stats_from_logits(ll.detach(), tt, vocab_start=start, inv_temp=1.0 / t, min_keep=None, keep_mask=keep)
                    p_lp, p_lse = _gathered_merge(tr, st, tz, ll.shape[1] // TILE if tr.world > 1 else None)
            if rows is None:
                lp, lse = p_lp, p_lse
            else:
                lp, lse = lp.index_copy(0, rows, p_lp), lse.index_copy(0, rows, p_lse)
        self._note(target=target, strict_entrypoint="sparse_nucleus_compact" if compact else "sparse_nucleus_masked",
                   runtime_platform="cuda" if local_logits.is_cuda else "cpu-reference", support_width=int(ids.shape[1]),
                   tp_group_present=tr.world > 1, tp_rank=tr.rank, tp_world_size=tr.world, vocab_start_index=start,
                   global_vocab_size=glob, real_vocab_size=real, restricted_support=True, logits_materialized=True)
        if not return_entropy:
            return lp
        return lp, self._support_entropy(tr, local_logits, ids, start, lse, pieces)

    @staticmethod
    def _support_entropy(tr: _Transport, local_logits, ids, start: int, lse, pieces) -> torch.Tensor:
        """Entropy of the restricted distribution: -sum_i p_i log p_i over the distinct ids of a row, from the same
        log-sum-exp the log-probs used (a metric: fp32 PyTorch arithmetic, no gradient)."""
        with torch.no_grad():
            inv = torch.ones(local_logits.shape[0], device=local_logits.device)
            for t, rows in pieces:
                if rows is None:
                    inv = inv / t
                else:
                    inv[rows] = 1.0 / t
            srt, _ = ids.sort(1)
            first = torch.ones_like(srt, dtype=torch.bool)
            first[:, 1:] = srt[:, 1:] != srt[:, :-1]                        # one term per distinct id
            loc = srt - start
            own = first & (loc >= 0) & (loc < local_logits.shape[1])
            z = local_logits.float().gather(1, loc.clamp(0, local_logits.shape[1] - 1)) * inv.reshape(-1, 1)
            logp = z - lse.reshape(-1, 1)
            term = torch.where(own, -torch.exp(logp) * logp, torch.zeros_like(logp)).sum(1)
            return tr.all_gather(term).sum(0) if tr.world > 1 else term

    def from_local_logits_top_p(self, local_logits: torch.Tensor, target_ids: torch.Tensor, replay_ids: torch.Tensor,
                                replay_logprobs: torch.Tensor, *, tp_group: Any = None, vocab_start_index: int = 0,
                                global_vocab_size: int | None = None, real_vocab_size: int | None = None, target: str = "rollout",
                                temperature: float | torch.Tensor | None = None) -> torch.Tensor:
        """The sampler's transport format: ``replay_ids`` [T, K] with ``replay_logprobs`` [T, K] finite exactly for the
        ids top-p retained.  Scores the targets over that support."""
        if replay_ids.shape != replay_logprobs.shape or replay_ids.shape[0] != local_logits.shape[0]:
            raise ValueError("top-p support must match the local-logit rows")
        return self.from_local_logits_sparse_nucleus(local_logits, target_ids, replay_ids, tp_group=tp_group,
                                                     vocab_start_index=vocab_start_index, global_vocab_size=global_vocab_size,
                                                     real_vocab_size=real_vocab_size, temperature=temperature, target=target,
                                                     valid=torch.isfinite(replay_logprobs))

    def from_replicated_logits_sparse_nucleus(self, logits: torch.Tensor, target_ids: torch.Tensor, nucleus_ids: torch.Tensor, *,
                                              real_vocab_size: int, temperature: float | torch.Tensor | None = None,
                                              return_entropy: bool = False, tp_group: Any = None):
        """Inference-only: the engine has already gathered the whole real vocabulary on every rank, so each rank scores
        alone (``tp_group`` is accepted for interface parity; nothing is exchanged)."""
        if torch.is_grad_enabled() and logits.requires_grad:
            raise RuntimeError("replicated sparse scoring is inference-only")
        if logits.ndim != 2 or logits.shape[1] != int(real_vocab_size):
            raise ValueError("replicated sparse scoring requires the complete real vocabulary")
        if nucleus_ids.ndim != 2 or nucleus_ids.shape[0] != logits.shape[0]:
            raise ValueError("replicated support rows must match logits")
        return LinearLogpWrapper(self.temperature).from_local_logits_sparse_nucleus(
            logits, target_ids, nucleus_ids, tp_group=None, vocab_start_index=0, global_vocab_size=int(real_vocab_size),
            real_vocab_size=int(real_vocab_size), temperature=temperature, target="rollout", return_entropy=return_entropy)


__all__ = ["COMPACT_REPLAY_WIDTH", "CONTRACT_VERSION", "LinearLogpWrapper", "RolloutLinearLogpContext", "alignment_tensor_summary",
           "clear_rollout_linear_logp_context", "publish_rollout_linear_logp_context", "take_rollout_linear_logp_context"]
