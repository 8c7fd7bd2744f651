"""Deterministic causal GQA attention (head_dim 128) with native forward and backward.

``causal_attention`` takes packed sequences (cu_seqlens) — padded batches are packed first — and
``decode_attention`` runs one query token per sequence against a KV cache; both go through the same
kernel and the same per-row program (csrc/attention/attn_fwd_sm100.cu), which is what makes rollout
and training log-probs bit-equal.  Parity: StrictFlashAttention4Core / StrictCUDAAttentionRuntime
(rl_engine/backends/cuda/attention/flash_attn.py:65, strict_runtime.py:40).
"""
from __future__ import annotations

import math

import torch

from rl_kernel_b200.ops._dispatch import use_native
from rl_kernel_b200.reference.attention.blockwise import blockwise_attention_reference


def varlen_tiles(cu_seqlens: list[int], hq: int, hkv: int, d: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """Forward/dQ tiles and dK/dV tiles for packed sequences with boundaries ``cu_seqlens``."""
    g = hq // hkv
    fw, kv = [], []
    for b in range(len(cu_seqlens) - 1):
        s0, S = cu_seqlens[b], cu_seqlens[b + 1] - cu_seqlens[b]
        nqt = (S + 127) // 128
        for qt in range(nqt - 1, -1, -1):
            for h in range(hq):
                row0 = s0 + qt * 128
                fw.append([row0, h * d, min(128, S - qt * 128), s0, (h // g) * d, qt * 128, 1, S, row0 * hq + h, hq, 0, 0])
        for kb in range(nqt):
            for hk in range(hkv):
                kv.append([s0 + kb * 128, hk * d, kb * 128, min(128, S - kb * 128), s0, 0, S, hk * g * d, g,
                           s0 * hq + hk * g, hq, 1])
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=device).reshape(-1, 12).contiguous()  # noqa: E731
    return mk(fw), mk(kv)


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, tiles, kvtiles, hq, hkv, scale):
        from rl_kernel_b200.backends import native as nv

        T = q.shape[0]
        o = torch.empty_like(q)
        lse = torch.empty(T, hq, device=q.device, dtype=torch.float32)
        nv.attn_fwd(q, [k], [v], o, lse, tiles, scale)
        ctx.save_for_backward(q, k, v, o, lse, tiles, kvtiles)
        ctx.meta = (hq, hkv, scale)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        from rl_kernel_b200.backends import native as nv

        q, k, v, o, lse, tiles, kvtiles = ctx.saved_tensors
        hq, hkv, scale = ctx.meta
        T = q.shape[0]
        do = do.contiguous()
        delta = torch.empty(T, hq, device=q.device, dtype=torch.float32)
        dq, dk, dv = torch.empty_like(q), torch.zeros_like(k), torch.zeros_like(v)
        nv.attn_bwd_delta(o, do, delta, T, hq)
        nv.attn_bwd_dq(q, do, k, v, lse, delta, dq, tiles, scale)
        nv.attn_bwd_dkv(q, do, k, v, lse, delta, dk, dv, kvtiles, scale)
        return dq, dk, dv, None, None, None, None, None


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens, *, scale: float | None = None,
                     return_lse: bool = False):
    """q [T, Hq, D], k/v [T, Hkv, D] packed; ``cu_seqlens`` list/tensor of boundaries. Differentiable."""
    T, hq, d = q.shape
    hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    cu = [int(x) for x in (cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)]
    if not use_native(q, k, v):
        outs, lses = [], []
        for b in range(len(cu) - 1):
            sl = slice(cu[b], cu[b + 1])
            o, l = blockwise_attention_reference(q[sl], k[sl], v[sl], torch.arange(cu[b + 1] - cu[b]), scale=scale,
                                                 strict=False)
            outs.append(o)
            lses.append(l)
        o, l = torch.cat(outs), torch.cat(lses)
        return (o, l) if return_lse else o
    if d != 128:
        raise ValueError("the sm_100a attention kernels need head_dim 128")
    tiles, kvtiles = varlen_tiles(cu, hq, hkv, d, q.device)
    o, lse = _AttnFn.apply(q.reshape(T, hq * d).contiguous(), k.reshape(T, hkv * d).contiguous(),
                           v.reshape(T, hkv * d).contiguous(), tiles, kvtiles, hq, hkv, scale)
    o = o.view(T, hq, d)
    return (o, lse) if return_lse else o


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor, *,
                     scale: float | None = None) -> torch.Tensor:
    """q [B, Hq, D] (one token per sequence at ``positions`` [B]); k_cache/v_cache [B, S_max, Hkv, D]
    already containing the token's own K/V.  Returns [B, Hq, D]; no gradient."""
    B, hq, d = q.shape
    smax, hkv = k_cache.shape[1], k_cache.shape[2]
    g = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if not use_native(q, k_cache, v_cache):
        outs = []
        for b in range(B):
            n = int(positions[b]) + 1
            o, _ = blockwise_attention_reference(q[b:b + 1], k_cache[b, :n], v_cache[b, :n], positions[b:b + 1].cpu(),
                                                 scale=scale, strict=False)
            outs.append(o[0])
        return torch.stack(outs)
    from rl_kernel_b200.backends import native as nv

    dev = q.device
    b_idx = torch.arange(B, device=dev).view(-1, 1)
    hk = torch.arange(hkv, device=dev).view(1, -1)
    z = torch.zeros(B, hkv, dtype=torch.long, device=dev)
    row0 = b_idx * hq + hk * g + z
    pos = positions.to(dev).long().view(-1, 1) + z
    tiles = torch.stack([row0, z, z + g, b_idx * smax + z, hk * d + z, pos, z, pos + 1, row0, z + 1, z, z],
                        dim=-1).reshape(-1, 12).to(torch.int32).contiguous()
    q2 = torch.zeros(B * hq + 128, d, device=dev, dtype=q.dtype)
    q2[: B * hq] = q.reshape(B * hq, d)
    o2 = torch.empty_like(q2)
    nv.attn_fwd(q2, [k_cache.reshape(B * smax, hkv * d)], [v_cache.reshape(B * smax, hkv * d)], o2, None, tiles, scale,
                decode=g <= 8)
    return o2[: B * hq].view(B, hq, d)


class AttentionOp:
    """Registry object ``attention`` (padded [B, S, H, D] interface of the reference ops)."""
    backend_id = "b200-tcgen05"
    backward_impl = "native"
    schedule = "canonical_128_key_blocks_no_splitkv"

    def __call__(self, q, k, v, *, causal: bool = True, key_padding_mask=None, scale=None, return_lse: bool = False):
        if not causal:
            raise NotImplementedError("the deterministic kernels implement causal attention")
        B, S = q.shape[:2]
        if key_padding_mask is not None:
            lens = key_padding_mask.bool().sum(1).tolist()
            if any(not bool(key_padding_mask[b, : lens[b]].all()) for b in range(B)):
                raise ValueError("only right padding is supported; pack the batch for other layouts")
        else:
            lens = [S] * B
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        pack = lambda t: torch.cat([t[b, : lens[b]] for b in range(B)])  # noqa: E731
        o, lse = causal_attention(pack(q), pack(k), pack(v), cu, scale=scale, return_lse=True)
        out = q.new_zeros(q.shape)
        lse_out = torch.full((B, S, q.shape[2]), float("-inf"), device=q.device)
        for b in range(B):
            out[b, : lens[b]] = o[cu[b]:cu[b + 1]]
            lse_out[b, : lens[b]] = lse[cu[b]:cu[b + 1]]
        return (out, lse_out) if return_lse else out

    forward = __call__
