"""Context-parallel attention drift by schedule (parity: benchmarks/distributed/benchmark_ws2_cp_attention_drift.py of the
reference): for CP degrees 2 / 4 / 8 and both layouts, the strict schedule (every rank walks the logical K/V in ascending
128-key blocks) against the ring schedules that merge per-arrival partial states, measured on the block-wise reference.
The strict rows must read exactly zero; the ring rows show what a merge-based schedule costs in bits.

    python -m rl_kernel_b200.benchmarks.cp_attention_drift --seq-len 512 --head-dim 64
"""
from __future__ import annotations

import argparse
import json

import torch

from rl_kernel_b200.reference.attention.cp_attention import DeterministicCPAttentionReferenceOp


def run(seq_len: int, q_heads: int, kv_heads: int, head_dim: int, degrees=(2, 4, 8), dtype=torch.bfloat16) -> list[dict]:
    g = torch.Generator().manual_seed(0)
    q = torch.randn(seq_len, q_heads, head_dim, generator=g).to(dtype)
    k = torch.randn(seq_len, kv_heads, head_dim, generator=g).to(dtype)
    v = torch.randn(seq_len, kv_heads, head_dim, generator=g).to(dtype)
    one_o, one_l = DeterministicCPAttentionReferenceOp(1, p_dtype=dtype)(q, k, v)
    rows = []
    for cp in degrees:
        for layout in ("zigzag", "contiguous"):
            if seq_len % (2 * cp if layout == "zigzag" else cp):
                continue
            for name, kw in (("strict", {}), ("ring_global_order", {"strict_bitwise": False}),
                             ("ring_arrival_order", {"strict_bitwise": False, "merge_order": "arrival"})):
                o, l = DeterministicCPAttentionReferenceOp(cp, layout, p_dtype=dtype, **kw)(q, k, v)
                rows.append({"cp": cp, "layout": layout, "schedule": name, "out_max_abs": float((o.float() - one_o.float()).abs().max()),
                             "lse_max_abs": float((l - one_l).abs().max()),
                             "out_bitwise_mismatches": int((o.view(torch.int16) != one_o.view(torch.int16)).sum()) if dtype == torch.bfloat16
                             else int((o != one_o).sum())})
    return rows


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--q-heads", type=int, default=4)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=64)
    a = ap.parse_args(argv)
    rows = run(a.seq_len, a.q_heads, a.kv_heads, a.head_dim)
    print(json.dumps({"bench": "cp_attention_drift", "rows": rows, "strict_all_zero": all(r["out_bitwise_mismatches"] == 0 for r in rows
                                                                                       if r["schedule"] == "strict")}))


if __name__ == "__main__":
    main()
