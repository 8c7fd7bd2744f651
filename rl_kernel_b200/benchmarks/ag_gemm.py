"""Fused all-gather + GEMM against NCCL all-gather followed by det_gemm, per tensor-parallel rank.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29544 -m rl_kernel_b200.benchmarks.ag_gemm --rows 12288 --out-features 6144 --in-features 4096

``--out-features`` is the full output width; each rank multiplies its N / W columns.  CUDA events, max over
ranks, L2 flushed between iterations.  Roofline: max(2 M N_loc K / measured bf16 peak,
(W-1)/W * M * K * 2 bytes / 770 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", dest="m", type=int, default=12288)
    ap.add_argument("--out-features", dest="n", type=int, default=6144)
    ap.add_argument("--in-features", dest="k", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.distributed.ag_gemm import AllGatherGemm
    from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective

    world, rank, local = (int(os.environ[k]) for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    coll = SymmetricMemoryCollective(None, dev, frame_bytes=1 << 20)
    M, K, Nl = a.m, a.k, a.n // world
    ag = AllGatherGemm(coll, dev, M, K)
    g = torch.Generator(device=dev).manual_seed(rank)
    shard = torch.randn(M // world, K, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(Nl, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    out, ref = torch.empty(M, Nl, device=dev, dtype=torch.bfloat16), torch.empty(M, Nl, device=dev, dtype=torch.bfloat16)
    full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def fused():
        ag.local_shard.copy_(shard)
        ag(w, out)

    def baseline():
        dist.all_gather_into_tensor(full, shard)
        nv.det_gemm(full, w, ref, M=M, N=Nl, K=K)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(); fn(); e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    t_f, t_b = timed(fused), timed(baseline)
    same = bool(torch.equal(out, ref))
    status = ext.poll_status(dev)
    if rank == 0:
        peaks = {"bf16_tflops": 1655.3, "nvlink_gbs": 770.0}
        floor = max(2.0 * M * Nl * K / peaks["bf16_tflops"] / 1e9, (world - 1) / world * M * K * 2 / peaks["nvlink_gbs"] / 1e6)
        print(json.dumps({"bench": "ag_gemm", "world": world, "M": M, "N_local": Nl, "K": K, "fused_ms": t_f,
                          "nccl_ag_plus_gemm_ms": t_b, "speedup": t_b / t_f, "roofline_ms": floor,
                          "fraction_of_roofline": floor / t_f, "bitwise_equal_to_gathered_gemm": same,
                          "device_status": status}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
