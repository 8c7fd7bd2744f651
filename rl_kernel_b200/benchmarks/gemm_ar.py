"""Row-parallel projection (o_proj, FFN down): fused GEMM + fixed-tree all-reduce in ONE kernel
against (a) det_gemm followed by this library's all-reduce kernel and (b) det_gemm followed by an
NCCL all-reduce, per tensor-parallel rank.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29545 -m rl_kernel_b200.benchmarks.gemm_ar --rows 12288 --out-features 4096 --in-features 12288

``--in-features`` is the full contraction width K; each rank multiplies its K / W slice (8 / W canonical
chunks).  CUDA events, max over ranks, L2 flushed between iterations.  Roofline per rank:
max(2 M N K_loc / measured bf16 peak, (W-1)/W * M * N * 2 bytes * 2 / 770 GB/s) -- an all-reduce moves
every element once in (reduce-scatter) and once out (all-gather) over each GPU's links.  The fused
kernel and (a) give the same bits (checked); NCCL's sum has no fixed order and is only timed.
The ``rs_*`` keys time the sequence-parallel exit (each rank keeps its M / W token rows): the fused GEMM + reduce-scatter
kernel against det_gemm + this library's reduce-scatter and det_gemm + NCCL ``reduce_scatter_tensor``.
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
    ap.add_argument("--out-features", dest="n", type=int, default=4096)
    ap.add_argument("--in-features", dest="k", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective

    world, rank, local = (int(os.environ[k]) for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    M, N, Kl = a.m, a.n, a.k // world
    nchunks = max(1, 8 // world)
    coll = SymmetricMemoryCollective(None, dev, frame_bytes=max(256 << 20, 2 * M * N))
    g = torch.Generator(device=dev).manual_seed(rank)
    x = torch.randn(M, Kl, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, Kl, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    out_f, part = (torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(2))
    out_o, out_n = torch.empty_like(part), torch.empty_like(part)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def fused():
        coll.gemm_all_reduce(x, w, out_f, nchunks)

    def own():
        nv.det_gemm(x, w, out_o, M=M, N=N, K=Kl, nchunks=nchunks, tile_n=128)
        coll.all_reduce_(out_o)

    def nccl():
        nv.det_gemm(x, w, out_n, M=M, N=N, K=Kl, nchunks=nchunks, tile_n=128)
        dist.all_reduce(out_n)

    def gemm_only():
        nv.det_gemm(x, w, part, M=M, N=N, K=Kl, nchunks=nchunks, tile_n=128)

    # sequence-parallel exit: every rank keeps its M / W token rows of the sum
    rs_ok = M % (128 * world) == 0
    out_rs = torch.empty(M // world if rs_ok else 1, N, device=dev, dtype=torch.bfloat16)
    out_rs_n = torch.empty_like(out_rs)

    def fused_rs():
        coll.gemm_reduce_scatter(x, w, out_rs, nchunks)

    def own_rs():
        nv.det_gemm(x, w, out_o, M=M, N=N, K=Kl, nchunks=nchunks, tile_n=128)
        return coll.reduce_scatter(out_o)

    def nccl_rs():
        nv.det_gemm(x, w, out_n, M=M, N=N, K=Kl, nchunks=nchunks, tile_n=128)
        dist.reduce_scatter_tensor(out_rs_n, out_n)

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

    t_f, t_o, t_n, t_g = timed(fused), timed(own), timed(nccl), timed(gemm_only)
    same = torch.tensor([int(torch.equal(out_f, out_o))], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    rs = {}
    if rs_ok:
        t_rf, t_ro, t_rn = timed(fused_rs), timed(own_rs), timed(nccl_rs)
        rows = slice(rank * M // world, (rank + 1) * M // world)
        same_rs = torch.tensor([int(torch.equal(out_rs, out_f[rows]))], device=dev)
        dist.all_reduce(same_rs, op=dist.ReduceOp.MIN)
        # a reduce-scatter moves every element once over each GPU's links (in), not twice
        floor_rs = max(2.0 * M * N * Kl / 1655.3 / 1e9, (world - 1) / world * M * N * 2 / 770.0 / 1e6)
        rs = {"rs_fused_ms": t_rf, "rs_gemm_plus_own_reduce_scatter_ms": t_ro, "rs_gemm_plus_nccl_reduce_scatter_ms": t_rn,
              "rs_speedup_vs_nccl": t_rn / t_rf, "rs_roofline_ms": floor_rs, "rs_fraction_of_roofline": floor_rs / t_rf,
              "rs_bitwise_equal_to_all_reduce_rows": bool(same_rs.item())}
    status = ext.poll_status(dev)
    if rank == 0:
        peak, link = 1655.3, 770.0
        floor = max(2.0 * M * N * Kl / peak / 1e9, (world - 1) / world * M * N * 2 * 2 / link / 1e6)
        print(json.dumps({"bench": "gemm_ar", "world": world, "M": M, "N": N, "K_local": Kl, "nchunks_local": nchunks,
                          "fused_ms": t_f, "gemm_plus_own_all_reduce_ms": t_o, "gemm_plus_nccl_all_reduce_ms": t_n,
                          "gemm_alone_ms": t_g, "speedup_vs_nccl": t_n / t_f, "roofline_ms": floor,
                          "fraction_of_roofline": floor / t_f, "bitwise_equal_to_unfused": bool(same.item()),
                          "device_status": status, **rs}))
    coll.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
