"""Weight-sync bridge: publish -> import -> release latency and bandwidth per transport, with and without checksums
(parity: benchmarks/e2e/benchmark_weight_sync_bridge.py of the reference).

    python -m rl_kernel_b200.benchmarks.weight_sync_bridge --transport local-clone --mb 512 --device cuda

Transports that stay inside one process (local-clone, shared-memory) run anywhere; cuda-ipc / cuda-vmm need a CUDA device.
The NVLink push between a trainer GPU and a rollout GPU is timed by ``benchmarks.collectives`` (two ranks)."""
from __future__ import annotations

import argparse
import json
import time

import torch

from rl_kernel_b200.integrations.common.weights import make_weight_bridge


def synthetic_state(total_mb: int, device: str, tensors: int = 16) -> dict[str, torch.Tensor]:
    n = total_mb * (1 << 20) // 2 // tensors
    g = torch.Generator().manual_seed(0)
    return {f"layers.{i}.weight": torch.randn(n, generator=g).bfloat16().to(device) for i in range(tensors)}


def run(transport: str, total_mb: int, device: str, iters: int) -> dict:
    state = synthetic_state(total_mb, device)
    bridge = make_weight_bridge(transport)
    sync = (lambda: torch.cuda.synchronize()) if device.startswith("cuda") else (lambda: None)
    pub, imp = [], []
    for v in range(1, iters + 2):
        sync()
        t0 = time.perf_counter()
        m = bridge.publish(state, weight_version=v)
        sync()
        t1 = time.perf_counter()
        got = bridge.import_update(m)
        sync()
        t2 = time.perf_counter()
        if v == 1:
            ok = all(torch.equal(got[k].to(state[k].device), state[k]) for k in state)
        else:
            pub.append(t1 - t0)
            imp.append(t2 - t1)
        bridge.release(m.update_id)
    nbytes = sum(t.numel() * t.element_size() for t in state.values())
    med = lambda xs: sorted(xs)[len(xs) // 2]  # noqa: E731
    return {"bench": "weight_sync_bridge", "transport": transport, "device": device, "mb": nbytes / 2 ** 20, "tensors": len(state),
            "publish_ms": med(pub) * 1e3, "import_ms": med(imp) * 1e3, "publish_gb_s": nbytes / med(pub) / 1e9,
            "round_trip_ok": bool(ok)}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--transport", default="local-clone")
    ap.add_argument("--mb", type=int, default=256)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args(argv)
    print(json.dumps(run(a.transport, a.mb, a.device, a.iters)))


if __name__ == "__main__":
    main()
