"""Operator profiler: CUDA-event timing with warm-up and L2 flush, peak memory, tokens/s and TFLOP/s
estimates, JSON / CSV output and a ``status`` of pass | blocked | oom per workload (parity:
PerformanceProfiler and WORKLOAD_REGISTRY, benchmarks/common/profiler.py:156-480 in the reference;
suite CLI: ``python -m rl_kernel_b200.benchmarks.run_profile_suite``).  Roofline fractions are taken
against the measured copy bandwidth and bf16 GEMM throughput of the box when a ``peaks`` mapping
({"hbm_gbs": ..., "bf16_tflops": ...}) is supplied.
"""
from __future__ import annotations

import csv
import json
import math
from dataclasses import asdict, dataclass, field
from typing import Callable

import torch


@dataclass
class ProfileResult:
    name: str
    status: str = "pass"                 # pass | blocked | oom
    reason: str = ""
    ms: float = float("nan")
    ms_min: float = float("nan")
    iters: int = 0
    peak_mem_mb: float = float("nan")
    tokens_per_s: float = float("nan")
    tflops: float = float("nan")
    gbs: float = float("nan")
    frac_of_bf16_peak: float = float("nan")
    frac_of_hbm_peak: float = float("nan")
    shape: dict = field(default_factory=dict)


@dataclass
class Workload:
    """``build(device) -> (fn, meta)``; meta may carry ``flops``, ``bytes``, ``tokens`` per call."""
    name: str
    build: Callable
    shape: dict = field(default_factory=dict)


WORKLOAD_REGISTRY: dict[str, Workload] = {}


def register_workload(name: str, shape: dict | None = None):
    def deco(fn):
        WORKLOAD_REGISTRY[name] = Workload(name, fn, shape or {})
        return fn
    return deco


class PerformanceProfiler:
    def __init__(self, device: torch.device | None = None, *, warmup: int = 3, iters: int = 10,
                 flush_l2: bool = True, peaks: dict | None = None):
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.warmup, self.iters, self.flush_l2, self.peaks = max(3, warmup), iters, flush_l2, peaks or {}
        self.results: list[ProfileResult] = []
        self._flush = None

    def _time(self, fn) -> tuple[float, float]:
        if self.flush_l2 and self._flush is None:
            self._flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.device)
        for _ in range(self.warmup):
            fn()
        ts = []
        for _ in range(self.iters):
            if self.flush_l2:
                self._flush.zero_()
            torch.cuda.synchronize(self.device)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize(self.device)
            ts.append(s.elapsed_time(e))
        ts.sort()
        return ts[len(ts) // 2], ts[0]

    def run(self, workload: Workload | str) -> ProfileResult:
        w = WORKLOAD_REGISTRY[workload] if isinstance(workload, str) else workload
        res = ProfileResult(w.name, shape=dict(w.shape))
        if not torch.cuda.is_available():
            res.status, res.reason = "blocked", "no CUDA device"
            self.results.append(res)
            return res
        try:
            torch.cuda.reset_peak_memory_stats(self.device)
            fn, meta = w.build(self.device)
            res.ms, res.ms_min = self._time(fn)
            res.iters = self.iters
            res.peak_mem_mb = torch.cuda.max_memory_allocated(self.device) / 2 ** 20
            if meta.get("tokens"):
                res.tokens_per_s = meta["tokens"] / res.ms * 1e3
            if meta.get("flops"):
                res.tflops = meta["flops"] / res.ms / 1e9
                if self.peaks.get("bf16_tflops"):
                    res.frac_of_bf16_peak = res.tflops / self.peaks["bf16_tflops"]
            if meta.get("bytes"):
                res.gbs = meta["bytes"] / res.ms / 1e6
                if self.peaks.get("hbm_gbs"):
                    res.frac_of_hbm_peak = res.gbs / self.peaks["hbm_gbs"]
        except torch.cuda.OutOfMemoryError as exc:
            res.status, res.reason = "oom", str(exc).splitlines()[0]
            torch.cuda.empty_cache()
        except (NotImplementedError, ValueError, ImportError) as exc:
            res.status, res.reason = "blocked", f"{type(exc).__name__}: {exc}"
        self.results.append(res)
        return res

    def to_json(self, path: str | None = None) -> str:
        def clean(v):
            return None if isinstance(v, float) and math.isnan(v) else v
        text = json.dumps([{k: clean(v) for k, v in asdict(r).items()} for r in self.results], indent=1)
        if path:
            with open(path, "w") as f:
                f.write(text)
        return text

    def to_csv(self, path: str) -> None:
        rows = [asdict(r) for r in self.results]
        with open(path, "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=list(rows[0].keys()) if rows else ["name"])
            wr.writeheader()
            for r in rows:
                r["shape"] = json.dumps(r["shape"])
                wr.writerow(r)


# ------------------------------------------------------------------------------------ workloads
def _bf16(dev, *shape, std=1.0):
    return (torch.randn(*shape, device=dev) * std).to(torch.bfloat16)


@register_workload("det_gemm_4096x12288x4096", {"M": 4096, "N": 12288, "K": 4096})
def _wl_gemm(dev):
    from rl_kernel_b200.backends import native as nv

    M, N, K = 4096, 12288, 4096
    a, b, c = _bf16(dev, M, K), _bf16(dev, N, K, std=0.02), torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    return (lambda: nv.det_gemm(a, b, c, M=M, N=N, K=K)), {"flops": 2.0 * M * N * K, "tokens": M}


@register_workload("attention_fwd_8x1536", {"batch": 8, "seq": 1536, "hq": 32, "hkv": 8})
def _wl_attn(dev):
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.models.qwen3.engine import train_tiles

    B, S, hq, hkv, d = 8, 1536, 32, 8, 128
    q, k, v = _bf16(dev, B * S, hq * d), _bf16(dev, B * S, hkv * d), _bf16(dev, B * S, hkv * d)
    o, lse = torch.empty_like(q), torch.empty(B * S, hq, device=dev)
    tiles, _ = train_tiles(B, S, hq, hkv, d, dev)
    return (lambda: nv.attn_fwd(q, [k], [v], o, lse, tiles, d ** -0.5)), {"flops": 4.0 * B * hq * d * S * S / 2, "tokens": B * S}


@register_workload("rmsnorm_fwd_12288x4096", {"rows": 12288, "H": 4096})
def _wl_rms(dev):
    from rl_kernel_b200.backends import native as nv

    x, w = _bf16(dev, 12288, 4096), _bf16(dev, 4096)
    y = torch.empty_like(x)
    return (lambda: nv.rmsnorm_fwd(x, w, y, 1e-6)), {"bytes": 2.0 * x.numel() * 2, "tokens": 12288}


@register_workload("linear_logp_fwd_4096x151936", {"rows": 4096, "H": 4096, "V": 151936})
def _wl_linear_logp(dev):
    from rl_kernel_b200.ops.logprob import linear_logp

    h, w = _bf16(dev, 4096, 4096), _bf16(dev, 151936, 4096, std=0.02)
    t = torch.randint(0, 151936, (4096,), device=dev)
    return (lambda: linear_logp(h, w, t)), {"flops": 2.0 * 4096 * 151936 * 4096, "tokens": 4096}


@register_workload("logp_from_logits_4096x151936", {"rows": 4096, "V": 151936})
def _wl_logp(dev):
    from rl_kernel_b200.ops.logprob import logp_from_logits

    lg = _bf16(dev, 4096, 151936)
    t = torch.randint(0, 151936, (4096,), device=dev)
    return (lambda: logp_from_logits(lg, t)), {"bytes": 2.0 * lg.numel(), "tokens": 4096}


@register_workload("qwen3_ffn_fwd_8192", {"tokens": 8192, "H": 4096, "I": 12288})
def _wl_ffn(dev):
    from rl_kernel_b200.backends import native as nv

    T, H, I = 8192, 4096, 12288
    x, wgu, wd = _bf16(dev, T, H), _bf16(dev, 2 * I, H, std=0.02), _bf16(dev, H, I, std=0.02)
    gu, act, out = (torch.empty(T, n, device=dev, dtype=torch.bfloat16) for n in (2 * I, I, H))

    def fn():
        nv.det_gemm(x, wgu, gu, M=T, N=2 * I, K=H)
        nv.swiglu_fwd(gu, act, I, I // 8)
        nv.det_gemm(act, wd, out, M=T, N=H, K=I, nchunks=8)
    return fn, {"flops": 6.0 * T * H * I, "tokens": T}
