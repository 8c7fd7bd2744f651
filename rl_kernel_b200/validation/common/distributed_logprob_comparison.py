"""Distributed comparison of the vocabulary-parallel log-prob reference (parity: rl_engine/validation/
common/distributed_logprob_comparison.py:61-840; also a torchrun entry point).

A case fixes a (TP, CP) topology, a vocabulary (real and padded size, tile count) and a token batch.
Rank r = cp_rank * TP + tp_rank holds the token rows of its CP shard and the vocabulary columns of
its TP shard of one canonical fp32 logits tensor (drawn from the seed on every rank, then sliced,
then rounded to the case dtype).  Every rank runs the contract-driven operator over its TP group,
compares its rows with an fp32 oracle over the real vocabulary and checks that the TP group's
outputs are replicated bit for bit; rank 0 gathers the payloads, adds the aggregate drift, the
worst token with its owner rank, and sha256 fingerprints of the assembled outputs (equal between
two topologies when the operator is topology-invariant) and writes one strict-JSON report.
"""
from __future__ import annotations

import argparse
import datetime
import hashlib
import json
import os
import shlex
import sys
from dataclasses import asdict, dataclass
from typing import Any, Sequence

import torch

from rl_kernel_b200.contracts.numerical import resolve_tolerance
from rl_kernel_b200.contracts.operators.logprob import (LogprobContract, LogprobDType, LogprobRole, MaskSpec, ReductionSpec,
                                                        ShardingSpec)
from rl_kernel_b200.reference.logprob.vocab_parallel_logp import BACKEND_ID, VocabParallelLogprobOp
from rl_kernel_b200.validation.common.logprob_drift import LogprobDriftStats, summarize_logprob_drift

_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
_TOL_KEYS = {"bf16": "bfloat16", "fp16": "float16", "fp32": "float32"}
_GROUP_TIMEOUT = datetime.timedelta(minutes=5)
SCHEMA_VERSION = 1


@dataclass(frozen=True)
class DistributedLogprobCase:
    tp_world_size: int
    cp_world_size: int
    dtype: str = "bf16"
    requested_backend: str = BACKEND_ID
    real_vocab_size: int = 151936
    padded_vocab_size: int = 151936
    num_vocab_tiles: int = 1187                      # 151936 / 128
    batch_size: int = 2
    sequence_length: int = 16
    prompt_tokens: int = 8
    seed: int = 123
    ignore_index: int = -100

    def __post_init__(self) -> None:
        for name in ("tp_world_size", "cp_world_size", "real_vocab_size", "padded_vocab_size", "num_vocab_tiles", "batch_size",
                     "sequence_length"):
            v = getattr(self, name)
            if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
                raise ValueError(f"{name} must be a positive integer")
        if self.dtype not in _DTYPES:
            raise ValueError(f"dtype must be one of {sorted(_DTYPES)}")
        if not self.requested_backend or self.requested_backend.lower() == "auto":
            raise ValueError("distributed cases require an explicit non-auto backend")
        if self.padded_vocab_size < self.real_vocab_size:
            raise ValueError("padded_vocab_size must be at least real_vocab_size")
        if self.num_vocab_tiles < self.tp_world_size:
            raise ValueError("num_vocab_tiles must be at least tp_world_size")
        if self.padded_vocab_size % self.num_vocab_tiles:
            raise ValueError("num_vocab_tiles must divide padded_vocab_size exactly")
        if not 0 <= self.prompt_tokens <= self.sequence_length:
            raise ValueError("prompt_tokens must be in [0, sequence_length]")
        if self.num_tokens < self.cp_world_size:
            raise ValueError("the batch must hold at least one token per CP rank")

    @property
    def world_size(self) -> int:
        return self.tp_world_size * self.cp_world_size

    @property
    def num_tokens(self) -> int:
        return self.batch_size * self.sequence_length

    @property
    def case_id(self) -> str:
        return hashlib.sha256(json.dumps(asdict(self), sort_keys=True, separators=(",", ":")).encode()).hexdigest()[:16]


@dataclass(frozen=True)
class RankTopology:
    global_rank: int
    world_size: int
    tp_rank: int
    tp_world_size: int
    cp_rank: int
    cp_world_size: int
    tp_group_ranks: tuple[int, ...]


@dataclass(frozen=True)
class DriftDetail:
    stats: LogprobDriftStats
    max_rel: float
    worst_global_token: int | None
    worst_target_id: int | None
    worst_owner_rank: int | None
    candidate_value: float | None
    reference_value: float | None
    atol: float
    rtol: float
    passed: bool


@dataclass(frozen=True)
class RankLogprobReport:
    global_rank: int
    tp_rank: int
    tp_world_size: int
    cp_rank: int
    cp_world_size: int
    sp_world_size: int
    dp_world_size: int
    token_start: int
    token_end: int
    vocab_start: int
    vocab_end: int
    device: str
    requested_backend: str
    actual_backend: str
    fallback: bool
    contract_fingerprint: str
    contract: dict[str, Any]
    capability: dict[str, Any]
    tp_outputs_bitwise_replicated: bool
    lse: DriftDetail
    dlogp: DriftDetail
    passed: bool


@dataclass(frozen=True)
class DistributedLogprobReport:
    schema_version: int
    case_id: str
    case: dict[str, Any]
    launch_command: str
    environment: dict[str, Any]
    ranks: tuple[RankLogprobReport, ...]
    aggregate: dict[str, DriftDetail]
    bitwise_fingerprints: dict[str, Any]
    passed: bool

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


def plan_distributed_logprob_cases(*, tp_world_sizes: Sequence[int] = (1, 2, 4), cp_world_sizes: Sequence[int] = (1, 2),
                                   **overrides: Any) -> tuple[DistributedLogprobCase, ...]:
    """The topology product in a fixed order (TP outer, CP inner)."""
    return tuple(DistributedLogprobCase(tp_world_size=tp, cp_world_size=cp, **overrides) for tp in tp_world_sizes
                 for cp in cp_world_sizes)


def rank_topology(case: DistributedLogprobCase, global_rank: int) -> RankTopology:
    if not 0 <= global_rank < case.world_size:
        raise ValueError(f"global_rank must be in [0, {case.world_size})")
    cp_rank, tp_rank = divmod(global_rank, case.tp_world_size)
    first = cp_rank * case.tp_world_size
    return RankTopology(global_rank, case.world_size, tp_rank, case.tp_world_size, cp_rank, case.cp_world_size,
                        tuple(range(first, first + case.tp_world_size)))


def token_shard_bounds(num_tokens: int, cp_world_size: int) -> tuple[tuple[int, int], ...]:
    """Contiguous token rows per CP rank; the first ``num_tokens % cp`` ranks take one row more."""
    if num_tokens < cp_world_size:
        raise ValueError("num_tokens must be at least cp_world_size")
    q, r = divmod(num_tokens, cp_world_size)
    out, at = [], 0
    for i in range(cp_world_size):
        n = q + (i < r)
        out.append((at, at + n))
        at += n
    return tuple(out)


def vocab_shard_bounds(case: DistributedLogprobCase) -> tuple[tuple[int, int], ...]:
    """Whole vocabulary tiles per TP rank; the first ``tiles % tp`` ranks take one tile more."""
    tile = case.padded_vocab_size // case.num_vocab_tiles
    q, r = divmod(case.num_vocab_tiles, case.tp_world_size)
    out, at = [], 0
    for i in range(case.tp_world_size):
        n = q + (i < r)
        out.append((at * tile, (at + n) * tile))
        at += n
    return tuple(out)


def format_launch_command(case: DistributedLogprobCase, *, output, device: str = "cuda", dist_backend: str | None = None) -> str:
    backend = dist_backend or ("nccl" if device == "cuda" else "gloo")
    return shlex.join(["python", "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
                       f"--nproc-per-node={case.world_size}", "-m", "rl_kernel_b200.validation.common.distributed_logprob_comparison",
                       "--tp", str(case.tp_world_size), "--cp", str(case.cp_world_size), "--dtype", case.dtype, "--backend",
                       case.requested_backend, "--real-vocab", str(case.real_vocab_size), "--padded-vocab",
                       str(case.padded_vocab_size), "--num-vocab-tiles", str(case.num_vocab_tiles), "--batch", str(case.batch_size),
                       "--seq", str(case.sequence_length), "--prompt-tokens", str(case.prompt_tokens), "--seed", str(case.seed),
                       "--device", device, "--dist-backend", backend, "--output", str(output)])


def canonical_inputs(case: DistributedLogprobCase) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(fp32 logits [N, padded vocab], targets [N] with ignore_index on prompt rows, active mask [N]); same on every rank."""
    g = torch.Generator().manual_seed(case.seed)
    logits = torch.randn(case.num_tokens, case.padded_vocab_size, generator=g)
    targets = torch.randint(0, case.real_vocab_size, (case.num_tokens,), generator=g)
    active = torch.ones(case.batch_size, case.sequence_length, dtype=torch.bool)
    active[:, : case.prompt_tokens] = False
    active = active.reshape(-1)
    return logits, targets.masked_fill(~active, case.ignore_index), active


def make_contract(case: DistributedLogprobCase, topo: RankTopology, active_local: torch.Tensor) -> LogprobContract:
    return LogprobContract(role=LogprobRole.TRAIN, dtype=LogprobDType(case.dtype),
                           mask=MaskSpec(int(active_local.numel()), tuple(bool(v) for v in active_local.tolist()), case.ignore_index),
                           sharding=ShardingSpec(tp_rank=topo.tp_rank, tp_world_size=case.tp_world_size,
                                                 vocab_shard_bounds=vocab_shard_bounds(case), real_vocab_size=case.real_vocab_size,
                                                 padded_vocab_size=case.padded_vocab_size, cp_rank=topo.cp_rank,
                                                 cp_world_size=case.cp_world_size),
                           reduction=ReductionSpec())


def fp32_oracle(logits: torch.Tensor, targets: torch.Tensor, active: torch.Tensor, real_vocab: int):
    real = logits[:, :real_vocab].float()
    lse = torch.logsumexp(real, -1)
    sel = real.gather(1, targets.masked_fill(~active, 0)[:, None])[:, 0]
    return torch.where(active, sel - lse, torch.zeros_like(lse)), lse


def _tolerance(dtype: str) -> tuple[float, float]:
    try:
        t = resolve_tolerance("vocab_parallel_logp", _TOL_KEYS[dtype])
    except KeyError:
        t = resolve_tolerance("linear_logp", _TOL_KEYS[dtype])
    return t.atol, t.rtol


def drift_detail(cand: torch.Tensor, ref: torch.Tensor, active: torch.Tensor, positions: torch.Tensor, targets: torch.Tensor,
                 owners: torch.Tensor | None, atol: float, rtol: float) -> DriftDetail:
    stats = summarize_logprob_drift(cand.float(), ref.float(), mask=active)
    if stats.active_count == 0:
        return DriftDetail(stats, 0.0, None, None, None, None, None, atol, rtol, True)
    diff = (cand.double() - ref.double()).abs().masked_fill(~active, -1.0)
    i = int(diff.argmax())
    rel = float((diff[active] / ref.double().abs()[active].clamp_min(1e-12)).max())
    ok = bool((diff[active] <= atol + rtol * ref.double().abs()[active]).all())
    return DriftDetail(stats, rel, int(positions[i]), int(targets[i]), None if owners is None else int(owners[i]), float(cand[i]),
                       float(ref[i]), atol, rtol, ok)


def _sha(t: torch.Tensor) -> str:
    t = t.detach().contiguous().cpu()
    return hashlib.sha256(str(t.dtype).encode() + str(tuple(t.shape)).encode() + t.view(torch.uint8).numpy().tobytes()).hexdigest()


def execute_rank(case: DistributedLogprobCase, topo: RankTopology, tp_group, device: torch.device) -> dict[str, Any]:
    """This rank's shard through the operator; the payload rank 0 aggregates."""
    logits, targets, active = canonical_inputs(case)
    t0, t1 = token_shard_bounds(case.num_tokens, case.cp_world_size)[topo.cp_rank]
    v0, v1 = vocab_shard_bounds(case)[topo.tp_rank]
    shard = logits[t0:t1, v0:v1].to(_DTYPES[case.dtype]).to(device)
    tg, act = targets[t0:t1].to(device), active[t0:t1]
    contract = make_contract(case, topo, act)
    op = VocabParallelLogprobOp()
    logp, lse = op.apply(shard, tg, contract=contract, tp_group=tp_group, num_vocab_tiles=case.num_vocab_tiles)
    logp, lse = logp.float().cpu(), lse.float().cpu()
    # the oracle sees the logits after the rounding to the case dtype, so that the drift is the operator's own
    ref_lp, ref_lse = fp32_oracle(logits[t0:t1].to(_DTYPES[case.dtype]).float(), targets[t0:t1], act, case.real_vocab_size)
    replicated = True
    if case.tp_world_size > 1:
        import torch.distributed as dist

        both = torch.stack([logp, lse]).to(device)
        gathered = [torch.empty_like(both) for _ in range(case.tp_world_size)]
        dist.all_gather(gathered, both, group=tp_group)
        replicated = all(torch.equal(g.view(torch.int32), gathered[0].view(torch.int32)) for g in gathered)
    atol, rtol = _tolerance(case.dtype)
    pos = torch.arange(t0, t1)
    d_lp = drift_detail(logp, ref_lp, act, pos, targets[t0:t1], None, atol, rtol)
    d_lse = drift_detail(lse, ref_lse, act, pos, targets[t0:t1], None, atol, rtol)
    rep = RankLogprobReport(topo.global_rank, topo.tp_rank, case.tp_world_size, topo.cp_rank, case.cp_world_size, 1, 1, t0, t1, v0, v1,
                            str(device), case.requested_backend, BACKEND_ID, case.requested_backend != BACKEND_ID,
                            contract.cross_rank_fingerprint(), contract.to_dict() if hasattr(contract, "to_dict") else {},
                            {"backend_id": BACKEND_ID, "implementation_kind": "reference"}, replicated, d_lse, d_lp,
                            replicated and d_lp.passed and d_lse.passed)
    return {"report": rep, "logp": logp, "lse": lse, "ref_logp": ref_lp, "ref_lse": ref_lse, "active": act, "targets": targets[t0:t1],
            "positions": pos}


def aggregate(case: DistributedLogprobCase, payloads: list[dict[str, Any]], *, launch_command: str = "",
              environment: dict | None = None) -> DistributedLogprobReport:
    """Assemble the ranks' rows (TP rank 0 of every CP shard) into the global order and judge the whole."""
    owners_first = sorted((p for p in payloads if p["report"].tp_rank == 0), key=lambda p: p["report"].cp_rank)
    cat = lambda k: torch.cat([p[k] for p in owners_first])  # noqa: E731
    owners = torch.cat([torch.full((p["logp"].numel(),), p["report"].global_rank) for p in owners_first])
    atol, rtol = _tolerance(case.dtype)
    agg = {"logp": drift_detail(cat("logp"), cat("ref_logp"), cat("active"), cat("positions"), cat("targets"), owners, atol, rtol),
           "lse": drift_detail(cat("lse"), cat("ref_lse"), cat("active"), cat("positions"), cat("targets"), owners, atol, rtol)}
    active = cat("active")
    prints = {"logp_active_sha256": _sha(cat("logp")[active]), "lse_active_sha256": _sha(cat("lse")[active]),
              "active_tokens": int(active.sum()), "topology": f"tp{case.tp_world_size}xcp{case.cp_world_size}"}
    ranks = tuple(sorted((p["report"] for p in payloads), key=lambda r: r.global_rank))
    return DistributedLogprobReport(SCHEMA_VERSION, case.case_id, asdict(case), launch_command, environment or {}, ranks, agg, prints,
                                    all(r.passed for r in ranks) and all(d.passed for d in agg.values()))


def run_distributed_logprob_case(case: DistributedLogprobCase, *, device: str = "cpu", dist_backend: str | None = None,
                                 output=None) -> DistributedLogprobReport | None:
    """Entry of every rank of a ``torch.distributed`` launch with ``case.world_size`` processes.  Rank 0 returns (and
    writes) the report; the others return None."""
    import torch.distributed as dist

    own_group = not dist.is_initialized()
    if own_group:
        dist.init_process_group(dist_backend or ("nccl" if device == "cuda" else "gloo"), timeout=_GROUP_TIMEOUT)
    try:
        if dist.get_world_size() != case.world_size:
            raise RuntimeError(f"the case needs {case.world_size} ranks, the launch has {dist.get_world_size()}")
        rank = dist.get_rank()
        topo = rank_topology(case, rank)
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank))) if device == "cuda" else torch.device("cpu")
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        groups = [dist.new_group(list(rank_topology(case, c * case.tp_world_size).tp_group_ranks), timeout=_GROUP_TIMEOUT)
                  for c in range(case.cp_world_size)]                   # every rank creates every group, in one order
        payload = execute_rank(case, topo, groups[topo.cp_rank] if case.tp_world_size > 1 else None, dev)
        gathered: list = [None] * case.world_size
        dist.all_gather_object(gathered, payload)
        if rank != 0:
            return None
        env = {"torch": torch.__version__, "dist_backend": dist.get_backend(), "device": device,
               "cuda_device": torch.cuda.get_device_name(dev) if dev.type == "cuda" else None}
        rep = aggregate(case, gathered, launch_command=format_launch_command(case, output=output or "report.json", device=device,
                                                                            dist_backend=dist_backend), environment=env)
        if output:
            with open(output, "w") as f:
                f.write(json.dumps(rep.to_dict(), indent=2, sort_keys=True, allow_nan=False) + "\n")
        return rep
    finally:
        if own_group:
            dist.destroy_process_group()


def main(argv: Sequence[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--dtype", choices=sorted(_DTYPES), default="bf16")
    ap.add_argument("--backend", default=BACKEND_ID)
    ap.add_argument("--real-vocab", type=int, default=151936)
    ap.add_argument("--padded-vocab", type=int, default=151936)
    ap.add_argument("--num-vocab-tiles", type=int, default=1187)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=16)
    ap.add_argument("--prompt-tokens", type=int, default=8)
    ap.add_argument("--seed", type=int, default=123)
    ap.add_argument("--device", choices=("cpu", "cuda"), default="cpu")
    ap.add_argument("--dist-backend", default=None)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    case = DistributedLogprobCase(a.tp, a.cp, a.dtype, a.backend, a.real_vocab, a.padded_vocab, a.num_vocab_tiles, a.batch, a.seq,
                                  a.prompt_tokens, a.seed)
    rep = run_distributed_logprob_case(case, device=a.device, dist_backend=a.dist_backend, output=a.output)
    if rep is not None:
        print(json.dumps({"case_id": rep.case_id, "passed": rep.passed, "fingerprints": rep.bitwise_fingerprints}, sort_keys=True))
        sys.exit(0 if rep.passed else 1)


__all__ = ["DistributedLogprobCase", "DistributedLogprobReport", "DriftDetail", "RankLogprobReport", "RankTopology", "aggregate",
           "canonical_inputs", "drift_detail", "execute_rank", "format_launch_command", "fp32_oracle", "make_contract",
           "plan_distributed_logprob_cases", "rank_topology", "run_distributed_logprob_case", "token_shard_bounds",
           "vocab_shard_bounds"]

if __name__ == "__main__":
    main()
