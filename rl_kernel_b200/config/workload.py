"""Workload manifest and logical-batch transforms (parity: rl_engine/config/workload.py:18-1212).

The manifest (``workloads/qwen3_8b.json``) pins what validation runs on: the model identity (full
Qwen3-8B architecture, never shrunk), the fixed token fixtures, the primary Batch x Chunked-Prefill
matrix, the backend profiles and the representative operator cases (shape, expected backend /
kernel, provenance).  ``validate_manifest`` fails closed on anything missing or inconsistent.

Logical vs physical.  A ``LogicalBatch`` is an ordered multiset of samples, each token identified
by (sample_id, position).  A physical layout says how those tokens are laid out for one run:
packed back to back, cut into prefill chunks, padded left or right, permuted, or one sample at a
time.  Every layout carries a restore map back to logical keys, so results of different layouts
are compared token by token, never by position in a tensor.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from functools import lru_cache
from pathlib import Path
from typing import Any, Mapping, Sequence

import torch

_DIR = Path(__file__).resolve().parent / "workloads"
_MANIFEST_PATH = _DIR / "qwen3_8b.json"

_REQUIRED_TOP_LEVEL = ("version", "workload_id", "seed", "model_identity", "chain_semantics", "stochastic_policy",
                       "primary_matrix", "fixtures", "logical_identity", "capabilities", "backend_profiles",
                       "representative_cases")
_REQUIRED_MATRIX_CELLS = ("B1-singleton_aggregate/full", "BN/full", "B1-singleton_aggregate/chunked", "BN/chunked")
_REQUIRED_PROFILES = ("b200_bf16", "reference_fp32")
_REQUIRED_CHAIN_NODES = ("embedding", "input_layernorm", "qkv_proj", "qk_norm", "rope", "attention", "o_proj",
                         "post_attention_layernorm", "gate_up_proj", "swiglu", "down_proj", "final_layernorm", "lm_head",
                         "logprob")
_FORBIDDEN_COMPARISON_ROLES = frozenset({"baseline", "singleton_aggregate"})
_OFFICIAL_FINGERPRINT = {
    "num_hidden_layers": 36, "hidden_size": 4096, "intermediate_size": 12288, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-06,
    "tie_word_embeddings": False, "attention_bias": False, "qk_norm": True,
}
_CASE_KEYS = ("case_id", "family", "shape", "expected_backend_id", "expected_kernel_config_id", "actual_backend_id",
              "actual_kernel_config_id", "provenance_status", "provenance_evidence", "algorithm_property",
              "architecture_identity", "fixture_id", "operator_spec")


class WorkloadError(ValueError):
    """The manifest, a fixture or a layout request is inconsistent."""


def _require(mapping: Mapping[str, Any], key: str, *, context: str) -> Any:
    if key not in mapping:
        raise WorkloadError(f"{context} lacks {key!r}")
    return mapping[key]


# ------------------------------------------------------------------------------------ logical / physical data model
@dataclass(frozen=True)
class LogicalToken:
    sample_id: str
    token_position: int
    token_id: int
    is_active: bool


@dataclass(frozen=True)
class LogicalSample:
    """One logical sequence; tokens at or beyond ``prompt_len`` are active (they carry the loss)."""
    sample_id: str
    token_ids: tuple[int, ...]
    prompt_len: int
    seq_len: int

    def __post_init__(self) -> None:
        if len(self.token_ids) != self.seq_len or not 0 <= self.prompt_len <= self.seq_len:
            raise WorkloadError(f"sample {self.sample_id}: {len(self.token_ids)} ids for seq_len {self.seq_len}, prompt "
                                f"{self.prompt_len}")

    def tokens(self) -> tuple[LogicalToken, ...]:
        return tuple(LogicalToken(self.sample_id, p, int(t), p >= self.prompt_len) for p, t in enumerate(self.token_ids))

    def active_tokens(self) -> tuple[LogicalToken, ...]:
        return tuple(t for t in self.tokens() if t.is_active)


@dataclass(frozen=True)
class LogicalBatch:
    workload_id: str
    seed: int
    samples: tuple[LogicalSample, ...]
    cell_id: str | None = None

    @property
    def sample_ids(self) -> tuple[str, ...]:
        return tuple(s.sample_id for s in self.samples)

    def sample(self, sample_id: str) -> LogicalSample:
        for s in self.samples:
            if s.sample_id == sample_id:
                return s
        raise KeyError(sample_id)

    def logical_keys(self, *, active_only: bool = False) -> tuple[tuple[str, int], ...]:
        return tuple((t.sample_id, t.token_position) for s in self.samples for t in s.tokens()
                     if t.is_active or not active_only)

    def active_token_count(self) -> int:
        return sum(len(s.active_tokens()) for s in self.samples)

    def token_multiset(self, *, active_only: bool = True) -> tuple[tuple[str, int, int], ...]:
        return tuple((t.sample_id, t.token_position, t.token_id) for s in self.samples for t in s.tokens()
                     if t.is_active or not active_only)


@dataclass(frozen=True)
class PaddedBatch:
    """Left- or right-padded [B, padded_len] layout; ``restore_map[b][p]`` is the logical key or None for padding."""
    physical_token_ids: tuple[tuple[int, ...], ...]
    physical_attention_mask: tuple[tuple[int, ...], ...]
    physical_loss_mask: tuple[tuple[int, ...], ...]
    physical_position_ids: tuple[tuple[int, ...], ...]
    pad_side: str
    pad_token_id: int
    padded_len: int
    restore_map: tuple[tuple[tuple[str, int] | None, ...], ...]
    sample_ids: tuple[str, ...]
    layout_kind: str = "padded"


@dataclass(frozen=True)
class PhysicalLayout:
    """Flattened tokens with their restore map.  ``packed``: one segment per sample, in batch order.
    ``chunked``: one segment per (sample, prefill chunk), a sample's chunks consecutive and ascending."""
    layout_kind: str
    physical_token_ids: tuple[int, ...]
    physical_loss_mask: tuple[int, ...]
    restore_map: tuple[tuple[str, int], ...]
    segment_offsets: tuple[int, ...]
    segment_lengths: tuple[int, ...]
    segment_sample_ids: tuple[str, ...] = ()
    segment_position_starts: tuple[int, ...] = ()

    @property
    def num_tokens(self) -> int:
        return len(self.physical_token_ids)

    def position_ids(self) -> tuple[int, ...]:
        return tuple(k[1] for k in self.restore_map)

    def cu_seqlens(self) -> tuple[int, ...]:
        return self.segment_offsets + (self.num_tokens,)


@dataclass(frozen=True)
class ChunkPlan:
    seq_len: int
    chunk_size: int
    chunk_spans: tuple[tuple[int, int], ...]        # half-open [start, end)

    @property
    def num_chunks(self) -> int:
        return len(self.chunk_spans)


@dataclass(frozen=True)
class SingletonAggregatePlan:
    """B = 1 x N runs that must reproduce one B = N run of the same multiset."""
    sample_ids: tuple[str, ...]
    run_sample_ids: tuple[tuple[str, ...], ...]
    aggregation_order: tuple[str, ...]
    denominator: str
    token_multiset: tuple[tuple[str, int, int], ...]


@dataclass
class WS1Manifest:
    raw: dict[str, Any]
    path: Path = field(default=_MANIFEST_PATH)

    @property
    def version(self) -> str:
        return str(self.raw["version"])

    @property
    def workload_id(self) -> str:
        return str(self.raw["workload_id"])

    @property
    def seed(self) -> int:
        return int(self.raw["seed"])

    @property
    def model_identity(self) -> dict[str, Any]:
        return dict(self.raw["model_identity"])

    @property
    def chain_semantics(self) -> dict[str, Any]:
        return dict(self.raw["chain_semantics"])

    @property
    def clip_interval(self) -> tuple[float, float]:
        lo, hi = self.raw["chain_semantics"]["clip_interval"]
        return float(lo), float(hi)

    @property
    def primary_matrix(self) -> dict[str, Any]:
        return dict(self.raw["primary_matrix"])

    @property
    def fixtures(self) -> dict[str, Any]:
        return dict(self.raw["fixtures"])

    @property
    def backend_profiles(self) -> dict[str, Any]:
        return dict(self.raw["backend_profiles"])

    @property
    def representative_cases(self) -> list[dict[str, Any]]:
        return list(self.raw["representative_cases"])

    # short forms kept for callers of the earlier, smaller manifest
    @property
    def cases(self) -> tuple:
        return tuple(self.raw["representative_cases"])

    def case(self, case_id: str) -> dict:
        return get_case(self, case_id)


def default_manifest_path() -> Path:
    return _MANIFEST_PATH


@lru_cache(maxsize=4)
def _load(path: str) -> WS1Manifest:
    raw = json.loads(Path(path).read_text())
    validate_manifest(raw)
    return WS1Manifest(raw, Path(path))


def load_manifest(path: str | Path | None = None) -> WS1Manifest:
    """``path``: a file, or the bare name of a manifest in ``workloads/`` (default ``qwen3_8b``)."""
    if path is None:
        p = _MANIFEST_PATH
    else:
        p = Path(path)
        if not p.suffix and not p.exists():
            p = _DIR / f"{path}.json"
    return _load(str(p))


# ------------------------------------------------------------------------------------ validation
def validate_manifest(raw: Mapping[str, Any]) -> None:
    for key in _REQUIRED_TOP_LEVEL:
        _require(raw, key, context="manifest")
    _validate_model_identity(raw["model_identity"])
    _validate_chain_semantics(raw["chain_semantics"])
    _validate_stochastic_policy(raw["stochastic_policy"])
    _validate_fixtures(raw["fixtures"], raw["primary_matrix"])
    _validate_primary_matrix(raw["primary_matrix"], raw["fixtures"])
    _validate_backend_profiles(raw["backend_profiles"])
    _validate_representative_cases(raw["representative_cases"], raw["fixtures"])
    want = raw.get("fixture_identity_sha256")
    if want is not None and want != manifest_identity_hash(raw):
        raise WorkloadError("fixture_identity_sha256 does not match the manifest's identity payload")


def _validate_model_identity(identity: Mapping[str, Any]) -> None:
    _require(identity, "model_id", context="model_identity")
    fp = _require(identity, "config_fingerprint", context="model_identity")
    for key, value in _OFFICIAL_FINGERPRINT.items():
        if fp.get(key) != value:
            raise WorkloadError(f"model_identity.config_fingerprint.{key} must be {value!r} (full Qwen3-8B); got {fp.get(key)!r}")


def _validate_chain_semantics(sem: Mapping[str, Any]) -> None:
    nodes = list(_require(sem, "nodes", context="chain_semantics"))
    missing = [n for n in _REQUIRED_CHAIN_NODES if n not in nodes]
    if missing:
        raise WorkloadError(f"chain_semantics.nodes lacks {missing}")
    lo, hi = _require(sem, "clip_interval", context="chain_semantics")
    if not 0 < lo < 1 < hi:
        raise WorkloadError("chain_semantics.clip_interval must bracket 1")
    if _require(sem, "loss_denominator", context="chain_semantics") != "active_token_count_across_all_samples":
        raise WorkloadError("chain loss must be normalised by the active tokens of all samples")


def _validate_stochastic_policy(policy: Mapping[str, Any]) -> None:
    if _require(policy, "dropout", context="stochastic_policy") not in (0, 0.0):
        raise WorkloadError("validation runs without dropout")
    if not _require(policy, "sampling_is_seeded", context="stochastic_policy"):
        raise WorkloadError("sampling must be seeded (Philox keys from seed, step, sequence, position)")


def _validate_fixtures(fx: Mapping[str, Any], matrix: Mapping[str, Any]) -> None:
    samples = _require(fx, "samples", context="fixtures")
    ids = [s["sample_id"] for s in samples]
    if len(set(ids)) != len(ids):
        raise WorkloadError("fixture sample ids must be unique")
    for s in samples:
        if len(s["token_ids"]) != s["seq_len"] or not 0 < s["prompt_len"] < s["seq_len"]:
            raise WorkloadError(f"fixture sample {s['sample_id']} is inconsistent")
        if max(s["token_ids"]) >= _OFFICIAL_FINGERPRINT["vocab_size"] or min(s["token_ids"]) < 0:
            raise WorkloadError(f"fixture sample {s['sample_id']} has ids outside the vocabulary")
    if list(_require(fx, "varlen_seq_lens", context="fixtures")) != [s["seq_len"] for s in samples]:
        raise WorkloadError("fixtures.varlen_seq_lens must list the samples' lengths")
    if len(set(fx["varlen_seq_lens"])) < 2:
        raise WorkloadError("the fixture must contain sequences of different lengths")
    pad = _require(fx, "padding", context="fixtures")
    if set(pad["modes"]) != {"left", "right"} or pad["primary_padded_len"] <= max(fx["varlen_seq_lens"]):
        raise WorkloadError("padding needs both sides and a padded length beyond the longest sample")
    if list(matrix.get("sample_ids", [])) != ids:
        raise WorkloadError("primary_matrix.sample_ids must equal the fixture sample order")
    _require(fx, "long_samples", context="fixtures")


def _validate_primary_matrix(matrix: Mapping[str, Any], fx: Mapping[str, Any]) -> None:
    cells = {c["cell_id"]: c for c in _require(matrix, "cells", context="primary_matrix")}
    for cid in _REQUIRED_MATRIX_CELLS:
        if cid not in cells:
            raise WorkloadError(f"primary_matrix lacks cell {cid}")
    n = int(_require(matrix, "N", context="primary_matrix"))
    if n != len(fx["samples"]) or n < 2:
        raise WorkloadError("primary_matrix.N must equal the number of fixture samples (at least 2)")
    perm = matrix["batch_permutation"]["permutation"]
    if sorted(perm) != list(range(n)) or perm == list(range(n)):
        raise WorkloadError("batch_permutation must be a non-identity permutation of the samples")
    chunk = int(matrix["chunk"]["chunk_size_tokens"])
    longest = max(fx["varlen_seq_lens"])
    if not (chunk < longest and longest % chunk):
        raise WorkloadError("the chunk size must cut the longest sample into >= 2 chunks and not divide it")
    for c in cells.values():
        if c["aggregation"]["denominator"] != "active_token_count_across_all_samples":
            raise WorkloadError(f"cell {c['cell_id']} must aggregate over the active tokens of all samples")
        if c.get("comparison_role") in _FORBIDDEN_COMPARISON_ROLES:
            raise WorkloadError(f"cell {c['cell_id']}: every cell is compared with every other; no cell is a baseline")


def _validate_backend_profiles(profiles: Mapping[str, Any]) -> None:
    for name in _REQUIRED_PROFILES:
        prof = _require(profiles, name, context="backend_profiles")
        for key in ("backend_family", "execution_dtype", "operators"):
            _require(prof, key, context=f"backend_profiles.{name}")
        missing = [n for n in _REQUIRED_CHAIN_NODES if n not in prof["operators"]]
        if missing:
            raise WorkloadError(f"backend profile {name} does not bind chain nodes {missing}")


def _validate_representative_cases(cases: Sequence[Mapping[str, Any]], fx: Mapping[str, Any]) -> None:
    if not cases:
        raise WorkloadError("representative_cases must be non-empty")
    ids = [c.get("case_id") for c in cases]
    if len(set(ids)) != len(ids):
        raise WorkloadError("representative_cases case_id values must be unique")
    fixture_ids = {"primary_varlen", "long_varlen", fx["short_full_model_fixture"]["fixture_id"], "decode_context"}
    for case in cases:
        for key in _CASE_KEYS:
            if key not in case:
                raise WorkloadError(f"case {case.get('case_id')} missing {key!r}")
        if case["architecture_identity"] != "full_qwen3_8b_dense":
            raise WorkloadError(f"case {case['case_id']} must pin architecture_identity=full_qwen3_8b_dense")
        if case["provenance_status"] != "runtime_evidence_required":
            raise WorkloadError(f"case {case['case_id']} must require runtime candidate evidence")
        if (case["actual_backend_id"], case["actual_kernel_config_id"]) != (case["expected_backend_id"],
                                                                             case["expected_kernel_config_id"]):
            raise WorkloadError(f"case {case['case_id']} actual backend / kernel differs from the expected one")
        ev = case["provenance_evidence"]
        if ev.get("kind") != "runtime_execution_via_operator_specs" or ev.get("resolved_path") != case["actual_kernel_config_id"]:
            raise WorkloadError(f"case {case['case_id']} lacks runtime provenance for its kernel")
        if not ev.get("algorithm_source") or not ev.get("runtime_evidence_command"):
            raise WorkloadError(f"case {case['case_id']} lacks an algorithm source or an evidence command")
        if case["fixture_id"] not in fixture_ids:
            raise WorkloadError(f"case {case['case_id']} names unknown fixture {case['fixture_id']!r}")
    for profile in _REQUIRED_PROFILES:
        mine = [c for c in cases if profile in c.get("profile_ids", [])]
        for family in ("gemm", "attention", "logprob"):
            if not any(c["family"] == family for c in mine):
                raise WorkloadError(f"profile {profile} has no {family} representative case")
        if len({int(c["shape"]["M"]) for c in mine if c["family"] == "gemm"}) < 2:
            raise WorkloadError(f"profile {profile} GEMM cases require multiple M values")
        if {c["shape"]["mode"] for c in mine if c["family"] == "attention"} < {"prefill", "decode"}:
            raise WorkloadError(f"profile {profile} attention cases require prefill and decode")


# ------------------------------------------------------------------------------------ building batches and layouts
def build_logical_batch(manifest: WS1Manifest | None = None, *, cell_id: str | None = "BN/full",
                        fixture: str = "samples") -> LogicalBatch:
    """The fixture's samples in their fixed order (``fixture="long_samples"``: lengths that cross 128-token blocks)."""
    m = manifest or load_manifest()
    samples = tuple(LogicalSample(s["sample_id"], tuple(int(t) for t in s["token_ids"]), int(s["prompt_len"]), int(s["seq_len"]))
                    for s in _expand_samples(m.fixtures[fixture]))
    return LogicalBatch(m.workload_id, m.seed, samples, cell_id)


def _expand_samples(entries: Sequence[Mapping[str, Any]]) -> list[dict]:
    """Samples are stored either with explicit ``token_ids`` or as ``{"token_rule": {"base", "stride", "mod"}}``
    (long fixtures: ids = (base + stride * p) mod mod, so the file stays small and the ids stay fixed)."""
    out = []
    for s in entries:
        s = dict(s)
        if "token_ids" not in s:
            r = s["token_rule"]
            s["token_ids"] = [(r["base"] + r["stride"] * p) % r["mod"] for p in range(s["seq_len"])]
        out.append(s)
    return out


def get_matrix_cell(manifest: WS1Manifest, cell_id: str) -> dict[str, Any]:
    for c in manifest.primary_matrix["cells"]:
        if c["cell_id"] == cell_id:
            return dict(c)
    raise WorkloadError(f"unknown matrix cell {cell_id!r}")


def matrix_cell_ids(manifest: WS1Manifest | None = None) -> tuple[str, ...]:
    return tuple(c["cell_id"] for c in (manifest or load_manifest()).primary_matrix["cells"])


def build_chunk_plan(seq_len: int, chunk_size: int) -> ChunkPlan:
    if seq_len <= 0 or chunk_size <= 0:
        raise WorkloadError("seq_len and chunk_size must be positive")
    return ChunkPlan(seq_len, chunk_size, tuple((a, min(seq_len, a + chunk_size)) for a in range(0, seq_len, chunk_size)))


def chunk_plan_from_manifest(manifest: WS1Manifest | None = None) -> ChunkPlan:
    m = manifest or load_manifest()
    return build_chunk_plan(max(m.fixtures["varlen_seq_lens"]), int(m.primary_matrix["chunk"]["chunk_size_tokens"]))


def apply_packing(batch: LogicalBatch) -> PhysicalLayout:
    ids, loss, restore, offs, lens = [], [], [], [], []
    for s in batch.samples:
        offs.append(len(ids))
        lens.append(s.seq_len)
        for t in s.tokens():
            ids.append(t.token_id)
            loss.append(int(t.is_active))
            restore.append((t.sample_id, t.token_position))
    return PhysicalLayout("packed", tuple(ids), tuple(loss), tuple(restore), tuple(offs), tuple(lens), batch.sample_ids,
                          (0,) * len(lens))


def apply_chunking(batch: LogicalBatch, *, chunk_size: int) -> PhysicalLayout:
    ids, loss, restore, offs, lens, sids, starts = [], [], [], [], [], [], []
    for s in batch.samples:
        toks = s.tokens()
        for a, b in build_chunk_plan(s.seq_len, chunk_size).chunk_spans:
            offs.append(len(ids))
            lens.append(b - a)
            sids.append(s.sample_id)
            starts.append(a)
            for t in toks[a:b]:
                ids.append(t.token_id)
                loss.append(int(t.is_active))
                restore.append((t.sample_id, t.token_position))
    return PhysicalLayout("chunked", tuple(ids), tuple(loss), tuple(restore), tuple(offs), tuple(lens), tuple(sids),
                          tuple(starts))


def restore_logical_order(layout: PhysicalLayout, values: Sequence[Any]) -> dict[tuple[str, int], Any]:
    if len(values) != layout.num_tokens:
        raise WorkloadError(f"{len(values)} values for a layout of {layout.num_tokens} tokens")
    return {key: values[i] for i, key in enumerate(layout.restore_map)}


def apply_padding(batch: LogicalBatch, *, pad_side: str, manifest: WS1Manifest | None = None,
                  padded_len: int | None = None) -> PaddedBatch:
    if pad_side not in ("left", "right"):
        raise WorkloadError("pad_side must be 'left' or 'right'")
    m = manifest or load_manifest()
    pad_id = int(m.fixtures["padding"]["pad_token_id"])
    longest = max(s.seq_len for s in batch.samples)
    L = padded_len or max(int(m.fixtures["padding"]["primary_padded_len"]), longest + 1)
    if L < longest:
        raise WorkloadError("padded_len is shorter than the longest sample")
    ids, att, loss, pos, restore = [], [], [], [], []
    for s in batch.samples:
        n, gap = s.seq_len, L - s.seq_len
        real_ids = list(s.token_ids)
        real_loss = [int(p >= s.prompt_len) for p in range(n)]
        keys: list[tuple[str, int] | None] = [(s.sample_id, p) for p in range(n)]
        if pad_side == "right":
            ids.append(tuple(real_ids + [pad_id] * gap))
            att.append(tuple([1] * n + [0] * gap))
            loss.append(tuple(real_loss + [0] * gap))
            pos.append(tuple(list(range(n)) + [0] * gap))
            restore.append(tuple(keys + [None] * gap))
        else:
            ids.append(tuple([pad_id] * gap + real_ids))
            att.append(tuple([0] * gap + [1] * n))
            loss.append(tuple([0] * gap + real_loss))
            pos.append(tuple([0] * gap + list(range(n))))
            restore.append(tuple([None] * gap + keys))
    return PaddedBatch(tuple(ids), tuple(att), tuple(loss), tuple(pos), pad_side, pad_id, L, tuple(restore), batch.sample_ids)


def restore_logical_order_from_padded(padded: PaddedBatch, values) -> dict[tuple[str, int], Any]:
    out = {}
    for b, row in enumerate(padded.restore_map):
        for p, key in enumerate(row):
            if key is not None:
                out[key] = values[b][p]
    return out


def permute_batch(batch, permutation=None, seed: int | None = None):
    """``permute_batch(LogicalBatch, permutation)`` -> the batch with its samples reordered.
    (A tensor as first argument keeps the row-permutation helper: ``(ids[perm], restore_fn)``.)"""
    if isinstance(batch, torch.Tensor):
        perm = torch.randperm(batch.shape[0], generator=torch.Generator().manual_seed(int(permutation or seed or 0)))
        inv = torch.argsort(perm)
        return batch[perm], lambda out: out[inv]
    perm = tuple(int(i) for i in permutation)
    if sorted(perm) != list(range(len(batch.samples))):
        raise WorkloadError("permutation must reorder exactly the batch's samples")
    return LogicalBatch(batch.workload_id, batch.seed, tuple(batch.samples[i] for i in perm), batch.cell_id)


def batch_permutation_from_manifest(manifest: WS1Manifest | None = None) -> tuple[int, ...]:
    return tuple(int(i) for i in (manifest or load_manifest()).primary_matrix["batch_permutation"]["permutation"])


def singleton_aggregate_plan(batch: LogicalBatch, manifest: WS1Manifest | None = None) -> SingletonAggregatePlan:
    m = manifest or load_manifest()
    cell = get_matrix_cell(m, "B1-singleton_aggregate/full")
    return SingletonAggregatePlan(batch.sample_ids, tuple((sid,) for sid in batch.sample_ids), batch.sample_ids,
                                  cell["aggregation"]["denominator"], batch.token_multiset())


def same_logical_multiset(a: LogicalBatch, b: LogicalBatch, *, active_only: bool = True) -> bool:
    return sorted(a.token_multiset(active_only=active_only)) == sorted(b.token_multiset(active_only=active_only))


def profile_required_nodes(manifest: WS1Manifest | None = None, profile: str = "b200_bf16") -> tuple[str, ...]:
    m = manifest or load_manifest()
    return tuple(n for n in m.chain_semantics["nodes"] if n in m.backend_profiles[profile]["operators"])


def profile_missing_required_nodes(manifest: WS1Manifest | None = None, profile: str = "b200_bf16") -> tuple[str, ...]:
    m = manifest or load_manifest()
    return tuple(n for n in _REQUIRED_CHAIN_NODES if n not in m.backend_profiles[profile]["operators"])


def get_case(manifest: WS1Manifest | None = None, case_id: str = "") -> dict[str, Any]:
    for c in (manifest or load_manifest()).representative_cases:
        if c["case_id"] == case_id:
            return dict(c)
    raise KeyError(case_id)


def case_ids(manifest: WS1Manifest | None = None) -> tuple[str, ...]:
    return tuple(c["case_id"] for c in (manifest or load_manifest()).representative_cases)


def assert_no_undeclared_randomness(manifest: WS1Manifest | None = None) -> None:
    pol = (manifest or load_manifest()).raw["stochastic_policy"]
    if pol.get("dropout") not in (0, 0.0) or not pol.get("sampling_is_seeded"):
        raise WorkloadError("the workload declares randomness that validation cannot replay")


def _digest(payload: Any) -> str:
    return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":")).encode("utf-8")).hexdigest()


def fixture_hash(manifest: WS1Manifest | None = None) -> str:
    return _digest((manifest or load_manifest()).fixtures)


def _manifest_identity_payload(raw: Mapping[str, Any]) -> dict[str, Any]:
    return {k: raw[k] for k in ("workload_id", "seed", "model_identity", "chain_semantics", "primary_matrix", "fixtures")}


def manifest_identity_hash(raw: Mapping[str, Any]) -> str:
    return _digest(_manifest_identity_payload(raw))


def weight_snapshot_hash(shards: Sequence[Mapping[str, Any]]) -> str:
    """Identity of a weight snapshot from its shard table (name, shape, dtype, sha256), independent of shard order."""
    return _digest(sorted(({k: s[k] for k in ("name", "shape", "dtype", "sha256")} for s in shards), key=lambda s: s["name"]))


def reference_payload(manifest: WS1Manifest | None = None, *, weights: Sequence[Mapping[str, Any]] = ()) -> dict[str, Any]:
    """What a stored reference artifact records next to its tensors so that a later run can refuse to compare against
    a reference of another workload, fixture set or weight snapshot."""
    m = manifest or load_manifest()
    return {"workload_id": m.workload_id, "seed": m.seed, "manifest_identity_sha256": manifest_identity_hash(m.raw),
            "fixture_sha256": fixture_hash(m), "weight_snapshot_sha256": weight_snapshot_hash(weights) if weights else None,
            "model_id": m.model_identity["model_id"]}


# ------------------------------------------------------------------------------------ tensor-level helpers
def chunk_batch(ids: torch.Tensor, size: int):
    return [ids[i:i + size] for i in range(0, ids.shape[0], size)], lambda outs: torch.cat(outs)


def pad_batch(ids: torch.Tensor, pad_to: int, side: str = "right", pad_id: int = 0):
    B, S = ids.shape
    if pad_to < S:
        raise ValueError("pad_to must be at least the sequence length")
    out = ids.new_full((B, pad_to), pad_id)
    mask = torch.zeros(B, pad_to, dtype=torch.bool)
    if side == "right":
        out[:, :S], mask[:, :S] = ids, True
        return out, mask, lambda r: r[:, :r.shape[1] - (pad_to - S)]
    out[:, pad_to - S:], mask[:, pad_to - S:] = ids, True
    return out, mask, lambda r: r[:, pad_to - S:]


def pack_batch(ids: torch.Tensor, lengths: torch.Tensor):
    flat = torch.cat([ids[b, : int(lengths[b])] for b in range(ids.shape[0])])
    cu = torch.cat([lengths.new_zeros(1), lengths.cumsum(0)])
    return flat, cu


__all__ = ["ChunkPlan", "LogicalBatch", "LogicalSample", "LogicalToken", "PaddedBatch", "PhysicalLayout",
           "SingletonAggregatePlan", "WS1Manifest", "WorkloadError", "apply_chunking", "apply_packing", "apply_padding",
           "assert_no_undeclared_randomness", "batch_permutation_from_manifest", "build_chunk_plan", "build_logical_batch",
           "case_ids", "chunk_batch", "chunk_plan_from_manifest", "default_manifest_path", "fixture_hash", "get_case",
           "get_matrix_cell", "load_manifest", "manifest_identity_hash", "matrix_cell_ids", "pack_batch", "pad_batch",
           "permute_batch", "profile_missing_required_nodes", "profile_required_nodes", "reference_payload",
           "restore_logical_order", "restore_logical_order_from_padded", "same_logical_multiset", "singleton_aggregate_plan",
           "validate_manifest", "weight_snapshot_hash"]
