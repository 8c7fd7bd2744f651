"""Train -> rollout weight-sync bridge.

The public surface follows the reference's module of the same path
(rl_engine/integrations/common/weights.py): the same dataclasses with the same field names and
value formats (``TensorDescriptor.name``, ``dtype == "torch.bfloat16"``, ``created_at``,
``metadata["layout"]`` as a mapping), the same exception classes, the same keyword-only bridge
constructors (``source_worker``, ``source_rank``), ``publish(model, *, weight_version, metadata)``,
``make_weight_bridge`` and the vLLM install adapters -- a manifest produced by the reference loads
here and the other way round.

Protocol: a publisher turns a model (or a name -> tensor mapping) into a ``WeightUpdateManifest``
{update_id, source_worker, source_rank, weight_version (strictly increasing), transport,
tensors{name -> TensorDescriptor}, created_at, metadata}; the consumer ``import_update``s it
(descriptors and checksums are verified against what the transport actually holds), installs the
tensors, then ``acknowledge``s or ``reject``s; a rejected or failed update leaves the previous
version active; ``release`` drops the transport's resources.

Transports:
  * ``LocalTensorCopyBridge``     ("local-clone")   same process, tensors are cloned
  * ``SharedMemoryTensorBridge``  ("shared-memory") POSIX shared memory, cross-process, CPU tensors
  * ``CUDAVMMTensorBridge``       ("cuda-vmm")      one cuMemCreate allocation, 256-byte packing, its
                                  POSIX descriptor handed over a unix socket; the importer maps the
                                  same physical memory (csrc/runtime/vmm.cu)
  * ``IPCWeightBridge``           ("cuda-ipc")      legacy cudaIpc handle of one packed buffer
  * ``NVLinkPushBridge``          ("nvlink-push")   ONE kernel pushes the trainer's flat shard into
                                  the rollout engines' buffers on peer GPUs and changes the tensor-
                                  parallel layout on the way (csrc/collectives/weight_sync.cu); the
                                  only transport that accepts a tensor-parallel layout
Extras over the reference, all with defaults: ``TensorDescriptor.offset`` (byte offset inside a
packed transport buffer), ``sha256 == ""`` meaning "not checksummed", JSON (de)serialisation of
manifests.
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import os
import socket
import tempfile
import threading
import time
import uuid
from dataclasses import asdict, dataclass, field
from multiprocessing import shared_memory
from typing import Any, Callable, Mapping, Optional, Protocol, runtime_checkable

import torch

_SUPPORTED_LAYOUT_KINDS = {"full-state", "replicated"}
_LAYOUT_AWARE_KINDS = {"tp-canonical"}          # accepted only by transports that reshard (NVLink push)
_BRIDGE_METADATA_KEY = "rl_kernel_bridge"
_PACK_ALIGN = 256


# ------------------------------------------------------------------------------- exceptions
class WeightBridgeError(RuntimeError):
    """Base class of every weight-bridge failure."""


class WeightBridgeUnavailableError(WeightBridgeError):
    """The requested transport or layout is not supported in this runtime."""


class WeightManifestValidationError(WeightBridgeError):
    """A manifest is incomplete or does not match what the transport holds."""


class WeightUpdateRejectedError(WeightBridgeError):
    """An update cannot be imported or acknowledged (unknown, rejected or released)."""


WeightSyncError = WeightBridgeError       # earlier name of the base class


# ------------------------------------------------------------------------------- layout
@dataclass(frozen=True)
class WeightLayout:
    """How the published state is laid out (rl_engine/integrations/common/weights.py:32-107)."""

    kind: str = "full-state"
    world_size: int = 1
    rank: int = 0
    tensor_parallel_size: int = 1
    data_parallel_size: int = 1
    zero_stage: int = 0
    node_count: int = 1
    rdma_enabled: bool = False

    @classmethod
    def from_metadata(cls, metadata: Optional[Mapping[str, Any]]) -> "WeightLayout":
        if metadata is None:
            return cls()
        raw = metadata.get("layout", {})
        if raw is None:
            return cls()
        if isinstance(raw, str):                 # shorthand: {"layout": "full-state"}
            raw = {"kind": raw}
        if not isinstance(raw, Mapping):
            raise WeightManifestValidationError("weight layout metadata must be a mapping")
        node_count = raw.get("node_count", metadata.get("node_count", 1))
        return cls(kind=str(raw.get("kind", "full-state")), world_size=int(raw.get("world_size", 1)),
                   rank=int(raw.get("rank", 0)), tensor_parallel_size=int(raw.get("tensor_parallel_size", 1)),
                   data_parallel_size=int(raw.get("data_parallel_size", 1)), zero_stage=int(raw.get("zero_stage", 0)),
                   node_count=int(node_count), rdma_enabled=bool(raw.get("rdma_enabled", False)))

    def to_metadata(self) -> dict[str, Any]:
        return asdict(self)

    def validate_supported(self, *, layout_aware: bool = False) -> None:
        kinds = _SUPPORTED_LAYOUT_KINDS | (_LAYOUT_AWARE_KINDS if layout_aware else set())
        if self.kind not in kinds:
            raise WeightBridgeUnavailableError(
                f"weight layout {self.kind!r} is not supported by this transport (supported: {sorted(kinds)}); "
                "publish a gathered full-state update or use the layout-aware NVLink push transport")
        if self.tensor_parallel_size != 1 and not layout_aware:
            raise WeightBridgeUnavailableError(
                "tensor-parallel weight layouts need the layout-aware transport (NVLinkPushBridge); "
                "this transport moves complete tensors only")
        if self.node_count != 1 or self.rdma_enabled:
            raise WeightBridgeUnavailableError("multi-node / RDMA weight transport is not implemented: one node only")
        if self.world_size < 1 or self.rank < 0 or self.rank >= self.world_size:
            raise WeightManifestValidationError(f"invalid layout rank/world_size: {self.rank}/{self.world_size}")
        if self.data_parallel_size < 1:
            raise WeightManifestValidationError("data_parallel_size must be >= 1")


def _validated_manifest_metadata(metadata: Optional[Mapping[str, Any]], *, layout_aware: bool = False) -> dict[str, Any]:
    md = dict(metadata or {})
    layout = WeightLayout.from_metadata(md)
    layout.validate_supported(layout_aware=layout_aware)
    md["layout"] = layout.to_metadata()
    return md


# ------------------------------------------------------------------------------- manifest
def _tensor_sha256(tensor: torch.Tensor) -> str:
    b = tensor.detach().contiguous().cpu()
    return hashlib.sha256(b.view(torch.uint8).numpy().tobytes()).hexdigest()


tensor_sha256 = _tensor_sha256


def _dtype_from_name(name: str) -> torch.dtype:
    dt = getattr(torch, str(name).removeprefix("torch."), None)
    if not isinstance(dt, torch.dtype):
        raise WeightManifestValidationError(f"unknown tensor dtype {name!r}")
    return dt


@dataclass(frozen=True)
class TensorDescriptor:
    """Transport-independent metadata of one tensor of an update."""

    name: str
    shape: tuple[int, ...]
    dtype: str                    # str(torch.dtype), e.g. "torch.bfloat16"
    stride: tuple[int, ...]
    device: str
    numel: int
    nbytes: int
    sha256: str = ""              # "" = the transport did not checksum this tensor
    offset: int = 0               # byte offset inside a packed transport buffer

    @classmethod
    def from_tensor(cls, name: str, tensor: torch.Tensor, *, checksum: bool = True, offset: int = 0) -> "TensorDescriptor":
        return cls(name=name, shape=tuple(int(d) for d in tensor.shape), dtype=str(tensor.dtype),
                   stride=tuple(int(s) for s in tensor.stride()), device=str(tensor.device), numel=int(tensor.numel()),
                   nbytes=int(tensor.numel() * tensor.element_size()),
                   sha256=_tensor_sha256(tensor) if checksum else "", offset=int(offset))

    def torch_dtype(self) -> torch.dtype:
        return _dtype_from_name(self.dtype)


@dataclass(frozen=True)
class WeightUpdateManifest:
    """Immutable public record of one complete published update."""

    update_id: str
    source_worker: str
    source_rank: int
    weight_version: int
    transport: str
    tensors: Mapping[str, TensorDescriptor]
    created_at: float
    metadata: Mapping[str, Any] = field(default_factory=dict)

    @property
    def tensor_count(self) -> int:
        return len(self.tensors)

    @property
    def total_nbytes(self) -> int:
        return sum(d.nbytes for d in self.tensors.values())

    def to_json(self) -> str:
        d = {"update_id": self.update_id, "source_worker": self.source_worker, "source_rank": self.source_rank,
             "weight_version": self.weight_version, "transport": self.transport, "created_at": self.created_at,
             "tensors": {k: asdict(v) for k, v in self.tensors.items()}, "metadata": dict(self.metadata)}
        return json.dumps(d, sort_keys=True)

    @classmethod
    def from_json(cls, text: str) -> "WeightUpdateManifest":
        return cls.from_dict(json.loads(text))

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "WeightUpdateManifest":
        """Accepts the reference's field names as they are (``name``, ``created_at``,
        ``"torch.float32"``) and fills this module's extras with their defaults."""
        tensors = {}
        for key, v in d["tensors"].items():
            v = dict(v)
            tensors[key] = TensorDescriptor(name=str(v.get("name", key)), shape=tuple(v["shape"]),
                                            dtype=str(_dtype_from_name(v["dtype"])), stride=tuple(v.get("stride", ())),
                                            device=str(v.get("device", "cpu")), numel=int(v["numel"]), nbytes=int(v["nbytes"]),
                                            sha256=str(v.get("sha256") or ""), offset=int(v.get("offset", 0)))
        return cls(update_id=str(d["update_id"]), source_worker=str(d["source_worker"]), source_rank=int(d["source_rank"]),
                   weight_version=int(d["weight_version"]), transport=str(d["transport"]), tensors=tensors,
                   created_at=float(d.get("created_at", d.get("created_ts", 0.0))), metadata=dict(d.get("metadata", {})))


# ------------------------------------------------------------------------------- protocols
@runtime_checkable
class WeightConsumer(Protocol):
    def import_update(self, manifest: WeightUpdateManifest) -> Mapping[str, torch.Tensor]: ...

    def acknowledge(self, update_id: str) -> None: ...

    def reject(self, update_id: str, reason: str) -> None: ...

    def release(self, update_id: str) -> None: ...


@runtime_checkable
class WeightBridge(WeightConsumer, Protocol):
    def publish(self, model: Any, *, weight_version: int, metadata: Optional[Mapping[str, Any]] = None
                ) -> WeightUpdateManifest: ...


@runtime_checkable
class WeightInstallAdapter(Protocol):
    def install(self, manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor]) -> None: ...

    def release(self, update_id: str) -> None: ...


class CallableInstallAdapter:
    """``WeightInstallAdapter`` from two callables: ``install_fn(manifest, tensors)`` must raise on failure."""

    def __init__(self, install_fn: Callable[[WeightUpdateManifest, Mapping[str, torch.Tensor]], None],
                 release_fn: Optional[Callable[[str], None]] = None):
        self._install, self._release = install_fn, release_fn
        self.active_weight_version: Optional[int] = None
        self.active_update_id: Optional[str] = None

    def install(self, manifest, tensors) -> None:
        self._install(manifest, tensors)
        self.active_weight_version, self.active_update_id = manifest.weight_version, manifest.update_id

    def release(self, update_id: str) -> None:
        if self._release is not None:
            self._release(update_id)
        if self.active_update_id == update_id:
            self.active_update_id = None


class WeightPublisher:
    """Publisher facade of a training worker: keeps the history and notifies a listener.  Any bridge
    is itself a publisher in the reference's sense (``publish(model, *, weight_version, metadata)``)."""

    def __init__(self, bridge, on_publish: Optional[Callable[[WeightUpdateManifest], None]] = None):
        self.bridge, self.on_publish = bridge, on_publish
        self.history: list[WeightUpdateManifest] = []

    def publish(self, model, weight_version: int, metadata: Optional[Mapping[str, Any]] = None) -> WeightUpdateManifest:
        m = self.bridge.publish(model, weight_version=weight_version, metadata=metadata)
        self.history.append(m)
        if self.on_publish:
            self.on_publish(m)
        return m

    def release(self, update_id: str) -> None:
        self.bridge.release(update_id)


# ------------------------------------------------------------------------------- local clone
@dataclass
class _LocalUpdateRecord:
    manifest: WeightUpdateManifest
    tensors: dict[str, torch.Tensor]
    state: str = "published"            # published -> imported -> acknowledged | rejected; released = gone
    import_count: int = 0
    rejection_reason: Optional[str] = None
    resources: dict = field(default_factory=dict)


class UpdateState:
    PUBLISHED, IMPORTED, ACKNOWLEDGED, REJECTED, RELEASED = "published", "imported", "acknowledged", "rejected", "released"


def _state_tensors(model) -> dict[str, torch.Tensor]:
    """``model``: an nn.Module (its state_dict) or a name -> tensor mapping."""
    src = model.state_dict() if hasattr(model, "state_dict") else model
    return {str(k): v for k, v in src.items() if isinstance(v, torch.Tensor)}


class LocalTensorCopyBridge:
    """Same-process transport: tensors are cloned at publish and again at import.  It carries the
    whole versioned publish / import / acknowledge / reject / release lifecycle that the zero-copy
    transports inherit."""

    transport = "local-clone"
    layout_aware = False
    checksum = True

    def __init__(self, *, source_worker: str = "local-training", source_rank: int = 0):
        self.source_worker, self.source_rank = source_worker, int(source_rank)
        self._updates: dict[str, _LocalUpdateRecord] = {}
        self._lock = threading.RLock()
        self._latest_published_weight_version = -1
        self.active_weight_version: Optional[int] = None
        self.active_update_id: Optional[str] = None
        self.rejections: dict[str, str] = {}

    # ---- publisher side
    def _begin_publish(self, weight_version: int, metadata) -> tuple[int, dict]:
        md = _validated_manifest_metadata(metadata, layout_aware=self.layout_aware)
        version = int(weight_version)
        if version <= self._latest_published_weight_version:
            raise WeightManifestValidationError(
                f"weight_version must increase monotonically (got {version}, latest {self._latest_published_weight_version})")
        return version, md

    def _finish_publish(self, version: int, md: dict, descriptors, tensors, resources=None) -> WeightUpdateManifest:
        m = WeightUpdateManifest(update_id=str(uuid.uuid4()), source_worker=self.source_worker, source_rank=self.source_rank,
                                 weight_version=version, transport=self.transport, tensors=descriptors,
                                 created_at=time.perf_counter(), metadata=md)
        with self._lock:
            self._updates[m.update_id] = _LocalUpdateRecord(m, tensors, resources=resources or {})
            self._latest_published_weight_version = version
        return m

    def publish(self, model, weight_version: Optional[int] = None, metadata: Optional[Mapping[str, Any]] = None
                ) -> WeightUpdateManifest:
        if weight_version is None:
            raise TypeError("publish() needs weight_version")
        version, md = self._begin_publish(weight_version, metadata)
        tensors = {k: v.detach().clone(memory_format=torch.preserve_format) for k, v in _state_tensors(model).items()}
        if not tensors:
            raise WeightManifestValidationError("model state_dict produced no tensors")
        descs = {k: TensorDescriptor.from_tensor(k, v, checksum=self.checksum) for k, v in tensors.items()}
        return self._finish_publish(version, md, descs, tensors)

    # ---- consumer side
    def _record_for_import(self, manifest: WeightUpdateManifest) -> _LocalUpdateRecord:
        rec = self._require_record(manifest.update_id)
        if rec.state == "rejected":
            raise WeightUpdateRejectedError(f"weight update {manifest.update_id} was rejected: {rec.rejection_reason}")
        self._validate_manifest(rec, manifest)
        rec.import_count += 1
        if rec.state == "published":
            rec.state = "imported"
        return rec

    def import_update(self, manifest: WeightUpdateManifest) -> Mapping[str, torch.Tensor]:
        rec = self._record_for_import(manifest)
        return {k: v.detach().clone(memory_format=torch.preserve_format) for k, v in rec.tensors.items()}

    def acknowledge(self, update_id: str) -> None:
        rec = self._require_record(update_id)
        if rec.state == "rejected":
            raise WeightUpdateRejectedError(f"cannot acknowledge rejected update {update_id}: {rec.rejection_reason}")
        if rec.import_count == 0:
            raise WeightUpdateRejectedError(f"cannot acknowledge update {update_id} before import_update succeeds")
        rec.state = "acknowledged"
        self.active_weight_version, self.active_update_id = rec.manifest.weight_version, update_id

    def reject(self, update_id: str, reason: str) -> None:
        rec = self._require_record(update_id)
        if rec.state == "acknowledged":
            raise WeightUpdateRejectedError(f"cannot reject acknowledged update {update_id}")
        rec.state, rec.rejection_reason = "rejected", reason
        self.rejections[update_id] = reason

    def release(self, update_id: str) -> None:
        with self._lock:
            rec = self._updates.pop(update_id, None)
        if rec is None:
            return
        self._free(rec)
        rec.tensors.clear()
        rec.state = "released"
        if self.active_update_id == update_id:
            self.active_update_id = None

    def update_status(self, update_id: str) -> str:
        rec = self._updates.get(update_id)
        return "released" if rec is None else rec.state

    state = update_status

    def get_manifest(self, update_id: str) -> WeightUpdateManifest:
        return self._require_record(update_id).manifest

    def debug_tensor_data_ptrs(self, update_id: str) -> Mapping[str, int]:
        return {k: int(v.data_ptr()) for k, v in self._require_record(update_id).tensors.items()}

    def close(self) -> None:
        for uid in list(self._updates):
            self.release(uid)

    def _free(self, rec: _LocalUpdateRecord) -> None:      # transports that own buffers override
        pass

    def _require_record(self, update_id: str) -> _LocalUpdateRecord:
        try:
            return self._updates[update_id]
        except KeyError as exc:
            raise WeightUpdateRejectedError(f"unknown weight update {update_id}") from exc

    def _validate_manifest(self, rec: _LocalUpdateRecord, manifest: WeightUpdateManifest) -> None:
        exp = rec.manifest
        WeightLayout.from_metadata(manifest.metadata).validate_supported(layout_aware=self.layout_aware)
        if manifest.transport != exp.transport:
            raise WeightManifestValidationError(f"transport mismatch: expected {exp.transport}, got {manifest.transport}")
        if manifest.weight_version != exp.weight_version:
            raise WeightManifestValidationError(
                f"weight_version mismatch: expected {exp.weight_version}, got {manifest.weight_version}")
        if set(manifest.tensors) != set(exp.tensors):
            raise WeightManifestValidationError(
                f"tensor manifest mismatch: missing={sorted(set(exp.tensors) - set(manifest.tensors))}, "
                f"extra={sorted(set(manifest.tensors) - set(exp.tensors))}")
        for name, d in exp.tensors.items():
            if manifest.tensors[name] != d:
                raise WeightManifestValidationError(f"tensor descriptor mismatch for {name}")
            if not d.sha256 or name not in rec.tensors:
                continue
            t = rec.tensors[name]
            if tuple(t.shape) != d.shape or str(t.dtype) != d.dtype:
                raise WeightManifestValidationError(f"stored tensor descriptor mismatch for {name}")
            got = _tensor_sha256(t)
            if got != d.sha256:
                raise WeightManifestValidationError(f"tensor checksum mismatch for {name}: expected {d.sha256}, got {got}")


# ------------------------------------------------------------------------------- packing
def _pack_plan(tensors: Mapping[str, torch.Tensor], *, checksum: bool) -> tuple[dict[str, TensorDescriptor], int]:
    """Every tensor contiguous at a 256-byte aligned offset of one buffer."""
    descs, off = {}, 0
    for k, v in tensors.items():
        c = v.detach().contiguous()
        d = TensorDescriptor.from_tensor(k, c, checksum=checksum, offset=off)
        descs[k] = d
        off = (off + d.nbytes + _PACK_ALIGN - 1) // _PACK_ALIGN * _PACK_ALIGN
    return descs, max(off, _PACK_ALIGN)


def _views_of_packed(packed: torch.Tensor, descs: Mapping[str, TensorDescriptor]) -> dict[str, torch.Tensor]:
    return {k: packed[d.offset:d.offset + d.nbytes].view(d.torch_dtype()).view(d.shape) for k, d in descs.items()}


# ------------------------------------------------------------------------------- shared memory
class SharedMemoryTensorBridge(LocalTensorCopyBridge):
    """Same-node transport through one POSIX shared-memory segment per update; an importer in
    another process attaches by name and gets tensors that alias the segment."""

    transport = "shared-memory"

    def publish(self, model, weight_version: Optional[int] = None, metadata=None) -> WeightUpdateManifest:
        if weight_version is None:
            raise TypeError("publish() needs weight_version")
        version, md = self._begin_publish(weight_version, metadata)
        cpu = {k: v.detach().contiguous().cpu() for k, v in _state_tensors(model).items()}
        if not cpu:
            raise WeightManifestValidationError("model state_dict produced no tensors")
        descs, total = _pack_plan(cpu, checksum=self.checksum)
        seg = shared_memory.SharedMemory(create=True, size=total)
        packed = torch.frombuffer(seg.buf, dtype=torch.uint8, count=total)
        for k, v in cpu.items():
            d = descs[k]
            packed[d.offset:d.offset + d.nbytes].copy_(v.view(torch.uint8).reshape(-1))
        md[_BRIDGE_METADATA_KEY] = {"format": "posix-shm-v1", "shm_name": seg.name, "shm_bytes": total}
        return self._finish_publish(version, md, descs, _views_of_packed(packed, descs), {"segment": seg, "packed": packed})

    def import_update(self, manifest: WeightUpdateManifest) -> Mapping[str, torch.Tensor]:
        if manifest.update_id not in self._updates:
            self._attach(manifest)
        rec = self._record_for_import(manifest)
        return dict(rec.tensors)          # aliases of the shared segment

    def _attach(self, manifest: WeightUpdateManifest) -> None:
        info = manifest.metadata.get(_BRIDGE_METADATA_KEY)
        if manifest.transport != self.transport or not isinstance(info, Mapping) or "shm_name" not in info:
            raise WeightManifestValidationError("manifest does not describe a shared-memory update")
        try:
            seg = shared_memory.SharedMemory(name=info["shm_name"])
        except FileNotFoundError as exc:
            raise WeightUpdateRejectedError(f"shared-memory segment {info['shm_name']} is gone") from exc
        packed = torch.frombuffer(seg.buf, dtype=torch.uint8, count=int(info["shm_bytes"]))
        self._updates[manifest.update_id] = _LocalUpdateRecord(manifest, _views_of_packed(packed, manifest.tensors),
                                                              resources={"segment": seg, "packed": packed, "attached": True})

    def _free(self, rec: _LocalUpdateRecord) -> None:
        seg = rec.resources.pop("segment", None)
        rec.resources.pop("packed", None)
        rec.tensors.clear()
        if seg is None:
            return
        try:
            seg.close()
        except BufferError:
            pass                          # a tensor view is still alive somewhere; the OS frees the mapping at exit
        if not rec.resources.get("attached"):
            try:
                seg.unlink()
            except FileNotFoundError:
                pass


# ------------------------------------------------------------------------------- device pointer helper
class _DevicePtrView:
    """Exposes a raw device pointer to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _native():
    from rl_kernel_b200.backends import extension

    return extension, extension.load()


# ------------------------------------------------------------------------------- CUDA VMM + fd broker
class CUDAVMMTensorBridge(LocalTensorCopyBridge):
    """Zero-copy same-GPU transport across processes: the state is packed into one
    virtual-memory-management allocation whose POSIX descriptor a small broker thread hands to
    importers over a unix socket (SCM_RIGHTS); the importer maps the same physical memory and
    returns tensors that alias it."""

    transport = "cuda-vmm"

    def __init__(self, *, source_worker: str = "local-training", source_rank: int = 0, device: torch.device | str | None = None,
                 socket_dir: Optional[str] = None):
        super().__init__(source_worker=source_worker, source_rank=source_rank)
        self.device = torch.device(device) if device is not None else None
        self._socket_dir = socket_dir

    def _device(self) -> torch.device:
        if self.device is None:
            if not torch.cuda.is_available():
                raise WeightBridgeUnavailableError("the cuda-vmm transport needs a CUDA device")
            self.device = torch.device("cuda", torch.cuda.current_device())
        return self.device

    def publish(self, model, weight_version: Optional[int] = None, metadata=None) -> WeightUpdateManifest:
        if weight_version is None:
            raise TypeError("publish() needs weight_version")
        version, md = self._begin_publish(weight_version, metadata)
        state = _state_tensors(model)
        if not state:
            raise WeightManifestValidationError("model state_dict produced no tensors")
        dev = self._device()
        ext, lib = _native()
        with torch.cuda.device(dev):
            if not lib.rlk_vmm_supported():
                raise WeightBridgeUnavailableError("this driver / device offers no POSIX-descriptor virtual memory")
            descs, total = _pack_plan(state, checksum=self.checksum)
            ptr, mapped, handle, fd = ctypes.c_void_p(0), ctypes.c_longlong(0), ctypes.c_ulonglong(0), ctypes.c_int(-1)
            ext.check(lib.rlk_vmm_create(ctypes.c_longlong(total), ctypes.byref(ptr), ctypes.byref(mapped),
                                         ctypes.byref(handle), ctypes.byref(fd)), "vmm_create")
            packed = torch.as_tensor(_DevicePtrView(ptr.value, mapped.value), device=dev)
            for k, v in state.items():
                d = descs[k]
                packed[d.offset:d.offset + d.nbytes].copy_(v.detach().contiguous().view(torch.uint8).reshape(-1))
            torch.cuda.synchronize(dev)
            descs = {k: TensorDescriptor(d.name, d.shape, d.dtype, d.stride, str(dev), d.numel, d.nbytes, d.sha256, d.offset)
                     for k, d in descs.items()}
        update_hint = uuid.uuid4().hex[:12]
        path, stop = self._start_fd_broker(update_hint, fd.value)
        md[_BRIDGE_METADATA_KEY] = {"format": "cuda-vmm-fd-v1", "socket_path": path, "mapped_nbytes": int(mapped.value),
                                    "device_index": int(dev.index or 0), "pid": os.getpid()}
        res = {"ptr": ptr.value, "mapped": int(mapped.value), "handle": int(handle.value), "fd": fd.value, "owner": True,
               "broker_stop": stop, "socket_path": path, "packed": packed}
        return self._finish_publish(version, md, descs, _views_of_packed(packed, descs), res)

    def _start_fd_broker(self, tag: str, fd: int) -> tuple[str, threading.Event]:
        """Serves the allocation's descriptor to whoever connects, until the update is released."""
        d = self._socket_dir or tempfile.gettempdir()
        path = os.path.join(d, f"rlk-vmm-{os.getpid()}-{tag}.sock")
        srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        srv.bind(path)
        srv.listen(8)
        srv.settimeout(0.2)
        stop = threading.Event()

        def serve():
            try:
                while not stop.is_set():
                    try:
                        conn, _ = srv.accept()
                    except socket.timeout:
                        continue
                    with conn:
                        socket.send_fds(conn, [b"fd"], [fd])
            finally:
                srv.close()
                try:
                    os.unlink(path)
                except FileNotFoundError:
                    pass

        threading.Thread(target=serve, name=f"rlk-vmm-broker-{tag}", daemon=True).start()
        return path, stop

    def import_update(self, manifest: WeightUpdateManifest) -> Mapping[str, torch.Tensor]:
        if manifest.update_id not in self._updates:
            self._attach(manifest)
        rec = self._record_for_import(manifest)
        return dict(rec.tensors)          # aliases of the publisher's allocation

    def _attach(self, manifest: WeightUpdateManifest) -> None:
        info = manifest.metadata.get(_BRIDGE_METADATA_KEY)
        if manifest.transport != self.transport or not isinstance(info, Mapping) or info.get("format") != "cuda-vmm-fd-v1":
            raise WeightManifestValidationError("manifest does not describe a cuda-vmm update")
        dev = torch.device("cuda", int(info["device_index"]))
        ext, lib = _native()
        with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as s:
            s.settimeout(30)
            try:
                s.connect(info["socket_path"])
            except OSError as exc:
                raise WeightUpdateRejectedError(f"the publisher's descriptor broker is gone: {exc}") from exc
            _, fds, _, _ = socket.recv_fds(s, 16, 1)
        if not fds:
            raise WeightUpdateRejectedError("the descriptor broker sent no descriptor")
        ptr, handle = ctypes.c_void_p(0), ctypes.c_ulonglong(0)
        with torch.cuda.device(dev):
            try:
                ext.check(lib.rlk_vmm_import(ctypes.c_int(fds[0]), ctypes.c_longlong(int(info["mapped_nbytes"])),
                                             ctypes.byref(ptr), ctypes.byref(handle)), "vmm_import")
            finally:
                os.close(fds[0])
        packed = torch.as_tensor(_DevicePtrView(ptr.value, int(info["mapped_nbytes"])), device=dev)
        res = {"ptr": ptr.value, "mapped": int(info["mapped_nbytes"]), "handle": int(handle.value), "owner": False,
               "packed": packed}
        self._updates[manifest.update_id] = _LocalUpdateRecord(manifest, _views_of_packed(packed, manifest.tensors), resources=res)

    def _free(self, rec: _LocalUpdateRecord) -> None:
        res = rec.resources
        if "broker_stop" in res:
            res["broker_stop"].set()
        rec.tensors.clear()
        res.pop("packed", None)
        if res.get("ptr"):
            ext, lib = _native()
            dev = self.device if self.device is not None else torch.device("cuda", 0)
            with torch.cuda.device(dev):
                lib.rlk_vmm_release(ctypes.c_void_p(res["ptr"]), ctypes.c_longlong(res["mapped"]), ctypes.c_ulonglong(res["handle"]))
            res["ptr"] = 0
        if res.get("owner") and res.get("fd", -1) >= 0:
            os.close(res["fd"])
            res["fd"] = -1


# ------------------------------------------------------------------------------- CUDA IPC (legacy handles)
class IPCWeightBridge(LocalTensorCopyBridge):
    """Packs the state into one cudaMalloc'ed buffer and exports it with a CUDA IPC handle; the
    consumer process maps it and sees the tensors without a copy."""

    transport = "cuda-ipc"

    def __init__(self, device: torch.device | str = "cuda:0", *, source_worker: str = "local-training", source_rank: int = 0):
        super().__init__(source_worker=source_worker, source_rank=source_rank)
        self.device = torch.device(device)

    def publish(self, model, weight_version: Optional[int] = None, metadata=None) -> WeightUpdateManifest:
        if weight_version is None:
            raise TypeError("publish() needs weight_version")
        version, md = self._begin_publish(weight_version, metadata)
        state = _state_tensors(model)
        ext, lib = _native()
        descs, total = _pack_plan(state, checksum=self.checksum)
        handle = ctypes.create_string_buffer(lib.rlk_symm_ipc_handle_bytes())
        ptr = ctypes.c_void_p(0)
        with torch.cuda.device(self.device):
            ext.check(lib.rlk_ipc_alloc(ctypes.c_longlong(total), ctypes.byref(ptr), handle), "ipc_alloc")
        packed = torch.as_tensor(_DevicePtrView(ptr.value, total), device=self.device)
        for k, v in state.items():
            d = descs[k]
            packed[d.offset:d.offset + d.nbytes].copy_(v.detach().contiguous().view(torch.uint8).reshape(-1))
        torch.cuda.synchronize(self.device)
        md[_BRIDGE_METADATA_KEY] = {"format": "cuda-ipc-packed-v1", "ipc_handle": handle.raw.hex(), "packed_bytes": total}
        return self._finish_publish(version, md, descs, _views_of_packed(packed, descs),
                                    {"ptr": ptr.value, "owner": True, "packed": packed})

    def import_update(self, manifest: WeightUpdateManifest) -> Mapping[str, torch.Tensor]:
        if manifest.update_id not in self._updates:
            info = manifest.metadata.get(_BRIDGE_METADATA_KEY)
            if not isinstance(info, Mapping) or "ipc_handle" not in info:
                raise WeightManifestValidationError("manifest does not describe a cuda-ipc update")
            ext, lib = _native()
            ptr = ctypes.c_void_p(0)
            with torch.cuda.device(self.device):
                ext.check(lib.rlk_ipc_open(bytes.fromhex(info["ipc_handle"]), ctypes.byref(ptr)), "ipc_open")
            packed = torch.as_tensor(_DevicePtrView(ptr.value, int(info["packed_bytes"])), device=self.device)
            self._updates[manifest.update_id] = _LocalUpdateRecord(
                manifest, _views_of_packed(packed, manifest.tensors), resources={"ptr": ptr.value, "owner": False, "packed": packed})
        rec = self._record_for_import(manifest)
        return dict(rec.tensors)

    def _free(self, rec: _LocalUpdateRecord) -> None:
        res = rec.resources
        rec.tensors.clear()
        res.pop("packed", None)
        if res.get("ptr"):
            _, lib = _native()
            (lib.rlk_ipc_free if res.get("owner") else lib.rlk_ipc_close)(ctypes.c_void_p(res["ptr"]))
            res["ptr"] = 0


CUDAIPCTensorBridge = IPCWeightBridge


# ------------------------------------------------------------------------------- NVLink push (K17)
def reshard_blocks(src_params, dst_params, dst_index: int, *, replicated_from_every_rank: bool = False) -> list[tuple]:
    """2-D block copies that move the part of ``src_params`` (a PackedParams shard of a TP group of
    size tp_s) that destination shard ``dst_params`` (TP size tp_d) needs.  Returns tuples
    (src_off, dst_off, src_pitch, dst_pitch, rows, row_bytes, dst_mask) in BYTES.
    Replicated vectors (norm gains) are sent by source rank 0 only, because every source rank holds
    the same values and all of them reach every destination; ``replicated_from_every_rank`` is for a
    source rank that is the ONLY writer of its destination (a rank that publishes into its own
    colocated rollout shard)."""
    out = []
    ts, rs = src_params.tp_size, src_params.tp_rank
    td, rd = dst_params.tp_size, dst_params.tp_rank
    for name, s in src_params.slots.items():
        d = dst_params.slots[name]
        if len(s.shape) == 1:                                       # replicated vector
            if rs == 0 or ts == 1 or replicated_from_every_rank:
                out.append((s.offset * 2, d.offset * 2, s.numel * 2, d.numel * 2, 1, s.numel * 2, 1 << dst_index))
            continue
        row_split = name.endswith(("wqkv", "wgu")) or name in ("embed", "lm_head")
        (sr, sc), (dr, dc) = s.shape, d.shape
        if row_split:      # shards are row ranges of the full matrix
            s0, d0 = rs * sr, rd * dr
            lo, hi = max(s0, d0), min(s0 + sr, d0 + dr)
            if lo < hi:
                out.append(((s.offset + (lo - s0) * sc) * 2, (d.offset + (lo - d0) * dc) * 2, sc * 2, dc * 2,
                            hi - lo, sc * 2, 1 << dst_index))
        else:              # wo / wd: shards are column ranges
            s0, d0 = rs * sc, rd * dc
            lo, hi = max(s0, d0), min(s0 + sc, d0 + dc)
            if lo < hi:
                out.append(((s.offset + (lo - s0)) * 2, (d.offset + (lo - d0)) * 2, sc * 2, dc * 2, sr, (hi - lo) * 2,
                            1 << dst_index))
    return out


class NVLinkPushBridge(LocalTensorCopyBridge):
    """The trainer pushes its flat bf16 shard into up to 8 destination buffers (peer-mapped rollout
    parameter buffers) with one kernel; the block list encodes the layout change.  The only
    transport that accepts a tensor-parallel ("tp-canonical") layout."""

    transport = "nvlink-push"
    layout_aware = True
    checksum = False

    def __init__(self, src_params, device: torch.device, *, source_worker: str = "local-training", source_rank: int = 0):
        super().__init__(source_worker=source_worker, source_rank=source_rank)
        self.src, self.device = src_params, device
        self._targets: list[tuple[int, int | None]] = []   # (base pointer, flag pointer)
        self._blocks: list[tuple] = []
        self._descs = None
        self._counter = torch.zeros(1, dtype=torch.int32, device=device)

    def add_target(self, dst_params, base_ptr: int | None = None, version_flag_ptr: int | None = None, *,
                   sole_writer: bool = False) -> int:
        """Register a destination shard; ``base_ptr`` is its flat buffer as mapped in THIS process
        (defaults to dst_params.flat for same-process targets).  ``sole_writer``: no other source
        rank pushes into this destination, so this rank also sends the replicated vectors."""
        idx = len(self._targets)
        if idx >= 8:
            raise WeightBridgeError("at most 8 destinations per push")
        self._targets.append((base_ptr if base_ptr is not None else dst_params.flat.data_ptr(), version_flag_ptr))
        self._blocks += reshard_blocks(self.src, dst_params, idx, replicated_from_every_rank=sole_writer)
        self._descs = None
        return idx

    def _desc_tensor(self) -> torch.Tensor:
        if self._descs is None:
            rows = []
            for (so, do, sp, dp, r, rb, mask) in self._blocks:
                if rb % 16 or so % 16 or do % 16 or (r > 1 and (sp % 16 or dp % 16)):
                    raise WeightBridgeError("weight blocks must be 16-byte aligned")
                rows.append([so, do, sp, dp, r | (rb << 32), mask])
            self._descs = torch.tensor(rows, dtype=torch.int64).to(self.device).contiguous()
        return self._descs

    def publish(self, model=None, weight_version: Optional[int] = None, metadata=None) -> WeightUpdateManifest:
        """``model`` is ignored (the source is the PackedParams given at construction); for
        convenience ``publish(7)`` is read as ``publish(weight_version=7)``."""
        from rl_kernel_b200.backends import native as nv

        if weight_version is None and isinstance(model, int):
            model, weight_version = None, model
        if weight_version is None:
            raise TypeError("publish() needs weight_version")
        md_in = dict(metadata or {})
        md_in.setdefault("layout", {"kind": "tp-canonical", "tensor_parallel_size": int(self.src.tp_size),
                                    "world_size": int(self.src.tp_size), "rank": int(self.src.tp_rank)})
        version, md = self._begin_publish(weight_version, md_in)
        ext, lib = _native()
        descs = self._desc_tensor()
        n = len(self._targets)
        bases = (ctypes.c_void_p * n)(*[t[0] for t in self._targets])
        flags = (ctypes.c_void_p * n)(*[t[1] or 0 for t in self._targets])
        ext.check(lib.rlk_weight_push(ext.ptr(self.src.flat), ext.ptr(descs), ctypes.c_int(descs.shape[0]), bases,
                                      flags, ctypes.c_int(n), ctypes.c_ulonglong(version),
                                      ext.ptr(self._counter), ext.stream_ptr(self.device)), "weight_push")
        nv._count()
        tensors = {k: TensorDescriptor(k, tuple(s.shape), "torch.bfloat16", (), str(self.device), s.numel, s.numel * 2, "",
                                       s.offset * 2) for k, s in self.src.slots.items()}
        md[_BRIDGE_METADATA_KEY] = {"format": "nvlink-push-v1", "targets": n, "blocks": int(descs.shape[0])}
        return self._finish_publish(version, md, tensors, {})

    def import_update(self, manifest: WeightUpdateManifest) -> Mapping[str, torch.Tensor]:
        self._record_for_import(manifest)
        return {}                         # the data is already in the destination buffers


# ------------------------------------------------------------------------------- vLLM install adapters
def _check_tensor_set(manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor], what: str) -> None:
    if set(tensors) != set(manifest.tensors):
        raise WeightManifestValidationError(
            f"{what} tensor set mismatch: missing={sorted(set(manifest.tensors) - set(tensors))}, "
            f"extra={sorted(set(tensors) - set(manifest.tensors))}")
    for name, d in manifest.tensors.items():
        t = tensors[name]
        if tuple(int(x) for x in t.shape) != tuple(d.shape):
            raise WeightManifestValidationError(f"{what} tensor shape mismatch for {name}: expected {d.shape}, got {tuple(t.shape)}")
        if str(t.dtype) != d.dtype:
            raise WeightManifestValidationError(f"{what} tensor dtype mismatch for {name}: expected {d.dtype}, got {t.dtype}")


def _engine_rpc(engine, method: str):
    """``engine.<method>(**kw)`` if it exists, else ``collective_rpc(method, kwargs=kw)`` of the engine or
    of its ``llm_engine``; None when the engine offers neither."""
    fn = getattr(engine, method, None)
    if callable(fn):
        return lambda **kw: fn(**kw)
    rpc = getattr(engine, "collective_rpc", None)
    if not callable(rpc):
        rpc = getattr(getattr(engine, "llm_engine", None), "collective_rpc", None)
    if callable(rpc):
        return lambda **kw: rpc(method, kwargs=kw)
    return None


class _AdapterBase:
    def __init__(self):
        self.active_weight_version: Optional[int] = None
        self.active_update_id: Optional[str] = None

    def _activated(self, manifest) -> None:
        self.active_weight_version, self.active_update_id = manifest.weight_version, manifest.update_id

    def release(self, update_id: str) -> None:
        if self.active_update_id == update_id:
            self.active_update_id = None


class VLLMWeightInstallAdapter(_AdapterBase):
    """Installs imported tensors into a rollout engine through capability hooks instead of private
    internals (rl_engine/integrations/common/weights.py:110-189): an explicit ``install_callable``,
    else ``engine.update_weights(request_builder(manifest, tensors))``, else one of the manifest-level
    methods an engine may offer."""

    _MANIFEST_METHODS = ("install_weight_update", "update_weights_from_manifest", "load_weights_from_manifest")

    def __init__(self, engine, *, install_callable=None, request_builder=None, release_callable=None):
        super().__init__()
        self.engine = engine
        self._install_callable, self._request_builder, self._release_callable = install_callable, request_builder, release_callable

    def install(self, manifest, tensors) -> None:
        tensors = dict(tensors)
        if self._install_callable is not None:
            self._install_callable(manifest, tensors)
        elif callable(getattr(self.engine, "update_weights", None)):
            if self._request_builder is None:
                raise WeightBridgeUnavailableError(
                    "engines that expose update_weights(request) need a request_builder: the public API does not "
                    "take a raw manifest / tensor mapping")
            try:
                self.engine.update_weights(self._request_builder(manifest, tensors))
            except Exception:
                rel = getattr(self._request_builder, "release", None)
                if callable(rel):
                    rel(manifest.update_id)
                raise
        else:
            for attr in self._MANIFEST_METHODS:
                fn = getattr(self.engine, attr, None)
                if callable(fn):
                    fn(manifest, tensors)
                    break
            else:
                raise WeightBridgeUnavailableError(
                    "this engine exposes no verified hot-weight install capability; pass install_callable")
        self._activated(manifest)

    def release(self, update_id: str) -> None:
        if self._release_callable is not None:
            self._release_callable(update_id)
        rel = getattr(self._request_builder, "release", None)
        if callable(rel):
            rel(update_id)
        super().release(update_id)


class VLLMIPCWeightUpdateRequestBuilder:
    """Builds ``{"update_info": {names, dtype_names, shapes, ipc_handles, is_checkpoint_format}}`` for an
    engine's IPC ``update_weights``; the source tensors stay alive until ``release(update_id)``
    (rl_engine/integrations/common/weights.py:191-325)."""

    def __init__(self, *, is_checkpoint_format: bool = True, reduce_tensor_fn=None, gpu_uuid: Optional[str] = None):
        self.is_checkpoint_format = bool(is_checkpoint_format)
        self._reduce, self._gpu_uuid = reduce_tensor_fn, gpu_uuid
        self._keepalive: dict[str, list[torch.Tensor]] = {}

    def __call__(self, manifest, tensors) -> dict[str, Any]:
        WeightLayout.from_metadata(manifest.metadata).validate_supported()
        tensors = dict(tensors)
        _check_tensor_set(manifest, tensors, "vLLM IPC")
        uuid_ = self._gpu_uuid or self._current_gpu_uuid()
        names, dtypes, shapes, handles, keep = [], [], [], [], []
        for name in manifest.tensors:
            t = tensors[name]
            if t.device.type != "cuda":
                raise WeightBridgeUnavailableError(f"vLLM IPC weight update requires CUDA tensors; {name} is on {t.device}")
            w = t.detach().contiguous()
            keep.append(w)
            names.append(name)
            dtypes.append(str(w.dtype).split(".")[-1])
            shapes.append([int(x) for x in w.shape])
            handles.append({uuid_: self._reduce_fn()(w)})
        self._keepalive[manifest.update_id] = keep
        return {"update_info": {"names": names, "dtype_names": dtypes, "shapes": shapes, "ipc_handles": handles,
                                "is_checkpoint_format": self.is_checkpoint_format}}

    def release(self, update_id: str) -> None:
        self._keepalive.pop(update_id, None)

    def _reduce_fn(self):
        if self._reduce is not None:
            return self._reduce
        from torch.multiprocessing.reductions import reduce_tensor

        return reduce_tensor

    def _current_gpu_uuid(self) -> str:
        if not torch.cuda.is_available():
            raise WeightBridgeUnavailableError("vLLM IPC weight update requires CUDA")
        return f"GPU-{torch.cuda.get_device_properties(torch.cuda.current_device()).uuid}"


class VLLMInProcessWeightReloadAdapter(_AdapterBase):
    """Single-process engines: hands ``[(name, tensor)]`` to ``reload_weights(weights_iterator=...)``
    (rl_engine/integrations/common/weights.py:327-433)."""

    def __init__(self, engine, *, target_dtype=None, target_device=None, is_checkpoint_format: bool = True,
                 synchronize_cuda: bool = True):
        super().__init__()
        self.engine, self.target_dtype, self.target_device = engine, target_dtype, target_device
        self.is_checkpoint_format, self.synchronize_cuda = bool(is_checkpoint_format), bool(synchronize_cuda)

    def install(self, manifest, tensors) -> None:
        WeightLayout.from_metadata(manifest.metadata).validate_supported()
        tensors = dict(tensors)
        _check_tensor_set(manifest, tensors, "vLLM reload")
        weights = []
        for name in manifest.tensors:
            w = tensors[name].detach()
            if self.target_dtype is not None and w.dtype != self.target_dtype:
                w = w.to(self.target_dtype)
            if self.target_device is not None and torch.device(self.target_device) != w.device:
                w = w.to(self.target_device)
            weights.append((name, w.contiguous()))
        call = _engine_rpc(self.engine, "reload_weights")
        if call is None:
            raise WeightBridgeUnavailableError("the engine exposes neither reload_weights(...) nor collective_rpc(...)")
        try:
            call(weights_iterator=weights, is_checkpoint_format=self.is_checkpoint_format)
            if self.synchronize_cuda and torch.cuda.is_available():
                torch.cuda.synchronize()
        except Exception:
            self.active_update_id = None
            raise
        self._activated(manifest)


class VLLMCheckpointWeightReloadAdapter(_AdapterBase):
    """Multi-process engines: the worker reloads from a checkpoint path itself, nothing crosses the
    RPC boundary (rl_engine/integrations/common/weights.py:436-540)."""

    def __init__(self, engine, *, weights_path: Optional[str] = None, weights_path_resolver=None,
                 metadata_key: str = "vllm_weights_path", is_checkpoint_format: bool = True, synchronize_cuda: bool = True):
        super().__init__()
        self.engine, self.weights_path, self.weights_path_resolver = engine, weights_path, weights_path_resolver
        self.metadata_key = metadata_key
        self.is_checkpoint_format, self.synchronize_cuda = bool(is_checkpoint_format), bool(synchronize_cuda)

    def _resolve_path(self, manifest, tensors) -> str:
        if self.weights_path:
            return self.weights_path
        if self.weights_path_resolver is not None:
            p = self.weights_path_resolver(manifest, tensors)
            if p:
                return str(p)
        p = manifest.metadata.get(self.metadata_key)
        if p:
            return str(p)
        raise WeightBridgeUnavailableError(
            f"checkpoint reload needs weights_path, a weights_path_resolver or manifest.metadata[{self.metadata_key!r}]")

    def install(self, manifest, tensors) -> None:
        WeightLayout.from_metadata(manifest.metadata).validate_supported()
        tensors = dict(tensors)
        if set(tensors) != set(manifest.tensors):
            raise WeightManifestValidationError("vLLM checkpoint reload tensor set mismatch")
        path = self._resolve_path(manifest, tensors)
        call = _engine_rpc(self.engine, "reload_weights")
        if call is None:
            raise WeightBridgeUnavailableError("the engine exposes neither reload_weights(...) nor collective_rpc(...)")
        try:
            call(weights_path=path, is_checkpoint_format=self.is_checkpoint_format)
            if self.synchronize_cuda and torch.cuda.is_available():
                torch.cuda.synchronize()
        except Exception:
            self.active_update_id = None
            raise
        self._activated(manifest)


class VLLMCUDAVMMExternalStorageAdapter(_AdapterBase):
    """Makes the engine's parameters ALIAS the imported tensors (a cuda-vmm import): every parameter
    named in the manifest gets ``param.data = imported tensor`` through ``apply_model`` (or the
    callable given), so a later publish into the same allocation is visible without another install
    (rl_engine/integrations/common/weights.py:543-745)."""

    def __init__(self, engine, *, apply_model: Optional[Callable[[Callable[[Any], Any]], Any]] = None,
                 name_map: Optional[Callable[[str], str]] = None):
        super().__init__()
        self.engine, self._apply, self._name_map = engine, apply_model, name_map or (lambda n: n)
        self._saved: dict[str, dict[str, torch.Tensor]] = {}

    def _resolve_apply(self):
        if self._apply is not None:
            return self._apply
        for owner in (self.engine, getattr(self.engine, "llm_engine", None)):
            fn = getattr(owner, "apply_model", None)
            if callable(fn):
                return fn
        if isinstance(self.engine, torch.nn.Module):
            return lambda f: f(self.engine)
        raise WeightBridgeUnavailableError("the engine exposes no apply_model(fn) and is not an nn.Module")

    def install(self, manifest, tensors) -> None:
        WeightLayout.from_metadata(manifest.metadata).validate_supported()
        tensors = dict(tensors)
        _check_tensor_set(manifest, tensors, "vLLM external storage")
        saved: dict[str, torch.Tensor] = {}

        def alias(model) -> dict[str, Any]:
            params = dict(model.named_parameters())
            missing = [n for n in tensors if self._name_map(n) not in params]
            if missing:
                raise WeightManifestValidationError(f"model has no parameters named {missing[:4]}")
            for n, t in tensors.items():
                p = params[self._name_map(n)]
                if tuple(p.shape) != tuple(t.shape) or p.dtype != t.dtype:
                    raise WeightManifestValidationError(f"parameter {n}: model {tuple(p.shape)}/{p.dtype}, update {tuple(t.shape)}/{t.dtype}")
                saved[n] = p.data
                p.data = t
            return {"aliased": len(tensors)}

        self._resolve_apply()(alias)
        self._saved[manifest.update_id] = saved
        self._activated(manifest)

    def release(self, update_id: str) -> None:
        saved = self._saved.pop(update_id, None)
        if saved and self.active_update_id == update_id:
            def restore(model):
                params = dict(model.named_parameters())
                for n, data in saved.items():
                    params[self._name_map(n)].data = data
            self._resolve_apply()(restore)
        super().release(update_id)


# ------------------------------------------------------------------------------- factory
def make_weight_bridge(transport: str = "local-clone", *, source_worker: str = "local-training", source_rank: int = 0):
    if transport in {"local", "local-clone", "local-copy"}:
        return LocalTensorCopyBridge(source_worker=source_worker, source_rank=source_rank)
    if transport in {"shared-memory", "shm"}:
        return SharedMemoryTensorBridge(source_worker=source_worker, source_rank=source_rank)
    if transport in {"cuda-vmm", "cuda-vmm-fd"}:
        return CUDAVMMTensorBridge(source_worker=source_worker, source_rank=source_rank)
    if transport in {"cuda-ipc", "ipc"}:
        return IPCWeightBridge(source_worker=source_worker, source_rank=source_rank)
    if transport in {"multi-node", "rdma", "nccl-rdma"}:
        raise WeightBridgeUnavailableError("multi-node / RDMA weight transport is not implemented: one node only")
    raise WeightBridgeUnavailableError(f"unknown weight bridge transport: {transport}")


__all__ = [
    "CUDAIPCTensorBridge", "CUDAVMMTensorBridge", "CallableInstallAdapter", "IPCWeightBridge", "LocalTensorCopyBridge",
    "NVLinkPushBridge", "SharedMemoryTensorBridge", "TensorDescriptor", "UpdateState", "VLLMCUDAVMMExternalStorageAdapter",
    "VLLMCheckpointWeightReloadAdapter", "VLLMInProcessWeightReloadAdapter", "VLLMIPCWeightUpdateRequestBuilder",
    "VLLMWeightInstallAdapter", "WeightBridge", "WeightBridgeError", "WeightBridgeUnavailableError", "WeightConsumer",
    "WeightInstallAdapter", "WeightLayout", "WeightManifestValidationError", "WeightPublisher", "WeightSyncError",
    "WeightUpdateManifest", "WeightUpdateRejectedError", "make_weight_bridge", "reshard_blocks", "tensor_sha256",
]
