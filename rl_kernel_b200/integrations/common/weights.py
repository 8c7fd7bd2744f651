"""Train -> rollout weight-sync bridge (parity: rl_engine/integrations/common/weights.py:84-2371).

Protocol (unchanged from the reference): a publisher turns a state into a ``WeightUpdateManifest``
{update_id, source_worker, source_rank, weight_version (monotonic), transport,
tensors{name -> TensorDescriptor(shape, dtype, stride, device, numel, nbytes, sha256)}, metadata};
the consumer ``import_update``s it, verifies checksums, installs, then ``acknowledge``s or
``reject``s; a rejected or failed update leaves the previous version active; only after an
acknowledgement is the previous update released.

Transports:
  * ``LocalTensorCopyBridge``     same process, device copy
  * ``SharedMemoryTensorBridge``  POSIX shared memory, cross-process (CPU tensors)
  * ``CUDAIPCTensorBridge``       CUDA IPC handles of a packed device buffer, cross-process
  * ``NVLinkPushBridge``          ONE kernel pushes the trainer's flat shard into the rollout
                                  engines' buffers on peer GPUs, resharding on the way
                                  (csrc/collectives/weight_sync.cu) — the B200-native path
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import threading
import time
import uuid
from dataclasses import asdict, dataclass, field
from multiprocessing import shared_memory
from typing import Callable, Mapping

import torch

SUPPORTED_LAYOUTS = ("full-state", "replicated", "tp-canonical")

_DTYPES = {str(d).removeprefix("torch."): d for d in (torch.bfloat16, torch.float16, torch.float32, torch.int64,
                                                       torch.int32, torch.uint8)}


class WeightSyncError(RuntimeError):
    pass


def tensor_sha256(t: torch.Tensor) -> str:
    b = t.detach().contiguous().cpu()
    return hashlib.sha256(b.view(torch.uint8).numpy().tobytes()).hexdigest()


@dataclass(frozen=True)
class TensorDescriptor:
    shape: tuple[int, ...]
    dtype: str
    stride: tuple[int, ...]
    device: str
    numel: int
    nbytes: int
    sha256: str | None = None
    offset: int = 0               # byte offset inside the transport's packed buffer

    @classmethod
    def of(cls, t: torch.Tensor, *, checksum: bool, offset: int = 0) -> "TensorDescriptor":
        return cls(tuple(t.shape), str(t.dtype).removeprefix("torch."), tuple(t.stride()), str(t.device), t.numel(),
                   t.numel() * t.element_size(), tensor_sha256(t) if checksum else None, offset)

    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype]


@dataclass
class WeightUpdateManifest:
    update_id: str
    source_worker: str
    source_rank: int
    weight_version: int
    transport: str
    tensors: dict[str, TensorDescriptor]
    metadata: dict = field(default_factory=dict)
    created_ts: float = field(default_factory=time.time)

    def to_json(self) -> str:
        d = asdict(self)
        return json.dumps(d, sort_keys=True)

    @classmethod
    def from_json(cls, text: str) -> "WeightUpdateManifest":
        d = json.loads(text)
        d["tensors"] = {k: TensorDescriptor(**{**v, "shape": tuple(v["shape"]), "stride": tuple(v["stride"])})
                        for k, v in d["tensors"].items()}
        return cls(**d)

    def validate(self) -> None:
        layout = self.metadata.get("layout", "full-state")
        if layout not in SUPPORTED_LAYOUTS:
            raise WeightSyncError(f"unsupported layout {layout!r}; supported: {SUPPORTED_LAYOUTS}")
        if self.metadata.get("node_count", 1) != 1:
            raise WeightSyncError("the weight bridge is single-node")
        if self.weight_version < 0:
            raise WeightSyncError("weight_version must be non-negative")


class UpdateState:
    PUBLISHED, IMPORTED, ACKNOWLEDGED, REJECTED, RELEASED = "published", "imported", "acknowledged", "rejected", "released"


class _BridgeBase:
    """Lifecycle bookkeeping shared by all transports."""
    transport = "base"

    def __init__(self, worker: str = "trainer", rank: int = 0, checksum: bool = True):
        self.worker, self.rank, self.checksum = worker, rank, checksum
        self._lock = threading.Lock()
        self._states: dict[str, str] = {}
        self._version = -1
        self._active_update: str | None = None
        self.rejections: dict[str, str] = {}

    # ---- publisher side
    def _new_manifest(self, tensors: dict[str, TensorDescriptor], weight_version: int, metadata: dict | None):
        with self._lock:
            if weight_version <= self._version:
                raise WeightSyncError(f"weight_version must increase monotonically: {weight_version} <= {self._version}")
            self._version = weight_version
            m = WeightUpdateManifest(uuid.uuid4().hex, self.worker, self.rank, weight_version, self.transport, tensors,
                                     dict(metadata or {}))
            m.metadata.setdefault("layout", "full-state")
            m.validate()
            self._states[m.update_id] = UpdateState.PUBLISHED
            return m

    # ---- consumer side
    def _verify(self, manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor]) -> None:
        for name, d in manifest.tensors.items():
            t = tensors[name]
            if tuple(t.shape) != d.shape or str(t.dtype).removeprefix("torch.") != d.dtype:
                raise WeightSyncError(f"{name}: got {tuple(t.shape)}/{t.dtype}, manifest says {d.shape}/{d.dtype}")
            if d.sha256 is not None and tensor_sha256(t) != d.sha256:
                raise WeightSyncError(f"{name}: checksum mismatch")

    def acknowledge(self, update_id: str) -> None:
        with self._lock:
            if self._states.get(update_id) not in (UpdateState.IMPORTED, UpdateState.PUBLISHED):
                raise WeightSyncError(f"cannot acknowledge update in state {self._states.get(update_id)!r}")
            prev, self._active_update = self._active_update, update_id
            self._states[update_id] = UpdateState.ACKNOWLEDGED
        if prev is not None and prev != update_id:
            self.release(prev)

    def reject(self, update_id: str, reason: str) -> None:
        with self._lock:
            self._states[update_id] = UpdateState.REJECTED
            self.rejections[update_id] = reason
        self._free(update_id)

    def release(self, update_id: str) -> None:
        with self._lock:
            self._states[update_id] = UpdateState.RELEASED
        self._free(update_id)

    def state(self, update_id: str) -> str | None:
        return self._states.get(update_id)

    def _free(self, update_id: str) -> None:  # transports that own buffers override
        pass

    def close(self) -> None:
        for uid, st in list(self._states.items()):
            if st not in (UpdateState.RELEASED, UpdateState.REJECTED):
                self._free(uid)


class LocalTensorCopyBridge(_BridgeBase):
    transport = "local-copy"

    def __init__(self, **kw):
        super().__init__(**kw)
        self._payload: dict[str, dict[str, torch.Tensor]] = {}

    def publish(self, state: Mapping[str, torch.Tensor], weight_version: int, metadata: dict | None = None):
        snap = {k: v.detach().clone() for k, v in state.items()}
        m = self._new_manifest({k: TensorDescriptor.of(v, checksum=self.checksum) for k, v in snap.items()},
                               weight_version, metadata)
        self._payload[m.update_id] = snap
        return m

    def import_update(self, manifest: WeightUpdateManifest) -> dict[str, torch.Tensor]:
        manifest.validate()
        if manifest.update_id not in self._payload:
            raise WeightSyncError(f"unknown update {manifest.update_id}")
        tensors = self._payload[manifest.update_id]
        self._verify(manifest, tensors)
        self._states[manifest.update_id] = UpdateState.IMPORTED
        return tensors

    def _free(self, update_id: str) -> None:
        self._payload.pop(update_id, None)


class SharedMemoryTensorBridge(_BridgeBase):
    """Packs the state 256-byte aligned into one POSIX shared-memory segment."""
    transport = "shared-memory"

    def __init__(self, **kw):
        super().__init__(**kw)
        self._segments: dict[str, shared_memory.SharedMemory] = {}

    def publish(self, state: Mapping[str, torch.Tensor], weight_version: int, metadata: dict | None = None):
        descs, off = {}, 0
        cpu = {k: v.detach().contiguous().cpu() for k, v in state.items()}
        for k, v in cpu.items():
            descs[k] = TensorDescriptor.of(v, checksum=self.checksum, offset=off)
            off = (off + v.numel() * v.element_size() + 255) // 256 * 256
        seg = shared_memory.SharedMemory(create=True, size=max(off, 256))
        for k, v in cpu.items():
            d = descs[k]
            seg.buf[d.offset:d.offset + d.nbytes] = v.view(torch.uint8).reshape(-1).numpy().tobytes()
        m = self._new_manifest(descs, weight_version, {**(metadata or {}), "shm_name": seg.name, "shm_bytes": off})
        self._segments[m.update_id] = seg
        return m

    def import_update(self, manifest: WeightUpdateManifest) -> dict[str, torch.Tensor]:
        manifest.validate()
        seg = self._segments.get(manifest.update_id)
        if seg is None:        # another process: attach by name
            seg = shared_memory.SharedMemory(name=manifest.metadata["shm_name"])
            self._segments[manifest.update_id] = seg
        out = {}
        for k, d in manifest.tensors.items():
            raw = bytes(seg.buf[d.offset:d.offset + d.nbytes])
            out[k] = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(d.torch_dtype()).view(d.shape).clone()
        self._verify(manifest, out)
        self._states[manifest.update_id] = UpdateState.IMPORTED
        return out

    def _free(self, update_id: str) -> None:
        seg = self._segments.pop(update_id, None)
        if seg is not None:
            seg.close()
            try:
                seg.unlink()
            except FileNotFoundError:
                pass


class CUDAIPCTensorBridge(_BridgeBase):
    """Packs the state into one cudaMalloc'ed buffer and exports it with a CUDA IPC handle; the
    consumer process maps it and sees the tensors without a copy."""
    transport = "cuda-ipc"

    def __init__(self, device: torch.device | str = "cuda:0", **kw):
        super().__init__(**kw)
        self.device = torch.device(device)
        self._bufs: dict[str, tuple[int, bool]] = {}     # update_id -> (device pointer, owned)

    def _lib(self):
        from rl_kernel_b200.backends import extension

        return extension.load()

    def publish(self, state: Mapping[str, torch.Tensor], weight_version: int, metadata: dict | None = None):
        from rl_kernel_b200.backends import extension as ext
        from rl_kernel_b200.distributed.transports.symm import _DevicePtrView

        descs, off = {}, 0
        for k, v in state.items():
            descs[k] = TensorDescriptor.of(v, checksum=self.checksum, offset=off)
            off = (off + v.numel() * v.element_size() + 255) // 256 * 256
        lib = self._lib()
        handle = ctypes.create_string_buffer(lib.rlk_symm_ipc_handle_bytes())
        ptr = ctypes.c_void_p(0)
        with torch.cuda.device(self.device):
            ext.check(lib.rlk_ipc_alloc(ctypes.c_longlong(max(off, 256)), ctypes.byref(ptr), handle), "ipc_alloc")
        packed = torch.as_tensor(_DevicePtrView(ptr.value, max(off, 256)), device=self.device)
        for k, v in state.items():
            d = descs[k]
            packed[d.offset:d.offset + d.nbytes].copy_(v.detach().contiguous().view(torch.uint8).reshape(-1))
        torch.cuda.synchronize(self.device)
        m = self._new_manifest(descs, weight_version, {**(metadata or {}), "ipc_handle": handle.raw.hex(),
                                                        "packed_bytes": max(off, 256)})
        self._bufs[m.update_id] = (ptr.value, True)
        return m

    def import_update(self, manifest: WeightUpdateManifest) -> dict[str, torch.Tensor]:
        from rl_kernel_b200.backends import extension as ext
        from rl_kernel_b200.distributed.transports.symm import _DevicePtrView

        manifest.validate()
        if manifest.update_id in self._bufs:
            base = self._bufs[manifest.update_id][0]
        else:
            ptr = ctypes.c_void_p(0)
            with torch.cuda.device(self.device):
                ext.check(self._lib().rlk_ipc_open(bytes.fromhex(manifest.metadata["ipc_handle"]), ctypes.byref(ptr)),
                          "ipc_open")
            base = ptr.value
            self._bufs[manifest.update_id] = (base, False)
        packed = torch.as_tensor(_DevicePtrView(base, manifest.metadata["packed_bytes"]), device=self.device)
        out = {k: packed[d.offset:d.offset + d.nbytes].view(d.torch_dtype()).view(d.shape)
               for k, d in manifest.tensors.items()}
        self._verify(manifest, out)
        self._states[manifest.update_id] = UpdateState.IMPORTED
        return out

    def _free(self, update_id: str) -> None:
        entry = self._bufs.pop(update_id, None)
        if entry is not None:
            lib = self._lib()
            (lib.rlk_ipc_free if entry[1] else lib.rlk_ipc_close)(ctypes.c_void_p(entry[0]))


# --------------------------------------------------------------------------- NVLink push (K17)
def reshard_blocks(src_params, dst_params, dst_index: int) -> list[tuple]:
    """2-D block copies that move the part of ``src_params`` (a PackedParams shard of a TP group of
    size tp_s) that destination shard ``dst_params`` (TP size tp_d) needs.  Returns tuples
    (src_off, dst_off, src_pitch, dst_pitch, rows, row_bytes, dst_mask) in BYTES."""
    out = []
    ts, rs = src_params.tp_size, src_params.tp_rank
    td, rd = dst_params.tp_size, dst_params.tp_rank
    for name, s in src_params.slots.items():
        d = dst_params.slots[name]
        if len(s.shape) == 1:                                       # replicated vector
            if rs == 0 or ts == 1:
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


class NVLinkPushBridge(_BridgeBase):
    """The trainer pushes its flat bf16 shard into up to 8 destination buffers (peer-mapped rollout
    parameter buffers) with one kernel; the block list encodes the layout change."""
    transport = "nvlink-push"

    def __init__(self, src_params, device: torch.device, **kw):
        super().__init__(checksum=False, **kw)
        self.src, self.device = src_params, device
        self._targets: list[tuple[int, int | None]] = []   # (base pointer, flag pointer)
        self._blocks: list[tuple] = []
        self._descs = None
        self._counter = torch.zeros(1, dtype=torch.int32, device=device)

    def add_target(self, dst_params, base_ptr: int | None = None, version_flag_ptr: int | None = None) -> int:
        """Register a destination shard; ``base_ptr`` is its flat buffer as mapped in THIS process
        (defaults to dst_params.flat for same-process targets)."""
        idx = len(self._targets)
        if idx >= 8:
            raise WeightSyncError("at most 8 destinations per push")
        self._targets.append((base_ptr if base_ptr is not None else dst_params.flat.data_ptr(), version_flag_ptr))
        self._blocks += reshard_blocks(self.src, dst_params, idx)
        self._descs = None
        return idx

    def _desc_tensor(self) -> torch.Tensor:
        if self._descs is None:
            rows = []
            for (so, do, sp, dp, r, rb, mask) in self._blocks:
                if rb % 16 or so % 16 or do % 16 or (r > 1 and (sp % 16 or dp % 16)):
                    raise WeightSyncError("weight blocks must be 16-byte aligned")
                rows.append([so, do, sp, dp, r | (rb << 32), mask])
            t = torch.tensor(rows, dtype=torch.int64)
            self._descs = t.to(self.device).contiguous()
        return self._descs

    def publish(self, weight_version: int, metadata: dict | None = None) -> WeightUpdateManifest:
        from rl_kernel_b200.backends import extension as ext
        from rl_kernel_b200.backends import native as nv

        descs = self._desc_tensor()
        n = len(self._targets)
        bases = (ctypes.c_void_p * n)(*[t[0] for t in self._targets])
        flags = (ctypes.c_void_p * n)(*[t[1] or 0 for t in self._targets])
        ext.check(ext.load().rlk_weight_push(ext.ptr(self.src.flat), ext.ptr(descs), ctypes.c_int(descs.shape[0]), bases,
                                             flags, ctypes.c_int(n), ctypes.c_ulonglong(weight_version),
                                             ext.ptr(self._counter), ext.stream_ptr(self.device)), "weight_push")
        nv._count()
        tensors = {k: TensorDescriptor(tuple(s.shape), "bfloat16", (), str(self.device), s.numel, s.numel * 2, None,
                                       s.offset * 2) for k, s in self.src.slots.items()}
        return self._new_manifest(tensors, weight_version, {**(metadata or {}), "layout": "tp-canonical",
                                                            "targets": n, "blocks": int(descs.shape[0])})

    def import_update(self, manifest: WeightUpdateManifest):
        manifest.validate()
        self._states[manifest.update_id] = UpdateState.IMPORTED
        return {}


class WeightPublisher:
    """Publisher facade used by training workers (parity: WeightPublisher.publish, weights.py:1360-1405)."""

    def __init__(self, bridge, on_publish: Callable[[WeightUpdateManifest], None] | None = None):
        self.bridge, self.on_publish = bridge, on_publish
        self.history: list[WeightUpdateManifest] = []

    def publish(self, state, weight_version: int, metadata: dict | None = None) -> WeightUpdateManifest:
        m = self.bridge.publish(state, weight_version, metadata) if state is not None else \
            self.bridge.publish(weight_version, metadata)
        self.history.append(m)
        if self.on_publish:
            self.on_publish(m)
        return m


class WeightInstallAdapter:
    """Installs imported tensors into an engine: ``install(tensors, manifest)`` must raise on failure."""

    def __init__(self, install_fn: Callable[[Mapping[str, torch.Tensor], WeightUpdateManifest], None]):
        self._fn = install_fn

    def install(self, tensors, manifest) -> None:
        self._fn(tensors, manifest)
