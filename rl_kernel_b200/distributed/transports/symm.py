"""Fixed-order collectives on CUDA symmetric memory (NVLink peer loads/stores, one node).

Bring-up mirrors the reference (rl_engine/distributed/algorithms/collectives.py:312-390): every rank
allocates a window, the IPC handles and host names are exchanged with ``all_gather_object`` (the
only host-side step, once), peers are mapped, and from then on each collective is one kernel on the
caller's stream.  Differences: device waits are bounded and report through a status word
(``CollectiveTimeout``), sequence numbers survive CUDA-graph replay (``graph_capture``), and the
sum tree continues det_gemm's canonical K-chunk tree.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
import socket
from ctypes import c_int, c_longlong, c_void_p

import torch

from rl_kernel_b200.backends import extension as ext
from rl_kernel_b200.backends import native as nv
from rl_kernel_b200.distributed.algorithms.collectives import CollectiveMismatchError, CollectiveTimeout

_DT = {torch.bfloat16: 0, torch.float32: 1}


class _DevicePtrView:
    """Exposes a raw device pointer to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3}


class SymmetricMemoryCollective:
    def __init__(self, group, device: torch.device, frame_bytes: int = 256 << 20):
        import torch.distributed as dist

        self._dist, self.group, self.device = dist, group, torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world & (self.world - 1) or self.world > 8:
            raise ValueError(f"world size must be 1, 2, 4 or 8, got {self.world}")
        self.frame_bytes = (int(frame_bytes) + 255) // 256 * 256
        self._lib = ext.load()
        self._lib.rlk_symm_frame_ptr.restype = c_void_p
        self._lib.rlk_symm_graph_end.restype = c_longlong
        self._state = c_void_p(0)
        self._closed = False
        # Debug aid (``RLK_SYMM_VERIFY=1`` or ``verify_signatures = True`` on every rank): before each call the ranks
        # compare (operation, shapes, dtype, call number) on the host and all raise CollectiveMismatchError when
        # they differ -- before any kernel is launched, so nobody is left waiting for a peer that will not come.
        self.verify_signatures = os.environ.get("RLK_SYMM_VERIFY", "0") not in ("", "0")
        self._calls = 0
        if self.world == 1:
            return
        with torch.cuda.device(self.device):
            hbytes = self._lib.rlk_symm_ipc_handle_bytes()
            handle = ctypes.create_string_buffer(hbytes)
            window = c_void_p(0)
            ext.check(self._lib.rlk_symm_alloc(c_longlong(self.frame_bytes), ctypes.byref(window), handle),
                      "symm_alloc")
            infos = [None] * self.world
            dist.all_gather_object(infos, (socket.gethostname(), bytes(handle.raw), self.frame_bytes), group=group)
            if len({i[0] for i in infos}) != 1:
                raise RuntimeError(f"symmetric-memory collectives need all ranks on one host, got {[i[0] for i in infos]}")
            if len({i[2] for i in infos}) != 1:
                raise RuntimeError(f"frame capacity differs across ranks: {[i[2] for i in infos]}")
            blob = b"".join(i[1] for i in infos)
            ext.check(self._lib.rlk_symm_create(window, blob, c_int(self.world), c_int(self.rank),
                                                c_longlong(self.frame_bytes), ctypes.byref(self._state)),
                      "symm_create")
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)

    # ------------------------------------------------------------------ helpers
    def _verify(self, op: str, *tensors: torch.Tensor, extra=()) -> None:
        """Host-side cross-rank comparison of the call (see ``verify_signatures``); skipped during graph capture."""
        self._calls += 1
        if not self.verify_signatures or self.world == 1 or torch.cuda.is_current_stream_capturing():
            return
        mine = (op, tuple((tuple(t.shape), str(t.dtype)) for t in tensors), tuple(extra), self._calls)
        sigs = [None] * self.world
        self._dist.all_gather_object(sigs, mine, group=self.group)
        if any(s != sigs[0] for s in sigs):
            raise CollectiveMismatchError(f"ranks disagree on collective call {self._calls}: {sigs}")

    def _check_open(self):
        if self._closed:
            raise RuntimeError("collective is closed")

    def frame_tensor(self, rank: int, frame: int, nbytes: int | None = None) -> torch.Tensor:
        """uint8 view of frame ``frame`` of rank ``rank``'s window as mapped in this process."""
        p = self._lib.rlk_symm_frame_ptr(self._state, c_int(rank), c_int(frame))
        return torch.as_tensor(_DevicePtrView(p, nbytes or self.frame_bytes), device=self.device)

    def staging_view(self, shape, dtype) -> torch.Tensor:
        """A tensor inside the frame the NEXT all_reduce will use: a producer (e.g. a GEMM) writes its
        partial result there and ``all_reduce_staged`` skips the copy-in."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        f = self._lib.rlk_symm_next_frame(self._state)
        return self.frame_tensor(self.rank, f, nbytes).view(dtype).view(shape)

    def raise_on_timeout(self) -> None:
        code = ext.poll_status(self.device)
        if code:
            raise CollectiveTimeout(f"a peer did not arrive within the wait limit (wait id {code})")

    # ------------------------------------------------------------------ collectives
    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        self._check_open()
        if t.dtype not in _DT or not t.is_contiguous():
            raise TypeError("all_reduce_ needs a contiguous bf16 or fp32 tensor")
        nbytes = t.numel() * t.element_size()
        if nbytes % 16:
            raise ValueError("all_reduce_: byte size must be a multiple of 16")
        self._verify("all_reduce", t)
        base = t.data_ptr()
        for off in range(0, nbytes, self.frame_bytes):       # larger than a frame: frame-sized pieces
            n = min(self.frame_bytes, nbytes - off)
            ext.check(self._lib.rlk_symm_all_reduce(self._state, c_void_p(base + off), c_void_p(base + off),
                                                    c_longlong(n), c_int(_DT[t.dtype]), c_int(0),
                                                    ext.stream_ptr(self.device)), "symm_all_reduce")
            nv._count()
        return t

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        return self.all_reduce_(t.clone())

    def all_reduce_staged(self, staged: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``staged`` must come from ``staging_view`` (same shape/dtype as ``out``)."""
        nbytes = out.numel() * out.element_size()
        ext.check(self._lib.rlk_symm_all_reduce(self._state, ext.ptr(staged), ext.ptr(out), c_longlong(nbytes),
                                                c_int(_DT[out.dtype]), c_int(1), ext.stream_ptr(self.device)),
                  "symm_all_reduce_staged")
        nv._count()
        return out

    def gemm_all_reduce(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, nchunks: int = 1) -> torch.Tensor:
        """out = tree-all-reduce over the group of (a_local @ b_local^T with canonical K chunks), as
        ONE kernel: tiles are exchanged over NVLink from inside the GEMM epilogue while later tiles
        are still being multiplied (csrc/gemm/det_gemm_sm100.cu, rlk_det_gemm_ar)."""
        self._check_open()
        self._verify("gemm_all_reduce", a, b, out, extra=(nchunks,))
        M, K = a.shape
        N = b.shape[0]
        ext.check(self._lib.rlk_det_gemm_ar(self._state, ext.ptr(a), ext.ptr(b), ext.ptr(out), c_int(M), c_int(N),
                                            c_int(K), c_longlong(a.stride(0)), c_longlong(b.stride(0)),
                                            c_longlong(out.stride(0)), c_int(nchunks), ext.stream_ptr(self.device)),
                  "det_gemm_ar")
        nv._count()
        return out

    def gemm_reduce_scatter(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, nchunks: int = 1) -> torch.Tensor:
        """out [M / world, N] = this rank's token rows of the tree-all-reduce of (a_local @ b_local^T), as ONE kernel
        (rlk_det_gemm_rs): the sequence-parallel form of ``gemm_all_reduce``.  Same bits per row; each partial tile
        crosses NVLink once.  M must be a multiple of 128 x world."""
        self._check_open()
        M, K = a.shape
        N = b.shape[0]
        if out.shape[0] * self.world != M or out.shape[1] != N:
            raise ValueError(f"out must be [{M // self.world}, {N}], got {tuple(out.shape)}")
        self._verify("gemm_reduce_scatter", a, b, out, extra=(nchunks,))
        ext.check(self._lib.rlk_det_gemm_rs(self._state, ext.ptr(a), ext.ptr(b), ext.ptr(out), c_int(M), c_int(N),
                                            c_int(K), c_longlong(a.stride(0)), c_longlong(b.stride(0)),
                                            c_longlong(out.stride(0)), c_int(nchunks), ext.stream_ptr(self.device)),
                  "det_gemm_rs")
        nv._count()
        return out

    def all_reduce_int_(self, t: torch.Tensor) -> torch.Tensor:
        """Integer sums are associative: gather and add (exact in any order)."""
        if self.world == 1:
            return t
        g = self.all_gather(t)
        t.copy_(g.sum(0))
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t.unsqueeze(0)
        self._check_open()
        self._verify("all_gather", t)
        t = t.contiguous()
        nbytes = t.numel() * t.element_size()
        pad = (-nbytes) % 16
        src = t
        if pad:
            src = torch.zeros(nbytes + pad, dtype=torch.uint8, device=t.device)
            src[:nbytes] = t.view(torch.uint8).reshape(-1)
        total = nbytes + pad
        out = torch.empty(self.world * total, dtype=torch.uint8, device=t.device)
        if total <= self.frame_bytes:
            ext.check(self._lib.rlk_symm_all_gather(self._state, ext.ptr(src), ext.ptr(out), c_longlong(total),
                                                    ext.stream_ptr(self.device)), "symm_all_gather")
            nv._count()
        else:
            # a rank's share is larger than a frame: frame-sized pieces, each gathered and then placed
            flat, rows = src.view(torch.uint8).reshape(-1), out.view(self.world, total)
            for off in range(0, total, self.frame_bytes):
                n = min(self.frame_bytes, total - off)
                piece = torch.empty(self.world * n, dtype=torch.uint8, device=t.device)
                ext.check(self._lib.rlk_symm_all_gather(self._state, ext.ptr(flat[off:off + n]), ext.ptr(piece),
                                                        c_longlong(n), ext.stream_ptr(self.device)), "symm_all_gather")
                nv._count()
                rows[:, off:off + n].copy_(piece.view(self.world, n))
        out = out.view(self.world, total)[:, :nbytes]
        if pad:
            out = out.contiguous()
        return out.view(t.dtype).view((self.world,) + tuple(t.shape))

    def all_gather_many(self, tensors):
        return [self.all_gather(t) for t in tensors]

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """t [world * n, ...] -> the fixed-tree sum of this rank's [n, ...] slice (one kernel: every
        rank stages the slices it does not own, the owner pulls and reduces them)."""
        if self.world == 1:
            return t
        self._check_open()
        n = t.shape[0] // self.world
        t = t.contiguous()
        per = t.numel() // self.world * t.element_size()
        if not (t.dtype not in _DT or t.shape[0] % self.world or per % 16 or per * self.world > self.frame_bytes):
            self._verify("reduce_scatter", t)
        if t.dtype not in _DT or t.shape[0] % self.world or per % 16 or per * self.world > self.frame_bytes:
            return self.all_reduce(t)[self.rank * n:(self.rank + 1) * n].contiguous()
        out = torch.empty((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        ext.check(self._lib.rlk_symm_reduce_scatter(self._state, ext.ptr(t), ext.ptr(out), c_longlong(per),
                                                    c_int(_DT[t.dtype]), ext.stream_ptr(self.device)),
                  "symm_reduce_scatter")
        nv._count()
        return out

    def broadcast_(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world > 1:
            t.copy_(self.all_gather(t)[src])
        return t

    def barrier(self) -> None:
        if self.world > 1:
            ext.check(self._lib.rlk_symm_barrier(self._state, ext.stream_ptr(self.device)), "symm_barrier")
            nv._count()

    # ------------------------------------------------------------------ CUDA graphs
    @contextlib.contextmanager
    def graph_capture(self):
        """Wrap the body of a ``torch.cuda.graph`` capture that contains collectives:

            with torch.cuda.graph(g), coll.graph_capture():
                ...
            coll.graph_commit()            # once, after the capture
            g.replay(); coll.graph_replayed(1)
        """
        if self.world == 1:
            yield
            return
        ext.check(self._lib.rlk_symm_graph_begin(self._state, ext.stream_ptr(self.device)), "graph_begin")
        try:
            yield
        finally:
            self._lib.rlk_symm_graph_end(self._state, ext.stream_ptr(self.device))

    def graph_commit(self) -> None:
        if self.world > 1:
            ext.check(self._lib.rlk_symm_graph_commit(self._state), "graph_commit")

    def graph_replayed(self, times: int = 1) -> None:
        if self.world > 1:
            self._lib.rlk_symm_graph_replayed(self._state, c_longlong(times))

    def resync(self) -> int:
        """After a ``CollectiveTimeout``: agree (on the host) on the highest sequence number any
        rank reached, rounded up to an even value so every rank also agrees on the frame parity."""
        if self.world == 1:
            return 0
        self._lib.rlk_symm_get_seq.restype = c_longlong
        torch.cuda.synchronize(self.device)
        t = torch.tensor([int(self._lib.rlk_symm_get_seq(self._state))], dtype=torch.int64, device=self.device)
        self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX, group=self.group)
        seq = (int(t.item()) + 2) // 2 * 2
        self._lib.rlk_symm_set_seq(self._state, c_longlong(seq))
        return seq

    def close(self) -> None:
        if not self._closed and self.world > 1 and self._state:
            torch.cuda.synchronize(self.device)
            self._dist.barrier(group=self.group)
            self._lib.rlk_symm_destroy(self._state, c_int(1))
        self._closed = True
