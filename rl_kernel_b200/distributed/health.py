"""Host-side failure detection for multi-rank jobs.

Device waits in this library are bounded and report through a status word, so a missing peer can
not hang a GPU -- but a rank should not even launch a collective whose peer is already known to be
gone.  ``PeerMonitor`` keeps one record per rank in a key-value store (torch.distributed's
TCPStore / FileStore): the last step the rank finished and, if it failed, why.  Every rank calls
``begin_step`` before it launches the step's kernels; it raises ``PeerFailure`` when a peer has
reported a failure or has fallen more than ``max_lag`` steps behind for longer than ``timeout_s``.
A rank leaves only between steps (``leave``), with none of its kernels in flight, and the others
learn of it here before their next launch.  (The reference has no such layer: its device waits
spin forever and a dead peer hangs the GPU, csrc/cuda/collectives/deterministic_collective.cu:
113-138; its launcher only refuses busy GPUs, rl_engine/entrypoints/repro.py:286-300.)
"""
from __future__ import annotations

import contextlib
import json
import time


class PeerFailure(RuntimeError):
    """A peer reported a failure, left, or stopped making progress."""

    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class PeerMonitor:
    def __init__(self, store, rank: int, world: int, *, prefix: str = "rlk/health", timeout_s: float = 30.0,
                 max_lag: int = 1, poll_s: float = 0.05):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self.timeout_s, self.max_lag, self.poll_s = timeout_s, max_lag, poll_s
        self._put({"step": -1, "state": "ok", "reason": ""})

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _put(self, rec: dict) -> None:
        self.store.set(self._key(self.rank), json.dumps(rec))

    def _get(self, rank: int) -> dict | None:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(rank)]):
                return None
            return json.loads(self.store.get(self._key(rank)).decode())
        except Exception:                       # a store that is gone is a failure of its host
            return {"step": -1, "state": "failed", "reason": "health store unreachable"}

    def begin_step(self, step: int) -> None:
        """Call before launching step ``step``: every peer must have finished step - 1 - max_lag
        and none may have failed or left."""
        deadline = time.monotonic() + self.timeout_s
        need = step - 1 - self.max_lag
        while True:
            behind = None
            for r in range(self.world):
                if r == self.rank:
                    continue
                rec = self._get(r)
                if rec is None:
                    behind = (r, "has not registered")
                    continue
                if rec["state"] != "ok":
                    raise PeerFailure(r, f"{rec['state']}: {rec['reason']}")
                if rec["step"] < need:
                    behind = (r, f"still at step {rec['step']}, step {need} needed")
            if behind is None:
                return
            if time.monotonic() > deadline:
                raise PeerFailure(behind[0], f"no progress within {self.timeout_s:.1f} s ({behind[1]})")
            time.sleep(self.poll_s)

    def end_step(self, step: int) -> None:
        self._put({"step": step, "state": "ok", "reason": ""})

    def fail(self, reason: str) -> None:
        self._put({"step": -1, "state": "failed", "reason": reason[:500]})

    def leave(self, reason: str = "left") -> None:
        """Announce an orderly exit (between steps, nothing in flight)."""
        self._put({"step": -1, "state": "left", "reason": reason})

    @contextlib.contextmanager
    def step(self, index: int):
        """``with monitor.step(i): ...`` = begin_step, body, end_step; an exception in the body is
        published to the peers before it propagates."""
        self.begin_step(index)
        try:
            yield
        except BaseException as exc:
            self.fail(f"{type(exc).__name__}: {exc}")
            raise
        self.end_step(index)
