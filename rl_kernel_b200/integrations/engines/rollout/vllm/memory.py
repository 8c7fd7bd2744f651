"""Worker memory preparation: symmetric-memory windows must be created BEFORE the engine grabs the
rest of the GPU for its KV / weight pools (parity: prepare_worker_ipc,
rl_engine/integrations/engines/rollout/vllm/memory.py:9-47)."""
from __future__ import annotations

_PREPARED: dict = {}


def prepare_worker_ipc(group, device, frame_bytes: int = 64 << 20):
    key = (id(group), str(device))
    if key not in _PREPARED:
        from rl_kernel_b200.distributed import create_deterministic_collective

        _PREPARED[key] = create_deterministic_collective(group, device, frame_bytes=frame_bytes)
    return _PREPARED[key]
