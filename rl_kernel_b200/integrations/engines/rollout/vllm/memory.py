"""Worker memory preparation (parity: rl_engine/integrations/engines/rollout/vllm/memory.py:9-91).

Symmetric-memory windows and peer-mapped page pools must exist BEFORE the engine sizes its KV / weight pools from
the free memory it sees, otherwise the later allocation fails or lands in an offloadable pool.
``prepare_worker_ipc`` creates the tensor-parallel collective and, under prefill context parallelism, a window large
enough for the CP exchange; ``patch_weight_pool`` repairs the known ``with pool and config`` pattern of some vLLM
releases that skips the weight pool in sleep mode.
"""
from __future__ import annotations

import ast
import inspect
import os
import textwrap
from functools import wraps

_PREPARED: dict = {}


def _collective(group, device, frame_bytes: int):
    key = (id(group), str(device))
    if key not in _PREPARED or _PREPARED[key][1] < frame_bytes:
        from rl_kernel_b200.distributed import create_deterministic_collective

        _PREPARED[key] = (create_deterministic_collective(group, device, frame_bytes=frame_bytes), frame_bytes)
    return _PREPARED[key][0]


def prepare_worker_ipc(group_or_worker, device=None, frame_bytes: int = 64 << 20):
    """``prepare_worker_ipc(group, device)`` builds (once) the collective of a process group.
    ``prepare_worker_ipc(worker)`` does what a vLLM worker needs: the TP collective, and for
    ``prefill_context_parallel_size > 1`` a CP window sized for K and V of the captured batch."""
    if device is not None or not hasattr(group_or_worker, "vllm_config"):
        return _collective(group_or_worker, device, frame_bytes)
    import torch
    from vllm.distributed import get_tp_group  # type: ignore

    worker = group_or_worker
    cfg = worker.vllm_config
    dev = getattr(worker, "device", torch.device("cuda", torch.cuda.current_device()))
    out = {}
    tp = get_tp_group()
    if tp.world_size > 1:
        out["tp"] = _collective(tp.device_group, dev, frame_bytes)
    cp = int(getattr(cfg.parallel_config, "prefill_context_parallel_size", 1))
    if cp > 1:
        from vllm.distributed import get_pcp_group  # type: ignore

        block = int(cfg.cache_config.block_size)
        capacity = ((cfg.model_config.max_model_len + cp * block - 1) // (cp * block)) * block
        requests = min(cfg.scheduler_config.max_num_seqs,
                       int(os.getenv("RL_KERNEL_VLLM_CUDAGRAPH_MAX_CAPTURE_SIZE", str(cfg.scheduler_config.max_num_seqs))))
        kv_heads = cfg.model_config.get_num_kv_heads(cfg.parallel_config)
        head = cfg.model_config.get_head_size()
        esize = torch.empty((), dtype=cfg.model_config.dtype).element_size()
        out["pcp"] = _collective(get_pcp_group().device_group, dev, 2 * requests * capacity * kv_heads * head * esize)
    return out


def patch_weight_pool(worker_class=None, prepare=None) -> bool:
    """Wrap ``load_model`` of workers whose source enters the weight pool as ``with pool and config`` (the pool
    context is dropped by the ``and``).  Returns whether a patch was applied."""
    if worker_class is None:
        from vllm.v1.worker.gpu_worker import Worker as worker_class  # type: ignore
    original = worker_class.load_model
    if getattr(original, "_rlk_weight_pool_fix", False):
        return False
    try:
        tree = ast.parse(textwrap.dedent(inspect.getsource(original)))
    except (OSError, TypeError, IndentationError, SyntaxError):
        return False
    broken = any(isinstance(node, ast.withitem) and isinstance(node.context_expr, ast.BoolOp)
                 and isinstance(node.context_expr.op, ast.And)
                 and any(isinstance(v, ast.Call) and isinstance(v.func, ast.Attribute)
                         and v.func.attr == "_maybe_get_memory_pool_context" for v in node.context_expr.values)
                 for node in ast.walk(tree))
    if not broken:
        return False

    @wraps(original)
    def load_model(self, *args, **kwargs):
        if not self.vllm_config.model_config.enable_sleep_mode:
            return original(self, *args, **kwargs)
        if prepare is not None:
            prepare(self)
        with self._maybe_get_memory_pool_context(tag="weights"):
            return original(self, *args, **kwargs)

    load_model._rlk_weight_pool_fix = True
    worker_class.load_model = load_model
    return True
