"""Helpers shared by the GPU tests."""
import torch

from rl_kernel_b200.backends import extension as ext


def sync_and_check():
    """Synchronise and fail if a bounded device wait timed out."""
    torch.cuda.synchronize()
    code = ext.poll_status()
    assert code == 0, f"device wait timed out (wait id {code})"


def dev():
    return torch.device("cuda:0")
