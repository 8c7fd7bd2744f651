"""Qwen3 dense: pinned spec, weights (HF key layout), fp32 reference model and the sm_100a engine."""
from rl_kernel_b200.models.qwen3.spec import OFFICIAL_FINGERPRINT, Qwen3DenseSpec  # noqa: F401
from rl_kernel_b200.models.qwen3.weights import Qwen3DenseWeights  # noqa: F401
