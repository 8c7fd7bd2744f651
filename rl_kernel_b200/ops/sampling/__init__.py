from rl_kernel_b200.ops.sampling.api import SamplerBackend, sample  # noqa: F401
from rl_kernel_b200.ops.sampling.policy import sampling_keep_mask, vocab_parallel_sampling_keep_mask  # noqa: F401
