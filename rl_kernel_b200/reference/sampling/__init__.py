from rl_kernel_b200.reference.sampling.policy import sampling_keep_mask, sample_from_logits  # noqa: F401
