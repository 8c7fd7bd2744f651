from rl_kernel_b200.config.workload import WS1Manifest, load_manifest  # noqa: F401
