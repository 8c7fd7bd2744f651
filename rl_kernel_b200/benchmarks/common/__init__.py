from rl_kernel_b200.benchmarks.common.profiler import (PerformanceProfiler, ProfileResult, WORKLOAD_REGISTRY,  # noqa: F401
                                                       register_workload)
