"""Operator and step micro-benchmarks (CUDA-event timing, warm-up excluded), runnable as
``python -m rl_kernel_b200.benchmarks.<name>``."""
