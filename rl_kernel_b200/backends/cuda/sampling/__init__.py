from rl_kernel_b200.backends.cuda.sampling.unique_scatter import copy_unique_rows_, scatter_permuted_columns  # noqa: F401
