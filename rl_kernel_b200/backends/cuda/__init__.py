"""Device operator classes under the names RL-Kernel users import (``rl_engine.backends.cuda.*``).

There is one device target here, sm_100a, so these modules are not a second backend: each class
is a thin, typed front of the tcgen05 / TMA kernels in ``csrc/`` with the reference's constructor
and call signatures, and each also answers to a Blackwell name (``RoPESM100Op`` next to
``RoPESM90Op``).  Parity: rl_engine/backends/cuda/__init__.py and the per-family packages below it.
"""
