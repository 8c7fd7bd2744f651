"""Device backends. There is exactly one: hand-written sm_100a CUDA in librlk_b200.so."""
