"""Validation harness: operator four-judgment matrices, forward/gradient invariance, the model
chain gate, the cross-configuration drift runner with resumable sealed artifacts, and drift reports
(parity: rl_engine/validation)."""
