"""Runnable examples (parity: examples/ of the reference)."""
