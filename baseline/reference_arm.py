"""Reference arm of bench.py: runs the unmodified reference installed under baseline/_ref."""
from __future__ import annotations


def run_reference(args) -> dict:
    return {"impl": "reference", "unavailable": "reference arm not wired yet"}
