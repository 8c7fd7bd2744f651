"""Diagnostic matrices: named grids of (case x judgment) cells with pass/fail/blocked status,
serialisable for reports (parity: rl_engine/contracts/diagnostics/*.py)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class Cell:
    status: str = "missing"      # pass | fail | blocked | missing
    detail: str = ""
    value: float | None = None


@dataclass
class DiagnosticMatrix:
    name: str
    rows: list[str]
    cols: list[str]
    cells: dict[tuple[str, str], Cell] = field(default_factory=dict)

    def set(self, row: str, col: str, status: str, detail: str = "", value: float | None = None) -> None:
        if row not in self.rows or col not in self.cols:
            raise KeyError((row, col))
        self.cells[(row, col)] = Cell(status, detail, value)

    def get(self, row: str, col: str) -> Cell:
        return self.cells.get((row, col), Cell())

    @property
    def green(self) -> bool:
        return all(self.get(r, c).status == "pass" for r in self.rows for c in self.cols)

    def red_cells(self) -> list[tuple[str, str, Cell]]:
        return [(r, c, self.get(r, c)) for r in self.rows for c in self.cols if self.get(r, c).status != "pass"]

    def to_dict(self) -> dict:
        return {"name": self.name, "rows": self.rows, "cols": self.cols,
                "cells": {f"{r}|{c}": vars(self.get(r, c)) for r in self.rows for c in self.cols}}

    def render(self) -> str:
        w = max(len(r) for r in self.rows) + 2
        head = " " * w + " ".join(f"{c:>12}" for c in self.cols)
        lines = [head]
        for r in self.rows:
            lines.append(f"{r:<{w}}" + " ".join(f"{self.get(r, c).status:>12}" for c in self.cols))
        return "\n".join(lines)
