"""How the tensor-core kernel of windowed attention (csrc/window_attention_mma.cu) wants the rows of a step cut:
tiles of up to 64 consecutive rows of one request.  The planner hands the tiles to the engine, which uploads them
with the step's own arrays (``parts.base.StepPlanner``)."""
from __future__ import annotations

from typing import Dict, Sequence, Tuple

import torch

from ..parts.base import StepPlanner

TILE_ROWS = 64


class WindowTilePlanner(StepPlanner):
    key = ("window_attention_tiles", TILE_ROWS)

    def max_words(self, rows: int) -> int:
        return 2 * rows                      # at worst every row is a tile of its own

    def plan(self, segments: Sequence[Tuple[int, int]]):
        row0, rows = [], []
        for first, n in segments:
            for a in range(0, n, TILE_ROWS):
                row0.append(first + a)
                rows.append(min(TILE_ROWS, n - a))
        return {"row0": row0, "rows": rows}, len(row0)

    def plan_decode(self, rows: int):
        return {"row0": list(range(rows)), "rows": [1] * rows}, rows

    def bind(self, arrays: Dict[str, torch.Tensor], facts):
        return arrays["row0"], arrays["rows"], int(facts)


_planner = WindowTilePlanner()


def planner() -> WindowTilePlanner:
    return _planner
