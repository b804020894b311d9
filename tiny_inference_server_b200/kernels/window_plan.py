"""How the tensor-core kernel of windowed attention (csrc/window_attention_mma.cu) wants the rows of a step cut:
tiles of consecutive rows of one request, as many as make 64 rows together with the query heads that share a kv head
(64 // group size).  The planner hands the tiles to the engine, which uploads them with the step's own arrays
(``parts.base.StepPlanner``)."""
from __future__ import annotations

from typing import Dict, Sequence, Tuple

import torch

from ..parts.base import StepPlanner

PACKED_ROWS = 64


class WindowTilePlanner(StepPlanner):
    def __init__(self, tile_rows: int):
        self.tile_rows = tile_rows
        self.key = ("window_attention_tiles", tile_rows)

    def max_words(self, rows: int) -> int:
        return 2 * rows                      # at worst every row is a tile of its own

    def plan(self, segments: Sequence[Tuple[int, int]]):
        row0, rows = [], []
        for first, n in segments:
            for a in range(0, n, self.tile_rows):
                row0.append(first + a)
                rows.append(min(self.tile_rows, n - a))
        return {"row0": row0, "rows": rows}, len(row0)

    def plan_decode(self, rows: int):
        return {"row0": list(range(rows)), "rows": [1] * rows}, rows

    def bind(self, arrays: Dict[str, torch.Tensor], facts):
        return arrays["row0"], arrays["rows"], int(facts)


_planners: Dict[int, WindowTilePlanner] = {}


def planner(group_size: int) -> WindowTilePlanner:
    """The planner for mixers with ``group_size`` query heads per kv head (at most 64)."""
    rows = max(1, PACKED_ROWS // group_size)
    if rows not in _planners:
        _planners[rows] = WindowTilePlanner(rows)
    return _planners[rows]
