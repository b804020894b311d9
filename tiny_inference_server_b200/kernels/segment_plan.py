"""The first row of every request in a step, for kernels that walk a request's rows in order (a recurrence over
time) and want one CTA per request instead of one per row (``parts.base.StepPlanner``)."""
from __future__ import annotations

from typing import Dict, Sequence, Tuple

import torch

from ..parts.base import StepPlanner


class SegmentPlanner(StepPlanner):
    key = ("segment_first_rows",)

    def max_words(self, rows: int) -> int:
        return rows

    def plan(self, segments: Sequence[Tuple[int, int]]):
        return {"row0": [first for first, _ in segments]}, len(segments)

    def plan_decode(self, rows: int):
        return {"row0": list(range(rows))}, rows

    def bind(self, arrays: Dict[str, torch.Tensor], facts):
        return arrays["row0"], int(facts)


_planner = SegmentPlanner()


def planner() -> SegmentPlanner:
    return _planner
