"""A short causal convolution over time on each channel, with per-request state."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from ..kernels import ops
from .base import BuildContext, Part, StateSpec, WeightSpec


class CausalConv(Part):
    """``y_t = [x_t +] sum_j w[:, j] * x_(t - taps + 1 + j)``, optionally through silu: the last column of
    ``w`` weighs the current position, inputs before the start of a sequence are zero, no bias.  The last
    ``taps - 1`` inputs of a request are its state (float32, ``state_floats`` per request), so that a step
    may bring any part of a sequence, down to one token.

    ``weight_names``: the tensors ``(channels_i, taps)`` whose channels lie one after the other in the
    rows this part is given (the projections of a mixer, convolved in one launch).  Used alone in front
    of a mixer (``residual=True``: the block's input filter) or inside a mixer on its projections."""

    def __init__(self, channels: Sequence[int], taps: int, weight_names: Sequence[str], prefix: str = "",
                 residual: bool = False, silu: bool = False):
        super().__init__(prefix)
        if not (1 <= taps <= 16):
            raise ValueError(f"a short convolution of {taps} taps: the kernel takes 1..16")
        self.sections = list(channels)
        self.channels = sum(self.sections)
        self.taps = taps
        self.weight_names = list(weight_names)
        self.residual = residual
        self.silu = silu
        self.weight: Optional[torch.Tensor] = None

    @property
    def state_floats(self) -> int:
        return (self.taps - 1) * self.channels

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((max(1, self.state_floats),), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {name: WeightSpec((c, self.taps)) for name, c in zip(self.weight_names, self.sections)}

    def load(self, tensors, ctx: BuildContext) -> None:
        w = torch.cat([tensors[self.prefix + name].to(torch.float32) for name in self.weight_names], dim=0)
        self.weight = w.t().contiguous().to(ctx.device)            # tap by tap: (taps, channels)

    def forward(self, x: torch.Tensor, step, state: torch.Tensor) -> torch.Tensor:
        """``x`` (n, channels), row stride free; ``state`` (slots, >= state_floats) float32."""
        out = torch.empty((x.shape[0], self.channels), dtype=x.dtype, device=x.device)
        return ops.causal_conv(x, self.weight, state, out, step.row_slot, step.row_last, residual=self.residual,
                               silu=self.silu)
