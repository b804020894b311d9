"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import BuildContext, FeedForward, WeightSpec


class SwiGLU(FeedForward):
    """``(silu(x W1) * (x W2)) W3`` (upstream ``swiglu`` and ``ffn_router``,
    main_models_new.py:44-60); weights ``(in, out)``: W1 gate and W2 up ``(width, hidden)``,
    W3 ``(hidden, width)``.  On the device gate and up are one matrix ``(width, 2*hidden)``
    whose columns alternate in blocks of 32 gates and 32 ups (when 32 divides the hidden size;
    else all gates, then all ups), so that one 64-column strip of the product holds both
    factors of 32 outputs and the gating can be the product's epilogue."""

    accepts_scaled_rows = True
    fuses_residual = True

    def __init__(self, width: int, hidden: int, prefix: str = "", names: Optional[Dict[str, str]] = None):
        super().__init__(prefix)
        self.width = width
        self.hidden = hidden
        self.names = {"gate": "swig.linear1.weight", "up": "swig.linear2.weight", "down": "fc.weight"}
        if names:
            self.names.update(names)
        self.w_gate_up = None
        self.w_down = None
        self.block = hidden

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int):
        return cls(cfg.hidden_size, cfg.ffn_hidden, prefix=prefix)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            self.names["gate"]: WeightSpec((self.width, self.hidden)),
            self.names["up"]: WeightSpec((self.width, self.hidden)),
            self.names["down"]: WeightSpec((self.hidden, self.width)),
        }

    def load(self, tensors, ctx: BuildContext) -> None:
        gate = tensors[self.prefix + self.names["gate"]]
        up = tensors[self.prefix + self.names["up"]]
        self.block = 32 if self.hidden % 32 == 0 else self.hidden
        nb = self.hidden // self.block
        both = torch.stack([gate.reshape(self.width, nb, self.block), up.reshape(self.width, nb, self.block)], dim=2)
        self.w_gate_up = both.reshape(self.width, 2 * self.hidden).to(device=ctx.device, dtype=ctx.dtype).contiguous()
        self.w_down = tensors[self.prefix + self.names["down"]].to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, x, step=None, residual=None):
        h = ops.gemm_swiglu(x, self.w_gate_up, self.hidden, self.block)
        return ops.gemm(h, self.w_down, sink=residual)


class ClampedGLU(FeedForward):
    """``g = min(W_gate h + b, limit)``, ``u = clamp(W_up h + b, -limit, limit)``,
    ``y = g * sigmoid(alpha * g) * (u + shift)``, output ``W_down y + b``.  Weights stored ``(out, in)``,
    names ``gate, up, down`` with biases ``gate.b, up.b, down.b``.  On the device gate and up are one matrix;
    the bias of the down projection is one more row of its matrix, met by a column of ones that the gating
    kernel writes, so that the product adds it."""

    accepts_scaled_rows = True

    def __init__(self, width: int, hidden: int, limit: float, alpha: float = 1.702, shift: float = 1.0,
                 prefix: str = ""):
        super().__init__(prefix)
        self.width, self.hidden = width, hidden
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        self.padded = (hidden + 1 + 7) // 8 * 8
        self.w_gate_up = self.w_down = self.b_gate = self.b_up = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int):
        f = cfg.layers[layer_index]["mlp"]
        return cls(cfg.hidden_size, f["ff"], f.get("limit", 0.0), prefix=prefix)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            "gate": WeightSpec((self.hidden, self.width)), "gate.b": WeightSpec((self.hidden,)),
            "up": WeightSpec((self.hidden, self.width)), "up.b": WeightSpec((self.hidden,)),
            "down": WeightSpec((self.width, self.hidden)), "down.b": WeightSpec((self.width,)),
        }

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        gu = torch.cat([tensors[p + "gate"], tensors[p + "up"]], dim=0).to(ctx.dtype).t()
        self.w_gate_up = gu.to(ctx.device).contiguous()
        down = torch.zeros((self.padded, self.width), dtype=ctx.dtype)
        down[:self.hidden] = tensors[p + "down"].to(ctx.dtype).t()
        down[self.hidden] = tensors[p + "down.b"].to(ctx.dtype)
        self.w_down = down.to(ctx.device).contiguous()
        self.b_gate = tensors[p + "gate.b"].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.b_up = tensors[p + "up.b"].to(device=ctx.device, dtype=torch.float32).contiguous()

    def forward(self, x, step=None):
        gu = ops.gemm(x, self.w_gate_up)
        y = torch.empty((gu.shape[0], self.padded), dtype=gu.dtype, device=gu.device)
        ops.glu_clamped(gu, self.b_gate, self.b_up, self.limit, self.alpha, self.shift, y, self.hidden)
        return ops.gemm(y, self.w_down)


register_part("ffn", "swiglu", SwiGLU)
register_part("ffn", "clamped_glu", ClampedGLU)
