"""Linear attention with a constant decay per head: a recurrent mixer with a matrix state and no softmax."""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from ..kernels import ops, segment_plan
from ..registry import register_part
from .base import BuildContext, LayerBinding, Mixer, StateSpec, WeightSpec
from .window_attention import pad8


class DecayLinearAttention(Mixer):
    """Per head a state ``S`` (``k_dim x v_dim``, float32, zero at the start of a sequence):

    * ``q = act(Wq h), k = act(Wk h)`` (``num_heads`` heads of ``k_dim``), ``v = act(Wv h)`` (heads of ``v_dim``),
      ``act`` = silu;
    * ``S <- decay[head] S + k v^T;  o = S^T q`` (o is read from the updated S; no other scale);
    * the heads' outputs side by side are divided by their root mean square over all of them (``eps`` inside the
      root), multiplied by ``norm`` (one weight per element) and by ``sigmoid(Wg h)``; then ``Wo``.

    ``decay``: one constant in (0, 1] per head.  Tensor names below the prefix: ``q, k, v, g, o`` (stored
    (out, in)) and ``norm``.  The state, the recurrence and the norm are 32-bit."""

    graph_safe = True
    fuses_residual = True

    def __init__(self, width: int, num_heads: int, k_dim: int, v_dim: int, decay: Sequence[float], eps: float,
                 prefix: str = ""):
        super().__init__(prefix)
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decay constants for {num_heads} heads")
        self.width, self.num_heads, self.k_dim, self.v_dim = width, num_heads, k_dim, v_dim
        self.decay_values = [float(d) for d in decay]
        self.eps = float(eps)
        self.nq = num_heads * k_dim
        self.nv = num_heads * v_dim
        self.gate_at = pad8(2 * self.nq + self.nv)          # columns of the fused input projection: q | k | v | gate
        self.cols = self.gate_at + pad8(self.nv)
        self.w_in = self.w_o = self.decay = self.norm_w = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int = 0, position=None):
        m = cfg.layers[layer_index]["mixer"]
        return cls(cfg.hidden_size, m["heads"], m["dim"], m["vdim"], m["decay"], cfg.rms_norm_eps, prefix=prefix)

    def step_planners(self):
        return (segment_plan.planner(),)

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_heads * self.k_dim * self.v_dim,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"q": WeightSpec((self.nq, self.width)), "k": WeightSpec((self.nq, self.width)),
                "v": WeightSpec((self.nv, self.width)), "g": WeightSpec((self.nv, self.width)),
                "norm": WeightSpec((self.nv,), init="ones_normal"), "o": WeightSpec((self.width, self.nv))}

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        w = torch.zeros((self.width, self.cols), dtype=ctx.dtype)
        at = 0
        for name, n in (("q", self.nq), ("k", self.nq), ("v", self.nv)):
            w[:, at:at + n] = tensors[p + name].to(ctx.dtype).t()
            at += n
        w[:, self.gate_at:self.gate_at + self.nv] = tensors[p + "g"].to(ctx.dtype).t()
        self.w_in = w.to(ctx.device).contiguous()
        self.w_o = tensors[p + "o"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()
        self.norm_w = tensors[p + "norm"].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(device=ctx.device, dtype=torch.float32)

    def forward(self, x, step, binding: LayerBinding, residual=None):
        n = x.shape[0]
        proj = ops.gemm(x, self.w_in)
        out = torch.empty((n, self.nv), dtype=x.dtype, device=x.device)
        ops.linear_attention(proj[:, :2 * self.nq + self.nv], proj[:, self.gate_at:self.gate_at + self.nv], self.decay,
                             self.norm_w, self.eps, binding.state, out, step.row_slot, step.row_last, self.num_heads,
                             self.k_dim, self.v_dim, requests=len(step.segments),
                             segments=step.plan(segment_plan.planner()))
        return ops.gemm(out, self.w_o, sink=residual)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
