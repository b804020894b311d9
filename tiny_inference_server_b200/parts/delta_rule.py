"""The delta rule with a decay per head and key channel: a recurrent mixer with a matrix state."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops, segment_plan
from ..registry import register_part
from .base import BuildContext, LayerBinding, Mixer, StateSpec, WeightSpec
from .short_conv import CausalConv
from .window_attention import pad8


class ChannelDeltaRule(Mixer):
    """Per head a state ``S`` (``k_dim x v_dim``, float32, zero at the start of a sequence):

    * ``q = Wq h, k = Wk h`` (``qk_heads`` heads of ``k_dim``), ``v = Wv h`` (``num_heads`` heads of ``v_dim``);
      each through a short causal convolution over time and silu; head h reads q/k head
      ``h // (num_heads / qk_heads)``; q and k to unit length per head (``unit_eps`` inside the root), q
      times ``k_dim ** -0.5``;
    * ``beta = sigmoid(Wb h)`` per head; decay ``g = exp(-exp(A_log[h]) * softplus(Wa2 (Wa1 h) + dt_bias))`` per
      head and key channel;
    * ``S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q`` (o is read from the updated S);
    * ``o / sqrt(mean(o^2) + eps) * norm`` per head (``norm`` of length ``v_dim``, shared by the heads), times
      ``sigmoid(Wg2 (Wg1 h))``; then ``Wo``.

    Tensor names below the prefix: ``q, k, v, o, b, a1, a2, g1, g2`` (stored (out, in)), ``q.conv, k.conv,
    v.conv``, ``A_log``, ``dt_bias``, ``norm``.  The state of a request is S of every head followed by the
    convolution's last inputs."""

    graph_safe = True
    fuses_residual = True
    UNIT_EPS = 1e-6

    def __init__(self, width: int, num_heads: int, qk_heads: int, k_dim: int, v_dim: int, conv_taps: int, eps: float,
                 decay_rank: int, gate_rank: int, prefix: str = ""):
        super().__init__(prefix)
        if num_heads % qk_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {qk_heads} query/key heads")
        self.width, self.num_heads, self.qk_heads, self.k_dim, self.v_dim = width, num_heads, qk_heads, k_dim, v_dim
        self.eps = float(eps)
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        self.nq = qk_heads * k_dim
        self.nv = num_heads * v_dim
        self.na = num_heads * k_dim
        self.conv = CausalConv([self.nq, self.nq, self.nv], conv_taps, ["q.conv", "k.conv", "v.conv"], prefix=prefix,
                               silu=True)
        self.state_matrix = num_heads * k_dim * v_dim
        # columns of the fused input projection: q | k | v | beta | a1 | g1, each block on a multiple of 8
        self.beta_at = pad8(2 * self.nq + self.nv)
        self.low_at = self.beta_at + pad8(num_heads)
        self.cols = self.low_at + pad8(decay_rank + gate_rank)
        self.gate_at = pad8(self.na)            # columns of the second low-rank product: decay | gate
        self.w_in = self.w_low = self.w_o = self.a_log = self.dt_bias = self.norm_w = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int = 0, position=None, ranks=None):
        m = cfg.layers[layer_index]["mixer"]
        decay_rank, gate_rank = ranks if ranks is not None else (m["decay_rank"], m["gate_rank"])
        return cls(cfg.hidden_size, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], cfg.rms_norm_eps,
                   decay_rank, gate_rank, prefix=prefix)

    def children(self):
        return (self.conv,)

    def step_planners(self):
        # the first row of every request of the step: the recurrence launches a CTA per request
        return (segment_plan.planner(),)

    def state_spec(self) -> StateSpec:
        return StateSpec((self.state_matrix + self.conv.state_floats,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            "q": WeightSpec((self.nq, self.width)), "k": WeightSpec((self.nq, self.width)),
            "v": WeightSpec((self.nv, self.width)), "b": WeightSpec((self.num_heads, self.width)),
            "A_log": WeightSpec((self.num_heads,), init="uniform", lo=-1.0, hi=1.0),
            "norm": WeightSpec((self.v_dim,), init="ones_normal"),
            "a1": WeightSpec((self.decay_rank, self.width)), "a2": WeightSpec((self.na, self.decay_rank)),
            "dt_bias": WeightSpec((self.na,), init="uniform", lo=-2.0, hi=1.0),
            "g1": WeightSpec((self.gate_rank, self.width)), "g2": WeightSpec((self.nv, self.gate_rank)),
            "o": WeightSpec((self.width, self.nv)),
        }

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        f32 = dict(device=ctx.device, dtype=torch.float32)
        w = torch.zeros((self.width, self.cols), dtype=ctx.dtype)
        at = 0
        for name, n in (("q", self.nq), ("k", self.nq), ("v", self.nv)):
            w[:, at:at + n] = tensors[p + name].to(ctx.dtype).t()
            at += n
        w[:, self.beta_at:self.beta_at + self.num_heads] = tensors[p + "b"].to(ctx.dtype).t()
        ra, rg = self.decay_rank, self.gate_rank
        w[:, self.low_at:self.low_at + ra] = tensors[p + "a1"].to(ctx.dtype).t()
        w[:, self.low_at + ra:self.low_at + ra + rg] = tensors[p + "g1"].to(ctx.dtype).t()
        self.w_in = w.to(ctx.device).contiguous()
        # the second factors of the two low-rank projections as one block-diagonal matrix
        low = torch.zeros((pad8(ra + rg), self.gate_at + pad8(self.nv)), dtype=ctx.dtype)
        low[:ra, :self.na] = tensors[p + "a2"].to(ctx.dtype).t()
        low[ra:ra + rg, self.gate_at:self.gate_at + self.nv] = tensors[p + "g2"].to(ctx.dtype).t()
        self.w_low = low.to(ctx.device).contiguous()
        self.w_o = tensors[p + "o"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()
        self.a_log = tensors[p + "A_log"].to(**f32).contiguous()
        self.dt_bias = tensors[p + "dt_bias"].to(**f32).contiguous()
        self.norm_w = tensors[p + "norm"].to(**f32).contiguous()

    def forward(self, x, step, binding: LayerBinding, residual=None):
        n = x.shape[0]
        proj = ops.gemm(x, self.w_in)
        nqkv = 2 * self.nq + self.nv
        qkv = self.conv.forward(proj[:, :nqkv], step, binding.state[:, self.state_matrix:])
        low = ops.gemm(proj[:, self.low_at:], self.w_low)
        out = torch.empty((n, self.nv), dtype=x.dtype, device=x.device)
        ops.delta_rule(qkv, proj[:, self.beta_at:self.beta_at + self.num_heads], low[:, :self.na],
                       low[:, self.gate_at:self.gate_at + self.nv], self.a_log, self.dt_bias, self.norm_w, self.eps,
                       self.UNIT_EPS, self.k_dim ** -0.5, binding.state, out, step.row_slot, step.row_last,
                       self.num_heads, self.qk_heads, self.k_dim, self.v_dim, requests=len(step.segments),
                       segments=step.plan(segment_plan.planner()))
        return ops.gemm(out, self.w_o, sink=residual)


class HeadDecayDeltaRule(Mixer):
    """The delta rule with one decay per head and token, and a full-rank gate.  Per head a state ``S``
    (``k_dim x v_dim``, float32, zero at the start of a sequence):

    * ``q = Wq h, k = Wk h`` (``qk_heads`` heads of ``k_dim``), ``v = Wv h`` (``num_heads`` heads of ``v_dim``);
      each through a short causal convolution over time and silu; head h reads q/k head
      ``h // (num_heads / qk_heads)``; q and k to unit length per head (``unit_eps`` inside the root), q
      times ``k_dim ** -0.5``;
    * ``beta = sigmoid(Wb h)`` and ``g = exp(-exp(A_log[h]) * softplus(Wa h + dt_bias[h]))``, one number each
      per head;
    * ``S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q`` (o is read from the updated S);
    * ``o / sqrt(mean(o^2) + eps) * norm`` per head (``norm`` of length ``v_dim``, shared by the heads), times
      ``gate_act(Wg h)`` with ``gate_act`` ``silu`` or ``sigmoid``; then ``Wo``.

    Tensor names below the prefix: ``q, k, v, o, b, a, g`` (stored (out, in)), ``q.conv, k.conv, v.conv``,
    ``A_log``, ``dt_bias``, ``norm``.  The state of a request is S of every head followed by the
    convolution's last inputs.  Decay, beta, unit norms, the recurrence and the output norm are computed in
    32-bit by the same kernels as ``ChannelDeltaRule``."""

    graph_safe = True
    fuses_residual = True
    UNIT_EPS = 1e-6

    def __init__(self, width: int, num_heads: int, qk_heads: int, k_dim: int, v_dim: int, conv_taps: int, eps: float,
                 gate_act: str = "silu", prefix: str = ""):
        super().__init__(prefix)
        if num_heads % qk_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {qk_heads} query/key heads")
        if gate_act not in ops.GATE_ACTS:
            raise ValueError(f"gate activation {gate_act!r}: one of {sorted(ops.GATE_ACTS)}")
        self.width, self.num_heads, self.qk_heads, self.k_dim, self.v_dim = width, num_heads, qk_heads, k_dim, v_dim
        self.eps, self.gate_act = float(eps), gate_act
        self.nq = qk_heads * k_dim
        self.nv = num_heads * v_dim
        self.conv = CausalConv([self.nq, self.nq, self.nv], conv_taps, ["q.conv", "k.conv", "v.conv"], prefix=prefix,
                               silu=True)
        self.state_matrix = num_heads * k_dim * v_dim
        # columns of the fused input projection: q | k | v | beta | a | gate, each block on a multiple of 8
        self.beta_at = pad8(2 * self.nq + self.nv)
        self.decay_at = self.beta_at + pad8(num_heads)
        self.gate_at = self.decay_at + pad8(num_heads)
        self.cols = self.gate_at + pad8(self.nv)
        self.w_in = self.w_o = self.a_log = self.dt_bias = self.norm_w = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int = 0, position=None):
        m = cfg.layers[layer_index]["mixer"]
        return cls(cfg.hidden_size, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], cfg.rms_norm_eps,
                   prefix=prefix)

    def children(self):
        return (self.conv,)

    def step_planners(self):
        return (segment_plan.planner(),)

    def state_spec(self) -> StateSpec:
        return StateSpec((self.state_matrix + self.conv.state_floats,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            "q": WeightSpec((self.nq, self.width)), "k": WeightSpec((self.nq, self.width)),
            "v": WeightSpec((self.nv, self.width)), "b": WeightSpec((self.num_heads, self.width)),
            "A_log": WeightSpec((self.num_heads,), init="uniform", lo=-1.0, hi=1.0),
            "norm": WeightSpec((self.v_dim,), init="ones_normal"),
            "a": WeightSpec((self.num_heads, self.width)),
            "dt_bias": WeightSpec((self.num_heads,), init="uniform", lo=-2.0, hi=1.0),
            "g": WeightSpec((self.nv, self.width)), "o": WeightSpec((self.width, self.nv)),
        }

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        f32 = dict(device=ctx.device, dtype=torch.float32)
        w = torch.zeros((self.width, self.cols), dtype=ctx.dtype)
        at = 0
        for name, n in (("q", self.nq), ("k", self.nq), ("v", self.nv)):
            w[:, at:at + n] = tensors[p + name].to(ctx.dtype).t()
            at += n
        w[:, self.beta_at:self.beta_at + self.num_heads] = tensors[p + "b"].to(ctx.dtype).t()
        w[:, self.decay_at:self.decay_at + self.num_heads] = tensors[p + "a"].to(ctx.dtype).t()
        w[:, self.gate_at:self.gate_at + self.nv] = tensors[p + "g"].to(ctx.dtype).t()
        self.w_in = w.to(ctx.device).contiguous()
        self.w_o = tensors[p + "o"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()
        self.a_log = tensors[p + "A_log"].to(**f32).contiguous()
        self.dt_bias = tensors[p + "dt_bias"].to(**f32).contiguous()
        self.norm_w = tensors[p + "norm"].to(**f32).contiguous()

    def forward(self, x, step, binding: LayerBinding, residual=None):
        n = x.shape[0]
        proj = ops.gemm(x, self.w_in)
        nqkv = 2 * self.nq + self.nv
        qkv = self.conv.forward(proj[:, :nqkv], step, binding.state[:, self.state_matrix:])
        out = torch.empty((n, self.nv), dtype=x.dtype, device=x.device)
        ops.delta_rule(qkv, proj[:, self.beta_at:self.beta_at + self.num_heads],
                       proj[:, self.decay_at:self.decay_at + self.num_heads],
                       proj[:, self.gate_at:self.gate_at + self.nv], self.a_log, self.dt_bias, self.norm_w, self.eps,
                       self.UNIT_EPS, self.k_dim ** -0.5, binding.state, out, step.row_slot, step.row_last,
                       self.num_heads, self.qk_heads, self.k_dim, self.v_dim, requests=len(step.segments),
                       segments=step.plan(segment_plan.planner()), decay_per_head=True, gate_act=self.gate_act)
        return ops.gemm(out, self.w_o, sink=residual)


register_part("mixer", "channel_delta_rule", ChannelDeltaRule)
register_part("mixer", "head_decay_delta_rule", HeadDecayDeltaRule)
