"""Attention over a window of the paged cache with a logarithmic distance bias."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops, window_plan
from ..registry import register_part
from .base import BuildContext, KVSpec, LayerBinding, Mixer, StateSpec, WeightSpec
from .short_conv import CausalConv


class ValueShare:
    """What the layers that mix their values share: the values of the first of them, for the rows of the
    step that is running (kept with the step, so that steps do not see each other's)."""

    def put(self, step, values: torch.Tensor) -> None:
        step.scratch[("value_share", id(self))] = values

    def get(self, step) -> torch.Tensor:
        return step.scratch[("value_share", id(self))]


def pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class BiasedWindowAttention(Mixer):
    """Grouped-query attention without rotation; positions enter through the window and through a bias.

    * ``q = Wq h, k = Wk h, v = Wv h`` (no biases), key/query width ``k_dim``, value width ``v_dim``;
    * ``conv_taps``: a short causal convolution over time on every channel of q, k and v (None: none);
    * ``qk_norm``: q and k, each as a whole (all heads at once), are divided by their root mean square
      (``eps`` inside the root) and multiplied by a weight of that length;
    * ``score = q . k * scale - r1[h] * ln(1 + r2[h] * (i - j))`` (``distance_bias``), keys
      ``i - window < j <= i``, softmax;
    * ``value_share``: v <- (1 - lambda) v + lambda v_first in every sharing layer but the first, whose
      values of the same token v_first is; the mixed values are what the cache holds;
    * ``gated``: the heads' outputs times ``sigmoid(Wg h)`` element by element; then ``Wo``.

    Tensor names below the prefix: ``q, k, v, o`` (stored (out, in)), ``q.conv, k.conv, v.conv``,
    ``q.norm, k.norm``, ``r1, r2``, ``vmix``, ``g``."""

    graph_safe = True
    fuses_residual = True

    def __init__(self, width: int, num_heads: int, kv_heads: int, k_dim: int, v_dim: int, scale: float,
                 window: Optional[int], eps: float, conv_taps: Optional[int] = None, qk_norm: bool = True,
                 distance_bias: bool = True, gated: bool = True, value_share: Optional[ValueShare] = None,
                 shares_first: bool = False, prefix: str = ""):
        super().__init__(prefix)
        if num_heads % kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {kv_heads} kv heads")
        self.width, self.num_heads, self.kv_heads, self.k_dim, self.v_dim = width, num_heads, kv_heads, k_dim, v_dim
        self.scale, self.window, self.eps = float(scale), window, float(eps)
        self.qk_norm, self.distance_bias, self.gated = qk_norm, distance_bias, gated
        self.value_share, self.shares_first = value_share, shares_first
        self.nq, self.nk, self.nv = num_heads * k_dim, kv_heads * k_dim, kv_heads * v_dim
        self.no = num_heads * v_dim
        self.conv = None
        if conv_taps is not None:
            self.conv = CausalConv([self.nq, self.nk, self.nv], conv_taps, ["q.conv", "k.conv", "v.conv"], prefix=prefix)
        self.gate_at = pad8(self.nq + self.nk + self.nv)
        self.w_in = self.w_o = self.q_weight = self.k_weight = self.r1 = self.r2 = self.mix = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int = 0, position=None, value_share=None,
                    shares_first: bool = False):
        m = cfg.layers[layer_index]["mixer"]
        mask = m.get("mask")
        return cls(cfg.hidden_size, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"],
                   mask["size"] if mask else None, cfg.rms_norm_eps, conv_taps=m.get("conv"),
                   value_share=value_share if m.get("v_mix") else None, shares_first=shares_first, prefix=prefix)

    def children(self):
        return (self.conv,) if self.conv is not None else ()

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.kv_heads, self.k_dim, self.window, 0, k_dim=self.k_dim, v_dim=self.v_dim)

    def state_spec(self) -> Optional[StateSpec]:
        return self.conv.state_spec() if self.conv is not None else None

    def step_planners(self):
        # the tiles of rows that the tensor-core kernel takes
        return (window_plan.planner(self.num_heads // self.kv_heads),)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"q": WeightSpec((self.nq, self.width)), "k": WeightSpec((self.nk, self.width)),
                 "v": WeightSpec((self.nv, self.width)), "o": WeightSpec((self.width, self.no))}
        if self.qk_norm:
            specs["q.norm"] = WeightSpec((self.nq,), init="ones_normal")
            specs["k.norm"] = WeightSpec((self.nk,), init="ones_normal")
        if self.distance_bias:
            specs["r1"] = WeightSpec((self.num_heads,), init="uniform", lo=0.1, hi=1.0)
            specs["r2"] = WeightSpec((self.num_heads,), init="uniform", lo=0.1, hi=2.0)
        if self.value_share is not None:
            specs["vmix"] = WeightSpec((), init="uniform", lo=0.2, hi=0.8)
        if self.gated:
            specs["g"] = WeightSpec((self.no, self.width))
        return specs

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        f32 = dict(device=ctx.device, dtype=torch.float32)
        cols = self.gate_at + (pad8(self.no) if self.gated else 0)
        w = torch.zeros((self.width, cols), dtype=ctx.dtype)
        at = 0
        for name, n in (("q", self.nq), ("k", self.nk), ("v", self.nv)):
            w[:, at:at + n] = tensors[p + name].to(ctx.dtype).t()
            at += n
        if self.gated:
            w[:, self.gate_at:self.gate_at + self.no] = tensors[p + "g"].to(ctx.dtype).t()
        self.w_in = w.to(ctx.device).contiguous()
        self.w_o = tensors[p + "o"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()
        if self.qk_norm:
            self.q_weight = tensors[p + "q.norm"].to(**f32).contiguous()
            self.k_weight = tensors[p + "k.norm"].to(**f32).contiguous()
        if self.distance_bias:
            self.r1 = tensors[p + "r1"].to(**f32).contiguous()
            self.r2 = tensors[p + "r2"].to(**f32).contiguous()
        if self.value_share is not None:
            self.mix = tensors[p + "vmix"].to(**f32).reshape(1).contiguous()

    def forward(self, x, step, binding: LayerBinding, residual=None):
        n = x.shape[0]
        g = binding.kv_group
        table, page_size = step.block_tables[g], step.page_sizes[g]
        proj = ops.gemm(x, self.w_in)
        nqkv = self.nq + self.nk + self.nv
        qkv = self.conv.forward(proj[:, :nqkv], step, binding.state) if self.conv is not None else proj[:, :nqkv]
        other = None
        if self.value_share is not None:
            if self.shares_first:
                self.value_share.put(step, qkv[:, self.nq + self.nk:])
            else:
                other = self.value_share.get(step)
        ops.norm_mix_store(qkv, self.nq, self.nk, self.nv, self.q_weight, self.k_weight, self.eps, other, self.mix,
                           binding.k_pages, binding.v_pages, table, step.positions, step.row_slot, page_size, step.fault)
        out = torch.empty((n, self.no), dtype=x.dtype, device=x.device)
        gate = proj[:, self.gate_at:self.gate_at + self.no] if self.gated else None
        ops.window_attention(qkv[:, :self.nq], gate, out, binding.k_pages, binding.v_pages, table, step.positions,
                             step.row_slot, self.num_heads, page_size, self.window, self.scale, self.r1, self.r2,
                             step.fault, step)
        return ops.gemm(out, self.w_o, sink=residual)


register_part("mixer", "biased_window_attention", BiasedWindowAttention)
