"""The Kefisun decoder, put together from parts: scaled embedding; pre-norm layers, each a mixer
(windowed attention with a logarithmic distance bias, or the delta rule with a decay per key channel)
behind a short causal convolution of its input, and a clamped gated feed-forward where the layer has one;
final norm; logits from the embedding matrix, scaled.

Tensor names::

    embed                        (vocab, width)
    l<i>.norm1, l<i>.norm2       (width,)          an offset from one: the norm multiplies by 1 + w
    l<i>.canon1                  (width, taps)     the convolution in front of the mixer
    l<i>.mix.*                   the mixer's tensors (``parts.window_attention``, ``parts.delta_rule``)
    l<i>.mlp.*                   the feed-forward's tensors (``parts.feed_forward.ClampedGLU``)
    final.norm                   (width,)

Linear weights are stored ``(out, in)``.
"""
from __future__ import annotations

from typing import List

from ..config.model_config import KefisunConfig
from ..parts.block import Block
from ..parts.delta_rule import ChannelDeltaRule
from ..parts.embedding import Embedding, LMHead
from ..parts.feed_forward import ClampedGLU
from ..parts.norms import RMSNormOnePlus
from ..parts.short_conv import CausalConv
from ..parts.stream import ResidualStream
from ..parts.window_attention import BiasedWindowAttention, ValueShare
from ..registry import register_architecture
from .base import Model, ScheduleEntry, StepOutput


class KefisunModel(Model):
    def __init__(self, cfg: KefisunConfig):
        super().__init__()
        self.config = cfg
        self.vocab_size = cfg.vocab_size
        self.max_positions = cfg.max_context
        width, eps = cfg.hidden_size, cfg.rms_norm_eps
        self.embedding = Embedding(cfg.vocab_size, width, weight_name="embed", scale=cfg.embedding_scale)
        share = ValueShare()
        shared = False
        self.blocks: List[Block] = []
        for i, layer in enumerate(cfg.layers):
            p = f"l{i}."
            if layer["type"] == "attention":
                mixes = bool(layer["mixer"].get("v_mix"))
                mixer = BiasedWindowAttention.from_config(cfg, prefix=p + "mix.", layer_index=i, value_share=share,
                                                          shares_first=mixes and not shared)
                shared = shared or mixes
            else:
                m = layer["mixer"]
                if "decay_rank" not in m or "gate_rank" not in m:
                    raise ValueError(f"layers[{i}].mixer: the ranks of the low-rank projections are not known "
                                     f"(read the configuration with registry.config_from_folder)")
                mixer = ChannelDeltaRule.from_config(cfg, prefix=p + "mix.", layer_index=i)
            has_ff = layer.get("mlp") is not None
            filt = None
            if cfg.canon_taps is not None:
                filt = CausalConv([width], cfg.canon_taps, ["canon1"], prefix=p, residual=True)
            self.blocks.append(Block(
                RMSNormOnePlus(width, eps, prefix=p + "norm1", weight_name=""),
                mixer,
                RMSNormOnePlus(width, eps, prefix=p + "norm2", weight_name="") if has_ff else None,
                ClampedGLU.from_config(cfg, prefix=p + "mlp.", layer_index=i) if has_ff else None,
                prefix=p, input_filter=filt))
        self.final_norm = RMSNormOnePlus(width, eps, prefix="final.norm", weight_name="")
        self.lm_head = LMHead(cfg.vocab_size, width, self.embedding, logit_scale=cfg.logit_scale)
        self.entries = [ScheduleEntry(b) for b in self.blocks]

    def top_parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.lm_head]

    def forward(self, step, want_rows, aux: bool = False) -> StepOutput:
        stream = ResidualStream(self.embedding.forward(step.tokens))
        for e in self.entries:
            e.block.forward(stream, step, e.binding)
        h = stream.normed(self.final_norm)
        if not getattr(step, "want_identity", False):
            h = h.index_select(0, want_rows)
        return StepOutput(main=self.lm_head.forward(h))


def build(cfg: KefisunConfig) -> KefisunModel:
    return KefisunModel(cfg)


register_architecture(KefisunConfig.architecture, KefisunConfig, build)
