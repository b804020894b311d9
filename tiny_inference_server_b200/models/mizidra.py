"""The Mizidra decoder, put together from parts: an embedding that passes a norm of its own before it starts the
residual stream; pre-norm layers, each with one of three mixers (the delta rule with a decay per head, attention
over compressed keys and values, linear attention with a constant decay) and, where the layer has one, a routed
mixture of gated units; final norm; an output matrix of its own.

Tensor names::

    embed                        (vocab, width)
    embed.norm                   (width,)
    l<i>.norm1, l<i>.norm2       (width,)          plain weights
    l<i>.mix.*                   the mixer's tensors (``parts.delta_rule.HeadDecayDeltaRule``,
                                 ``parts.latent_attention.LatentAttention``, ``parts.linear_attention.DecayLinearAttention``)
    l<i>.mlp.*                   the feed-forward's tensors (``parts.feed_forward.RoutedExperts``)
    final.norm                   (width,)
    head                         (vocab, width)

Linear weights are stored ``(out, in)``.
"""
from __future__ import annotations

from typing import List

from ..config.model_config import MizidraConfig
from ..parts.block import Block
from ..parts.delta_rule import HeadDecayDeltaRule
from ..parts.embedding import Embedding, LMHead
from ..parts.feed_forward import RoutedExperts
from ..parts.latent_attention import LatentAttention
from ..parts.linear_attention import DecayLinearAttention
from ..parts.norms import RMSNormMeanEps
from ..parts.stream import ResidualStream
from ..registry import register_architecture
from .base import Model, ScheduleEntry, StepOutput

#: ``layers[i].type`` of config.json -> the mixer part
MIXER_OF_TYPE = {"delta": HeadDecayDeltaRule, "latent_attention": LatentAttention, "lightning": DecayLinearAttention}


class MizidraModel(Model):
    def __init__(self, cfg: MizidraConfig):
        super().__init__()
        self.config = cfg
        self.vocab_size = cfg.vocab_size
        self.max_positions = cfg.max_context
        width, eps = cfg.hidden_size, cfg.rms_norm_eps
        self.embedding = Embedding(cfg.vocab_size, width, weight_name="embed")
        self.embed_norm = RMSNormMeanEps(width, eps, prefix="embed.norm", weight_name="", keep_f32=True)
        self.blocks: List[Block] = []
        for i, layer in enumerate(cfg.layers):
            p = f"l{i}."
            mixer = MIXER_OF_TYPE[layer["type"]].from_config(cfg, prefix=p + "mix.", layer_index=i)
            has_ff = layer.get("mlp") is not None
            self.blocks.append(Block(
                RMSNormMeanEps(width, eps, prefix=p + "norm1", weight_name=""),
                mixer,
                RMSNormMeanEps(width, eps, prefix=p + "norm2", weight_name="") if has_ff else None,
                RoutedExperts.from_config(cfg, prefix=p + "mlp.", layer_index=i) if has_ff else None,
                prefix=p))
        self.final_norm = RMSNormMeanEps(width, eps, prefix="final.norm", weight_name="")
        self.lm_head = LMHead(cfg.vocab_size, width, None, weight_name="head")
        self.entries = [ScheduleEntry(b) for b in self.blocks]

    def top_parts(self):
        return [self.embedding, self.embed_norm, *self.blocks, self.final_norm, self.lm_head]

    def forward(self, step, want_rows, aux: bool = False) -> StepOutput:
        # the stream starts as the normed embedding, in 32-bit
        stream = ResidualStream(self.embed_norm.forward(self.embedding.forward(step.tokens)))
        for e in self.entries:
            e.block.forward(stream, step, e.binding)
        h = stream.normed(self.final_norm)
        if not getattr(step, "want_identity", False):
            h = h.index_select(0, want_rows)
        return StepOutput(main=self.lm_head.forward(h))


def build(cfg: MizidraConfig) -> MizidraModel:
    return MizidraModel(cfg)


register_architecture(MizidraConfig.architecture, MizidraConfig, build)
