"""The Turudra decoder as a list of parts chosen from its configuration.

Fixed by the design: every layer is a parallel block (one RMSNorm; mixer and feed-forward read its output; their sum,
times the residual multiplier, is added to the stream); the experts' activation is the clamped gate
g' sigmoid(1.702 g') (u' + 1); the looped span of layers re-enters through a product over [stream; embedding].
Everything else -- sizes, the order and kinds of the layers, the loop, the constants -- comes from the configuration.
Tensor names: embed, loop.in, l<i>.norm1, l<i>.mix.*, l<i>.mlp.{router, e<j>.{gate,up,down}, shared.{gate,up,down}},
final.norm, head.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.turudra import NAME, LatentAttentionConfig, MLSTMConfig, TurudraConfig
from ..engine.model import ModelPlan, ScheduleEntry
from ..parts import (Embedding, GatedFeedForward, Head, LatentAttention, MLSTM, ParallelBlock, RMSNorm, Rope, RoutedExperts,
                     StreamJoin)

# no position table limits a request's length: the rotation takes any position and the recurrence has none
MAX_POSITIONS = 1 << 30


def build_turudra(cfg: TurudraConfig) -> ModelPlan:
    W, eps = cfg.width, cfg.norm_eps
    embedding = Embedding(cfg.vocab, W, "embed", scale=cfg.embedding_scale)
    blocks = []
    for i, lay in enumerate(cfg.layers):
        p = f"l{i}."
        m = lay.mixer
        if isinstance(m, LatentAttentionConfig):
            rope = Rope(m.rot_dim, m.rot_base, rotary_dim=m.rot_dims)
            mixer = LatentAttention(W, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.scale, rope, eps, prefix=p + "mix.")
        elif isinstance(m, MLSTMConfig):
            mixer = MLSTM(W, m.heads, m.dim, m.vdim, m.gate_cap, eps, prefix=p + "mix.")
        else:
            raise ValueError(f"layer {i}: unknown mixer configuration {type(m).__name__}")
        ff = None
        if lay.mlp is not None:
            f = lay.mlp
            shared = None
            if f.shared is not None:
                shared = GatedFeedForward(W, f.shared.ff, p + "mlp.shared.", "swish_clamp", gate="gate", up="up", down="down",
                                          limit=f.shared.limit)
            ff = RoutedExperts(W, f.experts, f.top, f.expert.ff, p + "mlp.", "swish_clamp", f.expert.limit, shared=shared)
        blocks.append(ParallelBlock(RMSNorm(W, eps, p + "norm1"), mixer, ff, cfg.residual_mult))
    stream_parts = [StreamJoin(W, "loop.in")] if cfg.loop is not None else []
    schedule = [ScheduleEntry(layer=i, before=0 if first else None) for i, first in cfg.layer_runs()]
    return ModelPlan(embedding=embedding, blocks=blocks, schedule=schedule, final_norm=RMSNorm(W, eps, "final.norm"),
                     head=Head(cfg.vocab, W, name="head", softcap=cfg.logit_softcap), width=W, vocab_size=cfg.vocab,
                     max_positions=MAX_POSITIONS, stream_parts=stream_parts)


register_architecture(NAME, TurudraConfig.from_dict, build_turudra, replace=True)
