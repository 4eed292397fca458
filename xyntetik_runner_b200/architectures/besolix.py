"""The Besolix decoder as a list of parts chosen from its configuration.

Fixed by the design: pre-norm layers with two residual additions; every norm on the stream is an RMSNorm whose stored
weight is an offset from one (factor 1 + w), the norms inside the mixers use their weights as stored; rotations pair elements
(2i, 2i + 1); the feed-forward is gated with the tanh form of GELU; the delta rule's constants (unit vectors with 1e-6
under the root, queries times D^-1/2).  Everything else -- sizes, the order and kinds of the layers, windows, rotation
bases and scaling, which layer reads whose cached rows -- comes from the configuration.
Tensor names: embed, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.{gate,up,down}, final.norm, head.
"""
from __future__ import annotations

from ..config.besolix import NAME, AttentionConfig, BesolixConfig, DeltaConfig, LatentConfig, RotationConfig
from ..config.llama import RopeScaling
from ..config.registry import register_architecture
from ..engine.model import ModelPlan, ScheduleEntry
from ..parts import Embedding, GatedDelta, GatedFeedForward, GQAAttention, Head, LatentAttention, PreNormBlock, RMSNorm, Rope
from ..weights.loader import TensorSpec

# no position table limits a request's length: the rotations take any position and the recurrence has none
MAX_POSITIONS = 1 << 30


def _rope(size: int, rot: RotationConfig) -> Rope:
    scaling = RopeScaling(rope_type="linear", factor=rot.factor) if rot.factor != 1.0 else None
    return Rope(size, rot.base, rotary_dim=rot.dims, scaling=scaling, pairing="adjacent")


class _Block(PreNormBlock):
    """A pre-norm layer; one without a feed-forward lets a checkpoint carry a second norm weight that nothing reads."""

    def __init__(self, *parts, spare: str = None):
        super().__init__(*parts)
        self.spare = spare

    def tensors(self):
        out = super().tensors()
        if self.spare is not None:
            out[self.spare] = TensorSpec((self.mixer_norm.width,), kind="vector", init="zeros", optional=True)
        return out


def build_besolix(cfg: BesolixConfig) -> ModelPlan:
    W, eps = cfg.width, cfg.norm_eps
    # the longest window among the layers that read a layer's cached rows (None: some reader sees every row)
    reach = {}
    for i, lay in enumerate(cfg.layers):
        m = lay.mixer
        if isinstance(m, LatentConfig):
            owner = i if m.kv_from is None else m.kv_from
            seen = reach.get(owner, 0)
            reach[owner] = None if (seen is None or m.window is None) else max(seen, m.window)
    blocks, schedule = [], []
    for i, lay in enumerate(cfg.layers):
        p = f"l{i}."
        m = lay.mixer
        cache_from = None
        if isinstance(m, AttentionConfig):
            mixer = GQAAttention(W, m.heads, m.kv_heads, m.dim, position=_rope(m.dim, m.rot), prefix=p + "mix.", window=m.window,
                                 scale=m.scale, q="q", k="k", v="v", o="o", weight_suffix="", value_dim=m.vdim, qk_norm=True,
                                 norm_eps=eps)
        elif isinstance(m, DeltaConfig):
            mixer = GatedDelta(W, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, eps, prefix=p + "mix.")
        elif isinstance(m, LatentConfig):
            cache_from = m.kv_from
            mixer = LatentAttention(W, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.scale, _rope(m.rot_dim, m.rot), eps,
                                    prefix=p + "mix.", gated=True, gate_each=True, q_rank=m.q_rank, window=m.window,
                                    retain=reach[i] if m.kv_from is None else m.window, own_rows=m.kv_from is None)
        else:
            raise ValueError(f"layer {i}: unknown mixer configuration {type(m).__name__}")
        norm1 = RMSNorm(W, eps, p + "norm1", one_plus=True)
        if lay.mlp is not None:
            ff = GatedFeedForward(W, lay.mlp.ff, p + "mlp.", "gelu_tanh", gate="gate", up="up", down="down")
            blocks.append(_Block(norm1, mixer, RMSNorm(W, eps, p + "norm2", one_plus=True), ff))
        else:
            blocks.append(_Block(norm1, mixer, spare=p + "norm2"))
        schedule.append(ScheduleEntry(layer=i, cache_from=cache_from))
    return ModelPlan(embedding=Embedding(cfg.vocab, W, "embed"), blocks=blocks, schedule=schedule,
                     final_norm=RMSNorm(W, eps, "final.norm", one_plus=True), head=Head(cfg.vocab, W, name="head"), width=W,
                     vocab_size=cfg.vocab, max_positions=MAX_POSITIONS)


register_architecture(NAME, BesolixConfig.from_dict, build_besolix, replace=True)
