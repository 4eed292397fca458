"""Typed configuration of the Besolix decoder, read from config.json.

A Besolix model is a list of pre-norm layers (x += mixer(norm1 x); x += ff(norm2 x)), each with one of three mixers:
"attention" (grouped-query softmax attention with a norm on every query and key head, a rotation over part of each
head, a sliding window), "delta" (the gated delta rule: a matrix per head that decays, is corrected and is read, behind
short causal convolutions) and "latent_attention" (keys and values expanded from a cached latent, queries through a
latent of their own, a sliding window, an element-wise output gate; a layer may read the rows another layer caches).
The feed-forward is gated with the tanh form of GELU, or absent.  Every size and every constant that can differ
between models is a field here; the parts and kernels carry none.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError
from .turudra import _get

NAME = "Besolix"


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int               # leading elements of a head (or of the rotated part) that are rotated, in pairs (2i, 2i + 1)
    factor: float = 1.0     # linear scaling: every frequency is divided by it

    @classmethod
    def from_dict(cls, d, where):
        if d is None:
            return cls(10000.0, 0, 1.0)
        sc = d.get("scaling") if isinstance(d, Mapping) else None
        c = cls(base=_get(d, "base", float, where), dims=_get(d, "dims", int, where),
                factor=_get(sc, "factor", float, where + ".scaling") if sc else 1.0)
        if c.dims % 2 or not c.base > 0 or not c.factor > 0:
            raise ConfigError(f"config.json: {where}: dims must be even, base and scaling.factor positive")
        return c

    def to_dict(self):
        d = {"base": self.base, "dims": self.dims}
        if self.factor != 1.0:
            d["scaling"] = {"factor": self.factor}
        return d


def _window(d, where) -> Optional[int]:
    mask = d.get("mask")
    if mask is None:
        return None
    size = _get(mask, "size", int, where + ".mask", None)
    if size is not None and size < 1:
        raise ConfigError(f"config.json: {where}.mask.size must be positive")
    return size


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int                # query/key elements per head
    vdim: int               # value elements per head
    scale: float
    rot: RotationConfig
    window: Optional[int]
    kind: str = "attention"

    @classmethod
    def from_dict(cls, d, where):
        heads = _get(d, "heads", int, where)
        c = cls(heads=heads, kv_heads=_get(d, "kv_heads", int, where, heads), dim=_get(d, "dim", int, where),
                vdim=_get(d, "vdim", int, where), scale=_get(d, "scale", float, where),
                rot=RotationConfig.from_dict(d.get("rot"), where + ".rot"), window=_window(d, where))
        if min(c.heads, c.kv_heads, c.dim, c.vdim) < 1 or c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")
        if c.rot.dims > c.dim:
            raise ConfigError(f"config.json: {where}.rot.dims exceeds dim")
        return c

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "rot": self.rot.to_dict()}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class DeltaConfig:
    heads: int              # value heads
    kv_heads: int           # query/key heads (each shared by heads / kv_heads value heads)
    dim: int
    vdim: int
    conv: int               # taps of the short convolutions
    kind: str = "delta"

    @classmethod
    def from_dict(cls, d, where):
        heads = _get(d, "heads", int, where)
        c = cls(heads=heads, kv_heads=_get(d, "kv_heads", int, where, heads), dim=_get(d, "dim", int, where),
                vdim=_get(d, "vdim", int, where), conv=_get(d, "conv", int, where))
        if min(c.heads, c.kv_heads, c.dim, c.vdim, c.conv) < 1 or c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")
        return c

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int                # unrotated query/key elements per head
    rot_dim: int            # rotated ones (the key's are shared by all heads)
    vdim: int
    kv_rank: int            # size of the cached latent
    q_rank: int             # size of the queries' latent
    scale: float
    rot: RotationConfig
    window: Optional[int]
    kv_from: Optional[int]  # the layer whose cached rows this one reads (None: its own)
    kind: str = "latent_attention"

    @classmethod
    def from_dict(cls, d, where):
        c = cls(heads=_get(d, "heads", int, where), dim=_get(d, "dim", int, where), rot_dim=_get(d, "rot_dim", int, where),
                vdim=_get(d, "vdim", int, where), kv_rank=_get(d, "kv_rank", int, where), q_rank=_get(d, "q_rank", int, where),
                scale=_get(d, "scale", float, where), rot=RotationConfig.from_dict(d.get("rot"), where + ".rot"),
                window=_window(d, where), kv_from=_get(d, "kv_from", int, where, None))
        if min(c.heads, c.vdim, c.kv_rank, c.q_rank) < 1 or c.dim + c.rot_dim < 1:
            raise ConfigError(f"config.json: {where}: heads, vdim, kv_rank, q_rank and dim + rot_dim must be positive")
        if c.rot.dims > c.rot_dim:
            raise ConfigError(f"config.json: {where}.rot.dims exceeds rot_dim")
        return c

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "q_rank": self.q_rank, "scale": self.scale, "rot": self.rot.to_dict()}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class DenseConfig:
    ff: int

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "kind", str, where, "dense")
        if kind != "dense":
            raise ConfigError(f"config.json: {where}.kind '{kind}' is not supported (known: dense)")
        c = cls(ff=_get(d, "ff", int, where))
        if c.ff < 1:
            raise ConfigError(f"config.json: {where}.ff must be positive")
        return c


@dataclass(frozen=True)
class LayerConfig:
    mixer: Any                       # AttentionConfig | DeltaConfig | LatentConfig
    mlp: Optional[DenseConfig]


@dataclass(frozen=True)
class BesolixConfig:
    architecture: str
    vocab: int
    width: int
    layers: Tuple[LayerConfig, ...]
    norm_eps: float
    torch_dtype: str = "bfloat16"

    MIXERS = {"attention": AttentionConfig, "delta": DeltaConfig, "latent_attention": LatentConfig}

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BesolixConfig":
        top = "top level"
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(raw):
            where = f"layers[{i}]"
            kind = _get(lr, "type", str, where)
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not supported (known: {', '.join(sorted(cls.MIXERS))})")
            if not isinstance(lr.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} lacks 'mixer'")
            md = lr["mixer"]
            j = md.get("kv_from")
            if kind == "latent_attention" and isinstance(j, int) and not isinstance(j, bool) and 0 <= j < i \
                    and isinstance(raw[j], Mapping) and isinstance(raw[j].get("mixer"), Mapping):
                # what a reader of another layer's rows shares with that layer may be left to it
                md = dict(md)
                for key in ("kv_rank", "rot_dim", "rot"):
                    if md.get(key) is None and raw[j]["mixer"].get(key) is not None:
                        md[key] = raw[j]["mixer"][key]
            mixer = cls.MIXERS[kind].from_dict(md, where + ".mixer")
            mlp = DenseConfig.from_dict(lr["mlp"], where + ".mlp") if lr.get("mlp") else None
            layers.append(LayerConfig(mixer, mlp))
        for i, lay in enumerate(layers):
            m = lay.mixer
            if isinstance(m, LatentConfig) and m.kv_from is not None:
                src = layers[m.kv_from].mixer if 0 <= m.kv_from < i else None
                if not isinstance(src, LatentConfig) or src.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from must name an earlier latent_attention layer that keeps rows of its own")
                if (src.kv_rank, src.rot_dim, src.rot) != (m.kv_rank, m.rot_dim, m.rot):
                    raise ConfigError(f"config.json: layers[{i}].mixer: kv_rank, rot_dim and rot must equal those of layer {m.kv_from}")
        norm = d.get("norm") or {}
        cfg = cls(architecture=NAME, vocab=_get(d, "vocab", int, top), width=_get(d, "width", int, top), layers=tuple(layers),
                  norm_eps=_get(norm, "eps", float, "norm"), torch_dtype=_get(d, "torch_dtype", str, top, "bfloat16"))
        if cfg.vocab < 1 or cfg.width < 1:
            raise ConfigError("config.json: vocab and width must be positive")
        return cfg

    def to_dict(self) -> dict:
        """The config.json of this configuration."""
        return {"architecture": NAME, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "layers": [{"type": l.mixer.kind, "mixer": l.mixer.to_dict(),
                            "mlp": None if l.mlp is None else {"kind": "dense", "ff": l.mlp.ff}} for l in self.layers],
                "torch_dtype": self.torch_dtype}
