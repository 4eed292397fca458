"""Typed configuration of the Turudra decoder, read from config.json.

A Turudra model is a list of layers, each with one mixer ("latent_attention" or "mlstm"), an optional
mixture-of-experts feed-forward beside it (both read the layer's one norm), a residual multiplier, an optional span
of layers that runs several times with the same weights (the embedding is joined to the stream again at the start of
every pass), a scaled embedding and soft-capped logits.  Every size and constant is a field here and comes from
config.json; the parts and kernels carry none.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError

NAME = "Turudra"
DIM_MAX = 1 << 20


def _get(d: Mapping[str, Any], key: str, kind, where: str, default=...):
    if not isinstance(d, Mapping):
        raise ConfigError(f"config.json: {where} must be an object")
    if key not in d or d[key] is None:
        if default is ...:
            raise ConfigError(f"config.json: {where} lacks '{key}'")
        return default
    v = d[key]
    if kind is float and isinstance(v, (int, float)) and not isinstance(v, bool):
        return float(v)
    if kind is int and isinstance(v, int) and not isinstance(v, bool):
        if not (0 <= v <= DIM_MAX):
            raise ConfigError(f"config.json: {where}.{key} = {v} is out of range")
        return v
    if kind is str and isinstance(v, str):
        return v
    if kind is dict and isinstance(v, Mapping):
        return v
    raise ConfigError(f"config.json: {where}.{key} must be {kind.__name__}")


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int               # unrotated query/key elements per head
    rot_dim: int           # rotated query/key elements per head (the key's are shared by all heads)
    vdim: int
    kv_rank: int           # size of the cached latent
    scale: float
    rot_base: float
    rot_dims: int          # leading elements of the rotated part that are actually rotated
    kind: str = "latent_attention"

    @classmethod
    def from_dict(cls, d, where):
        rot = _get(d, "rot", dict, where)
        c = cls(heads=_get(d, "heads", int, where), dim=_get(d, "dim", int, where), rot_dim=_get(d, "rot_dim", int, where),
                vdim=_get(d, "vdim", int, where), kv_rank=_get(d, "kv_rank", int, where), scale=_get(d, "scale", float, where),
                rot_base=_get(rot, "base", float, where + ".rot"), rot_dims=_get(rot, "dims", int, where + ".rot"))
        if min(c.heads, c.vdim, c.kv_rank) < 1 or c.dim + c.rot_dim < 1:
            raise ConfigError(f"config.json: {where}: heads, vdim, kv_rank and dim + rot_dim must be positive")
        if c.rot_dims % 2 or c.rot_dims > c.rot_dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most rot_dim")
        return c


@dataclass(frozen=True)
class MLSTMConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float
    kind: str = "mlstm"

    @classmethod
    def from_dict(cls, d, where):
        c = cls(heads=_get(d, "heads", int, where), dim=_get(d, "dim", int, where), vdim=_get(d, "vdim", int, where),
                gate_cap=_get(d, "gate_cap", float, where))
        if min(c.heads, c.dim, c.vdim) < 1 or not c.gate_cap > 0:
            raise ConfigError(f"config.json: {where}: heads, dim, vdim and gate_cap must be positive")
        return c


@dataclass(frozen=True)
class ExpertConfig:
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, d, where):
        c = cls(ff=_get(d, "ff", int, where), limit=_get(d, "limit", float, where))
        if c.ff < 1:
            raise ConfigError(f"config.json: {where}.ff must be positive")
        return c


@dataclass(frozen=True)
class MoEConfig:
    experts: int
    top: int
    expert: ExpertConfig
    shared: Optional[ExpertConfig]

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "kind", str, where, "moe")
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind '{kind}' is not supported (known: moe)")
        router = _get(d, "router", dict, where)
        c = cls(experts=_get(router, "experts", int, where + ".router"), top=_get(router, "top", int, where + ".router"),
                expert=ExpertConfig.from_dict(_get(d, "expert", dict, where), where + ".expert"),
                shared=ExpertConfig.from_dict(d["shared"], where + ".shared") if d.get("shared") else None)
        if not (1 <= c.top <= c.experts):
            raise ConfigError(f"config.json: {where}.router: top must be between 1 and experts")
        return c


@dataclass(frozen=True)
class LayerConfig:
    mixer: Any                       # LatentAttentionConfig | MLSTMConfig
    mlp: Optional[MoEConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class TurudraConfig:
    architecture: str
    vocab: int
    width: int
    layers: Tuple[LayerConfig, ...]
    loop: Optional[LoopConfig]
    embedding_scale: float
    residual_mult: float
    norm_eps: float
    logit_softcap: Optional[float]
    torch_dtype: str = "bfloat16"

    MIXERS = {"latent_attention": LatentAttentionConfig, "mlstm": MLSTMConfig}

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "TurudraConfig":
        top = "top level"
        layers_raw = d.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            kind = _get(lr, "type", str, where)
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not supported (known: {', '.join(sorted(cls.MIXERS))})")
            if not isinstance(lr.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} lacks 'mixer'")
            mixer = cls.MIXERS[kind].from_dict(lr["mixer"], where + ".mixer")
            mlp = MoEConfig.from_dict(lr["mlp"], where + ".mlp") if lr.get("mlp") else None
            layers.append(LayerConfig(mixer, mlp))
        loop = None
        if d.get("loop"):
            lp = d["loop"]
            loop = LoopConfig(_get(lp, "start", int, "loop"), _get(lp, "stop", int, "loop"), _get(lp, "times", int, "loop"))
            if not (0 <= loop.start < loop.stop <= len(layers)) or loop.times < 1:
                raise ConfigError("config.json: loop needs 0 <= start < stop <= number of layers and times >= 1")
        emb = d.get("embedding") or {}
        norm = d.get("norm") or {}
        cap = _get(d, "logit_softcap", float, top, None)
        cfg = cls(architecture=NAME, vocab=_get(d, "vocab", int, top), width=_get(d, "width", int, top), layers=tuple(layers),
                  loop=loop, embedding_scale=_get(emb, "scale", float, "embedding", 1.0),
                  residual_mult=_get(d, "residual_mult", float, top, 1.0), norm_eps=_get(norm, "eps", float, "norm"),
                  logit_softcap=cap if cap else None, torch_dtype=_get(d, "torch_dtype", str, top, "bfloat16"))
        if cfg.vocab < 1 or cfg.width < 1:
            raise ConfigError("config.json: vocab and width must be positive")
        return cfg

    def layer_runs(self):
        """[(layer index, first of a pass)] in the order the layers run."""
        L = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(L)]
        a, b, times = self.loop.start, self.loop.stop, self.loop.times
        runs = [(i, False) for i in range(a)]
        for _ in range(times):
            runs += [(i, i == a) for i in range(a, b)]
        return runs + [(i, False) for i in range(b, L)]

    def to_dict(self) -> dict:
        """The config.json of this configuration."""
        def mixer(m):
            if isinstance(m, MLSTMConfig):
                return {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "gate_cap": m.gate_cap}
            return {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale,
                    "rot": {"base": m.rot_base, "dims": m.rot_dims}}

        def mlp(f):
            if f is None:
                return None
            out = {"kind": "moe", "router": {"experts": f.experts, "top": f.top}, "expert": {"ff": f.expert.ff, "limit": f.expert.limit}}
            out["shared"] = {"ff": f.shared.ff, "limit": f.shared.limit} if f.shared else None
            return out
        d = {"architecture": NAME, "vocab": self.vocab, "width": self.width, "embedding": {"scale": self.embedding_scale},
             "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps}, "logit_softcap": self.logit_softcap,
             "layers": [{"type": l.mixer.kind, "mixer": mixer(l.mixer), "mlp": mlp(l.mlp)} for l in self.layers],
             "loop": None if self.loop is None else {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times},
             "torch_dtype": self.torch_dtype}
        return d
