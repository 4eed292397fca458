"""Small Turudra configurations with random weights for the tests, as config.json + model.safetensors folders.

The sizes are awkward on purpose: widths that are no multiple of 8, head counts of 1, 3 and 5, value sizes that differ
from key sizes, layers of one kind with different sizes (so that they get cache groups of their own), a rotation over
part of the rotated elements, a loop that starts at layer 0 or covers one layer, layers without a feed-forward,
`top` equal to the number of experts, a single expert, no shared expert.
"""
import json
import os

import numpy as np
import torch


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, dims=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                   "scale": scale, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}}


def _mlstm(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def _moe(experts, top, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


def _layer(mixer, mlp):
    d = dict(mixer)
    d["mlp"] = mlp
    return d


CONFIGS = {
    # both mixers, a loop over the two middle layers run three times, sparse routing with a shared expert
    "mix": {"architecture": "Turudra", "vocab": 203, "width": 96, "embedding": {"scale": 2.0}, "residual_mult": 0.7,
            "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
            "layers": [_layer(_latent(3, 16, 8, 24, 40, 0.2), _moe(6, 2, 48, 2.0, (40, 1.0))),
                       _layer(_mlstm(2, 24, 40, 15.0), _moe(6, 2, 48, 2.0, (40, 1.0))),
                       _layer(_latent(2, 24, 16, 8, 56, 0.15, base=500.0), _moe(5, 3, 32, 1.2, None)),
                       _layer(_mlstm(3, 8, 16, 6.0), None)],
            "loop": {"start": 1, "stop": 3, "times": 3}},
    # a width that is no multiple of 8, one head, a rotation over part of the rotated elements, every expert chosen
    "odd": {"architecture": "Turudra", "vocab": 131, "width": 68, "embedding": {"scale": 1.0}, "residual_mult": 1.0,
            "norm": {"eps": 1e-6}, "logit_softcap": None,
            "layers": [_layer(_mlstm(1, 20, 36, 9.0), _moe(3, 3, 20, 3.0, None)),
                       _layer(_latent(5, 12, 6, 10, 24, 0.3, base=100.0, dims=4), _moe(3, 3, 20, 3.0, (12, 0.8)))],
            "loop": None},
    # latent attention alone, one expert, the whole model looped twice from layer 0
    "attn": {"architecture": "Turudra", "vocab": 97, "width": 64, "embedding": {"scale": 1.5}, "residual_mult": 0.5,
             "norm": {"eps": 1e-5}, "logit_softcap": 50.0,
             "layers": [_layer(_latent(4, 8, 8, 16, 32, 0.25), _moe(1, 1, 24, 1.5, None)),
                        _layer(_latent(1, 32, 4, 40, 16, 0.18), None)],
             "loop": {"start": 0, "stop": 2, "times": 2}},
    # the recurrence alone (no layer keeps a row per token), a loop over one layer
    "rec": {"architecture": "Turudra", "vocab": 77, "width": 48, "embedding": {"scale": 1.0}, "residual_mult": 0.8,
            "norm": {"eps": 1e-5}, "logit_softcap": 10.0,
            "layers": [_layer(_mlstm(4, 8, 8, 12.0), None),
                       _layer(_mlstm(2, 16, 24, 8.0), _moe(4, 4, 16, 2.5, (16, 2.5)))],
            "loop": {"start": 1, "stop": 2, "times": 2}},
    # sizes that the tensor-core kernels take (latent sizes 64 and 128, twenty heads = two tiles of sixteen, experts'
    # widths that are multiples of 8), every expert chosen; scores kept moderate, so that no position hangs on a near tie of two
    # keys that a bfloat16 rounding can turn
    "tc": {"architecture": "Turudra", "vocab": 151, "width": 128, "embedding": {"scale": 1.0}, "residual_mult": 0.6,
           "norm": {"eps": 1e-5}, "logit_softcap": 25.0,
           "layers": [_layer(_latent(3, 16, 8, 24, 64, 0.08), _moe(4, 4, 32, 2.0, (24, 1.0))),
                      _layer(_mlstm(2, 16, 32, 10.0), _moe(4, 4, 32, 2.0, None)),
                      _layer(_latent(20, 8, 16, 8, 128, 0.08, base=1000.0, dims=8), None)],
           "loop": {"start": 0, "stop": 2, "times": 2}},
}
SEEDS = {"mix": 11, "odd": 12, "attn": 13, "rec": 14, "tc": 16}


def shapes(cfg):
    """Tensor names and shapes of a configuration."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    if cfg.get("loop"):
        out["loop.in"] = (W, 2 * W)
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        out[p + "norm1"] = (W,)
        if lay["type"] == "mlstm":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * D, W), p + "mix.k": (H * D, W), p + "mix.v": (H * V, W), p + "mix.g": (H * V, W),
                        p + "mix.o": (W, H * V), p + "mix.norm": (H * V,), p + "mix.i": (H, W), p + "mix.i.b": (H,),
                        p + "mix.f": (H, W), p + "mix.f.b": (H,)})
        else:
            H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({p + "mix.q": (H * (D + R), W), p + "mix.dkv": (C + R, W), p + "mix.dkv.norm": (C,),
                        p + "mix.uk": (H * D, C), p + "mix.uv": (H * V, C), p + "mix.g": (H, W), p + "mix.o": (W, H * V)})
        f = lay.get("mlp")
        if f:
            out[p + "mlp.router"] = (f["router"]["experts"], W)
            for e in range(f["router"]["experts"]):
                ff = f["expert"]["ff"]
                out.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
            if f.get("shared"):
                ff = f["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (ff, W), p + "mlp.shared.up": (ff, W), p + "mlp.shared.down": (W, ff)})
    return out


def draw(cfg, seed, dtype=torch.bfloat16):
    """Random tensors: matrices N(0, 1/fan_in) (the router four times that), norm weights around 1, gate biases that
    spread the forget gates between quick and slow forgetting."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes(cfg).items():
        if name.endswith("norm") or name.endswith("norm1"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("i.b"):
            t = torch.randn(shape, generator=g)
        elif name.endswith("f.b"):
            t = 2.0 + 2.0 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
            if name.endswith("router"):
                t = t * 4.0
            if name.endswith("mix.q") or name.endswith("mix.dkv") or name.endswith("mix.k"):
                t = t * 2.0
        out[name] = t.to(dtype)
    return out


def make_folder(path, name, tensors=None, cfg=None):
    """Write config.json + model.safetensors (bfloat16) for configuration `name` (or `cfg`); returns (path, cfg, tensors)."""
    from xyntetik_runner_b200.weights.safetensors_io import write_safetensors
    cfg = cfg or CONFIGS[name]
    tensors = tensors if tensors is not None else draw(cfg, SEEDS.get(name, 1))
    os.makedirs(path, exist_ok=True)
    write_safetensors(os.path.join(path, "model.safetensors"), list(tensors.items()), metadata={"format": "pt"})
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    return path, cfg, tensors


def plain_logits(cfg, tensors, tokens):
    import plain_turudra
    return plain_turudra.forward(cfg, tensors, tokens, dtype=torch.float64).to(torch.float32).numpy()


def plain_greedy(cfg, tensors, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(plain_logits(cfg, tensors, toks)[-1])))
    return toks[len(prompt):]


def recurrence_conditioning(cfg, tensors, tokens, rounding=4e-3):
    """How far the recurrence's denominator max(|n . q|, exp(-m)) stays above what a rounding of q and k to bfloat16 does
    to n . q (about `rounding` * |n| |q|), as the smallest ratio over the request's tokens, heads and layer runs.  Where
    n and q are nearly orthogonal the sum cancels, and below a ratio of about 2 a bfloat16 run legitimately differs from
    the plain implementation by more than rounding at that token: the design's own conditioning, not the engine's."""
    import plain_turudra as P
    worst = [float("inf")]
    orig = P.mlstm

    def spy(h, w, m, eps, state=None):
        T, H, D, cap = h.shape[0], m["heads"], m["dim"], m["gate_cap"]
        q = (h @ w["q"].T).view(T, H, D) * D ** -0.5
        k = (h @ w["k"].T).view(T, H, D)
        li = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
        lf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
        n = torch.zeros(H, D, dtype=h.dtype)
        mx = torch.zeros(H, dtype=h.dtype)
        for t in range(T):
            mn = torch.maximum(lf[t] + mx, li[t])
            n = torch.exp(lf[t] + mx - mn)[:, None] * n + torch.exp(li[t] - mn)[:, None] * k[t]
            mx = mn
            den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx))
            worst[0] = min(worst[0], float((den / (rounding * n.norm(dim=-1) * q[t].norm(dim=-1) + 1e-30)).min()))
        return orig(h, w, m, eps, state)
    P.mlstm = spy
    try:
        P.forward(cfg, {k: v for k, v in tensors.items()}, tokens, dtype=torch.float64)
    finally:
        P.mlstm = orig
    return worst[0]
