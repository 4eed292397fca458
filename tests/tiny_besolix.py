"""Small Besolix configurations with random weights for the tests, as config.json + model.safetensors folders.

The sizes are awkward on purpose: widths that are no multiple of 8, one head, key sizes that differ from value sizes and
are no multiple of 16, fewer key heads than heads, rotations over all, part or none of a head, with and without scaling,
layers with and without a window (windows of one token, windows that end inside a page), a layer that reads another
layer's cached rows through a longer or a shorter window than the owner's, convolutions of one to five taps, layers
without a feed-forward, every order of the three mixers.
"""
import json
import os

import numpy as np
import torch


def _rot(base, dims, factor=None):
    d = {"base": base, "dims": dims}
    if factor is not None:
        d["scaling"] = {"factor": factor}
    return d


def attention(heads, kv_heads, dim, vdim, scale, rot, window=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, window=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": _rot(base, rot_dim), "rot_dim": rot_dim}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def layer(mixer, ff):
    d = dict(mixer)
    d["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return d


def model(vocab, width, eps, layers):
    return {"architecture": "Besolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # every mixer; fewer key heads than heads; a reader of layer 1's rows with a longer window than layer 1's own
    "mix": model(211, 96, 1e-5, [
        layer(delta(4, 2, 12, 20, 3), 80),
        layer(latent(3, 16, 8, 24, 40, 24, 0.2, base=500.0, window=19), 64),
        layer(attention(4, 2, 24, 16, 0.21, _rot(1000.0, 8, 2.0), window=33), None),
        layer(latent(2, 8, 8, 12, 40, 16, 0.3, base=500.0, window=37, kv_from=1), 48),
        layer(delta(2, 2, 16, 8, 2), 32)]),
    # a width that is no multiple of 8, one head, no windows, no scaling, a rotation over the whole head, one tap
    "odd": model(131, 68, 1e-6, [
        layer(attention(5, 5, 10, 14, 0.3, _rot(100.0, 10)), 36),
        layer(delta(1, 1, 20, 36, 1), None),
        layer(latent(5, 12, 6, 10, 24, 20, 0.25, base=100.0), 20),
        layer(attention(1, 1, 18, 6, 0.2, _rot(10000.0, 0)), 28)]),
    # sizes that the tensor-core kernels take; two readers of layer 0's rows, one with a shorter window, one with none
    "tc": model(160, 128, 1e-5, [
        layer(latent(4, 16, 16, 32, 64, 48, 0.1, window=50), 96),
        layer(attention(4, 2, 64, 64, 0.12, _rot(20000.0, 32, 8.0), window=40), 64),
        layer(delta(4, 2, 32, 64, 4), 64),
        layer(latent(20, 8, 16, 16, 64, 32, 0.1, window=30, kv_from=0), None),
        layer(attention(2, 1, 32, 128, 0.15, _rot(500.0, 16)), 32),
        layer(latent(2, 32, 16, 64, 64, 64, 0.1, kv_from=0), 32)]),
    # the recurrence alone (no layer keeps a row per token): five taps, value heads of their own, then shared ones
    "rec": model(77, 48, 1e-5, [
        layer(delta(4, 1, 8, 8, 5), None),
        layer(delta(2, 2, 40, 24, 2), 40)]),
    # windows of one, two and three tokens beside pages of four; a reader with a window of one
    "win": model(90, 64, 1e-5, [
        layer(attention(2, 1, 16, 16, 0.3, _rot(10.0, 16), window=1), 24),
        layer(latent(2, 8, 4, 8, 16, 8, 0.4, base=10.0, window=3), 24),
        layer(attention(2, 2, 8, 24, 0.3, _rot(10.0, 4, 1.5), window=2), None),
        layer(latent(1, 4, 4, 8, 16, 8, 0.4, base=10.0, window=1, kv_from=1), 24)]),
}
SEEDS = {"mix": 21, "odd": 22, "tc": 23, "rec": 24, "win": 25}


def shapes(cfg):
    """Tensor names and shapes of a configuration."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        out[p + "norm1"] = (W,)
        if lay["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * D, W), p + "mix.k": (G * D, W), p + "mix.v": (G * V, W), p + "mix.q.norm": (D,),
                        p + "mix.k.norm": (D,), p + "mix.o": (W, H * V)})
        elif lay["type"] == "delta":
            H, G, D, V, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            out.update({p + "mix.q": (G * D, W), p + "mix.q.conv": (G * D, K), p + "mix.k": (G * D, W), p + "mix.k.conv": (G * D, K),
                        p + "mix.v": (H * V, W), p + "mix.v.conv": (H * V, K), p + "mix.b": (H, W), p + "mix.A_log": (H,),
                        p + "mix.norm": (V,), p + "mix.a": (H, W), p + "mix.dt_bias": (H,), p + "mix.g": (H * V, W),
                        p + "mix.o": (W, H * V)})
        else:
            H, D, R, V, C, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({p + "mix.dq": (Q, W), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (D + R), Q), p + "mix.uk": (H * D, C),
                        p + "mix.uv": (H * V, C), p + "mix.g": (H * V, W), p + "mix.o": (W, H * V)})
            if m.get("kv_from") is None:
                out.update({p + "mix.dkv": (C + R, W), p + "mix.dkv.norm": (C,)})
        if lay.get("mlp"):
            ff = lay["mlp"]["ff"]
            out.update({p + "norm2": (W,), p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    return out


def draw(cfg, seed, dtype=torch.bfloat16, slow_decay=False):
    """Random tensors: matrices N(0, 1/fan_in); the stream's norm weights around 0 (they are offsets from one), the mixers'
    own around 1; convolution taps N(0, 1/2); decays spread between quick and slow forgetting (`slow_decay`: all slow)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes(cfg).items():
        r = lambda: torch.randn(shape, generator=g)
        if name.endswith(("norm1", "norm2", "final.norm")):
            t = 0.1 * r()
        elif name.endswith("norm"):
            t = 1.0 + 0.1 * r()
        elif name.endswith("conv"):
            t = 0.7 * r()
        elif name.endswith("A_log"):
            t = (-5.0 + 0.3 * r()) if slow_decay else (-1.0 + 1.0 * r())
        elif name.endswith("dt_bias"):
            t = r()
        else:
            t = r() / shape[-1] ** 0.5
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
    import plain_besolix
    return plain_besolix.forward(cfg, tensors, tokens, dtype=torch.float64).to(torch.float32).numpy()


def plain_greedy(cfg, tensors, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(plain_logits(cfg, tensors, toks)[-1])))
    return toks[len(prompt):]


def rounding_sensitivity(cfg, tensors, tokens, draws=3):
    """How far a rounding of every layer's input to bfloat16 moves each position's logits in the plain implementation, as a
    fraction of the largest logit: the largest of `draws` runs, the first with the rounding alone, the others with a relative
    nudge of up to 2^-8 before it.  Positions where this is large (two keys whose scores nearly tie, a recurrence's read-out
    that nearly cancels) differ by more than the usual rounding in ANY bfloat16 run; that is the design's own conditioning
    at that position, and a bfloat16 comparison allows for it position by position."""
    import plain_besolix as P
    ref = plain_logits(cfg, tensors, tokens)
    scale = float(np.abs(ref).max())
    orig = P.norm_one_plus
    g = torch.Generator().manual_seed(len(tokens))
    worst = np.zeros(len(tokens))
    try:
        for d in range(draws):
            def rounded(x, w, eps, d=d):
                y = orig(x, w, eps)
                if d:
                    y = y * (1.0 + (torch.rand(y.shape, generator=g, dtype=torch.float64) - 0.5) * 2.0 ** -7)
                return y.to(torch.bfloat16).to(x.dtype)
            P.norm_one_plus = rounded
            worst = np.maximum(worst, np.abs(plain_logits(cfg, tensors, tokens) - ref).max(axis=1) / scale)
    finally:
        P.norm_one_plus = orig
    return worst


def assert_close_bfloat16(got, ref, sens, what=""):
    """The fixed bfloat16 tolerance of `traces` at every position, except that a position may differ by three times what the
    rounding of the layers' inputs alone does to it in the plain implementation (`sens`, from ``rounding_sensitivity``); few
    positions may need that, and the mean over all (of a request of sixteen tokens or more) stays within the fixed mean."""
    import traces
    tol = traces.TOL["bfloat16"]
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    scale = float(np.abs(ref).max())
    diff = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    err = diff.max(axis=1) / scale
    allowed = np.maximum(tol["max_rel"], 3.0 * sens)
    bad = np.nonzero(err > allowed)[0]
    assert len(bad) == 0, f"{what}: positions {bad[:10].tolist()} differ by {err[bad[:10]].round(4).tolist()} of the largest logit, allowed {allowed[bad[:10]].round(4).tolist()}"
    over = int((err > tol["max_rel"]).sum())
    assert over <= max(1, len(err) // 20), f"{what}: {over} of {len(err)} positions beyond the fixed tolerance"
    if len(err) >= 16:              # (a mean over a handful of positions is no mean)
        assert diff.mean() <= tol["mean_rel"] * scale, f"{what}: mean |diff| {diff.mean():.3e} > {tol['mean_rel']:.1e} * {scale:.3f}"
