"""A plain, slow implementation of the Turudra decoder: one function per mechanism, whole sequences, no cache.

Everything is computed on the CPU in one dtype (float64 by default) from a configuration dict and a dict of
tensors by name.  It shares no code with the engine: the tests compare the engine's logits with it.

Notation.  x: residual stream [T, width]; h: normed input of a layer; p: position (from 0).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def rotate_half_layout(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """v [T, ..., D]: the first `dims` elements are rotated; element i pairs with i + dims/2."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]                  # [T, half]
    while ang.dim() < v.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], dim=-1)


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Causal softmax attention whose keys and values are expanded from a normed latent; one rotated key part is
    shared by all heads; a sigmoid gate per head multiplies the head's output."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w["q"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], q[..., D:]
    down = h @ w["dkv"].T
    latent = rms_norm(down[:, :C], w["dkv.norm"], eps)
    k_rot = down[:, C:]
    rot = m["rot"]
    q_rot = rotate_half_layout(q_rot, pos, rot["dims"], rot["base"])
    k_rot = rotate_half_layout(k_rot, pos, rot["dims"], rot["base"])
    k_plain = (latent @ w["uk"].T).view(T, H, D)
    val = (latent @ w["uv"].T).view(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    a = torch.softmax(scores, dim=-1)
    o = torch.einsum("hij,jhv->ihv", a, val)
    gate = torch.sigmoid(h @ w["g"].T)                                     # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * V) @ w["o"].T


def mlstm(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, state: Optional[dict] = None) -> torch.Tensor:
    """Matrix memory with exponential input gate and a stabilising running maximum that starts at 0."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).view(T, H, D)
    v = (h @ w["v"].T).view(T, H, V)
    ig = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)                # log input gate   [T, H]
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    if state is None:
        state = {"S": torch.zeros(H, D, V, dtype=h.dtype), "n": torch.zeros(H, D, dtype=h.dtype),
                 "m": torch.zeros(H, dtype=h.dtype)}
    S, n, mx = state["S"], state["n"], state["m"]
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(fg[t] + mx, ig[t])
        decay = torch.exp(fg[t] + mx - m_new)
        inp = torch.exp(ig[t] - m_new)
        S = decay[:, None, None] * S + inp[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = decay[:, None] * n + inp[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    state["S"], state["n"], state["m"] = S, n, mx
    o = rms_unit(out, eps).reshape(T, H * V) * w["norm"]
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return y @ down.T


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict, chosen: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`chosen` [T, top] (optional): take these experts instead of the `top` largest logits (their weights are still the
    softmax of their own logits): for comparing with a run whose rounding turned a near tie the other way."""
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ w["router"].T
    best, idx = torch.topk(z, top, dim=-1)
    if chosen is not None:
        idx = chosen.to(torch.long)
        best = torch.gather(z, 1, idx)
    wt = torch.softmax(best, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wt[t, j] * expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], f["shared"]["limit"])
    return out


def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer_order(cfg: dict) -> List[tuple]:
    """[(layer index, first of a pass)] in the order the layers run."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(L)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, L)]


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens, dtype=torch.float64, trace: Optional[list] = None,
            routing: Optional[list] = None, round_inputs: bool = False) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  `trace` collects the residual stream after every layer run.  `routing`:
    the experts to take ([T, top] per layer run that has experts, in the order the layers run) instead of the router's choice.
    `round_inputs`: every layer's normed input is rounded to bfloat16, the one rounding of a bfloat16 run that a layer with
    a cancelling sum (the first tokens of the recurrence, where k . q may be near zero before the unit norm) amplifies
    beyond all others; what is left between this and a bfloat16 run is rounding inside the layers."""
    routing = list(routing) if routing is not None else None
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    x0 = x
    for i, first in layer_order(cfg):
        lay = cfg["layers"][i]
        if first:
            x = torch.cat([x, x0], dim=-1) @ W["loop.in"].T
        h = rms_norm(x, W[f"l{i}.norm1"], eps)
        if round_inputs:
            h = h.to(torch.bfloat16).to(dtype)
        wm = sub(W, f"l{i}.mix.")
        if lay["type"] == "latent_attention":
            y = latent_attention(h, wm, lay["mixer"], eps)
        elif lay["type"] == "mlstm":
            y = mlstm(h, wm, lay["mixer"], eps)
        else:
            raise ValueError(lay["type"])
        if lay.get("mlp"):
            y = y + moe(h, sub(W, f"l{i}.mlp."), lay["mlp"], routing.pop(0) if routing else None)
        x = x + mult * y
        if trace is not None:
            trace.append(x.clone())
    hn = rms_norm(x, W["final.norm"], eps)
    logits = hn @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
