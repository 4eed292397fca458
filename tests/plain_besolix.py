"""A plain, slow implementation of the Besolix decoder: one function per mechanism, whole sequences, no cache.

Everything is computed on the CPU in one dtype (float64 by default) from a configuration dict and a dict of tensors
by name.  It shares no code with the engine: the tests compare the engine's logits with it.

Notation.  x: residual stream [T, width]; h: a layer's normed input; p: position (from 0); a window of size w lets
position i see the positions j with 0 <= i - j < w.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Weight used as it is."""
    return unit_rms(x, eps) * w


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The stored weight is the factor's distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_adjacent(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float, factor: float = 1.0) -> torch.Tensor:
    """v [T, ..., D]: of the first `dims` elements, 2i and 2i + 1 are a pair turned by p * base^(-2i/dims) / factor."""
    if dims == 0:
        return v
    i = torch.arange(dims // 2, dtype=v.dtype)
    freq = base ** (-2.0 * i / dims) / factor
    ang = positions.to(v.dtype)[:, None] * freq[None, :]
    while ang.dim() < v.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def window_mask(T: int, size: Optional[int]) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if size is not None:
        m &= (i - j) < size
    return m


def softmax_rows(scores: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return torch.softmax(scores.masked_fill(~mask, float("-inf")), dim=-1)


def _rot(m: dict):
    r = m.get("rot") or {}
    return r.get("dims", 0), r.get("base", 10000.0), ((r.get("scaling") or {}).get("factor", 1.0))


def _window(m: dict) -> Optional[int]:
    return (m.get("mask") or {}).get("size")


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Grouped-query softmax attention with a norm on every query and key head before the rotation."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = norm_plain((h @ w["q"].T).view(T, H, D), w["q.norm"], eps)
    k = norm_plain((h @ w["k"].T).view(T, G, D), w["k.norm"], eps)
    v = (h @ w["v"].T).view(T, G, V)
    dims, base, factor = _rot(m)
    q, k = rotate_adjacent(q, pos, dims, base, factor), rotate_adjacent(k, pos, dims, base, factor)
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    a = softmax_rows(torch.einsum("ihd,jhd->hij", q, k) * m["scale"], window_mask(T, _window(m)))
    return torch.einsum("hij,jhv->ihv", a, v).reshape(T, H * V) @ w["o"].T


def short_conv(z: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """z [T, C], taps [C, K]: out[t, c] = sum_j taps[c, K-1-j] z[t-j, c], zeros before the start."""
    T, K = z.shape[0], taps.shape[1]
    out = torch.zeros_like(z)
    for j in range(min(K, T)):
        out[j:] += z[:T - j] * taps[:, K - 1 - j]
    return out


def delta(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Gated delta rule: a matrix S per head that decays, is corrected towards the value at the key, and is read by the query."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).view(T, G, D)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).view(T, G, D)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ w["b"].T)                                                      # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * torch.nn.functional.softplus(h @ w["a"].T + w["dt_bias"]))
    S = torch.zeros(H, D, V, dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        S = S * decay[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps) * w["norm"] * silu(h @ w["g"].T).view(T, H, V)
    return o.reshape(T, H * V) @ w["o"].T


def latent_rows(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """What a latent-attention layer keeps per token: the normed latent and the rotated key part shared by all heads."""
    T = h.shape[0]
    C = m["kv_rank"]
    down = h @ w["dkv"].T
    dims, base, factor = _rot(m)
    return norm_plain(down[:, :C], w["dkv.norm"], eps), rotate_adjacent(down[:, C:], torch.arange(T), dims, base, factor)


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, rows=None) -> torch.Tensor:
    """Softmax attention whose keys and values are expanded from a latent; queries pass a normed latent of their own; an
    element-wise sigmoid gate on the heads' outputs.  `rows`: the (latent, rotated key part) of another layer."""
    T = h.shape[0]
    H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    dims, base, factor = _rot(m)
    q = (norm_plain(h @ w["dq"].T, w["dq.norm"], eps) @ w["uq"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_adjacent(q[..., D:], torch.arange(T), dims, base, factor)
    latent, k_rot = rows if rows is not None else latent_rows(h, w, m, eps)
    k_plain = (latent @ w["uk"].T).view(T, H, D)
    val = (latent @ w["uv"].T).view(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    a = softmax_rows(scores, window_mask(T, _window(m)))
    o = torch.einsum("hij,jhv->ihv", a, val).reshape(T, H * V) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def _sub(tensors: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[List] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  `layers_out`, if a list, receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    t = {k: v.to(dtype) for k, v in tensors.items()}
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        m, kind = lay["mixer"], lay["type"]
        w = _sub(t, p + "mix.", dtype)
        h = norm_one_plus(x, t[p + "norm1"], eps)
        if kind == "attention":
            y = attention(h, w, m, eps)
        elif kind == "delta":
            y = delta(h, w, m, eps)
        elif kind == "latent_attention":
            if m.get("kv_from") is not None:
                y = latent_attention(h, w, m, eps, rows=kept[m["kv_from"]])
            else:
                kept[i] = latent_rows(h, w, m, eps)
                y = latent_attention(h, w, m, eps, rows=kept[i])
        else:
            raise ValueError(f"layer {i}: unknown type '{kind}'")
        x = x + y
        if lay.get("mlp") is not None:
            x = x + feed_forward(norm_one_plus(x, t[p + "norm2"], eps), _sub(t, p + "mlp.", dtype))
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_one_plus(x, t["final.norm"], eps) @ t["head"].T
