"""Routed experts with an optional shared expert.

    z = W_router h (float32);  the `top` experts with the largest z;  weights = softmax over the chosen z alone
    out = sum_j weight_j * expert_{e_j}(h)  (+ shared(h))
    expert(h) = W_down gate_act(W_gate h, W_up h), no biases
The activation is one of ``kernels.ACTIVATIONS`` (with its `limit` where it has one).  Experts' matrices are kept as
[experts, rows, columns] arrays; the (token, choice) pairs are put in the order of their experts on the device and every
expert multiplies the rows that chose it (csrc/moe.cu), so no step waits for the host.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import FeedForward, register_feed_forward
from .feed_forward import GatedFeedForward, _act_id
from .linear import Linear


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, width: int, experts: int, top: int, inner: int, prefix: str, activation: str = "silu",
                 limit: float = 0.0, shared: Optional[GatedFeedForward] = None, router: str = "router",
                 expert: str = "e{}.", gate: str = "gate", up: str = "up", down: str = "down"):
        if not (1 <= top <= experts):
            raise ValueError(f"{prefix}: top {top} of {experts} experts")
        self.width, self.E, self.top, self.inner, self.prefix = width, experts, top, inner, prefix
        self.act, self.limit, self.shared = _act_id(activation), float(limit), shared
        self.router_name = prefix + router
        self.expert_names = [tuple(prefix + expert.format(e) + s for s in (gate, up, down)) for e in range(experts)]
        self.router = self.w_gate_up = self.w_down = None

    def tensors(self):
        t = {self.router_name: TensorSpec((self.E, self.width))}
        for g, u, d in self.expert_names:
            t[g] = TensorSpec((self.inner, self.width))
            t[u] = TensorSpec((self.inner, self.width))
            t[d] = TensorSpec((self.width, self.inner))
        if self.shared is not None:
            t.update(self.shared.tensors())
        return t

    def bind(self, tensors, rt):
        self.router = Linear(tensors[self.router_name]).prepare(rt)
        ws = [tensors.pop(n) for names in self.expert_names for n in names]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        # [E][2F][width]: an expert's gate rows, then its up rows; [E][width][F]
        self.w_gate_up = torch.stack([torch.cat([ws[3 * e], ws[3 * e + 1]], dim=0) for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([ws[3 * e + 2] for e in range(self.E)]).contiguous()
        del ws
        if self.shared is not None:
            self.shared.bind(tensors, rt)

    def weight_bytes(self):
        # a step reads the router, the shared expert, and at most all experts
        own = self.router.nbytes() + (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()
        return own + (self.shared.weight_bytes() if self.shared is not None else 0)

    def forward(self, ctx, h, x):
        n, top, E = h.shape[0], self.top, self.E
        pairs = n * top
        z = ctx.buf("moe_logits", (n, E), torch.float32)
        self.router.forward(h, z)
        ids = ctx.buf("moe_ids", (n, top), torch.int32)
        wts = ctx.buf("moe_weights", (n, top), torch.float32)
        kernels.route_topk(z, ids, wts, top)
        row_pair = ctx.buf("moe_row_pair", (pairs,), torch.int32)
        pair_row = ctx.buf("moe_pair_row", (pairs,), torch.int32)
        tile_info = ctx.buf("moe_tiles", (3 * kernels.moe_max_tiles(pairs, E),), torch.int32)
        counts = ctx.buf("moe_counts", (4,), torch.int32)
        kernels.moe_plan(ids, row_pair, pair_row, tile_info, counts, E)
        y = ctx.buf("moe_act", (pairs, self.inner), ctx.act_dtype)
        kernels.moe_gemm(h, self.w_gate_up, y, row_pair, tile_info, counts, pairs, top, True, self.act, self.limit)
        zz = ctx.buf("moe_out", (pairs, self.width), torch.float32)
        kernels.moe_gemm(y, self.w_down, zz, row_pair, tile_info, counts, pairs, top, False)
        ctx.materialize(x)
        kernels.moe_combine(x, zz, wts, pair_row, top)
        if self.shared is not None:
            self.shared.forward(ctx, h, x)


register_feed_forward("routed_experts", RoutedExperts)
