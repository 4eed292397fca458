"""Parts that act on the residual stream between layers.

``StreamJoin``: x <- W [x; x0], one product over the stream and the embedding's output side by side (W is
[width, 2 width], the stream's columns first).  A model that runs a span of layers several times with the same
weights feeds the embedding back in this way at the start of every pass.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Part
from .linear import Linear


class StreamJoin(Part):
    graph_safe = True

    def __init__(self, width: int, name: str):
        self.width, self.name = width, name
        self.linear = None

    def tensors(self):
        return {self.name: TensorSpec((self.width, 2 * self.width))}

    def bind(self, tensors, rt):
        self.linear = Linear(tensors[self.name]).prepare(rt)

    def weight_bytes(self):
        return self.linear.nbytes()

    def forward(self, ctx, x: torch.Tensor, x0: torch.Tensor) -> None:
        ctx.materialize(x)
        both = ctx.buf("stream_join", (x.shape[0], 2 * self.width), ctx.act_dtype)
        kernels.concat_cast(x, x0, both)
        self.linear.forward(both, x)
