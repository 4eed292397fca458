"""The gated delta rule as a mixer with a fixed-size state per request.

With h the mixer's input, H value heads of size V, G query/key heads of size D (value head i reads query/key head
i / (H / G)), short causal convolutions of `taps` taps per channel (the last column of a convolution's weight is the
current token's, zeros before a request's first token):
    q = silu(conv(W_q h)),  k = silu(conv(W_k h)),  v = silu(conv(W_v h))
    q <- q / sqrt(sum q^2 + 1e-6) * D^-1/2,   k <- k / sqrt(sum k^2 + 1e-6)                       per head
    beta = sigmoid(W_b h),   g = exp(-exp(A_log) softplus(W_a h + dt_bias))                       per value head
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                              S [D, V] per value head
    y = W_o (concat_i(o_i / rms(o_i)) * w * silu(W_g h))                                          w: V values for all heads
S starts at zero and lives in float32 in the request's state slot together with the last taps - 1 rows that entered the
convolutions; the projections' sums and everything after them are float32 in both precisions (csrc/delta.cu).  The state after a token
does not depend on how tokens were cut into steps.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_mixer
from .linear import Linear


class GatedDelta(Mixer):
    graph_safe = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float, prefix: str,
                 q: str = "q", k: str = "k", v: str = "v", g: str = "g", o: str = "o", norm: str = "norm", b: str = "b",
                 a: str = "a", a_log: str = "A_log", dt_bias: str = "dt_bias", conv_suffix: str = ".conv"):
        if heads % kv_heads:
            raise ValueError(f"{prefix}: heads must be a multiple of kv_heads")
        if dim > 256:
            raise ValueError(f"{prefix}: key size {dim}: the recurrence kernel takes up to 256")
        self.width, self.H, self.G, self.D, self.V, self.taps = width, heads, kv_heads, dim, vdim, taps
        self.eps, self.prefix = float(eps), prefix
        self.names = {x: prefix + y for x, y in dict(q=q, k=k, v=v, g=g, o=o, norm=norm, b=b, a=a, a_log=a_log, dt_bias=dt_bias).items()}
        for x in ("q", "k", "v"):
            self.names[x + "c"] = self.names[x] + conv_suffix
        self.channels = 2 * kv_heads * dim + heads * vdim
        self.proj = self.gates = self.out = self.norm_w = self.conv_w = self.neg_a = self.dt_bias = None

    def state_need(self):
        return StateNeed((kernels.delta_state_floats(self.H, self.G, self.D, self.V, self.taps),), torch.float32)

    def tensors(self):
        n, H, G, D, V, W, K = self.names, self.H, self.G, self.D, self.V, self.width, self.taps
        return {n["q"]: TensorSpec((G * D, W)), n["k"]: TensorSpec((G * D, W)), n["v"]: TensorSpec((H * V, W)),
                n["qc"]: TensorSpec((G * D, K), "vector", "normal"), n["kc"]: TensorSpec((G * D, K), "vector", "normal"),
                n["vc"]: TensorSpec((H * V, K), "vector", "normal"),
                n["g"]: TensorSpec((H * V, W)), n["o"]: TensorSpec((W, H * V)), n["norm"]: TensorSpec((V,), "vector", "ones_jitter"),
                n["b"]: TensorSpec((H, W)), n["a"]: TensorSpec((H, W)),
                n["a_log"]: TensorSpec((H,), "vector", "zeros"), n["dt_bias"]: TensorSpec((H,), "vector", "zeros")}

    def bind(self, tensors, rt):
        n = self.names
        ws = [tensors.pop(n[x]) for x in ("q", "k", "v", "g")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        # one product for the convolutions' channels (q, k, v, in this order from column 0) and the output gate
        self.proj = Linear(torch.cat(ws, dim=0)).prepare(rt)
        del ws
        gs = [tensors.pop(n["b"]), tensors.pop(n["a"])]
        if len({w.dtype for w in gs}) > 1:
            gs = [w.to(torch.float32) for w in gs]
        # the two scalars per head leave their product in float32
        self.gates = Linear(torch.cat(gs, dim=0)).prepare(rt)
        self.out = Linear(tensors[n["o"]]).prepare(rt)
        f32 = lambda name: tensors[name].to(torch.float32).contiguous()
        self.norm_w = f32(n["norm"])
        self.conv_w = torch.cat([f32(n["qc"]), f32(n["kc"]), f32(n["vc"])], dim=0).contiguous()
        self.neg_a = (-torch.exp(f32(n["a_log"]))).contiguous()
        self.dt_bias = f32(n["dt_bias"])

    def weight_bytes(self):
        return self.proj.nbytes() + self.gates.nbytes() + self.out.nbytes() + self.conv_w.numel() * 4

    def forward(self, ctx, h, x, lay):
        n, H, V, CH = h.shape[0], self.H, self.V, self.channels
        total = CH + H * V
        ld = -(-total // 8) * 8
        # the projections leave their product in float32: what enters the convolutions and the recurrence is rounded once, at the
        # product's input, and the convolutions' tail holds exactly what the rows held
        proj = ctx.buf("delta_proj", (n, ld), torch.float32)[:, :total]
        self.proj.forward(h, proj)
        gates = ctx.buf("delta_gates", (n, 2 * H), torch.float32)
        self.gates.forward(h, gates)
        qkv = ctx.buf("delta_qkv", (n, CH), torch.float32)
        coef = ctx.buf("delta_coef", (n, 2 * H), torch.float32)
        o = ctx.buf("delta_o", (n, H * V), torch.float32)
        kernels.delta(proj, self.conv_w, gates, self.neg_a, self.dt_bias, lay.state, qkv, coef, o, ctx.tok_seg, ctx.seg_start,
                      ctx.seg_len, ctx.seg_slot, ctx.n_seg, H, self.G, self.D, V, self.taps)
        y = ctx.buf("attn_out", (n, H * V), ctx.act_dtype)
        kernels.head_norm_gate(o, proj, CH, self.norm_w, y, H, V, self.eps, per_head_weight=False, silu=True)
        ctx.set_pending(x, self.out.forward(y, x, accumulate=True, defer=True))


register_mixer("gated_delta", GatedDelta)
