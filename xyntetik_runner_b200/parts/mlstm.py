"""Matrix-memory recurrence (the mLSTM cell of xLSTM) as a mixer with a fixed-size state per request.

With h the mixer's input, H heads, key size D, value size V and gate cap c:
    q = W_q h * D^-1/2,  k = W_k h,  v = W_v h
    li = c tanh((W_i h + b_i) / c),  lf = logsigmoid(c tanh((W_f h + b_f) / c))          per head
    m' = max(lf + m, li);  S' = exp(lf + m - m') S + exp(li - m') k v^T;  n' likewise with k alone
    o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
    y = W_o (concat_h(o_h / rms(o_h)) * w * sigmoid(W_g h))
S, n, m start at zero and live in float32 in the request's state slot ([H][D V + D + 1] floats); gates, decays and the
recurrence are float32 (csrc/mlstm.cu).  The state after a token does not depend on how tokens were cut into steps.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_mixer
from .linear import Linear


class MLSTM(Mixer):
    graph_safe = True

    def __init__(self, width: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float, prefix: str,
                 q: str = "q", k: str = "k", v: str = "v", g: str = "g", o: str = "o", norm: str = "norm",
                 i: str = "i", f: str = "f", bias_suffix: str = ".b"):
        self.width, self.H, self.D, self.V = width, heads, dim, vdim
        self.cap, self.eps, self.prefix = float(gate_cap), float(eps), prefix
        self.names = {a: prefix + b for a, b in dict(q=q, k=k, v=v, g=g, o=o, norm=norm, i=i, f=f).items()}
        self.names["ib"], self.names["fb"] = self.names["i"] + bias_suffix, self.names["f"] + bias_suffix
        self.proj = self.gates = self.out = self.norm_w = None

    def state_need(self):
        return StateNeed((kernels.mlstm_state_floats(self.H, self.D, self.V),), torch.float32)

    def tensors(self):
        n, H, D, V, W = self.names, self.H, self.D, self.V, self.width
        return {n["q"]: TensorSpec((H * D, W)), n["k"]: TensorSpec((H * D, W)), n["v"]: TensorSpec((H * V, W)),
                n["g"]: TensorSpec((H * V, W)), n["o"]: TensorSpec((W, H * V)),
                n["norm"]: TensorSpec((H * V,), "vector", "ones_jitter"),
                n["i"]: TensorSpec((H, W)), n["ib"]: TensorSpec((H,), "vector", "zeros"),
                n["f"]: TensorSpec((H, W)), n["fb"]: TensorSpec((H,), "vector", "zeros")}

    def bind(self, tensors, rt):
        n = self.names
        ws = [tensors.pop(n[a]) for a in ("q", "k", "v", "g")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.proj = Linear(torch.cat(ws, dim=0)).prepare(rt)
        del ws
        gs = [tensors.pop(n["i"]), tensors.pop(n["f"])]
        if len({w.dtype for w in gs}) > 1:
            gs = [w.to(torch.float32) for w in gs]
        bias = torch.cat([tensors[n["ib"]].to(torch.float32), tensors[n["fb"]].to(torch.float32)])
        # the gates' pre-activations leave their product in float32
        self.gates = Linear(torch.cat(gs, dim=0), bias).prepare(rt)
        self.out = Linear(tensors[n["o"]]).prepare(rt)
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()

    def weight_bytes(self):
        return self.proj.nbytes() + self.gates.nbytes() + self.out.nbytes()

    def forward(self, ctx, h, x, lay):
        n, H, D, V = h.shape[0], self.H, self.D, self.V
        total = 2 * H * D + 2 * H * V
        ld = -(-total // 8) * 8
        proj = ctx.buf("mlstm_proj", (n, ld), ctx.act_dtype)[:, :total]
        self.proj.forward(h, proj)
        gates = ctx.buf("mlstm_gates", (n, 2 * H), torch.float32)
        self.gates.forward(h, gates)
        coef = ctx.buf("mlstm_coef", (n, 3 * H), torch.float32)
        o = ctx.buf("mlstm_o", (n, H * V), torch.float32)
        y = ctx.buf("attn_out", (n, H * V), ctx.act_dtype)
        kernels.mlstm(proj, (0, H * D, 2 * H * D, 2 * H * D + H * V), gates, lay.state, coef, o, self.norm_w, y,
                      ctx.seg_start, ctx.seg_len, ctx.seg_slot, ctx.n_seg, H, D, V, self.cap, self.eps)
        ctx.set_pending(x, self.out.forward(y, x, accumulate=True, defer=True))


register_mixer("mlstm", MLSTM)
