"""Latent attention: keys and values of all heads are expanded from one small latent vector per token.

With h the mixer's input, H heads, per head D plain and R rotated query/key elements, value size V, latent size C:
    q = W_q h                   heads laid out as [D plain | R rotated]
    [c' | r'] = W_dkv h         c = RMSNorm(c') * w (the latent), r = rotate(r') (one rotated key part for all heads)
    k_h = [W_uk,h c | r],  v_h = W_uv,h c
    s_ij = (q_plain . W_uk,h c_j + rotate(q_rot) . r_j) * scale,  j <= i;  a = softmax(s);  o_h = sum_j a_ij v_hj
    y = W_o concat_h(sigmoid(W_g h)_h * o_h)
Only [c | r] is cached: one row of C + R values per token (one plane, one "kv head"), whatever H is.  The kernels
never expand a key: the query is taken into the latent space, attention runs over the cached rows, and the result is
expanded by W_uv afterwards (csrc/latent_attention.cu).  The rotation uses the first `rotary_dim` of the R elements
in the pairing the position encoding names (half-split or adjacent).

Options, all off by default:
    q_rank Q:    the queries pass a latent of their own, q = W_uq (RMSNorm(W_dq h) * w_dq);
    window w:    position i sees the positions j with 0 <= i - j < w;
    gate_each:   the gate has H V elements and multiplies the heads' outputs element by element (else one per head);
    own_rows False: the layer has no W_dkv and reads the rows that another layer caches (the schedule entry's
                 `cache_from`); `retain` is then the longest window among the readers of a layer's rows.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, PositionEncoding, register_mixer
from . import linear_tc
from .linear import Linear


# the tensor-core kernel for the sizes it takes (a module attribute, so that a test can compare the two kernels)
USE_MMA = True
counters = {"mma": 0, "simt": 0}


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, width: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float,
                 position: PositionEncoding, eps: float, prefix: str, gated: bool = True,
                 q: str = "q", dkv: str = "dkv", dkv_norm: str = "dkv.norm", uk: str = "uk", uv: str = "uv", g: str = "g", o: str = "o",
                 q_rank: Optional[int] = None, dq: str = "dq", dq_norm: str = "dq.norm", uq: str = "uq",
                 window: Optional[int] = None, retain: Optional[int] = ..., gate_each: bool = False, own_rows: bool = True):
        if kv_rank > 1024:
            raise ValueError(f"{prefix}: latent size {kv_rank}: the attention kernel takes up to 1024")
        self.width, self.H, self.D, self.R, self.V, self.C = width, heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.position, self.eps, self.prefix, self.gated = float(scale), position, float(eps), prefix, gated
        self.Q, self.window, self.gate_each, self.own_rows = q_rank, window, bool(gate_each), bool(own_rows)
        # how long the cached rows are kept: this layer's window unless a reader of its rows looks further back
        self.retain = window if retain is ... else retain
        self.names = {k: prefix + v for k, v in dict(q=q, dkv=dkv, norm=dkv_norm, uk=uk, uv=uv, g=g, o=o, dq=dq, dq_norm=dq_norm,
                                                     uq=uq).items()}
        self.proj = self.out = self.w_uk = self.w_uv = self.norm_w = self.freq = self.up_q = self.q_norm_w = None
        self.w_uk_packed = self.w_uv_packed = None
        self.rot_dims = 0
        self.adjacent = False

    def kv_need(self):
        return KVNeed(1, self.C + self.R, self.retain, planes=1)

    def gate_width(self) -> int:
        return 0 if not self.gated else (self.H * self.V if self.gate_each else self.H)

    def tensors(self):
        n, H, D, R, V, C, W = self.names, self.H, self.D, self.R, self.V, self.C, self.width
        t = {n["uk"]: TensorSpec((H * D, C)), n["uv"]: TensorSpec((H * V, C)), n["o"]: TensorSpec((W, H * V))}
        if self.Q is None:
            t[n["q"]] = TensorSpec((H * (D + R), W))
        else:
            t.update({n["dq"]: TensorSpec((self.Q, W)), n["dq_norm"]: TensorSpec((self.Q,), "vector", "ones_jitter"),
                      n["uq"]: TensorSpec((H * (D + R), self.Q))})
        if self.own_rows:
            t.update({n["dkv"]: TensorSpec((C + R, W)), n["norm"]: TensorSpec((C,), "vector", "ones_jitter")})
        if self.gated:
            t[n["g"]] = TensorSpec((self.gate_width(), W))
        return t

    def bind(self, tensors, rt):
        n = self.names
        ws = [tensors.pop(n["q"] if self.Q is None else n["dq"])] + ([tensors.pop(n["dkv"])] if self.own_rows else []) \
            + ([tensors.pop(n["g"])] if self.gated else [])
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        # one product for the queries (or their latent), the down projection and the gates
        self.proj = Linear(torch.cat(ws, dim=0)).prepare(rt)
        del ws
        if self.Q is not None:
            self.up_q = Linear(tensors.pop(n["uq"])).prepare(rt)
            self.q_norm_w = tensors[n["dq_norm"]].to(torch.float32).contiguous()
        self.out = Linear(tensors[n["o"]]).prepare(rt)
        self.w_uk, self.w_uv = tensors[n["uk"]].contiguous(), tensors[n["uv"]].contiguous()
        # for the tensor-core products per head: W_uk,h^T ([C, D]: the query goes into the latent space) and W_uv,h ([V, C])
        self.w_uk_packed = self.w_uv_packed = None
        if (linear_tc.ENABLED and rt.act_dtype == torch.bfloat16 and self.w_uk.dtype == torch.bfloat16 and self.w_uv.dtype == torch.bfloat16
                and self.w_uk.is_cuda and self.D % 8 == 0 and self.D >= 8 and self.C % 8 == 0):
            self.w_uk_packed = kernels.pack_weight_groups(self.w_uk.view(self.H, self.D, self.C).transpose(1, 2).contiguous())
            self.w_uv_packed = kernels.pack_weight_groups(self.w_uv.view(self.H, self.V, self.C))
        self._heads_of_tiles = {}
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous() if self.own_rows else None
        self.position.prepare(rt)
        rot = self.position.rotary()
        if rot is not None and rot.rotary_dim:
            if rot.mscale != 1.0 or rot.rotary_dim > self.R:
                raise ValueError(f"{self.prefix}: this mixer rotates the first rotary_dim <= rot_dim elements, cosines and sines unscaled")
            self.rot_dims = rot.rotary_dim
            self.adjacent = rot.pairing == "adjacent"
            # angles are position * frequency in float64; the frequencies come from the position encoding
            f64 = getattr(self.position, "inv_freq64_host", None)
            f64 = rot.inv_freq.double().cpu().numpy() if f64 is None else f64
            self.freq = torch.from_numpy(np.ascontiguousarray(f64, dtype=np.float64)).to(rt.device)

    def _tile_heads(self, tiles_per_head: int, device) -> torch.Tensor:
        """int32 [H * tiles_per_head]: the head whose matrix a tile of rows meets in the grouped per-head products."""
        t = self._heads_of_tiles.get(tiles_per_head)
        if t is None:
            t = torch.arange(self.H, dtype=torch.int32, device=device).repeat_interleave(tiles_per_head).contiguous()
            self._heads_of_tiles[tiles_per_head] = t
        return t

    def weight_bytes(self):
        return (self.proj.nbytes() + self.out.nbytes() + self.w_uk.numel() * self.w_uk.element_size()
                + self.w_uv.numel() * self.w_uv.element_size() + (self.up_q.nbytes() if self.up_q is not None else 0))

    def forward(self, ctx, h, x, lay):
        n, H, D, R, V, C = h.shape[0], self.H, self.D, self.R, self.V, self.C
        if lay.writes_cache != self.own_rows:
            raise ValueError(f"{self.prefix}: a layer with rows of its own writes its cache entry, one without reads another's")
        q_cols = H * (D + R)
        first = q_cols if self.Q is None else self.Q
        down_col = first
        gate_col = first + (C + R if self.own_rows else 0)
        total = gate_col + self.gate_width()
        ld = -(-total // 8) * 8                      # rows start on 16-byte boundaries
        proj = ctx.buf("latent_proj", (n, ld), ctx.act_dtype)[:, :total]
        self.proj.forward(h, proj)
        if self.Q is None:
            qt = proj[:, :q_cols]
        else:
            # the queries' latent is normed in float32 and taken up to the heads' queries
            cq = ctx.buf("latent_cq", (n, self.Q), ctx.act_dtype)
            kernels.rmsnorm_act(proj[:, :self.Q], self.q_norm_w, cq, self.eps)
            qt = ctx.buf("latent_queries", (n, -(-q_cols // 8) * 8), ctx.act_dtype)[:, :q_cols]
            self.up_q.forward(cq, qt)
        cache_ptr, page_stride, _ = ctx.cache_layer(lay)
        bt = ctx.block_tables[lay.group]
        kernels.latent_prep(qt, proj[:, down_col:down_col + C + R] if self.own_rows else None, ctx.positions, ctx.tok_seg, bt, self.freq,
                            self.norm_w, cache_ptr if lay.writes_cache else None, page_stride, H, D, R, C, self.rot_dims,
                            ctx.max_pages, ctx.page_size, self.eps, adjacent=self.adjacent)
        o = ctx.buf("attn_out", (n, H * V), ctx.act_dtype)
        gate = proj if self.gated else None
        window = self.window or 0
        if USE_MMA and D > 0 and kernels.latent_attention_mma_supported(ctx.act_dtype, D, R, C):
            reach = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
            chunk, splits = ctx.once(("latent_splits", H, window), lambda: kernels.latent_attention_splits(n, H, reach))
            po = pm = None
            if splits > 1:
                mt = -(-H // 16)
                po = ctx.buf("latent_part_o", (n * mt * splits * 16 * C,), torch.float32)
                pm = ctx.buf("latent_part_ml", (n * mt * splits * 32,), torch.float32)
            args = (cache_ptr, page_stride, ctx.positions, ctx.tok_seg, bt, H, C, R, ctx.max_pages, ctx.page_size, self.scale, chunk, splits)
            if self.w_uk_packed is not None:
                # the two per-head products on tcgen05: rows of one head together (n_pad a head), one grouped product each
                bn = 16 if n <= 16 else (32 if n <= 32 else (64 if n <= 64 else 128))
                n_pad = -(-n // bn) * bn
                groups = self._tile_heads(n_pad // bn, h.device)
                qh = ctx.buf("latent_qh", (H * n_pad, D), torch.bfloat16)
                kernels.heads_gather(qt, 0, D + R, qh, n, n_pad, H, D)
                ql = ctx.buf("latent_q", (H * n_pad, C), torch.bfloat16)
                kernels.gemm_tc_grouped(qh, self.w_uk_packed, ql, groups, bn, C)
                ol = ctx.buf("latent_o", (H * n_pad, C), torch.bfloat16)
                kernels.latent_attention_mma(ql, qt, D, D + R, ol, po, pm, *args, n_pad=n_pad, window=window)
                oh = ctx.buf("latent_oh", (H * n_pad, V), torch.float32)
                kernels.gemm_tc_grouped(ol, self.w_uv_packed, oh, groups, bn, V)
                kernels.heads_scatter_gate(oh, o, gate, gate_col, n, n_pad, H, V, gate_each=self.gate_each)
            else:
                # the plain query parts, taken through W_uk^T into the latent space (bfloat16: an operand of the tensor cores)
                ql = ctx.buf("latent_q", (n, H * C), torch.bfloat16)
                kernels.head_matmul(qt, 0, D + R, self.w_uk, False, ql, n, H, D, C)
                ol = ctx.buf("latent_o", (n, H * C), torch.float32)
                kernels.latent_attention_mma(ql, qt, D, D + R, ol, po, pm, *args, window=window)
                kernels.head_matmul(ol, 0, C, self.w_uv, True, o, n, H, C, V, gate=gate, gate_col=gate_col, gate_each=self.gate_each)
            counters["mma"] += 1
        else:
            ql = ctx.buf("latent_q", (n, H * C), torch.float32)
            if D > 0:
                kernels.head_matmul(qt, 0, D + R, self.w_uk, False, ql, n, H, D, C)
            else:
                ql.zero_()                       # no plain query part: the scores come from the rotated parts alone
            ol = ctx.buf("latent_o", (n, H * C), torch.float32)
            kernels.latent_attention(ql, qt, D, D + R, ol, cache_ptr, page_stride, ctx.positions, ctx.tok_seg, bt, H, C, R,
                                     ctx.max_pages, ctx.page_size, self.scale, window=window)
            kernels.head_matmul(ol, 0, C, self.w_uv, True, o, n, H, C, V, gate=gate, gate_col=gate_col, gate_each=self.gate_each)
            counters["simt"] += 1
        ctx.set_pending(x, self.out.forward(o, x, accumulate=True, defer=True))


register_mixer("latent_attention", LatentAttention)
