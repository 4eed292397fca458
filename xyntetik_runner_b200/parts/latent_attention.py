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
in the half-split pairing.
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
                 q: str = "q", dkv: str = "dkv", dkv_norm: str = "dkv.norm", uk: str = "uk", uv: str = "uv", g: str = "g", o: str = "o"):
        if kv_rank > 1024:
            raise ValueError(f"{prefix}: latent size {kv_rank}: the attention kernel takes up to 1024")
        self.width, self.H, self.D, self.R, self.V, self.C = width, heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.position, self.eps, self.prefix, self.gated = float(scale), position, float(eps), prefix, gated
        self.names = {k: prefix + v for k, v in dict(q=q, dkv=dkv, norm=dkv_norm, uk=uk, uv=uv, g=g, o=o).items()}
        self.proj = self.out = self.w_uk = self.w_uv = self.norm_w = self.freq = None
        self.w_uk_packed = self.w_uv_packed = None
        self.rot_dims = 0

    def kv_need(self):
        return KVNeed(1, self.C + self.R, None, planes=1)

    def tensors(self):
        n, H, D, R, V, C, W = self.names, self.H, self.D, self.R, self.V, self.C, self.width
        t = {n["q"]: TensorSpec((H * (D + R), W)), n["dkv"]: TensorSpec((C + R, W)),
             n["norm"]: TensorSpec((C,), "vector", "ones_jitter"), n["uk"]: TensorSpec((H * D, C)),
             n["uv"]: TensorSpec((H * V, C)), n["o"]: TensorSpec((W, H * V))}
        if self.gated:
            t[n["g"]] = TensorSpec((H, W))
        return t

    def bind(self, tensors, rt):
        n = self.names
        ws = [tensors.pop(n["q"]), tensors.pop(n["dkv"])] + ([tensors.pop(n["g"])] if self.gated else [])
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        # one product for the queries, the down projection and the heads' gates
        self.proj = Linear(torch.cat(ws, dim=0)).prepare(rt)
        del ws
        self.out = Linear(tensors[n["o"]]).prepare(rt)
        self.w_uk, self.w_uv = tensors[n["uk"]].contiguous(), tensors[n["uv"]].contiguous()
        # for the tensor-core products per head: W_uk,h^T ([C, D]: the query goes into the latent space) and W_uv,h ([V, C])
        self.w_uk_packed = self.w_uv_packed = None
        if (linear_tc.ENABLED and rt.act_dtype == torch.bfloat16 and self.w_uk.dtype == torch.bfloat16 and self.w_uv.dtype == torch.bfloat16
                and self.w_uk.is_cuda and self.D % 8 == 0 and self.D >= 8 and self.C % 8 == 0):
            self.w_uk_packed = kernels.pack_weight_groups(self.w_uk.view(self.H, self.D, self.C).transpose(1, 2).contiguous())
            self.w_uv_packed = kernels.pack_weight_groups(self.w_uv.view(self.H, self.V, self.C))
        self._heads_of_tiles = {}
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()
        self.position.prepare(rt)
        rot = self.position.rotary()
        if rot is not None and rot.rotary_dim:
            if rot.pairing != "half" or rot.mscale != 1.0 or rot.rotary_dim > self.R:
                raise ValueError(f"{self.prefix}: this mixer rotates the first rotary_dim <= rot_dim elements in the half-split pairing")
            self.rot_dims = rot.rotary_dim
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
                + self.w_uv.numel() * self.w_uv.element_size())

    def forward(self, ctx, h, x, lay):
        n, H, D, R, V, C = h.shape[0], self.H, self.D, self.R, self.V, self.C
        q_cols = H * (D + R)
        total = q_cols + C + R + (H if self.gated else 0)
        ld = -(-total // 8) * 8                      # rows start on 16-byte boundaries
        proj = ctx.buf("latent_proj", (n, ld), ctx.act_dtype)[:, :total]
        self.proj.forward(h, proj)
        cache_ptr, page_stride, _ = ctx.cache_layer(lay)
        bt = ctx.block_tables[lay.group]
        kernels.latent_prep(proj, q_cols, ctx.positions, ctx.tok_seg, bt, self.freq, self.norm_w,
                            cache_ptr if lay.writes_cache else None, page_stride, H, D, R, C, self.rot_dims,
                            ctx.max_pages, ctx.page_size, self.eps)
        o = ctx.buf("attn_out", (n, H * V), ctx.act_dtype)
        gate = proj if self.gated else None
        if USE_MMA and D > 0 and kernels.latent_attention_mma_supported(ctx.act_dtype, D, R, C):
            chunk, splits = ctx.once(("latent_splits", H), lambda: kernels.latent_attention_splits(n, H, ctx.max_kv_len))
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
                kernels.heads_gather(proj, 0, D + R, qh, n, n_pad, H, D)
                ql = ctx.buf("latent_q", (H * n_pad, C), torch.bfloat16)
                kernels.gemm_tc_grouped(qh, self.w_uk_packed, ql, groups, bn, C)
                ol = ctx.buf("latent_o", (H * n_pad, C), torch.bfloat16)
                kernels.latent_attention_mma(ql, proj, D, D + R, ol, po, pm, *args, n_pad=n_pad)
                oh = ctx.buf("latent_oh", (H * n_pad, V), torch.float32)
                kernels.gemm_tc_grouped(ol, self.w_uv_packed, oh, groups, bn, V)
                kernels.heads_scatter_gate(oh, o, gate, q_cols + C + R, n, n_pad, H, V)
            else:
                # the plain query parts, taken through W_uk^T into the latent space (bfloat16: an operand of the tensor cores)
                ql = ctx.buf("latent_q", (n, H * C), torch.bfloat16)
                kernels.head_matmul(proj, 0, D + R, self.w_uk, False, ql, n, H, D, C)
                ol = ctx.buf("latent_o", (n, H * C), torch.float32)
                kernels.latent_attention_mma(ql, proj, D, D + R, ol, po, pm, *args)
                kernels.head_matmul(ol, 0, C, self.w_uv, True, o, n, H, C, V, gate=gate, gate_col=q_cols + C + R)
            counters["mma"] += 1
        else:
            ql = ctx.buf("latent_q", (n, H * C), torch.float32)
            if D > 0:
                kernels.head_matmul(proj, 0, D + R, self.w_uk, False, ql, n, H, D, C)
            else:
                ql.zero_()                       # no plain query part: the scores come from the rotated parts alone
            ol = ctx.buf("latent_o", (n, H * C), torch.float32)
            kernels.latent_attention(ql, proj, D, D + R, ol, cache_ptr, page_stride, ctx.positions, ctx.tok_seg, bt, H, C, R,
                                     ctx.max_pages, ctx.page_size, self.scale)
            kernels.head_matmul(ol, 0, C, self.w_uv, True, o, n, H, C, V, gate=gate, gate_col=q_cols + C + R)
            counters["simt"] += 1
        ctx.set_pending(x, self.out.forward(o, x, accumulate=True, defer=True))


register_mixer("latent_attention", LatentAttention)
