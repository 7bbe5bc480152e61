"""Latent attention: keys and values of all heads come from one small row per token.

Per token, with h the mixer's input (H heads; per head dn unrotated and dr rotated query/key entries,
dv value entries; R the latent's size):

    q = W_q h                      per head [q_n (dn) | q_r (dr)]
    [a | k_r] = W_dkv h            a (R), k_r (dr, one for all heads)
    c = a / sqrt(mean(a^2) + eps) * g
    k_n,h = W_uk,h c;   v_h = W_uv,h c
    s_h(i, j) = (q_n,h(i) . k_n,h(j) + rot(q_r,h(i), i) . rot(k_r(j), j)) * scale,   0 <= i - j < window
    p = softmax over j with exp(sink_h) added to the denominator;   o_h = sum_j p v_h(j);   y = W_o [o_1 .. o_H]

Without ``sink`` the softmax is the ordinary one.  With ``gate`` the heads' results are multiplied element by element
by sigmoid(W_g h) before the output product: y = W_o ([o_1 .. o_H] * sigmoid(W_g h)), W_g being further rows of the
input product.

Only [c | rot(k_r)] is cached, one row of R + dr entries per token, and attention runs in the latent's
space: since q_n . (W_uk c) = (W_uk^T q_n) . c, every head's query becomes [W_uk,h^T q_n,h | rot(q_r,h)] and
all heads share the cached row as their key; the weighted sum of cached rows is projected up by W_uv,h
afterwards.  That is attention with one key/value head of size R + dr whose values are its keys, which is
what the framework's attention kernels run (the sink being one more term of their softmax).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..cache import KVSpec
from .base import ParamSpec, Part, register_part
from .linear import linear


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class LatentAttention(Part):
    kind = "mixer"
    graph_safe = True

    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float,
                 eps: float, window: Optional[int] = None, sink: bool = True, position: Optional[Part] = None,
                 gate: bool = False):
        self.has_gate = bool(gate)
        self.hidden, self.heads, self.dn, self.dr, self.dv, self.rank = hidden, heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.eps = float(scale), float(eps)
        self.window = int(window) if window else None
        self.has_sink = bool(sink)
        self.position = position
        if position is not None and position.rotary_dim > rot_dim:
            raise ValueError("latent attention: more rotated dimensions than the rotated part has")
        # the cached row, padded with zeros to a width every attention kernel takes
        self.row = _round_up(kv_rank + rot_dim, 16)
        if self.row > 512:
            raise ValueError(f"latent attention: a cached row of {self.row} entries is beyond the kernels' limit of 512")
        self.q_cols = heads * (dim + rot_dim)

    def param_specs(self):
        specs = {"q": ParamSpec((self.q_cols, self.hidden)), "dkv": ParamSpec((self.rank + self.dr, self.hidden)),
                 "dkv_norm": ParamSpec((self.rank,), "vector"), "uk": ParamSpec((self.heads * self.dn, self.rank)),
                 "uv": ParamSpec((self.heads * self.dv, self.rank)), "o": ParamSpec((self.hidden, self.heads * self.dv))}
        if self.has_sink:
            specs["sink"] = ParamSpec((self.heads,), "vector")
        if self.has_gate:
            specs["g"] = ParamSpec((self.heads * self.dv, self.hidden))
        return specs

    def bind(self, params):
        kinds = {params[n].dtype for n in ("q", "dkv", "uk", "uv", "dkv_norm") + (("g",) if self.has_gate else ())}
        if len(kinds) > 1:
            raise TypeError("latent attention: its matrices and the latent's gain must have one element type")
        # one product for the queries, the compressed row and the gate's logits: rows [Wq; Wdkv; Wg]
        self.w_in = torch.cat([params["q"], params["dkv"]] + ([params["g"]] if self.has_gate else []), dim=0).contiguous()
        self.gate_from = self.q_cols + self.rank + self.dr
        self.gain = params["dkv_norm"].contiguous()
        # per head: W_uk^T (R, dn) for the queries' way into the latent's space, W_uv (dv, R) for the way out
        self.w_qk = params["uk"].view(self.heads, self.dn, self.rank).transpose(1, 2).contiguous()
        self.w_uv = params["uv"].view(self.heads, self.dv, self.rank).contiguous()
        self.w_o = params["o"]
        self.sink = params["sink"].float().contiguous() if self.has_sink else None
        self.params = {}

    def cache_spec(self):
        return KVSpec(1, self.row, self.window, values=False)

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def forward(self, x: torch.Tensor, ctx, entry, writes_cache: bool = True) -> torch.Tensor:
        """x (tokens, hidden) in the step's element type -> (tokens, hidden) float32 (or partial sums)."""
        pages, _, table, ring, page = ctx.kv(entry)
        T, H, D = x.shape[0], self.heads, self.row
        if x.dtype != self.w_in.dtype:
            x = x.to(self.w_in.dtype)
        proj = linear(x, self.w_in, out_dtype=x.dtype)
        lat = torch.empty((T, D), dtype=x.dtype, device=x.device)
        q = torch.empty((T, H * D), dtype=x.dtype, device=x.device)
        pos = self.position
        kernels.latent_rows(proj, self.q_cols, ctx.positions, pos.table if pos is not None else None,
                            pos.rotary_dim if pos is not None else 0, self.gain, self.eps, H, self.dn, self.dr,
                            self.rank, lat, q, pages if writes_cache else None,
                            ctx.cache_rows[entry.group_id] if writes_cache else None)
        kernels.heads_linear(proj, self.dn + self.dr, self.w_qk, q, D)        # columns 0 .. R of every head of q
        out = torch.empty((T, H * D), dtype=x.dtype, device=x.device)
        common = dict(n_kv=1, group=H, head_dim=D, scale=self.scale, cap=0.0, window=self.window or 0,
                      batch=ctx.batch, sink=self.sink)
        tensor_cores = x.dtype == torch.bfloat16 and D <= 256
        if ctx.mode == "prefill" and writes_cache:
            # the step's own rows, still packed: a prompt longer than the window needs rows the ring no longer holds
            if tensor_cores:
                kernels.attention_prefill_mma(q, out, ctx.cu_q, lat, lat, max_q_len=ctx.max_q_len, **common)
            else:
                kernels.attention_simt(q, out, ctx.cu_q, ctx.kv_len, k=lat, v=lat, max_q_len=ctx.max_q_len, **common)
        elif tensor_cores and ctx.mode == "decode" and page == 64 and H <= 16:
            splits = kernels.decode_splits(ctx.batch, 1, ctx.max_kv_len, self.window or 0,
                                           ragged=getattr(ctx, "ragged", False))
            if H * D >= 2048:
                # every split leaves H * D floats for the block that merges them; up to four are merged in one
                # round trip, and with all heads on one cached row a split is cheap to run and dear to merge
                splits = min(splits, 4)
            kernels.attention_decode_mma(q, out, ctx.cu_q, ctx.kv_len, pages, pages, table, ring=ring, page_size=page,
                                         n_splits=splits, **common)
        else:
            if ctx.mode == "prefill" and self.window and ctx.max_kv_len > ring:
                raise NotImplementedError("a layer that reads another layer's windowed cache cannot take a "
                                          "prompt longer than the ring in one step")
            kernels.attention_simt(q, out, ctx.cu_q, ctx.kv_len, k_pages=pages, v_pages=pages, page_table=table,
                                   ring=ring, page_size=page, max_q_len=ctx.max_q_len, **common)
        o = torch.empty((T, H * self.dv), dtype=x.dtype, device=x.device)
        kernels.heads_linear(out, D, self.w_uv, o, self.dv)
        if self.has_gate:
            gated = torch.empty_like(o)
            kernels.norm_sigmoid_gate(o, proj[:, self.gate_from:], None, 0.0, gated)
            o = gated
        return linear(o, self.w_o, out_dtype=torch.float32, parts_ok=True)


register_part("mixer", "latent_attention", LatentAttention)
