"""The attention mixer: grouped-query attention with rotary positions, a
score scale of its own, tanh soft-capping of the scores and an optional
sliding window, over a paged cache.

Formulas as wlejon/brolm computes them (src/gemma2.cpp:349-369): fused q/k/v
projection without bias, rotation of q and k at the absolute position, k and
v into the cache, scores = q.k * scale -> cap * tanh(./cap) -> causal/window
mask -> softmax, then the output projection.  Key j is visible from position
p iff 0 <= p - j < window.

Options beside those: value heads of a size of their own (``v_dim``); an RMS
norm of the whole query row and of the whole key row, one statistic over all
heads, with a gain per element (``qk_norm="whole"``, tensors ``q_norm`` and
``k_norm``); a chunked mask (``chunk`` = C: key j is visible from p iff j <= p
and j >= p - p % C, chunks counted from position 0), kept in the cache as a
ring of C places like a window.  A layer that uses one of them runs its
projection with a float result, the row-wise kernel that norms and fills the
cache, and the exact attention kernel.

A third set of options works one head at a time between the projection and
the attention (``headwise``; the notation: H query heads, G key/value heads,
head h reads kv head h // (H / G)):

* ``bias``: q, k, v and the output projection have a bias each;
* ``taps`` = K > 0: a causal convolution per channel over time on the projected
  q, k and v (``y_t = sum_j w[:, j] u_(t - K + 1 + j)``, zeros before the
  sequence's start), whose last K - 1 inputs are kept per sequence in a state
  entry beside the keys and values;
* ``qk_norm="head"``: every q and k head divided by its own root mean square
  (``eps``), no gain; with ``qk_gain`` the normed heads are multiplied by a gain of
  ``head_dim`` numbers, one for all query heads (tensor ``q_norm``) and one for
  all key heads (``k_norm``);
* ``sink``: a learned number per query head (tensor ``sink``) whose exponential
  joins the softmax's denominator: it has no key and no value, and is neither
  scaled nor capped;
* ``distance_rows`` = B > 0 with ``distance_far`` = D: a learned bias by distance
  (tensor ``rel``, B rows of one number per query head) is added to the score
  after the scale and the cap; key j at distance n = p - j reads row n for
  n < B/2, else min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(D / (B/2)) (B - B/2)));
  with ``distance_rows_free`` B is whatever the checkpoint's tensor has, and
  ``distance_rows`` only says how many rows a tensor made at random gets;
* a rotation of part of a head, in either pairing, also with ``v_dim``;
* ``slope_power`` = s > 0: slope_h * (p - j) is taken off the scaled score of
  key j at query position p, slope_h = 2^(-s (h + 1) / H);
* ``keep_first`` = F with a window: keys at positions below F stay visible
  however far back they lie, at their true positions;
* ``talk``: the heads' softmax weights are mixed by an H x H matrix before they
  meet the values, w'_h = sum_g talk[h, g] w_g, head h applying w'_h to the
  values of its own kv head.  The attention kernel applies every head's
  weights to the values of every kv head (float results [H, G, v_dim]) and a
  row-wise kernel takes the sums over g;  in bfloat16 that kernel, like the
  one for slopes, kept first keys and value rows of their own size, runs on
  the tensor cores (``attention_headmix_*``);
* ``gate``: head h's result is multiplied by sigmoid(W_g x)_h, W_g being H rows
  of the fused projection;
* ``v_mix``: "source" leaves the layer's values of the step's tokens (float,
  before rounding) under ``v_mix_key`` for later layers of the same pass;
  "mixed" makes v <- (1 - lambda) v + lambda v_source with a learned scalar
  lambda, and that is what the cache keeps.  Both hold a tensor ``vmix``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels
from ..cache import KVSpec, StateSpec
from .base import ParamSpec, Part, register_part
from .linear import linear


def distance_buckets(rows: int, far: float) -> list:
    """The row of a distance-bias table that each distance n = 0, 1, ... reads, up to and including the first
    distance that reads the last row (every larger one reads it too): n itself below rows // 2, then steps that
    grow like the logarithm of n, reaching the last row at ``far``."""
    half = rows // 2
    out, n = [], 0
    while True:
        if n < half:
            b = n
        else:
            b = min(rows - 1, half + math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))
        out.append(b)
        if b == rows - 1:
            return out
        n += 1


class Attention(Part):
    kind = "mixer"
    graph_safe = True

    def __init__(self, hidden: int, n_q: int, n_kv: int, head_dim: int, scale: float, softcap: float = 0.0,
                 window: Optional[int] = None, position: Optional[Part] = None, v_dim: Optional[int] = None,
                 qk_norm: str = "none", eps: float = 0.0, chunk: Optional[int] = None, bias: bool = False, taps: int = 0,
                 slope_power: float = 0.0, keep_first: int = 0, talk: bool = False, gate: bool = False,
                 v_mix: Optional[str] = None, v_mix_key: str = "v_first", qk_gain: bool = False, sink: bool = False,
                 distance_rows: int = 0, distance_far: float = 0.0, distance_rows_free: bool = False):
        if n_q % n_kv:
            raise ValueError("attention: the number of query heads must be a multiple of the kv heads")
        rotation = getattr(position, "pairing", "half")
        self.headwise = bool(bias or taps or qk_norm == "head" or slope_power or keep_first or talk or gate or v_mix
                             or sink or distance_rows
                             or (position is not None and ((v_dim and v_dim != head_dim) or rotation != "half")))
        plain = not (v_dim and v_dim != head_dim) and qk_norm == "none" and not chunk and not self.headwise
        if plain and head_dim % 16:
            raise ValueError(f"attention: head_dim {head_dim} is not a multiple of 16; the kernels refuse it")
        if head_dim > 512:
            raise ValueError(f"attention: head_dim {head_dim} is beyond the kernels' limit of 512")
        if qk_norm not in ("none", "whole", "head"):
            raise ValueError(f"attention: unknown qk_norm '{qk_norm}' (none, whole, head)")
        if v_mix not in (None, "source", "mixed"):
            raise ValueError(f"attention: unknown v_mix '{v_mix}' (source, mixed)")
        if taps < 0 or keep_first < 0 or slope_power < 0:
            raise ValueError("attention: taps, keep_first and slope_power cannot be negative")
        if keep_first and not window:
            keep_first = 0                    # every key is visible anyway
        if self.headwise and qk_norm == "whole":
            raise ValueError("attention: a whole-row norm together with the head-wise options is not built")
        if self.headwise and softcap and talk:
            raise ValueError("attention: a soft cap together with mixed heads' weights is not built")
        if qk_gain and qk_norm != "head":
            raise ValueError("attention: a gain per head element goes with qk_norm='head'")
        if distance_rows < 0 or (distance_rows and (distance_rows < 2 or not distance_far > distance_rows // 2)):
            raise ValueError("attention: the distance bias needs at least two rows and distance_far beyond half of them")
        if (sink or distance_rows) and talk:
            raise ValueError("attention: a sink or a distance bias together with mixed heads' weights is not built")
        if keep_first and chunk:
            raise ValueError("attention: kept first keys together with a chunked mask are not built")
        self.hidden, self.n_q, self.n_kv, self.head_dim = hidden, n_q, n_kv, head_dim
        self.v_dim = int(v_dim) if v_dim else head_dim
        self.scale, self.softcap = float(scale), float(softcap or 0.0)
        self.window = int(window) if window else None
        self.chunk = int(chunk) if chunk else None
        self.qk_norm, self.eps = qk_norm, float(eps)
        self.position = position
        self.q_dim, self.kv_dim, self.v_cols = n_q * head_dim, n_kv * head_dim, n_kv * self.v_dim
        # the options of the second paragraph above: their own row-wise kernel and the exact attention
        self.bias, self.taps, self.slope_power, self.keep_first = bool(bias), int(taps), float(slope_power), int(keep_first)
        self.talk, self.gate, self.v_mix, self.v_mix_key = bool(talk), bool(gate), v_mix, v_mix_key
        self.qk_gain, self.has_sink = bool(qk_gain), bool(sink)
        self.distance_rows, self.distance_far = int(distance_rows), float(distance_far)
        self.distance_rows_free = bool(distance_rows_free)
        self.cols = self.q_dim + self.kv_dim + self.v_cols
        self.slopes = None
        self.rowwise = (self.v_dim != head_dim or qk_norm != "none" or self.chunk is not None) and not self.headwise
        if self.headwise and (self.v_dim > 512 or n_q > 128):
            raise ValueError("attention: v_dim beyond 512 or more than 128 heads are beyond the head-wise kernels")
        if self.rowwise:
            if self.v_dim > 512:
                raise ValueError(f"attention: v_dim {self.v_dim} is beyond the kernels' limit of 512")
            if position is not None:
                raise ValueError("attention: a rotation together with v_dim, qk_norm or chunk is not built")

    def param_specs(self):
        specs = {"q": ParamSpec((self.q_dim, self.hidden)), "k": ParamSpec((self.kv_dim, self.hidden)),
                 "v": ParamSpec((self.v_cols, self.hidden)), "o": ParamSpec((self.hidden, self.n_q * self.v_dim))}
        if self.qk_norm == "whole":
            specs["q_norm"] = ParamSpec((self.q_dim,), "vector")
            specs["k_norm"] = ParamSpec((self.kv_dim,), "vector")
        if self.qk_gain:
            specs["q_norm"] = ParamSpec((self.head_dim,), "vector")
            specs["k_norm"] = ParamSpec((self.head_dim,), "vector")
        if self.has_sink:
            specs["sink"] = ParamSpec((self.n_q,), "vector")
        if self.distance_rows:
            specs["rel"] = ParamSpec((-self.distance_rows if self.distance_rows_free else self.distance_rows, self.n_q),
                                     "vector")
        if self.bias:
            specs.update(q_bias=ParamSpec((self.q_dim,), "vector"), k_bias=ParamSpec((self.kv_dim,), "vector"),
                         v_bias=ParamSpec((self.v_cols,), "vector"), o_bias=ParamSpec((self.hidden,), "vector"))
        if self.taps:
            specs.update(q_conv=ParamSpec((self.q_dim, self.taps), "vector"), k_conv=ParamSpec((self.kv_dim, self.taps), "vector"),
                         v_conv=ParamSpec((self.v_cols, self.taps), "vector"))
        if self.talk:
            specs["talk"] = ParamSpec((self.n_q, self.n_q), "vector")
        if self.gate:
            specs["gate"] = ParamSpec((self.n_q, self.hidden))
        if self.v_mix:
            specs["vmix"] = ParamSpec((), "vector")
        return specs

    def bind(self, params):
        # one projection for q, k and v: rows [Wq; Wk; Wv]
        kinds = {params[n].dtype for n in ("q", "k", "v")}
        dt = torch.float32 if (len(kinds) > 1 or torch.float32 in kinds) else next(iter(kinds))
        rows = [params["q"].to(dt), params["k"].to(dt), params["v"].to(dt)]
        if self.gate:
            rows.append(params["gate"].to(dt))               # the gates' logits are columns of the same product
        self.w_qkv = torch.cat(rows, dim=0).contiguous()
        self.w_o = params["o"]
        f32 = lambda *names: torch.cat([params[n].float() for n in names], dim=0).contiguous()
        self.in_bias = f32("q_bias", "k_bias", "v_bias") if self.bias else None
        self.o_bias = params["o_bias"].float().contiguous() if self.bias else None
        self.conv = f32("q_conv", "k_conv", "v_conv") if self.taps else None
        self.w_talk = params["talk"].float().contiguous() if self.talk else None
        self.lam = params["vmix"].float().reshape(1).contiguous() if self.v_mix == "mixed" else None
        self.q_gain = self.k_gain = None
        if self.qk_gain:
            self.q_gain, self.k_gain = params["q_norm"].float().contiguous(), params["k_norm"].float().contiguous()
        self.sink = params["sink"].float().contiguous() if self.has_sink else None
        self.dist_bias = None
        if self.distance_rows:
            # laid out by distance: [head][n] for n up to the first distance that reads the last row (all further do)
            n_rows = params["rel"].shape[0]
            if n_rows < 2 or not self.distance_far > n_rows // 2:
                raise ValueError(f"attention: a distance bias of {n_rows} rows does not go with distance_far "
                                 f"{self.distance_far}")
            rows = torch.tensor(distance_buckets(n_rows, self.distance_far), device=params["rel"].device)
            self.dist_bias = params["rel"].float().index_select(0, rows).t().contiguous()
        if self.qk_norm == "whole":
            gd = torch.float32 if params["q_norm"].dtype != params["k_norm"].dtype else params["q_norm"].dtype
            self.q_gain, self.k_gain = params["q_norm"].to(gd).contiguous(), params["k_norm"].to(gd).contiguous()
        self.params = {}

    def cache_spec(self):
        if self.headwise:
            kv = KVSpec(self.n_kv, self.head_dim, self.window, v_dim=self.v_dim if self.v_dim != self.head_dim else None,
                        chunk=self.chunk, keep_first=self.keep_first)
            if not self.taps:
                return kv
            # the convolution's last taps - 1 inputs (the projected q | k | v of those tokens, biases included)
            return (kv, StateSpec((max(1, (self.taps - 1) * self.cols),), torch.float32))
        if self.rowwise:
            return KVSpec(self.n_kv, self.head_dim, self.window, v_dim=self.v_dim if self.v_dim != self.head_dim else None,
                          chunk=self.chunk)
        return KVSpec(self.n_kv, self.head_dim, self.window)

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)
        if self.slope_power and (self.slopes is None or self.slopes.device != torch.device(device)):
            h = torch.arange(1, self.n_q + 1, dtype=torch.float64)
            self.slopes = torch.pow(torch.tensor(2.0, dtype=torch.float64), -self.slope_power * h / self.n_q) \
                .to(torch.float32).to(device)

    def forward(self, x: torch.Tensor, ctx, entry, writes_cache: bool = True) -> torch.Tensor:
        """x (tokens, hidden) in the step's element type -> (tokens, hidden) float32, or
        [parts, tokens, hidden] partial sums that the residual kernel adds."""
        if self.headwise:
            return self._forward_headwise(x, ctx, entry, writes_cache)
        k_pages, v_pages, table, ring, page = ctx.kv(entry)
        if self.rowwise:
            return self._forward_rowwise(x, ctx, entry, writes_cache)
        rot = self.position.rotary_dim if self.position is not None else 0
        cos_sin = self.position.table if self.position is not None else None
        kept = (k_pages, v_pages, ctx.cache_rows[entry.group_id]) if writes_cache else (None, None, None)
        if kernels.skinny_ok(x, self.w_qkv) and (cos_sin is None or rot == self.head_dim):
            # a few tokens: the rotation and the write into the cache are the product's epilogue
            qkv = torch.empty((x.shape[0], self.q_dim + 2 * self.kv_dim), dtype=ctx.dtype, device=x.device)
            kernels.skinny_qkv_rope(x, self.w_qkv, qkv, ctx.positions, cos_sin, self.n_q, self.n_kv, self.head_dim,
                                    *kept, page)
        elif kernels.stream_rows(x, self.w_qkv) and (cos_sin is None or rot == self.head_dim):
            # 17 to 128 tokens: the weights stream once through tcgen05, cut along K so that every SM takes
            # part; the kernel that rotates q and k and fills the cache adds the slices on its way
            slices = kernels.gemm_stream_parts(x, self.w_qkv)
            sums = torch.empty((slices, x.shape[0], self.q_dim + 2 * self.kv_dim), dtype=torch.float32, device=x.device)
            kernels.gemm_stream(x, self.w_qkv, sums)
            qkv = torch.empty((x.shape[0], self.q_dim + 2 * self.kv_dim), dtype=ctx.dtype, device=x.device)
            kernels.rope_kv_write_parts(sums, qkv, ctx.positions, cos_sin, self.n_q, self.n_kv, self.head_dim, *kept,
                                        page)
        else:
            qkv = linear(x, self.w_qkv, out_dtype=ctx.dtype)
            kernels.rope_kv_write(qkv, ctx.positions, cos_sin, self.n_q, self.n_kv, self.head_dim, rot, *kept, page)
        q = qkv[:, :self.q_dim]
        out = torch.empty((qkv.shape[0], self.q_dim), dtype=ctx.dtype, device=x.device)
        common = dict(n_kv=self.n_kv, group=self.n_q // self.n_kv, head_dim=self.head_dim, scale=self.scale,
                      cap=self.softcap, window=self.window or 0, batch=ctx.batch, max_q_len=ctx.max_q_len)
        if ctx.mode == "prefill" and writes_cache:
            # the step's own keys and values, still packed: a prompt longer than
            # the window needs keys the ring no longer holds
            k = qkv[:, self.q_dim:self.q_dim + self.kv_dim]
            v = qkv[:, self.q_dim + self.kv_dim:]
            self.attend_packed(q, k, v, out, ctx, common)
        else:
            if ctx.mode == "prefill" and self.window and ctx.max_kv_len > ring:
                raise NotImplementedError("a layer that reads another layer's windowed cache cannot take a "
                                          "prompt longer than the ring in one step")
            self.attend_paged(q, out, ctx, common, k_pages, v_pages, table, ring, page)
        return linear(out, self.w_o, out_dtype=torch.float32, parts_ok=True)

    def _forward_rowwise(self, x, ctx, entry, writes_cache):
        """The path of a layer with a whole-row norm, value heads of their own size or a chunked mask."""
        k_pages, v_pages, table, ring, page = ctx.kv(entry)
        if ctx.mode == "prefill" and not writes_cache:
            raise NotImplementedError("a layer of this kind that reads another layer's cache cannot take a prompt")
        proj = linear(x, self.w_qkv, out_dtype=torch.float32)
        qkv = proj if ctx.dtype == torch.float32 else torch.empty(proj.shape, dtype=ctx.dtype, device=x.device)
        kept = (k_pages, v_pages, ctx.cache_rows[entry.group_id]) if writes_cache else (None, None, None)
        kernels.qkv_norm_write(proj, self.q_dim, self.kv_dim, self.v_cols, self.q_gain, self.k_gain, self.eps,
                               ctx.positions, qkv, self.n_kv, *kept, page)
        q = qkv[:, :self.q_dim]
        out = torch.empty((qkv.shape[0], self.n_q * self.v_dim), dtype=ctx.dtype, device=x.device)
        common = dict(n_kv=self.n_kv, group=self.n_q // self.n_kv, head_dim=self.head_dim, scale=self.scale,
                      cap=self.softcap, window=self.window or 0, batch=ctx.batch, max_q_len=ctx.max_q_len,
                      v_dim=self.v_dim, chunk=self.chunk or 0)
        # bfloat16 with key and value rows of one size runs on the tensor cores; all else on the exact kernel
        tensor = self._tensor_cores(ctx) and self.v_dim == self.head_dim and self.head_dim % 16 == 0
        k, v = qkv[:, self.q_dim:self.q_dim + self.kv_dim], qkv[:, self.q_dim + self.kv_dim:]
        if ctx.mode == "prefill" and tensor:
            kernels.attention_prefill_mma(q, out, ctx.cu_q, k, v, **{n: a for n, a in common.items() if n != "v_dim"})
        elif ctx.mode == "prefill":
            kernels.attention_simt(q, out, ctx.cu_q, ctx.kv_len, k=k, v=v, **common)
        elif tensor and page == 64:
            span = min(self.window or (1 << 30), self.chunk or (1 << 30))
            splits = kernels.decode_splits(ctx.batch, self.n_kv, ctx.max_kv_len, span if span < (1 << 30) else 0,
                                           ragged=getattr(ctx, "ragged", False))
            kernels.attention_decode_mma(q, out, ctx.cu_q, ctx.kv_len, k_pages, v_pages, table, ring=ring, page_size=page,
                                         n_splits=splits, **{n: a for n, a in common.items() if n not in ("v_dim", "max_q_len")})
        else:
            kernels.attention_simt(q, out, ctx.cu_q, ctx.kv_len, k_pages=k_pages, v_pages=v_pages, page_table=table,
                                   ring=ring, page_size=page, **common)
        return linear(out, self.w_o, out_dtype=torch.float32, parts_ok=True)

    def _forward_headwise(self, x, ctx, entry, writes_cache):
        """The path of a layer with one of the head-wise options of the module's third paragraph."""
        if not writes_cache:
            raise NotImplementedError("a layer of this kind cannot run on another layer's cache")
        kv_entry, conv_entry = (entry.parts[0], entry.parts[1]) if self.taps else (entry, None)
        k_pages, v_pages, table, ring, page = ctx.kv(kv_entry)
        T, cols, dev = x.shape[0], self.cols, x.device
        proj = linear(x, self.w_qkv, out_dtype=torch.float32)             # [ q | k | v | gate logits ]
        rows, bias = proj[:, :cols], self.in_bias
        if self.taps:
            seq = (ctx.cu_q, ctx.kv_len, ctx.slots_dev, ctx.state(conv_entry))
            conv = torch.empty((T, cols), dtype=torch.float32, device=dev)
            kernels.causal_conv(rows, bias, self.conv, None, "none", ctx.tok_seq, ctx.positions, *seq, 0, conv)
            kernels.conv_tail(rows, bias, self.taps, *seq, 0, ctx.batch)
            rows, bias = conv, None
        mix = v_first = v_keep = None
        if self.v_mix == "source":
            v_keep = ctx.carry[self.v_mix_key] = torch.empty((T, self.v_cols), dtype=torch.float32, device=dev)
        elif self.v_mix == "mixed":
            if self.v_mix_key not in ctx.carry:
                raise RuntimeError(f"attention: no earlier layer of this pass left '{self.v_mix_key}'")
            mix, v_first = self.lam, ctx.carry[self.v_mix_key]
        qkv = torch.empty((T, cols), dtype=ctx.dtype, device=dev)
        pos = self.position
        kernels.qkv_finish(rows, bias, self.n_q, self.n_kv, self.head_dim, self.v_dim, ctx.positions, qkv,
                           head_norm=self.qk_norm == "head", eps=self.eps,
                           cos_sin=pos.table if pos is not None else None,
                           rotary_dim=pos.rotary_dim if pos is not None else 0,
                           pairing=pos.pairing if pos is not None else "half", mix=mix, v_first=v_first, v_keep=v_keep,
                           q_gain=self.q_gain, k_gain=self.k_gain, k_pages=k_pages, v_pages=v_pages, cache_rows=ctx.cache_rows[kv_entry.group_id], page_size=page)
        q = qkv[:, :self.q_dim]
        k, v = qkv[:, self.q_dim:self.q_dim + self.kv_dim], qkv[:, self.q_dim + self.kv_dim:]
        group = self.n_q // self.n_kv
        common = dict(n_kv=self.n_kv, group=group, head_dim=self.head_dim, scale=self.scale, cap=self.softcap,
                      window=self.window or 0, batch=ctx.batch, max_q_len=ctx.max_q_len)
        out = torch.empty((T, self.n_q * self.v_dim), dtype=ctx.dtype, device=dev)
        scored = bool(self.softcap or self.has_sink or self.dist_bias is not None)     # options of the score itself
        special = self.talk or self.gate or self.slopes is not None or self.keep_first or self.chunk
        same_size = self.v_dim == self.head_dim and self.head_dim % 16 == 0 and self._tensor_cores(ctx)
        if not special and same_size and scored and (ctx.mode == "prefill" or page == 64):
            # key and value rows of one size: the plain layers' mma.sync kernels, which know the cap, the sink and
            # the distance table (and stage keys and values through more buffers than the head-wise ones)
            more = dict(sink=self.sink, dist_bias=self.dist_bias)
            if ctx.mode == "prefill":
                kernels.attention_prefill_mma(q, out, ctx.cu_q, k, v, **common, **more)
            else:
                splits = kernels.decode_splits(ctx.batch, self.n_kv, ctx.max_kv_len, self.window or 0,
                                               ragged=getattr(ctx, "ragged", False))
                kernels.attention_decode_mma(q, out, ctx.cu_q, ctx.kv_len, k_pages, v_pages, table, ring=ring,
                                             page_size=page, n_splits=splits, **more,
                                             **{n: a for n, a in common.items() if n != "max_q_len"})
        elif not special and not scored and same_size:
            # nothing the tensor-core kernels do not know: the same attention as a plain layer's
            if ctx.mode == "prefill":
                self.attend_packed(q, k, v, out, ctx, common)
            else:
                self.attend_paged(q, out, ctx, common, k_pages, v_pages, table, ring, page)
        else:
            exact = dict(common, v_dim=self.v_dim, chunk=self.chunk or 0, slopes=self.slopes, keep_first=self.keep_first,
                         sink=self.sink, dist_bias=self.dist_bias)
            if ctx.mode == "prefill":
                source = dict(k=k, v=v)
            else:
                source = dict(k_pages=k_pages, v_pages=v_pages, page_table=table, ring=ring, page_size=page,
                              ring_from=ctx.ring_from(kv_entry))
            # bfloat16 without a chunked mask runs on the tensor cores, all else on the exact kernel
            tensor = self._tensor_cores(ctx) and not self.chunk and not (scored and self.talk) and \
                kernels.attention_headmix_ok(self.head_dim, self.v_dim, group, ctx.mode != "prefill", page)

            def attend(dst, all_values=False):
                if not tensor:
                    if all_values:
                        kernels.attention_all_values(q, dst, ctx.cu_q, ctx.kv_len, **exact, **source)
                    else:
                        kernels.attention_simt(q, dst, ctx.cu_q, ctx.kv_len, **exact, **source)
                    return
                args = dict(n_kv=self.n_kv, group=group, head_dim=self.head_dim, v_dim=self.v_dim, scale=self.scale,
                            window=self.window or 0, batch=ctx.batch, slopes=self.slopes, keep_first=self.keep_first,
                            all_values=all_values, cap=self.softcap, sink=self.sink, dist_bias=self.dist_bias)
                if ctx.mode == "prefill":
                    kernels.attention_headmix_prefill(q, dst, ctx.cu_q, k, v, max_q_len=ctx.max_q_len, **args)
                else:
                    shares = kernels.attention_headmix_shares_keys(self.head_dim, self.v_dim, self.n_kv, group, all_values)
                    rows = self.n_kv * (self.n_kv if all_values and not shares else 1)
                    splits = kernels.headmix_splits(ctx.batch, rows, ctx.max_kv_len, self.window or 0, self.keep_first,
                                                    rounds=1 if shares else None)
                    kernels.attention_headmix_decode(q, dst, ctx.cu_q, ctx.kv_len, k_pages, v_pages, table, ring=ring,
                                                     ring_from=ctx.ring_from(kv_entry), page_size=page,
                                                     n_splits=splits, **args)

            if self.talk:
                # every head's weights on the values of every kv head, then the mixing (and the gate) row by row
                acc = torch.empty((T, self.n_q * self.n_kv * self.v_dim), dtype=torch.float32, device=dev)
                attend(acc, all_values=True)
                kernels.heads_mix(acc, self.w_talk, proj[:, cols:] if self.gate else None, out, self.n_q, self.n_kv,
                                  self.v_dim)
            elif self.gate:
                acc = torch.empty((T, self.n_q * self.v_dim), dtype=torch.float32, device=dev)
                attend(acc)
                kernels.heads_mix(acc, None, proj[:, cols:], out, self.n_q, self.n_kv, self.v_dim)
            else:
                attend(out)
        y = linear(out, self.w_o, out_dtype=torch.float32, parts_ok=True)
        if self.o_bias is None:
            return y
        biased = torch.empty((T, self.hidden), dtype=torch.float32, device=dev)
        kernels.bias_act(y, self.o_bias, "none", biased)
        return biased

    # bfloat16 runs on the tensor cores when the sizes allow; everything else, and
    # all of float32, takes the exact CUDA-core kernel
    def _tensor_cores(self, ctx) -> bool:
        return ctx.dtype == torch.bfloat16 and self.head_dim <= 256 and self.n_q // self.n_kv <= 16

    def attend_packed(self, q, k, v, out, ctx, common):
        if self._tensor_cores(ctx) and kernels.attention_prefill_tc_ok(self.head_dim, self.n_q // self.n_kv):
            kernels.attention_prefill_tc(q, out, ctx.cu_q, k, v, **common)         # tcgen05, scores in tensor memory
        elif self._tensor_cores(ctx):
            kernels.attention_prefill_mma(q, out, ctx.cu_q, k, v, **common)
        else:
            kernels.attention_simt(q, out, ctx.cu_q, ctx.kv_len, k=k, v=v, **common)

    def attend_paged(self, q, out, ctx, common, k_pages, v_pages, table, ring, page):
        if self._tensor_cores(ctx) and ctx.mode == "decode" and page == 64:
            args = {k: v for k, v in common.items() if k != "max_q_len"}
            splits = kernels.decode_splits(ctx.batch, self.n_kv, ctx.max_kv_len, self.window or 0,
                                           ragged=getattr(ctx, "ragged", False))
            kernels.attention_decode_mma(q, out, ctx.cu_q, ctx.kv_len, k_pages, v_pages, table, ring=ring,
                                         page_size=page, n_splits=splits, **args)
        else:
            kernels.attention_simt(q, out, ctx.cu_q, ctx.kv_len, k_pages=k_pages, v_pages=v_pages, page_table=table,
                                   ring=ring, page_size=page, **common)


register_part("mixer", "attention", Attention)
