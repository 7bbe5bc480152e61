"""Norm parts and the residual sum around them."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ParamSpec, Part, register_part


class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * (offset + w).

    Gemma 2 uses offset 1 (wlejon/brolm src/gemma2.cpp:154-175 folds it into
    the gain at load; here the gain stays as stored and the kernel adds it).
    Statistics and the product are float32.

    ``groups`` > 1: the row is cut into that many equal consecutive parts and every part is divided by its own
    root mean square; the gain still spans the whole row.
    """

    kind = "norm"
    graph_safe = True

    def __init__(self, size: int, eps: float, offset: float = 0.0, groups: int = 1):
        if groups < 1 or size % groups:
            raise ValueError(f"norm: {groups} groups do not divide a row of {size}")
        self.size, self.eps, self.offset, self.groups = size, float(eps), float(offset), int(groups)

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), "vector")}

    @property
    def weight(self) -> torch.Tensor:
        return self.params["weight"]

    def apply(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = rows.numel() if rows is not None else x.shape[0]
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        if self.groups > 1:
            kernels.group_rmsnorm(x, self.weight, self.eps, self.offset, self.groups, out, rows)
        else:
            kernels.rmsnorm(x, self.weight, self.eps, self.offset, out, rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)


class Cast(Part):
    """No norm at all: the rows as they are, in the element type asked for.  It stands where an arrangement
    whose sublayers read the residual stream itself needs an entry "norm"; in float32 the stream is handed
    on as it is, without a copy (every sublayer has read its input before the stream takes its result)."""

    kind = "norm"
    graph_safe = True

    def __init__(self, size: int):
        self.size = size

    def apply(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if rows is not None:
            x = x.index_select(0, rows.long())
        if x.dtype == out_dtype:
            return x
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        kernels.cast(x, out)
        return out


register_part("norm", "cast", Cast)


def add_then_norm(h: torch.Tensor, y: torch.Tensor, post: Optional[Part], nxt: Optional[Part],
                  out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """h += post(y) (or y);  return nxt(h) when ``nxt`` is given.

    h is the float32 residual stream and is updated in place.  Two RMSNorms
    run in one kernel with the sum; any other norm part is applied through its
    own ``apply`` and only the sum stays fused.
    """
    fused_post = post is None or isinstance(post, RMSNorm)
    plain_next = isinstance(nxt, Cast)          # no norm ahead of the next block: it wants the stream itself
    fused_next = nxt is None or plain_next or isinstance(nxt, RMSNorm)
    # norms in groups have a fused kernel of their own, which takes one number of groups for both norms
    counts = {n.groups for n in (post, nxt) if isinstance(n, RMSNorm)}
    groups = max(counts) if counts else 1
    if len(counts) > 1:
        fused_next = plain_next or nxt is None
    if fused_post and fused_next and post is not None and nxt is not None and not plain_next \
            and post.weight.dtype != nxt.weight.dtype:
        fused_next = False
    if y.dim() == 3 and not fused_post:
        y = y.sum(dim=0)                       # partial sums, and a norm that wants the whole
    if not fused_post:
        y = post.apply(y, torch.float32)
        post = None
    out = None
    if fused_next and nxt is not None and not (plain_next and out_dtype == torch.float32):
        out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
    normed_next = fused_next and nxt is not None and not plain_next
    args = (h, y,
            post.weight if post is not None else None, post.eps if post is not None else 0.0,
            post.offset if post is not None else 0.0,
            nxt.weight if normed_next else None, nxt.eps if normed_next else 0.0,
            nxt.offset if normed_next else 0.0)
    if groups > 1 and (post is not None or normed_next):
        kernels.residual_group_rmsnorm(*args, post.groups if post is not None else groups, out)
    else:
        kernels.residual_rmsnorm(*args, out)
    if plain_next and out is None:
        return h                               # float32: the stream is handed on as it is
    if nxt is not None and not fused_next:
        out = nxt.apply(h, out_dtype)
    return out
