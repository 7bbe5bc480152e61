"""Python face of the hand-written CUDA kernels.

Every function takes CUDA tensors, checks what the kernel cannot check itself,
and launches on the current torch stream.  There is no CPU path and no
library fallback: a missing build or a CPU tensor raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from .build import KernelBuildError, build_all, library_loaded, load_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {
    10001: "unsupported element type",
    10002: "a size the kernel does not take",
    10003: "a size beyond the kernel's limit",
    10004: "a stride or pointer that is not aligned as the kernel needs",
}
# gated activations: act(gate) * up for the first two; "clamped_gate" is min(g, limit) * sigmoid(1.702 min(g, limit))
# * (clamp(up, -limit, limit) + 1) and takes ``limit`` wherever an activation is named
ACTIVATIONS = {"gelu_tanh": 0, "gelu_pytorch_tanh": 0, "silu": 1, "clamped_gate": 2}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not float32 or bfloat16") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("brolm_b200 kernels run on CUDA tensors only; there is no CPU path")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


B200_SMS = 148
_sms: dict = {}


def device_sms(device=None) -> int:
    """How many SMs the device of the kernels' launches has, asked once per device.  Without a CUDA
    device (the policy functions below are plain arithmetic and are tested on the CPU) the B200's 148."""
    if not torch.cuda.is_available():
        return B200_SMS
    index = torch.device(device).index if device is not None else None
    if index is None:
        index = torch.cuda.current_device()
    n = _sms.get(index)
    if n is None:
        n = _sms[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return n


_launches = 0


def launch_count() -> int:
    """How many of this library's own kernels have been launched by this process."""
    return _launches


def add_launches(n: int) -> None:
    """Count kernels that ran without passing through this module (a replayed CUDA graph)."""
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    if status in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[status]}")
    raise KernelError(f"{what}: CUDA error {status}")


_fn_cache: dict[str, ctypes._CFuncPtr] = {}


def _fn(lib: str, name: str, argtypes: list) -> ctypes._CFuncPtr:
    f = _fn_cache.get(name)
    if f is None:
        f = getattr(load_library(lib), name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[name] = f
    return f


# ---------------------------------------------------------------------------
def embed_scale(ids: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    """out[t] = float(table[ids[t]]) * scale;  ids int32, out float32 (tokens, hidden)."""
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous() and out.is_contiguous()
    f = _fn("core", "brolm_embed_scale", [c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(table), _code(table), scale, _ptr(out), ids.numel(), table.shape[1], _stream()),
           "embed_scale")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * (offset + weight)."""
    assert x.is_contiguous() and out.is_contiguous() and weight.is_contiguous()
    n = out.shape[0]
    hidden = x.shape[-1]
    assert weight.numel() == hidden and out.shape[-1] == hidden
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n
    else:
        assert x.shape[0] == n
    f = _fn("core", "brolm_rmsnorm", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_int,
                                      c_int, c_int, c_void_p])
    _check(f(_ptr(x), _code(x), _ptr(rows), _ptr(weight), _code(weight), eps, offset, _ptr(out), _code(out), n,
             hidden, _stream()), "rmsnorm")


def residual_rmsnorm(h: torch.Tensor, y: torch.Tensor, post_weight: Optional[torch.Tensor], post_eps: float,
                     post_offset: float, next_weight: Optional[torch.Tensor], next_eps: float, next_offset: float,
                     out: Optional[torch.Tensor]) -> None:
    """h += rmsnorm(y; post) (or y when post_weight is None); out = rmsnorm(h; next) when next_weight is given;
    with ``out`` but no ``next_weight``, out = the new h in out's element type.

    ``y`` may be [parts, rows, hidden]: partial sums that are added in order first."""
    assert h.dtype == torch.float32 and h.is_contiguous() and y.is_contiguous() and tuple(y.shape[-2:]) == tuple(h.shape)
    n_parts, part_stride = (y.shape[0], y.stride(0)) if y.dim() == 3 else (1, 0)
    wd = None
    for w in (post_weight, next_weight):
        if w is not None:
            assert w.is_contiguous() and w.numel() == h.shape[-1]
            if wd is not None and w.dtype != wd:
                raise KernelError("residual_rmsnorm: both gains must have one element type")
            wd = w.dtype
    if next_weight is not None:
        assert out is not None
    if out is not None:
        assert out.is_contiguous() and out.shape == h.shape
    f = _fn("core", "brolm_residual_rmsnorm", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_float, c_float,
                                               c_void_p, c_float, c_float, c_int, c_void_p, c_int, c_int, c_int,
                                               c_void_p])
    _check(f(_ptr(h), _ptr(y), _code(y), n_parts, part_stride, _ptr(post_weight), post_eps, post_offset, _ptr(next_weight), next_eps,
             next_offset, _CODES[wd] if wd is not None else F32, _ptr(out) if out is not None else None,
             _code(out) if out is not None else F32, h.shape[0], h.shape[-1], _stream()),
           "residual_rmsnorm")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: Optional[torch.Tensor], n_q: int, n_kv: int,
                  head_dim: int, rotary_dim: int, k_pages: Optional[torch.Tensor] = None,
                  v_pages: Optional[torch.Tensor] = None, cache_rows: Optional[torch.Tensor] = None,
                  page_size: int = 64) -> None:
    """Rotate q and k inside qkv (tokens, (n_q + 2 n_kv) * head_dim) and write k, v into the cache pages.

    ``cache_rows[t]`` = page * page_size + place of token t, negative when the token is not kept."""
    assert qkv.is_contiguous() and qkv.shape[1] == (n_q + 2 * n_kv) * head_dim
    assert positions.dtype == torch.int32 and positions.numel() == qkv.shape[0]
    if k_pages is not None:
        assert v_pages is not None and cache_rows is not None
        assert k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype
        assert k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim), (k_pages.shape, n_kv, page_size, head_dim)
        assert cache_rows.dtype == torch.int32 and cache_rows.numel() == qkv.shape[0]
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1:] == (rotary_dim // 2, 2)
    f = _fn("core", "brolm_rope_kv_write", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                            c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(qkv), _code(qkv), _ptr(positions), _ptr(cos_sin), n_q, n_kv, head_dim, rotary_dim, _ptr(k_pages),
             _ptr(v_pages), _ptr(cache_rows) if k_pages is not None else None, page_size, qkv.shape[0], _stream()),
           "rope_kv_write")


def rope_kv_write_parts(parts: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor,
                        cos_sin: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int,
                        k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                        cache_rows: Optional[torch.Tensor] = None, page_size: int = 64) -> None:
    """``rope_kv_write`` for a q/k/v projection that arrives as float32 partial sums of K slices,
    ``parts`` [slices, tokens, width]: the slices are added in order, q and k rotated over the whole head,
    and the result rounded once to bfloat16 into ``qkv`` (tokens, width) and into the cache pages."""
    width = (n_q + 2 * n_kv) * head_dim
    assert parts.dtype == torch.float32 and parts.dim() == 3 and parts.shape[2] == width and parts.stride(2) == 1
    assert parts.stride(1) == width and qkv.dtype == torch.bfloat16 and qkv.shape == (parts.shape[1], width)
    assert qkv.stride(1) == 1 and head_dim % 16 == 0
    assert positions.dtype == torch.int32 and positions.numel() == qkv.shape[0]
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1:] == (head_dim // 2, 2)
    if k_pages is not None:
        assert v_pages is not None and cache_rows is not None and k_pages.dtype == torch.bfloat16
        assert k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim)
        assert cache_rows.dtype == torch.int32 and cache_rows.numel() == qkv.shape[0]
    f = _fn("core", "brolm_rope_kv_write_parts", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                                  c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(parts), parts.shape[0], parts.stride(0), _ptr(qkv), qkv.stride(0), _ptr(positions), _ptr(cos_sin),
             n_q, n_kv, head_dim, _ptr(k_pages), _ptr(v_pages), _ptr(cache_rows) if k_pages is not None else None,
             page_size, qkv.shape[0], _stream()), "rope_kv_write_parts")


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, activation: str, limit: float = 0.0) -> None:
    """out = act(gate) * up for gate_up = [gate | up] (tokens, 2 * inter); ``limit`` for "clamped_gate"."""
    assert gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype
    assert gate_up.shape[1] == 2 * out.shape[1] and gate_up.shape[0] == out.shape[0]
    if activation not in ACTIVATIONS:
        raise KernelError(f"gated_act: unknown activation '{activation}' (known: {sorted(ACTIVATIONS)})")
    f = _fn("core", "brolm_gated_act", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), _code(out), out.shape[0], out.shape[1], ACTIVATIONS[activation], limit, _stream()),
           "gated_act")


def softcap(x: torch.Tensor, out: torch.Tensor, cap: float) -> None:
    """out (float32) = cap * tanh(x / cap); cap <= 0 only converts."""
    assert x.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32 and x.numel() == out.numel()
    f = _fn("core", "brolm_softcap", [c_void_p, c_int, c_void_p, c_longlong, c_float, c_void_p])
    _check(f(_ptr(x), _code(x), _ptr(out), x.numel(), cap, _stream()), "softcap")


def embed_pairs(ids: torch.Tensor, positions: torch.Tensor, tok_seq: torch.Tensor, cu_q: torch.Tensor,
                slots: torch.Tensor, last_token: torch.Tensor, table: torch.Tensor, pairs: torch.Tensor, scale: float,
                mul_prev: int, mul_cur: int, buckets: int, out: torch.Tensor) -> None:
    """out[t] = table[ids[t]] * scale + pairs[(prev * mul_prev + ids[t] * mul_cur) % buckets], prev being the
    token before ids[t] in its sequence (this step's, or ``last_token[slot]`` from the step before); a
    sequence's first token takes row ``buckets``.  Leaves each sequence's last token in ``last_token``."""
    for t in (ids, positions, tok_seq, cu_q, slots, last_token):
        assert t.dtype == torch.int32 and t.is_contiguous()
    assert out.dtype == torch.float32 and table.is_contiguous() and pairs.is_contiguous() and out.is_contiguous()
    assert table.dtype == pairs.dtype and pairs.shape == (buckets + 1, table.shape[1])
    assert positions.numel() == ids.numel() and tok_seq.numel() == ids.numel()
    f = _fn("core", "brolm_embed_pairs", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int, c_float, c_longlong, c_longlong, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(ids), _ptr(positions), _ptr(tok_seq), _ptr(cu_q), _ptr(slots), _ptr(last_token), _ptr(table),
             _ptr(pairs), _code(table), scale, mul_prev, mul_cur, buckets, _ptr(out), ids.numel(), table.shape[1],
             _stream()), "embed_pairs")


def concat_cast(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [a[t] | b[t]] in out's element type; a and b float32 (tokens, hidden)."""
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and a.shape == b.shape
    assert a.is_contiguous() and b.is_contiguous() and out.is_contiguous() and out.shape == (a.shape[0], 2 * a.shape[1])
    f = _fn("core", "brolm_concat_cast", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(a), _ptr(b), _ptr(out), _code(out), a.shape[0], a.shape[1], _stream()), "concat_cast")


def latent_rows(proj: torch.Tensor, q_cols: int, positions: torch.Tensor, cos_sin: Optional[torch.Tensor], rotary_dim: int,
                gain: torch.Tensor, eps: float, heads: int, dn: int, dr: int, rank: int, lat: torch.Tensor,
                qlat: torch.Tensor, pages: Optional[torch.Tensor] = None,
                cache_rows: Optional[torch.Tensor] = None) -> None:
    """The row-wise step of latent attention.  ``proj`` (tokens, q_cols + rank + dr): per head [dn | dr] queries,
    then the compressed row [rank | dr].  Writes ``lat`` (tokens, Dp) = [rmsnorm(compressed) * gain | rotated key
    part | zeros], the same row into ``pages`` at ``cache_rows`` (negative: not kept), and the rotated query
    parts into columns rank .. of every head of ``qlat`` (tokens, heads * Dp)."""
    Dp = lat.shape[1]
    assert proj.stride(1) == 1 and proj.shape[1] >= q_cols + rank + dr and q_cols == heads * (dn + dr)
    assert lat.dtype == proj.dtype and qlat.dtype == proj.dtype and gain.dtype == proj.dtype
    assert lat.is_contiguous() and qlat.is_contiguous() and qlat.shape == (proj.shape[0], heads * Dp)
    assert gain.is_contiguous() and gain.numel() == rank
    assert positions.dtype == torch.int32 and positions.numel() == proj.shape[0]
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1:] == (rotary_dim // 2, 2)
    if pages is not None:
        assert pages.dtype == proj.dtype and pages.is_contiguous() and pages.shape[-1] == Dp
        assert cache_rows is not None and cache_rows.dtype == torch.int32 and cache_rows.numel() == proj.shape[0]
    f = _fn("latent", "brolm_latent_rows", [c_int, c_void_p, c_long, c_int, c_void_p, c_void_p, c_int, c_void_p, c_float,
                                            c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_int, c_void_p])
    _check(f(_code(proj), _ptr(proj), proj.stride(0), q_cols, _ptr(positions), _ptr(cos_sin),
             rotary_dim if cos_sin is not None else 0, _ptr(gain), eps, heads, dn, dr, rank, Dp, _ptr(lat), _ptr(qlat),
             _ptr(pages), _ptr(cache_rows) if pages is not None else None, proj.shape[0], _stream()), "latent_rows")


ROUTE_MODES = {"logistic": 0, "softmax": 1}


def _check_route(mode: str, correction: Optional[torch.Tensor], experts: int) -> None:
    if mode not in ROUTE_MODES:
        raise KernelError(f"router: unknown mode '{mode}' (known: {sorted(ROUTE_MODES)})")
    if correction is not None:
        assert mode == "softmax" and correction.dtype == torch.float32 and correction.is_contiguous()
        assert correction.numel() == experts


def _route_opts(mode: str, experts: int, top: int, groups: int, keep: int, renorm: bool, scale: float) -> tuple:
    if (groups, keep, renorm, scale) != (1, 1, True, 1.0) and mode != "softmax":
        raise KernelError("router: groups, unnormalised weights and a scale go with the softmax mode")
    if groups < 1 or not 1 <= keep <= groups or experts % groups or top > keep * (experts // groups):
        raise KernelError(f"router: {experts} experts in {groups} groups of which {keep} stay open cannot give {top} choices")
    return int(groups), int(keep), 1 if renorm else 0, float(scale)


def route_topk(x: torch.Tensor, router: torch.Tensor, top: int, ids: torch.Tensor, weights: torch.Tensor,
               mode: str = "logistic", correction: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 1,
               renorm: bool = True, scale: float = 1.0) -> None:
    """ids, weights [tokens, top]: the ``top`` experts with the largest score, best first (ties: the lower index).
    ``mode`` "logistic": the score is z = router.x (float32 sums) and the weight its logistic function.
    ``mode`` "softmax": s = softmax(z) over all experts, the choice goes by s + ``correction`` (float32 [experts],
    no part of the weights) and the weights are the chosen s over their sum (+ 1e-20).  In that mode the experts may
    form ``groups`` equal groups of neighbours, of which only the ``keep`` with the largest best score stay open to
    the choice; ``renorm`` False leaves the chosen s undivided; ``scale`` multiplies the weights."""
    assert x.dtype == router.dtype and x.stride(1) == 1 and router.is_contiguous() and router.shape[1] == x.shape[1]
    assert ids.dtype == torch.int32 and weights.dtype == torch.float32 and ids.is_contiguous() and weights.is_contiguous()
    assert ids.shape == (x.shape[0], top) and weights.shape == ids.shape
    _check_route(mode, correction, router.shape[0])
    opts = _route_opts(mode, router.shape[0], top, groups, keep, renorm, scale)
    f = _fn("grouped", "brolm_route_topk", [c_int, c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                            c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_code(x), _ptr(x), x.stride(0), _ptr(router), x.shape[0], router.shape[0], x.shape[1], top, _ptr(ids),
             _ptr(weights), ROUTE_MODES[mode], _ptr(correction), *opts, _stream()), "route_topk")


def route_pick(z: torch.Tensor, top: int, ids: torch.Tensor, weights: torch.Tensor, mode: str = "logistic",
               correction: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 1, renorm: bool = True,
               scale: float = 1.0) -> None:
    """The choice of ``route_topk`` from scores z [tokens, experts] float32 that a matrix product left in memory."""
    assert z.dtype == torch.float32 and z.dim() == 2 and z.stride(1) == 1 and z.shape[1] <= 1024
    assert ids.dtype == torch.int32 and weights.dtype == torch.float32 and ids.is_contiguous() and weights.is_contiguous()
    assert ids.shape == (z.shape[0], top) and weights.shape == ids.shape
    _check_route(mode, correction, z.shape[1])
    opts = _route_opts(mode, z.shape[1], top, groups, keep, renorm, scale)
    f = _fn("grouped", "brolm_route_pick", [c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                            c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(z), z.stride(0), z.shape[0], z.shape[1], top, _ptr(ids), _ptr(weights), ROUTE_MODES[mode],
             _ptr(correction), *opts, _stream()), "route_pick")


GROUP_ROWS = 64          # rows of a tile of the grouped product
GROUP_ROWS_TC = 128      # ... of the tcgen05 grouped product


def group_tiles(pairs: int, experts: int, rows: int = GROUP_ROWS) -> int:
    """Room the tile list of ``group_pairs`` needs: every expert may end with a tile that is not full."""
    return (pairs + rows - 1) // rows + experts


def group_pairs(ids: torch.Tensor, experts: int, perm: torch.Tensor, offsets: torch.Tensor, tiles: torch.Tensor,
                rows: int = GROUP_ROWS) -> None:
    """Sort the (token, choice) pairs of ``ids`` [tokens, top] by expert, on the device: ``perm`` [pairs] the
    pairs in expert order, ``offsets`` [experts + 1] each expert's first row, ``tiles`` [2, group_tiles]
    (expert, first row) of every tile of ``rows`` rows, expert -1 beyond the last."""
    pairs = ids.numel()
    for t in (ids, perm, offsets, tiles):
        assert t.dtype == torch.int32 and t.is_contiguous()
    assert rows in (GROUP_ROWS, GROUP_ROWS_TC)
    assert perm.numel() == pairs and offsets.numel() == experts + 1
    assert tiles.shape == (2, group_tiles(pairs, experts, rows))
    f = _fn("grouped", "brolm_group_pairs", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                             c_int, c_void_p])
    _check(f(_ptr(ids), pairs, experts, _ptr(perm), _ptr(offsets), _ptr(tiles[0]), _ptr(tiles[1]), tiles.shape[1],
             rows, _stream()), "group_pairs")


# From how many pairs per expert on the experts' products run on tcgen05 (128-row tiles): below it most of
# a tile would be rows that are dropped, and the mma.sync kernel with its 64-row tiles is ahead.
EXPERTS_TC_ROWS = int(os.environ.get("BROLM_EXPERTS_TC_ROWS", "64"))


def experts_tc_ok(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, pairs: int) -> bool:
    """Whether the two products of routed experts over ``pairs`` (token, choice) pairs go to the tcgen05
    grouped kernel: bfloat16 on the device, enough rows per expert, sizes a TMA box takes."""
    E, F, W = w_up.shape
    return (x.is_cuda and x.dtype == torch.bfloat16 and w_up.dtype == torch.bfloat16 and W % 8 == 0 and F % 8 == 0
            and w_down.shape[2] % 8 == 0       # (gated experts: the second product's rows are half as wide as F)
            and x.stride(0) % 8 == 0 and pairs >= max(GROUP_ROWS_TC, EXPERTS_TC_ROWS * E))


def gather_rows(x: torch.Tensor, perm: torch.Tensor, top: int, out: torch.Tensor) -> None:
    """out[s, :] = x[perm[s] // top, :]: the tokens' rows in the order of their sorted pairs (bfloat16)."""
    assert x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and x.stride(1) == 1 and out.is_contiguous()
    assert perm.dtype == torch.int32 and out.shape == (perm.numel(), x.shape[1])
    f = _fn("grouped_tc", "brolm_gather_rows", [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(perm), top, perm.numel(), x.shape[1], _ptr(out), _stream()), "gather_rows")


def experts_linear_tc(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, perm: torch.Tensor,
                      offsets: torch.Tensor, tiles: torch.Tensor, top: int, tokens: int,
                      scale: Optional[torch.Tensor] = None, activation: str = "none", down: bool = False) -> None:
    """``experts_linear`` on tcgen05, for rows already in expert order: a (pairs, K); ``tiles`` the list of
    128-row tiles.  First product: out (pairs, N) = act(scale[pair] * (W[e] a[row])), the gate applied to the
    float sums; second: out float32 [top, tokens, N]."""
    E, N, K = weight.shape
    pairs = perm.numel()
    assert a.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.is_contiguous()
    assert a.stride(1) == 1 and out.is_contiguous() and a.shape == (pairs, K) and pairs == top * tokens
    assert tiles.shape == (2, group_tiles(pairs, E, GROUP_ROWS_TC))
    if down:
        assert out.dtype == torch.float32 and tuple(out.shape) == (top, tokens, N)
    else:
        assert scale is None or (scale.dtype == torch.float32 and scale.numel() == pairs and scale.is_contiguous())
        assert tuple(out.shape) == (pairs, N) and out.dtype in (torch.float32, torch.bfloat16)
    if activation not in EXPERT_ACTS:
        raise KernelError(f"experts_linear_tc: unknown activation '{activation}' (known: {sorted(EXPERT_ACTS)})")
    f = _fn("grouped_tc", "brolm_experts_linear_tc", [c_int, c_void_p, c_long, c_long, c_void_p, c_int, c_void_p, c_long,
                                                      c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                      c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(1 if down else 0, _ptr(a), a.stride(0), pairs, _ptr(weight), E, _ptr(out), N,
             1 if out.dtype == torch.float32 else 0, EXPERT_ACTS[activation], N, K, _ptr(tiles[0]), _ptr(tiles[1]),
             _ptr(offsets), _ptr(perm), _ptr(scale) if scale is not None else None, top, tokens, tiles.shape[1],
             _stream()), "experts_linear_tc")


def grouped_tc_status(reset: bool = False) -> int:
    """0 if no bounded wait inside the tcgen05 grouped product ever ran out; otherwise its code.  Synchronises."""
    if not library_loaded("grouped_tc"):
        return 0
    f = load_library("grouped_tc").brolm_grouped_tc_status
    f.argtypes = [c_int]
    f.restype = c_int
    return f(1 if reset else 0)


def heads_linear(a: torch.Tensor, a_head: int, weight: torch.Tensor, out: torch.Tensor, o_head: int) -> None:
    """A product per head: out[t, h * o_head + n] = sum_k weight[h, n, k] * a[t, h * a_head + k].
    ``weight`` [heads, N, K]; a and out are packed rows whose heads lie ``a_head`` / ``o_head`` apart (a head's
    slice may be wider than K or N).  float32 everywhere, or bfloat16 operands with a bfloat16 or float32 result."""
    H, N, K = weight.shape
    assert a.dtype == weight.dtype and weight.is_contiguous() and a.stride(1) == 1 and out.stride(1) == 1
    assert a.shape[0] == out.shape[0] and K <= a_head and N <= o_head
    assert (H - 1) * a_head + K <= a.shape[1] and (H - 1) * o_head + N <= out.shape[1]
    assert out.dtype in (torch.float32, a.dtype)
    f = _fn("grouped", "brolm_heads_linear", [c_int, c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p, c_long,
                                              c_long, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_code(a), _ptr(a), a.stride(0), a_head, _ptr(weight), K, N * K, _ptr(out), out.stride(0), o_head,
             1 if out.dtype == torch.float32 else 0, a.shape[0], H, N, K, _stream()), "heads_linear")


EXPERT_ACTS = {"none": 0, "relu2": 1}


def experts_linear(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, perm: torch.Tensor, offsets: torch.Tensor,
                   tiles: torch.Tensor, top: int, tokens: int, scale: Optional[torch.Tensor] = None,
                   activation: str = "none", down: bool = False) -> None:
    """One of the two products of routed experts over the pairs that ``group_pairs`` sorted.  ``weight``
    [experts, N, K].  First product (``down`` False): a (tokens, K) the tokens' rows, each pair's row multiplied
    by ``scale[pair]`` and rounded to the operands' type; out (pairs, N) in expert order, with the activation.
    Second (``down`` True): a (pairs, K) in expert order; out float32 [top, tokens, N], a pair's result at
    [its choice, its token]."""
    E, N, K = weight.shape
    pairs = perm.numel()
    assert a.dtype == weight.dtype and weight.is_contiguous() and a.stride(1) == 1 and out.is_contiguous()
    assert a.shape[1] == K and pairs == top * tokens
    if down:
        assert out.dtype == torch.float32 and tuple(out.shape) == (top, tokens, N) and a.shape[0] == pairs
    else:
        assert scale is None or (scale.dtype == torch.float32 and scale.numel() == pairs and scale.is_contiguous())
        assert tuple(out.shape) == (pairs, N) and a.shape[0] == tokens and out.dtype in (torch.float32, a.dtype)
    if activation not in EXPERT_ACTS:
        raise KernelError(f"experts_linear: unknown activation '{activation}' (known: {sorted(EXPERT_ACTS)})")
    f = _fn("grouped", "brolm_experts_linear", [c_int, c_int, c_void_p, c_long, c_void_p, c_long, c_long, c_int, c_void_p, c_long,
                                                c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_code(a), 1 if down else 0, _ptr(a), a.stride(0), _ptr(weight), K, N * K, E, _ptr(out), N,
             1 if out.dtype == torch.float32 else 0, EXPERT_ACTS[activation], N, K, _ptr(tiles[0]), _ptr(tiles[1]),
             _ptr(offsets), _ptr(perm), _ptr(scale), top, tokens, tiles.shape[1], _stream()), "experts_linear")


# --- row-wise steps (csrc/rowwise.cu) ---------------------------------------
ROW_ACTS = {"none": 0, "relu2": 1, "gelu_tanh": 2, "silu": 3}


def cast(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x in out's element type (float32 or bfloat16)."""
    assert x.is_contiguous() and out.is_contiguous() and x.numel() == out.numel()
    f = _fn("rowwise", "brolm_cast", [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_ptr(x), _code(x), _ptr(out), _code(out), x.numel(), _stream()), "cast")


def bias_act(y: torch.Tensor, bias: Optional[torch.Tensor], activation: str, out: torch.Tensor) -> None:
    """out (rows, cols) = act(y + bias); y may be [parts, rows, cols] partial sums, which are added in order first."""
    if activation not in ROW_ACTS:
        raise KernelError(f"bias_act: unknown activation '{activation}' (known: {sorted(ROW_ACTS)})")
    n_parts, part_stride = (y.shape[0], y.stride(0)) if y.dim() == 3 else (1, 0)
    rows, cols = out.shape
    assert tuple(y.shape[-2:]) == (rows, cols) and y.stride(-1) == 1 and out.stride(1) == 1
    if bias is not None:
        assert bias.is_contiguous() and bias.numel() == cols
    f = _fn("rowwise", "brolm_bias_act", [c_void_p, c_int, c_int, c_longlong, c_long, c_void_p, c_int, c_int, c_void_p, c_int,
                                          c_long, c_int, c_int, c_void_p])
    _check(f(_ptr(y), _code(y), n_parts, part_stride, y.stride(-2), _ptr(bias), _code(bias) if bias is not None else F32,
             ROW_ACTS[activation], _ptr(out), _code(out), out.stride(0), rows, cols, _stream()), "bias_act")


def scaled_sum(a: torch.Tensor, sa: float, b: torch.Tensor, sb: float, out: torch.Tensor) -> None:
    """out = sa * a + sb * b, float32; a and b may each be [parts, rows, cols] partial sums."""
    for t in (a, b):
        assert t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape[-2:]) == tuple(out.shape)
    assert out.dtype == torch.float32 and out.is_contiguous()
    ap, astr = (a.shape[0], a.stride(0)) if a.dim() == 3 else (1, 0)
    bp, bstr = (b.shape[0], b.stride(0)) if b.dim() == 3 else (1, 0)
    f = _fn("rowwise", "brolm_scaled_sum", [c_void_p, c_int, c_longlong, c_float, c_void_p, c_int, c_longlong, c_float,
                                            c_void_p, c_longlong, c_void_p])
    _check(f(_ptr(a), ap, astr, sa, _ptr(b), bp, bstr, sb, _ptr(out), out.numel(), _stream()), "scaled_sum")


def qkv_norm_write(proj: torch.Tensor, q_cols: int, k_cols: int, v_cols: int, q_gain: Optional[torch.Tensor],
                   k_gain: Optional[torch.Tensor], eps: float, positions: torch.Tensor, out: torch.Tensor, n_kv: int,
                   k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                   cache_rows: Optional[torch.Tensor] = None, page_size: int = 64) -> None:
    """proj (tokens, q_cols + k_cols + v_cols) -> out of the same layout in out's element type, the whole query
    row and the whole key row each RMS-normed over all of their heads at once when gains are given, and keys and
    values written into the cache pages (k rows of k_cols / n_kv, value rows of v_cols / n_kv)."""
    assert proj.stride(1) == 1 and out.stride(1) == 1 and proj.shape == out.shape
    assert proj.shape[1] == q_cols + k_cols + v_cols
    assert positions.dtype == torch.int32 and positions.numel() == proj.shape[0]
    whole = q_gain is not None
    if whole:
        assert k_gain is not None and q_gain.dtype == k_gain.dtype and q_gain.numel() == q_cols and k_gain.numel() == k_cols
        assert q_gain.is_contiguous() and k_gain.is_contiguous()
    if k_pages is not None:
        assert v_pages is not None and cache_rows is not None and k_pages.dtype == out.dtype and v_pages.dtype == out.dtype
        assert k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (n_kv, page_size, k_cols // n_kv)
        assert tuple(v_pages.shape[1:]) == (n_kv, page_size, v_cols // n_kv)
        assert cache_rows.dtype == torch.int32 and cache_rows.numel() == proj.shape[0]
    f = _fn("rowwise", "brolm_qkv_norm_write", [c_void_p, c_int, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                                c_float, c_int, c_void_p, c_void_p, c_int, c_long, c_void_p, c_void_p,
                                                c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(proj), _code(proj), proj.stride(0), q_cols, k_cols, v_cols, _ptr(q_gain), _ptr(k_gain),
             _code(q_gain) if whole else F32, eps, 1 if whole else 0, _ptr(positions), _ptr(out), _code(out), out.stride(0),
             _ptr(k_pages), _ptr(v_pages), _ptr(cache_rows) if k_pages is not None else None, n_kv, page_size,
             proj.shape[0], _stream()), "qkv_norm_write")


ROPE_PAIRINGS = {"half": 0, "interleaved": 1}


def qkv_finish(proj: torch.Tensor, bias: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int, v_dim: int,
               positions: torch.Tensor, out: torch.Tensor, *, head_norm: bool = False, eps: float = 0.0,
               cos_sin: Optional[torch.Tensor] = None, rotary_dim: int = 0, pairing: str = "half",
               mix: Optional[torch.Tensor] = None, v_first: Optional[torch.Tensor] = None,
               v_keep: Optional[torch.Tensor] = None, k_pages: Optional[torch.Tensor] = None,
               v_pages: Optional[torch.Tensor] = None, cache_rows: Optional[torch.Tensor] = None,
               page_size: int = 64, q_gain: Optional[torch.Tensor] = None, k_gain: Optional[torch.Tensor] = None) -> None:
    """A projection's rows [q: n_q * head_dim | k: n_kv * head_dim | v: n_kv * v_dim] made ready for attention:
    ``proj`` (tokens, cols) or float32 partial sums [parts, tokens, cols] plus ``bias`` (float32 [cols]); every q
    and k head divided by its root mean square (``head_norm``; times ``q_gain`` / ``k_gain`` when given); the first ``rotary_dim`` elements of
    every q and k head rotated with ``cos_sin`` [positions, rotary_dim / 2, 2], pairs (i, i + rotary_dim / 2)
    ("half") or (2i, 2i + 1) ("interleaved"); v <- (1 - mix) v + mix v_first with ``mix`` a float32 scalar on
    the device and ``v_first`` float32 (tokens, n_kv * v_dim); ``v_keep`` (float32, contiguous) takes this layer's
    own values as they are before the mixing; the result in ``out``'s element type into ``out`` and the cache."""
    cols = (n_q + n_kv) * head_dim + n_kv * v_dim
    parts, part_stride = (proj.shape[0], proj.stride(0)) if proj.dim() == 3 else (1, 0)
    assert proj.shape[-1] == cols and proj.stride(-1) == 1 and out.stride(1) == 1 and out.shape == (proj.shape[-2], cols)
    assert parts == 1 or proj.dtype == torch.float32
    assert positions.dtype == torch.int32 and positions.numel() == out.shape[0]
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == cols)
    if pairing not in ROPE_PAIRINGS:
        raise KernelError(f"qkv_finish: unknown pairing '{pairing}' (known: {sorted(ROPE_PAIRINGS)})")
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1:] == (rotary_dim // 2, 2)
        assert 0 < rotary_dim <= head_dim and rotary_dim % 2 == 0
    ld_first = 0
    if v_first is not None:
        assert mix is not None and mix.dtype == torch.float32 and mix.numel() == 1
        assert v_first.dtype == torch.float32 and v_first.stride(1) == 1 and v_first.shape == (out.shape[0], n_kv * v_dim)
        ld_first = v_first.stride(0)
    if v_keep is not None:
        assert v_keep.dtype == torch.float32 and v_keep.is_contiguous() and v_keep.shape == (out.shape[0], n_kv * v_dim)
    for gain in (q_gain, k_gain):              # float32 [head_dim]: multiplies every normed head of its kind
        assert gain is None or (head_norm and gain.dtype == torch.float32 and gain.is_contiguous() and gain.numel() == head_dim)
    if k_pages is not None:
        assert v_pages is not None and cache_rows is not None and k_pages.dtype == out.dtype and v_pages.dtype == out.dtype
        assert k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim)
        assert tuple(v_pages.shape[1:]) == (n_kv, page_size, v_dim)
        assert cache_rows.dtype == torch.int32 and cache_rows.numel() == out.shape[0]
    f = _fn("headwise", "brolm_qkv_finish", [c_void_p, c_int, c_int, c_longlong, c_long, c_void_p, c_int, c_int, c_int,
                                             c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                             c_long, c_void_p, c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p,
                                             c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(proj), _code(proj), parts, part_stride, proj.stride(-2), _ptr(bias), n_q, n_kv, head_dim, v_dim,
             1 if head_norm else 0, eps, _ptr(positions), _ptr(cos_sin), rotary_dim, ROPE_PAIRINGS[pairing],
             _ptr(mix) if v_first is not None else None, _ptr(v_first), ld_first, _ptr(v_keep), _ptr(out), _code(out),
             out.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(cache_rows) if k_pages is not None else None, page_size,
             out.shape[0], _ptr(q_gain), _ptr(k_gain), _stream()), "qkv_finish")


def heads_mix(acc: torch.Tensor, talk: Optional[torch.Tensor], gate: Optional[torch.Tensor], out: torch.Tensor,
              heads: int, n_kv: int, v_dim: int) -> None:
    """out[t, h] = sigmoid(gate[t, h]) * sum_g talk[h, g] * acc[t, g, kv head of h]: ``acc`` float32
    (tokens, heads * n_kv * v_dim) holds every head's weights applied to the values of every kv head, ``talk``
    float32 [heads, heads] mixes the heads' weights, ``gate`` float32 (tokens, heads) logits or None.
    Without ``talk`` acc is (tokens, heads * v_dim), every head's own result, and only the gate is applied."""
    assert acc.dtype == torch.float32 and acc.stride(1) == 1
    assert acc.shape[1] == heads * v_dim * (n_kv if talk is not None else 1)
    assert talk is None or (talk.dtype == torch.float32 and talk.is_contiguous() and talk.shape == (heads, heads))
    assert out.stride(1) == 1 and out.shape == (acc.shape[0], heads * v_dim)
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == (acc.shape[0], heads)
    f = _fn("headwise", "brolm_heads_mix", [c_void_p, c_long, c_void_p, c_void_p, c_long, c_void_p, c_int, c_long, c_int,
                                            c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(acc), acc.stride(0), _ptr(talk), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out),
             _code(out), out.stride(0), heads, n_kv, v_dim, acc.shape[0], _stream()), "heads_mix")


def group_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float, groups: int, out: torch.Tensor,
                  rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[rows[r] or r], every one of ``groups`` equal consecutive parts of the row divided by its own
    sqrt(mean(part^2) + eps), the whole times (offset + weight)."""
    assert x.is_contiguous() and out.is_contiguous() and weight.is_contiguous()
    n, hidden = out.shape[0], x.shape[-1]
    assert weight.numel() == hidden and out.shape[-1] == hidden and hidden % groups == 0
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n
    else:
        assert x.shape[0] == n
    f = _fn("groupnorm", "brolm_group_rmsnorm", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p,
                                                 c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _code(x), _ptr(rows), _ptr(weight), _code(weight), eps, offset, _ptr(out), _code(out), n, hidden,
             groups, _stream()), "group_rmsnorm")


def residual_group_rmsnorm(h: torch.Tensor, y: torch.Tensor, post_weight: Optional[torch.Tensor], post_eps: float,
                           post_offset: float, next_weight: Optional[torch.Tensor], next_eps: float, next_offset: float,
                           groups: int, out: Optional[torch.Tensor]) -> None:
    """``residual_rmsnorm`` with both norms taken in ``groups`` equal consecutive parts of the row."""
    assert h.dtype == torch.float32 and h.is_contiguous() and y.is_contiguous() and tuple(y.shape[-2:]) == tuple(h.shape)
    n_parts, part_stride = (y.shape[0], y.stride(0)) if y.dim() == 3 else (1, 0)
    wd = None
    for w in (post_weight, next_weight):
        if w is not None:
            assert w.is_contiguous() and w.numel() == h.shape[-1]
            if wd is not None and w.dtype != wd:
                raise KernelError("residual_group_rmsnorm: both gains must have one element type")
            wd = w.dtype
    if next_weight is not None:
        assert out is not None
    if out is not None:
        assert out.is_contiguous() and out.shape == h.shape
    f = _fn("groupnorm", "brolm_residual_group_rmsnorm", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_float,
                                                          c_float, c_void_p, c_float, c_float, c_int, c_void_p, c_int,
                                                          c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(y), _code(y), n_parts, part_stride, _ptr(post_weight), post_eps, post_offset,
             _ptr(next_weight), next_eps, next_offset, _CODES[wd] if wd is not None else F32,
             _ptr(out) if out is not None else None, _code(out) if out is not None else F32, h.shape[0], h.shape[-1],
             groups, _stream()), "residual_group_rmsnorm")


def gate_group_norm(y: torch.Tensor, z: torch.Tensor, gain: torch.Tensor, eps: float, groups: int,
                    out: torch.Tensor) -> None:
    """out = rmsnorm over each of ``groups`` equal parts of (y * silu(z)), times gain.  y float32 (tokens, n);
    z (tokens, n) may be a strided view."""
    n = y.shape[1]
    assert y.dtype == torch.float32 and y.stride(1) == 1 and z.stride(1) == 1 and out.stride(1) == 1
    assert z.shape == y.shape and out.shape == y.shape and n % groups == 0 and gain.is_contiguous() and gain.numel() == n
    f = _fn("rowwise", "brolm_gate_group_norm", [c_void_p, c_long, c_void_p, c_int, c_long, c_void_p, c_int, c_float, c_int,
                                                 c_int, c_void_p, c_int, c_long, c_int, c_void_p])
    _check(f(_ptr(y), y.stride(0), _ptr(z), _code(z), z.stride(0), _ptr(gain), _code(gain), eps, groups, n // groups,
             _ptr(out), _code(out), out.stride(0), y.shape[0], _stream()), "gate_group_norm")


def experts_combine(y: Optional[torch.Tensor], ids: torch.Tensor, weights: torch.Tensor, n_real: int, x: torch.Tensor,
                    shared: Optional[torch.Tensor], out: torch.Tensor, shared_gate: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum over t's choices c of weights[t, c] * (y[c, t] if ids[t, c] < n_real else x[t]) + shared[t].
    y float32 [top, tokens, hidden] (None when there is no real expert); shared float32 (tokens, hidden) or
    [parts, tokens, hidden], or None.  ``shared_gate`` (hidden numbers of x's type): the shared result is multiplied
    by sigmoid(shared_gate . x[t]), one number per token."""
    tokens, top = ids.shape
    hidden = out.shape[1]
    assert ids.dtype == torch.int32 and weights.dtype == torch.float32 and ids.is_contiguous() and weights.is_contiguous()
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape[0] == tokens and x.stride(1) == 1
    if y is not None:
        assert y.dtype == torch.float32 and y.is_contiguous() and tuple(y.shape) == (top, tokens, hidden)
    else:
        assert n_real == 0
    sp, sstr = 0, 0
    if shared is not None:
        assert shared.dtype == torch.float32 and shared.is_contiguous() and tuple(shared.shape[-2:]) == (tokens, hidden)
        sp, sstr = (shared.shape[0], shared.stride(0)) if shared.dim() == 3 else (1, 0)
    if shared_gate is not None:
        assert shared_gate.dtype == x.dtype and shared_gate.is_contiguous() and shared_gate.numel() == hidden
        assert x.shape[1] == hidden
    f = _fn("rowwise", "brolm_experts_combine", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_long,
                                                 c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(y), _ptr(ids), _ptr(weights), top, n_real, _ptr(x), _code(x), x.stride(0), _ptr(shared), sp, sstr,
             _ptr(out), tokens, hidden, _ptr(shared_gate), _stream()), "experts_combine")


def norm_sigmoid_gate(y: torch.Tensor, z: torch.Tensor, gain: Optional[torch.Tensor], eps: float, out: torch.Tensor) -> None:
    """out = n(y) * sigmoid(z) row by row: n(y) = y * rsqrt(mean(y^2) + eps) * gain over the whole row, or y itself
    when ``gain`` is None.  y, z (tokens, cols), possibly strided views; float arithmetic."""
    tokens, cols = y.shape
    assert z.shape == y.shape and out.shape == y.shape and y.stride(1) == 1 and z.stride(1) == 1 and out.stride(1) == 1
    assert gain is None or (gain.is_contiguous() and gain.numel() == cols)
    f = _fn("rowwise", "brolm_norm_sigmoid_gate", [c_void_p, c_int, c_long, c_void_p, c_int, c_long, c_void_p, c_int, c_float,
                                                   c_int, c_void_p, c_int, c_long, c_int, c_void_p])
    _check(f(_ptr(y), _code(y), y.stride(0), _ptr(z), _code(z), z.stride(0), _ptr(gain), _code(gain) if gain is not None else F32,
             eps, cols, _ptr(out), _code(out), out.stride(0), tokens, _stream()), "norm_sigmoid_gate")


# --- mixers with a state (csrc/recurrent.cu) --------------------------------
CONV_ACTS = {"none": 0, "silu": 1}


def _seq(ctx_cu_q, kv_len, slots, state):
    assert ctx_cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32 and slots.dtype == torch.int32
    assert state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
    return _ptr(ctx_cu_q), _ptr(kv_len), _ptr(slots), _ptr(state), state.stride(0)


def causal_conv(x: torch.Tensor, in_bias: Optional[torch.Tensor], taps: torch.Tensor, bias: Optional[torch.Tensor],
                activation: str, tok_seq: torch.Tensor, positions: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                slots: torch.Tensor, state: torch.Tensor, tail_off: int, out: torch.Tensor) -> None:
    """out (tokens, C) float32 = act(causal convolution per channel of (x + in_bias) + bias).  ``taps`` float32
    (C, K), column K - 1 weighs the token itself.  Inputs before the step come from the K - 1 rows that
    ``state[slot, tail_off:]`` keeps as [K - 1, C] (zeros before a sequence's start); ``conv_tail`` moves them on."""
    C, K = taps.shape
    assert x.stride(1) == 1 and x.shape[1] == C and out.dtype == torch.float32 and out.stride(1) == 1
    assert tuple(out.shape) == (x.shape[0], C) and taps.dtype == torch.float32 and taps.is_contiguous()
    for v in (in_bias, bias):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == C)
    assert tok_seq.dtype == torch.int32 and positions.dtype == torch.int32 and positions.numel() == x.shape[0]
    assert tail_off + (K - 1) * C <= state.shape[1]
    if activation not in CONV_ACTS:
        raise KernelError(f"causal_conv: unknown activation '{activation}'")
    f = _fn("recurrent", "brolm_causal_conv", [c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_long,
                                               c_void_p, c_long, c_int, c_void_p])
    _check(f(_ptr(x), _code(x), x.stride(0), _ptr(in_bias), _ptr(taps), _ptr(bias), C, K, CONV_ACTS[activation],
             _ptr(tok_seq), _ptr(positions), *_seq(cu_q, kv_len, slots, state), tail_off, _ptr(out), out.stride(0),
             x.shape[0], _stream()), "causal_conv")


def conv_tail(x: torch.Tensor, in_bias: Optional[torch.Tensor], K: int, cu_q: torch.Tensor, kv_len: torch.Tensor,
              slots: torch.Tensor, state: torch.Tensor, tail_off: int, batch: int) -> None:
    """Move every sequence's kept K - 1 convolution inputs on by the step's tokens (after all that read them)."""
    C = x.shape[1]
    assert x.stride(1) == 1 and tail_off + (K - 1) * C <= state.shape[1]
    assert in_bias is None or (in_bias.dtype == torch.float32 and in_bias.numel() == C)
    f = _fn("recurrent", "brolm_conv_tail", [c_void_p, c_int, c_long, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_long, c_long, c_int, c_void_p])
    _check(f(_ptr(x), _code(x), x.stride(0), _ptr(in_bias), C, K, *_seq(cu_q, kv_len, slots, state), tail_off, batch,
             _stream()), "conv_tail")


def gated_scan(pre: torch.Tensor, u: torch.Tensor, y_raw: torch.Tensor, y_bias: Optional[torch.Tensor],
               r_bias: torch.Tensor, i_bias: torch.Tensor, lam: torch.Tensor, decay_scale: float, block: int,
               positions: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor, slots: torch.Tensor, state: torch.Tensor,
               out: torch.Tensor, batch: int, max_q_len: int, pre_lo: Optional[torch.Tensor] = None) -> None:
    """The gated diagonal recurrence over the packed tokens: per channel c of block c // block,
    r, i = sigmoid(pre[t, blk, 0 / 1, o] + bias), a = exp(-decay_scale * r * softplus(lam)),
    S <- a S + sqrt(1 - a^2) i u[t, c], out[t, c] = S * gelu_tanh(y_raw[t, c] + y_bias).  S is ``state[slot, :width]``.
    ``pre`` is overwritten.  A sequence of more than 32 tokens is scanned as 32 runs side by side that are then joined.
    ``pre_lo``: the gates' sums are pre + pre_lo (two products over the halves that ``split_halves`` makes)."""
    width = u.shape[1]
    assert pre.dtype == torch.float32 and u.dtype == torch.float32 and pre.stride(1) == 1 and u.stride(1) == 1
    assert pre.shape[1] == 2 * width and y_raw.stride(1) == 1 and y_raw.shape[1] == width and out.stride(1) == 1
    assert positions.dtype == torch.int32 and positions.numel() == u.shape[0]
    if pre_lo is not None:
        assert pre_lo.dtype == torch.float32 and pre_lo.shape == pre.shape and pre_lo.stride() == pre.stride()
    for v in (y_bias, r_bias, i_bias, lam):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.numel() == width)
    f = _fn("recurrent", "brolm_gated_scan", [c_void_p, c_void_p, c_long, c_void_p, c_long, c_void_p, c_int, c_long, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_long, c_void_p, c_int, c_long, c_int, c_int, c_int,
                                              c_void_p])
    _check(f(_ptr(pre), _ptr(pre_lo), pre.stride(0), _ptr(u), u.stride(0), _ptr(y_raw), _code(y_raw), y_raw.stride(0), _ptr(y_bias),
             _ptr(r_bias), _ptr(i_bias), _ptr(lam), decay_scale, width, block, _ptr(positions),
             *_seq(cu_q, kv_len, slots, state), _ptr(out), _code(out), out.stride(0), batch, u.shape[0], max_q_len,
             _stream()), "gated_scan")
    global _launches
    _launches += 1                      # two kernels


def split_halves(u: torch.Tensor, out: torch.Tensor) -> None:
    """out (2 rows, cols) bfloat16 = [bf16(u); bf16(u - bf16(u))] for float32 u (rows, cols): 16 bits of u in two halves."""
    rows, cols = u.shape
    assert u.dtype == torch.float32 and out.dtype == torch.bfloat16 and u.stride(1) == 1 and out.stride(1) == 1
    assert tuple(out.shape) == (2 * rows, cols)
    f = _fn("recurrent", "brolm_split_halves", [c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_void_p])
    _check(f(_ptr(u), u.stride(0), _ptr(out), out.stride(0), rows, cols, _stream()), "split_halves")


def block_matvec_ok(rows: int, k: int) -> bool:
    """Whether ``block_matvec_f32`` takes this many rows of this length."""
    return 0 < rows <= 16 and rows * k <= 12288


def block_matvec_f32(a: torch.Tensor, a_head: int, weight: torch.Tensor, out: torch.Tensor, o_head: int) -> None:
    """``heads_linear`` for a handful of float32 rows: out[t, h * o_head + n] = sum_k weight[h, n, k] * a[t, h * a_head + k],
    one coalesced pass over every matrix row, used for all tokens."""
    H, N, K = weight.shape
    assert a.dtype == torch.float32 and weight.dtype == torch.float32 and out.dtype == torch.float32
    assert weight.is_contiguous() and a.stride(1) == 1 and out.stride(1) == 1 and a.shape[0] == out.shape[0]
    assert (H - 1) * a_head + K <= a.shape[1] and (H - 1) * o_head + N <= out.shape[1] and block_matvec_ok(a.shape[0], K)
    f = _fn("recurrent", "brolm_block_matvec_f32", [c_void_p, c_long, c_long, c_void_p, c_void_p, c_long, c_long, c_int, c_int,
                                                    c_int, c_int, c_void_p])
    _check(f(_ptr(a), a.stride(0), a_head, _ptr(weight), _ptr(out), out.stride(0), o_head, a.shape[0], H, N, K, _stream()),
           "block_matvec_f32")


def ssm_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d: torch.Tensor,
             heads: int, groups: int, head_size: int, n_state: int, cu_q: torch.Tensor, kv_len: torch.Tensor,
             slots: torch.Tensor, state: torch.Tensor, y: torch.Tensor, batch: int, max_q_len: int) -> None:
    """The selective state space over the packed tokens.  xbc float32 (tokens, heads * P + 2 * groups * N) =
    [x | B | C]; dt_raw (tokens, heads) may be a strided view; per head S (kept as [P][N] in ``state[slot]``):
    dt = softplus(dt_raw + dt_bias), S <- exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + d x."""
    P, N = head_size, n_state
    assert xbc.dtype == torch.float32 and xbc.stride(1) == 1 and xbc.shape[1] == heads * P + 2 * groups * N
    assert dt_raw.dtype == torch.float32 and dt_raw.stride(1) == 1 and dt_raw.shape[1] == heads
    assert y.dtype == torch.float32 and y.stride(1) == 1
    assert y.shape[1] == heads * P and state.shape[1] >= heads * P * N
    for v in (dt_bias, a_log, d):
        assert v.dtype == torch.float32 and v.is_contiguous() and v.numel() == heads
    f = _fn("recurrent", "brolm_ssm_scan", [c_void_p, c_long, c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_int,
                                            c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_void_p,
                                            c_long, c_int, c_int, c_void_p])
    _check(f(_ptr(xbc), xbc.stride(0), _ptr(dt_raw), _code(dt_raw), dt_raw.stride(0), _ptr(dt_bias), _ptr(a_log), _ptr(d),
             heads, groups, P, N, *_seq(cu_q, kv_len, slots, state), _ptr(y), y.stride(0), batch, max_q_len, _stream()),
           "ssm_scan")


SCAN_ACTS = {"none": 0, "silu": 1}


def decay_state_size(heads: int, dim: int, v_dim: int) -> int:
    """Floats of a sequence's state row that ``decay_scan`` keeps: [head][value column][dim padded to four]."""
    return heads * v_dim * ((dim + 3) // 4 * 4)


def decay_scan(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, dim: int, v_dim: int, activation: str,
               decay_m1: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor, slots: torch.Tensor, state: torch.Tensor,
               out: torch.Tensor, batch: int, max_q_len: int = 0) -> None:
    """Linear attention with a fixed decay per head over the packed tokens: S <- decay_h S + k v^T, out = S^T q.
    q, k (``dim`` per head) and v (``v_dim`` per head) are columns of ``qkv`` (tokens, cols) from ``q_off``, ``k_off``,
    ``v_off`` on, head by head; ``activation`` ("none", "silu") is applied to them as they are read.  ``decay_m1``
    float32 [heads] holds decay - 1.  S is the first ``decay_state_size`` floats of ``state[slot]``.  ``out`` float32
    (tokens, heads * v_dim).  ``max_q_len`` 1 says that every sequence brings one token (the launch then takes part
    in programmatic launch); 0: unknown."""
    assert qkv.stride(1) == 1 and out.dtype == torch.float32 and out.stride(1) == 1 and out.shape == (qkv.shape[0], heads * v_dim)
    assert decay_m1.dtype == torch.float32 and decay_m1.is_contiguous() and decay_m1.numel() == heads
    assert max(q_off, k_off) + heads * dim <= qkv.shape[1] and v_off + heads * v_dim <= qkv.shape[1]
    assert state.shape[1] >= decay_state_size(heads, dim, v_dim)
    if activation not in SCAN_ACTS:
        raise KernelError(f"decay_scan: unknown activation '{activation}'")
    f = _fn("linear_attn", "brolm_decay_scan", [c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_long,
                                                c_int, c_int, c_void_p])
    _check(f(_ptr(qkv), _code(qkv), qkv.stride(0), q_off, k_off, v_off, heads, dim, v_dim, SCAN_ACTS[activation],
             _ptr(decay_m1), *_seq(cu_q, kv_len, slots, state), _ptr(out), out.stride(0), batch, int(max_q_len), _stream()),
           "decay_scan")


def linear_f32(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out (M, N) = x (M, K) @ weight (N, K)^T, all float32, rows may be strided."""
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and out.dtype == torch.float32
    assert x.dim() == 2 and weight.dim() == 2 and out.dim() == 2
    assert x.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and tuple(out.shape) == (M, N)
    f = _fn("linear_f32", "brolm_linear_f32", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                               c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, _stream()),
           "linear_f32")


SKINNY_MAX_ROWS = 16


def skinny_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the few-token product kernel takes these operands."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and
            0 < x.shape[0] <= SKINNY_MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1 and
            x.stride(0) % 8 == 0 and weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and
            x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def _stream_share(fill: float) -> float:
    """Which part of the memory's rate a stream of weights reaches while an SM holds ``fill`` of the
    blocks it has room for (their weights in flight against the memory's latency): measured with the
    few-token product, 0.45 with one block of three, 0.75 with two, 0.95 with all three."""
    pts = ((0.0, 0.0), (1.0 / 3, 0.45), (2.0 / 3, 0.75), (1.0, 0.95))
    for (x0, y0), (x1, y1) in zip(pts, pts[1:]):
        if fill <= x1:
            return y0 + (y1 - y0) * (fill - x0) / (x1 - x0)
    return 0.95


def _rounds_cost(blocks: int, per_sm: int, sms: int, nbytes: float) -> float:
    """Estimated time, in bytes at the memory's full rate, of ``blocks`` equal blocks that stream ``nbytes``
    in all, ``per_sm`` of them fitting an SM at a time: round after round of blocks, each round at the
    rate its fill allows, plus 1.5 us for a round's start and end."""
    left, cost = blocks, 0.0
    while left > 0:
        now = min(left, per_sm * sms)
        cost += 1.5e-6 * 6.5e12 + nbytes * now / blocks / _stream_share(now / float(per_sm * sms))
        left -= now
    return cost


def skinny_rope_tiles(width: int, k: int, sms: Optional[int] = None) -> int:
    """16-row tiles of W per block (1 or 2) for the fused q/k/v projection, which cannot be cut along K:
    whichever fills the rounds of blocks better.  4096 rows (Gemma 2 2B): 256 blocks of one tile, three
    to an SM; 8192 rows (9B, 27B): 512 such blocks would be one round and a thin second one, 256 blocks of
    two tiles, two to an SM, are one round."""
    sms = sms or device_sms()
    tiles = (width + 15) // 16
    if tiles % 2:
        return 1
    nbytes = float(width) * k * 2.0
    return 1 if _rounds_cost(tiles, 3, sms, nbytes) <= _rounds_cost(tiles // 2, 2, sms, nbytes) else 2


def skinny_parts(x: torch.Tensor, weight: torch.Tensor, sms: Optional[int] = None) -> int:
    """Into how many slices of K a few-token product is cut.

    A block streams 16 rows of W over its slice, three blocks share an SM, and a stream runs near the
    memory's rate only while the SMs hold about three blocks each: with one block an SM reaches about
    0.45 of its share, with two 0.75, with three 0.95 (the weights of a block in flight against the
    memory's latency).  The slices decide how many blocks there are and so how full the rounds of
    blocks are; a last round of a few blocks streams slowly and is what to avoid.  The number of
    slices (at most 8, at least 8 blocks of 64 k each) with the shortest estimated time is taken; every
    slice is another float copy of the output for the kernel after it to add, which counts too.
    Measured, product + residual kernel, microseconds at 8 tokens, by slices 1 / 2 / 3 / 4:
    2304 x 9216 (2B down) 14.4 / 12.5 / 11.8 / 14.8; 4608 x 36864 (27B down) 74.0 / 72.9 / 63.2 / 67.4;
    3584 x 4096 (9B o) 10.7 / 11.8 / 12.2 / 12.0."""
    sms = sms or device_sms(x.device if x.is_cuda else None)
    blocks = (weight.shape[0] + 15) // 16
    kblocks = (x.shape[1] + 63) // 64
    nbytes = float(weight.shape[0]) * x.shape[1] * 2.0
    best, best_cost = 1, None
    for parts in range(1, 9):
        if parts > 1 and kblocks // parts < 8:
            break
        cost = _rounds_cost(blocks * parts, 3, sms, nbytes)
        cost += (parts - 1) * x.shape[0] * weight.shape[0] * 8.0 + (parts - 1) * 0.3e-6 * 6.5e12
        if best_cost is None or cost < best_cost * 0.98:
            best, best_cost = parts, cost
    return best


def skinny_gemm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "store",
                activation: str = "gelu_tanh", cap: float = 0.0, limit: float = 0.0) -> None:
    """out = x @ weight^T for at most 16 rows of x (bfloat16 in, float32 accumulation).

    ``epilogue``: "store" (out bfloat16 or float32), "gated" (weight = [Wg; Wu],
    out = act(x Wg^T) * (x Wu^T)), "softcap" (out float32 = cap * tanh(. / cap)).
    """
    assert skinny_ok(x, weight) and out.stride(-1) == 1 and out.shape[-2] == x.shape[0]
    M, K = x.shape
    assert weight.shape[1] == K
    code = {"store": 0, "gated": 1, "softcap": 2}[epilogue]
    N = out.shape[-1]
    ksplit, part_stride = 1, 0
    if out.dim() == 3:                      # [parts, M, N] float32 partial sums along K
        assert code == 0 and out.dtype == torch.float32 and out.stride(1) == N
        ksplit, part_stride = out.shape[0], out.stride(0)
    assert weight.shape[0] == (2 * N if code == 1 else N)
    if code == 1:
        if activation not in ACTIVATIONS:
            raise KernelError(f"skinny_gemm: unknown activation '{activation}'")
        # a gate tile and an up tile per block, two blocks to an SM, whatever the width: blocks of four tiles (one
        # to an SM) measured slower at every size (8 tokens: 9B 40.7 against 34.5 us, 27B 109.4 against 104.6 us,
        # 2B 17.4 against 16.2 us): their last, thin round of blocks streams twice the bytes per block
        tiles = 2
    else:
        tiles = 2 if N >= 64 * device_sms(x.device) else 1
    if code == 2:
        assert out.dtype == torch.float32
    f = _fn("skinny_gemm", "brolm_skinny_gemm", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                                 c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_longlong,
                                                 c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(-2), M, N, K, code,
             1 if out.dtype == torch.float32 else 0, ACTIVATIONS.get(activation, 0), limit if code == 1 else cap, tiles,
             ksplit, part_stride, _stream()), "skinny_gemm")


def skinny_qkv_rope(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                    cos_sin: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int,
                    k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                    cache_rows: Optional[torch.Tensor] = None, page_size: int = 64) -> None:
    """out = x @ [Wq; Wk; Wv]^T for at most 16 rows of x, with q and k rotated over the whole head
    (pairs i, i + head_dim/2; ``cos_sin`` [positions, head_dim/2, 2], None: no rotation) and k, v written
    into the cache pages as well: ``rope_kv_write`` as the epilogue of the product, one rounding to
    bfloat16 instead of two.  Rows with a negative position are not written."""
    assert skinny_ok(x, weight) and out.dtype == torch.bfloat16 and out.stride(1) == 1
    width = (n_q + 2 * n_kv) * head_dim
    assert weight.shape == (width, x.shape[1]) and out.shape == (x.shape[0], width) and head_dim % 16 == 0
    assert positions.dtype == torch.int32 and positions.numel() == x.shape[0]
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] == head_dim // 2
    if k_pages is not None:
        assert v_pages is not None and cache_rows is not None and k_pages.dtype == torch.bfloat16
        assert k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim)
        assert cache_rows.dtype == torch.int32 and cache_rows.numel() == x.shape[0]
    f = _fn("skinny_gemm", "brolm_skinny_qkv_rope", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                                     c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                                     c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), x.shape[0], x.shape[1],
             _ptr(positions), _ptr(cos_sin), n_q, n_kv, head_dim, _ptr(k_pages), _ptr(v_pages), _ptr(cache_rows),
             page_size, skinny_rope_tiles(width, x.shape[1], device_sms(x.device)), _stream()), "skinny_qkv_rope")


USE_TC_GEMM = True      # False: many-token bfloat16 products go to the library (cuBLAS) instead
USE_PAIR_GEMM = True    # False: the tcgen05 product runs one block per tile instead of a pair of SMs per tile


def gemm_tc_ok(x: torch.Tensor, weight: torch.Tensor, gated: bool = False, sms: Optional[int] = None) -> bool:
    """Whether the tcgen05 product kernel takes these operands and has enough
    128 x 256 tiles of output to put one on every SM (fewer tiles would leave
    SMs idle while the rest stream the weights)."""
    sms = sms or device_sms(x.device if x.is_cuda else None)
    out_cols = weight.shape[0] // 2 if gated else weight.shape[0]
    tiles = ((x.shape[0] + 127) // 128) * ((out_cols + (127 if gated else 255)) // (128 if gated else 256))
    return (USE_TC_GEMM and tiles >= sms and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and
            x.shape[0] > SKINNY_MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and
            weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and
            weight.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "store",
            activation: str = "gelu_tanh", pairs: Optional[bool] = None, limit: float = 0.0) -> None:
    """out = x @ weight^T on the tcgen05 tensor cores (bfloat16 in, float32 accumulation in tensor memory).

    Runs on pairs of SMs (``gemm_tc2``: 256 x 256 tiles, tcgen05 cta_group::2) unless ``pairs`` is False or
    ``USE_PAIR_GEMM`` is off; then one block per 128 x 256 tile.

    ``epilogue``: "store" (out bfloat16 or float32) or "gated" (weight = [Wg; Wu], out = act(x Wg^T) * (x Wu^T),
    out width a multiple of 128)."""
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and out.stride(1) == 1
    M, K = x.shape
    N = out.shape[1]
    code = {"store": 0, "gated": 1}[epilogue]
    assert weight.shape == ((2 * N if code else N), K) and out.shape[0] == M
    if activation not in ACTIVATIONS:
        raise KernelError(f"gemm_tc: unknown activation '{activation}'")
    if USE_PAIR_GEMM and pairs is not False:
        return gemm_tc2(x, weight, out, epilogue, activation, limit)
    f = _fn("gemm_tc", "brolm_gemm_tc", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                         c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, code,
             1 if out.dtype == torch.float32 else 0, ACTIVATIONS[activation], limit, _stream()), "gemm_tc")


def gemm_tc2(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "store",
             activation: str = "gelu_tanh", limit: float = 0.0) -> None:
    """``gemm_tc`` on pairs of SMs (tcgen05 cta_group::2): 256 x 256 tiles, each block of a pair loads half
    of the weight tile.  Same operands and epilogues."""
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    assert weight.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == x.shape[0]
    M, K = x.shape
    code = {"store": 0, "gated": 1}[epilogue]
    N = out.shape[1]
    assert weight.shape == ((2 * N if code == 1 else N), K)
    f = _fn("gemm_tc2", "brolm_gemm_tc2", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K, code,
             1 if out.dtype == torch.float32 else 0, ACTIVATIONS[activation], limit, _stream()), "gemm_tc2")


def gemm_tc2_status(reset: bool = False) -> int:
    """0 if no bounded wait inside gemm_tc2 ever ran out; otherwise its code.  Synchronises."""
    if not library_loaded("gemm_tc2"):
        return 0
    f = load_library("gemm_tc2").brolm_gemm_tc2_status
    f.argtypes = [c_int]
    f.restype = c_int
    return f(1 if reset else 0)


def gemm_tc_status(reset: bool = False) -> int:
    """0 if no bounded wait inside gemm_tc (either form) ever ran out; otherwise the code of the first one.
    Synchronises."""
    pair = gemm_tc2_status(reset)
    if pair or not library_loaded("gemm_tc"):
        return pair                # (a library none of whose kernels ever ran is not built or loaded for the question)
    f = load_library("gemm_tc").brolm_gemm_tc_status
    f.argtypes = [c_int]
    f.restype = c_int
    return f(1 if reset else 0)


WAIT_LIBRARIES = ("gemm_tc", "gemm_tc2", "gemm_stream", "attn_tc", "grouped_tc")


def wait_control(library: str, cycles: int = 0, stall_code: int = 0) -> None:
    """The limit of the bounded waits inside one of the tcgen05 libraries, in clock cycles (0: the default of
    about a second), and, for tests of the give-up path, the code of the waits that shall behave as if
    their barrier never completed (0: none).  A wait that runs out ends its kernel early; the library's
    status function then reports the code and ``Engine.step`` raises ``StepError``."""
    if library not in WAIT_LIBRARIES:
        raise KernelError(f"wait_control: '{library}' has no bounded waits (libraries: {WAIT_LIBRARIES})")
    f = getattr(load_library(library), f"brolm_{library}_wait_control")
    f.argtypes = [c_longlong, c_int]
    f.restype = c_int
    status = f(int(cycles), int(stall_code))
    if status:
        raise KernelError(f"wait_control: CUDA error {status}")


STREAM_MAX_ROWS = 128
# Up to how many tokens the per-layer products of a step go to the tcgen05 weight stream rather than to the
# library (cuBLAS).  Measured at the Gemma 2 2B sizes, context 1280 (tokens/s, own stream against library):
# 24 rows 9,598 / 9,582; 32 rows 12,708 / 12,660; 48 rows 14,076 / 14,436; 64 rows 18,676 / 19,152;
# 96 rows 20,727 / 22,622; 128 rows 23,901 / 25,584.  With 64 and 128 token columns a stage of the ring is a
# third and a half tokens, so fewer bytes of weights are in flight per SM; up to 32 it is at least even.
# BROLM_STREAM_ROWS=128 takes every product of up to 128 tokens to the own kernel, =16 none.
STREAM_ROWS = int(os.environ.get("BROLM_STREAM_ROWS", "32"))


def stream_rows(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether a product of this many tokens is one for the tcgen05 weight stream: more rows than the
    mma.sync kernel takes (16), at most STREAM_ROWS, operands it takes."""
    return x.dim() == 2 and SKINNY_MAX_ROWS < x.shape[0] <= STREAM_ROWS and gemm_stream_ok(x, weight)


def gemm_stream_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the tcgen05 weight-streaming product (few tokens) takes these operands."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and
            0 < x.shape[0] <= STREAM_MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1 and
            x.stride(0) % 8 == 0 and weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and
            x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_stream_parts(x: torch.Tensor, weight: torch.Tensor, sms: Optional[int] = None) -> int:
    """Slices of K so that every SM gets a (128-row tile, slice) item of the weight stream."""
    sms = sms or device_sms(x.device if x.is_cuda else None)
    row_tiles = (weight.shape[0] + 127) // 128
    nkb = (x.shape[1] + 63) // 64
    want = max(1, sms // row_tiles)
    # at least a ring's worth of K blocks (8) per item: a shorter run is over before its loads are all
    # in flight, and every further slice is another float copy of the output for the reader to add
    per = max(min(8, nkb), (nkb + want - 1) // want)
    return max(1, (nkb + per - 1) // per)


def gemm_stream(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "store",
                activation: str = "gelu_tanh", cap: float = 0.0, limit: float = 0.0) -> None:
    """out = x @ weight^T for at most 128 rows of x on tcgen05, the weights streamed through a TMA ring.

    ``epilogue``: "store" (out bfloat16 or float32, or [parts, M, N] float32 partial sums of K slices),
    "gated" (weight = [Wg; Wu], out = act(x Wg^T) * (x Wu^T), width a multiple of 64), "softcap" (float32)."""
    assert gemm_stream_ok(x, weight) and out.stride(-1) == 1 and out.shape[-2] == x.shape[0]
    M, K = x.shape
    code = {"store": 0, "gated": 1, "softcap": 2}[epilogue]
    N = out.shape[-1]
    assert weight.shape == ((2 * N if code == 1 else N), K)
    ksplit, part_stride = 1, 0
    if out.dim() == 3:
        assert code == 0 and out.dtype == torch.float32 and out.stride(1) == N
        ksplit, part_stride = out.shape[0], out.stride(0)
    if code == 2:
        assert out.dtype == torch.float32
    if activation not in ACTIVATIONS:
        raise KernelError(f"gemm_stream: unknown activation '{activation}'")
    f = _fn("gemm_stream", "brolm_gemm_stream", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                 c_int, c_int, c_int, c_float, c_int, c_longlong, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(-2), M, N, K, code,
             1 if out.dtype == torch.float32 else 0, ACTIVATIONS[activation], limit if code == 1 else cap, ksplit,
             part_stride, _stream()), "gemm_stream")


def gemm_stream_status(reset: bool = False) -> int:
    """0 if no bounded wait inside gemm_stream ever ran out; otherwise its code.  Synchronises."""
    if not library_loaded("gemm_stream"):
        return 0                   # none of its kernels ever ran: nothing is built or loaded for the question
    f = load_library("gemm_stream").brolm_gemm_stream_status
    f.argtypes = [c_int]
    f.restype = c_int
    return f(1 if reset else 0)


def attention_simt(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor, *, n_kv: int,
                   group: int, head_dim: int, scale: float, cap: float, window: int, batch: int, max_q_len: int,
                   k: Optional[torch.Tensor] = None, v: Optional[torch.Tensor] = None,
                   k_pages: Optional[torch.Tensor] = None, v_pages: Optional[torch.Tensor] = None,
                   page_table: Optional[torch.Tensor] = None, ring: int = 0, page_size: int = 0,
                   sink: Optional[torch.Tensor] = None, v_dim: Optional[int] = None, chunk: int = 0,
                   slopes: Optional[torch.Tensor] = None, keep_first: int = 0, ring_from: int = 0,
                   v_all: int = 0, v_from: int = 0, dist_bias: Optional[torch.Tensor] = None) -> None:
    """Exact attention on CUDA cores.  Keys come from (k, v) packed like q, or from cache pages.
    ``sink``: float32 [query heads]; exp(sink) joins every softmax's denominator (a key with no value).
    ``v_dim``: size of a value row and of an output row when it is not ``head_dim``.
    ``chunk`` > 0: a query at position p sees no key before p - p % chunk.
    ``slopes``: float32 [query heads]; slopes[h] * (p - j) is taken off the scaled score of key j.
    ``keep_first``: with a window, keys at positions below it stay visible; the pages then hold the first
    ``ring_from`` places (a multiple of the page size, at least keep_first) for good, the ring behind them.
    ``v_all`` > 0: every query head's weights are applied to the value rows of ``v_all`` kv heads from
    ``v_from`` on; ``out`` is then (tokens, heads * n_kv * v_dim), head h's row being [n_kv][v_dim], of which
    the call fills those kv heads' part (``attention_all_values`` covers all of them).
    ``out`` may be float32 whatever the element type of q.
    ``dist_bias``: float32 [query heads, L]; key j adds entry min(p - j, L - 1) of its head's row to the score
    after the scale and the cap."""
    _check_dist_bias(dist_bias, n_kv * group)
    _check_sink(sink, n_kv * group)
    _check_sink(slopes, n_kv * group)
    vd = v_dim or head_dim
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and (q.dtype == out.dtype or out.dtype == torch.float32)
    assert out.shape[-1] >= n_kv * group * vd * (n_kv if v_all else 1) and 0 <= v_from <= n_kv - v_all
    assert cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    kv_stride = v_stride = pt_stride = 0
    if k_pages is not None:
        assert page_table is not None and page_table.dtype == torch.int32 and page_table.stride(1) == 1
        assert k_pages.dtype == q.dtype and v_pages.dtype == q.dtype and k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim)
        assert tuple(v_pages.shape[1:]) == (n_kv, page_size, vd)
        pt_stride = page_table.stride(0)
    else:
        assert k is not None and v is not None and k.dtype == q.dtype and v.dtype == q.dtype
        assert k.stride(-1) == 1 and v.stride(-1) == 1
        kv_stride, v_stride = k.stride(0), v.stride(0)
    f = _fn("attn_simt", "brolm_attn_simt", [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                             c_int, c_int, c_int, c_float, c_float, c_int, c_void_p, c_int, c_int,
                                             c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                             c_int, c_void_p])
    _check(f(_code(q), _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cu_q), _ptr(kv_len), _ptr(k), _ptr(v),
             kv_stride, _ptr(k_pages), _ptr(v_pages), _ptr(page_table), pt_stride, ring, page_size, n_kv, group,
             head_dim, scale, cap, window, _ptr(sink), batch, max_q_len, vd, v_stride, int(chunk), _ptr(slopes),
             int(keep_first), int(ring_from), int(v_all), int(v_from), 1 if out.dtype == torch.float32 else 0,
             _ptr(dist_bias), dist_bias.shape[1] if dist_bias is not None else 0, _stream()),
           "attention_simt")


ALL_VALUES_ROW = 512        # the exact kernel's limit for an output row of one head


def attention_all_values(q: torch.Tensor, acc: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor, *, n_kv: int,
                         v_dim: int, **args) -> None:
    """``attention_simt`` with every query head's weights applied to the values of every kv head: ``acc`` float32
    (tokens, heads * n_kv * v_dim).  As many kv heads a call as fit the kernel's row; the scores are computed anew
    by each call, in the same order, so the weights of all calls are the same bits."""
    assert acc.dtype == torch.float32
    per_call = max(1, min(n_kv, ALL_VALUES_ROW // v_dim))
    for first in range(0, n_kv, per_call):
        attention_simt(q, acc, cu_q, kv_len, n_kv=n_kv, v_dim=v_dim, v_all=min(per_call, n_kv - first), v_from=first,
                       **args)


def attention_headmix_ok(head_dim: int, v_dim: int, group: int, decode: bool, page_size: int = 64) -> bool:
    """Whether the tensor-core kernels with the head-wise options take these sizes (bfloat16 only)."""
    ok = head_dim % 16 == 0 and v_dim % 16 == 0 and 0 < head_dim <= 256 and 0 < v_dim <= 256
    return ok and (not decode or (group <= 16 and page_size == 64))


HEADMIX_ROUNDS = int(os.environ.get("BROLM_HEADMIX_ROUNDS", "2"))


def attention_headmix_shares_keys(head_dim: int, v_dim: int, n_kv: int, group: int, all_values: bool) -> bool:
    """Whether a decode step of these sizes runs the kernel that keeps the value rows of every kv head in one
    block (at most 8 query heads per kv head, n_kv * v_dim up to 512, a stage of keys and values twice in shared
    memory): its grid has n_kv block rows a sequence, the other kernel's n_kv * n_kv.  The launcher's own rule."""
    key = (head_dim, v_dim, n_kv, group, bool(all_values))
    got = _shares_memo.get(key)
    if got is None:
        f = _fn("attn_headmix", "brolm_attn_headmix_decode_shares_keys", [c_int, c_int, c_int, c_int, c_int, c_int])
        got = _shares_memo[key] = bool(f(head_dim, v_dim, n_kv, group, 1 if all_values else 0, 40))
    return got


_shares_memo: dict = {}


def headmix_splits(batch: int, blocks_y: int, max_kv_len: int, window: int, keep_first: int,
                   sms: Optional[int] = None, rounds: Optional[int] = None) -> int:
    """How many blocks share the visible keys of one (sequence, block row) when decoding: ``rounds`` blocks per
    SM over the whole grid (default ``HEADMIX_ROUNDS``: a block walks its tiles one after another and two are
    resident on an SM, so with many block rows short walks beat one round of long ones; the kernel that keeps
    every value head in a block holds an SM alone and takes one round), at least two tiles a block, at most 40."""
    sms = sms or device_sms()
    keys = min(max_kv_len, window + 63 + (keep_first + 63) // 64 * 64) if window > 0 else max_kv_len
    tiles = max(1, (keys + 63) // 64)
    if batch * blocks_y > 65536:
        return 1                       # more block rows than the splits' tickets
    return max(1, min((rounds or HEADMIX_ROUNDS) * sms // max(1, batch * blocks_y), (tiles + 1) // 2, 40))


def attention_headmix_prefill(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                              n_kv: int, group: int, head_dim: int, v_dim: int, scale: float, window: int, batch: int,
                              max_q_len: int, slopes: Optional[torch.Tensor] = None, keep_first: int = 0,
                              all_values: bool = False, cap: float = 0.0, sink: Optional[torch.Tensor] = None,
                              dist_bias: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention (bfloat16 operands) of whole prompts that start at position 0, with value rows of
    their own size, distance slopes and a window that keeps first keys.  ``out`` is bfloat16 or float32,
    (tokens, heads * v_dim); with ``all_values`` every head's weights meet the values of every kv head and
    ``out`` is (tokens, heads * n_kv * v_dim), head h's row being [n_kv][v_dim].  ``cap``, ``sink`` and
    ``dist_bias`` as in ``attention_simt`` (not together with ``all_values``)."""
    _check_sink(slopes, n_kv * group)
    _check_sink(sink, n_kv * group)
    _check_dist_bias(dist_bias, n_kv * group)
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    assert out.dtype in (torch.bfloat16, torch.float32)
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert out.shape[-1] >= n_kv * group * v_dim * (n_kv if all_values else 1) and cu_q.dtype == torch.int32
    f = _fn("attn_headmix", "brolm_attn_headmix_prefill",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_float, c_int, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), 1 if out.dtype == torch.float32 else 0, _ptr(cu_q),
             _ptr(k), k.stride(0), _ptr(v), v.stride(0), n_kv, group, head_dim, v_dim, scale, int(window),
             int(keep_first), _ptr(slopes), 1 if all_values else 0, batch, max_q_len, float(cap), _ptr(sink),
             _ptr(dist_bias), dist_bias.shape[1] if dist_bias is not None else 0, _stream()),
           "attention_headmix_prefill")


def attention_headmix_decode(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                             k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor, *, ring: int,
                             ring_from: int, page_size: int, n_kv: int, group: int, head_dim: int, v_dim: int,
                             scale: float, window: int, batch: int, n_splits: int,
                             slopes: Optional[torch.Tensor] = None, keep_first: int = 0,
                             all_values: bool = False, cap: float = 0.0, sink: Optional[torch.Tensor] = None,
                             dist_bias: Optional[torch.Tensor] = None) -> None:
    """The same attention for one new token per sequence over the paged cache (pages of 64 keys, at most 16
    query heads per kv head).  The splits' partial results go through float32 scratch made here; the block
    that finishes last among them merges them."""
    _check_sink(slopes, n_kv * group)
    _check_sink(sink, n_kv * group)
    _check_dist_bias(dist_bias, n_kv * group)
    assert q.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and v_pages.dtype == torch.bfloat16
    assert out.dtype in (torch.bfloat16, torch.float32) and q.stride(-1) == 1 and out.stride(-1) == 1
    assert k_pages.is_contiguous() and v_pages.is_contiguous()
    assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim) and tuple(v_pages.shape[1:]) == (n_kv, page_size, v_dim)
    assert page_table.dtype == torch.int32 and page_table.stride(1) == 1
    assert cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    n_vh = n_kv if all_values else 1
    assert out.shape[-1] >= n_kv * group * v_dim * n_vh
    part_o = part_ml = None
    if n_splits > 1:
        n = batch * n_kv * group * n_vh * n_splits
        both = torch.empty(n * (v_dim + 2), dtype=torch.float32, device=q.device)
        part_o, part_ml = both[:n * v_dim], both[n * v_dim:]
    f = _fn("attn_headmix", "brolm_attn_headmix_decode",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
             c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), 1 if out.dtype == torch.float32 else 0, _ptr(cu_q),
             _ptr(kv_len), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.stride(0), ring, int(ring_from),
             page_size, n_kv, group, head_dim, v_dim, scale, int(window), int(keep_first), _ptr(slopes),
             1 if all_values else 0, batch, n_splits, _ptr(part_o), _ptr(part_ml), float(cap), _ptr(sink), _ptr(dist_bias),
             dist_bias.shape[1] if dist_bias is not None else 0, _stream()),
           "attention_headmix_decode")


def _check_dist_bias(table: Optional[torch.Tensor], n_q: int) -> None:
    if table is not None:
        assert table.dtype == torch.float32 and table.is_contiguous() and table.dim() == 2 and table.shape[0] == n_q
        assert table.shape[1] >= 1


def _check_sink(sink: Optional[torch.Tensor], n_q: int) -> None:
    if sink is not None:
        assert sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == n_q


def attention_prefill_mma(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                          n_kv: int, group: int, head_dim: int, scale: float, cap: float, window: int, batch: int,
                          max_q_len: int, sink: Optional[torch.Tensor] = None, chunk: int = 0,
                          dist_bias: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention of whole prompts that start at position 0 (bfloat16, head_dim <= 256).
    ``chunk`` > 0: a query at position p sees no key before p - p % chunk.  ``dist_bias`` as in ``attention_simt``."""
    _check_sink(sink, n_kv * group)
    _check_dist_bias(dist_bias, n_kv * group)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert k.stride(0) == v.stride(0) and cu_q.dtype == torch.int32
    f = _fn("attn_mma", "brolm_attn_prefill_mma", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                   c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p, c_int,
                                                   c_int, c_int, c_void_p, c_int, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cu_q), _ptr(k), _ptr(v), k.stride(0), n_kv, group,
             head_dim, scale, cap, window, _ptr(sink), batch, max_q_len, int(chunk), _ptr(dist_bias),
             dist_bias.shape[1] if dist_bias is not None else 0, _stream()), "attention_prefill_mma")


def attention_prefill_tc_ok(head_dim: int, group: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes these sizes."""
    return head_dim in (64, 128, 256) and group > 0 and 128 % group == 0


def attention_prefill_tc_split(max_q_len: int, n_kv: int, group: int, window: int, batch: int) -> int:
    """How many of the heaviest row blocks of every (sequence, kv head) the tcgen05 prompt attention cuts in
    two along the keys (0: none): with few kv heads and a prompt of a few thousand tokens the causal blocks
    are few and of very different lengths, and halves fill the SMs better.  The launcher's own rule."""
    key = (max_q_len, n_kv, group, window, batch, torch.cuda.current_device())
    got = _split_memo.get(key)
    if got is None:
        f = _fn("attn_tc", "brolm_attn_prefill_tc_plan", [c_int, c_int, c_int, c_int, c_int])
        if len(_split_memo) > 64:
            _split_memo.clear()
        got = _split_memo[key] = int(f(max_q_len, n_kv, group, window, batch))
    return got


_split_memo: dict = {}


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                         n_kv: int, group: int, head_dim: int, scale: float, cap: float, window: int, batch: int,
                         max_q_len: int, v_lbo: int = 0, v_sbo: int = 0, n_split: Optional[int] = None) -> None:
    """tcgen05 attention of whole prompts that start at position 0 (bfloat16; head_dim 64, 128 or 256).
    ``n_split``: how many of the heaviest row blocks run as two halves of their keys, merged by the half
    that finishes second (None: ``attention_prefill_tc_split`` decides)."""
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert k.stride(0) == v.stride(0) and cu_q.dtype == torch.int32 and q.shape[0] == k.shape[0] == v.shape[0]
    if n_split is None:
        n_split = attention_prefill_tc_split(max_q_len, n_kv, group, window, batch) if PREFILL_SPLIT else 0
    part_o = part_ml = None
    if n_split > 0:
        pairs = n_split * n_kv * batch
        both = torch.empty(pairs * 2 * 128 * (head_dim + 2), dtype=torch.float32, device=q.device)
        part_o, part_ml = both[:pairs * 2 * 128 * head_dim], both[pairs * 2 * 128 * head_dim:]
    f = _fn("attn_tc", "brolm_attn_prefill_tc", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int,
                                                 c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cu_q), _ptr(k), _ptr(v), k.stride(0), q.shape[0],
             n_kv, group, head_dim, scale, cap, window, batch, max_q_len, v_lbo, v_sbo, n_split, _ptr(part_o),
             _ptr(part_ml), _stream()),
           "attention_prefill_tc")


# BROLM_PREFILL_SPLIT=0: the tcgen05 prompt attention never cuts a row block's keys in two
PREFILL_SPLIT = os.environ.get("BROLM_PREFILL_SPLIT", "1") != "0"


def attention_tc_status(reset: bool = False) -> int:
    """0 if no bounded wait inside the tcgen05 attention ever ran out; otherwise its code.  Synchronises."""
    if not library_loaded("attn_tc"):
        return 0                   # none of its kernels ever ran: nothing is built or loaded for the question
    f = load_library("attn_tc").brolm_attn_tc_status
    f.argtypes = [c_int]
    f.restype = c_int
    return f(1 if reset else 0)


RAGGED_WAVES = int(os.environ.get("BROLM_RAGGED_WAVES", "5"))


def decode_splits(batch: int, n_kv: int, max_kv_len: int, window: int, sms: Optional[int] = None,
                  ragged: bool = False) -> int:
    """How many blocks share the keys of one (sequence, kv head): as many as make one wave of blocks
    over the SMs (a block holds an SM's shared memory alone), at least two pages per block and at
    most 40 splits (the last block's merge reads every split's partial result).
    Measured on a B200 at 8 kv-head pairs x 4: 4 splits (one wave) read 8192 keys in 54 us, 9 splits
    (two waves) in 58 us; one sequence with 4 kv heads and 8192 keys: 37 splits (148 blocks) 1.600 ms
    per decode step of the 2B sizes against 1.632 ms with 20 splits (80 blocks).

    ``ragged``: the sequences' lengths are far from equal.  One round of blocks then ends with the longest
    sequence's blocks running alone, so every sequence is cut into enough pieces for ``RAGGED_WAVES``
    rounds and the SMs even the lengths out as they take block after block.  Measured at 16 sequences of
    1,280 to 6,400 keys and 8 kv heads (128 pairs): 1 / 2 / 4 / 6 / 8 / 12 splits 147 / 128 / 118 / 114 /
    116 / 126 us; with equal lengths more than one round only costs (152 / 163 / 167 us for 1 / 2 / 4).
    (Pieces of one size for all sequences, so that a short sequence is one block and a long one many,
    were measured too: 111 to 113 us, no better than equal shares, and are not in the kernel.)"""
    sms = sms or device_sms()
    keys = min(max_kv_len, window + 63) if window > 0 else max_kv_len
    tiles = max(1, (keys + 63) // 64)
    want = max(1, sms // max(1, batch * n_kv))
    if ragged:
        want = max(want, -(-RAGGED_WAVES * sms // max(1, batch * n_kv)))
    return max(1, min(want, (tiles + 1) // 2, 40))


def attention_decode_mma(q: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                         k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor, *, ring: int,
                         page_size: int, n_kv: int, group: int, head_dim: int, scale: float, cap: float, window: int,
                         batch: int, n_splits: int, scratch: Optional[tuple] = None,
                         sink: Optional[torch.Tensor] = None, chunk: int = 0,
                         dist_bias: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention of one new token per sequence over the paged cache
    (bfloat16, head_dim <= 256, group <= 16, pages of 64 keys).  With more than
    one split the partial results go through float32 scratch: ``scratch`` =
    (part_o [batch * n_q * n_splits * head_dim], part_ml [batch * n_q * n_splits * 2]),
    made here when it is not given.  ``cu_q``, ``kv_len`` and ``page_table`` are read before the kernel
    waits for the launch before it (they are the host's description of the step, copied in before the
    step's first kernel); ``q`` and the pages are read after.  ``v_pages`` may be ``k_pages`` itself
    (the cached row is key and value at once): a tile is then fetched once."""
    _check_sink(sink, n_kv * group)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert tuple(k_pages.shape[1:]) == (n_kv, page_size, head_dim)
    assert page_table.dtype == torch.int32 and page_table.stride(1) == 1
    assert cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    part_o = part_ml = None
    if n_splits > 1:
        n = batch * n_kv * group * n_splits
        if scratch is None:
            part_o = torch.empty(n * head_dim, dtype=torch.float32, device=q.device)
            part_ml = torch.empty(n * 2, dtype=torch.float32, device=q.device)
        else:
            part_o, part_ml = scratch
            assert part_o.numel() >= n * head_dim and part_ml.numel() >= n * 2
    f = _fn("attn_mma", "brolm_attn_decode_mma", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                  c_float, c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                  c_int, c_void_p, c_int, c_void_p])
    _check(f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cu_q), _ptr(kv_len), _ptr(k_pages), _ptr(v_pages),
             _ptr(page_table), page_table.stride(0), ring, page_size, n_kv, group, head_dim, scale, cap, window,
             _ptr(sink), batch, n_splits, _ptr(part_o), _ptr(part_ml), int(chunk), _ptr(dist_bias),
             dist_bias.shape[1] if dist_bias is not None else 0, _stream()), "attention_decode_mma")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] (int32) = first index of the maximum of logits[r] (float32)."""
    assert logits.dtype == torch.float32 and logits.is_contiguous() and out.dtype == torch.int32
    f = _fn("sampling", "brolm_argmax", [c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.shape[0], logits.shape[1], _ptr(out), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, streams: torch.Tensor,
           counter: int, out: torch.Tensor) -> None:
    """One draw per row from softmax(logits / temperature) after top-k and top-p."""
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert streams.dtype == torch.int32 and out.dtype == torch.int32 and streams.numel() == logits.shape[0]
    f = _fn("sampling", "brolm_sample", [c_void_p, c_int, c_int, c_float, c_int, c_float, c_ulonglong, c_void_p,
                                         c_ulonglong, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.shape[0], logits.shape[1], temperature, top_k, top_p, seed & (2 ** 64 - 1),
             _ptr(streams), counter, _ptr(out), _stream()), "sample")


__all__ = ["KernelBuildError", "KernelError", "build_all", "launch_count", "device_sms", "wait_control", "embed_scale",
           "embed_pairs", "concat_cast", "latent_rows", "route_topk", "route_pick", "group_tiles", "group_pairs", "experts_tc_ok", "gather_rows", "experts_linear_tc", "grouped_tc_status", "heads_linear",
           "experts_linear", "rmsnorm", "residual_rmsnorm",
           "rope_kv_write", "rope_kv_write_parts", "gated_act", "softcap", "linear_f32", "skinny_gemm", "skinny_qkv_rope", "skinny_ok", "skinny_parts", "skinny_rope_tiles", "gemm_tc", "gemm_tc2", "gemm_tc2_status", "gemm_tc_ok", "gemm_tc_status", "gemm_stream", "gemm_stream_ok", "gemm_stream_parts", "stream_rows",
           "gemm_stream_status", "attention_simt", "attention_prefill_mma", "attention_prefill_tc", "attention_prefill_tc_ok", "attention_prefill_tc_split", "attention_tc_status", "attention_decode_mma",
           "decode_splits", "argmax", "sample", "cast", "bias_act", "scaled_sum", "qkv_norm_write", "gate_group_norm",
           "experts_combine", "causal_conv", "conv_tail", "gated_scan", "ssm_scan", "block_matvec_f32", "block_matvec_ok", "split_halves"]
