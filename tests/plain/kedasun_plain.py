"""Kedasun restated plainly: one function per mechanism, float64, whole sequences, quadratic attention.

Nothing here is shared with the package: the configuration is the parsed config.json (a dict), the weights a dict of
tensors by checkpoint name.  Notation: T tokens, W width, H / G query / key-value heads, d / dv key / value head sizes,
K taps.  ``F64`` can be set to float32 to see what the same arithmetic loses in 32 bits.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def grouped_rms_norm(x, gain, groups: int, eps: float):
    """x [T, W] cut into ``groups`` equal consecutive parts, each over its own sqrt(mean(part^2) + eps), times gain."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)
    return parts.reshape(T, W) * gain


def unit_heads(x, eps: float):
    """x [T, heads, d]: every head over its own root mean square, no gain."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rotate_pairs(x, base: float, dims: int):
    """x [T, heads, d]: the pair (2i, 2i + 1) of the first ``dims`` elements of a head turns by t * base^(-2i/dims)."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=F64)
    ang = torch.arange(T, dtype=F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def short_convolution(u, taps):
    """u [T, C], taps [C, K]: y_t = sum_j taps[:, j] u_(t - K + 1 + j), zeros before the start."""
    T, K = u.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, u.shape[1], dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + taps[:, j] * padded[j:j + T]
    return y


def visible(T: int, window=None, keep_first: int = 0):
    """[T, T] bool: j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def head_slopes(H: int, power: float = 8.0):
    return torch.tensor([2.0 ** (-power * (h + 1) / H) for h in range(H)], dtype=F64)


def softmax_weights(q, k, scale: float, mask, slopes=None):
    """q [T, H, d], k [T, G, d] -> [H, T, T] weights; slopes[h] * (i - j) is taken off the scaled score."""
    H, G = q.shape[1], k.shape[1]
    kk = k.repeat_interleave(H // G, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if slopes is not None:
        T = q.shape[0]
        dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(F64)
        s = s - slopes[:, None, None] * dist[None]
    s = s.masked_fill(~mask[None], -math.inf)
    return torch.softmax(s, -1)


def apply_weights(w, v, H: int):
    """w [H, T, T], v [T, G, dv] -> [T, H, dv]; head h reads kv head h // (H / G)."""
    vv = v.repeat_interleave(H // v.shape[1], 1)
    return torch.einsum("hij,jhd->ihd", w, vv)


def mix_values(v, v_first, lam):
    """v, v_first [T, G, dv] (the first layer's may be cut into heads differently: the rows are mixed flat)."""
    return (1.0 - lam) * v + lam * v_first.reshape(v.shape)


def clamped_feed_forward(h, w_gate, w_up, w_down, limit: float):
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def mixer(kind: str, m: dict, h, w: dict, p: str, eps: float, v_first):
    """One mixer on its normed input h [T, W].  Returns (result [T, W], this layer's own values or None)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    slopes = None
    if kind == "attention":
        q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
        rot = m.get("rot") or {}
        if rot.get("dims"):
            q, k = rotate_pairs(q, rot["base"], rot["dims"]), rotate_pairs(k, rot["base"], rot["dims"])
        mask = visible(T)
    else:
        q, k, v = q + w[p + "q.b"], k + w[p + "k.b"], v + w[p + "v.b"]
        q, k, v = (short_convolution(q, w[p + "q.conv"]), short_convolution(k, w[p + "k.conv"]),
                   short_convolution(v, w[p + "v.conv"]))
        q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
        q, k = unit_heads(q, eps), unit_heads(k, eps)
        window = m.get("mask") or {}
        mask = visible(T, window.get("size"), window.get("keep_first") or 0)
        slopes = head_slopes(H)
    own = None
    if m.get("v_mix"):
        if v_first is None:
            own = v
        else:
            v = mix_values(v, v_first, w[p + "vmix"])
    weights = softmax_weights(q, k, m["scale"], mask, slopes)
    if kind == "attention_2":
        weights = torch.einsum("hg,gij->hij", w[p + "talk"], weights)
    o = apply_weights(weights, v, H)
    if kind == "attention_2":
        o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    y = o.reshape(T, H * dv) @ w[p + "o"].T
    if kind == "attention_2":
        y = y + w[p + "o.b"]
    return y, own


def forward(config: dict, weights: dict, tokens, streams=None):
    """Logits [T, vocab] of one sequence; ``streams`` (a list) takes the residual stream after every layer."""
    w = {n: t.to(F64) for n, t in weights.items()}
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    x = w["embed"][torch.tensor(list(tokens))] * config["embedding"]["scale"]
    v_first = None
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        y, own = mixer(layer["type"], layer["mixer"], grouped_rms_norm(x, w[p + "norm1"], groups, eps), w, p + "mix.", eps,
                       v_first)
        if own is not None:
            v_first = own
        x = x + grouped_rms_norm(y, w[p + "norm1b"], groups, eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = grouped_rms_norm(x, w[p + "norm2"], groups, eps)
            y = clamped_feed_forward(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"], mlp["limit"])
            x = x + grouped_rms_norm(y, w[p + "norm2b"], groups, eps)
        if streams is not None:
            streams.append(x.clone())
    return grouped_rms_norm(x, w["final.norm"], groups, eps) @ w["head"].T
