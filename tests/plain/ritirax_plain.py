"""Ritirax restated plainly: whole sequences, float64, one function per mechanism.

Nothing here is shared with the package: the functions take the tensors of a checkpoint by name (a dict
of float64 tensors) and the configuration as the dict config.json holds.  Notation: T tokens, W width,
x the residual stream (T, W), n the input of a layer's two sublayers (the normed stream).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def layer_norm(x, gain, eps):
    """The layers' norm: the gain is stored around zero."""
    return unit_rms(x, eps) * (1.0 + gain)


# --- the distance bias of the soft-capped attention -----------------------------------------------------------
def distance_bucket(n: int, rows: int, far: float) -> int:
    """Which row of the bias table a key n places back reads: exact below rows/2, logarithmic steps up to
    ``far`` behind that, the last row for everything further."""
    half = rows // 2
    if n < half:
        return n
    step = math.floor(math.log(n / half) / math.log(far / half) * (rows - half))
    return min(rows - 1, half + step)


def biased_attention(q, k, v, scale, cap, rel, far, sink, first=0):
    """q (Tq, H, d) at positions first, first + 1, ...; k (Tk, G, d), v (Tk, G, dv) at positions 0, 1, ...;
    rel (rows, H) or None; sink (H,) or None.  Returns (Tq, H, dv)."""
    Tq, H, _ = q.shape
    Tk, G, _ = k.shape
    i = torch.arange(Tq)[:, None] + first
    j = torch.arange(Tk)[None, :]
    seen = j <= i
    which = None
    if rel is not None:
        rows = rel.shape[0]
        which = torch.tensor([[distance_bucket(int(a) - b, rows, far) if b <= int(a) else 0 for b in range(Tk)]
                              for a in i[:, 0]])
    outs = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        if which is not None:
            s = s + rel[which, h]
        s = s.masked_fill(~seen, float("-inf"))
        top = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[h])
        e = torch.exp(s - top)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - top)
        outs.append((e / den) @ v[:, g])
    return torch.stack(outs, dim=1)


def capped_attention(n, t, p, m, eps):
    """Grouped-query attention without a rotation: per-head RMS norm of q and k, a tanh cap on the scaled
    score, a learned bias by distance, every earlier key visible, and a sink in the softmax's denominator."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = n.shape[0]
    q = unit_rms((n @ t[p + "q"].T).view(T, H, d), eps) * t[p + "q.norm"]
    k = unit_rms((n @ t[p + "k"].T).view(T, G, d), eps) * t[p + "k.norm"]
    v = (n @ t[p + "v"].T).view(T, G, dv)
    o = biased_attention(q, k, v, m["scale"], m.get("softcap") or 0.0, t[p + "rel"], m["bias_max"], t[p + "sink"])
    return o.reshape(T, H * dv) @ t[p + "o"].T


# --- rotation with stretched frequencies ------------------------------------------------------------------------
def stretched_angles(T: int, rot: dict):
    """(cos, sin) of shape (T, dims/2) with YaRN's blend of stretched and plain frequencies, both already
    multiplied by its magnitude factor."""
    dims, base = rot["dims"], float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def where(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(where(float(sc["fast"]))), 0)
        hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    a = torch.arange(T, dtype=F64)[:, None] * f[None, :]
    return torch.cos(a) * mag, torch.sin(a) * mag


def rotate_half(x, cos, sin):
    """x (T, ..., r): dimension i pairs with i + dims/2 over the first dims = 2 * cos.shape[1] entries."""
    half = cos.shape[1]
    u, v, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    while cos.dim() < u.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], dim=-1)


def latent_attention(n, t, p, m, eps):
    """Keys and values of all heads expanded from one small normed row per token, one rotated key part for
    all heads, ordinary softmax, and a sigmoid gate on the heads' results."""
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = n.shape[0]
    q = (n @ t[p + "q"].T).view(T, H, d + r)
    down = n @ t[p + "dkv"].T
    c = unit_rms(down[:, :R], eps) * t[p + "dkv.norm"]
    cos, sin = stretched_angles(T, m["rot"])
    k_rot = rotate_half(down[:, R:], cos, sin)                     # (T, r)
    q_rot = rotate_half(q[..., d:], cos, sin)                      # (T, H, r)
    k_plain = (c @ t[p + "uk"].T).view(T, H, d)
    v = (c @ t[p + "uv"].T).view(T, H, dv)
    seen = torch.tril(torch.ones(T, T, dtype=torch.bool))
    outs = []
    for h in range(H):
        s = (q[:, h, :d] @ k_plain[:, h].T + q_rot[:, h] @ k_rot.T) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        outs.append(torch.softmax(s, dim=-1) @ v[:, h])
    o = torch.cat(outs, dim=-1) * torch.sigmoid(n @ t[p + "g"].T)
    return o @ t[p + "o"].T


def decay_recurrence(q, k, v, decay, S=None):
    """q, k (T, H, d), v (T, H, dv), decay (H,): S <- decay S + k v^T, o = S^T q, token by token.
    Returns (o (T, H, dv), the last S (H, d, dv))."""
    T, H, d = q.shape
    if S is None:
        S = torch.zeros(H, d, v.shape[-1], dtype=q.dtype)
    rows = []
    for i in range(T):
        S = decay[:, None, None] * S + k[i][:, :, None] * v[i][:, None, :]
        rows.append(torch.einsum("hdv,hd->hv", S, q[i]))
    return torch.stack(rows), S


def lightning(n, t, p, m, eps):
    """Linear attention with one fixed decay per head, a norm over all heads' results together, a sigmoid gate."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = n.shape[0]
    q = silu(n @ t[p + "q"].T).view(T, H, d)
    k = silu(n @ t[p + "k"].T).view(T, H, d)
    v = silu(n @ t[p + "v"].T).view(T, H, dv)
    o, _ = decay_recurrence(q, k, v, torch.tensor(m["decay"], dtype=F64))
    o = unit_rms(o.reshape(T, H * dv), eps) * t[p + "norm"]
    return (o * torch.sigmoid(n @ t[p + "g"].T)) @ t[p + "o"].T


# --- feed-forwards ---------------------------------------------------------------------------------------------
def dense_ff(n, t, p):
    return torch.relu(n @ t[p + "up"].T) ** 2 @ t[p + "down"].T


def gated_ff(n, t, p):
    return (silu(n @ t[p + "gate"].T) * (n @ t[p + "up"].T)) @ t[p + "down"].T


def choose_experts(s, top: int, groups: int, keep: int):
    """s (E,) scores of one token -> the chosen experts: the ``top`` largest among the experts of the ``keep``
    groups of neighbours whose best score is largest (ties: the lower index)."""
    E = s.numel()
    size = E // groups
    best = [max(float(s[g * size + j]) for j in range(size)) for g in range(groups)]
    kept = sorted(range(groups), key=lambda g: (-best[g], g))[:keep]
    open_to = [e for e in range(E) if e // size in kept]
    return sorted(open_to, key=lambda e: (-float(s[e]), e))[:top]


def routed_ff(n, t, p, mlp):
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.softmax(n @ t[p + "router"].T, dim=-1)
    out = torch.zeros_like(n)
    for i in range(n.shape[0]):
        for e in choose_experts(s[i], top, grp["count"], grp["keep"]):
            out[i] += float(r.get("scale", 1.0)) * s[i, e] * gated_ff(n[i:i + 1], t, f"{p}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(n @ t[p + "shared.sg"].T) * gated_ff(n, t, p + "shared.")
    return out


# --- the model ----------------------------------------------------------------------------------------------------
MIXERS = {"attention": capped_attention, "latent_attention": latent_attention, "lightning": lightning}


def forward(config: dict, tensors: dict, tokens, streams=None):
    """Logits (T, vocab) of one sequence; ``streams`` (a list) receives the residual stream after every layer."""
    t = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = t["embed"][torch.tensor(tokens)] * float(config["embedding"]["scale"])
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        n = layer_norm(x, t[p + "norm1"], eps)
        y = MIXERS[layer["type"]](n, t, p + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + (dense_ff(n, t, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(n, t, p + "mlp.", mlp))
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, t["final.norm"], eps) @ t["head"].T
