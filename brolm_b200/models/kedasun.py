"""Kedasun as a layout of parts.

Every layer is a sandwich: x += n1b(mixer(n1(x))), x += n2b(ff(n2(x))), all norms RMS norms taken in groups of the
row.  Two kinds of mixer, both the framework's attention part with different options:

* ``attention``: grouped-query attention with value heads of their own size, rotary positions on the first part of a
  head with the pairs (2i, 2i + 1), every earlier key visible;
* ``attention_2``: biased projections, a short causal convolution over time on q, k and v, unit-norm q and k heads,
  no rotation but a distance bias with a slope per head, a sliding window that keeps a sequence's first keys, the
  heads' softmax weights mixed by a matrix, and a gate per head on the result.

Layers that say so mix their values with those of the first such layer of the same token.  The feed-forward is gated
with the clamped pair function.  The embedding is scaled; the output matrix is a tensor of its own.  Every size and
constant of config.json is read from there; what the design fixes stands below.

Tensor names: ``embed``, ``final.norm``, ``head`` and, for layer i, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``,
``l<i>.norm2b``, ``l<i>.mix.{q,k,v,o,vmix}``, for the second kind also ``l<i>.mix.{q.b,k.b,v.b,o.b,q.conv,k.conv,
v.conv,talk,g}``, and ``l<i>.mlp.{gate,up,down}``.
"""
from __future__ import annotations

from ..config import KedasunConfig, register_architecture
from ..parts import BlockSpec, EmbeddingSpec, HeadSpec, LayerCall, ModelLayout, PartSpec

SLOPE_POWER = 8.0        # slope of head h of H: 2^(-8 (h + 1) / H); fixed by the design
V_MIX_KEY = "v_first"    # the name under which the first mixing layer leaves its values for the pass


def _mixer(cfg: KedasunConfig, i: int, p: str) -> PartSpec:
    layer = cfg.layers[i]
    m = layer["mixer"]
    W = cfg.width
    first = cfg.first_mixing_layer()
    args = dict(hidden=W, n_q=m["heads"], n_kv=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"], scale=float(m["scale"]),
                eps=cfg.eps, v_mix=(None if not m.get("v_mix") else "source" if i == first else "mixed"),
                v_mix_key=V_MIX_KEY)
    names = {n: p + n for n in ("q", "k", "v", "o")}
    if m.get("v_mix"):
        names["vmix"] = p + "vmix"
    if layer["type"] == "attention":
        rot = m.get("rot") or {}
        if rot.get("dims"):
            args["position"] = PartSpec("position", "rope", dict(head_dim=m["dim"], theta=float(rot["base"]),
                                                                 rotary_dim=rot["dims"], pairing="interleaved"))
        return PartSpec("mixer", "attention", args, names)
    mask = m.get("mask") or {}
    args.update(bias=True, taps=m["conv"], qk_norm="head", slope_power=SLOPE_POWER, window=mask.get("size"),
                keep_first=mask.get("keep_first") or 0, talk=True, gate=True)
    names.update({"q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b", "o_bias": p + "o.b",
                  "q_conv": p + "q.conv", "k_conv": p + "k.conv", "v_conv": p + "v.conv", "talk": p + "talk",
                  "gate": p + "g"})
    return PartSpec("mixer", "attention", args, names)


def kedasun_layout(cfg: KedasunConfig) -> ModelLayout:
    W = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("norm", "rmsnorm", dict(size=W, eps=cfg.eps, offset=0.0, groups=cfg.norm_groups), {"weight": name})

    blocks, unused = [], {}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mlp = layer.get("mlp")
        ff = None
        if mlp is not None:
            ff = PartSpec("feedforward", "gated", dict(hidden=W, inter=mlp["ff"], activation="clamped_gate",
                                                       limit=float(mlp["limit"])),
                          {n: f"{p}mlp.{n}" for n in ("gate", "up", "down")})
        else:
            unused.update({p + "norm2": (W,), p + "norm2b": (W,)})       # norms of a sublayer that is not there
        if not layer["mixer"].get("v_mix"):
            unused[p + "mix.vmix"] = ()
        blocks.append(BlockSpec(mixer=_mixer(cfg, i, p + "mix."), feedforward=ff,
                                pre_mixer_norm=norm(p + "norm1"), post_mixer_norm=norm(p + "norm1b"),
                                pre_ffn_norm=norm(p + "norm2") if ff is not None else None,
                                post_ffn_norm=norm(p + "norm2b") if ff is not None else None))
    return ModelLayout(
        embedding=EmbeddingSpec("embed", cfg.vocab, W, scale=cfg.embedding_scale),
        blocks=blocks,
        schedule=[LayerCall(i) for i in range(len(cfg.layers))],
        final_norm=norm("final.norm"),
        head=HeadSpec("head"),
        unused_tensors=unused)


register_architecture(KedasunConfig, kedasun_layout)
