"""Ritirax as a layout of parts.

Layers in the parallel arrangement with one norm (x += mixer(n(x)) + ff(n(x)), the gain stored around zero); three
kinds of mixer: attention without a rotation (a norm with a gain per query and key head, soft-capped scores, a
learned bias by distance, a sink, value heads of their own size), latent attention (a stretched rotation on the
rotated part, ordinary softmax, a sigmoid gate on the heads' results) and linear attention with a fixed decay per
head; a dense feed-forward (the square of relu) or routed experts (softmax scores, groups of which some stay open,
unnormalised scaled weights, a gated shared expert); the embedding scaled; an output matrix of its own.  Every size
and constant comes from config.json.

Tensor names: ``embed``, ``final.norm``, ``head`` and, for layer i, ``l<i>.norm1``,
``l<i>.mix.{q,k,v,q.norm,k.norm,rel,sink,o}`` (attention), ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}`` (latent attention),
``l<i>.mix.{q,k,v,g,norm,o}`` (lightning), ``l<i>.mlp.{up,down}`` (dense) or
``l<i>.mlp.{router,e<j>.{gate,up,down},shared.{gate,up,down,sg}}``.
"""
from __future__ import annotations

from ..config import RitiraxConfig, register_architecture
from ..parts import BlockSpec, EmbeddingSpec, HeadSpec, LayerCall, ModelLayout, PartSpec


REL_ROWS = 16      # rows of a distance-bias table made at random when the configuration names none (key bias_rows)


def _attention(W: int, m: dict, eps: float, p: str) -> PartSpec:
    # the table's rows are the one size that only the tensor's shape gives
    names = {n: p + n for n in ("q", "k", "v", "o", "rel", "sink")} | {"q_norm": p + "q.norm", "k_norm": p + "k.norm"}
    return PartSpec("mixer", "attention",
                    dict(hidden=W, n_q=m["heads"], n_kv=m["kv_heads"], head_dim=m["dim"], scale=float(m["scale"]),
                         softcap=float(m.get("softcap") or 0.0), v_dim=m["vdim"], qk_norm="head", qk_gain=True, eps=eps,
                         sink=True, distance_rows=int(m.get("bias_rows") or REL_ROWS), distance_rows_free=True,
                         distance_far=float(m["bias_max"])), names)


def _latent(W: int, m: dict, eps: float, p: str) -> PartSpec:
    rot = m["rot"]
    position = PartSpec("position", "rope", dict(head_dim=m["rot_dim"], theta=float(rot["base"]), rotary_dim=rot["dims"],
                                                 stretch=rot.get("scaling")))
    return PartSpec("mixer", "latent_attention",
                    dict(hidden=W, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"],
                         kv_rank=m["kv_rank"], scale=float(m["scale"]), eps=eps, window=None, sink=False,
                         position=position, gate=True),
                    {"q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv",
                     "g": p + "g", "o": p + "o"})


def _lightning(W: int, m: dict, eps: float, p: str) -> PartSpec:
    return PartSpec("mixer", "decay_attention",
                    dict(hidden=W, heads=m["heads"], dim=m["dim"], v_dim=m["vdim"], decay=tuple(m["decay"]), eps=eps,
                         activation="silu", norm=True, gate=True),
                    {n: p + n for n in ("q", "k", "v", "g", "o", "norm")})


def _feedforward(W: int, mlp: dict, p: str) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("feedforward", "dense", dict(hidden=W, inter=mlp["ff"], activation="relu2", bias=False),
                        {"up": p + "up", "down": p + "down"})
    router = mlp["router"]
    n = router["experts"]
    names = {"router": p + "router"}
    for e in range(n):
        for mat in ("gate", "up", "down"):
            names[f"e{e}.{mat}"] = f"{p}e{e}.{mat}"
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("feedforward", "gated", dict(hidden=W, inter=mlp["shared"]["ff"], activation="silu"),
                          {mat: f"{p}shared.{mat}" for mat in ("gate", "up", "down")})
        names["shared_gate"] = p + "shared.sg"
    groups = router.get("groups") or {"count": 1, "keep": 1}
    return PartSpec("feedforward", "routed_experts",
                    dict(hidden=W, inter=mlp["expert"]["ff"], experts=n, top=router["top"], activation="silu",
                         scale_input=False, router="softmax", gated=True, shared=shared, shared_gate=shared is not None,
                         groups=(groups["count"], groups["keep"]), renorm=False,
                         weight_scale=float(router.get("scale") if router.get("scale") is not None else 1.0)), names)


def ritirax_layout(cfg: RitiraxConfig) -> ModelLayout:
    W, eps = cfg.width, cfg.eps

    def norm(name: str) -> PartSpec:
        return PartSpec("norm", "rmsnorm", dict(size=W, eps=eps, offset=1.0), {"weight": name})

    blocks = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "attention":
            mixer = _attention(W, m, eps, p + "mix.")
        elif layer["type"] == "latent_attention":
            mixer = _latent(W, m, eps, p + "mix.")
        else:
            mixer = _lightning(W, m, eps, p + "mix.")
        mlp = layer.get("mlp")
        blocks.append(BlockSpec(kind="parallel_one_norm", mixer=mixer, pre_mixer_norm=norm(p + "norm1"),
                                feedforward=_feedforward(W, mlp, p + "mlp.") if mlp is not None else None))
    return ModelLayout(
        embedding=EmbeddingSpec("embed", cfg.vocab, W, scale=cfg.embedding_scale),
        blocks=blocks,
        schedule=[LayerCall(i) for i in range(len(cfg.layers))],
        final_norm=norm("final.norm"),
        head=HeadSpec("head"))


register_architecture(RitiraxConfig, ritirax_layout)
