"""Shared by the Ritirax tests: small configurations that differ from one another in every size and option,
model folders with random weights, and the oracle's view of them."""
from __future__ import annotations

import json
import os

import torch

import brolm_b200 as bb


def lightning(heads, dim, vdim, decay, mlp=None):
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay)), mlp=mlp)


def attention(heads, kv_heads, dim, vdim, scale, softcap, bias_max, bias_rows, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, bias_max=bias_max, bias_rows=bias_rows)
    if softcap:
        m["softcap"] = softcap
    return dict(type="attention", mixer=m, mlp=mlp)


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, scaling=None, mlp=None):
    rot = dict(base=base, dims=rot_dim)
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return dict(type="latent_attention", mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank,
                                                    scale=scale, rot=rot), mlp=mlp)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, top, scale=None, groups=None, shared=None):
    router = dict(experts=experts, top=top)
    if scale is not None:
        router["scale"] = scale
    if groups:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    d = dict(kind="moe", expert=dict(ff=ff), router=router)
    if shared:
        d["shared"] = dict(ff=shared)
    return d


# S: every routed layer uses all of its experts and keeps all of its groups, so nothing hangs on a discrete choice
# and a rounded run can be held against the oracle.  Key and value heads of unequal sizes both ways, a layer without
# a feed-forward, a decay of one half beside one close to 1, a table of 8 rows that ends at distance 40.
CFG_S = dict(
    architecture="Ritirax", vocab=96, width=48, norm=dict(eps=1e-5), embedding=dict(scale=3.0),
    layers=[lightning(3, 8, 16, (0.5, 0.9, 0.99), mlp=dense(40)),
            attention(4, 2, 16, 8, 0.3, 20.0, 40, 8, mlp=moe(24, 3, 3, scale=1.5, shared=16)),
            latent(2, 8, 8, 16, 24, 0.3, 100.0, scaling=(2.0, 32, 8.0, 1.0), mlp=moe(24, 4, 4, scale=0.7, groups=(2, 2))),
            lightning(3, 8, 16, (0.5, 0.9, 0.99))])

# T: real routing (3 of 6 in 2 of 3 groups; 1 of 4 in groups of one expert that all stay open, no scale, no shared
# expert), as many key heads as
# query heads, head sizes that are no multiples of 8 or of 4, no soft cap, a table with an odd number of rows, a rotated
# part smaller than the unrotated one and no stretching, one lightning head, sizes that are no multiples of 16.
CFG_T = dict(
    architecture="Ritirax", vocab=50, width=40, norm=dict(eps=1e-6), embedding=dict(scale=0.5),
    layers=[attention(3, 3, 12, 20, 0.25, 0.0, 25, 7, mlp=moe(20, 6, 3, scale=2.0, groups=(3, 2), shared=12)),
            lightning(1, 6, 12, (0.97,), mlp=moe(36, 4, 1, groups=(4, 4))),
            latent(3, 12, 4, 8, 20, 0.2, 10000.0, mlp=dense(56)),
            attention(6, 1, 8, 8, 0.35, 5.0, 300, 12, mlp=dense(24))])

# U: distances far into the logarithmic rows and beyond the last (a table of 32 rows that ends at 200, prompts of 300),
# positions far beyond the stretch's original length, key and value heads of one size that is a multiple of 16, a decay
# of exactly 1 and one of 0.999 over hundreds of tokens; every routed layer uses all of its experts, so that a rounded
# run can be held against the oracle here too.
CFG_U = dict(
    architecture="Ritirax", vocab=64, width=32, norm=dict(eps=1e-5), embedding=dict(scale=5.5),
    layers=[latent(4, 16, 16, 16, 32, 0.18, 1000.0, scaling=(8.0, 64, 16.0, 2.0), mlp=moe(16, 4, 4, scale=1.0, groups=(2, 2))),
            attention(4, 1, 32, 32, 0.18, 25.0, 200, 32, mlp=dense(24)),
            lightning(2, 32, 64, (0.999, 1.0), mlp=moe(16, 2, 2, scale=3.0, shared=24)),
            attention(2, 2, 16, 48, 0.25, 0.0, 9, 4)])

CONFIGS = {"S": (CFG_S, 3, 0.15), "T": (CFG_T, 4, 0.2), "U": (CFG_U, 5, 0.2)}      # name -> (config, seed, weight std)


def make_folder(tmp_path, name: str, store=torch.float32) -> str:
    cfg, seed, std = CONFIGS[name]
    folder = os.path.join(str(tmp_path), f"ritirax_{name}_{str(store).split('.')[-1]}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        bb.write_random_model(bb.RitiraxConfig.from_dict(cfg), folder, seed=seed, weight_std=std, norm_std=0.5,
                              dtype=store)
    return folder


def oracle_inputs(folder: str):
    """(config dict, {name: tensor}) read without the framework's own reader."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as fh:
        config = json.load(fh)
    return config, load_file(os.path.join(folder, "model.safetensors"))


def random_prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
