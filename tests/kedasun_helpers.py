"""Shared by the Kedasun tests: small configurations that differ from one another in every size and option, model
folders with random weights (with mixing weights and head-mixing matrices large enough to matter), and the oracle's
view of them."""
from __future__ import annotations

import json
import os

import torch

import brolm_b200 as bb


def rotary(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, v_mix=True, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, v_mix=v_mix)
    if rot_dims is not None:
        m["rot"] = dict(base=base, dims=rot_dims)
    return dict(type="attention", mixer=m, mlp=mlp)


def windowed(heads, kv_heads, dim, vdim, scale, conv, size=None, keep_first=None, v_mix=True, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, conv=conv, v_mix=v_mix)
    if size is not None:
        m["mask"] = dict(size=size) if keep_first is None else dict(size=size, keep_first=keep_first)
    return dict(type="attention_2", mixer=m, mlp=mlp)


def dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


# S: grouped-query heads (4 over 2), value heads larger than key heads, half of a head rotated, three norm groups; a
# window below a page (9) that keeps three first keys, four taps; the first mixing layer is a rotary one; a layer without
# a feed-forward; a layer that mixes no values.
CFG_S = dict(
    architecture="Kedasun", vocab=96, width=48, embedding=dict(scale=2.5), norm=dict(eps=1e-5, groups=3),
    layers=[rotary(4, 2, 8, 16, 0.3, 4, mlp=dense(40, 1.5)),
            windowed(4, 2, 12, 16, 0.4, 4, size=9, keep_first=3, mlp=dense(24, 0.7)),
            rotary(4, 2, 8, 16, 0.3, 4, v_mix=False),
            windowed(2, 2, 6, 16, 0.5, 2, size=20, keep_first=1, mlp=dense(56, 3.0)),
            rotary(2, 1, 16, 32, 0.25, 16, base=500.0, mlp=dense(40, 1.5))])

# T: one norm group (the ordinary RMS norm), as many key heads as query heads, the first mixing layer is a windowed
# one (its values come out of the convolution), a window of one page exactly (64) with no kept keys, a window across
# a page border (70) that keeps more keys than a page holds (66), a convolution of one tap (no kept inputs), head
# sizes that are no multiples of 8, a whole head rotated, an embedding scale of one, sizes that are no multiples of 16.
CFG_T = dict(
    architecture="Kedasun", vocab=50, width=40, embedding=dict(scale=1.0), norm=dict(eps=1e-6, groups=1),
    layers=[windowed(3, 3, 10, 6, 0.35, 3, size=64, keep_first=0, mlp=dense(20, 1.0)),
            rotary(3, 3, 12, 6, 0.2, 12, mlp=dense(36, 2.0)),
            windowed(6, 1, 12, 18, 0.45, 1, size=70, keep_first=66, mlp=dense(28, 1.2)),
            rotary(2, 1, 20, 18, 0.3, 6, base=77.0)])

# U: key and value heads of one size that is a multiple of 16 (in bfloat16 the rotary layers run on the tensor cores),
# a layer without rotation at all, a windowed layer without a mask (every earlier key visible), a window of one (a token
# sees itself and the kept first keys), five taps, no layer mixes values, eight norm groups.
CFG_U = dict(
    architecture="Kedasun", vocab=64, width=64, embedding=dict(scale=0.5), norm=dict(eps=1e-5, groups=8),
    layers=[rotary(4, 2, 16, 16, 0.25, 8, v_mix=False, mlp=dense(32, 2.0)),
            windowed(4, 4, 8, 8, 0.4, 5, v_mix=False, mlp=dense(32, 2.0)),
            rotary(2, 2, 32, 32, 0.2, None, v_mix=False),
            windowed(2, 1, 16, 8, 0.3, 2, size=1, keep_first=2, v_mix=False, mlp=dense(24, 0.9)),
            rotary(4, 1, 16, 16, 0.25, 16, v_mix=False, mlp=dense(48, 1.1))])

# V: head sizes that are multiples of 16, keys and values of different sizes: in bfloat16 every layer's attention runs on
# the tensor cores; windows across a page's border that keep keys within and beyond the first page, several key/value
# heads under mixed weights, a rotary layer with value rows of their own size.
CFG_V = dict(
    architecture="Kedasun", vocab=80, width=64, embedding=dict(scale=1.5), norm=dict(eps=1e-5, groups=2),
    layers=[windowed(4, 2, 32, 48, 0.3, 3, size=70, keep_first=5, mlp=dense(48, 1.5)),
            rotary(4, 2, 16, 48, 0.3, 8, mlp=dense(40, 2.0)),
            windowed(6, 3, 16, 32, 0.35, 2, size=64, keep_first=66, mlp=dense(32, 1.0)),
            windowed(2, 1, 48, 16, 0.25, 4, size=130, keep_first=1, v_mix=False),
            rotary(2, 2, 32, 48, 0.25, 32, base=300.0, mlp=dense(40, 1.5))])

CONFIGS = {"S": (CFG_S, 3, 0.15), "T": (CFG_T, 4, 0.2), "U": (CFG_U, 5, 0.2), "V": (CFG_V, 6, 0.15)}      # name -> (config, seed, weight std)


def shape_up(tensors: dict, seed: int) -> dict:
    """Random weights leave a few tensors near zero that the design means to matter: the scalars that mix values become
    0.2 to 0.7, the head-mixing matrices an identity plus noise, the convolutions' newest tap about one."""
    g = torch.Generator().manual_seed(seed)
    out = dict(tensors)
    for name, t in tensors.items():
        if name.endswith(".vmix"):
            out[name] = (0.2 + 0.5 * torch.rand((), generator=g)).to(t.dtype)
        elif name.endswith(".talk"):
            out[name] = (torch.eye(t.shape[0]) + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif name.endswith(".conv"):
            w = 0.4 * torch.randn(t.shape, generator=g)
            w[:, -1] += 1.0
            out[name] = w.to(t.dtype)
    return out


def write_folder(config: dict, folder: str, seed: int, std: float, store=torch.float32) -> str:
    """config.json and model.safetensors with random weights, shaped up; returns the folder."""
    from safetensors.torch import load_file, save_file
    bb.write_random_model(bb.KedasunConfig.from_dict(config), folder, seed=seed, weight_std=std, norm_std=0.5, dtype=store)
    path = os.path.join(folder, "model.safetensors")
    save_file({n: t.contiguous() for n, t in shape_up(load_file(path), seed).items()}, path)
    return folder


def make_folder(tmp_path, name: str, store=torch.float32) -> str:
    cfg, seed, std = CONFIGS[name]
    folder = os.path.join(str(tmp_path), f"kedasun_{name}_{str(store).split('.')[-1]}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_folder(cfg, folder, seed, std, store)
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
