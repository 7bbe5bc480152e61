"""Kedasun models drawn at random (layer order, head counts, head sizes that the tensor cores take and that they do not,
rotation, taps, windows and kept keys around the pages' borders, norm groups, layers without a feed-forward or without
value mixing) through a prompt step of three unequal requests and twelve tokens decoded together, twice on the same
slots, against the plain implementation, in float32 and in bfloat16."""
import os
import random

import pytest
import torch

import brolm_b200 as bb
from tests.kedasun_helpers import dense, oracle_inputs, rotary, windowed, write_folder
from tests.plain import kedasun_plain as plain
from tests.test_kedasun_gpu import STORE, check

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def draw(seed: int) -> dict:
    r = random.Random(seed)
    W = r.choice([48, 64, 96, 128, 160])
    # parts of at least 16 elements: a part of four whose elements all happen to be small is divided by a tiny root mean
    # square, and in bfloat16 the rounding of such a position is several times that of its neighbours
    groups = r.choice([g for g in (1, 2, 4, 8) if W % g == 0 and W // g >= 16])
    G = r.choice([1, 2, 3, 4, 8])
    sixteen = r.random() < 0.6                       # head sizes the tensor cores take, or others
    dims = [16, 32, 48, 64, 96] if sixteen else [8, 12, 20, 24, 40]
    vdim = r.choice(dims[:4])
    layers = []
    kinds = ["attention", "attention_2"] + [r.choice(["attention", "attention_2"]) for _ in range(r.randint(1, 3))]
    r.shuffle(kinds)
    for kind in kinds:
        H = G * r.choice([1, 2, 3, 4] if G < 8 else [1, 2])
        d = r.choice(dims)
        mlp = dense(r.choice([24, 40, 72, 136]), r.choice([0.6, 1.5, 4.0, 9.0])) if r.random() < 0.8 else None
        v_mix = r.random() < 0.75
        scale = r.uniform(0.5, 1.5) / d ** 0.5
        if kind == "attention":
            rot = r.choice([None, d, d // 2, 4, 8])
            layers.append(rotary(H, G, d, vdim, scale, rot, base=r.choice([50.0, 10000.0, 500000.0]), v_mix=v_mix, mlp=mlp))
        else:
            size = r.choice([None, 1, 7, 63, 64, 65, 100, 128, 136, 200])
            keep = r.choice([None, 0, 1, 6, 63, 64, 65, 70]) if size else None
            layers.append(windowed(H, G, d, vdim, scale * 4.0, r.choice([1, 2, 3, 4, 6]), size=size, keep_first=keep,
                                   v_mix=v_mix, mlp=mlp))
    return dict(architecture="Kedasun", vocab=r.randint(40, 300), width=W, embedding=dict(scale=r.choice([1.0, 2.0, 7.5])),
                norm=dict(eps=r.choice([1e-6, 1e-5]), groups=groups), layers=layers)


@pytest.mark.parametrize("seed", range(int(os.environ.get("BROLM_TEST_DRAWS", "10"))))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_drawn_at_random(tmp_path, seed, dtype):
    cfg = draw(seed)
    folder = write_folder(cfg, str(tmp_path / "m"), seed=100 + seed, std=0.15, store=STORE[dtype])
    config, weights = oracle_inputs(folder)
    model = bb.load_model(folder, dtype=dtype, device=DEV)
    eng = bb.Engine(model, max_tokens=1024)
    g = torch.Generator().manual_seed(seed)
    more = 12
    for again in range(2):                           # the second time slots, pages and kept inputs are used again
        lens = [230, 90, 7] if again == 0 else [3, 140, 66]
        ids = [torch.randint(0, config["vocab"], (n + more,), generator=g).tolist() for n in lens]
        refs = [plain.forward(config, weights, p) for p in ids]
        slots = eng.open(3)
        got = eng.step(slots, [p[:n] for p, n in zip(ids, lens)], want=[list(range(n)) for n in lens])
        rows = list(got.split(lens))
        tails = [[] for _ in lens]
        for t in range(more):
            out = eng.step(slots, [[p[n + t]] for p, n in zip(ids, lens)])
            for b in range(3):
                tails[b].append(out[b:b + 1].clone())
        eng.close(slots)
        for b in range(3):
            check(torch.cat([rows[b]] + tails[b]), refs[b], dtype, f"model {seed}, request of {lens[b]} + {more}")
