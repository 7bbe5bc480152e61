"""Ritirax models drawn at random (layer order, every size, head counts, tables, decays, stretches, experts, groups)
through the engine against the plain implementation: a prompt step of three unequal requests, twelve tokens one by one,
and the same once more on the slots, pages and states that were given back.  In float32 the bar of a request is the
larger of 2e-5 and eight times the error the plain implementation itself makes when it runs in float32.  In bfloat16
the drawn routers use all their experts (no discrete choice) and sizes that reach the tensor-core kernels are drawn
more often; the bar is on the typical row."""
import os
import random

import pytest
import torch

import brolm_b200 as bb
from tests.plain import ritirax_plain as plain
from tests.ritirax_helpers import attention, dense, latent, lightning, moe, oracle_inputs, random_prompts

pytestmark = pytest.mark.gpu


def draw_mlp(rng, discrete):
    kind = rng.choice(["none", "dense", "moe", "moe"])
    if kind == "none":
        return None
    if kind == "dense":
        return dense(rng.choice([8, 20, 48, 130]))
    count = rng.choice([1, 1, 2, 3, 4])
    experts = count * rng.choice([1, 2, 3])
    keep = rng.randint(1, count) if discrete else count
    top = rng.randint(1, min(keep * (experts // count), 4)) if discrete else experts
    return moe(rng.choice([8, 12, 40, 72]), experts, top, scale=rng.choice([None, 0.5, 1.75]),
               groups=(count, keep) if (count > 1 or rng.random() < 0.5) else None, shared=rng.choice([None, 8, 56]))


def draw_layer(rng, discrete, tensor_sizes):
    kind = rng.choice(["attention", "latent_attention", "lightning"])
    mlp = draw_mlp(rng, discrete)
    if kind == "attention":
        kv = rng.choice([1, 2, 3])
        d = rng.choice([16, 32, 64] if tensor_sizes else [4, 6, 8, 16, 20, 32, 64])
        dv = rng.choice([d, d, 16, 48, 80] if tensor_sizes else [d, 4, 8, 12, 32, 80])
        rows = rng.choice([2, 3, 4, 7, 8, 16, 32])
        return attention(kv * rng.choice([1, 2, 4]), kv, d, dv, rng.choice([0.1, 0.3, 1.0]), rng.choice([0.0, 5.0, 30.0]),
                         rows // 2 + rng.choice([1, 2, 7, 60, 300]), rows, mlp=mlp)
    if kind == "latent_attention":
        r = rng.choice([2, 4, 8, 16])
        scaling = rng.choice([None, (2.0, 16, 4.0, 1.0), (8.0, 64, 32.0, 1.0), (40.0, 128, 16.0, 2.0)])
        return latent(rng.choice([1, 2, 3, 5]), rng.choice([4, 6, 8, 16, 24]), r, rng.choice([4, 8, 12, 32]),
                      rng.choice([8, 12, 24, 48, 64]), rng.choice([0.1, 0.25, 0.5]), rng.choice([100.0, 10000.0]),
                      scaling=scaling, mlp=mlp)
    heads = rng.choice([1, 2, 3, 6])
    return lightning(heads, rng.choice([4, 6, 8, 20, 32, 64]), rng.choice([4, 7, 16, 32, 64]),
                     [rng.choice([0.5, 0.9, 0.97, 0.999, 1.0]) for _ in range(heads)], mlp=mlp)


def draw_config(seed, discrete=True, tensor_sizes=False):
    rng = random.Random(seed)
    return dict(architecture="Ritirax", vocab=rng.choice([37, 64, 200, 577]), width=rng.choice([24, 40, 72, 136, 312]),
                norm=dict(eps=rng.choice([1e-5, 1e-6])), embedding=dict(scale=rng.choice([0.5, 1.0, 4.0, 12.0])),
                layers=[draw_layer(rng, discrete, tensor_sizes) for _ in range(rng.randint(1, 5))])


def run_twice(folder, dtype, reqs, lens):
    eng = bb.Engine(bb.load_model(folder, dtype=dtype), max_tokens=1024, max_slots=3)
    rounds = []
    for _ in range(2):
        slots = eng.open(3)
        got = [[] for _ in reqs]
        first = eng.step(slots, [p[:n] for p, n in zip(reqs, lens)], want=[list(range(n)) for n in lens])
        at = 0
        for b, n in enumerate(lens):
            got[b].append(first[at:at + n].clone())
            at += n
        for j in range(12):
            out = eng.step(slots, [[p[n + j]] for p, n in zip(reqs, lens)])
            for b in range(3):
                got[b].append(out[b:b + 1].clone())
        eng.close(slots)
        rounds.append([torch.cat(g).cpu() for g in got])
    return rounds


@pytest.mark.parametrize("seed", range(14))
def test_a_drawn_model_prompt_decode_and_the_same_again(tmp_path, seed):
    folder = os.path.join(str(tmp_path), "drawn")
    bb.write_random_model(bb.RitiraxConfig.from_dict(draw_config(seed)), folder, seed=seed, weight_std=0.15, norm_std=0.5,
                          dtype=torch.float32)
    config, weights = oracle_inputs(folder)
    rng = random.Random(seed + 1000)
    lens = [rng.choice([1, 2, 17, 40, 66, 130, 200]) for _ in range(3)]
    reqs = random_prompts(config["vocab"], [n + 12 for n in lens], seed)
    refs = [plain.forward(config, weights, p) for p in reqs]
    plain.F64 = torch.float32
    try:
        own = [float((plain.forward(config, weights, p).double() - r).abs().max() / r.abs().max()) for p, r in zip(reqs, refs)]
    finally:
        plain.F64 = torch.float64
    bars = [max(2e-5, 8 * e) for e in own]
    rounds = run_twice(folder, "float32", reqs, lens)
    for b, (r, bar) in enumerate(zip(refs, bars)):
        err = float((rounds[0][b].double() - r).abs().max() / r.abs().max())
        assert err <= bar, f"request {b} of {lens[b]} + 12 tokens: {err:.2e} against a bar of {bar:.1e}"
        assert torch.equal(rounds[0][b], rounds[1][b]), "the second tenants of the slots see something of the first"


@pytest.mark.parametrize("seed", range(100, 108))
def test_a_drawn_model_in_bfloat16(tmp_path, seed):
    folder = os.path.join(str(tmp_path), "drawn16")
    bb.write_random_model(bb.RitiraxConfig.from_dict(draw_config(seed, discrete=False, tensor_sizes=True)), folder, seed=seed,
                          weight_std=0.15, norm_std=0.5, dtype=torch.bfloat16)
    config, weights = oracle_inputs(folder)
    rng = random.Random(seed + 1000)
    lens = [rng.choice([1, 2, 17, 40, 66, 130, 200]) for _ in range(3)]
    reqs = random_prompts(config["vocab"], [n + 12 for n in lens], seed)
    rounds = run_twice(folder, "bfloat16", reqs, lens)
    errs = []
    for b, p in enumerate(reqs):
        ref = plain.forward(config, weights, p)
        errs += ((rounds[0][b].double() - ref).abs().amax(dim=1) / ref.abs().max()).tolist()
        assert torch.equal(rounds[0][b], rounds[1][b]), "the second tenants of the slots see something of the first"
    errs.sort()
    assert errs[len(errs) // 2] <= 2e-2 and errs[int(0.9 * (len(errs) - 1))] <= 6e-2, (errs[len(errs) // 2], errs[-1])
