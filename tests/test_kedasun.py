"""Kedasun without a GPU: configuration, layout, tensor names, what the cache keeps and where, the oracle's own
consistency."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import brolm_b200 as bb
from brolm_b200.cache import Cache, CacheEntries, KVSpec, StateSpec
from brolm_b200.config import ConfigError
from tests.kedasun_helpers import CFG_S, CFG_T, CFG_U, make_folder, oracle_inputs, random_prompts
from tests.plain import kedasun_plain as plain


def test_config_is_chosen_by_its_architecture_key(tmp_path):
    path = os.path.join(str(tmp_path), "config.json")
    with open(path, "w") as fh:
        json.dump(CFG_S, fh)
    cfg = bb.load_config(path)
    assert isinstance(cfg, bb.KedasunConfig) and cfg.width == 48 and len(cfg.layers) == 5
    assert bb.KedasunConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.norm_groups == 3 and cfg.embedding_scale == 2.5 and cfg.first_mixing_layer() == 0
    assert bb.KedasunConfig.from_dict(CFG_T).first_mixing_layer() == 0
    assert bb.KedasunConfig.from_dict(CFG_U).first_mixing_layer() is None


@pytest.mark.parametrize("edit,what", [
    (lambda c: c["layers"][0].update(type="other"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].pop("base"), "base"),
    (lambda c: c["layers"][0]["mixer"].update(scale=0.0), "scale"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][1]["mixer"].update(v_mix="yes"), "v_mix"),
    (lambda c: c["layers"][4]["mixer"].update(vdim=16), "mixes values"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c.pop("embedding"), "embedding"),
])
def test_bad_configurations_are_named(edit, what):
    c = copy.deepcopy(CFG_S)
    edit(c)
    with pytest.raises(ConfigError) as e:
        bb.KedasunConfig.from_dict(c)
    assert what in str(e.value)


def test_layout_names_and_caches():
    m = bb.Model(bb.KedasunConfig.from_dict(CFG_S), dtype="float32", device="cpu")
    names = m.expected_tensors()
    for n in ("embed", "head", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.q", "l0.mix.vmix",
              "l0.mix.o", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down", "l1.mix.q.b", "l1.mix.k.b", "l1.mix.v.b", "l1.mix.o.b",
              "l1.mix.q.conv", "l1.mix.k.conv", "l1.mix.v.conv", "l1.mix.talk", "l1.mix.g", "l1.mix.vmix"):
        assert n in names and not names[n].optional, n
    assert "l0.mix.q.b" not in names and "l0.mix.talk" not in names and "l2.mlp.gate" not in names
    # what a checkpoint may carry although nothing reads it
    for n in ("l2.norm2", "l2.norm2b", "l2.mix.vmix"):
        assert names[n].optional
    assert names["l0.mix.q"].shape == (32, 48) and names["l0.mix.v"].shape == (32, 48) and names["l0.mix.o"].shape == (48, 64)
    assert names["l1.mix.q.conv"].shape == (48, 4) and names["l1.mix.v.conv"].shape == (32, 4)
    assert names["l1.mix.talk"].shape == (4, 4) and names["l1.mix.g"].shape == (4, 48) and names["l1.mix.vmix"].shape == ()
    assert names["head"].shape == (96, 48) and names["l0.mlp.gate"].shape == (40, 48)
    specs = m.cache_specs()
    assert specs[0] == KVSpec(2, 8, None, v_dim=16)
    kv, state = specs[1]
    assert kv == KVSpec(2, 12, 9, v_dim=16, keep_first=3) and state == StateSpec((3 * (48 + 24 + 32),), torch.float32)
    # one tap keeps no inputs: the state is a single unused number
    t = bb.Model(bb.KedasunConfig.from_dict(CFG_T), dtype="float32", device="cpu").cache_specs()
    assert t[2][0] == KVSpec(1, 12, 70, v_dim=18, keep_first=66) and t[2][1] == StateSpec((1,), torch.float32)
    # a windowed layer without a mask keeps every key and no first ones
    u = bb.Model(bb.KedasunConfig.from_dict(CFG_U), dtype="float32", device="cpu").cache_specs()
    assert u[1][0] == KVSpec(4, 8, None) and u[3][0] == KVSpec(1, 16, 1, v_dim=8, keep_first=2)


def test_random_folder_has_every_tensor_and_loads_on_the_cpu_reader(tmp_path):
    folder = make_folder(tmp_path, "S")
    config, weights = oracle_inputs(folder)
    m = bb.Model(bb.KedasunConfig.from_dict(config), dtype="float32", device="cpu")
    need = {n for n, e in m.expected_tensors().items() if not e.optional}
    assert need == set(weights)
    assert weights["l1.mix.vmix"].shape == () and 0.2 <= float(weights["l1.mix.vmix"]) <= 0.7


def test_kept_first_places_stay_ahead_of_the_ring():
    """Positions below the kept head live at their own place for good; the ring begins behind them."""
    cache = Cache([(KVSpec(1, 8, 70, keep_first=66), StateSpec((4,), torch.float32)), KVSpec(1, 8, 70)], 2048,
                  torch.float32, "cpu", max_slots=2)
    assert isinstance(cache.entries[0], CacheEntries)
    g = cache.entries[0].parts[0].group
    assert g.head == 128 and g.ring == 128 and g.pages_for(5) == 1 and g.pages_for(1000) == 4
    pos = np.arange(0, 700)
    place = g.place(pos)
    assert (place[:128] == pos[:128]).all() and (place[128:] >= 128).all() and place.max() == 255
    assert g.place(128 + 128) == 128 and g.place(127) == 127 and g.place(128 + 129) == 129
    # any 70 consecutive positions beyond the head occupy 70 different places
    for a in (128, 200, 500):
        assert len(set(place[a:a + 70].tolist())) == 70
    plain_ring = cache.entries[1].group
    assert plain_ring.head == 0 and plain_ring.place(300) == 300 % 128


def test_rows_of_a_prompt_longer_than_head_and_ring():
    cache = Cache([KVSpec(1, 8, 20, keep_first=3)], 1024, torch.float32, "cpu", max_slots=2)
    g = cache.kv_groups[0]
    assert g.head == 64 and g.ring == 64
    slot = cache.alloc_slot()
    cache.reserve({slot: 300})
    rows = cache.write_rows(0, [slot], [0], [300])
    pages = g.pages[slot]
    assert len(pages) == 2
    kept = rows >= 0
    # the first page's places are all written; of the rest only the newest ring's worth
    assert kept[:64].all() and not kept[64:300 - 64].any() and kept[300 - 64:].all()
    assert (rows[:64] == pages[0] * 64 + np.arange(64)).all()
    assert len(set(rows[kept].tolist())) == int(kept.sum())


def test_oracle_is_causal_and_its_window_has_the_edges_it_should():
    mask = plain.visible(12, window=4, keep_first=2)
    assert mask[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert mask[3].tolist() == [True] * 4 + [False] * 8 and mask[5].tolist() == [True, True, True, True, True, True] + [False] * 6
    assert plain.visible(5)[4].all() and not plain.visible(5)[0, 1:].any()
    assert plain.visible(6, window=1, keep_first=0).int().sum() == 6


def test_oracle_prefix_logits_do_not_depend_on_what_follows(tmp_path):
    folder = make_folder(tmp_path, "S")
    config, weights = oracle_inputs(folder)
    p = random_prompts(config["vocab"], [40], seed=1)[0]
    whole = plain.forward(config, weights, p)
    part = plain.forward(config, weights, p[:17])
    assert torch.allclose(whole[:17], part, atol=1e-12)


def test_oracle_mechanisms_alone():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 12, generator=g, dtype=torch.float64)
    w = torch.randn(12, generator=g, dtype=torch.float64)
    y = plain.grouped_rms_norm(x, w, 3, 1e-5)
    for part in range(3):
        a = x[:, 4 * part:4 * part + 4]
        assert torch.allclose(y[:, 4 * part:4 * part + 4], a / torch.sqrt(a.pow(2).mean(-1, keepdim=True) + 1e-5) * w[4 * part:4 * part + 4])
    # a rotation keeps every pair's length and leaves the unrotated rest alone; position 0 is unchanged
    q = torch.randn(7, 2, 10, generator=g, dtype=torch.float64)
    r = plain.rotate_pairs(q, 100.0, 6)
    assert torch.equal(r[..., 6:], q[..., 6:]) and torch.allclose(r[0], q[0])
    assert torch.allclose(r[..., 0:6:2] ** 2 + r[..., 1:6:2] ** 2, q[..., 0:6:2] ** 2 + q[..., 1:6:2] ** 2)
    # the score of rotated q and k depends on the distance alone
    one = torch.randn(1, 1, 6, generator=g, dtype=torch.float64).expand(9, 1, 6).contiguous()
    rq = plain.rotate_pairs(one, 50.0, 6)
    s = torch.einsum("ihd,jhd->ij", rq, rq)
    assert torch.allclose(s[5, 2], s[8, 5]) and torch.allclose(s[3, 3], s[0, 0])
    # the newest tap weighs the token itself, the oldest the token taps - 1 back
    u = torch.randn(6, 3, generator=g, dtype=torch.float64)
    taps = torch.randn(3, 4, generator=g, dtype=torch.float64)
    c = plain.short_convolution(u, taps)
    assert torch.allclose(c[0], taps[:, 3] * u[0])
    assert torch.allclose(c[4], taps[:, 3] * u[4] + taps[:, 2] * u[3] + taps[:, 1] * u[2] + taps[:, 0] * u[1])
    slopes = plain.head_slopes(4)
    assert torch.allclose(slopes, torch.tensor([0.25, 0.0625, 2.0 ** -6, 2.0 ** -8], dtype=torch.float64))
    # mixed heads' weights: an identity matrix changes nothing, a swap exchanges the heads' weights but not their values
    wts = torch.softmax(torch.randn(2, 4, 4, generator=g, dtype=torch.float64), -1)
    v = torch.randn(4, 2, 3, generator=g, dtype=torch.float64)
    swap = torch.tensor([[0.0, 1.0], [1.0, 0.0]], dtype=torch.float64)
    o = plain.apply_weights(torch.einsum("hg,gij->hij", swap, wts), v, 2)
    assert torch.allclose(o[:, 0], torch.einsum("ij,jd->id", wts[1], v[:, 0]))
    ff = plain.clamped_feed_forward(torch.tensor([[10.0, -10.0]], dtype=torch.float64), torch.eye(2, dtype=torch.float64),
                                    torch.eye(2, dtype=torch.float64), torch.eye(2, dtype=torch.float64), 2.0)
    assert torch.allclose(ff[0, 0], torch.tensor(2.0 * (1 / (1 + np.exp(-3.404))) * 3.0, dtype=torch.float64))
    assert torch.allclose(ff[0, 1], torch.tensor(-10.0 * (1 / (1 + np.exp(17.02))) * -1.0, dtype=torch.float64))
