"""Ritirax without a GPU: configuration, layout, tensor names, what the cache keeps, a size left to the checkpoint's
tensor, the tables the parts build on the host, and the oracle's own consistency."""
import copy
import json
import math
import os

import pytest
import torch

import brolm_b200 as bb
from brolm_b200.cache import KVSpec, StateSpec
from brolm_b200.config import ConfigError
from brolm_b200.parts import RotaryEmbedding
from brolm_b200.parts.attention import distance_buckets
from brolm_b200.weights import WeightsError
from tests.ritirax_helpers import CFG_S, make_folder, oracle_inputs
from tests.plain import ritirax_plain as plain


def test_config_is_chosen_by_its_architecture_key(tmp_path):
    path = os.path.join(str(tmp_path), "config.json")
    with open(path, "w") as fh:
        json.dump(CFG_S, fh)
    cfg = bb.load_config(path)
    assert isinstance(cfg, bb.RitiraxConfig) and cfg.width == 48 and len(cfg.layers) == 4
    assert bb.RitiraxConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.embedding_scale == 3.0 and cfg.eps == 1e-5


@pytest.mark.parametrize("edit,what", [
    (lambda c: c["layers"][0].update(type="other"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.9]), "decay"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.9, 1.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("bias_max"), "bias_max"),
    (lambda c: c["layers"][1]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=4), "top"),
    (lambda c: c["layers"][2]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][2]["mlp"]["router"]["groups"].update(keep=1), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="other"), "kind"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.pop("embedding"), "scale"),
])
def test_bad_configurations_are_named(edit, what):
    c = copy.deepcopy(CFG_S)
    edit(c)
    with pytest.raises(ConfigError) as e:
        bb.RitiraxConfig.from_dict(c)
    assert what in str(e.value)


def test_layout_names_and_caches():
    m = bb.Model(bb.RitiraxConfig.from_dict(CFG_S), dtype="float32", device="cpu")
    names = m.expected_tensors()
    for n in ("embed", "head", "final.norm", "l0.norm1", "l0.mix.q", "l0.mix.g", "l0.mix.norm", "l0.mlp.up", "l0.mlp.down",
              "l1.mix.q.norm", "l1.mix.k.norm", "l1.mix.rel", "l1.mix.sink", "l1.mlp.router", "l1.mlp.e2.gate",
              "l1.mlp.shared.up", "l1.mlp.shared.sg", "l2.mix.dkv", "l2.mix.dkv.norm", "l2.mix.uk", "l2.mix.uv", "l2.mix.g",
              "l2.mlp.e3.down", "l3.mix.o"):
        assert n in names, n
    assert not any(n.endswith("norm2") for n in names)                   # one norm a layer
    assert not any(n.startswith("l3.mlp") for n in names) and "l2.mlp.shared.sg" not in names
    assert names["l1.mix.q"].shape == (64, 48) and names["l1.mix.v"].shape == (16, 48) and names["l1.mix.o"].shape == (48, 32)
    assert names["l1.mix.q.norm"].shape == (16,) and names["l1.mix.sink"].shape == (4,)
    assert names["l1.mix.rel"].shape == (-8, 4)                          # the rows are the tensor's to say
    assert names["l2.mix.q"].shape == (32, 48) and names["l2.mix.dkv"].shape == (32, 48) and names["l2.mix.g"].shape == (32, 48)
    assert names["l1.mlp.shared.sg"].shape == (1, 48) and not names["head"].optional
    specs = m.cache_specs()
    assert specs[0] == StateSpec((3 * 16 * 8,), torch.float32) and specs[3] == specs[0]
    assert specs[1] == KVSpec(2, 16, None, v_dim=8)
    assert specs[2] == KVSpec(1, 32, None, values=False)                  # the latent row: 24 + 8


def test_the_bias_tables_rows_come_from_the_tensor(tmp_path):
    """A checkpoint whose table has other rows than a random model would get loads; a wrong second size does not."""
    folder = make_folder(tmp_path, "S")
    config, weights = oracle_inputs(folder)
    cfg = bb.RitiraxConfig.from_dict(config)
    weights["l1.mix.rel"] = torch.randn(14, 4)
    bb.Model(cfg, dtype="float32", device="cpu").load_weights(weights)
    weights["l1.mix.rel"] = torch.randn(14, 5)
    with pytest.raises(WeightsError) as e:
        bb.Model(cfg, dtype="float32", device="cpu").load_weights(weights)
    assert "l1.mix.rel" in str(e.value)


@pytest.mark.parametrize("rows,far", [(8, 40.0), (7, 25.0), (32, 200.0), (4, 9.0), (12, 300.0), (16, 128.0), (2, 1.5)])
def test_rows_by_distance_against_the_oracle(rows, far):
    table = distance_buckets(rows, far)
    assert table[-1] == rows - 1 and rows - 1 not in table[:-1]
    for n in range(len(table) + 50):
        assert plain.distance_bucket(n, rows, far) == table[min(n, len(table) - 1)], n
    assert table[:rows // 2] == list(range(rows // 2)) and table == sorted(table)
    assert len(table) - 1 <= math.ceil(far)


@pytest.mark.parametrize("rot", [dict(base=100.0, dims=8, scaling=dict(factor=2.0, original=32, fast=8.0, slow=1.0)),
                                 dict(base=10000.0, dims=4),
                                 dict(base=1000.0, dims=16, scaling=dict(factor=8.0, original=64, fast=16.0, slow=2.0)),
                                 dict(base=10000.0, dims=64, scaling=dict(factor=40.0, original=4096, fast=32.0, slow=1.0))])
def test_stretched_rotation_table_against_the_oracle(rot):
    part = RotaryEmbedding(head_dim=rot["dims"], theta=rot["base"], rotary_dim=rot["dims"], stretch=rot.get("scaling"))
    part.prepare(700, torch.device("cpu"))
    cos, sin = plain.stretched_angles(700, rot)
    assert torch.allclose(part.table[..., 0].double(), cos, atol=1e-6) and torch.allclose(part.table[..., 1].double(), sin, atol=1e-6)
    if rot.get("scaling"):
        plainer = plain.stretched_angles(700, dict(base=rot["base"], dims=rot["dims"]))[0]
        assert float((cos - plainer).abs().max()) > 0.05                  # the stretch is not a no-op


def test_oracle_is_causal_and_its_parts_add_up():
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        folder = make_folder(tmp, "T")
        config, weights = oracle_inputs(folder)
    g = torch.Generator().manual_seed(5)
    p = torch.randint(0, config["vocab"], (60,), generator=g).tolist()
    full = plain.forward(config, weights, p)
    assert torch.allclose(plain.forward(config, weights, p[:37]), full[:37], atol=1e-9)
    assert full.shape == (60, config["vocab"]) and bool(torch.isfinite(full).all())


def test_oracle_recurrence_against_its_quadratic_form():
    g = torch.Generator().manual_seed(1)
    T, H, d, dv = 40, 3, 6, 5
    q, k = torch.randn(T, H, d, generator=g, dtype=torch.float64), torch.randn(T, H, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, H, dv, generator=g, dtype=torch.float64)
    decay = torch.tensor([0.5, 0.97, 1.0], dtype=torch.float64)
    o, S = plain.decay_recurrence(q, k, v, decay)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    for h in range(H):
        w = (q[:, h] @ k[:, h].T) * torch.where(j <= i, decay[h] ** (i - j).clamp(min=0).double(), torch.zeros(()).double())
        assert torch.allclose(w @ v[:, h], o[:, h], atol=1e-10)
    a, Sa = plain.decay_recurrence(q[:25], k[:25], v[:25], decay)
    b, Sb = plain.decay_recurrence(q[25:], k[25:], v[25:], decay, Sa)
    assert torch.allclose(torch.cat([a, b]), o, atol=1e-12) and torch.allclose(Sb, S, atol=1e-12)


def test_oracle_choice_of_experts():
    s = torch.tensor([0.05, 0.30, 0.02, 0.03, 0.25, 0.20, 0.10, 0.05])
    assert plain.choose_experts(s, 3, 1, 1) == [1, 4, 5]
    # groups of two: best scores 0.30, 0.03, 0.25, 0.10 -> groups 0 and 2 stay open
    assert plain.choose_experts(s, 3, 4, 2) == [1, 4, 5]
    assert plain.choose_experts(s, 4, 4, 2) == [1, 4, 5, 0]
    # groups of four: 0.30 and 0.25; one group open: only experts 0 .. 3
    assert plain.choose_experts(s, 3, 2, 1) == [1, 0, 3]
    assert plain.choose_experts(torch.tensor([0.25, 0.25, 0.25, 0.25]), 2, 2, 1) == [0, 1]      # ties: the lower index


def test_oracle_distance_bias_sink_and_cap_show():
    """One key that carries the weight: moving it one row of the table on, adding a sink or a cap changes the result."""
    g = torch.Generator().manual_seed(2)
    T, H, d = 30, 2, 8
    k = torch.randn(T, 1, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, 1, 4, generator=g, dtype=torch.float64)
    q = torch.zeros(T, H, d, dtype=torch.float64)
    q[-1] = 4.0 * k[10, 0]
    rel = torch.zeros(6, H, dtype=torch.float64)
    base = plain.biased_attention(q, k, v, 1.0, 0.0, rel, 25.0, None)[-1]
    rel2 = rel.clone()
    rel2[plain.distance_bucket(19, 6, 25.0)] = -50.0                       # the far key's row
    assert float((plain.biased_attention(q, k, v, 1.0, 0.0, rel2, 25.0, None)[-1] - base).abs().max()) > 0.1
    sunk = plain.biased_attention(q, k, v, 1.0, 0.0, rel, 25.0, torch.tensor([60.0, -60.0], dtype=torch.float64))[-1]
    assert float(sunk[0].abs().max()) < 1e-6 and torch.allclose(sunk[1], base[1], atol=1e-9)
    capped = plain.biased_attention(q, k, v, 1.0, 2.0, rel, 25.0, None)[-1]
    assert float((capped - base).abs().max()) > 0.1
