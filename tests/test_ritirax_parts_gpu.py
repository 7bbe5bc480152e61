"""The mechanisms Ritirax added, each alone against the plain implementation, with inputs made so that a fault shows:
a key that carries the weight at every step of the distance table (packed and from scattered pages), a sink that
swallows a head, scores beyond the cap, the choice of experts among groups, the shared expert's gate, the norm with a
sigmoid gate, the per-head gains, and the decayed recurrence through prompts, single tokens and slots used again."""
import math

import pytest
import torch

from brolm_b200 import kernels
from tests.plain import ritirax_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def close(got, ref, dtype, what=""):
    tol = 2e-5 if dtype == torch.float32 else 2.5e-2
    scale = max(float(ref.abs().max()), 1e-3)
    err = float((got.double().cpu() - ref.double()).abs().max()) / scale
    assert err <= tol, f"{what}: relative error {err:.3e} exceeds {tol:.0e}"


def steps_of(rows, far):
    """Distances at which the table's row changes, each with the distance before it, and a few beyond the last."""
    out, n = set(), 1
    while plain.distance_bucket(n - 1, rows, far) < rows - 1:
        if plain.distance_bucket(n, rows, far) != plain.distance_bucket(n - 1, rows, far):
            out.update((n - 1, n))
        n += 1
    return sorted(out | {0, n + 3, n + 40})


def dist_table(rel, far):
    """The table as the kernels take it: [heads][distance], made with the oracle's own rule."""
    rows = rel.shape[0]
    n = 0
    while plain.distance_bucket(n, rows, far) < rows - 1:
        n += 1
    idx = torch.tensor([plain.distance_bucket(i, rows, far) for i in range(n + 1)])
    return rel[idx].t().contiguous().float()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,vd,rows,far,cap", [(4, 2, 16, 8, 8, 40.0, 20.0), (3, 3, 12, 20, 7, 25.0, 0.0),
                                                    (4, 1, 32, 32, 32, 200.0, 30.0), (2, 2, 64, 96, 12, 90.0, 5.0)])
def test_a_key_that_carries_the_weight_at_every_step_of_the_table(dtype, H, G, hd, vd, rows, far, cap):
    """Packed (a prompt): the last queries each look for one key at a distance where the table's row changes; the
    table's rows differ by several units, so a row that is one off moves the weights."""
    g = torch.Generator().manual_seed(rows + hd)
    dists = steps_of(rows, far)
    T = max(dists) + len(dists) + 2
    k = torch.randn(T, G, hd, generator=g)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(T, G, vd, generator=g)
    q = 0.1 * torch.randn(T, H, hd, generator=g)
    for i, n in enumerate(dists):
        p = T - 1 - i
        for h in range(H):
            q[p, h] = 9.0 * k[p - n, h // (H // G)]
    rel = 3.0 * torch.randn(rows, H, generator=g)
    sink = torch.randn(H, generator=g)
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    ref = plain.biased_attention(q.double(), k.double(), v.double(), 1.0, cap, rel.double(), far, sink.double())
    out = torch.empty(T, H * vd, dtype=dtype, device=DEV)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    kvl = torch.tensor([T], dtype=torch.int32, device=DEV)
    kernels.attention_simt(q.reshape(T, -1).to(DEV), out, cu, kvl, n_kv=G, group=H // G, head_dim=hd, scale=1.0, cap=cap,
                           window=0, batch=1, max_q_len=T, k=k.reshape(T, -1).to(DEV), v=v.reshape(T, -1).to(DEV), v_dim=vd,
                           sink=sink.to(DEV), dist_bias=dist_table(rel, far).to(DEV))
    close(out.view(T, H, vd), ref, dtype, "packed")
    # the same without the table is far away: the table matters in this test
    kernels.attention_simt(q.reshape(T, -1).to(DEV), out, cu, kvl, n_kv=G, group=H // G, head_dim=hd, scale=1.0, cap=cap,
                           window=0, batch=1, max_q_len=T, k=k.reshape(T, -1).to(DEV), v=v.reshape(T, -1).to(DEV), v_dim=vd,
                           sink=sink.to(DEV))
    assert float((out.view(T, H, vd).double().cpu() - ref).abs().max()) > 0.05
    if dtype == torch.bfloat16 and kernels.attention_headmix_ok(hd, vd, H // G, False):
        # the same on the tensor cores
        out.zero_()
        kernels.attention_headmix_prefill(q.reshape(T, -1).to(DEV), out, cu, k.reshape(T, -1).to(DEV), v.reshape(T, -1).to(DEV),
                                          n_kv=G, group=H // G, head_dim=hd, v_dim=vd, scale=1.0, window=0, batch=1,
                                          max_q_len=T, cap=cap, sink=sink.to(DEV), dist_bias=dist_table(rel, far).to(DEV))
        close(out.view(T, H, vd), ref, dtype, "packed, tensor cores")
        if hd == vd:
            # ... and on the kernel for key and value rows of one size
            out.zero_()
            kernels.attention_prefill_mma(q.reshape(T, -1).to(DEV), out, cu, k.reshape(T, -1).to(DEV), v.reshape(T, -1).to(DEV),
                                          n_kv=G, group=H // G, head_dim=hd, scale=1.0, cap=cap, window=0, batch=1,
                                          max_q_len=T, sink=sink.to(DEV), dist_bias=dist_table(rel, far).to(DEV))
            close(out.view(T, H, vd), ref, dtype, "packed, tensor cores, rows of one size")


@pytest.mark.parametrize("dtype,vd", [(torch.float32, 48), (torch.bfloat16, 48), (torch.bfloat16, 16)])
def test_far_keys_from_scattered_pages(dtype, vd):
    """Decoding: one query per sequence over pages in a scattered order with NaN in the places never written; the key
    that carries the weight lies at a page's last place, at the next page's first, and far beyond the table's end."""
    g = torch.Generator().manual_seed(7)
    H, G, hd, rows, far, page = 4, 2, 16, 8, 40.0, 64
    lengths = [1, 64, 65, 130, 400, 41]
    targets = [0, 63, 64, 63, 5, 1]                                   # position of the key each sequence's query looks for
    rel = 3.0 * torch.randn(rows, H, generator=g)
    sink = torch.randn(H, generator=g)
    ks, vs, qs = [], [], []
    for n, tgt in zip(lengths, targets):
        k = torch.randn(n, G, hd, generator=g)
        k = k / k.norm(dim=-1, keepdim=True)
        ks.append(k.to(dtype))
        vs.append(torch.randn(n, G, vd, generator=g).to(dtype))
        qs.append(torch.stack([9.0 * k[tgt, h // (H // G)] for h in range(H)]).to(dtype))
    pages_per = [(n + page - 1) // page for n in lengths]
    n_pages = sum(pages_per) + 3
    order = iter(torch.randperm(n_pages, generator=g).tolist())
    pt = torch.zeros(len(lengths), max(pages_per), dtype=torch.int32)
    kp = torch.full((n_pages, G, page, hd), float("nan")).to(dtype)
    vp = torch.full((n_pages, G, page, vd), float("nan")).to(dtype)
    for b, n in enumerate(lengths):
        for j in range(pages_per[b]):
            pt[b, j] = next(order)
        for p in range(n):
            kp[int(pt[b, p // page]), :, p % page] = ks[b][p]
            vp[int(pt[b, p // page]), :, p % page] = vs[b][p]
    B = len(lengths)
    out = torch.empty(B, H * vd, dtype=dtype, device=DEV)
    kernels.attention_simt(torch.stack(qs).reshape(B, -1).to(DEV), out, torch.arange(B + 1, dtype=torch.int32, device=DEV),
                           torch.tensor(lengths, dtype=torch.int32, device=DEV), n_kv=G, group=H // G, head_dim=hd, scale=1.0,
                           cap=15.0, window=0, batch=B, max_q_len=1, k_pages=kp.to(DEV), v_pages=vp.to(DEV),
                           page_table=pt.to(DEV), ring=1 << 30, page_size=page, v_dim=vd, sink=sink.to(DEV),
                           dist_bias=dist_table(rel, far).to(DEV))
    assert bool(torch.isfinite(out.float()).all()), "a place of the cache that was never written was read"
    refs = [plain.biased_attention(qs[b].double()[None], ks[b].double(), vs[b].double(), 1.0, 15.0, rel.double(), far,
                                   sink.double(), first=n - 1)[0] for b, n in enumerate(lengths)]
    for b, n in enumerate(lengths):
        close(out[b].view(H, vd), refs[b], dtype, f"sequence of {n}")
    if dtype == torch.bfloat16:
        # the same on the tensor cores, the keys of a sequence in one piece and cut into three and seven
        for splits in (1, 3, 7):
            out.zero_()
            kernels.attention_headmix_decode(torch.stack(qs).reshape(B, -1).to(DEV), out,
                                             torch.arange(B + 1, dtype=torch.int32, device=DEV),
                                             torch.tensor(lengths, dtype=torch.int32, device=DEV), kp.to(DEV), vp.to(DEV),
                                             pt.to(DEV), ring=1 << 30, ring_from=0, page_size=page, n_kv=G, group=H // G,
                                             head_dim=hd, v_dim=vd, scale=1.0, window=0, batch=B, n_splits=splits, cap=15.0,
                                             sink=sink.to(DEV), dist_bias=dist_table(rel, far).to(DEV))
            for b, n in enumerate(lengths):
                close(out[b].view(H, vd), refs[b], dtype, f"sequence of {n}, tensor cores, {splits} splits")
            if hd == vd:
                out.zero_()
                kernels.attention_decode_mma(torch.stack(qs).reshape(B, -1).to(DEV), out,
                                             torch.arange(B + 1, dtype=torch.int32, device=DEV),
                                             torch.tensor(lengths, dtype=torch.int32, device=DEV), kp.to(DEV), vp.to(DEV),
                                             pt.to(DEV), ring=1 << 30, page_size=page, n_kv=G, group=H // G, head_dim=hd,
                                             scale=1.0, cap=15.0, window=0, batch=B, n_splits=splits, sink=sink.to(DEV),
                                             dist_bias=dist_table(rel, far).to(DEV))
                for b, n in enumerate(lengths):
                    close(out[b].view(H, vd), refs[b], dtype, f"sequence of {n}, rows of one size, {splits} splits")


def test_a_sink_that_swallows_a_head():
    g = torch.Generator().manual_seed(3)
    T, H, hd = 20, 2, 16
    q, k, v = (torch.randn(T, H, hd, generator=g) for _ in range(3))
    sink = torch.tensor([40.0, -40.0])
    out = torch.empty(T, H * hd, dtype=torch.float32, device=DEV)
    kernels.attention_simt(q.reshape(T, -1).to(DEV), out, torch.tensor([0, T], dtype=torch.int32, device=DEV),
                           torch.tensor([T], dtype=torch.int32, device=DEV), n_kv=H, group=1, head_dim=hd, scale=0.25, cap=0.0,
                           window=0, batch=1, max_q_len=T, k=k.reshape(T, -1).to(DEV), v=v.reshape(T, -1).to(DEV),
                           sink=sink.to(DEV))
    out = out.view(T, H, hd).cpu()
    assert float(out[:, 0].abs().max()) < 1e-6
    ref = plain.biased_attention(q.double(), k.double(), v.double(), 0.25, 0.0, None, 0.0, None)
    close(out[:, 1], ref[:, 1], torch.float32)


@pytest.mark.parametrize("E,top,groups,keep,tokens", [(10, 4, 5, 3, 50), (6, 3, 3, 2, 9), (4, 2, 4, 3, 300), (8, 2, 2, 1, 70),
                                                      (12, 5, 1, 1, 33), (64, 6, 8, 4, 300), (4, 4, 2, 2, 5)])
def test_choice_among_groups(E, top, groups, keep, tokens):
    g = torch.Generator().manual_seed(E * 7 + top)
    W = 48
    x = torch.randn(tokens, W, generator=g)
    router = torch.randn(E, W, generator=g) * 0.3
    ids = torch.empty(tokens, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(tokens, top, dtype=torch.float32, device=DEV)
    s = torch.softmax(x.double() @ router.double().T, dim=-1)
    for use_product in (False, True):
        if use_product:
            z = (x.double() @ router.double().T).float().to(DEV)
            kernels.route_pick(z, top, ids, wts, "softmax", None, groups=groups, keep=keep, renorm=False, scale=1.75)
        else:
            kernels.route_topk(x.to(DEV), router.to(DEV), top, ids, wts, "softmax", None, groups=groups, keep=keep,
                               renorm=False, scale=1.75)
        for t in range(tokens):
            want = plain.choose_experts(s[t], top, groups, keep)
            assert ids[t].tolist() == want, (t, ids[t].tolist(), want)
            assert torch.allclose(wts[t].double().cpu(), 1.75 * s[t][want], rtol=1e-5)
    # the plain softmax router is what it was: weights over their sum
    kernels.route_topk(x.to(DEV), router.to(DEV), top, ids, wts, "softmax", None)
    assert torch.allclose(wts.sum(dim=1).cpu(), torch.ones(tokens), atol=1e-5)


def test_a_group_that_is_shut_out_whatever_its_second_best():
    """Group 1 holds the second and third largest scores but not a group's best among the kept ones."""
    z = torch.tensor([[5.0, 0.0, 4.9, 4.8, 4.95, 0.1]]).to(DEV)        # groups of two: best 5.0, 4.9, 4.95 -> 0 and 2 stay
    ids = torch.empty(1, 3, dtype=torch.int32, device=DEV)
    wts = torch.empty(1, 3, dtype=torch.float32, device=DEV)
    kernels.route_pick(z, 3, ids, wts, "softmax", None, groups=3, keep=2, renorm=False, scale=1.0)
    assert ids[0].tolist() == [0, 4, 5]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_shared_expert_gate_in_the_sum(dtype):
    g = torch.Generator().manual_seed(4)
    T, W, top = 37, 72, 3
    y = torch.randn(top, T, W, generator=g)
    shared = torch.randn(2, T, W, generator=g)
    x = torch.randn(T, W, generator=g).to(dtype)
    sg = (torch.randn(W, generator=g) * 0.4).to(dtype)
    ids = torch.randint(0, 5, (T, top), generator=g).to(torch.int32)
    wts = torch.rand(T, top, generator=g)
    out = torch.empty(T, W, dtype=torch.float32, device=DEV)
    kernels.experts_combine(y.to(DEV), ids.to(DEV), wts.to(DEV), 5, x.to(DEV), shared.to(DEV), out, sg.to(DEV))
    gate = torch.sigmoid(x.double() @ sg.double())
    ref = torch.einsum("tc,ctw->tw", wts.double(), y.double()) + gate[:, None] * shared.double().sum(dim=0)
    close(out, ref, torch.float32)
    kernels.experts_combine(y.to(DEV), ids.to(DEV), wts.to(DEV), 5, x.to(DEV), shared.to(DEV), out)       # no gate: as before
    close(out, torch.einsum("tc,ctw->tw", wts.double(), y.double()) + shared.double().sum(dim=0), torch.float32)


@pytest.mark.parametrize("cols", [48, 192, 1000])
@pytest.mark.parametrize("with_gain", [True, False])
def test_norm_with_a_sigmoid_gate(cols, with_gain):
    g = torch.Generator().manual_seed(cols)
    T = 19
    y = torch.randn(T, cols, generator=g) * 3
    wide = torch.randn(T, cols + 24, generator=g)
    gain = torch.randn(cols, generator=g) if with_gain else None
    ref = (plain.unit_rms(y.double(), 1e-5) * gain.double() if with_gain else y.double()) * torch.sigmoid(wide[:, 24:].double())
    for od in (torch.float32, torch.bfloat16):
        out = torch.empty(T, cols, dtype=od, device=DEV)
        kernels.norm_sigmoid_gate(y.to(DEV), wide.to(DEV)[:, 24:], gain.to(DEV) if with_gain else None, 1e-5, out)
        close(out, ref, od)


@pytest.mark.parametrize("n_q,n_kv,hd,vd", [(4, 2, 16, 8), (3, 3, 12, 20), (2, 1, 64, 80)])
def test_per_head_norm_with_gains(n_q, n_kv, hd, vd):
    g = torch.Generator().manual_seed(hd)
    T = 11
    cols = (n_q + n_kv) * hd + n_kv * vd
    proj = torch.randn(T, cols, generator=g) * 2
    qg, kg = torch.randn(hd, generator=g), torch.randn(hd, generator=g)
    out = torch.empty(T, cols, dtype=torch.float32, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    kernels.qkv_finish(proj.to(DEV), None, n_q, n_kv, hd, vd, pos, out, head_norm=True, eps=1e-5, q_gain=qg.to(DEV), k_gain=kg.to(DEV))
    p = proj.double()
    q = plain.unit_rms(p[:, :n_q * hd].view(T, n_q, hd), 1e-5) * qg.double()
    k = plain.unit_rms(p[:, n_q * hd:(n_q + n_kv) * hd].view(T, n_kv, hd), 1e-5) * kg.double()
    ref = torch.cat([q.reshape(T, -1), k.reshape(T, -1), p[:, (n_q + n_kv) * hd:]], dim=1)
    close(out, ref, torch.float32)


def scan(q, k, v, decay, cuts, state, slot, dtype=torch.float32):
    """Run one sequence through decay_scan in pieces of the given lengths; q, k, v (T, H, .)."""
    T, H, d = q.shape
    dv = v.shape[-1]
    row = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(dtype).to(DEV)
    dm1 = torch.tensor([x - 1.0 for x in decay], dtype=F64).float().to(DEV)
    outs, at = [], 0
    for n in cuts:
        out = torch.empty(n, H * dv, dtype=torch.float32, device=DEV)
        kernels.decay_scan(row[at:at + n], 0, H * d, 2 * H * d, H, d, dv, "none", dm1,
                           torch.tensor([0, n], dtype=torch.int32, device=DEV), torch.tensor([at + n], dtype=torch.int32, device=DEV),
                           torch.tensor([slot], dtype=torch.int32, device=DEV), state, out, 1)
        outs.append(out)
        at += n
    return torch.cat(outs).view(T, H, dv)


@pytest.mark.parametrize("H,d,dv", [(3, 8, 16), (1, 6, 12), (2, 32, 64), (2, 128, 128), (5, 20, 7), (1, 256, 40)])
def test_decayed_recurrence_in_pieces(H, d, dv):
    g = torch.Generator().manual_seed(d + dv)
    T = 150
    q, k = torch.randn(T, H, d, generator=g) * 0.3, torch.randn(T, H, d, generator=g) * 0.3
    v = torch.randn(T, H, dv, generator=g)
    decay = [0.5, 0.999, 1.0, 0.9, 0.97][:H]
    ref, S = plain.decay_recurrence(q.double(), k.double(), v.double(), torch.tensor(decay, dtype=F64))
    size = kernels.decay_state_size(H, d, dv)
    for cuts in ([T], [1] * T, [64, 1, 1, 20, 2, 62], [149, 1]):
        state = torch.zeros(3, size + 8, dtype=torch.float32, device=DEV)
        state[0] = float("nan")                                        # another sequence's row is never touched
        got = scan(q, k, v, decay, cuts, state, slot=1)
        close(got, ref, torch.float32, f"cuts {cuts[:4]}")
        kept = state[1, :size].view(H, dv, -1)[:, :, :d].transpose(1, 2)
        close(kept, S, torch.float32, "the state after the last token")
        assert bool(torch.isnan(state[0]).all()) and float(state[2].abs().max()) == 0.0


def test_a_first_token_that_lasts_and_one_that_fades():
    """3,000 tokens: with a decay of 1 the first token's key still answers at the end; with 0.99 it is gone, and with
    0.999 it is there at a twentieth (a decay rounded to a float before the recurrence would lose three digits)."""
    T, d, dv = 3000, 8, 8
    q = torch.zeros(T, 3, d)
    k = torch.zeros(T, 3, d)
    v = torch.zeros(T, 3, dv)
    k[0, :, 0] = 1.0
    v[0, :, 3] = 2.0
    q[-1, :, 0] = 1.0
    decay = [1.0, 0.99, 0.999]
    state = torch.zeros(1, kernels.decay_state_size(3, d, dv), dtype=torch.float32, device=DEV)
    got = scan(q, k, v, decay, [2000, 999, 1], state, slot=0)[-1].cpu().double()
    want = torch.tensor([2.0, 2.0 * 0.99 ** 2999, 2.0 * 0.999 ** 2999], dtype=F64)
    assert torch.allclose(got[:, 3], want, rtol=2e-6, atol=1e-30), (got[:, 3], want)


def test_activation_and_bfloat16_rows():
    g = torch.Generator().manual_seed(9)
    T, H, d, dv = 40, 2, 16, 24
    raw = torch.randn(T, 2 * H * d + H * dv + 5, generator=g).to(torch.bfloat16)
    q, k = raw[:, :H * d].double().view(T, H, d), raw[:, H * d:2 * H * d].double().view(T, H, d)
    v = raw[:, 2 * H * d:2 * H * d + H * dv].double().view(T, H, dv)
    ref, _ = plain.decay_recurrence(plain.silu(q), plain.silu(k), plain.silu(v), torch.tensor([0.9, 0.8], dtype=F64))
    state = torch.zeros(2, kernels.decay_state_size(H, d, dv), dtype=torch.float32, device=DEV)
    out = torch.empty(T, H * dv, dtype=torch.float32, device=DEV)
    kernels.decay_scan(raw.to(DEV), 0, H * d, 2 * H * d, H, d, dv, "silu", torch.tensor([-0.1, -0.2], device=DEV),
                       torch.tensor([0, T], dtype=torch.int32, device=DEV), torch.tensor([T], dtype=torch.int32, device=DEV),
                       torch.tensor([1], dtype=torch.int32, device=DEV), state, out, 1)
    close(out.view(T, H, dv), ref, torch.float32)


def test_a_batch_of_unequal_sequences_and_a_padding_row():
    g = torch.Generator().manual_seed(10)
    H, d, dv = 2, 12, 20
    lens = [5, 1, 33, 0]                                               # the last row is padding: no tokens, length 0
    total = sum(lens)
    q, k = torch.randn(total, H, d, generator=g) * 0.3, torch.randn(total, H, d, generator=g) * 0.3
    v = torch.randn(total, H, dv, generator=g)
    row = torch.cat([q.reshape(total, -1), k.reshape(total, -1), v.reshape(total, -1)], dim=1).to(DEV)
    size = kernels.decay_state_size(H, d, dv)
    state = torch.zeros(5, size, dtype=torch.float32, device=DEV)
    state[4] = 7.0                                                     # the padding rows' spare row
    cu = torch.tensor([0, 5, 6, 39, 39], dtype=torch.int32, device=DEV)
    out = torch.zeros(total, H * dv, dtype=torch.float32, device=DEV)
    kernels.decay_scan(row, 0, H * d, 2 * H * d, H, d, dv, "none", torch.tensor([-0.05, -0.2], device=DEV), cu,
                       torch.tensor([5, 1, 33, 0], dtype=torch.int32, device=DEV),
                       torch.tensor([2, 0, 3, 4], dtype=torch.int32, device=DEV), state, out, 4)
    at = 0
    for n in lens[:3]:
        ref, _ = plain.decay_recurrence(q[at:at + n].double(), k[at:at + n].double(), v[at:at + n].double(),
                                        torch.tensor([0.95, 0.8], dtype=F64))
        close(out[at:at + n].view(n, H, dv), ref, torch.float32, f"sequence of {n}")
        at += n
    assert float((state[4] - 7.0).abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0
