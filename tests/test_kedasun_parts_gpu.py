"""The kernels that Kedasun brought, each alone against the plain function of the same mechanism: norms in groups
(alone and fused with the residual sum), the clamped pair function, the row-wise kernel between the projection and
the attention (biases, unit-norm heads, rotation of interleaved pairs over part of a head, values mixed with an
earlier layer's, pages filled), the short convolution with an input bias through a prompt and then token by token,
and the mixing of the heads' results with the gate.  Sizes are other than any model's here and include values that
make two mechanisms coincide (one group, one kv head, one tap, a whole head rotated, a mixing weight of 0 and 1)."""
import pytest
import torch

from brolm_b200 import kernels
from tests.plain import kedasun_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, scale=1.0):
    return scale * torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)


def close(got, ref, tol, what=""):
    err = float((got.double().cpu() - ref).abs().max()) / max(float(ref.abs().max()), 1e-6)
    assert err <= tol, f"{what}: relative error {err:.3e} exceeds {tol:.0e}"


@pytest.mark.parametrize("W,groups", [(48, 3), (40, 1), (64, 8), (96, 96), (2048, 4), (130, 2)])
def test_norm_in_groups_alone_and_with_the_residual_sum(W, groups):
    T, eps = 7, 1e-5
    x, y, h = rnd(T, W, seed=1, scale=3.0), rnd(T, W, seed=2), rnd(T, W, seed=3)
    x[2] *= 1e-3                                       # a row so small that eps matters
    g1, g2 = rnd(W, seed=4), rnd(W, seed=5)
    out = torch.empty(T, W, dtype=torch.float32, device=DEV)
    kernels.group_rmsnorm(x.float().to(DEV), g1.float().to(DEV), eps, 0.0, groups, out)
    close(out, plain.grouped_rms_norm(x.float().double(), g1.float().double(), groups, eps), 2e-6, "norm alone")
    # h += norm(y); out = norm(h) for the next sublayer, partial sums of y added first
    parts = torch.stack([0.25 * y, 0.75 * y]).float().to(DEV).contiguous()
    hd = h.float().to(DEV).contiguous()
    nxt = torch.empty(T, W, dtype=torch.float32, device=DEV)
    kernels.residual_group_rmsnorm(hd, parts, g1.float().to(DEV), eps, 0.0, g2.float().to(DEV), eps, 0.0, groups, nxt)
    ysum = parts.double().cpu().sum(0)
    h_ref = h.float().double() + plain.grouped_rms_norm(ysum, g1.float().double(), groups, eps)
    close(hd, h_ref, 2e-6, "the stream after the sum")
    close(nxt, plain.grouped_rms_norm(h_ref, g2.float().double(), groups, eps), 4e-6, "the next input")


@pytest.mark.parametrize("limit", [0.7, 3.0, 50.0])
def test_clamped_pair_function(limit):
    T, n = 5, 72
    gu = rnd(T, 2 * n, seed=6, scale=2.5).float()
    gu[0, :4] = torch.tensor([limit, limit + 1e-3, -limit, 40.0])          # the gate is only cut from above
    gu[0, n:n + 4] = torch.tensor([limit, -limit - 1.0, limit + 1.0, -1.0])  # the other half from both sides; -1 gives zero
    out = torch.empty(T, n, dtype=torch.float32, device=DEV)
    kernels.gated_act(gu.to(DEV).contiguous(), out, "clamped_gate", limit)
    g, u = gu[:, :n].double().clamp(max=limit), gu[:, n:].double().clamp(-limit, limit)
    close(out, g * torch.sigmoid(1.702 * g) * (u + 1.0), 2e-6)
    eye = torch.eye(n, dtype=torch.float64)
    close(out, plain.clamped_feed_forward(torch.cat([gu[:, :n], gu[:, n:]], 1).double(),
                                          torch.cat([eye, 0 * eye], 1), torch.cat([0 * eye, eye], 1), eye, limit), 2e-6)


CASES = [  # H, G, d, dv, rot, pairing, head_norm, lam
    (4, 2, 8, 16, 4, "interleaved", False, 0.4),
    (6, 3, 12, 6, 12, "interleaved", True, 1.0),
    (2, 1, 20, 18, 6, "interleaved", False, 0.0),
    (4, 4, 16, 16, 0, "interleaved", True, None),
    (8, 2, 64, 128, 32, "interleaved", False, 0.25),
]


@pytest.mark.parametrize("H,G,d,dv,rot,pairing,head_norm,lam", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rows_between_projection_and_attention(H, G, d, dv, rot, pairing, head_norm, lam, dtype):
    T, eps, base, page = 70, 1e-5, 300.0, 64
    cols = (H + G) * d + G * dv
    proj, bias = rnd(T, cols, seed=7).float(), rnd(cols, seed=8).float()
    v_first = rnd(T, G * dv, seed=9).float()
    pos = torch.arange(T, dtype=torch.int32)
    pos[40:] -= 40                                      # two sequences: 40 and 30 tokens
    table = None
    if rot:
        i = torch.arange(rot // 2, dtype=torch.float64)
        ang = torch.arange(64, dtype=torch.float64)[:, None] * base ** (-2.0 * i / rot)[None, :]
        table = torch.stack([ang.cos(), ang.sin()], -1).float().contiguous().to(DEV)
    k_pages = torch.zeros(3, G, page, d, dtype=dtype, device=DEV)
    v_pages = torch.zeros(3, G, page, dv, dtype=dtype, device=DEV)
    rows = torch.cat([torch.arange(40) + 2 * page, torch.arange(30)]).to(torch.int32)   # page 2, then page 0
    out = torch.empty(T, cols, dtype=dtype, device=DEV)
    keep = torch.empty(T, G * dv, dtype=torch.float32, device=DEV)
    kernels.qkv_finish(proj.to(DEV), bias.to(DEV), H, G, d, dv, pos.to(DEV), out, head_norm=head_norm, eps=eps, cos_sin=table,
                       rotary_dim=rot, pairing=pairing, mix=torch.tensor([lam or 0.0], dtype=torch.float32, device=DEV),
                       v_first=v_first.to(DEV) if lam is not None else None, v_keep=keep, k_pages=k_pages,
                       v_pages=v_pages, cache_rows=rows.to(DEV), page_size=page)
    x = proj.double() + bias.double()
    q, k, v = x[:, :H * d].reshape(T, H, d), x[:, H * d:(H + G) * d].reshape(T, G, d), x[:, (H + G) * d:].reshape(T, G, dv)
    if head_norm:
        q, k = plain.unit_heads(q, eps), plain.unit_heads(k, eps)
    if rot:
        for lo, hi in ((0, 40), (40, 70)):
            q[lo:hi], k[lo:hi] = plain.rotate_pairs(q[lo:hi], base, rot), plain.rotate_pairs(k[lo:hi], base, rot)
    close(keep, v.reshape(T, -1), 1e-6, "the layer's own values")
    if lam is not None:
        v = plain.mix_values(v, v_first.double().reshape(T, G, dv), lam)
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    close(out[:, :H * d], q.reshape(T, -1), tol, "q")
    close(out[:, H * d:(H + G) * d], k.reshape(T, -1), tol, "k")
    close(out[:, (H + G) * d:], v.reshape(T, -1), tol, "v")
    close(k_pages[2, :, :40].transpose(0, 1), k[:40], tol, "keys of the first sequence in their page")
    close(v_pages[0, :, :30].transpose(0, 1), v[40:], tol, "values of the second sequence in their page")
    assert float(k_pages[1].abs().max()) == 0.0 and float(k_pages[0, :, 30:].abs().max()) == 0.0


@pytest.mark.parametrize("C,K", [(24, 4), (40, 1), (16, 2), (130, 7)])
def test_short_convolution_with_an_input_bias_through_prompt_and_single_tokens(C, K):
    lens, more = [9, 1, 30], 6
    taps, bias = rnd(C, K, seed=10).float(), rnd(C, seed=11).float()
    seqs = [rnd(n + more, C, seed=20 + i).float() for i, n in enumerate(lens)]
    refs = [plain.short_convolution(s.double() + bias.double(), taps.double()) for s in seqs]
    B = len(lens)
    state = torch.zeros(B + 1, max(1, (K - 1) * C), dtype=torch.float32, device=DEV)
    slots = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)

    def step(xs, starts):
        n = [x.shape[0] for x in xs]
        cu = torch.tensor([0] + list(torch.tensor(n).cumsum(0)), dtype=torch.int32, device=DEV)
        kv_len = torch.tensor([s + m for s, m in zip(starts, n)], dtype=torch.int32, device=DEV)
        tok_seq = torch.cat([torch.full((m,), b, dtype=torch.int32) for b, m in enumerate(n)]).to(DEV)
        pos = torch.cat([torch.arange(s, s + m, dtype=torch.int32) for s, m in zip(starts, n)]).to(DEV)
        x = torch.cat(xs).to(DEV).contiguous()
        out = torch.empty(x.shape, dtype=torch.float32, device=DEV)
        seq = (cu, kv_len, slots, state)
        kernels.causal_conv(x, bias.to(DEV), taps.to(DEV), None, "none", tok_seq, pos, *seq, 0, out)
        kernels.conv_tail(x, bias.to(DEV), K, *seq, 0, B)
        return out.cpu().split(n)

    got = [[o] for o in step([s[:n] for s, n in zip(seqs, lens)], [0] * B)]
    for t in range(more):
        for b, o in enumerate(step([s[n + t:n + t + 1] for s, n in zip(seqs, lens)], [n + t for n in lens])):
            got[b].append(o)
    for b in range(B):
        close(torch.cat(got[b]), refs[b], 2e-6, f"sequence {b}")


@pytest.mark.parametrize("H,G,dv,talk,gate", [(4, 2, 16, True, True), (6, 1, 10, True, False), (3, 3, 8, True, True),
                                              (4, 2, 16, False, True), (16, 4, 128, True, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_heads_results_mixed_and_gated(H, G, dv, talk, gate, dtype):
    T = 9
    acc = rnd(T, H, G if talk else 1, dv, seed=12).float()
    mat = (torch.eye(H, dtype=torch.float64) + 0.5 * rnd(H, H, seed=13)).float()
    logit = rnd(T, H, seed=14, scale=2.0).float()
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    kernels.heads_mix(acc.reshape(T, -1).to(DEV).contiguous(), mat.to(DEV) if talk else None,
                      logit.to(DEV) if gate else None, out, H, G, dv)
    a = acc.double()
    if talk:
        own = torch.tensor([h // (H // G) for h in range(H)])
        ref = torch.stack([torch.einsum("g,tgd->td", mat[h].double(), a[:, :, own[h]]) for h in range(H)], 1)
    else:
        ref = a[:, :, 0]
    if gate:
        ref = ref * torch.sigmoid(logit.double())[:, :, None]
    close(out, ref.reshape(T, -1), 2e-6 if dtype == torch.float32 else 8e-3)
