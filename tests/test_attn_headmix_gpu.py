"""The tensor-core attention with head-wise options (value rows of their own size, distance slopes, a window that
keeps first keys, every head's weights on every kv head's values) against a plain float64 computation of the same
rounded inputs: prompts of unequal lengths, and one token over a paged cache with a ring behind kept places, with
pages in scattered order and every number of splits.  One far key and one kept first key are scaled so that their
scores stand out: a key lost or seen wrongly moves the result by far more than rounding."""
import pytest
import torch

from brolm_b200 import kernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def plain(q, k, v, pos, n_kv, scale, window, keep, slopes, all_values):
    """q [H, hd] at position pos over k [L, G, hd], v [L, G, vd] (float64) -> [H, vd] or [H, G, vd]."""
    H, G = q.shape[0], n_kv
    j = torch.arange(k.shape[0])
    seen = (j <= pos) & (((pos - j) < window) | (j < keep) if window else torch.ones_like(j, dtype=torch.bool))
    out = []
    for h in range(H):
        s = (k[:, h // (H // G)] @ q[h]) * scale
        if slopes is not None:
            s = s - slopes[h].double() * (pos - j)
        w = torch.softmax(s.masked_fill(~seen, float("-inf")), dim=0)
        out.append(torch.einsum("j,jgd->gd", w, v) if all_values else w @ v[:, h // (H // G)])
    return torch.stack(out)


def inputs(T, H, G, hd, vd, seed, loud=()):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H * hd, generator=g)
    k = torch.randn(T, G * hd, generator=g)
    v = torch.randn(T, G * vd, generator=g)
    for j in loud:                          # keys whose scores stand out from wherever they are seen
        if j < T:
            k[j] *= 3.0
    bf = lambda t: t.to(torch.bfloat16).to(DEV)
    return bf(q), bf(k), bf(v)


CASES = [  # H, G, hd, vd, window, keep, slopes, all_values
    (4, 2, 32, 16, 70, 3, True, True),
    (6, 3, 16, 48, 64, 0, True, True),
    (4, 1, 64, 64, 130, 66, True, True),
    (2, 2, 48, 80, 0, 0, False, False),
    (8, 2, 128, 128, 100, 1, True, True),
    (4, 4, 16, 32, 1, 2, True, False),
    (16, 1, 80, 144, 200, 65, False, True),
    (20, 2, 16, 32, 90, 2, True, True),         # ten heads a kv head: too many for the decode kernel that shares keys
    (8, 4, 64, 128, 150, 7, True, True),        # 32 tiles of 16 value elements: that kernel's largest form
    (8, 8, 32, 128, 70, 3, True, True),         # 64 such tiles: beyond it
]


@pytest.mark.parametrize("H,G,hd,vd,window,keep,sl,allv", CASES)
@pytest.mark.parametrize("f32", [True, False])
def test_prompts(H, G, hd, vd, window, keep, sl, allv, f32):
    lens = [1, 63, 64, 65, 200, 331]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    T = int(cu[-1])
    loud = [int(c) + d for c in cu[:-1] for d in (0, keep - 1 if keep else 1, keep)]
    q, k, v = inputs(T, H, G, hd, vd, 1, loud)
    slopes = torch.pow(2.0, -8.0 * torch.arange(1, H + 1) / H).float().to(DEV) if sl else None
    width = H * vd * (G if allv else 1)
    out = torch.full((T, width), float("nan"), dtype=torch.float32 if f32 else torch.bfloat16, device=DEV)
    kernels.attention_headmix_prefill(q, out, cu.to(DEV), k, v, n_kv=G, group=H // G, head_dim=hd, v_dim=vd,
                                      scale=0.2, window=window, batch=len(lens), max_q_len=max(lens), slopes=slopes,
                                      keep_first=keep, all_values=allv)
    torch.cuda.synchronize()
    qd, kd, vd_ = q.double().cpu(), k.double().cpu(), v.double().cpu()
    worst = 0.0
    for b, n in enumerate(lens):
        lo = int(cu[b])
        picks = sorted({min(n - 1, p) for p in (0, 1, n // 2, n - 1, window, window + keep, keep + window - 1, 64, 127, 128)})
        for p in picks:
            ref = plain(qd[lo + p].view(H, hd), kd[lo:lo + n].view(n, G, hd), vd_[lo:lo + n].view(n, G, vd), p, G, 0.2,
                        window, keep, slopes.cpu() if sl else None, allv)
            got = out[lo + p].double().cpu().view(ref.shape)
            worst = max(worst, float((got - ref).abs().max()))
    assert worst <= (2e-2 if f32 else 4e-2), f"largest difference {worst:.3e}"
    assert not torch.isnan(out.float()).any()


@pytest.mark.parametrize("H,G,hd,vd,window,keep,sl,allv", CASES)
def test_one_token_over_pages(H, G, hd, vd, window, keep, sl, allv):
    page = 64
    ring = (window + page - 1) // page * page if window else (1 << 30)
    head = (keep + page - 1) // page * page if (window and keep) else 0
    lens = [1, 2, 64, 65, 129, window + 1 if window else 130, window + keep + 70 if window else 500, 700]
    B = len(lens)
    slopes = torch.pow(2.0, -8.0 * torch.arange(1, H + 1) / H).float().to(DEV) if sl else None
    place = lambda p: p if (p < head or not window) else head + (p - head) % ring
    per_seq = [(min(n, head + ring) + page - 1) // page if window else (n + page - 1) // page for n in lens]
    n_pages = sum(per_seq) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(5)).tolist()
    k_pages = torch.zeros(n_pages, G, page, hd, dtype=torch.bfloat16, device=DEV)
    v_pages = torch.zeros(n_pages, G, page, vd, dtype=torch.bfloat16, device=DEV)
    table = torch.zeros(B, max(per_seq), dtype=torch.int32)
    qs, refs = [], []
    for b, n in enumerate(lens):
        for e in range(per_seq[b]):
            table[b, e] = order.pop()
        q, k, v = inputs(n, H, G, hd, vd, 10 + b, loud=(0, max(0, keep - 1), keep, max(0, n - window), max(0, n - 1 - window)))
        for p in range(n):                  # a place keeps the newest key that was written there
            pl = place(p)
            pg = int(table[b, pl // page])
            k_pages[pg, :, pl % page] = k[p].view(G, hd)
            v_pages[pg, :, pl % page] = v[p].view(G, vd)
        qs.append(q[n - 1])
        refs.append(plain(q[n - 1].double().cpu().view(H, hd), k.double().cpu().view(n, G, hd), v.double().cpu().view(n, G, vd),
                          n - 1, G, 0.2, window, keep, slopes.cpu() if sl else None, allv))
    q = torch.stack(qs)
    cu = torch.arange(B, dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    width = H * vd * (G if allv else 1)
    for splits in (1, 2, 3, 7):
        for dt in (torch.float32, torch.bfloat16):
            out = torch.full((B, width), float("nan"), dtype=dt, device=DEV)
            kernels.attention_headmix_decode(q, out, cu, kv_len, k_pages, v_pages, table.to(DEV), ring=ring, ring_from=head,
                                             page_size=page, n_kv=G, group=H // G, head_dim=hd, v_dim=vd, scale=0.2,
                                             window=window, batch=B, n_splits=splits, slopes=slopes, keep_first=keep,
                                             all_values=allv)
            torch.cuda.synchronize()
            for b in range(B):
                d = float((out[b].double().cpu().view(refs[b].shape) - refs[b]).abs().max())
                assert d <= (2e-2 if dt == torch.float32 else 4e-2), f"sequence of {lens[b]}, {splits} splits: {d:.3e}"
