#!/usr/bin/env python3
"""Decode and prefill throughput of brolm_b200 on one B200, one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--size 2b|9b|27b] [--batch B] [--context C] [--layers L]

The default run (``--size 2b``) has the layer sizes of Gemma 2 2B with random
bfloat16 weights, a batch of 8 and a context of 8192 tokens.  A step is one
decode step of the whole batch.  ``value`` is decoded tokens a second, timed on
the device: the median of ``repeats`` timed regions of exactly K steps each;
``e2e`` is the same through ``brolm_b200.generate`` with host tokens in and
out; ``prefill`` is one prompt of 2,048 tokens; ``points`` holds decoding at
batch 1 and 64, ``points_roofline`` their fractions of the memory's rate.

``--size 9b``: Gemma 2 9B sizes, 16 prompts of 128 to 6,144 tokens (seeded) in
one prefill step, then decode steps of the 16 sequences (K defaults to 128).
``--size 27b``: Gemma 2 27B sizes, a prompt of 2,048 tokens and decoding at
batch 8 (headline) and batch 1 (a point).  Same JSON shape.

``--arch banevik [--size s|m]``: the Banevik design (latent attention with a window and a sink, routed
experts, a looped span of layers) at layer sizes of a real model, beside a Gemma 2 model of the same
width, heads, window, layer runs and active feed-forward size: one prompt of 2,048 tokens and decoding at
batch 8, both through the engine, and a table of the device time of each kernel of both models with the
main kernels' fractions of their rooflines.  One JSON line of its own shape; the default run is untouched.

``--arch neburax [--size s|m]``: the same for the Neburax design (state-space layers, chunked attention beside a
gated recurrence, routed experts with a shared expert), beside Gemma 2 at equal sizes.

``--arch ritirax [--size s|m]``: the Ritirax design (linear attention with a fixed decay per head, capped attention with
a distance bias and a sink, gated latent attention, routed experts chosen among groups with a gated shared expert) beside
the closest design the library has, Neburax (state-space layers, attention beside a recurrence, routed experts with a
shared expert), built to the same width, heads, experts and layer count.

More than one GPU is not what this library does: ``--gpus N`` with N > 1 says
so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The layer sizes of the three workloads (the keys of Gemma 2's config.json; 2B is the configuration's default).
SIZES = {
    "2b": dict(),
    "9b": dict(num_hidden_layers=42, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8, head_dim=256,
               intermediate_size=14336, query_pre_attn_scalar=256.0),
    "27b": dict(num_hidden_layers=46, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16, head_dim=128,
                intermediate_size=36864, query_pre_attn_scalar=144.0),
}
REPEATS = 3


def peaks() -> dict:
    """The roofline's denominators: measured on this pool when the file is there, else the fallback.
    ``bf16_burst`` is the product peak of a kernel timed alone (what the prompt's fraction is taken
    against: the prompt is timed alone, between synchronisations and after an L2 flush);
    ``bf16_sustained`` the peak of a seconds-long loop under the power cap."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            raw = json.load(fh)
        burst = float(raw["bf16_tflops"])
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_burst": burst,
                "bf16_sustained": float(raw.get("bf16_tflops_sustained") or burst), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read only)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines: list[str] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# Decode steps that every run puts between its prompt and its warm-up steps.  The prompt (batch x
# context tokens at full compute power) leaves the GPU with lowered clocks for some tens of
# milliseconds: the first 10-30 decode steps after it take up to 1.4 times as long as the steady
# ones that the metric is about (measured: 3.4, then 2.8, then 2.45 ms at batch 8, context 8192).
SETTLE = 32


def decode_bytes(cfg, layers: int, lengths, itemsize: int = 2) -> float:
    """Bytes a decode step has to read: every weight once and the cache of the live requests,
    ``lengths`` being the tokens each of them holds (a windowed layer holds at most its window)."""
    if isinstance(lengths, tuple) and len(lengths) == 2:         # (batch, context): equal lengths
        lengths = [lengths[1]] * lengths[0]
    H, F = cfg.hidden_size, cfg.intermediate_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * F * H + 4 * H
    weights = (layers * per_layer + cfg.vocab_size * H + H) * itemsize
    kv = 0.0
    for i in range(layers):
        for n in lengths:
            keys = min(n, cfg.sliding_window) if cfg.is_sliding(i) else n
            kv += keys * 2 * cfg.kv_dim * itemsize
    return float(weights + kv)


def prefill_flops(cfg, layers: int, tokens) -> float:
    """Floating-point operations of one prefill step; ``tokens``: a prompt length or a list of them."""
    lengths = [tokens] if isinstance(tokens, int) else list(tokens)
    H, F = cfg.hidden_size, cfg.intermediate_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * F * H
    linear = 2.0 * sum(lengths) * per_layer * layers
    attn = 0.0
    for i in range(layers):
        for n in lengths:
            w = cfg.sliding_window if cfg.is_sliding(i) else n
            full = min(n, w)
            keys = full * (full + 1) // 2 + (n - full) * w          # sum over positions of min(p + 1, w)
            attn += 4.0 * cfg.q_dim * keys
    return linear + attn + 2.0 * cfg.vocab_size * H * len(lengths)


# --arch banevik: layer sizes (a cached row of kv_rank + rot_dim = 256 entries, the widest the tensor-core
# attention kernels take; sixteen heads, the most a decode tile has rows for)
BANEVIK_SIZES = {
    "s": dict(width=2048, heads=16, dim=64, rot_dim=64, vdim=64, kv_rank=192, window=1024, experts=32, top=4,
              ff=1024, layers=4, loop=(1, 3, 2), vocab=32768),
    "m": dict(width=3072, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=192, window=2048, experts=64, top=6,
              ff=1024, layers=4, loop=(1, 3, 2), vocab=65536),
}


def measure_design(cfg, vocab, dev, flush, steps, warmup, batch, context, prompt_len):
    """One prompt timed alone after an L2 flush, then decode steps through the generation loop's captured step,
    both with the device's own record of every kernel."""
    import torch

    import brolm_b200 as bb
    from brolm_b200 import kernels
    from brolm_b200.kernels.microbench import _cuda_events

    model = bb.Model(cfg, dtype="bfloat16", device=dev).init_random(seed=0, on_device=True)
    g = torch.Generator().manual_seed(1)
    out = {}
    # one prompt, timed alone after an L2 flush: the median of three after three untimed ones
    eng = bb.Engine(model, max_tokens=prompt_len + 64, max_slots=1, max_seq_len=prompt_len + 1)
    prompt = torch.randint(0, vocab, (prompt_len,), generator=g).tolist()
    times = []
    for it in range(6):
        (s,) = eng.open(1)
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([s], [prompt])
        e1.record()
        torch.cuda.synchronize()
        eng.close([s])
        if it >= 3:
            times.append(e0.elapsed_time(e1))

    def one_prompt():
        (s,) = eng.open(1)
        eng.step([s], [prompt])
        eng.close([s])
    out["prefill_ms"] = statistics.median(times)
    out["prefill_kernels"] = _by_kernel(_cuda_events(one_prompt))
    del eng
    # decoding: the generation loop's own steps, ids fed on the device
    total = SETTLE + warmup + steps
    eng = bb.Engine(model, max_tokens=batch * ((context + 63) // 64 * 64), max_slots=batch, max_seq_len=context + 1)
    prompts = [torch.randint(0, vocab, (context - total - 1,), generator=g).tolist() for _ in range(batch)]
    sampler = bb.Sampler(bb.SamplingParams(temperature=0.0))
    streams = torch.arange(batch, dtype=torch.int32, device=dev)
    pick = list(range(batch))
    slots = eng.open(batch)
    state = {"ids": sampler(eng.step(slots, prompts), streams, 0), "n": 1}

    def go(n):
        for _ in range(n):
            state["ids"] = sampler(eng.step_from(slots, state["ids"], pick), streams, state["n"])
            state["n"] += 1
    go(SETTLE + warmup)
    with ClockSampler() as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = kernels.launch_count()
        e0.record()
        go(steps)
        e1.record()
        torch.cuda.synchronize()
    out["decode_ms"] = e0.elapsed_time(e1) / steps
    out["launches"] = kernels.launch_count() - before
    out["clocks"] = clocks.summary()
    out["decode_kernels"] = _by_kernel(_cuda_events(lambda: go(1)))
    eng.close(slots)
    return out



def banevik_main(args, pk) -> int:
    import torch

    import brolm_b200 as bb
    from brolm_b200 import kernels
    from brolm_b200.kernels.microbench import _cuda_events

    z = BANEVIK_SIZES[args.size if args.size in BANEVIK_SIZES else "s"]
    dev = "cuda:0"
    torch.cuda.set_device(0)
    layer = dict(type="latent_attention",
                 mixer=dict(heads=z["heads"], dim=z["dim"], rot_dim=z["rot_dim"], vdim=z["vdim"], kv_rank=z["kv_rank"],
                            scale=(z["dim"] + z["rot_dim"]) ** -0.5, rot=dict(base=10000.0, dims=z["rot_dim"]),
                            mask=dict(size=z["window"])),
                 mlp=dict(kind="moe", expert=dict(ff=z["ff"]), router=dict(experts=z["experts"], top=z["top"])))
    bcfg = bb.BanevikConfig.from_dict(dict(
        architecture="Banevik", vocab=z["vocab"], width=z["width"], layers=[layer] * z["layers"],
        loop=dict(start=z["loop"][0], stop=z["loop"][1], times=z["loop"][2]), norm=dict(eps=1e-5),
        embedding=dict(bigram=dict(buckets=65521, mul_prev=8191, mul_cur=127)), logit_softcap=30.0))
    runs = len(bcfg.runs())
    inter = (2 * z["top"] * z["ff"] // 3 + 255) // 256 * 256          # three matrices there, two per expert here
    gcfg = bb.Gemma2Config(vocab_size=z["vocab"], hidden_size=z["width"], intermediate_size=inter,
                           num_hidden_layers=runs, num_attention_heads=z["heads"], num_key_value_heads=z["heads"] // 4,
                           head_dim=z["dim"] + z["rot_dim"], query_pre_attn_scalar=float(z["dim"] + z["rot_dim"]),
                           sliding_window=z["window"], layer_types=("sliding_attention",) * runs,
                           max_position_embeddings=8192)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    steps, warmup, batch, context, prompt_len = args.steps or 64, max(args.warmup, 3), args.batch or 8, 1280, 2048

    common = (dev, flush, steps, warmup, batch, context, prompt_len)
    b, gm = measure_design(bcfg, z["vocab"], *common), measure_design(gcfg, z["vocab"], *common)
    W, H, D, R = z["width"], z["heads"], z["kv_rank"] + z["rot_dim"], z["kv_rank"]
    T, top, ff, win = prompt_len, z["top"], z["ff"], z["window"]
    keys = win * (win + 1) // 2 + (T - win) * win if T > win else T * (T + 1) // 2
    hd = z["dim"] + z["rot_dim"]
    tf, gb = pk["bf16_burst"] * 1e12, pk["hbm_gbs"] * 1e9
    active = min(z["experts"], batch * top)
    # (kernel-name fragment, calls per layer run, flops or bytes per call, bound) for the main kernels of both models
    rows = [
        ("banevik prefill", b["prefill_kernels"], [
            ("grouped_tc_kernel", 2, 2.0 * T * top * ff * W * 2, "flops"),
            ("fast_kernel<128, 32, 4, false>", 2, 2.0 * T * top * ff * W * 2, "flops"),
            ("attn_prefill_mma", 1, 4.0 * H * D * keys, "flops"),
        ]),
        ("closest prefill", gm["prefill_kernels"], [
            ("gemm_tc2_kernel<1>", 1, 2.0 * T * W * 2 * inter, "flops"),
            ("attn_prefill_tc", 1, 4.0 * H * hd * keys, "flops"),
        ]),
        ("banevik decode", b["decode_kernels"], [
            ("fast_kernel<64, 64, 4, false>", 2, active * ff * W * 2.0 * 2, "bytes"),
            ("attn_decode_mma", 1, batch * min(context, win) * D * 2.0, "bytes"),
        ]),
        ("closest decode", gm["decode_kernels"], [
            ("skinny_kernel<2, 1, 1>", 1, 2 * inter * W * 2.0, "bytes"),
            ("attn_decode_mma", 1, batch * min(context, win) * 2 * (H // 4) * hd * 2.0, "bytes"),
        ]),
    ]
    table = []
    for title, kern, wanted in rows:
        for frag, calls, work, bound in wanted:
            us = sum(v["us"] for k, v in kern.items() if frag in k)
            n = sum(v["n"] for k, v in kern.items() if frag in k)
            if not n:
                continue
            per_run = us / runs
            total_work = work * runs                       # (work: of all the kernel's launches in one layer run)
            frac = total_work / (us * 1e-6) / (tf if bound.startswith("flops") else gb)
            table.append({"step": title, "kernel": frag, "launches": n, "us_per_layer_run": round(per_run, 2),
                          "bound": "tensor" if bound.startswith("flops") else "hbm", "frac_of_measured_peak": round(frac, 4)})
    result = {
        "metric": f"Banevik decode tokens/s (size {args.size if args.size in BANEVIK_SIZES else 's'}, batch {batch}, "
                  f"context {context}) beside Gemma 2 at equal sizes",
        "value": round(batch * 1000.0 / b["decode_ms"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(b["decode_ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "brolm_b200", "clocks": b["clocks"], "gpu_launches": b["launches"],
        "config": {"model": "Banevik", **{k: v for k, v in z.items()}, "layer_runs": runs, "global_batch": batch,
                   "seq_len": context, "closest": {"model": "Gemma 2", "hidden": W, "heads": H, "kv_heads": H // 4,
                                                   "head_dim": hd, "intermediate": inter, "layers": runs,
                                                   "sliding_window": win},
                   "l2": "the prompt is timed after an L2 flush; a decode step reads more than the L2 holds",
                   "peaks": pk["source"]},
        "banevik": {"prefill_tok_s": round(T * 1000.0 / b["prefill_ms"], 1), "prefill_ms": round(b["prefill_ms"], 3),
                    "decode_tok_s": round(batch * 1000.0 / b["decode_ms"], 1), "decode_ms": round(b["decode_ms"], 4)},
        "closest": {"prefill_tok_s": round(T * 1000.0 / gm["prefill_ms"], 1), "prefill_ms": round(gm["prefill_ms"], 3),
                    "decode_tok_s": round(batch * 1000.0 / gm["decode_ms"], 1), "decode_ms": round(gm["decode_ms"], 4)},
        "kernels": table,
        "by_kernel_us": {"banevik_prefill": _top(b["prefill_kernels"]), "closest_prefill": _top(gm["prefill_kernels"]),
                         "banevik_decode": _top(b["decode_kernels"]), "closest_decode": _top(gm["decode_kernels"])},
    }
    print(json.dumps(result))
    return 0


# --arch neburax: a state-space layer with a dense feed-forward, a layer of chunked attention beside a gated
# recurrence with routed experts, a state-space layer with routed experts, and the second layer's tensors once more
NEBURAX_SIZES = {
    "s": dict(width=2048, ssm_heads=32, ssm_vdim=128, state=128, groups=8, heads=16, kv_heads=4, dim=128, vdim=128,
              chunk=1024, rec_width=2048, rec_blocks=8, experts=32, identity=2, top=4, ff=1024, shared=1024,
              dense_ff=4096, vocab=32768),
    "m": dict(width=3072, ssm_heads=48, ssm_vdim=128, state=128, groups=8, heads=24, kv_heads=4, dim=128, vdim=128,
              chunk=2048, rec_width=3072, rec_blocks=12, experts=64, identity=2, top=6, ff=1024, shared=2048,
              dense_ff=6144, vocab=65536),
}


def neburax_main(args, pk) -> int:
    import torch

    import brolm_b200 as bb

    name = args.size if args.size in NEBURAX_SIZES else "s"
    z = NEBURAX_SIZES[name]
    dev = "cuda:0"
    torch.cuda.set_device(0)
    W = z["width"]
    moe = dict(kind="moe", expert=dict(ff=z["ff"]), router=dict(experts=z["experts"], top=z["top"], identity=z["identity"]),
               shared=dict(ff=z["shared"]))
    ssm = dict(heads=z["ssm_heads"], vdim=z["ssm_vdim"], state=z["state"], groups=z["groups"], norm_groups=z["groups"], conv=4)
    pair = dict(left=dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["dim"], vdim=z["vdim"], scale=z["dim"] ** -0.5,
                          mask=dict(size=z["chunk"])),
                right=dict(width=z["rec_width"], blocks=z["rec_blocks"], conv=4), left_scale=1.0, right_scale=1.0)
    layers = [dict(type="mamba2", mixer=ssm, mlp=dict(kind="dense", ff=z["dense_ff"])),
              dict(type="parallel", mixer=pair, mlp=moe), dict(type="mamba2", mixer=ssm, mlp=moe),
              dict(type="parallel", mixer=pair, mlp=moe, weights_of=1)]
    ncfg = bb.NeburaxConfig.from_dict(dict(architecture="Neburax", vocab=z["vocab"], width=W, layers=layers,
                                           norm=dict(eps=1e-5)))
    runs = len(layers)
    inter = ((z["top"] * z["ff"] + z["shared"]) + 255) // 256 * 256         # a token's active feed-forward width
    gcfg = bb.Gemma2Config(vocab_size=z["vocab"], hidden_size=W, intermediate_size=inter, num_hidden_layers=runs,
                           num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"], head_dim=z["dim"],
                           query_pre_attn_scalar=float(z["dim"]), sliding_window=z["chunk"],
                           layer_types=("sliding_attention",) * runs, max_position_embeddings=8192)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    steps, warmup, batch, context, prompt_len = args.steps or 64, max(args.warmup, 3), args.batch or 8, 1280, 2048
    common = (dev, flush, steps, warmup, batch, context, prompt_len)
    b, gm = measure_design(ncfg, z["vocab"], *common), measure_design(gcfg, z["vocab"], *common)
    T, top, ff, H, G, d, dv, C = prompt_len, z["top"], z["ff"], z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["chunk"]
    full, part = divmod(T, C)
    keys = full * (C * (C + 1) // 2) + part * (part + 1) // 2                  # visible (query, key) pairs of a prompt
    gkeys = C * (C + 1) // 2 + (T - C) * C if T > C else T * (T + 1) // 2      # ... under a window of the same size
    nh, P, N, grp = z["ssm_heads"], z["ssm_vdim"], z["state"], z["groups"]
    inner, cols = nh * P, nh * P + 2 * grp * N
    tf, gb = pk["bf16_burst"] * 1e12, pk["hbm_gbs"] * 1e9
    # experts that a step of `batch` tokens is expected to touch (uniform choices; identity choices touch none)
    active = z["experts"] * (1.0 - (1.0 - top / (z["experts"] + z["identity"])) ** batch)
    n_pair, n_ssm, n_moe = 2, 2, 3
    # (kernel-name fragment, work of all its launches in one pass over the layers, bound)
    rows = [
        ("neburax prefill", b["prefill_kernels"], [
            ("grouped_tc_kernel", n_moe * 2.0 * T * top * ff * W * 3, "flops"),
            ("attn_prefill", n_pair * 2.0 * H * (d + dv) * keys, "flops"),
            ("attn_simt", n_pair * 2.0 * H * (d + dv) * keys, "flops"),
            ("ssm_", n_ssm * T * (cols + inner + nh) * 4.0, "bytes"),
            ("gated_scan", n_pair * T * z["rec_width"] * (4 * 4.0 + 2), "bytes"),
        ]),
        ("closest prefill", gm["prefill_kernels"], [
            ("gemm_tc2_kernel<1>", runs * 2.0 * T * W * 2 * inter, "flops"),
            ("attn_prefill_tc", runs * 4.0 * H * d * gkeys, "flops"),
        ]),
        ("neburax decode", b["decode_kernels"], [
            ("fast_kernel<64, 64, 4, false>", n_moe * active * ff * W * 2.0 * 3, "bytes"),
            ("attn_decode", n_pair * batch * min(context, C) * G * (d + dv) * 2.0, "bytes"),
            ("attn_simt", n_pair * batch * min(context, C) * G * (d + dv) * 2.0, "bytes"),
            ("ssm_", n_ssm * batch * nh * P * N * 4.0 * 2, "bytes"),
        ]),
        ("closest decode", gm["decode_kernels"], [
            ("skinny_kernel<2, 1, 1>", runs * 2 * inter * W * 2.0, "bytes"),
            ("attn_decode_mma", runs * batch * min(context, C) * 2 * G * d * 2.0, "bytes"),
        ]),
    ]
    table = []
    for title, kern, wanted in rows:
        for frag, work, bound in wanted:
            us = sum(v["us"] for k, v in kern.items() if frag in k)
            n = sum(v["n"] for k, v in kern.items() if frag in k)
            if not n:
                continue
            frac = work / (us * 1e-6) / (tf if bound == "flops" else gb)
            table.append({"step": title, "kernel": frag, "launches": n, "us": round(us, 2),
                          "bound": "tensor" if bound == "flops" else "hbm", "frac_of_measured_peak": round(frac, 4)})
    result = {
        "metric": f"Neburax decode tokens/s (size {name}, batch {batch}, context {context}) beside Gemma 2 at equal sizes",
        "value": round(batch * 1000.0 / b["decode_ms"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(b["decode_ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "brolm_b200", "clocks": b["clocks"], "gpu_launches": b["launches"],
        "config": {"model": "Neburax", **{k: v for k, v in z.items()}, "layer_runs": runs, "global_batch": batch,
                   "seq_len": context, "closest": {"model": "Gemma 2", "hidden": W, "heads": H, "kv_heads": G,
                                                   "head_dim": d, "intermediate": inter, "layers": runs,
                                                   "sliding_window": C},
                   "l2": "the prompt is timed after an L2 flush; a decode step reads more than the L2 holds",
                   "peaks": pk["source"]},
        "neburax": {"prefill_tok_s": round(T * 1000.0 / b["prefill_ms"], 1), "prefill_ms": round(b["prefill_ms"], 3),
                    "decode_tok_s": round(batch * 1000.0 / b["decode_ms"], 1), "decode_ms": round(b["decode_ms"], 4)},
        "closest": {"prefill_tok_s": round(T * 1000.0 / gm["prefill_ms"], 1), "prefill_ms": round(gm["prefill_ms"], 3),
                    "decode_tok_s": round(batch * 1000.0 / gm["decode_ms"], 1), "decode_ms": round(gm["decode_ms"], 4)},
        "kernels": table,
        "by_kernel_us": {"neburax_prefill": _top(b["prefill_kernels"], 24), "closest_prefill": _top(gm["prefill_kernels"]),
                         "neburax_decode": _top(b["decode_kernels"], 24), "closest_decode": _top(gm["decode_kernels"])},
    }
    print(json.dumps(result))
    return 0


# --arch kedasun: rotary layers (values mixed across layers) alternating with windowed layers that keep a sequence's
# first keys (short convolutions, unit-norm heads, distance slopes, mixed heads' weights, a gate per head), each with a
# dense clamped feed-forward between grouped norms
KEDASUN_SIZES = {
    "s": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, rot=64, window=1024, keep_first=4, conv=4, ff=8192,
              groups=4, vocab=32768),
    "m": dict(width=3072, heads=24, kv_heads=8, dim=128, vdim=64, rot=64, window=2048, keep_first=8, conv=3, ff=12288,
              groups=8, vocab=65536),
}


def kedasun_main(args, pk) -> int:
    import torch

    import brolm_b200 as bb

    name = args.size if args.size in KEDASUN_SIZES else "s"
    z = KEDASUN_SIZES[name]
    dev = "cuda:0"
    torch.cuda.set_device(0)
    W, H, G, d, dv, ff, win = z["width"], z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["ff"], z["window"]
    mlp = dict(kind="dense", ff=ff, limit=7.0)
    rotary = dict(type="attention", mlp=mlp,
                  mixer=dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=d ** -0.5, rot=dict(base=10000.0, dims=z["rot"]),
                             v_mix=True))
    windowed = dict(type="attention_2", mlp=mlp,
                    mixer=dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=d ** -0.5, conv=z["conv"],
                               mask=dict(size=win, keep_first=z["keep_first"]), v_mix=True))
    layers = [rotary, windowed, rotary, windowed]
    kcfg = bb.KedasunConfig.from_dict(dict(architecture="Kedasun", vocab=z["vocab"], width=W, layers=layers,
                                           embedding=dict(scale=1.0), norm=dict(eps=1e-5, groups=z["groups"])))
    runs = len(layers)
    gcfg = bb.Gemma2Config(vocab_size=z["vocab"], hidden_size=W, intermediate_size=ff, num_hidden_layers=runs,
                           num_attention_heads=H, num_key_value_heads=G, head_dim=d, query_pre_attn_scalar=float(d),
                           sliding_window=win, layer_types=("full_attention", "sliding_attention") * (runs // 2),
                           max_position_embeddings=8192)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    steps, warmup, batch = args.steps or 64, max(args.warmup, 3), args.batch or 8
    context, prompt_len = args.context or 2304, 2048
    common = (dev, flush, steps, warmup, batch, context, prompt_len)
    b, gm = measure_design(kcfg, z["vocab"], *common), measure_design(gcfg, z["vocab"], *common)
    T = prompt_len
    full = T * (T + 1) // 2                                                   # visible (query, key) pairs, every key
    wkeys = win * (win + 1) // 2 + (T - win) * win if T > win else full       # ... under a window
    kept = sum(min(z["keep_first"], max(0, p + 1 - win)) for p in range(T))   # ... and the kept first keys beyond it
    tf, gb = pk["bf16_burst"] * 1e12, pk["hbm_gbs"] * 1e9
    n_rot, n_win = 2, 2
    cols = H * d + G * d + G * dv
    dec_full = batch * context * G * (d + dv) * 2.0
    dec_win = batch * min(context, win + z["keep_first"]) * G * (d + dv) * 2.0
    # (kernel-name fragment, work of all its launches in one pass over the layers, bound)
    rows = [
        ("kedasun prefill", b["prefill_kernels"], [
            ("gemm_tc2_kernel<1>", runs * 2.0 * T * W * 2 * ff, "flops"),
            ("attn_prefill", n_rot * 2.0 * H * (d + dv) * full, "flops"),
            ("attn_headmix_prefill", n_win * 2.0 * H * (d + dv) * (wkeys + kept), "flops"),
            ("attn_simt", n_rot * 2.0 * H * (d + dv) * full, "flops"),
            ("attn_all_values", n_win * 2.0 * H * (d + G * dv) * (wkeys + kept), "flops"),
            ("qkv_finish", runs * T * cols * (4.0 + 2.0 + 2.0), "bytes"),
            ("causal_conv", n_win * T * cols * 8.0, "bytes"),
            ("group_norm", 4 * runs * T * W * 8.0, "bytes"),
        ]),
        ("closest prefill", gm["prefill_kernels"], [
            ("gemm_tc2_kernel<1>", runs * 2.0 * T * W * 2 * ff, "flops"),
            ("attn_prefill", n_rot * 4.0 * H * d * full + n_win * 4.0 * H * d * wkeys, "flops"),
            ("rope_kv_write", runs * T * (H * d + 2 * G * d) * (2.0 + 2.0 + 2.0), "bytes"),
            ("rmsnorm", 4 * runs * T * W * 8.0, "bytes"),
        ]),
        ("kedasun decode", b["decode_kernels"], [
            ("skinny_kernel<2, 1, 1>", runs * 2 * ff * W * 2.0, "bytes"),
            ("attn_decode", n_rot * dec_full, "bytes"),
            ("attn_headmix_decode", n_win * dec_win, "bytes"),
            ("attn_simt", n_rot * dec_full, "bytes"),
            ("attn_all_values", n_win * dec_win, "bytes"),
        ]),
        ("closest decode", gm["decode_kernels"], [
            ("skinny_kernel<2, 1, 1>", runs * 2 * ff * W * 2.0, "bytes"),
            ("attn_decode_mma", (n_rot * batch * context + n_win * batch * min(context, win)) * 2 * G * d * 2.0, "bytes"),
        ]),
    ]
    table = []
    for title, kern, wanted in rows:
        for frag, work, bound in wanted:
            us = sum(v["us"] for k, v in kern.items() if frag in k)
            n = sum(v["n"] for k, v in kern.items() if frag in k)
            if not n:
                continue
            frac = work / (us * 1e-6) / (tf if bound == "flops" else gb)
            table.append({"step": title, "kernel": frag, "launches": n, "us": round(us, 2),
                          "bound": "tensor" if bound == "flops" else "hbm", "frac_of_measured_peak": round(frac, 4)})
    result = {
        "metric": f"Kedasun decode tokens/s (size {name}, batch {batch}, context {context}) beside Gemma 2 at equal sizes",
        "value": round(batch * 1000.0 / b["decode_ms"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(b["decode_ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "brolm_b200", "clocks": b["clocks"], "gpu_launches": b["launches"],
        "config": {"model": "Kedasun", **{k: v for k, v in z.items()}, "layer_runs": runs, "global_batch": batch,
                   "seq_len": context, "prompt": prompt_len,
                   "closest": {"model": "Gemma 2", "hidden": W, "heads": H, "kv_heads": G, "head_dim": d,
                               "intermediate": ff, "layers": runs, "sliding_window": win},
                   "l2": "the prompt is timed after an L2 flush; a decode step reads more than the L2 holds",
                   "peaks": pk["source"]},
        "kedasun": {"prefill_tok_s": round(T * 1000.0 / b["prefill_ms"], 1), "prefill_ms": round(b["prefill_ms"], 3),
                    "decode_tok_s": round(batch * 1000.0 / b["decode_ms"], 1), "decode_ms": round(b["decode_ms"], 4)},
        "closest": {"prefill_tok_s": round(T * 1000.0 / gm["prefill_ms"], 1), "prefill_ms": round(gm["prefill_ms"], 3),
                    "decode_tok_s": round(batch * 1000.0 / gm["decode_ms"], 1), "decode_ms": round(gm["decode_ms"], 4)},
        "kernels": table,
        "by_kernel_us": {"kedasun_prefill": _top(b["prefill_kernels"], 24), "closest_prefill": _top(gm["prefill_kernels"]),
                         "kedasun_decode": _top(b["decode_kernels"], 24), "closest_decode": _top(gm["decode_kernels"])},
    }
    print(json.dumps(result))
    return 0


# --arch ritirax: a lightning layer with a dense feed-forward, a capped attention layer, a latent attention layer and a
# second lightning layer, the last three with routed experts (the sizes of the Neburax run of the same letter; the
# latent layer has sixteen heads, the most a decode tile of the tensor-core kernel has rows for)
RITIRAX_SIZES = {
    "s": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, lat_heads=16, lat_dim=64, lat_rot=64, lat_vdim=64, kv_rank=192,
              experts=32, groups=8, keep=4, top=4, ff=1024, shared=1024, dense_ff=4096, vocab=32768),
    "m": dict(width=3072, heads=24, kv_heads=4, dim=128, vdim=128, lat_heads=16, lat_dim=128, lat_rot=64, lat_vdim=128, kv_rank=192,
              experts=64, groups=8, keep=4, top=6, ff=1024, shared=2048, dense_ff=6144, vocab=65536),
}


def ritirax_main(args, pk) -> int:
    import torch

    import brolm_b200 as bb

    name = args.size if args.size in RITIRAX_SIZES else "s"
    z, nz = RITIRAX_SIZES[name], NEBURAX_SIZES[name]
    dev = "cuda:0"
    torch.cuda.set_device(0)
    W, H, G, d, dv = z["width"], z["heads"], z["kv_heads"], z["dim"], z["vdim"]
    moe = dict(kind="moe", expert=dict(ff=z["ff"]), shared=dict(ff=z["shared"]),
               router=dict(experts=z["experts"], top=z["top"], scale=2.0, groups=dict(count=z["groups"], keep=z["keep"])))
    decay = [1.0 - 2.0 ** (-3.0 - 7.0 * h / max(H - 1, 1)) for h in range(H)]
    light = dict(heads=H, dim=d, vdim=dv, decay=decay)
    attn = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=d ** -0.5, softcap=30.0, bias_max=128, bias_rows=32)
    lat = dict(heads=z["lat_heads"], dim=z["lat_dim"], rot_dim=z["lat_rot"], vdim=z["lat_vdim"], kv_rank=z["kv_rank"],
               scale=(z["lat_dim"] + z["lat_rot"]) ** -0.5,
               rot=dict(base=10000.0, dims=z["lat_rot"], scaling=dict(factor=8.0, original=1024, fast=32.0, slow=1.0)))
    layers = [dict(type="lightning", mixer=light, mlp=dict(kind="dense", ff=z["dense_ff"])),
              dict(type="attention", mixer=attn, mlp=moe), dict(type="latent_attention", mixer=lat, mlp=moe),
              dict(type="lightning", mixer=light, mlp=moe)]
    rcfg = bb.RitiraxConfig.from_dict(dict(architecture="Ritirax", vocab=z["vocab"], width=W, layers=layers,
                                           norm=dict(eps=1e-5), embedding=dict(scale=W ** 0.5)))
    # the closest design at the same sizes: the Neburax run of the same letter
    nmoe = dict(kind="moe", expert=dict(ff=nz["ff"]), router=dict(experts=nz["experts"], top=nz["top"], identity=nz["identity"]),
                shared=dict(ff=nz["shared"]))
    ssm = dict(heads=nz["ssm_heads"], vdim=nz["ssm_vdim"], state=nz["state"], groups=nz["groups"], norm_groups=nz["groups"], conv=4)
    pair = dict(left=dict(heads=nz["heads"], kv_heads=nz["kv_heads"], dim=nz["dim"], vdim=nz["vdim"], scale=nz["dim"] ** -0.5,
                          mask=dict(size=4096)),
                right=dict(width=nz["rec_width"], blocks=nz["rec_blocks"], conv=4), left_scale=1.0, right_scale=1.0)
    nlayers = [dict(type="mamba2", mixer=ssm, mlp=dict(kind="dense", ff=nz["dense_ff"])),
               dict(type="parallel", mixer=pair, mlp=nmoe), dict(type="mamba2", mixer=ssm, mlp=nmoe),
               dict(type="parallel", mixer=pair, mlp=nmoe, weights_of=1)]
    ncfg = bb.NeburaxConfig.from_dict(dict(architecture="Neburax", vocab=nz["vocab"], width=W, layers=nlayers,
                                           norm=dict(eps=1e-5)))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    steps, warmup, batch, context, prompt_len = args.steps or 64, max(args.warmup, 3), args.batch or 8, 1280, 2048
    common = (dev, flush, steps, warmup, batch, context, prompt_len)
    r, nb = measure_design(rcfg, z["vocab"], *common), measure_design(ncfg, z["vocab"], *common)
    T, top, ff = prompt_len, z["top"], z["ff"]
    keys = T * (T + 1) // 2                                                    # visible (query, key) pairs of a prompt
    row = (z["kv_rank"] + z["lat_rot"] + 15) // 16 * 16                        # the cached row of the latent layer
    nh, P, N, grp = nz["ssm_heads"], nz["ssm_vdim"], nz["state"], nz["groups"]
    inner, cols = nh * P, nh * P + 2 * grp * N
    tf, gb = pk["bf16_burst"] * 1e12, pk["hbm_gbs"] * 1e9
    active = z["experts"] * (1.0 - (1.0 - top / z["experts"]) ** batch)
    nactive = nz["experts"] * (1.0 - (1.0 - nz["top"] / (nz["experts"] + nz["identity"])) ** batch)
    # (kernel-name fragment, work of all its launches in one pass over the layers, bound)
    rows = [
        ("ritirax prefill", r["prefill_kernels"], [
            ("grouped_tc_kernel", 3 * 2.0 * T * top * ff * W * 3, "flops"),
            ("attn_headmix_prefill", 2.0 * H * (d + dv) * keys, "flops"),
            (f"attn_prefill_mma_kernel<{d}", 2.0 * H * (d + dv) * keys, "flops"),
            (f"attn_prefill_mma_kernel<{row}", 2.0 * z["lat_heads"] * 2 * row * keys, "flops"),
            ("decay_scan", 2 * T * (H * (2 * d + dv) + H * dv) * 4.0, "bytes"),
        ]),
        ("closest prefill", nb["prefill_kernels"], [
            ("grouped_tc_kernel", 3 * 2.0 * T * nz["top"] * nz["ff"] * W * 3, "flops"),
            ("attn_prefill", 2 * 2.0 * nz["heads"] * (nz["dim"] + nz["vdim"]) * keys, "flops"),
            ("ssm_", 2 * T * (cols + inner + nh) * 4.0, "bytes"),
            ("gated_scan", 2 * T * nz["rec_width"] * (4 * 4.0 + 2), "bytes"),
        ]),
        ("ritirax decode", r["decode_kernels"], [
            ("fast_kernel<64, 64, 4, false>", 3 * active * ff * W * 2.0 * 3, "bytes"),
            ("attn_headmix_decode", batch * context * G * (d + dv) * 2.0, "bytes"),
            (f"attn_decode_mma_kernel<{d}", batch * context * G * (d + dv) * 2.0, "bytes"),
            (f"attn_decode_mma_kernel<{row}", batch * context * row * 2.0, "bytes"),
            ("decay_scan", 2 * batch * H * d * dv * 4.0 * 2, "bytes"),
        ]),
        ("closest decode", nb["decode_kernels"], [
            ("fast_kernel<64, 64, 4, false>", 3 * nactive * nz["ff"] * W * 2.0 * 3, "bytes"),
            ("attn_decode", 2 * batch * context * nz["kv_heads"] * (nz["dim"] + nz["vdim"]) * 2.0, "bytes"),
            ("ssm_", 2 * batch * nh * P * N * 4.0 * 2, "bytes"),
        ]),
    ]
    table = []
    for title, kern, wanted in rows:
        for frag, work, bound in wanted:
            us = sum(v["us"] for k, v in kern.items() if frag in k)
            n = sum(v["n"] for k, v in kern.items() if frag in k)
            if not n:
                continue
            frac = work / (us * 1e-6) / (tf if bound == "flops" else gb)
            table.append({"step": title, "kernel": frag, "launches": n, "us": round(us, 2),
                          "bound": "tensor" if bound == "flops" else "hbm", "frac_of_measured_peak": round(frac, 4)})
    result = {
        "metric": f"Ritirax decode tokens/s (size {name}, batch {batch}, context {context}) beside Neburax at equal sizes",
        "value": round(batch * 1000.0 / r["decode_ms"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(r["decode_ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "brolm_b200", "clocks": r["clocks"], "gpu_launches": r["launches"],
        "config": {"model": "Ritirax", **{k: v for k, v in z.items()}, "layers": len(layers), "global_batch": batch,
                   "seq_len": context, "closest": {"model": "Neburax", **{k: v for k, v in nz.items()}},
                   "l2": "the prompt is timed after an L2 flush; a decode step reads more than the L2 holds",
                   "peaks": pk["source"]},
        "ritirax": {"prefill_tok_s": round(T * 1000.0 / r["prefill_ms"], 1), "prefill_ms": round(r["prefill_ms"], 3),
                    "decode_tok_s": round(batch * 1000.0 / r["decode_ms"], 1), "decode_ms": round(r["decode_ms"], 4)},
        "closest": {"prefill_tok_s": round(T * 1000.0 / nb["prefill_ms"], 1), "prefill_ms": round(nb["prefill_ms"], 3),
                    "decode_tok_s": round(batch * 1000.0 / nb["decode_ms"], 1), "decode_ms": round(nb["decode_ms"], 4)},
        "kernels": table,
        "by_kernel_us": {"ritirax_prefill": _top(r["prefill_kernels"], 28), "closest_prefill": _top(nb["prefill_kernels"], 24),
                         "ritirax_decode": _top(r["decode_kernels"], 28), "closest_decode": _top(nb["decode_kernels"], 24)},
    }
    print(json.dumps(result))
    return 0


def _by_kernel(events) -> dict:
    """Device records -> {kernel name: {"us": total time, "n": launches}}."""
    out: dict = {}
    for e in events:
        name = e.name.replace("void ", "").replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
        name = name.split("(")[0][:72]
        d = out.setdefault(name, {"us": 0.0, "n": 0})
        d["us"] += e.time_range.end - e.time_range.start
        d["n"] += 1
    return out


def _top(kern: dict, n: int = 14) -> dict:
    return {k: [round(v["us"], 1), v["n"]] for k, v in sorted(kern.items(), key=lambda kv: -kv[1]["us"])[:n]}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="gemma2", choices=["gemma2", "banevik", "neburax", "kedasun", "ritirax"],
                    help="banevik, neburax, kedasun: that design at real layer sizes beside Gemma 2 at equal sizes (--size s|m); "
                         "ritirax: beside Neburax at equal sizes")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="decode steps in a timed region (default 64; 128 for 9b)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="brolm_b200")
    ap.add_argument("--size", default="2b", choices=sorted(SIZES) + sorted(BANEVIK_SIZES))
    ap.add_argument("--batch", type=int, default=0, help="sequences of the headline run (default: the workload's)")
    ap.add_argument("--context", type=int, default=0,
                    help="tokens a sequence holds after the last timed step (default 8192; 2304 for 27b)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all)")
    ap.add_argument("--repeats", type=int, default=REPEATS, help="timed regions of K steps each; value = their median")
    ap.add_argument("--no-points", action="store_true", help="skip the other batch sizes and the prefill measurement")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "wlejon/brolm is a C++ project without a Python "
                          "package (pip: neither setup.py nor pyproject.toml) and needs the absent sibling library "
                          "brotensor to build; it also has no batched Gemma 2 decode to time"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: brolm_b200 is a one-GPU library; --gpus {args.gpus} is not supported")
        return 2
    if args.arch == "banevik":
        return banevik_main(args, peaks())
    if args.arch == "neburax":
        return neburax_main(args, peaks())
    if args.arch == "kedasun":
        return kedasun_main(args, peaks())
    if args.arch == "ritirax":
        return ritirax_main(args, peaks())
    if args.size not in SIZES:
        print(f"bench.py: --size {args.size} goes with --arch banevik, neburax or kedasun")
        return 2
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    steps = args.steps or (128 if args.size == "9b" else 64)
    context = args.context or (2048 + 256 if args.size == "27b" else 8192)

    import torch

    import brolm_b200 as bb
    from brolm_b200 import kernels

    pk = peaks()
    cfg = bb.Gemma2Config(**SIZES[args.size])
    full_layers = cfg.num_hidden_layers
    if args.layers:
        cfg.num_hidden_layers = args.layers
    layers = cfg.num_hidden_layers
    dev = "cuda:0"
    torch.cuda.set_device(0)
    model = bb.Model(cfg, dtype="bfloat16", device=dev).init_random(seed=0, on_device=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # larger than the 126 MB L2

    def decode_run(prompt_lengths, steps: int, warmup: int, repeats: int, e2e: bool):
        """Decode after one prefill step of prompts of ``prompt_lengths``: SETTLE + ``warmup`` untimed
        steps, then ``repeats`` timed regions of ``steps`` steps each.

        A step reads every weight and the live cache once, gigabytes against an L2 of 126 MB, so
        nothing of one step is still cached for the next and no flush is put between steps.
        Device timing: the generation loop's own steps (``Engine.step_from``: the ids a step's sampler
        drew feed the next step on the device), queued without reading anything back, CUDA events
        around each region.  End to end (``e2e``): ``brolm_b200.generate`` with host token ids in and
        out; every step copies its description from pinned host memory to the device and reads the
        sampled ids back; host clock between the callbacks that follow those reads."""
        batch = len(prompt_lengths)
        warmup += SETTLE
        total = warmup + repeats * steps
        longest = max(prompt_lengths) + total + 1
        need = sum((n + total + 1 + 63) // 64 * 64 for n in prompt_lengths)
        engine = bb.Engine(model, max_tokens=need, max_slots=batch, max_seq_len=longest)
        g = torch.Generator().manual_seed(42)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in prompt_lengths]
        opts = bb.GenerateOptions(max_new_tokens=total + 1, sampling=bb.SamplingParams(temperature=0.0),
                                  stop_on_eos=False)
        e2e_tok_s = None
        with ClockSampler() as clocks:
            if e2e:
                stamps: list[float] = []
                # called after each step's tokens reached the host; call 0 follows the prefill
                out = bb.generate(engine, prompts, eos_id=-1, opts=opts,
                                  on_step=lambda produced, active: stamps.append(time.perf_counter()))
                torch.cuda.synchronize()
                assert all(len(o) == total + 1 for o in out)
                rates = [batch * steps / (stamps[warmup + (r + 1) * steps] - stamps[warmup + r * steps])
                         for r in range(repeats)]
                e2e_tok_s = statistics.median(rates)

            sampler = bb.Sampler(opts.sampling)
            streams = torch.arange(batch, dtype=torch.int32, device=dev)
            pick = list(range(batch))
            slots = engine.open(batch)
            logits = engine.step(slots, prompts)
            ids = sampler(logits, streams, 0)
            marks, launches = [], []
            for i in range(total):
                if i >= warmup and (i - warmup) % steps == 0:
                    ev = torch.cuda.Event(enable_timing=True)
                    ev.record()
                    marks.append(ev)
                    launches.append(kernels.launch_count())
                logits = engine.step_from(slots, ids, pick)
                ids = sampler(logits, streams, i + 1)
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append(ev)
            launches.append(kernels.launch_count())
            torch.cuda.synchronize()
            engine.close(slots)
        region_ms = [marks[r].elapsed_time(marks[r + 1]) / steps for r in range(repeats)]
        # what each region had to read: the lengths at its middle step
        region_bytes = [decode_bytes(cfg, layers, [n + 1 + warmup + r * steps + steps // 2 for n in prompt_lengths])
                        for r in range(repeats)]
        gbs = [b / (ms * 1e-3) / 1e9 for b, ms in zip(region_bytes, region_ms)]
        ms = statistics.median(region_ms)
        return {"tok_s": batch * 1000.0 / ms, "ms": ms, "best_tok_s": batch * 1000.0 / min(region_ms),
                "e2e_tok_s": e2e_tok_s, "launches": launches[1] - launches[0], "clocks": clocks.summary(),
                "h2d": engine.last_h2d_bytes, "d2h": 4 * batch, "gbs": statistics.median(gbs),
                "bytes": statistics.median(region_bytes), "final": [n + total + 1 for n in prompt_lengths]}

    def equal_prompts(batch: int, context: int, steps: int, warmup: int, repeats: int):
        """Prompts such that the last timed step ends at ``context`` tokens."""
        return [context - (SETTLE + warmup + repeats * steps) - 1] * batch

    def prefill_run(lengths):
        """One prefill step of prompts of ``lengths`` (logits of each last token), the median of three
        after three untimed ones, the L2 flushed before each."""
        need = sum((n + 63) // 64 * 64 for n in lengths) + 64
        engine = bb.Engine(model, max_tokens=need, max_slots=len(lengths), max_seq_len=max(lengths) + 1)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lengths]
        times = []
        for it in range(3 + 3):
            slots = engine.open(len(lengths))
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step(slots, prompts)
            e1.record()
            torch.cuda.synchronize()
            engine.close(slots)
            if it >= 3:
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        fl = prefill_flops(cfg, layers, list(lengths))
        T = sum(lengths)
        return {"value": round(T * 1000.0 / ms, 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(fl / (ms * 1e-3) / (pk["bf16_burst"] * 1e12), 4),
                "frac_sustained": round(fl / (ms * 1e-3) / (pk["bf16_sustained"] * 1e12), 4),
                "tflops": round(fl / (ms * 1e-3) / 1e12, 1), "peak": pk["bf16_burst"],
                "of": f"{pk['source']} bf16 burst peak (the step is timed alone after an L2 flush)"}

    if args.size == "9b":
        g = torch.Generator().manual_seed(9)
        prompt_lengths = torch.randint(128, 6144 + 1, (args.batch or 16,), generator=g).tolist()
        what = f"{len(prompt_lengths)} prompts of 128 to 6144 tokens"
    else:
        batch = args.batch or 8
        prompt_lengths = equal_prompts(batch, context, steps, args.warmup, args.repeats)
        what = f"batch {batch}, context {context}"
    main_run = decode_run(prompt_lengths, steps, args.warmup, args.repeats, e2e=True)
    name = {"2b": "Gemma 2 2B", "9b": "Gemma 2 9B", "27b": "Gemma 2 27B"}[args.size]

    result = {
        "metric": f"decode tokens/s ({name} sizes, {what})",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0, 0.02), uniform random token ids)",
        "impl": "brolm_b200",
        "config": {"model": f"gemma-2-{args.size} sizes", "layers": layers, "layers_of_configuration": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "sliding_window": cfg.sliding_window, "global_batch": len(prompt_lengths),
                   "seq_len": max(main_run["final"]), "seq_len_min": min(main_run["final"]),
                   "parallelism": "none (1 GPU)", "settle_steps": SETTLE, "repeats": args.repeats,
                   "l2": f"inputs larger than L2 ({main_run['bytes'] / 1e9:.1f} GB read per step)",
                   "peaks": pk["source"]},
        "clocks": main_run["clocks"],
        "repeats": {"n": args.repeats, "median": round(main_run["tok_s"], 1), "best": round(main_run["best_tok_s"], 1)},
        "e2e": {"value": round(main_run["e2e_tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": main_run["h2d"],
                "d2h_bytes_per_step": main_run["d2h"]},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(main_run["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main_run["gbs"] / pk["hbm_gbs"], 4), "of": pk["source"]},
    }

    if not args.no_points:
        points, fracs, best = {}, {}, {}

        def point(key: str, lengths, k: int) -> None:
            r = decode_run(lengths, k, 3, args.repeats, e2e=False)
            points[key] = round(r["tok_s"], 1)
            best[key] = round(r["best_tok_s"], 1)
            fracs[key] = round(r["gbs"] / pk["hbm_gbs"], 4)

        if args.size == "2b":
            for b in (1, 64):
                point(f"decode_b{b}", equal_prompts(b, context, 64, 3, args.repeats), 64)
            # the workload of the configuration's own description: prompts of 1,024 tokens, 256 generated
            for b in (1, 8, 64):
                point(f"decode_b{b}_ctx1280", equal_prompts(b, 1024 + 256, 64, 3, args.repeats), 64)
        elif args.size == "27b":
            # prompts of 2,048 tokens, 256 generated
            point("decode_b1", equal_prompts(1, context, 64, 3, args.repeats), 64)
        result["points"] = points
        result["points_best"] = best
        result["points_roofline"] = fracs
        result["prefill"] = prefill_run(prompt_lengths if args.size == "9b" else [2048])
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
