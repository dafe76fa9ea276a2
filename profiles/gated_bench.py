"""Prefill / decode throughput of the Fegolorn decoder (gated, normed and scaled sublayer results; attention with rotated values;
windowed latent attention with an output gate; clamped gated feed-forward and experts chosen by logit; layers that borrow weights)
beside Tafopel, Tipetar and Qwen3 at equal width, depth and feed-forward size, plus a per-kernel roofline table of its kernels and
their counterparts in those models (``python bench.py --gated``).

Same rules as hybrid_bench.py, whose engine set-up, throughput loop and timing helper it uses: random weights, synthetic token
ids, device time between CUDA events after warm-up, a 256 MB write between the timed launches of the per-kernel table.
"""
from __future__ import annotations

import json
import os
import sys
import time

import hybrid_bench as hb
import window_bench as wb  # noqa: F401  (registers Tipetar with the throughput loop)

ROOT = hb.ROOT
VOCAB = hb.VOCAB

SIZES = {
    # name: (width, heads, kv_heads, kv_rank, window, experts, top)  -- head size 128, rotated part 64; eight layers, of which the last two
    # run with the weights of layers 2 and 3; Tafopel / Tipetar / Qwen3 beside it: hybrid_bench.SIZES, window_bench.SIZES
    "w1024": (1024, 16, 8, 256, 1024, 16, 2),
    "w2048": (2048, 16, 8, 512, 2048, 32, 4),
}


def fegolorn_config(size: str):
    from nanovllm.models.fegolorn import FegolornConfig
    width, H, G, R, window, E, top = SIZES[size]
    lat = {"type": "latent_attention", "mixer": {"heads": H, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": R, "scale": 192 ** -0.5,
                                                 "mask": {"size": window}, "rot": {"dims": 64, "base": 5e4}}}
    att = {"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                          "rot": {"dims": 64, "base": 5e5, "scaling": {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 8192}}}}
    dense = {"kind": "dense", "ff": 3 * width, "limit": 7.0}
    moe = {"kind": "moe", "router": {"experts": E, "top": top}, "expert": {"ff": 3 * width // (2 * top)}, "shared": {"ff": width}}
    layers = [dict(lat, mlp=dense), dict(att, mlp=moe), dict(lat, mlp=dense), dict(att, mlp=moe), dict(lat, mlp=dense), dict(att, mlp=moe)]
    layers += [dict(layers[2], weights_of=2), dict(layers[3], weights_of=3)]
    return FegolornConfig({"architecture": "Fegolorn", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6}, "logit_softcap": 50.0,
                           "embedding": {"scale": width ** 0.5, "bigram": {"buckets": 65521, "mul_prev": 40503, "mul_cur": 9973}},
                           "layers": layers})


hb.EXTRA_KINDS["fegolorn"] = fegolorn_config


def kernel_table(size: str, peaks: dict):
    import torch
    from nanovllm import mixops
    from nanovllm.layers.rotary_embedding import build_banded_cos_sin, build_interleaved_cos_sin
    width, H, G, R, window, E, top = SIZES[size]
    d, rd, bs, dev, bf = 128, 64, 256, "cuda", torch.bfloat16
    hbm, tc = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    fma = 148 * 128 * 2 * 1.9e9
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    rows = []

    def add(name, fn, nbytes, flops, pipe="hbm"):
        t = hb.timed(fn, flush)
        peak = tc if pipe == "tensor" else fma
        roof = max(nbytes / hbm, flops / peak if flops else 0.0)
        rows.append(dict(kernel=name, us=round(t * 1e6, 1), gbs=round(nbytes / t / 1e9, 1), tflops=round(flops / t / 1e12, 2),
                         bound="hbm" if nbytes / hbm >= (flops / peak if flops else 0) else pipe, of_roofline=round(roof / t, 3)))

    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *s, dt=bf: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(dt)

    def spans(S, q, k):
        if q > 1:
            cu = torch.arange(0, S + 1, dtype=torch.int32, device=dev)
            return mixops.StepSpans(S, q, cu * q, cu * k, None)
        return mixops.StepSpans(S, 1, None, None, torch.full((S,), k, dtype=torch.int32, device=dev))

    table = build_banded_cos_sin(rd, 8192, 5e4, None, dev)
    vtab = build_banded_cos_sin(d, 8192, 5e5, None, dev)
    sink = torch.zeros(H, device=dev)
    for label, S, q, k in (("prefill 4x2048", 4, 2048, 2048), ("decode 64x4096", 64, 1, 4096)):
        nblk = S * (k // bs)
        bt = torch.arange(nblk, dtype=torch.int32, device=dev).view(S, -1)
        n = S * q
        spn = spans(S, q, k)
        # ---- latent attention: windowed without a sink (this design) and causal with a sink (Tafopel), same rows ----
        D = R + rd
        cache = rn(nblk * bs, D)
        q_lat, q_raw = rn(H, n, R), rn(n, H, d + rd)
        for win in (window, 0):
            vis = (lambda i: min(i + 1, win)) if win else (lambda i: i + 1)
            pairs = S * (sum(vis(i) for i in range(k - q, k)))
            keys_read = S * (k if q > 1 else vis(k - 1))
            flops = pairs * H * 2 * (D + R)
            nbytes = keys_read * D * 2 + n * H * (2 * R + d + rd) * 2
            name = f"latent_attention window {win}, no sink" if win else "latent_attention causal + sink (tafopel form)"
            add(f"{name} {label}", lambda: mixops.latent_attention(q_lat, q_raw, d, cache, bt, bs, spn, None if win else sink, table, 0.07, window=win,
                                                                   layout=mixops.ROT_HALVES if win else mixops.ROT_PAIRS), nbytes, flops, "tensor")
        if q == 1:                                          # Tafopel's form over as many keys as the window leaves visible: like for like
            kk = min(window, k)
            nb2 = S * (kk // bs)
            bt2 = torch.arange(nb2, dtype=torch.int32, device=dev).view(S, -1)
            add(f"latent_attention causal + sink (tafopel form) decode {S}x{kk}", lambda: mixops.latent_attention(q_lat, q_raw, d, cache, bt2, bs, spans(S, 1, kk),
                sink, table, 0.07), S * kk * D * 2 + n * H * (2 * R + d + rd) * 2, S * kk * H * 2 * (D + R), "tensor")
        # ---- grouped-query attention, causal, fp32 sums (this design; the turn back follows) and the windowed form of Tipetar ----
        cache2 = rn(nblk * bs, G * 2 * d)
        qkv = rn(n, H * d)
        for win, f32 in ((0, True), (window, False)):
            vis = (lambda i: min(i + 1, win)) if win else (lambda i: i + 1)
            pairs = S * (sum(vis(i) for i in range(k - q, k)))
            keys_read = S * (k if q > 1 else vis(k - 1))
            name = "window_attention causal, fp32 sums" if f32 else f"window_attention window {win} (tipetar form)"
            add(f"{name} {label}", lambda: mixops.window_attention(qkv, cache2, bt, bs, spn, H, G, d, d, 0.088, None, win, out_f32=f32),
                keys_read * G * 2 * d * 2 + n * H * d * 2 + n * H * d * (4 if f32 else 2), pairs * H * 4 * d, "tensor")
    # ---- row-wise kernels, 8192 rows ----
    n = 8192
    pos = torch.arange(n, dtype=torch.int64, device=dev)
    sl = torch.arange(n, dtype=torch.int32, device=dev)
    acc, gate = torch.randn(n, H, d, device=dev), rn(n, H * d)
    add("head_rotate_gate turn back 8192 rows", lambda: mixops.head_rotate_gate(acc, bf, vtab, pos, sign=-1.0), n * H * d * (4 + 2) + n * d * 4, 0)
    o_lat = rn(H, n, d)
    add("head_rotate_gate gate only 8192 rows", lambda: mixops.head_rotate_gate(o_lat.permute(1, 0, 2), bf, gate=gate), n * H * d * (2 + 2 + 2), 0)
    qk_tab = build_interleaved_cos_sin(64, 8192, 5e5, None, dev)
    proj = rn(n, (H + 2 * G) * d)
    cache3 = torch.zeros(n, G * 2 * d, dtype=bf, device=dev)
    wq, wk = rn(d), rn(d)
    for vt, name in ((vtab, "headnorm_rope_store + rotated values"), (None, "headnorm_rope_store (musavik form, unit-RMS values)")):
        add(f"{name} 8192 rows", lambda: mixops.headnorm_rope_store(proj, 0, H * d, (H + G) * d, H, G, d, d, wq, wk, vt is None, qk_tab, pos, sl, cache3, 1e-6,
                                                                   v_cos_sin=vt), n * ((2 * H + 4 * G) * d) * 2 + n * (64 + (d if vt is not None else 0)) * 4, 0)
    dkv, cache4, wn = rn(n, R + rd), torch.zeros(n, R + rd, dtype=bf, device=dev), rn(R)
    for lay, name in ((mixops.ROT_HALVES, "latent_store, half-split pairs"), (mixops.ROT_PAIRS, "latent_store, neighbour pairs (tafopel form)")):
        add(f"{name} 8192 rows", lambda: mixops.latent_store(dkv, wn, table, pos, sl, cache4, R, rd, 1e-6, layout=lay), n * (R + rd) * 4 + n * rd * 4, 0)
    x, yb, y32 = torch.randn(n, width, device=dev), rn(n, width), torch.randn(n, width, device=dev)
    wide = rn(n, 3 * width)
    w32, w32b, wb16, wb16b = torch.rand(width, device=dev), torch.rand(width, device=dev), rn(width), rn(width)
    add("gated_add_normed_norm 8192 rows", lambda: mixops.gated_add_normed_norm(x, yb, wide[:, 2 * width:], w32, 1e-6, bf, 1.0, w32b),
        n * width * (4 + 4 + 2 + 2 + 2), 0)
    add("gated_add_normed_norm fp32 branch 8192 rows", lambda: mixops.gated_add_normed_norm(x, y32, wide[:, 2 * width:], w32, 1e-6, bf, 1.0, w32b),
        n * width * (4 + 4 + 4 + 2 + 2), 0)
    add("add_normed_norm (musavik form) 8192 rows", lambda: mixops.add_normed_norm(x, yb, wb16, 1e-6, 1.0, next_weight=wb16b, next_offset=1.0),
        n * width * (4 + 4 + 2 + 2), 0)
    ff = 3 * width
    gu = rn(n, 2 * ff + width)
    add("ff_glu_clamped 8192 rows", lambda: mixops.ff_glu_clamped(gu[:, :2 * ff], 7.0, 1.702), n * ff * 6, 0)
    gu2 = rn(n, 2 * ff)
    add("ff_act silu * up (tipetar form) 8192 rows", lambda: mixops.ff_act(gu2, mixops.FF_SILU_MUL), n * ff * 6, 0)
    logits = torch.randn(n, VOCAB, device=dev)
    add("softcap 8192 x vocab", lambda: mixops.softcap_(logits, 50.0), n * VOCAB * 8, 0)
    z = torch.randn(n, E, device=dev)
    zero = torch.zeros(E, device=dev)
    add("moe_route_grouped, one group (top-k by logit) 8192 rows", lambda: mixops.moe_route_grouped(z, E, top, zero, 1, 1, E), n * (E * 4 + top * 8), 0)
    return rows


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="w1024,w2048")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new-tokens", type=int, default=48)
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--no-models", action="store_true")
    a = ap.parse_args(argv)
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = dict(json.load(open(pk)), source="measured")
    out = {"bench": "gated", "dtype": "bf16", "data": "synthetic token ids, random weights", "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")},
           "workload": {"batch": a.batch, "prompt": a.prompt, "new_tokens": a.new_tokens}, "sizes": {}}
    for size in a.sizes.split(","):
        t0 = time.time()
        entry = {"dims": dict(zip(("width", "heads", "kv_heads", "kv_rank", "window", "experts", "top"), SIZES[size]))}
        for kind in () if a.no_models else ("fegolorn", "tafopel", "tipetar", "qwen3"):
            entry[kind] = hb.throughput(kind, size, a.batch, a.prompt, a.new_tokens)
        if not a.no_kernels:
            entry["kernels"] = kernel_table(size, peaks)
        entry["seconds"] = round(time.time() - t0, 1)
        out["sizes"][size] = entry
        print(json.dumps({size: entry}), file=sys.stderr, flush=True)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
