"""Prefill / decode throughput of the Musavik decoder (gated diagonal recurrence; windowed attention with kept first tokens and
mixed heads beside a gated delta rule; repeated layers) beside Tafopel, Tipetar and Qwen3 at equal width, number of layer runs and
feed-forward size, plus a per-kernel roofline table of its kernels and their counterparts (``python bench.py --recurrent``).

Same rules as hybrid_bench.py, whose engine set-up, throughput loop and timing helper it uses: random weights, synthetic token
ids, device time between CUDA events after warm-up, a 256 MB write between the timed launches of the per-kernel table.
"""
from __future__ import annotations

import json
import os
import sys
import time

import hybrid_bench as hb
import window_bench as wb

ROOT = hb.ROOT
VOCAB = hb.VOCAB

SIZES = {
    # name: (width, heads, kv_heads, window, keep_first, delta heads, delta q/k heads, gate blocks)  -- head size 128; six layers of which
    # layers 2..3 run twice: eight layer runs, as many as the eight layers of the models beside it
    "w1024": (1024, 16, 4, 1024, 4, 8, 4, 8),
    "w2048": (2048, 16, 4, 2048, 4, 16, 4, 16),
}


def musavik_config(size: str):
    from nanovllm.models.musavik import MusavikConfig
    width, H, G, window, keep, dh, dg, blocks = SIZES[size]
    rec = {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": 4}}
    par = {"type": "parallel", "mixer": {
        "left": {"heads": H, "kv_heads": G, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": window, "keep_first": keep},
                 "rot": {"dims": 64, "base": 5e5}},
        "right": {"heads": dh, "kv_heads": dg, "dim": 128, "vdim": 128, "conv": 4}, "left_scale": 1.0, "right_scale": 1.0}}
    mlp = {"kind": "dense", "ff": 3 * width}
    layers = [dict(l, mlp=mlp) for l in (rec, par, rec, par, rec, par)]
    return MusavikConfig({"architecture": "Musavik", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6},
                          "embedding": {"scale": width ** 0.5, "bigram": {"buckets": 65521, "mul_prev": 40503, "mul_cur": 9973}},
                          "layers": layers, "loop": {"start": 2, "stop": 4, "times": 2}})


hb.EXTRA_KINDS["musavik"] = musavik_config


def kernel_table(size: str, peaks: dict):
    import torch
    from nanovllm import mixops
    width, H, G, window, keep, dh, dg, blocks = SIZES[size]
    d, bs, dev, bf = 128, 256, "cuda", torch.bfloat16
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

    # ---- attention: every head's weights on every value head (what the head mixing needs), and the plain windowed form beside it ----
    for label, S, q, k in (("prefill 4x2048", 4, 2048, 2048), ("decode 64x4096", 64, 1, 4096)):
        nblk = S * (k // bs)
        cache = rn(nblk * bs, G * 2 * d)
        bt = torch.arange(nblk, dtype=torch.int32, device=dev).view(S, -1)
        n = S * q
        qkv = rn(n, H * d)
        spn = spans(S, q, k)
        vis = lambda i: min(i + 1, window) + max(0, min(keep, i + 1 - window))
        pairs = S * (sum(vis(i) for i in range(q)) if q > 1 else vis(k - 1))
        keys_read = S * (k if q > 1 else vis(k - 1))
        for mixed in (True, False):
            vsets = G if mixed else 1
            flops = pairs * H * 2 * d * (1 + vsets)
            nbytes = keys_read * G * 2 * d * 2 + n * H * d * 2 + n * H * vsets * d * (4 if mixed else 2)
            name = "window_attention all values + kept first" if mixed else "window_attention own values (tipetar form)"
            add(f"{name} {label}", lambda: mixops.window_attention(qkv, cache, bt, bs, spn, H, G, d, d, 0.088, None, window, keep_first=keep if mixed else 0,
                                                                  all_values=mixed, out_f32=mixed), nbytes, flops, "tensor")
    n = 8192
    acc = torch.randn(n, H, G, d, device=dev)
    T = torch.randn(H, H, device=dev)
    gate = rn(n, H * d)
    add("head_mix_gate 8192 rows", lambda: mixops.head_mix_gate(acc, T, gate, bf), n * H * d * (G * 4 + 2 + 2), n * H * H * d * 2, "fma")
    # ---- per-head norms, rotation and cache store; Tipetar's whole-projection norm + store beside it ----
    from nanovllm.layers.rotary_embedding import build_interleaved_cos_sin
    table = build_interleaved_cos_sin(64, 8192, 5e5, None, dev)
    qkv = rn(n, (H + 2 * G) * d)
    cache = torch.zeros(n, G * 2 * d, dtype=bf, device=dev)
    sl = torch.arange(n, dtype=torch.int32, device=dev)
    pos = torch.arange(n, dtype=torch.int64, device=dev)
    wq, wk = rn(d), rn(d)
    add("headnorm_rope_store 8192 rows", lambda: mixops.headnorm_rope_store(qkv, 0, H * d, (H + G) * d, H, G, d, d, wq, wk, True, table, pos, sl, cache, 1e-6),
        n * ((2 * H + 4 * G) * d) * 2, 0)
    wq2, wk2 = rn(H * d), rn(G * d)
    add("tipetar qk_norm_store 8192 rows", lambda: mixops.qk_norm_store(qkv, H * d, G * d, G * d, wq2, wk2, sl, cache, 1e-6), n * ((2 * H + 4 * G) * d) * 2, 0)
    # ---- recurrences: a prompt step of 4 x 2048 tokens and a decode step of 64 rows; Tafopel's selective scan beside them ----
    C, cb = width, width // blocks
    for label, S, q in (("prefill 4x2048", 4, 2048), ("decode 64", 64, 1)):
        n = S * q
        spn = spans(S, q, q if q > 1 else 100)
        slots = torch.arange(S, dtype=torch.int32, device=dev)
        u, y = rn(n, C), rn(n, C)
        gates = torch.randn(blocks, n, 2 * cb, device=dev)
        gb, rate = torch.zeros(blocks, 2 * cb, device=dev), -torch.rand(C, device=dev)
        st = torch.zeros(S, C, device=dev)
        add(f"diag_scan {label}", lambda: mixops.diag_scan(u, gates, gb, rate, y, st, slots, spn), n * C * (2 + 8 + 2 + 2), n * C * 40, "fma")
        x = rn(n, 2 * dg * d + dh * d)
        ba = torch.randn(n, 2 * dh, device=dev)
        rt, db = -torch.rand(dh, device=dev), torch.zeros(dh, device=dev)
        sd = torch.zeros(S, dh, d, d, device=dev)
        add(f"gated_delta {label}", lambda: mixops.gated_delta(x, 0, dg * d, 2 * dg * d, ba, rt, db, sd, slots, spn, dh, dg, d, d, d ** -0.5),
            n * ((2 * dg + dh) * d * 2 + dh * d * 4) + 2 * S * dh * d * d * 4, n * dh * d * d * 6, "fma")
        o = torch.randn(n, dh, d, device=dev)
        gz = rn(n, dh * d)
        add(f"head_rmsnorm_gate {label}", lambda: mixops.head_rmsnorm_gate(o, wq, gz, 1e-6, bf), n * dh * d * (4 + 2 + 2), 0)
        xc, wc, cs = rn(n, C), rn(C, 4), torch.zeros(S, 3, C, device=dev)
        add(f"causal_conv {label}", lambda: mixops.causal_conv(xc, wc, None, cs, slots, spn, silu=False), n * C * 4, 0)
        # Tafopel's selective scan at the same channel count, 16 states per channel
        N = 16
        dt, Bm, Cm, z = rn(n, C), rn(n, N), rn(n, N), rn(n, C)
        A, Dv, dtb = -torch.rand(C, N, device=dev), rn(C), rn(C)
        ss = torch.zeros(S, C, N, device=dev)
        add(f"tafopel selective_scan {label}", lambda: mixops.selective_scan(u, dt, dtb, A, Bm, Cm, Dv, z, ss, slots, spn), n * (C * 8 + N * 4) + 2 * S * C * N * 4,
            n * C * N * 8, "fma")
    # ---- row-wise ops, 8192 rows ----
    n = 8192
    x, yb, w, w2 = torch.randn(n, width, device=dev), rn(n, width), rn(width), rn(width)
    add("add_normed_norm 8192 rows", lambda: mixops.add_normed_norm(x, yb, w, 1e-6, 1.0, next_weight=w2, next_offset=1.0), n * width * (4 + 4 + 2 + 2), 0)
    copy = torch.empty(n, width, dtype=bf, device=dev)
    add("tipetar add_normed 8192 rows", lambda: mixops.add_normed(x, yb, w, 0.5, 1e-6, 1.0, copy), n * width * (4 + 4 + 2 + 2), 0)
    ids = torch.randint(0, VOCAB, (n,), device=dev)
    tab, pair = rn(VOCAB, width), rn(65522, width)
    prev, sl4 = torch.zeros(4, dtype=torch.int64, device=dev), torch.arange(4, dtype=torch.int32, device=dev)
    add("embed_pair 8192 rows", lambda: mixops.embed_pair(ids, tab, 3.0, spans(4, 2048, 2048), pair, 65521, 40503, 9973, prev, sl4), n * width * (2 + 2 + 4), 0)
    add("tafopel embed 8192 rows", lambda: mixops.embed(ids, tab), n * width * (2 + 4), 0)
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
    out = {"bench": "recurrent", "dtype": "bf16", "data": "synthetic token ids, random weights", "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")},
           "workload": {"batch": a.batch, "prompt": a.prompt, "new_tokens": a.new_tokens}, "sizes": {}}
    for size in a.sizes.split(","):
        t0 = time.time()
        entry = {"dims": dict(zip(("width", "heads", "kv_heads", "window", "keep_first", "delta_heads", "delta_qk_heads", "gate_blocks"), SIZES[size]))}
        for kind in () if a.no_models else ("musavik", "tafopel", "tipetar", "qwen3"):
            entry[kind] = hb.throughput(kind, size, a.batch, a.prompt, a.new_tokens)
        if not a.no_kernels:
            entry["kernels"] = kernel_table(size, peaks)
        entry["seconds"] = round(time.time() - t0, 1)
        out["sizes"][size] = entry
        print(json.dumps({size: entry}), file=sys.stderr, flush=True)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
