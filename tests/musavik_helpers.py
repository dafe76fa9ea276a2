"""Small Musavik configurations with random weights for the tests, written out as checkpoint directories."""
from __future__ import annotations

import torch

from tafopel_helpers import tokens, write_checkpoint  # noqa: F401  (shared: token streams, checkpoint writer)


def rglru(width=48, blocks=3, conv=4):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def left(heads=4, kv_heads=2, dim=16, vdim=16, window=24, keep=3, rot_dims=8, base=10000.0, scale=0.25):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window, "keep_first": keep}}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return m


def right(heads=4, kv_heads=2, dim=12, vdim=8, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(l=None, r=None, left_scale=1.3, right_scale=0.8):
    return {"type": "parallel", "mixer": {"left": l or left(), "right": r or right(), "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def config(layers, width=64, vocab=97, eps=2e-5, loop=None, pair=(53, 7, 11), scale=2.5):
    cfg = {"architecture": "Musavik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
           "layers": [dict(l, mlp=mlp) for l, mlp in layers]}
    if pair:
        cfg["embedding"]["bigram"] = {"buckets": pair[0], "mul_prev": pair[1], "mul_cur": pair[2]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def config_a():
    """both mixer kinds, a loop of two layers run three times in the middle, a layer without feed-forward, windows shorter than a
    page and than two, kept first tokens, half-rotated heads, three query heads on one key/value head."""
    return config([(rglru(), dense()),
                   (parallel(), dense(40)),
                   (rglru(width=40, blocks=5, conv=2), None),
                   (parallel(left(heads=3, kv_heads=1, dim=8, vdim=24, window=9, keep=0, rot_dims=8, scale=0.3),
                             right(heads=2, kv_heads=2, dim=8, vdim=20, conv=2), 0.7, 1.1), dense(56))], loop=(1, 3, 3))


def config_b():
    """no pair embedding, the loop opens at the first layer, one head, a fully rotated head, a window of one token with kept first
    tokens, a window longer than any test sequence, one block, one tap, odd sizes."""
    return config([(parallel(left(heads=1, kv_heads=1, dim=12, vdim=20, window=1, keep=2, rot_dims=12, scale=0.3),
                             right(heads=1, kv_heads=1, dim=10, vdim=6, conv=1), 1.0, 1.0), dense(24)),
                   (rglru(width=28, blocks=1, conv=1), dense(36)),
                   (parallel(left(heads=5, kv_heads=5, dim=8, vdim=4, window=100000, keep=4, rot_dims=2, base=50.0, scale=0.35),
                             right(heads=6, kv_heads=2, dim=20, vdim=12, conv=5), 0.5, 1.5), None)],
                  width=44, vocab=61, eps=1e-6, loop=(0, 2, 2), pair=None, scale=1.0)


def config_c():
    """sizes of the tensor-core attention path (heads of 64 and 32, four query heads per key/value head and one), windows around
    the 64-key tile with kept first tokens below and above a tile, unrotated heads, a 64 x 64 delta state, no loop."""
    return config([(parallel(left(heads=8, kv_heads=2, dim=64, vdim=64, window=65, keep=5, rot_dims=32, scale=0.125),
                             right(heads=4, kv_heads=1, dim=64, vdim=64, conv=4)), dense(96)),
                   (rglru(width=160, blocks=2, conv=3), dense(64)),
                   (parallel(left(heads=4, kv_heads=4, dim=32, vdim=32, window=64, keep=70, rot_dims=0, scale=0.18),
                             right(heads=2, kv_heads=2, dim=32, vdim=40, conv=2), 1.0, 0.6), None)], width=128, vocab=211, pair=(211, 3, 5))


def shapes(cfg):
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    if cfg["embedding"].get("bigram"):
        out["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, W)
    if cfg.get("loop"):
        out["loop.in"] = (W, 2 * W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out.update({p + "norm1": (W,), p + "norm1b": (W,)})
        if layer["type"] == "rglru":
            C, nb, K = m["width"], m["blocks"], m["conv"]
            cb = C // nb
            out.update({p + "mix.y": (C, W), p + "mix.y.b": (C,), p + "mix.x": (C, W), p + "mix.x.b": (C,), p + "mix.conv": (C, K),
                        p + "mix.conv.b": (C,), p + "mix.ra": (nb, cb, cb), p + "mix.ra.b": (nb, cb), p + "mix.ri": (nb, cb, cb),
                        p + "mix.ri.b": (nb, cb), p + "mix.lam": (C,), p + "mix.o": (W, C)})
        else:
            l, r = m["left"], m["right"]
            H, G, d, vd = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            q = p + "mix.left."
            out.update({q + "q": (H * d, W), q + "q.b": (H * d,), q + "k": (G * d, W), q + "k.b": (G * d,), q + "v": (G * vd, W),
                        q + "v.b": (G * vd,), q + "q.norm": (d,), q + "k.norm": (d,), q + "talk": (H, H), q + "g": (H * vd, W),
                        q + "o": (W, H * vd)})
            H, G, d, vd, K = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            q = p + "mix.right."
            out.update({q + "q": (G * d, W), q + "q.conv": (G * d, K), q + "k": (G * d, W), q + "k.conv": (G * d, K), q + "v": (H * vd, W),
                        q + "v.conv": (H * vd, K), q + "b": (H, W), q + "a": (H, W), q + "A_log": (H,), q + "dt_bias": (H,),
                        q + "norm": (vd,), q + "g": (H * vd, W), q + "o": (W, H * vd)})
        mlp = layer.get("mlp")
        if mlp is not None:
            out.update({p + "norm2": (W,), p + "norm2b": (W,), p + "mlp.up": (mlp["ff"], W), p + "mlp.up.b": (mlp["ff"],),
                        p + "mlp.down": (W, mlp["ff"]), p + "mlp.down.b": (W,)})
    return out


def random_weights(cfg, seed=0):
    """bf16 tensors (what a checkpoint holds).  Scales keep activations O(1), make the recurrences remember for tens of tokens and
    the head mixing far from the identity."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in shapes(cfg).items():
        leaf = name.split(".")[-1]
        rnd = lambda s=1.0: torch.randn(shape, generator=g) * s
        if leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            w = rnd(0.3)
        elif leaf == "norm":
            w = 1.0 + rnd(0.3)
        elif leaf == "b" and len(shape) == 1:
            w = rnd(0.5)
        elif leaf == "lam":
            w = -2.0 + rnd(1.5)                                 # softplus(lam) in (0.01, 1): decays from 0.9 per token down to e^-8
        elif leaf == "A_log":
            w = torch.log(0.2 + 2.0 * torch.rand(shape, generator=g))
        elif leaf == "dt_bias":
            w = rnd(1.0)
        elif leaf == "talk":
            w = torch.eye(shape[0]) * 0.6 + rnd(0.5)
        elif leaf == "conv":
            w = rnd(0.6)
        elif name in ("embed", "bigram"):
            w = rnd(1.0)
        else:
            w = rnd(1.5 / shape[-1] ** 0.5)
        W[name] = w.to(torch.bfloat16)
    return W
