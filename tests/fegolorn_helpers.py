"""Small Fegolorn configurations with random weights for the tests, written out as checkpoint directories."""
from __future__ import annotations

import copy

import torch

from tafopel_helpers import tokens, write_checkpoint  # noqa: F401  (shared: token streams, checkpoint writer)


def attention(heads=4, kv_heads=2, dim=16, vdim=8, rot_dims=8, base=5000.0, scale=0.3, scaling=None, window=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot_dims, "base": base}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if window:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=16, rot_dim=8, vdim=12, kv_rank=24, window=9, base=300.0, scale=0.25, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": {"dims": rot_dim, "base": base}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def dense(ff=40, limit=0.8):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=6, top=2, ff=24, shared=16):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(layers, width=64, vocab=97, eps=2e-5, pair=(53, 7, 11), scale=2.5, softcap=12.0):
    """layers: (mixer entry, mlp) pairs, or an int j for a layer that runs with layer j's weights."""
    out = []
    for entry in layers:
        if isinstance(entry, int):
            out.append(dict(copy.deepcopy(out[entry]), weights_of=entry))
        else:
            out.append(dict(copy.deepcopy(entry[0]), mlp=copy.deepcopy(entry[1])))
    cfg = {"architecture": "Fegolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale}, "layers": out}
    if pair:
        cfg["embedding"]["bigram"] = {"buckets": pair[0], "mul_prev": pair[1], "mul_cur": pair[2]}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


def config_a():
    """both mixers and both feed-forwards, two layers that borrow weights (one of them twice removed in depth), a layer without
    feed-forward, a window shorter than a page, banded frequencies that fall in all three bands, three query heads on one latent."""
    return config([(latent(), dense()),
                   (attention(scaling=(4.0, 1.0, 4.0, 64)), moe()),
                   1,
                   (latent(heads=2, dim=8, rot_dim=4, vdim=20, kv_rank=16, window=33, scaling=(2.0, 1.0, 2.0, 16)), None),
                   0,
                   1])


def config_b():
    """no pair table, no soft cap, one head, a window of one token and one longer than any test sequence, fully rotated heads,
    every expert chosen, a single expert, no shared expert, one key/value head per query head, odd sizes."""
    return config([(latent(heads=1, dim=12, rot_dim=6, vdim=10, kv_rank=20, window=1), moe(experts=3, top=3, ff=20, shared=0)),
                   (attention(heads=5, kv_heads=5, dim=8, vdim=4, rot_dims=8, base=50.0, scale=0.35), dense(36, 1.0)),
                   (latent(heads=5, dim=4, rot_dim=2, vdim=6, kv_rank=10, window=100000), moe(experts=1, top=1, ff=12, shared=28)),
                   (attention(heads=1, kv_heads=1, dim=12, vdim=20, rot_dims=2, scale=0.3), None)],
                  width=44, vocab=61, eps=1e-6, pair=None, scale=1.0, softcap=None)


def config_c():
    """sizes of the tensor-core attention paths (latent rows of 96 and 160 elements, heads of 64 and 32), windows around the 64-key
    tile, four query heads per key/value head and sixteen heads on one latent, more experts."""
    return config([(latent(heads=8, dim=32, rot_dim=32, vdim=32, kv_rank=64, window=65, base=10000.0, scale=0.12), dense(96, 1.5)),
                   (attention(heads=8, kv_heads=2, dim=64, vdim=64, rot_dims=32, base=100000.0, scale=0.125, scaling=(8.0, 1.0, 4.0, 256)), moe(8, 3, 64, 48)),
                   (latent(heads=16, dim=16, rot_dim=32, vdim=16, kv_rank=128, window=64, scale=0.15), None),
                   1,
                   (attention(heads=4, kv_heads=4, dim=32, vdim=32, rot_dims=32, scale=0.18), dense(64, 0.5))], width=128, vocab=211, pair=(211, 3, 5))


def mixer_shapes(layer, W):
    m = layer["mixer"]
    if layer["type"] == "attention":
        H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        return {"q": (H * d, W), "k": (G * d, W), "v": (G * vd, W), "q.norm": (d,), "k.norm": (d,), "o": (W, H * vd)}
    H, d, rd, vd, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    return {"q": (H * (d + rd), W), "dkv": (R + rd, W), "dkv.norm": (R,), "uk": (H * d, R), "uv": (H * vd, R), "g": (H * vd, W), "o": (W, H * vd)}


def mlp_shapes(mlp, W):
    if mlp["kind"] == "dense":
        return {"gate": (mlp["ff"], W), "up": (mlp["ff"], W), "down": (W, mlp["ff"])}
    out, f = {"router": (mlp["router"]["experts"], W), "router.b": (mlp["router"]["experts"],)}, mlp["expert"]["ff"]
    for k in range(mlp["router"]["experts"]):
        out.update({f"e{k}.gate": (f, W), f"e{k}.up": (f, W), f"e{k}.down": (W, f)})
    if mlp.get("shared"):
        s = mlp["shared"]["ff"]
        out.update({"shared.gate": (s, W), "shared.up": (s, W), "shared.down": (W, s)})
    return out


def shapes(cfg):
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": ()}
    if cfg["embedding"].get("bigram"):
        out["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, W)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p = f"l{i}."
        out.update({p + "norm1": (), p + "norm1b": (), p + "ls1": (W,), p + "rg1": (W, W), p + "rg1.b": (W,)})
        out.update({p + "mix." + k: v for k, v in mixer_shapes(layer, W).items()})
        if layer.get("mlp") is not None:
            out.update({p + "norm2": (), p + "norm2b": (), p + "ls2": (W,), p + "rg2": (W, W), p + "rg2.b": (W,)})
            out.update({p + "mlp." + k: v for k, v in mlp_shapes(layer["mlp"], W).items()})
    return out


def random_tensor(name, shape, g):
    leaf = name.split(".")[-1]
    rnd = lambda s=1.0: torch.randn(shape, generator=g) * s
    if shape == ():
        return 0.7 + 0.6 * torch.rand((), generator=g)                      # the norms' single numbers, away from 1
    if leaf in ("ls1", "ls2"):
        return 0.6 + rnd(0.3)
    if leaf == "norm":
        return 1.0 + rnd(0.3)
    if leaf == "b":
        return rnd(0.7)
    if name in ("embed", "bigram"):
        return rnd(1.0)
    if leaf == "router":
        return rnd(3.0 / shape[-1] ** 0.5)                                  # clear choices: no test rests on a close call
    return rnd(1.5 / shape[-1] ** 0.5)


def random_weights(cfg, seed=0):
    """bf16 tensors (what a checkpoint holds).  Scales keep activations O(1) and let the clamps, gates and routing matter."""
    g = torch.Generator().manual_seed(seed)
    return {name: random_tensor(name, shape, g).to(torch.bfloat16) for name, shape in shapes(cfg).items()}
