"""Plain float64 implementation of the Fegolorn decoder: whole sequences, no cache, no batching, one function per mechanism.
It shares no code with the product path and is the yardstick of tests/test_gpu_fegolorn.py.

A model is (cfg, tensors): cfg the parsed config.json, tensors a dict name -> torch tensor (any float type; int tables none).

    embedding   x_t = E[tok_t] * s + B[(tok_{t-1} * a + tok_t * b) mod n]         (row n of B for t = 0)
    layer       x <- x + ls1 * rms1(mixer(h) * sigmoid(R1 h + r1), g1b),  h = rms1(x, g1)       rms1: one number as weight
                x <- x + ls2 * rms1(ff(h') * sigmoid(R2 h' + r2), g2b),   h' = rms1(x, g2)
    output      softcap(head rms1(x, g_final))
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    return rms(x, eps) * g.to(F64).reshape(())


def embed(tokens, E, scale, pair_table=None, pair=None):
    x = E.to(F64)[tokens] * scale
    if pair_table is not None:
        n, a, b = int(pair["buckets"]), int(pair["mul_prev"]), int(pair["mul_cur"])
        rows = [n] + [(int(tokens[t - 1]) * a + int(tokens[t]) * b) % n for t in range(1, len(tokens))]
        x = x + pair_table.to(F64)[torch.tensor(rows)]
    return x


def frequencies(dims: int, base: float, scaling: dict | None = None) -> torch.Tensor:
    """f_i = base^(-2i/dims); with ``scaling`` the long wavelengths are slowed by `factor`, the short ones kept, and the band
    between original/low and original/high blended linearly in original/wavelength."""
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    if scaling:
        fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f.tolist():
            wave = 2.0 * math.pi / fi
            if wave < orig / hi:
                out.append(fi)
            elif wave > orig / lo:
                out.append(fi / fac)
            else:
                s = (orig / wave - lo) / (hi - lo)
                out.append((1.0 - s) * fi / fac + s * fi)
        f = torch.tensor(out, dtype=F64)
    return f


def rotate(x: torch.Tensor, pos: torch.Tensor, freq: torch.Tensor, layout: str, sign: float = 1.0) -> torch.Tensor:
    """x [T, ..., d]: the first 2 * len(freq) elements are turned by sign * pos * freq; pairs (2i, 2i+1) for 'interleaved',
    (i, i + n) for 'halves'."""
    n = freq.numel()
    if n == 0:
        return x
    ang = sign * pos.to(F64)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [n]
    c, s = ang.cos().reshape(shape), ang.sin().reshape(shape)
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2] = u * c - v * s
        out[..., 1:2 * n:2] = v * c + u * s
    else:
        u, v = x[..., :n], x[..., n:2 * n]
        out[..., :n] = u * c - v * s
        out[..., n:2 * n] = v * c + u * s
    return out


def softmax_attend(scores: torch.Tensor, visible: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    """scores [H, T, T], visible bool [T, T], values [H, T, vd] -> [T, H, vd]."""
    p = torch.softmax(scores.masked_fill(~visible[None], float("-inf")), -1)
    return torch.einsum("hij,hjd->ihd", p, values)


def attention(h, w, m, eps, pos=None):
    """Grouped-query attention: per-head RMS norm of q and k (one weight of `dim` numbers for all heads), interleaved rotation of the
    first rot.dims elements, values turned by their own position over the whole vdim and every head's sum turned back by the
    query's position, causal softmax (over the last mask.size positions when the mixer has a mask)."""
    T = h.shape[0]
    H, G, d, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T) if pos is None else pos
    q = (h @ w["q"].to(F64).T).view(T, H, d)
    k = (h @ w["k"].to(F64).T).view(T, G, d)
    v = (h @ w["v"].to(F64).T).view(T, G, vd)
    q = rms(q, eps) * w["q.norm"].to(F64)
    k = rms(k, eps) * w["k.norm"].to(F64)
    rot = m.get("rot")
    if rot and int(rot["dims"]) > 0:
        f = frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        q, k = rotate(q, pos, f, "interleaved"), rotate(k, pos, f, "interleaved")
    base = float(rot["base"]) if rot else 10000.0
    fv = frequencies(vd, base)
    v = rotate(v, pos, fv, "interleaved")
    rep = H // G
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * float(m["scale"])
    dist = pos[:, None] - pos[None, :]
    vis = dist >= 0
    size = int((m.get("mask") or {}).get("size") or 0)
    if size:
        vis = vis & (dist < size)
    o = softmax_attend(s, vis, vv.transpose(0, 1))
    o = rotate(o, pos, fv, "interleaved", sign=-1.0)
    return o.reshape(T, H * vd) @ w["o"].to(F64).T


def latent_attention(h, w, m, eps, pos=None):
    """Latent attention with per-head keys and values written out: k[h] = [W_uk[h] c | k_rot], v[h] = W_uv[h] c."""
    T = h.shape[0]
    H, d, rd, vd, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(T) if pos is None else pos
    q = (h @ w["q"].to(F64).T).view(T, H, d + rd)
    dkv = h @ w["dkv"].to(F64).T
    c = rms(dkv[:, :R], eps) * w["dkv.norm"].to(F64)
    k_rot = dkv[:, R:]
    f = frequencies(int(m["rot"]["dims"]), float(m["rot"]["base"]), m["rot"].get("scaling"))
    q_rot = rotate(q[..., d:], pos, f, "halves")
    k_rot = rotate(k_rot, pos, f, "halves")
    k_nope = (c @ w["uk"].to(F64).T).view(T, H, d)
    v = (c @ w["uv"].to(F64).T).view(T, H, vd)
    s = (torch.einsum("ihd,jhd->hij", q[..., :d], k_nope) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    dist = pos[:, None] - pos[None, :]
    vis = dist >= 0
    size = int((m.get("mask") or {}).get("size") or 0)
    if size:
        vis = vis & (dist < size)
    o = softmax_attend(s, vis, v.transpose(0, 1)).reshape(T, H * vd)
    if "g" in w:
        o = o * torch.sigmoid(h @ w["g"].to(F64).T)
    return o @ w["o"].to(F64).T


def clamped_glu(h, w, limit: float):
    g = (h @ w["gate"].to(F64).T).clamp(max=limit)
    u = (h @ w["up"].to(F64).T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].to(F64).T


def silu_expert(h, gate, up, down):
    z = h @ gate.to(F64).T
    return (z * torch.sigmoid(z) * (h @ up.to(F64).T)) @ down.to(F64).T


def routed_experts(h, w, mlp):
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ w["router"].to(F64).T + w["router.b"].to(F64)
    val, idx = z.topk(top, -1)
    p = torch.softmax(val, -1)
    out = torch.zeros_like(h)
    for e in range(E):
        ye = silu_expert(h, w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])
        out = out + ye * (p * (idx == e)).sum(-1, keepdim=True)
    if mlp.get("shared"):
        out = out + silu_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: dict, tokens, taps: list | None = None) -> torch.Tensor:
    """-> float64 logits [T, vocab]; ``taps`` collects the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    emb = cfg.get("embedding") or {}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = embed(tokens, tensors["embed"], float(emb.get("scale", 1.0)), tensors.get("bigram"), emb.get("bigram"))
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        p = f"l{src}."
        t = sub(tensors, p)
        m = layer["mixer"]
        h = scalar_norm(x, t["norm1"], eps)
        w = sub(t, "mix.")
        y = attention(h, w, m, eps) if layer["type"] == "attention" else latent_attention(h, w, m, eps)
        if "rg1" in t:
            y = y * torch.sigmoid(h @ t["rg1"].to(F64).T + t["rg1.b"].to(F64))
        y = scalar_norm(y, t["norm1b"], eps)
        if "ls1" in t:
            y = y * t["ls1"].to(F64)
        x = x + y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = scalar_norm(x, t["norm2"], eps)
            w = sub(t, "mlp.")
            y = clamped_glu(h, w, float(mlp["limit"])) if mlp["kind"] == "dense" else routed_experts(h, w, mlp)
            if "rg2" in t:
                y = y * torch.sigmoid(h @ t["rg2"].to(F64).T + t["rg2.b"].to(F64))
            y = scalar_norm(y, t["norm2b"], eps)
            if "ls2" in t:
                y = y * t["ls2"].to(F64)
            x = x + y
        if taps is not None:
            taps.append(x.clone())
    z = scalar_norm(x, tensors["final.norm"], eps) @ tensors["head"].to(F64).T
    cap = cfg.get("logit_softcap")
    if cap:
        z = float(cap) * torch.tanh(z / float(cap))
    return z
