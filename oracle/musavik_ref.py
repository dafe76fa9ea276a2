"""Plain implementation of the Musavik decoder: float64, whole sequences, no cache, no batching, one function per mechanism.
Test infrastructure only: it shares no code with the product path and is written from the design's equations.

Weights: a dict name -> tensor (any float dtype; cast to float64 here).  Linear weights are [out, in] and applied as W x.

    embedding:    x = E[t] * s + B[(t_prev * a + t * b) mod n]      (row n of B for a sequence's first token)
    layer order:  layers [start, stop) run `times` times in a row with the same weights; every pass opens with
                  x <- W_in [x ; x0], x0 the embedding output
    layer:        x <- x + zc_norm(mixer(zc_norm(x)));  x <- x + zc_norm(ff(zc_norm(x)))        (four weights per layer)
    zc_norm:      y / sqrt(mean(y^2) + eps) * (1 + g)
    mixers:       'rglru'    two branches, a gated diagonal linear recurrence on one of them
                  'parallel' windowed attention with kept first tokens and head mixing  +  a gated delta-rule recurrence
    ff:           W_down gelu_tanh(W_up h + b) + b
    output:       logits = head zc_norm(x)
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

F64 = torch.float64


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def zc_norm(y: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is stored around zero."""
    return unit_rms(y, eps) * (1.0 + g.to(F64))


def embedding(W: dict, cfg: dict, tokens: list[int]) -> torch.Tensor:
    e = cfg["embedding"]
    x = W["embed"].to(F64)[tokens] * float(e["scale"])
    bg = e.get("bigram")
    if bg:
        n = int(bg["buckets"])
        rows = [n] + [(tokens[i - 1] * int(bg["mul_prev"]) + tokens[i] * int(bg["mul_cur"])) % n for i in range(1, len(tokens))]
        x = x + W["bigram"].to(F64)[rows]
    return x


def causal_conv(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """x [n, C], w [C, taps]: y[t, c] = sum_j w[c, taps - 1 - j] x[t - j, c], zeros before the start."""
    n, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        if j < n:
            y[j:] += x[:n - j] * w[:, taps - 1 - j]
    return y if bias is None else y + bias


def rglru(W: dict, p: str, m: dict, h: torch.Tensor) -> torch.Tensor:
    """Gated diagonal recurrence: S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t,  a_t = exp(-8 r_t softplus(lam)),
    r, i = sigmoid(block-diagonal maps of u); out = W_o (S * gelu_tanh(W_y h + b))."""
    w = lambda leaf: W[p + leaf].to(F64)
    C, nb = int(m["width"]), int(m["blocks"])
    y = gelu_tanh(h @ w("y").T + w("y.b"))
    u = causal_conv(h @ w("x").T + w("x.b"), w("conv"), w("conv.b"))
    n = h.shape[0]
    ub = u.view(n, nb, C // nb)
    r = torch.sigmoid(torch.einsum("nbi,boi->nbo", ub, w("ra")) + w("ra.b")).reshape(n, C)
    i = torch.sigmoid(torch.einsum("nbi,boi->nbo", ub, w("ri")) + w("ri.b")).reshape(n, C)
    log_a = -8.0 * r * F.softplus(w("lam"))
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(C, dtype=F64)
    out = torch.empty_like(u)
    for t in range(n):
        S = a[t] * S + drive[t]
        out[t] = S
    return (out * y) @ w("o").T


def rotate_pairs(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [n, heads, d]: the pairs (2i, 2i + 1), i < dims / 2, of the token at position p turn by p * base^(-2i / dims)."""
    n = x.shape[0]
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    ang = torch.arange(n, dtype=F64)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def visible(n: int, window: int, keep_first: int) -> torch.Tensor:
    """[n, n] bool: query i sees key j when j <= i and (i - j < window or j < keep_first)."""
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    return (j <= i) & ((i - j < window) | (j < keep_first))


def mixed_head_attention(W: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Grouped-query attention: per-head query/key norm, partial pair rotation, unit-RMS values, sliding window with kept first
    tokens, softmax, then the heads' weight matrices are mixed by T before they meet the values; sigmoid output gate."""
    w = lambda leaf: W[p + leaf].to(F64)
    H, G, d, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    n = h.shape[0]
    q = (h @ w("q").T + w("q.b")).view(n, H, d)
    k = (h @ w("k").T + w("k.b")).view(n, G, d)
    v = (h @ w("v").T + w("v.b")).view(n, G, vd)
    q = unit_rms(q, eps) * w("q.norm")
    k = unit_rms(k, eps) * w("k.norm")
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, int(rot["dims"]), float(rot["base"]))
        k = rotate_pairs(k, int(rot["dims"]), float(rot["base"]))
    v = unit_rms(v, eps)
    mask = m.get("mask") or {}
    see = visible(n, int(mask.get("size") or n + 1), int(mask.get("keep_first") or 0))
    P = []
    for hh in range(H):
        s = (q[:, hh] @ k[:, hh // (H // G)].T) * float(m["scale"])
        P.append(torch.softmax(torch.where(see, s, torch.full_like(s, -math.inf)), -1))
    P = torch.stack(P)                                           # [H, n, n]
    T = w("talk")
    mixed = torch.einsum("hg,gij->hij", T, P)
    o = torch.cat([mixed[hh] @ v[:, hh // (H // G)] for hh in range(H)], -1)
    o = o * torch.sigmoid(h @ w("g").T)
    return o @ w("o").T


def gated_delta(W: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Per head a matrix state S [dim, vdim]:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    w = lambda leaf: W[p + leaf].to(F64)
    H, G, d, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    n = h.shape[0]
    silu = lambda z: z * torch.sigmoid(z)
    q = silu(causal_conv(h @ w("q").T, w("q.conv"))).view(n, G, d)
    k = silu(causal_conv(h @ w("k").T, w("k.conv"))).view(n, G, d)
    v = silu(causal_conv(h @ w("v").T, w("v.conv"))).view(n, H, vd)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w("b").T)                                               # [n, H]
    decay = torch.exp(-torch.exp(w("A_log")) * F.softplus(h @ w("a").T + w("dt_bias")))   # [n, H]
    out = torch.empty(n, H, vd, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(d, vd, dtype=F64)
        for t in range(n):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hh] = S.T @ q[t, g]
    out = unit_rms(out, eps) * w("norm")
    out = out.reshape(n, H * vd) * silu(h @ w("g").T)
    return out @ w("o").T


def parallel_mixer(W: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    return float(m["left_scale"]) * mixed_head_attention(W, p + "left.", m["left"], h, eps) + \
        float(m["right_scale"]) * gated_delta(W, p + "right.", m["right"], h, eps)


def dense_ff(W: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    w = lambda leaf: W[p + leaf].to(F64)
    return gelu_tanh(h @ w("up").T + w("up.b")) @ w("down").T + w("down.b")


def layer_runs(cfg: dict) -> list[tuple[int, bool]]:
    """(layer index, whether a pass of the loop opens right before it) in execution order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(cfg: dict, W: dict, tokens: list[int], taps: list | None = None) -> torch.Tensor:
    """-> logits [n, vocab] (float64).  ``taps`` collects the residual stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x0 = embedding(W, cfg, tokens)
    x = x0
    for i, opens in layer_runs(cfg):
        if opens:
            x = torch.cat([x, x0], -1) @ W["loop.in"].to(F64).T
        layer, p = cfg["layers"][i], f"l{i}."
        h = zc_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "rglru":
            y = rglru(W, p + "mix.", layer["mixer"], h)
        elif layer["type"] == "parallel":
            y = parallel_mixer(W, p + "mix.", layer["mixer"], h, eps)
        else:
            raise ValueError(layer["type"])
        x = x + zc_norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = dense_ff(W, p + "mlp.", zc_norm(x, W[p + "norm2"], eps))
            x = x + zc_norm(y, W[p + "norm2b"], eps)
        if taps is not None:
            taps.append(x.clone())
    return zc_norm(x, W["final.norm"], eps) @ W["head"].to(F64).T
