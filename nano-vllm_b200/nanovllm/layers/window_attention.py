"""Grouped-query attention with a sliding window and a linear distance bias, without any rotation.

    q = norm_all(W_q h) * g_q        k = norm_all(W_k h) * g_k        v = W_v h
        (norm_all: ONE root mean square over the whole projection of a token, all heads together, then a weight per column)
    s[h, i, j] = (q_i[h] . k_j[h // (H / G)]) * scale - slope[h] * (i - j),   slope[h] = 2^(-8 (h + 1) / H)
    visible j:  0 <= i - j < window        p = softmax over the visible j        out = W_o concat_h (sum_j p_j v_j)

Positions enter only through the bias and the window, so the cached keys are position-free: per token the cache holds one
row ``[k (G * dim) | v (G * vdim)]`` (keys after their norm) for every layer that owns a key/value projection.  A layer with
``kv_from`` has no key/value tensors: it reads the named layer's cache rows with its own queries, window, scale and bias.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops


def distance_slopes(heads: int, device) -> torch.Tensor:
    """slope[h] = 2^(-8 (h + 1) / heads), fp32."""
    h = torch.arange(1, heads + 1, dtype=torch.float64)
    return torch.exp2(-8.0 * h / heads).to(torch.float32).to(device)


class BiasedWindowAttention:
    kind = "attention"

    def __init__(self, width: int, m: dict, eps: float, dtype, device):
        self.width, self.eps, self.dtype, self.device = width, eps, dtype, device
        self.heads, self.kv_heads = int(m["heads"]), int(m["kv_heads"])
        self.dim, self.vdim = int(m["dim"]), int(m["vdim"])
        self.scale = float(m["scale"])
        mask = m.get("mask") or {}
        self.window = int(mask.get("size") or 0)                  # 0: every earlier token is visible
        self.kv_from = m.get("kv_from")
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if self.vdim > 512:
            raise ValueError(f"vdim {self.vdim}: the attention kernels hold at most 512 output columns per query row")
        self.q_cols = self.heads * self.dim
        self.k_cols = 0 if self.kv_from is not None else self.kv_heads * self.dim
        self.v_cols = 0 if self.kv_from is not None else self.kv_heads * self.vdim
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.w_qkv = e(self.q_cols + self.k_cols + self.v_cols, width)       # [W_q ; W_k ; W_v]: one GEMM reads h once
        self.q_norm = e(self.q_cols)
        self.k_norm = e(self.k_cols) if self.kv_from is None else None
        self.w_o = e(width, self.heads * self.vdim)
        self.slopes = distance_slopes(self.heads, device)
        self.cache = None                                 # [num_blocks * block_size, G * (dim + vdim)]; the source layer's when kv_from
        self.block_size = 0

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        own = self.kv_from is None
        if leaf == "q":
            self.w_qkv[:self.q_cols].copy_(w)
        elif leaf == "k" and own:
            self.w_qkv[self.q_cols:self.q_cols + self.k_cols].copy_(w)
        elif leaf == "v" and own:
            self.w_qkv[self.q_cols + self.k_cols:].copy_(w)
        elif leaf == "q.norm":
            self.q_norm.copy_(w)
        elif leaf == "k.norm" and own:
            self.k_norm.copy_(w)
        elif leaf == "o":
            self.w_o.copy_(w)
        else:
            return False
        return True

    def weight_shapes(self, width: int) -> dict:
        out = {"q": (self.q_cols, width), "q.norm": (self.q_cols,), "o": (width, self.heads * self.vdim)}
        if self.kv_from is None:
            out.update({"k": (self.k_cols, width), "v": (self.v_cols, width), "k.norm": (self.k_cols,)})
        return out

    def cache_row_elems(self) -> int:
        """Cached elements per token (0 for a layer that borrows another layer's cache)."""
        return self.k_cols + self.v_cols

    def forward(self, h: torch.Tensor, ctx, spans: mixops.StepSpans) -> torch.Tensor:
        qkv = F.linear(h, self.w_qkv)
        mixops.qk_norm_store(qkv, self.q_cols, self.k_cols, self.v_cols, self.q_norm, self.k_norm, ctx.slot_mapping,
                             self.cache if self.kv_from is None else None, self.eps)
        o = mixops.window_attention(qkv, self.cache, ctx.block_tables, self.block_size, spans, self.heads, self.kv_heads, self.dim,
                                    self.vdim, self.scale, self.slopes, self.window)
        return F.linear(o, self.w_o)


class MixedHeadWindowAttention:
    """Grouped-query attention with per-head query/key norms, a partial pair rotation, unit-RMS values, a sliding window that
    keeps a sequence's first tokens, head mixing after the softmax and a sigmoid output gate.

        q = W_q h + b_q,  k = W_k h + b_k,  v = W_v h + b_v
        q[h] <- rotate(rms(q[h]) * g_q),  k[g] <- rotate(rms(k[g]) * g_k)     (g_q, g_k: `dim` weights shared by the heads; rotation of the
                                                                                first rot.dims elements, pair (2i, 2i+1) by p * base^(-2i / dims))
        v[g] <- v[g] / rms(v[g])                                                (no weight; cached so)
        s[h, i, j] = (q_i[h] . k_j[h // (H / G)]) * scale,   visible j:  j <= i and (i - j < window or j < keep_first)
        p[h] = softmax over the visible j;   p'[h] = sum_g T[h, g] p[g];   o[h] = sum_j p'[h]_ij v_j[h // (H / G)]
        out = W_o (concat_h o[h] * sigmoid(W_g h))

    Keys are cached after norm and rotation, values after their norm: one row ``[k (G * dim) | v (G * vdim)]`` per token, pass and
    layer.  The head mixing is linear in the weight matrices, so it commutes with the product by the values: the attention
    kernel applies every head's weights to the values of every value head (one online-softmax pass, fp32 results), and a
    row-wise kernel forms ``sum_g T[h, g] (p[g] V[h // (H / G)])`` and the gate.

    The input projection ``[W_q ; W_k ; W_v ; W_g]``, its bias and the output projection may be views into the merged weights
    of a block that runs this mixer beside another one on the same input (``ParallelMixer``).
    """
    kind = "mixed_head_attention"

    def __init__(self, width: int, m: dict, eps: float, dtype, device, max_position: int, w_in=None, b_in=None, w_o=None):
        from .rotary_embedding import build_interleaved_cos_sin
        self.width, self.eps, self.dtype, self.device = width, eps, dtype, device
        self.heads, self.kv_heads = int(m["heads"]), int(m["kv_heads"])
        self.dim, self.vdim = int(m["dim"]), int(m["vdim"])
        self.scale = float(m["scale"])
        mask = m.get("mask") or {}
        self.window = int(mask.get("size") or 0)                  # 0: every earlier token is visible
        self.keep_first = int(mask.get("keep_first") or 0) if self.window else 0
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if self.vdim > 512:
            raise ValueError(f"vdim {self.vdim}: the attention kernels hold at most 512 output columns per query row")
        H, G, d, vd = self.heads, self.kv_heads, self.dim, self.vdim
        self.q_cols, self.k_cols, self.v_cols = H * d, G * d, G * vd
        self.in_cols, self.out_cols = self.q_cols + self.k_cols + self.v_cols + H * vd, H * vd
        rot = m.get("rot")
        self.cos_sin, self.rot_key = None, None
        if rot and int(rot["dims"]) > 0:
            dims = int(rot["dims"])
            if dims > d or dims % 2:
                raise ValueError("rot.dims must be even and at most dim")
            self.rot_key = (dims, float(rot["base"]), max_position)
            self.cos_sin = build_interleaved_cos_sin(dims, max_position, float(rot["base"]), None, device)
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.w_in = w_in if w_in is not None else e(self.in_cols, width)          # [W_q ; W_k ; W_v ; W_g]: one GEMM reads h once
        self.b_in = b_in if b_in is not None else torch.zeros(self.in_cols, dtype=dtype, device=device)
        self.w_o = w_o if w_o is not None else e(width, self.out_cols)
        assert self.w_in.shape == (self.in_cols, width) and self.b_in.shape == (self.in_cols,) and self.w_o.shape == (width, self.out_cols)
        self.q_norm, self.k_norm = e(d), e(d)
        self.talk = torch.zeros(H, H, dtype=torch.float32, device=device)
        self.cache: list = []                             # per pass [num_blocks * block_size, G * (dim + vdim)]
        self.block_size = 0

    @staticmethod
    def projection_cols(m: dict) -> tuple[int, int]:
        """(rows of the wide input projection, columns of the output projection) for a mixer configuration."""
        H, G, d, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        return H * d + G * d + G * vd + H * vd, H * vd

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        q, k, v = self.q_cols, self.k_cols, self.v_cols
        spans = {"q": (0, q), "k": (q, q + k), "v": (q + k, q + k + v), "g": (q + k + v, self.in_cols)}
        if leaf in spans:
            self.w_in[spans[leaf][0]:spans[leaf][1]].copy_(w)
        elif leaf in ("q.b", "k.b", "v.b"):
            a, b = spans[leaf[0]]
            self.b_in[a:b].copy_(w)
        elif leaf == "q.norm":
            self.q_norm.copy_(w)
        elif leaf == "k.norm":
            self.k_norm.copy_(w)
        elif leaf == "talk":
            self.talk.copy_(w.float())
        elif leaf == "o":
            self.w_o.copy_(w)
        else:
            return False
        return True

    def weight_shapes(self, width: int) -> dict:
        H = self.heads
        return {"q": (self.q_cols, width), "q.b": (self.q_cols,), "k": (self.k_cols, width), "k.b": (self.k_cols,), "v": (self.v_cols, width),
                "v.b": (self.v_cols,), "q.norm": (self.dim,), "k.norm": (self.dim,), "talk": (H, H), "g": (H * self.vdim, width),
                "o": (width, H * self.vdim)}

    def cache_row_elems(self) -> int:
        return self.k_cols + self.v_cols

    def state_slot_bytes(self) -> int:
        return 0

    def bind(self, num_blocks: int, block_size: int, num_slots: int, copies: int = 1) -> None:
        self.block_size = block_size
        self.cache = [torch.zeros(num_blocks * block_size, self.cache_row_elems(), dtype=self.dtype, device=self.device) for _ in range(copies)]

    def unbind(self) -> None:
        self.cache = []

    def mix(self, proj: torch.Tensor, h: torch.Tensor, positions, ctx, spans: mixops.StepSpans, inst: int, out: torch.Tensor | None = None,
            out_scale: float = 1.0) -> torch.Tensor:
        """proj [n, in_cols] = h W_in^T + b_in (a row-strided view) -> the output projection's operand [n, heads * vdim]."""
        q, k, v = self.q_cols, self.k_cols, self.v_cols
        cache = self.cache[inst]
        mixops.headnorm_rope_store(proj, 0, q, q + k, self.heads, self.kv_heads, self.dim, self.vdim, self.q_norm, self.k_norm, True,
                                   self.cos_sin, positions, ctx.slot_mapping, cache, self.eps)
        acc = mixops.window_attention(proj, cache, ctx.block_tables, self.block_size, spans, self.heads, self.kv_heads, self.dim, self.vdim,
                                      self.scale, None, self.window, keep_first=self.keep_first, all_values=True,
                                      out_f32=self.dtype != torch.float32)
        return mixops.head_mix_gate(acc, self.talk, proj[:, q + k + v:], self.dtype, out=out, out_scale=out_scale)

    def forward(self, h: torch.Tensor, positions, ctx, spans: mixops.StepSpans, inst: int = 0) -> torch.Tensor:
        return F.linear(self.mix(F.linear(h, self.w_in, self.b_in), h, positions, ctx, spans, inst), self.w_o)


class RotatedValueAttention:
    """Grouped-query attention with per-head query/key norms, a banded partial pair rotation, and values that carry their own
    position:

        q = W_q h,  k = W_k h,  v = W_v h
        q[h] <- rotate(rms(q[h]) * g_q, p),  k[g] <- rotate(rms(k[g]) * g_k, p)      (g_q, g_k: `dim` weights shared by the heads; the first
                                                                                      rot.dims elements turn, pair (2i, 2i+1) by p * f_i, f_i banded)
        v[g] at position j <- turn every pair (2m, 2m+1) of vdim by j * base^(-2m / vdim);   cached so
        s[h, i, j] = (q_i[h] . k_j[h // (H / G)]) * scale,  visible j: j <= i (and i - j < window when the mask has a size)
        o[h]_i = turn_back( sum_j softmax(s)_ij v_j, i )                                    (every pair by -i * base^(-2m / vdim))
        out = W_o concat_h o[h]

    One row ``[k (G * dim) | v (G * vdim)]`` per token, layer instance and page slot; keys after norm and rotation, values after
    theirs.  The attention kernel leaves fp32 sums, which a row-wise kernel turns back and rounds once.  ``extra_rows`` more rows
    (with a bias) that read the same input ride in the input projection; ``forward`` returns their columns as a view.
    """
    kind = "attention"

    def __init__(self, width: int, m: dict, eps: float, dtype, device, max_position: int, extra_rows: int = 0):
        from .rotary_embedding import build_banded_cos_sin
        self.width, self.eps, self.dtype, self.device = width, eps, dtype, device
        self.heads, self.kv_heads = int(m["heads"]), int(m["kv_heads"])
        self.dim, self.vdim = int(m["dim"]), int(m["vdim"])
        self.scale = float(m["scale"])
        self.window = int((m.get("mask") or {}).get("size") or 0)           # 0: every earlier token is visible
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if self.vdim > 512:
            raise ValueError(f"vdim {self.vdim}: the attention kernels hold at most 512 output columns per query row")
        H, G, d, vd = self.heads, self.kv_heads, self.dim, self.vdim
        self.q_cols, self.k_cols, self.v_cols = H * d, G * d, G * vd
        self.in_cols, self.extra = self.q_cols + self.k_cols + self.v_cols, extra_rows
        rot = m.get("rot")
        self.cos_sin = self.v_cos_sin = None
        self.rot_key = self.v_rot_key = None
        if rot:
            dims, base = int(rot.get("dims") or 0), float(rot["base"])
            if dims > d or dims % 2 or vd % 2:
                raise ValueError("rot.dims must be even and at most dim, and vdim even")
            if dims > 0:
                self.rot_key = ("pairs", dims, base, repr(rot.get("scaling")), max_position)
                self.cos_sin = build_banded_cos_sin(dims, max_position, base, rot.get("scaling"), device)
            self.v_rot_key = ("pairs", vd, base, "None", max_position)
            self.v_cos_sin = build_banded_cos_sin(vd, max_position, base, None, device)
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.w_in = e(self.in_cols + extra_rows, width)                    # [W_q ; W_k ; W_v ; extra]: one GEMM reads h once
        self.b_in = torch.zeros(self.in_cols + extra_rows, dtype=dtype, device=device) if extra_rows else None
        self.w_extra = self.w_in[self.in_cols:] if extra_rows else None
        self.b_extra = self.b_in[self.in_cols:] if extra_rows else None
        self.w_o = e(width, H * vd)
        self.q_norm, self.k_norm = e(d), e(d)
        self.cache: list = []                                              # per instance [num_blocks * block_size, G * (dim + vdim)]
        self.block_size = 0

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        q, k, v = self.q_cols, self.k_cols, self.v_cols
        spans = {"q": (0, q), "k": (q, q + k), "v": (q + k, q + k + v)}
        if leaf in spans:
            self.w_in[spans[leaf][0]:spans[leaf][1]].copy_(w)
        elif leaf == "q.norm":
            self.q_norm.copy_(w)
        elif leaf == "k.norm":
            self.k_norm.copy_(w)
        elif leaf == "o":
            self.w_o.copy_(w)
        else:
            return False
        return True

    def weight_shapes(self, width: int) -> dict:
        return {"q": (self.q_cols, width), "k": (self.k_cols, width), "v": (self.v_cols, width), "q.norm": (self.dim,), "k.norm": (self.dim,),
                "o": (width, self.heads * self.vdim)}

    def cache_row_elems(self) -> int:
        return self.k_cols + self.v_cols

    def state_slot_bytes(self) -> int:
        return 0

    def bind(self, num_blocks: int, block_size: int, num_slots: int, copies: int = 1) -> None:
        self.block_size = block_size
        self.cache = [torch.zeros(num_blocks * block_size, self.cache_row_elems(), dtype=self.dtype, device=self.device) for _ in range(copies)]

    def unbind(self) -> None:
        self.cache = []

    def forward(self, h: torch.Tensor, positions, ctx, spans: mixops.StepSpans, inst: int = 0):
        """-> (mixer output [n, width], the extra rows' projection of h (a view) or None)."""
        n, q, k = h.shape[0], self.q_cols, self.k_cols
        proj = F.linear(h, self.w_in, self.b_in)
        cache = self.cache[inst]
        mixops.headnorm_rope_store(proj, 0, q, q + k, self.heads, self.kv_heads, self.dim, self.vdim, self.q_norm, self.k_norm, False,
                                   self.cos_sin, positions, ctx.slot_mapping, cache, self.eps, v_cos_sin=self.v_cos_sin)
        acc = mixops.window_attention(proj, cache, ctx.block_tables, self.block_size, spans, self.heads, self.kv_heads, self.dim, self.vdim,
                                      self.scale, None, self.window, out_f32=self.dtype != torch.float32)
        o = mixops.head_rotate_gate(acc.view(n, self.heads, self.vdim), self.dtype, self.v_cos_sin, positions, sign=-1.0,
                                    layout=mixops.ROT_PAIRS)
        return F.linear(o, self.w_o), (proj[:, self.in_cols:] if self.extra else None)
