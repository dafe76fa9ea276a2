"""Latent attention: queries and keys/values pass through low-rank latents, only the key/value latent and one rotated
key part shared by all heads are cached, and the softmax denominator carries a learned per-head sink.

    c_q = rms(W_dq h) * g_q                       q[h] = W_uq[h] c_q = [q_nope (dim) | q_rot (rot_dim)]
    [c_raw | k_rot_raw] = W_dkv h                 c = rms(c_raw) * g_kv,  k_rot = rotate(k_rot_raw)       <- cached per token
    s[h, j] = (q_nope[h] . W_uk[h] c_j + rotate(q_rot[h]) . k_rot_j) * scale,  j <= i
    p = exp(s) / (sum_j exp(s_j) + exp(sink[h]))
    out = W_o concat_h ( W_uv[h] sum_j p_j c_j )

The product path never materialises per-head keys or values: ``q_nope . W_uk c = (W_uk^T q_nope) . c`` moves W_uk to the
query side (one batched GEMM over the step's tokens) and W_uv is applied to the attention output, so the attention kernel
runs multi-query over the cached rows.  A layer with ``kv_from`` reads another layer's cache (it has no W_dkv) with its own
W_uk / W_uv, queries and sink.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops
from .rotary_embedding import build_interleaved_cos_sin


class LatentAttention:
    kind = "latent_attention"

    def __init__(self, width: int, m: dict, eps: float, dtype, device, max_position: int):
        self.width, self.eps, self.dtype, self.device = width, eps, dtype, device
        self.heads, self.dim, self.rot_dim, self.vdim = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
        self.kv_rank, self.q_rank = int(m["kv_rank"]), int(m["q_rank"])
        self.scale = float(m["scale"])
        self.kv_from = m.get("kv_from")
        rot = m["rot"]
        self.rope_dims = int(rot["dims"])
        assert self.rope_dims <= self.rot_dim and self.rope_dims % 2 == 0
        if self.kv_rank > 512:
            raise ValueError(f"kv_rank {self.kv_rank}: the attention kernels hold at most 512 latent columns per query row")
        self.cos_sin = build_interleaved_cos_sin(self.rope_dims, max_position, float(rot["base"]), rot.get("scaling"), device)
        self.rot_key = (self.rope_dims, float(rot["base"]), repr(rot.get("scaling")))
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        H, qd = self.heads, self.dim + self.rot_dim
        down = self.q_rank + (0 if self.kv_from is not None else self.kv_rank + self.rot_dim)
        self.w_down = e(down, width)                      # [W_dq ; W_dkv]: one GEMM reads h once
        self.q_norm = e(self.q_rank)
        self.kv_norm = e(self.kv_rank) if self.kv_from is None else None
        self.w_uq = e(H * qd, self.q_rank)
        self.w_uk = e(H, self.dim, self.kv_rank)          # q_lat[h] = q_nope[h] @ w_uk[h]
        self.w_uv = e(H, self.vdim, self.kv_rank)
        self.w_o = e(width, H * self.vdim)
        self.sink = torch.zeros(H, dtype=torch.float32, device=device)
        self.cache = None                                 # [num_blocks * block_size, kv_rank + rot_dim]; the source layer's when kv_from
        self.block_size = 0

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "dq":
            self.w_down[:self.q_rank].copy_(w)
        elif leaf == "dkv" and self.kv_from is None:
            self.w_down[self.q_rank:].copy_(w)
        elif leaf == "dq.norm":
            self.q_norm.copy_(w)
        elif leaf == "dkv.norm" and self.kv_from is None:
            self.kv_norm.copy_(w)
        elif leaf == "uq":
            self.w_uq.copy_(w)
        elif leaf == "uk":
            self.w_uk.copy_(w.view(self.heads, self.dim, self.kv_rank))
        elif leaf == "uv":
            self.w_uv.copy_(w.view(self.heads, self.vdim, self.kv_rank))
        elif leaf == "o":
            self.w_o.copy_(w)
        elif leaf == "sink":
            self.sink.copy_(w.float())
        else:
            return False
        return True

    def cache_row_elems(self) -> int:
        """Cached elements per token (0 for a layer that borrows another layer's cache)."""
        return 0 if self.kv_from is not None else self.kv_rank + self.rot_dim

    def forward(self, h: torch.Tensor, positions: torch.Tensor, ctx, spans: mixops.StepSpans) -> torch.Tensor:
        n, H, d, rd, R = h.shape[0], self.heads, self.dim, self.rot_dim, self.kv_rank
        down = F.linear(h, self.w_down)
        cq = mixops.rmsnorm(down, self.q_norm, self.eps, cols=self.q_rank)
        q = F.linear(cq, self.w_uq).view(n, H, d + rd)
        if self.kv_from is None:
            mixops.latent_store(down[:, self.q_rank:], self.kv_norm, self.cos_sin, positions, ctx.slot_mapping, self.cache,
                                R, rd, self.eps)
        q_lat = torch.bmm(q[:, :, :d].transpose(0, 1), self.w_uk)                       # [H, n, R]
        o_lat = mixops.latent_attention(q_lat, q, d, self.cache, ctx.block_tables, self.block_size, spans, self.sink,
                                        self.cos_sin, self.scale)
        o = torch.bmm(o_lat, self.w_uv.transpose(1, 2))                                 # [H, n, vdim]
        return F.linear(o.transpose(0, 1).reshape(n, H * self.vdim), self.w_o)


class GatedWindowLatentAttention:
    """Latent attention with full-rank queries, a sliding window, an ordinary softmax and a sigmoid output gate:

        q[h] = W_q[h] h = [q_nope (dim) | q_rot (rot_dim)]
        [c_raw | k_rot_raw] = W_dkv h                 c = rms(c_raw) * g_kv,  k_rot = rotate(k_rot_raw)       <- cached per token
        s[h, i, j] = (q_nope[h] . W_uk[h] c_j + rotate(q_rot[h]) . k_rot_j) * scale,   visible j: 0 <= i - j < window (0: all j <= i)
        out = W_o ( concat_h ( W_uv[h] sum_j softmax(s)_j c_j ) * sigmoid(W_g h) )

    The rotation pairs element i of the rotated part with element i + rot.dims / 2 (banded frequencies).  As in ``LatentAttention``
    per-head keys and values are never formed: W_uk moves to the query side, W_uv to the output, and the attention kernel runs
    multi-query over the cached rows ``[c | k_rot]``, one per token, layer instance and page slot.  ``[W_q ; W_dkv ; W_g]`` and
    ``extra_rows`` more rows (with a bias) that read the same input are one GEMM; ``forward`` returns the extra columns as a view.
    """
    kind = "latent_attention"

    def __init__(self, width: int, m: dict, eps: float, dtype, device, max_position: int, extra_rows: int = 0):
        from .rotary_embedding import build_banded_cos_sin
        self.width, self.eps, self.dtype, self.device = width, eps, dtype, device
        self.heads, self.dim, self.rot_dim, self.vdim = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
        self.kv_rank = int(m["kv_rank"])
        self.scale = float(m["scale"])
        self.window = int((m.get("mask") or {}).get("size") or 0)
        rot = m["rot"]
        self.rope_dims = int(rot["dims"])
        if self.rope_dims > self.rot_dim or self.rope_dims % 2:
            raise ValueError("rot.dims must be even and at most rot_dim")
        if self.kv_rank > 512:
            raise ValueError(f"kv_rank {self.kv_rank}: the attention kernels hold at most 512 latent columns per query row")
        self.rot_key = ("halves", self.rope_dims, float(rot["base"]), repr(rot.get("scaling")), max_position)
        self.cos_sin = build_banded_cos_sin(self.rope_dims, max_position, float(rot["base"]), rot.get("scaling"), device)
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        H, qd, R = self.heads, self.dim + self.rot_dim, self.kv_rank
        self.q_cols, self.kv_cols, self.g_cols = H * qd, R + self.rot_dim, H * self.vdim
        self.in_cols, self.extra = self.q_cols + self.kv_cols + self.g_cols, extra_rows
        self.w_in = e(self.in_cols + extra_rows, width)                    # [W_q ; W_dkv ; W_g ; extra]: one GEMM reads h once
        self.b_in = torch.zeros(self.in_cols + extra_rows, dtype=dtype, device=device) if extra_rows else None
        self.w_extra = self.w_in[self.in_cols:] if extra_rows else None
        self.b_extra = self.b_in[self.in_cols:] if extra_rows else None
        self.kv_norm = e(R)
        self.w_uk = e(H, self.dim, R)                                      # q_lat[h] = q_nope[h] @ w_uk[h]
        self.w_uv = e(H, self.vdim, R)
        self.w_o = e(width, H * self.vdim)
        self.cache: list = []                                              # per instance [num_blocks * block_size, kv_rank + rot_dim]
        self.block_size = 0

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        q, kv = self.q_cols, self.kv_cols
        if leaf == "q":
            self.w_in[:q].copy_(w)
        elif leaf == "dkv":
            self.w_in[q:q + kv].copy_(w)
        elif leaf == "g":
            self.w_in[q + kv:self.in_cols].copy_(w)
        elif leaf == "dkv.norm":
            self.kv_norm.copy_(w)
        elif leaf == "uk":
            self.w_uk.copy_(w.view(self.heads, self.dim, self.kv_rank))
        elif leaf == "uv":
            self.w_uv.copy_(w.view(self.heads, self.vdim, self.kv_rank))
        elif leaf == "o":
            self.w_o.copy_(w)
        else:
            return False
        return True

    def weight_shapes(self, width: int) -> dict:
        H, R = self.heads, self.kv_rank
        return {"q": (self.q_cols, width), "dkv": (self.kv_cols, width), "dkv.norm": (R,), "uk": (H * self.dim, R), "uv": (H * self.vdim, R),
                "g": (self.g_cols, width), "o": (width, H * self.vdim)}

    def cache_row_elems(self) -> int:
        return self.kv_cols

    def state_slot_bytes(self) -> int:
        return 0

    def bind(self, num_blocks: int, block_size: int, num_slots: int, copies: int = 1) -> None:
        self.block_size = block_size
        self.cache = [torch.zeros(num_blocks * block_size, self.kv_cols, dtype=self.dtype, device=self.device) for _ in range(copies)]

    def unbind(self) -> None:
        self.cache = []

    def forward(self, h: torch.Tensor, positions, ctx, spans: mixops.StepSpans, inst: int = 0):
        """-> (mixer output [n, width], the extra rows' projection of h (a view) or None)."""
        n, H, d, rd, R = h.shape[0], self.heads, self.dim, self.rot_dim, self.kv_rank
        proj = F.linear(h, self.w_in, self.b_in)
        q = proj[:, :self.q_cols].view(n, H, d + rd)
        cache = self.cache[inst]
        mixops.latent_store(proj[:, self.q_cols:], self.kv_norm, self.cos_sin, positions, ctx.slot_mapping, cache, R, rd, self.eps,
                            layout=mixops.ROT_HALVES)
        q_lat = torch.bmm(q[:, :, :d].transpose(0, 1), self.w_uk)                       # [H, n, R]
        o_lat = mixops.latent_attention(q_lat, q, d, cache, ctx.block_tables, self.block_size, spans, None, self.cos_sin, self.scale,
                                        window=self.window, layout=mixops.ROT_HALVES)
        o = torch.bmm(o_lat, self.w_uv.transpose(1, 2))                                 # [H, n, vdim]
        gated = mixops.head_rotate_gate(o.permute(1, 0, 2), self.dtype, gate=proj[:, self.q_cols + self.kv_cols:self.in_cols])
        return F.linear(gated, self.w_o), (proj[:, self.in_cols:] if self.extra else None)
