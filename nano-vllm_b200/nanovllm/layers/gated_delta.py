"""Gated delta-rule mixer: per head a matrix state that is decayed, corrected towards the new value along the new key, and read
out with the query.

    q = silu(conv(W_q h)), k = silu(conv(W_k h))   [kv_heads, dim]        v = silu(conv(W_v h))   [heads, vdim]     (depthwise causal, no bias)
    q <- q / sqrt(|q|^2 + 1e-6) * dim^-1/2,  k <- k / sqrt(|k|^2 + 1e-6)                  (per head; head h reads q/k head h // (heads / kv_heads))
    beta = sigmoid(W_b h)                            g = exp(-exp(A_log) softplus(W_a h + dt_bias))                 (one of each per head, fp32)
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                        (S fp32 [dim, vdim], from zero)
    out = W_o (o / rms(o) * w_norm * silu(W_g h))                                        (norm per head over vdim, weight shared by the heads)

Per sequence and pass the layer keeps S and the last taps - 1 inputs of the three convolutions (one channel-concatenated
convolution) in a state slot.  The write strength and decay inputs come from a small GEMM with an fp32 result; the unit
norms, gates and the state never leave fp32 (``mixops.gated_delta``).

The wide input projection ``[W_q ; W_k ; W_v ; W_g]`` and the output projection may be views into the merged weights of a
block that runs this mixer beside another one on the same input (``ParallelMixer``).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops


class GatedDeltaMixer:
    kind = "gated_delta"
    UNIT_EPS = 1e-6            # inside the root of the query / key normaliser (fixed in the kernel)

    def __init__(self, width: int, m: dict, eps: float, dtype, device, w_in=None, w_o=None):
        self.width, self.eps, self.dtype, self.device = width, eps, dtype, device
        self.heads, self.kv_heads = int(m["heads"]), int(m["kv_heads"])
        self.dim, self.vdim, self.taps = int(m["dim"]), int(m["vdim"]), int(m["conv"])
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if self.dim > 256:
            raise ValueError(f"dim {self.dim}: the delta-rule kernel holds at most 256 state rows per column")
        H, G, d, vd = self.heads, self.kv_heads, self.dim, self.vdim
        self.qk_cols, self.v_cols = G * d, H * vd
        self.conv_cols = 2 * self.qk_cols + self.v_cols                   # [q | k | v]
        self.in_cols = self.conv_cols + self.v_cols                       # ... | output gate
        self.out_cols = self.v_cols
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.w_in = w_in if w_in is not None else e(self.in_cols, width)
        self.w_o = w_o if w_o is not None else e(width, self.out_cols)
        assert self.w_in.shape == (self.in_cols, width) and self.w_o.shape == (width, self.out_cols)
        self.w_ba = e(2 * H, width)                                       # [W_b ; W_a]: fp32 result
        self.conv_w = e(self.conv_cols, self.taps)
        self.norm_w = e(vd)
        self.rate = torch.zeros(H, dtype=torch.float32, device=device)    # -exp(A_log)
        self.dt_bias = torch.zeros(H, dtype=torch.float32, device=device)
        self.conv_state: list = []     # per pass [slots, taps - 1, conv_cols] fp32
        self.state: list = []          # per pass [slots, heads, vdim, dim] fp32
        self._mm_f32_out = dtype != torch.float32

    @staticmethod
    def projection_cols(m: dict) -> tuple[int, int]:
        """(rows of the wide input projection, columns of the output projection) for a mixer configuration."""
        qk, v = int(m["kv_heads"]) * int(m["dim"]), int(m["heads"]) * int(m["vdim"])
        return 2 * qk + 2 * v, v

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        Q, V, H = self.qk_cols, self.v_cols, self.heads
        if leaf == "q":
            self.w_in[:Q].copy_(w)
        elif leaf == "k":
            self.w_in[Q:2 * Q].copy_(w)
        elif leaf == "v":
            self.w_in[2 * Q:2 * Q + V].copy_(w)
        elif leaf == "g":
            self.w_in[2 * Q + V:].copy_(w)
        elif leaf == "q.conv":
            self.conv_w[:Q].copy_(w)
        elif leaf == "k.conv":
            self.conv_w[Q:2 * Q].copy_(w)
        elif leaf == "v.conv":
            self.conv_w[2 * Q:].copy_(w)
        elif leaf == "b":
            self.w_ba[:H].copy_(w)
        elif leaf == "a":
            self.w_ba[H:].copy_(w)
        elif leaf == "A_log":
            self.rate.copy_(-torch.exp(w.float()))
        elif leaf == "dt_bias":
            self.dt_bias.copy_(w.float())
        elif leaf == "norm":
            self.norm_w.copy_(w)
        elif leaf == "o":
            self.w_o.copy_(w)
        else:
            return False
        return True

    def weight_shapes(self, width: int) -> dict:
        Q, V, H, K = self.qk_cols, self.v_cols, self.heads, self.taps
        return {"q": (Q, width), "q.conv": (Q, K), "k": (Q, width), "k.conv": (Q, K), "v": (V, width), "v.conv": (V, K), "b": (H, width),
                "a": (H, width), "A_log": (H,), "dt_bias": (H,), "norm": (self.vdim,), "g": (V, width), "o": (width, V)}

    def cache_row_elems(self) -> int:
        return 0

    def state_slot_bytes(self) -> int:
        return 4 * (max(self.taps - 1, 1) * self.conv_cols + self.heads * self.vdim * self.dim)

    def bind(self, num_blocks: int, block_size: int, num_slots: int, copies: int = 1) -> None:
        z = lambda *s: torch.zeros(*s, dtype=torch.float32, device=self.device)
        self.conv_state = [z(num_slots, max(self.taps - 1, 1), self.conv_cols) for _ in range(copies)]
        self.state = [z(num_slots, self.heads, self.vdim, self.dim) for _ in range(copies)]

    def unbind(self) -> None:
        self.conv_state, self.state = [], []

    def _write_and_decay_inputs(self, h: torch.Tensor) -> torch.Tensor:
        if self._mm_f32_out:
            try:
                return torch.mm(h, self.w_ba.t(), out_dtype=torch.float32)
            except (RuntimeError, TypeError):
                self._mm_f32_out = False
        return F.linear(h, self.w_ba).float()

    def mix(self, proj: torch.Tensor, h: torch.Tensor, positions, ctx, spans: mixops.StepSpans, inst: int, out: torch.Tensor | None = None,
            out_scale: float = 1.0) -> torch.Tensor:
        """proj [n, in_cols] = h W_in^T (a row-strided view) -> the output projection's operand [n, heads * vdim]."""
        Q, V = self.qk_cols, self.v_cols
        qkv = mixops.causal_conv(proj[:, :self.conv_cols], self.conv_w, None, self.conv_state[inst], ctx.state_slots, spans)
        o = mixops.gated_delta(qkv, 0, Q, 2 * Q, self._write_and_decay_inputs(h), self.rate, self.dt_bias, self.state[inst], ctx.state_slots,
                               spans, self.heads, self.kv_heads, self.dim, self.vdim, self.dim ** -0.5)
        return mixops.head_rmsnorm_gate(o, self.norm_w, proj[:, self.conv_cols:self.conv_cols + V], self.eps, self.dtype, silu=True, out=out,
                                        out_scale=out_scale)

    def forward(self, h: torch.Tensor, positions, ctx, spans: mixops.StepSpans, inst: int = 0) -> torch.Tensor:
        return F.linear(self.mix(F.linear(h, self.w_in), h, positions, ctx, spans, inst), self.w_o)
