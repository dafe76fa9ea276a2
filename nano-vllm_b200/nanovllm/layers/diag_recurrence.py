"""Gated diagonal linear recurrence (the recurrent block of Griffin-style decoders; kind ``rglru``).

    y = gelu_tanh(W_y h + b_y)                          u = conv(W_x h + b_x) + b_c      (depthwise, `taps` wide, causal, no activation)
    r = sigmoid(A_r[b] u_b + c_r[b]),  i = sigmoid(A_i[b] u_b + c_i[b])                  (u in `blocks` equal parts, one square map per part)
    a = exp(-8 r softplus(lam))                         S <- a S + sqrt(1 - a^2) (i u)   (S fp32 [channels], from zero)
    out = W_o (S * y)

Per sequence and pass the layer keeps S and the last taps - 1 inputs of the convolution in a state slot; the slot index of every
sequence of a step arrives in ``ctx.state_slots``.  The two input projections run as one GEMM with the biases in its epilogue,
the two block-diagonal gate maps as one batched GEMM with an fp32 result; gates, decay and state never leave fp32
(``mixops.diag_scan``).  A model that runs the layer several times in a row binds one state per pass (``copies``).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops

DECAY_SHARPNESS = 8.0          # the constant c of a = exp(-c r softplus(lam))


class GatedDiagonalRecurrence:
    kind = "rglru"

    def __init__(self, width: int, m: dict, dtype, device):
        self.width, self.dtype, self.device = width, dtype, device
        self.channels, self.blocks, self.taps = int(m["width"]), int(m["blocks"]), int(m["conv"])
        if self.channels % self.blocks:
            raise ValueError("the recurrence width must be a multiple of its block count")
        C, cb = self.channels, self.channels // self.blocks
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.w_in, self.b_in = e(2 * C, width), e(2 * C)                 # [W_y ; W_x]: one GEMM reads h once
        self.conv_w, self.conv_b = e(C, self.taps), e(C)
        self.w_gates = e(self.blocks, 2 * cb, cb)                        # per block [A_r ; A_i]
        self.gate_bias = torch.zeros(self.blocks, 2 * cb, dtype=torch.float32, device=device)
        self.rate = torch.zeros(C, dtype=torch.float32, device=device)   # -c softplus(lam), formed once in fp32
        self.w_o = e(width, C)
        self.conv_state: list = []     # per pass [slots, taps - 1, channels] fp32
        self.state: list = []          # per pass [slots, channels] fp32
        self._bmm_f32_out = dtype != torch.float32

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        C, cb = self.channels, self.channels // self.blocks
        if leaf == "y":
            self.w_in[:C].copy_(w)
        elif leaf == "y.b":
            self.b_in[:C].copy_(w)
        elif leaf == "x":
            self.w_in[C:].copy_(w)
        elif leaf == "x.b":
            self.b_in[C:].copy_(w)
        elif leaf == "conv":
            self.conv_w.copy_(w)
        elif leaf == "conv.b":
            self.conv_b.copy_(w)
        elif leaf == "ra":
            self.w_gates[:, :cb].copy_(w)
        elif leaf == "ri":
            self.w_gates[:, cb:].copy_(w)
        elif leaf == "ra.b":
            self.gate_bias[:, :cb].copy_(w.float())
        elif leaf == "ri.b":
            self.gate_bias[:, cb:].copy_(w.float())
        elif leaf == "lam":
            self.rate.copy_(-DECAY_SHARPNESS * F.softplus(w.float()))
        elif leaf == "o":
            self.w_o.copy_(w)
        else:
            return False
        return True

    def weight_shapes(self, width: int) -> dict:
        C, nb, cb = self.channels, self.blocks, self.channels // self.blocks
        return {"y": (C, width), "y.b": (C,), "x": (C, width), "x.b": (C,), "conv": (C, self.taps), "conv.b": (C,),
                "ra": (nb, cb, cb), "ra.b": (nb, cb), "ri": (nb, cb, cb), "ri.b": (nb, cb), "lam": (C,), "o": (width, C)}

    def cache_row_elems(self) -> int:
        return 0

    def state_slot_bytes(self) -> int:
        return 4 * (max(self.taps - 1, 1) * self.channels + self.channels)

    def bind(self, num_blocks: int, block_size: int, num_slots: int, copies: int = 1) -> None:
        z = lambda *s: torch.zeros(*s, dtype=torch.float32, device=self.device)
        self.conv_state = [z(num_slots, max(self.taps - 1, 1), self.channels) for _ in range(copies)]
        self.state = [z(num_slots, self.channels) for _ in range(copies)]

    def unbind(self) -> None:
        self.conv_state, self.state = [], []

    def _gates(self, u: torch.Tensor) -> torch.Tensor:
        """u [n, C] -> fp32 [blocks, n, 2 cb]: both block-diagonal maps as one batched GEMM over the blocks."""
        n = u.shape[0]
        ub = u.view(n, self.blocks, -1).transpose(0, 1)                  # [blocks, n, cb], strided
        wt = self.w_gates.transpose(1, 2)                                # [blocks, cb, 2 cb]
        if self._bmm_f32_out:
            try:
                return torch.bmm(ub, wt, out_dtype=torch.float32)        # bf16 operands, fp32 accumulator written as is
            except (RuntimeError, TypeError):
                self._bmm_f32_out = False
        return torch.bmm(ub, wt).float()

    def forward(self, h: torch.Tensor, positions, ctx, spans: mixops.StepSpans, inst: int = 0) -> torch.Tensor:
        C = self.channels
        yx = F.linear(h, self.w_in, self.b_in)
        u = mixops.causal_conv(yx[:, C:], self.conv_w, self.conv_b, self.conv_state[inst], ctx.state_slots, spans, silu=False)
        s = mixops.diag_scan(u, self._gates(u), self.gate_bias, self.rate, yx[:, :C], self.state[inst], ctx.state_slots, spans)
        return F.linear(s, self.w_o)
