"""Two sequence mixers side by side on the same input, their results summed with fixed weights:
``out = c_left * left(h) + c_right * right(h)``.

Both read h, so their input projections are one GEMM over the merged rows ``[W_in_left ; W_in_right]`` (biases in the
epilogue), and both end in an output projection, so ``c_l W_ol a + c_r W_or b = [W_ol | W_or] [c_l a ; c_r b]`` is one GEMM too:
each mixer writes its scaled operand into its columns of one buffer.  The sub-mixers hold views into the merged weights and load
their own tensors (``left.*`` / ``right.*``).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops


class ParallelMixer:
    kind = "parallel"

    def __init__(self, width: int, left_cls, left_cfg: dict, right_cls, right_cfg: dict, left_scale: float, right_scale: float, dtype, device,
                 **common):
        self.width, self.dtype, self.device = width, dtype, device
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        probe_l, probe_r = left_cls.projection_cols(left_cfg), right_cls.projection_cols(right_cfg)
        (li, lo), (ri, ro) = probe_l, probe_r
        self.w_in = torch.empty(li + ri, width, dtype=dtype, device=device)
        self.b_in = torch.zeros(li + ri, dtype=dtype, device=device)
        self.w_o = torch.empty(width, lo + ro, dtype=dtype, device=device)
        self.left = left_cls(width, left_cfg, dtype=dtype, device=device, w_in=self.w_in[:li], b_in=self.b_in[:li], w_o=self.w_o[:, :lo], **common)
        self.right = right_cls(width, right_cfg, dtype=dtype, device=device, w_in=self.w_in[li:], w_o=self.w_o[:, lo:],
                               **{k: v for k, v in common.items() if k == "eps"})
        self.split_in, self.split_out = li, lo

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        side, _, rest = leaf.partition(".")
        if side == "left":
            return self.left.load(rest, w)
        if side == "right":
            return self.right.load(rest, w)
        return False

    def weight_shapes(self, width: int) -> dict:
        out = {"left." + k: v for k, v in self.left.weight_shapes(width).items()}
        out.update({"right." + k: v for k, v in self.right.weight_shapes(width).items()})
        return out

    def cache_row_elems(self) -> int:
        return self.left.cache_row_elems() + self.right.cache_row_elems()

    def state_slot_bytes(self) -> int:
        return self.left.state_slot_bytes() + self.right.state_slot_bytes()

    def bind(self, num_blocks: int, block_size: int, num_slots: int, copies: int = 1) -> None:
        self.left.bind(num_blocks, block_size, num_slots, copies)
        self.right.bind(num_blocks, block_size, num_slots, copies)

    def unbind(self) -> None:
        self.left.unbind()
        self.right.unbind()

    def forward(self, h: torch.Tensor, positions, ctx, spans: mixops.StepSpans, inst: int = 0) -> torch.Tensor:
        proj = F.linear(h, self.w_in, self.b_in)
        both = torch.empty(h.shape[0], self.w_o.shape[1], dtype=self.dtype, device=self.device)
        self.left.mix(proj[:, :self.split_in], h, positions, ctx, spans, inst, out=both[:, :self.split_out], out_scale=self.left_scale)
        self.right.mix(proj[:, self.split_in:], h, positions, ctx, spans, inst, out=both[:, self.split_out:], out_scale=self.right_scale)
        return F.linear(both, self.w_o)
