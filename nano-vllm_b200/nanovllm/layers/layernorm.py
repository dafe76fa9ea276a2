"""RMSNorm module (reference nanovllm/layers/layernorm.py:5-50) on the CUDA kernels."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size), requires_grad=False)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        """``norm(x)``, or ``(norm(x + residual), bf16(x + residual))`` when a residual is given.

        The fused form updates ``residual`` in place and returns it (the reference returns a new tensor
        with the same values)."""
        if residual is None:
            return ops.rmsnorm(x, self.weight, self.eps)
        return ops.add_rmsnorm(x, residual, self.weight, self.eps)


class ResidualLayerNorm:
    """Weight-only layer norm reading an fp32 residual stream, fused with the stream's update: ``x += a + b`` (the two
    branches of a parallel block, summed first), then ``(x - mean) / sqrt(var + eps) * w`` in the model's activation type.
    A plain object (no nn.Module): ``weight`` is a device tensor set by the model's loader."""

    def __init__(self, width: int, eps: float, dtype, device):
        self.eps = eps
        self.weight = torch.ones(width, dtype=dtype, device=device)

    def __call__(self, x, a=None, b=None, b32=None, rows_idx=None):
        from .. import mixops
        return mixops.add_layernorm(x, self.weight, self.eps, a=a, b=b, b32=b32, rows_idx=rows_idx)


class SublayerOutputNorm:
    """RMS norm on a sublayer's OUTPUT with a weight stored around zero, fused with the scaled residual update of an fp32
    stream: ``x += mult * y / sqrt(mean(y^2) + eps) * (1 + w)``.  ``copy`` receives the updated rows in the activation type
    (the next sublayer's GEMM operand; the sublayers read the stream itself, not a normed copy)."""

    def __init__(self, width: int, eps: float, dtype, device):
        self.eps = eps
        self.weight = torch.zeros(width, dtype=dtype, device=device)

    def __call__(self, x, y, mult: float, copy=None) -> None:
        from .. import mixops
        mixops.add_normed(x, y, self.weight, mult, self.eps, w_offset=1.0, copy=copy)


class SandwichNorm:
    """The norms around one sublayer of a block that norms a sublayer on both sides, ``x <- x + norm_out(f(norm_in(x)))``, both RMS norms
    with weights stored around zero (``x / sqrt(mean(x^2) + eps) * (1 + w)``) over an fp32 stream.  ``open`` norms the stream
    for the sublayer; ``close`` norms the sublayer's output, updates the stream and, given the sublayer that follows, opens
    that one in the same pass (``copy``: the updated rows in the activation type instead, for a consumer that reads the stream itself)."""

    def __init__(self, width: int, eps: float, dtype, device):
        self.eps = eps
        self.w_in = torch.zeros(width, dtype=dtype, device=device)
        self.w_out = torch.zeros(width, dtype=dtype, device=device)

    def open(self, x):
        from .. import mixops
        return mixops.rmsnorm_rows(x, self.w_in, self.eps, w_offset=1.0)

    def close(self, x, y, then: "SandwichNorm | None" = None, copy=None):
        from .. import mixops
        return mixops.add_normed_norm(x, y, self.w_out, self.eps, w_offset=1.0, next_weight=then.w_in if then is not None else None,
                                      next_offset=1.0, copy=copy)


class GatedScaledSandwich:
    """The norms, gate and column scale around one sublayer of a block that reads a normed stream and gates, norms and scales the
    sublayer's result:

        h = rms(x) * g_in                          (g_in, g_out: ONE number each)
        x <- x + ls * rms(f(h) * sigmoid(W_r h + b_r)) * g_out

    over an fp32 stream.  The gate's pre-activation ``W_r h + b_r`` comes from the sublayer (its rows ride in the sublayer's input
    projection, which reads the same h).  ``g_out * ls`` is folded into one fp32 vector when either is loaded; ``g_in`` is kept as a
    vector in the activation type (the opening norm of a step) and in fp32 (the opening norm fused into the previous close)."""

    def __init__(self, width: int, eps: float, dtype, device):
        self.eps, self.dtype = eps, dtype
        self.g_out = torch.ones(1, dtype=torch.float32, device=device)
        self.ls = torch.ones(width, dtype=torch.float32, device=device)
        self.w_out = torch.ones(width, dtype=torch.float32, device=device)        # g_out * ls
        self.w_in32 = torch.ones(width, dtype=torch.float32, device=device)       # g_in on every column
        self.w_in = torch.ones(width, dtype=dtype, device=device)

    def load(self, which: str, w: torch.Tensor) -> None:
        w = w.to(self.w_out.device, torch.float32).reshape(-1)
        if which == "in":
            self.w_in32.copy_(w.expand_as(self.w_in32))
            self.w_in.copy_(self.w_in32)
            return
        if which == "out":
            self.g_out.copy_(w)
        else:
            self.ls.copy_(w)
        torch.mul(self.ls, self.g_out, out=self.w_out)

    def open(self, x):
        from .. import mixops
        return mixops.rmsnorm_rows(x, self.w_in, self.eps)

    def close(self, x, y, gate, then: "GatedScaledSandwich | None" = None):
        """x += ls * norm_out(y * sigmoid(gate)); with ``then`` also returns that sublayer's normed input."""
        from .. import mixops
        return mixops.gated_add_normed_norm(x, y, gate, self.w_out, self.eps, self.dtype, next_scale=1.0 if then is not None else None,
                                            w_next=then.w_in32 if then is not None else None)
