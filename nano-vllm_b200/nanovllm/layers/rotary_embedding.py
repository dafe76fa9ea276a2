"""NeoX rotary embedding table (reference nanovllm/layers/rotary_embedding.py:17-59).

The rotation itself is fused with q/k-norm and the KV scatter in ``ops.qknorm_rope_store``; this
module owns the fp32 ``[max_pos, head_dim] = cat(cos, sin)`` table the kernel gathers from.
"""
from __future__ import annotations

from functools import lru_cache

import torch


def build_cos_sin(head_size: int, max_position: int, base: float, device=None) -> torch.Tensor:
    exponent = torch.arange(0, head_size, 2, dtype=torch.float) / head_size
    inv_freq = 1.0 / (base ** exponent)
    angles = torch.outer(torch.arange(max_position, dtype=torch.float), inv_freq)
    table = torch.cat((angles.cos(), angles.sin()), dim=-1).contiguous()
    return table.to(device) if device is not None else table


@lru_cache(4)
def get_rope(head_size: int, rotary_dim: int, max_position: int, base: float, device: str = "cuda") -> torch.Tensor:
    assert rotary_dim == head_size
    return build_cos_sin(head_size, max_position, base, device)


def build_interleaved_cos_sin(dims: int, max_position: int, base: float, scaling: dict | None = None, device=None) -> torch.Tensor:
    """fp32 ``[max_position, dims] = cat(cos, sin)`` for the interleaved layout (element 2i pairs with 2i+1), with optional
    YaRN frequency interpolation.  ``scaling`` = {factor, original, fast, slow}: with
    ``d(t) = dims * ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(d(fast)), 0)``, ``hi = min(ceil(d(slow)), dims - 1)``
    and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, pair i turns at ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``
    and both tables carry the magnitude ``0.1 ln(factor) + 1``.  Angles are formed in float64 (positions reach the
    thousands, where an fp32 product would already cost several ulps of the cosine) and rounded once."""
    import math
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = float(base) ** (-2.0 * i / dims)
    magnitude = 1.0
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])
        turn = lambda t: dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(float(base)))
        lo = max(math.floor(turn(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        freq = freq / factor * ramp + freq * (1.0 - ramp)
        magnitude = 0.1 * math.log(factor) + 1.0
    angles = torch.outer(torch.arange(max_position, dtype=torch.float64), freq)
    table = (torch.cat((angles.cos(), angles.sin()), dim=-1) * magnitude).to(torch.float32).contiguous()
    return table.to(device) if device is not None else table


def banded_frequencies(dims: int, base: float, scaling: dict | None = None) -> torch.Tensor:
    """float64 [dims / 2]: f_i = base^(-2i / dims).  ``scaling`` = {factor, low, high, original} rescales by wavelength bands
    (w = 2 pi / f): short waves (w < original / high) keep f, long ones (w > original / low) turn at f / factor, and in between the two
    are blended with s = (original / w - low) / (high - low): (1 - s) f / factor + s f."""
    import math
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = float(base) ** (-2.0 * i / dims)
    if scaling:
        factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        wave = 2.0 * math.pi / freq
        s = (original / wave - low) / (high - low)
        blended = (1.0 - s) * freq / factor + s * freq
        freq = torch.where(wave < original / high, freq, torch.where(wave > original / low, freq / factor, blended))
    return freq


def build_banded_cos_sin(dims: int, max_position: int, base: float, scaling: dict | None = None, device=None) -> torch.Tensor:
    """fp32 ``[max_position, dims] = cat(cos, sin)`` of position * banded_frequencies: pair i of a rotated vector turns by column i
    (which two elements form pair i is the consuming kernel's layout).  Angles are formed in float64 and rounded once."""
    angles = torch.outer(torch.arange(max_position, dtype=torch.float64), banded_frequencies(dims, base, scaling))
    table = torch.cat((angles.cos(), angles.sin()), dim=-1).to(torch.float32).contiguous()
    return table.to(device) if device is not None else table
