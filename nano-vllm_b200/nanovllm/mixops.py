"""Tensor-facing wrappers over libb200mix.so (include/b200_mixers.h): the mixers of hybrid decoders and their row-wise
ops.  Like ``ops``: every function is one launch (``causal_conv``: two) of a hand-written sm_100a kernel on the current
stream, PyTorch only supplies memory and streams, and there is no CPU path.

Activations, weights and caches are bf16 or fp32 (one type per call, taken from the tensors); residual stream, recurrent
state, router logits and softmax statistics are fp32 in both.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _native as nat
from . import ops


@dataclass
class StepSpans:
    """Which tokens of a step belong to which sequence, in the two forms the kernels take.

    varlen step:  cu_q, cu_k int32 [S + 1] (cumulative tokens of this step / tokens held after it), max_q on the host
    decode step:  ctx_lens int32 [S] (tokens held after the step, 0 = padding row), one token per row
    """
    num_seqs: int
    max_q: int
    cu_q: torch.Tensor | None = None
    cu_k: torch.Tensor | None = None
    ctx_lens: torch.Tensor | None = None


def _is32(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise nat.B200Error("tensors must be on a CUDA device (there is no CPU path)")
    if t.dtype == torch.float32:
        return 1
    if t.dtype == torch.bfloat16:
        return 0
    raise nat.B200Error(f"unsupported dtype {t.dtype}")


def _same(is32: int, *tensors):
    for t in tensors:
        if t is not None and _is32(t) != is32:
            raise nat.B200Error("all tensors of a call must share one dtype")


def _p(t):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return ops._stream()          # counts the launch too


_SMS = [0]


def _sm_count() -> int:
    if not _SMS[0]:
        _SMS[0] = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _SMS[0]


def _call(name, *args):
    nat.check_mix(getattr(nat.load_mix(), name)(*args))


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None, copy: torch.Tensor | None = None) -> torch.Tensor:
    """ids int64 [n] -> fp32 [n, width]; ``copy`` (table's dtype, [n, width]) receives the same rows unconverted."""
    assert ids.dtype == torch.int64 and ids.is_contiguous() and table.is_contiguous()
    n, width = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty(n, width, dtype=torch.float32, device=table.device)
    assert copy is None or (copy.dtype == table.dtype and copy.is_contiguous() and copy.shape == out.shape)
    _call("b200m_embed", ids.data_ptr(), table.data_ptr(), out.data_ptr(), _p(copy), n, width, table.shape[0], _is32(table), _stream())
    return out


def embed_pair(ids: torch.Tensor, table: torch.Tensor, scale: float, spans: "StepSpans", pair: torch.Tensor | None = None,
               buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0, prev_tok: torch.Tensor | None = None,
               state_slots: torch.Tensor | None = None, copy: torch.Tensor | None = None) -> torch.Tensor:
    """ids int64 [n] -> fp32 [n, width] = table[id] * scale + pair[(prev * mul_prev + id * mul_cur) % buckets]; the first token
    of a sequence takes row ``buckets`` of ``pair``.  ``prev_tok`` (int64 [slots]) supplies the token before a portion and is
    left holding the portion's last token."""
    assert ids.dtype == torch.int64 and ids.is_contiguous() and table.is_contiguous()
    n, width = ids.numel(), table.shape[1]
    is32 = _is32(table)
    out = torch.empty(n, width, dtype=torch.float32, device=table.device)
    if pair is not None:
        _same(is32, pair)
        assert pair.is_contiguous() and pair.shape == (buckets + 1, width) and prev_tok.dtype == torch.int64
        assert state_slots.dtype == torch.int32 and state_slots.numel() >= spans.num_seqs
        ops.LAUNCHES[0] += 1
    assert copy is None or (copy.dtype == table.dtype and copy.is_contiguous() and copy.shape == out.shape)
    _call("b200m_embed_pair", ids.data_ptr(), table.data_ptr(), scale, _p(pair), buckets, mul_prev, mul_cur, _p(prev_tok),
          _p(state_slots), _p(spans.cu_q), _p(spans.cu_k), _p(spans.ctx_lens), out.data_ptr(), _p(copy), spans.num_seqs, spans.max_q,
          width, table.shape[0], is32, _stream())
    return out


def add_normed_norm(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, w_offset: float = 0.0, mult: float = 1.0,
                    next_weight: torch.Tensor | None = None, next_offset: float = 0.0, copy: torch.Tensor | None = None):
    """``add_normed``, then the RMS norm of the updated rows with ``next_weight`` (the next sublayer's input), returned in the
    weight's dtype (None without ``next_weight``)."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2 and y.is_contiguous() and y.shape == x.shape
    is32 = _is32(weight)
    y32 = y.dtype == torch.float32 and not is32
    if not y32:
        _same(is32, y)
    _same(is32, next_weight, copy)
    out = torch.empty(x.shape, dtype=weight.dtype, device=x.device) if next_weight is not None else None
    _call("b200m_add_normed_norm", x.data_ptr(), None if y32 else y.data_ptr(), y.data_ptr() if y32 else None, weight.data_ptr(), mult,
          w_offset, _p(copy), _p(next_weight), next_offset, _p(out), x.shape[0], x.shape[1], eps, is32, _stream())
    return out


def add_normed(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, mult: float, eps: float, w_offset: float = 0.0,
               copy: torch.Tensor | None = None) -> None:
    """x (fp32 [rows, cols], in place) += mult * rms_norm(y) * (w_offset + weight): the norm sits on the sublayer's output.
    y: the activation type of ``weight``, or fp32.  ``copy`` ([rows, cols], weight's dtype): the updated rows, rounded."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2 and y.is_contiguous() and y.shape == x.shape
    is32 = _is32(weight)
    y32 = y.dtype == torch.float32 and not is32
    if not y32:
        _same(is32, y)
    assert copy is None or (copy.dtype == weight.dtype and copy.is_contiguous() and copy.shape == x.shape)
    _call("b200m_add_normed", x.data_ptr(), None if y32 else y.data_ptr(), y.data_ptr() if y32 else None, weight.data_ptr(),
          mult, w_offset, _p(copy), x.shape[0], x.shape[1], eps, is32, _stream())


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, w_offset: float = 0.0, rows_idx: torch.Tensor | None = None):
    """RMS norm of rows of the fp32 stream (all, or those named by int32 ``rows_idx``) -> weight's dtype."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
    assert rows_idx is None or rows_idx.dtype == torch.int32
    n = x.shape[0] if rows_idx is None else rows_idx.numel()
    out = torch.empty(n, x.shape[1], dtype=weight.dtype, device=x.device)
    _call("b200m_rmsnorm_rows", x.data_ptr(), _p(rows_idx), weight.data_ptr(), w_offset, out.data_ptr(), n, x.shape[1], eps,
          _is32(weight), _stream())
    return out


def add_layernorm(x: torch.Tensor, weight: torch.Tensor | None, eps: float, a=None, b=None, b32=None, rows_idx=None,
                  out: torch.Tensor | None = None, norm: bool = True):
    """x (fp32 [rows, cols], updated in place) += a + b + b32; returns the weight-only layer norm of the updated rows
    (dtype of ``weight``), or None with ``norm=False``.  ``rows_idx``: normalise these rows only, add nothing."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
    rows, cols = x.shape
    for t in (a, b, b32):
        assert t is None or (t.is_contiguous() and t.shape == x.shape)
    assert b32 is None or b32.dtype == torch.float32
    ref = weight if weight is not None else (a if a is not None else b)
    is32 = _is32(ref) if ref is not None else 1
    _same(is32, a, b, weight)
    n_out = rows
    if rows_idx is not None:
        assert rows_idx.dtype == torch.int32 and a is None and b is None and b32 is None
        n_out = rows_idx.numel()
    if norm and out is None:
        out = torch.empty(n_out, cols, dtype=weight.dtype, device=x.device)
    _call("b200m_add_layernorm", x.data_ptr(), _p(a), _p(b), _p(b32), _p(weight), _p(out) if norm else None, _p(rows_idx),
          n_out, cols, eps, is32, _stream())
    return out if norm else None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, cols: int | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """RMS norm over the first ``cols`` elements of each row of a 2-D, unit-inner-stride x."""
    assert x.dim() == 2 and x.stride(1) == 1
    cols = x.shape[1] if cols is None else cols
    is32 = _is32(x)
    _same(is32, weight)
    if out is None:
        out = torch.empty(x.shape[0], cols, dtype=x.dtype, device=x.device)
    _call("b200m_rmsnorm", x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0), x.shape[0], cols, eps,
          is32, _stream())
    return out


FF_GELU_TANH_MUL, FF_RELU2, FF_SILU_MUL, FF_GELU_TANH = 0, 1, 2, 3


def ff_glu_clamped(x: torch.Tensor, limit: float, alpha: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [rows, 2n] = [gate | up] (a row-strided view) -> g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
    assert x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 2 == 0
    n = x.shape[1] // 2
    if out is None:
        out = torch.empty(x.shape[0], n, dtype=x.dtype, device=x.device)
    _call("b200m_ff_glu_clamped", x.data_ptr(), x.stride(0), out.data_ptr(), x.shape[0], n, float(limit), float(alpha), _is32(x), _stream())
    return out


def gated_add_normed_norm(x: torch.Tensor, y: torch.Tensor, gate: torch.Tensor | None, w_out: torch.Tensor, eps: float, dtype,
                          next_scale: float | None = None, w_next: torch.Tensor | None = None):
    """x (fp32 [rows, cols], in place) += rms_norm(y * sigmoid(gate)) * w_out; then, with ``next_scale``, returns
    rms_norm(x) * next_scale * w_next in ``dtype`` (the next sublayer's input).  y: ``dtype`` or fp32, contiguous; gate: ``dtype``, a
    row-strided view; w_out, w_next: fp32 [cols]."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2 and y.is_contiguous() and y.shape == x.shape
    is32 = int(dtype == torch.float32)
    y32 = y.dtype == torch.float32 and not is32
    assert y32 or y.dtype == dtype
    assert gate is None or (gate.dtype == dtype and gate.stride(1) == 1 and gate.shape == x.shape)
    assert w_out.dtype == torch.float32 and w_out.numel() == x.shape[1] and (w_next is None or (w_next.dtype == torch.float32 and w_next.numel() == x.shape[1]))
    out = torch.empty(x.shape, dtype=dtype, device=x.device) if next_scale is not None else None
    _call("b200m_gated_add_normed_norm", x.data_ptr(), None if y32 else y.data_ptr(), y.data_ptr() if y32 else None, _p(gate),
          gate.stride(0) if gate is not None else 0, w_out.data_ptr(), _p(w_next), float(next_scale or 0.0), _p(out), x.shape[0], x.shape[1],
          eps, is32, _stream())
    return out


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x (fp32, contiguous) <- cap * tanh(x / cap), in place."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.is_cuda
    _call("b200m_softcap", x.data_ptr(), x.numel(), float(cap), _stream())
    return x


def ff_act(x: torch.Tensor, kind: int, out: torch.Tensor | None = None) -> torch.Tensor:
    assert x.dim() == 2 and x.is_contiguous()
    n = x.shape[1] if kind in (FF_RELU2, FF_GELU_TANH) else x.shape[1] // 2
    if out is None:
        out = torch.empty(x.shape[0], n, dtype=x.dtype, device=x.device)
    _call("b200m_ff_act", x.data_ptr(), out.data_ptr(), x.shape[0], n, kind, _is32(x), _stream())
    return out


# ---- latent attention ----------------------------------------------------------------------------------------------------
ROT_PAIRS, ROT_HALVES = 0, 1          # which elements of a rotated vector form a pair: (2i, 2i+1) or (i, i + dims / 2)


def latent_store(dkv: torch.Tensor, norm_w: torch.Tensor, cos_sin: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                 cache: torch.Tensor, rank: int, rot_dim: int, eps: float, layout: int = ROT_PAIRS) -> None:
    """dkv [n, >= rank + rot_dim] -> cache rows [slots_total, rank + rot_dim] at ``slots`` (int32, -1 = skip)."""
    assert dkv.dim() == 2 and dkv.stride(1) == 1 and cache.is_contiguous() and cache.shape[-1] == rank + rot_dim
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    assert positions.dtype == torch.int64 and slots.dtype == torch.int32 and slots.numel() == dkv.shape[0]
    is32 = _is32(dkv)
    _same(is32, norm_w, cache)
    _call("b200m_latent_store", dkv.data_ptr(), dkv.stride(0), norm_w.data_ptr(), cos_sin.data_ptr(), cos_sin.shape[1],
          positions.data_ptr(), slots.data_ptr(), cache.data_ptr(), dkv.shape[0], rank, rot_dim, eps, int(layout), is32, _stream())


def latent_attention(q_lat: torch.Tensor, q_raw: torch.Tensor, q_rot_off: int, cache: torch.Tensor, block_tables: torch.Tensor,
                     block_size: int, spans: StepSpans, sink: torch.Tensor | None, cos_sin: torch.Tensor, scale: float,
                     out: torch.Tensor | None = None, fma: bool = False, window: int = 0, layout: int = ROT_PAIRS) -> torch.Tensor:
    """q_lat [H, n, rank], q_raw [n, H, >= q_rot_off + rot_dim] (any token / head strides) -> [H, n, rank].  bf16 runs on the tensor cores unless ``fma``.
    ``sink`` None: ordinary softmax.  ``window`` > 0: a query sees itself and the window - 1 keys before it."""
    H, n, rank = q_lat.shape
    rot_dim = cache.shape[-1] - rank
    assert q_lat.is_contiguous() and q_raw.stride(2) == 1 and q_raw.shape[:2] == (n, H) and cache.is_contiguous()
    assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1 and (sink is None or sink.dtype == torch.float32)
    is32 = _is32(q_lat)
    _same(is32, q_raw, cache)
    if out is None:
        out = torch.empty_like(q_lat)
    # single-token steps: few (sequence) CTAs would each walk a whole context; share the key tiles out so that about two
    # CTAs per SM are in flight.  The bound comes from the block-table width (static, so it also holds inside a CUDA graph).
    splits, part = 1, None
    if not is32 and not fma and spans.cu_q is None and H <= 64:
        keys = block_tables.shape[1] * block_size
        tiles = -(-(min(keys, window + 63) if window > 0 else keys) // 64)          # a window straddles one tile more than it fills
        chunks = -(-rank // (128 if rank <= 128 else 256))
        splits = max(1, min(tiles, 32, (2 * _sm_count()) // max(spans.num_seqs * chunks, 1)))      # whole waves: never a few CTAs over
        if splits > 1:
            part = torch.empty(spans.num_seqs * splits * 4 * H * (rank + 2), dtype=torch.float32, device=q_lat.device)   # x4: one partial per warp when H <= 16
            ops.LAUNCHES[0] += 1
    _call("b200m_latent_attention", q_lat.data_ptr(), q_raw.data_ptr(), q_raw.stride(0), q_raw.stride(1), q_rot_off, cache.data_ptr(),
          block_tables.data_ptr(), block_tables.stride(0), block_size, _p(spans.cu_q), _p(spans.cu_k), _p(spans.ctx_lens),
          _p(sink), cos_sin.data_ptr(), cos_sin.shape[1], out.data_ptr(), n, spans.num_seqs, spans.max_q, H, rank,
          rot_dim, scale, int(window), int(layout), is32, int(fma), splits, _p(part), _stream())
    return out


# ---- windowed grouped-query attention --------------------------------------------------------------------------------------
def qk_norm_store(qkv: torch.Tensor, q_cols: int, k_cols: int, v_cols: int, q_norm: torch.Tensor | None, k_norm: torch.Tensor | None,
                  slots: torch.Tensor | None, cache: torch.Tensor | None, eps: float) -> None:
    """qkv [n, q_cols + k_cols + v_cols]: whole-projection RMS norm of q in place; [norm(k) | v] -> cache rows at ``slots``."""
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= q_cols + k_cols + v_cols
    is32 = _is32(qkv)
    _same(is32, q_norm, k_norm, cache)
    if k_cols + v_cols:
        assert slots.dtype == torch.int32 and slots.numel() == qkv.shape[0] and cache.is_contiguous() and cache.shape[-1] == k_cols + v_cols
    _call("b200m_qk_norm_store", qkv.data_ptr(), qkv.stride(0), q_cols, k_cols, v_cols, _p(q_norm), _p(k_norm), _p(slots), _p(cache),
          qkv.shape[0], eps, is32, _stream())


def window_attention(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, block_size: int, spans: StepSpans,
                     heads: int, kv_heads: int, dim: int, vdim: int, scale: float, slopes: torch.Tensor | None = None,
                     window: int = 0, fma: bool = False, splits: int | None = None, keep_first: int = 0, all_values: bool = False,
                     out_f32: bool = False) -> torch.Tensor:
    """q [n, >= heads * dim] (row-strided view), cache [slots, kv_heads * (dim + vdim)] -> [n, heads * vdim].
    ``keep_first``: the first tokens of a sequence that stay visible beyond the window.  ``all_values``: every head's weights
    meet the values of every value head, -> [n, heads, kv_heads, vdim] (``head_mix_gate`` mixes them).  ``out_f32``: fp32 result."""
    n = q.shape[0]
    assert q.dim() == 2 and q.stride(1) == 1 and cache.is_contiguous() and cache.shape[-1] == kv_heads * (dim + vdim)
    assert block_tables.dtype == torch.int32 and block_tables.stride(1) == 1
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == heads)
    is32 = _is32(q)
    _same(is32, cache)
    vsets = kv_heads if all_values else 1
    out = torch.empty(n, heads * vsets * vdim, dtype=torch.float32 if out_f32 else q.dtype, device=q.device)
    part, nsplit = None, 1
    if splits is None:
        splits = window_attention_splits(spans, block_tables.shape[1] * block_size, window, kv_heads * vsets, keep_first) \
            if (not is32 and not fma) else 1
    if splits > 1 and spans.cu_q is None and not is32 and not fma:
        nsplit = splits
        part = torch.empty(spans.num_seqs * nsplit * heads * vsets * (vdim + 2), dtype=torch.float32, device=q.device)
        ops.LAUNCHES[0] += 1
    _call("b200m_window_attention", q.data_ptr(), q.stride(0), cache.data_ptr(), cache.shape[-1], kv_heads * dim,
          block_tables.data_ptr(), block_tables.stride(0), block_size, _p(spans.cu_q), _p(spans.cu_k), _p(spans.ctx_lens),
          _p(slopes), int(window), int(keep_first), int(all_values), out.data_ptr(), n, spans.num_seqs, spans.max_q, heads, kv_heads,
          dim, vdim, scale, is32, int(fma) | (2 if out_f32 else 0), nsplit, _p(part), _stream())
    return out.view(n, heads, vsets, vdim) if all_values else out


def window_attention_splits(spans: StepSpans, max_keys: int, window: int, kv_heads: int, keep_first: int = 0) -> int:
    """How many CTAs share the visible keys of one decode row: enough for about two CTAs per SM, at least two 64-key tiles each.
    Static per (batch rows, table width), so the choice also holds inside a captured graph."""
    if spans.cu_q is not None:
        return 1
    keys = min(max_keys, window + keep_first) if window > 0 else max_keys
    tiles = -(-keys // 64)
    return max(1, min(tiles // 2, 32, (2 * _sm_count()) // max(spans.num_seqs * kv_heads, 1)))


def headnorm_rope_store(x: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, kv_heads: int, dim: int, vdim: int,
                        q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, v_unit_norm: bool, cos_sin: torch.Tensor | None,
                        positions: torch.Tensor | None, slots: torch.Tensor | None, cache: torch.Tensor | None, eps: float,
                        v_cos_sin: torch.Tensor | None = None) -> None:
    """x [n, cols] (q heads at q_off, key heads at k_off, value heads at v_off): per-head RMS norm of q and k with one weight of
    ``dim`` elements shared by the heads, pair rotation by cos_sin [positions, rope_dims] (fp32), q in place; normed, rotated keys
    and (unit-RMS) values into cache rows [k (kv_heads * dim) | v (kv_heads * vdim)] at ``slots``.  ``v_cos_sin`` (fp32
    [positions, v_dims]): the value pairs are turned by the token's position before the store."""
    assert x.dim() == 2 and x.stride(1) == 1
    is32 = _is32(x)
    _same(is32, q_norm, k_norm, cache)
    rope_dims = 0
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and positions.dtype == torch.int64
        rope_dims = cos_sin.shape[1]
    v_dims = 0
    if v_cos_sin is not None:
        assert v_cos_sin.dtype == torch.float32 and v_cos_sin.is_contiguous() and positions.dtype == torch.int64
        v_dims = v_cos_sin.shape[1]
    if cache is not None:
        assert cache.is_contiguous() and cache.shape[-1] == kv_heads * (dim + vdim) and slots.dtype == torch.int32 and slots.numel() == x.shape[0]
    _call("b200m_headnorm_rope_store", x.data_ptr(), x.stride(0), q_off, k_off, v_off, heads, kv_heads, dim, vdim, _p(q_norm), _p(k_norm),
          int(v_unit_norm), _p(cos_sin), rope_dims, _p(v_cos_sin), v_dims, _p(positions), _p(slots), _p(cache), x.shape[0], eps, is32,
          _stream())


def head_rotate_gate(acc: torch.Tensor, dtype, cos_sin: torch.Tensor | None = None, positions: torch.Tensor | None = None,
                     sign: float = 1.0, layout: int = ROT_PAIRS, gate: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """acc [n, H, vdim] (any token / head strides, unit inner stride; fp32 or ``dtype``) -> [n, H * vdim] in ``dtype``: every head
    turned by ``sign`` times the token's position (cos_sin fp32 [positions, dims]: the first ``dims`` elements of a head), then
    multiplied by sigmoid(gate) (gate [n, H * vdim], a row-strided view)."""
    n, H, vdim = acc.shape
    assert acc.stride(2) == 1 and acc.dtype in (torch.float32, dtype)
    dims = 0
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and positions.dtype == torch.int64 and positions.numel() == n
        dims = cos_sin.shape[1]
    assert gate is None or (gate.stride(1) == 1 and gate.shape == (n, H * vdim) and gate.dtype == dtype)
    if out is None:
        out = torch.empty(n, H * vdim, dtype=dtype, device=acc.device)
    assert out.dtype == dtype and out.shape == (n, H * vdim) and out.stride(1) == 1
    _call("b200m_head_rotate_gate", acc.data_ptr(), int(acc.dtype == torch.float32), acc.stride(0), acc.stride(1), _p(cos_sin), dims,
          int(layout), float(sign), _p(positions), _p(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(), out.stride(0),
          n, H, vdim, int(dtype == torch.float32), _stream())
    return out


def head_mix_gate(acc: torch.Tensor, mix: torch.Tensor, gate: torch.Tensor | None, dtype, out: torch.Tensor | None = None,
                  out_scale: float = 1.0) -> torch.Tensor:
    """acc [n, H, G, vdim] (head g's weights on value head v), mix fp32 [H, H], gate [n, H * vdim] (row-strided view) ->
    [n, H * vdim] = out_scale * sigmoid(gate) * sum_g mix[h, g] acc[:, g, h // (H / G)]; ``out`` may be a row-strided view."""
    n, H, G, vdim = acc.shape
    assert acc.is_contiguous() and mix.dtype == torch.float32 and mix.is_contiguous() and mix.shape == (H, H)
    assert gate is None or (gate.stride(1) == 1 and gate.shape == (n, H * vdim) and gate.dtype == dtype)
    if out is None:
        out = torch.empty(n, H * vdim, dtype=dtype, device=acc.device)
    assert out.dtype == dtype and out.shape == (n, H * vdim) and out.stride(1) == 1
    _call("b200m_head_mix_gate", acc.data_ptr(), int(acc.dtype == torch.float32), mix.data_ptr(), _p(gate), gate.stride(0) if gate is not None else 0,
          out.data_ptr(), out.stride(0), out_scale, n, H, G, vdim, int(dtype == torch.float32), _stream())
    return out


# ---- gated diagonal recurrence and gated delta rule ------------------------------------------------------------------------
def diag_scan(u: torch.Tensor, gates: torch.Tensor, gate_bias: torch.Tensor, rate: torch.Tensor, y: torch.Tensor, state: torch.Tensor,
              state_slots: torch.Tensor, spans: StepSpans, chunk: int = 64) -> torch.Tensor:
    """u [n, C]; gates fp32 [C / cb, n, 2 cb] (per block: pre-activations of r, then of i); gate_bias fp32 [C / cb, 2 cb];
    rate fp32 [C] (<= 0); y [n, C] (row-strided view); state fp32 [slots, C] -> S * gelu_tanh(y), [n, C]."""
    n, C = u.shape
    nb, rows, cb2 = gates.shape
    assert u.stride(1) == 1 and y.stride(1) == 1 and gates.dtype == torch.float32 and gates.is_contiguous() and rows == n and nb * cb2 == 2 * C
    assert gate_bias.dtype == torch.float32 and gate_bias.is_contiguous() and gate_bias.numel() == 2 * C
    assert rate.dtype == torch.float32 and rate.numel() == C and state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == C
    is32 = _is32(u)
    _same(is32, y)
    out = torch.empty(n, C, dtype=u.dtype, device=u.device)
    ws = None
    if spans.max_q > 2 * chunk:            # long portions: chunks in parallel (three launches) instead of one serial walk
        ws = torch.empty(spans.num_seqs * (-(-spans.max_q // chunk)) * C * 2, dtype=torch.float32, device=u.device)
        ops.LAUNCHES[0] += 2
    _call("b200m_diag_scan", u.data_ptr(), u.stride(0), gates.data_ptr(), n, gate_bias.data_ptr(), rate.data_ptr(), y.data_ptr(), y.stride(0),
          state.data_ptr(), state_slots.data_ptr(), _p(spans.cu_q), _p(spans.cu_k), _p(spans.ctx_lens), out.data_ptr(), spans.num_seqs,
          spans.max_q, C, cb2 // 2, chunk, _p(ws), is32, _stream())
    return out


def gated_delta(x: torch.Tensor, q_off: int, k_off: int, v_off: int, ba: torch.Tensor, rate: torch.Tensor, dt_bias: torch.Tensor,
                state: torch.Tensor, state_slots: torch.Tensor, spans: StepSpans, heads: int, kv_heads: int, dim: int, vdim: int,
                q_scale: float) -> torch.Tensor:
    """x [n, cols]: convolved q, k ([kv_heads, dim] at q_off / k_off) and v ([heads, vdim] at v_off); ba fp32 [n, 2 heads];
    state fp32 [slots, heads, vdim, dim] -> fp32 [n, heads, vdim]."""
    n = x.shape[0]
    assert x.dim() == 2 and x.stride(1) == 1 and ba.dtype == torch.float32 and ba.stride(1) == 1 and ba.shape == (n, 2 * heads)
    assert rate.dtype == torch.float32 and dt_bias.dtype == torch.float32 and rate.numel() == heads and dt_bias.numel() == heads
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, vdim, dim)
    out = torch.empty(n, heads, vdim, dtype=torch.float32, device=x.device)
    _call("b200m_gated_delta", x.data_ptr(), x.stride(0), q_off, k_off, v_off, ba.data_ptr(), ba.stride(0), rate.data_ptr(), dt_bias.data_ptr(),
          state.data_ptr(), state_slots.data_ptr(), _p(spans.cu_q), _p(spans.cu_k), _p(spans.ctx_lens), out.data_ptr(), spans.num_seqs, heads,
          kv_heads, dim, vdim, q_scale, _is32(x), _stream())
    return out


def head_rmsnorm_gate(x: torch.Tensor, weight: torch.Tensor | None, gate: torch.Tensor | None, eps: float, dtype, silu: bool = True,
                      out: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor:
    """x fp32 [n, H, vdim] -> [n, H * vdim] = out_scale * x / rms(x) * weight * act(gate), per head; act = silu or sigmoid;
    ``out`` may be a row-strided view."""
    n, H, vdim = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    assert gate is None or (gate.stride(1) == 1 and gate.shape == (n, H * vdim) and gate.dtype == dtype)
    assert weight is None or (weight.dtype == dtype and weight.numel() == vdim)
    if out is None:
        out = torch.empty(n, H * vdim, dtype=dtype, device=x.device)
    assert out.dtype == dtype and out.shape == (n, H * vdim) and out.stride(1) == 1
    _call("b200m_head_rmsnorm_gate", x.data_ptr(), _p(weight), _p(gate), gate.stride(0) if gate is not None else 0, int(silu), out.data_ptr(),
          out.stride(0), out_scale, n, H, vdim, eps, int(dtype == torch.float32), _stream())
    return out


# ---- selective scan ------------------------------------------------------------------------------------------------------
SCAN_CHUNK = 64          # tokens per chunk of the chunk-parallel form


def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, conv_state: torch.Tensor,
                state_slots: torch.Tensor, spans: StepSpans, out: torch.Tensor | None = None, silu: bool = True) -> torch.Tensor:
    """x [n, channels] (row-strided view) -> silu(conv(x) + bias) [n, channels] (``silu=False``: no activation); conv_state [slots, taps - 1, channels] fp32
    is read for the history and left holding the inputs that follow."""
    channels, taps = weight.shape
    assert x.dim() == 2 and x.stride(1) == 1 and x.shape[1] == channels and weight.is_contiguous()
    assert conv_state.dtype == torch.float32 and conv_state.is_contiguous() and state_slots.dtype == torch.int32
    is32 = _is32(x)
    _same(is32, weight, bias)
    if out is None:
        out = torch.empty(x.shape[0], channels, dtype=x.dtype, device=x.device)
    _call("b200m_causal_conv", x.data_ptr(), x.stride(0), weight.data_ptr(), _p(bias), conv_state.data_ptr(), state_slots.data_ptr(),
          _p(spans.cu_q), _p(spans.cu_k), _p(spans.ctx_lens), out.data_ptr(), spans.num_seqs, spans.max_q, channels, taps, int(silu),
          is32, _stream())
    if taps > 1:
        ops.LAUNCHES[0] += 1
    return out


def selective_scan(u, dt_raw, dt_bias, A, Bm, Cm, Dv, z, state, state_slots, spans: StepSpans, out=None) -> torch.Tensor:
    """u, dt_raw [n, C]; Bm, Cm [n, N] and z [n, C] may be column slices of wider rows; A fp32 [C, N]; state fp32 [slots, C, N]."""
    n, channels = u.shape
    nstate = A.shape[1]
    assert u.is_contiguous() and dt_raw.is_contiguous() and A.dtype == torch.float32 and A.is_contiguous()
    assert Bm.stride(1) == 1 and Cm.stride(1) == 1 and Bm.stride(0) == Cm.stride(0) and z.stride(1) == 1
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (channels, nstate)
    is32 = _is32(u)
    _same(is32, dt_raw, dt_bias, Bm, Cm, Dv, z)
    if out is None:
        out = torch.empty_like(u)
    ws, chunk = None, SCAN_CHUNK
    if spans.max_q > 2 * chunk:            # long portions: chunks in parallel (three launches) instead of one serial walk
        nchunks = -(-spans.max_q // chunk)
        ws = torch.empty(spans.num_seqs * nchunks * channels * (nstate + 1), dtype=torch.float32, device=u.device)
        ops.LAUNCHES[0] += 2
    _call("b200m_selective_scan", u.data_ptr(), dt_raw.data_ptr(), dt_bias.data_ptr(), A.data_ptr(), Bm.data_ptr(), Cm.data_ptr(),
          Bm.stride(0), Dv.data_ptr(), z.data_ptr(), z.stride(0), state.data_ptr(), state_slots.data_ptr(), _p(spans.cu_q),
          _p(spans.cu_k), _p(spans.ctx_lens), out.data_ptr(), spans.num_seqs, channels, nstate, chunk, spans.max_q, _p(ws), is32, _stream())
    return out


# ---- routed experts ------------------------------------------------------------------------------------------------------
def moe_tile_rows() -> int:
    return nat.load_mix().b200m_moe_tile_rows()


def moe_capacity(pairs: int, num_experts: int) -> int:
    """Rows of the grouped buffers for `pairs` (token, choice) pairs: every expert's run is padded to a row tile."""
    bm = moe_tile_rows()
    return (pairs + num_experts * (bm - 1) + bm - 1) // bm * bm


def moe_route(logits: torch.Tensor, num_experts: int, top: int):
    """logits fp32 [n, >= num_experts] -> (idx int32 [n, top], weights fp32 [n, top])."""
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    n = logits.shape[0]
    idx = torch.empty(n, top, dtype=torch.int32, device=logits.device)
    wgt = torch.empty(n, top, dtype=torch.float32, device=logits.device)
    _call("b200m_moe_route", logits.data_ptr(), logits.stride(0), n, num_experts, top, idx.data_ptr(), wgt.data_ptr(), _stream())
    return idx, wgt


def moe_route_grouped(logits: torch.Tensor, num_outputs: int, top: int, correction: torch.Tensor | None = None, groups: int = 1,
                      keep: int = 1, num_real: int | None = None, sigmoid: bool = False, renorm: bool = True, scale: float = 1.0):
    """logits fp32 [n, >= num_outputs] -> (idx int32 [n, top], weights fp32 [n, top]).  Softmax (or sigmoid) scores; the choice
    is made on score + correction within the `keep` best of `groups` equal groups; weights are the plain scores of the chosen,
    renormalised and scaled.  Router outputs from ``num_real`` on are identity experts: idx -1."""
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == num_outputs)
    n = logits.shape[0]
    idx = torch.empty(n, top, dtype=torch.int32, device=logits.device)
    wgt = torch.empty(n, top, dtype=torch.float32, device=logits.device)
    _call("b200m_moe_route_grouped", logits.data_ptr(), logits.stride(0), n, num_outputs, top, _p(correction), groups, keep,
          num_outputs if num_real is None else num_real, int(sigmoid), int(renorm), scale, idx.data_ptr(), wgt.data_ptr(), _stream())
    return idx, wgt


def moe_align(idx: torch.Tensor, num_experts: int):
    """-> (sorted_rows [cap], pos_of [pairs], tile_expert [cap / tile], num_tiles [1]) int32, all on the device."""
    pairs = idx.numel()
    cap = moe_capacity(pairs, num_experts)
    dev = idx.device
    sorted_rows = torch.empty(cap, dtype=torch.int32, device=dev)
    pos_of = torch.empty(pairs, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(cap // moe_tile_rows(), dtype=torch.int32, device=dev)
    num_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    counts = torch.empty(2 * num_experts, dtype=torch.int32, device=dev)
    _call("b200m_moe_align", idx.data_ptr(), pairs, num_experts, sorted_rows.data_ptr(), cap, pos_of.data_ptr(),
          tile_expert.data_ptr(), num_tiles.data_ptr(), counts.data_ptr(), _stream())
    return sorted_rows, pos_of, tile_expert, num_tiles


def moe_gemm(A: torch.Tensor, sorted_rows, tile_expert, num_tiles, W: torch.Tensor, wgt: torch.Tensor | None = None, top: int = 1,
             act: int = 0, out_f32: bool = False, gather: bool = False) -> torch.Tensor:
    """W [experts, N, K].  With ``wgt`` or ``gather``: row i is token (pair // top) of A (times the pair's weight); else row i
    of A.  act 1: relu^2; act 2: W = [gate rows ; up rows], the result silu(gate) * up has N / 2 columns."""
    assert A.dim() == 2 and A.stride(1) == 1 and W.dim() == 3 and W.is_contiguous() and A.shape[1] == W.shape[2]
    is32 = _is32(A)
    _same(is32, W)
    cap = sorted_rows.numel()
    out = torch.empty(cap, W.shape[1] // 2 if act == 2 else W.shape[1], dtype=torch.float32 if out_f32 else A.dtype, device=A.device)
    _call("b200m_moe_gemm", A.data_ptr(), A.stride(0), sorted_rows.data_ptr(), _p(wgt), top, int(wgt is not None or gather),
          tile_expert.data_ptr(), num_tiles.data_ptr(), tile_expert.numel(), W.data_ptr(), W.shape[1], W.shape[2], out.data_ptr(),
          int(out_f32), act, is32, _stream())
    return out


def moe_combine(rows: torch.Tensor, pos_of: torch.Tensor, top: int, n: int, shared: torch.Tensor | None = None,
                gate_logit: torch.Tensor | None = None, wgt: torch.Tensor | None = None, ident: torch.Tensor | None = None) -> torch.Tensor:
    """rows fp32 [cap, width] -> fp32 [n, width]; gate_logit: fp32 column view [n] (any stride); wgt fp32 [n, top] weights the
    choices' rows; ident fp32 [n, width] stands in for the row of a choice without an expert (pos_of < 0)."""
    assert rows.dtype == torch.float32 and rows.is_contiguous()
    width = rows.shape[1]
    out = torch.empty(n, width, dtype=torch.float32, device=rows.device)
    is32 = _is32(shared) if shared is not None else 1
    gld = gate_logit.stride(0) if gate_logit is not None else 0
    assert gate_logit is None or gate_logit.dtype == torch.float32
    assert wgt is None or (wgt.dtype == torch.float32 and wgt.is_contiguous() and wgt.numel() == n * top)
    assert ident is None or (ident.dtype == torch.float32 and ident.is_contiguous() and ident.shape == out.shape)
    _call("b200m_moe_combine", rows.data_ptr(), pos_of.data_ptr(), top, _p(shared), _p(gate_logit), gld, _p(wgt), _p(ident),
          out.data_ptr(), n, width, is32, _stream())
    return out
