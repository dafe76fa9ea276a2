"""Musavik: a decoder whose layers norm every sublayer on both sides, ``x <- x + norm(mixer(norm(x)))`` then
``x <- x + norm(ff(norm(x)))``, all four RMS norms with weights stored around zero.  The token embedding is scaled by a constant
and joined by a hashed embedding of the (previous token, token) pair.  The mixer of a layer is a gated diagonal recurrence
(``rglru``) or two mixers side by side (``parallel``): windowed attention with kept first tokens and head mixing, and a gated
delta-rule recurrence.  A run of consecutive layers may be repeated several times with the same weights; every repetition
(pass) opens with ``x <- W_in [x ; x0]`` (x0: the embedding output) and has caches and states of its own.  The feed-forward is
an ungated dense block with biases, or absent.  config.json (``"architecture": "Musavik"``) lists the layers and gives every
size and constant.

The residual stream is fp32 in both number formats; projections, caches and branch outputs are bf16 (serving) or fp32; what
enters a recurrence, attention statistics and norms are fp32 in both.  Like the other models of this package it is a plain
object: named device tensors and a flat list of launches per step, the same for prompt portions, mixed batches and (captured in
CUDA graphs) decode steps.

Cache and state: per attention mixer and pass a paged key/value cache (``[blocks * block_size, kv_heads * (dim + vdim)]``,
addressed through the engine's block tables and slot numbers); per recurrent mixer and pass a state slot per live sequence
(recurrent state and convolution history); one more slot entry holds the sequence's last token for the pair embedding.  The
engine's block manager hands out pages and slots.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops
from ..layers.diag_recurrence import GatedDiagonalRecurrence
from ..layers.gated_delta import GatedDeltaMixer
from ..layers.layernorm import SandwichNorm
from ..layers.moe import BiasedDenseFF
from ..layers.parallel_mixer import ParallelMixer
from ..layers.window_attention import MixedHeadWindowAttention
from ..utils.context import get_context

MIXER_TYPES = ("rglru", "parallel")


def layer_runs(num_layers: int, loop: dict | None) -> list[tuple[int, int, bool]]:
    """Execution order: (layer, pass, whether a pass opens right before it).  Layers [start, stop) run `times` times in a row."""
    if not loop:
        return [(i, 0, False) for i in range(num_layers)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    if not (0 <= a < b <= num_layers) or times < 1:
        raise ValueError("loop: need 0 <= start < stop <= number of layers and times >= 1")
    runs = [(i, 0, False) for i in range(a)]
    for k in range(times):
        runs += [(i, k, i == a) for i in range(a, b)]
    return runs + [(i, 0, False) for i in range(b, num_layers)]


class MusavikConfig:
    """The parsed config.json plus the attribute names the engine reads from any model configuration."""
    architectures = ["Musavik"]

    def __init__(self, raw: dict, max_position_embeddings: int = 1 << 20):
        self.raw = raw
        self.layers = raw["layers"]
        self.vocab_size = int(raw["vocab"])
        self.hidden_size = int(raw["width"])
        self.norm_eps = float(raw["norm"]["eps"])
        emb = raw.get("embedding") or {}
        self.embed_scale = float(emb.get("scale", 1.0))
        self.pair = emb.get("bigram") or None           # {buckets, mul_prev, mul_cur}
        self.loop = raw.get("loop") or None
        self.num_hidden_layers = len(self.layers)
        self.max_position_embeddings = int(raw.get("max_position", max_position_embeddings))
        self.eos_token_id = raw.get("eos")
        self.runs = layer_runs(len(self.layers), self.loop)
        for i, layer in enumerate(self.layers):
            if layer["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")

    def passes_of(self, layer: int) -> int:
        return max(k for i, k, _ in self.runs if i == layer) + 1


class _Block:
    __slots__ = ("norm1", "mixer", "norm2", "ff", "passes")


class MusavikForCausalLM:
    needs_block_tables = True        # attention always reads keys through the block tables, also in a first portion
    has_recurrent_state = True       # the pair embedding alone keeps a token per sequence
    supports_prefix_cache = False    # a cached prefix cannot be skipped: the recurrent state at its end is not kept
    zero_centred = ("norm1", "norm1b", "norm2", "norm2b", "final.norm")      # 1-D tensors whose neutral value is 0, not 1 (random initialisation)

    def __init__(self, hf_config: MusavikConfig, tp_rank: int = 0, tp_size: int = 1, device="cuda", max_position: int | None = None,
                 dtype=torch.bfloat16):
        if tp_size != 1:
            raise NotImplementedError("Musavik runs on one GPU (no tensor-parallel sharding of its mixers yet)")
        c = hf_config
        self.cfg, self.device, self.dtype = c, torch.device(device), dtype
        self.hidden, self.eps = c.hidden_size, c.norm_eps
        self.vocab_shard = c.vocab_size
        self.tp_rank, self.tp_size = tp_rank, tp_size
        max_position = int(max_position or c.max_position_embeddings)
        W = self.hidden
        e = lambda *s: torch.empty(*s, dtype=dtype, device=self.device)
        self.embed, self.lm_head = e(c.vocab_size, W), e(c.vocab_size, W)
        self.pair_table = e(int(c.pair["buckets"]) + 1, W) if c.pair else None
        self.loop_in = e(W, 2 * W) if c.loop else None
        self.final_norm = torch.zeros(W, dtype=dtype, device=self.device)
        self.blocks: list[_Block] = []
        tables: dict = {}
        for i, layer in enumerate(c.layers):
            b = _Block()
            b.passes = c.passes_of(i)
            b.norm1 = SandwichNorm(W, self.eps, dtype, self.device)
            m = layer["mixer"]
            if layer["type"] == "rglru":
                b.mixer = GatedDiagonalRecurrence(W, m, dtype, self.device)
            else:
                b.mixer = ParallelMixer(W, MixedHeadWindowAttention, m["left"], GatedDeltaMixer, m["right"], m["left_scale"], m["right_scale"],
                                        dtype, self.device, eps=self.eps, max_position=max_position)
                att = b.mixer.left
                if att.cos_sin is not None:
                    att.cos_sin = tables.setdefault(att.rot_key, att.cos_sin)       # layers with one rotation share its table
            mlp = layer.get("mlp")
            b.ff = BiasedDenseFF(W, mlp, dtype, self.device) if mlp is not None else None
            b.norm2 = SandwichNorm(W, self.eps, dtype, self.device) if mlp is not None else None
            self.blocks.append(b)
        self.prev_tok = None              # int64 [slots]: the last token of every live sequence
        self.block_size = 0
        self._bound = False
        self._mm_f32_out = True

    # ---- weights -----------------------------------------------------------------------------------------------------
    def load_hf_tensor(self, name: str, w: torch.Tensor) -> None:
        """Place one checkpoint tensor: ``embed``, ``bigram``, ``loop.in``, ``head``, ``final.norm``, ``l<i>.norm1|norm1b|norm2|norm2b``,
        ``l<i>.mix.<leaf>``, ``l<i>.mlp.<leaf>``."""
        top = {"embed": self.embed, "head": self.lm_head, "final.norm": self.final_norm, "bigram": self.pair_table, "loop.in": self.loop_in}
        if name in top:
            if top[name] is None:
                raise KeyError(f"checkpoint tensor {name} has no counterpart in the configuration")
            top[name].copy_(w)
            return
        head, _, rest = name.partition(".")
        if not (head.startswith("l") and head[1:].isdigit()) or int(head[1:]) >= len(self.blocks):
            raise KeyError(f"unexpected checkpoint tensor {name}")
        b = self.blocks[int(head[1:])]
        norms = {"norm1": (b.norm1, "w_in"), "norm1b": (b.norm1, "w_out"), "norm2": (b.norm2, "w_in"), "norm2b": (b.norm2, "w_out")}
        ok = False
        if rest in norms and norms[rest][0] is not None:
            getattr(*norms[rest]).copy_(w); ok = True
        elif rest.startswith("mix."):
            ok = b.mixer.load(rest[4:], w)
        elif rest.startswith("mlp.") and b.ff is not None:
            ok = b.ff.load(rest[4:], w)
        if not ok:
            raise KeyError(f"unexpected checkpoint tensor {name}")

    def weight_shapes(self) -> dict:
        """name -> shape of every checkpoint tensor of this configuration (random initialisation, tests)."""
        c, W = self.cfg, self.hidden
        out = {"embed": (c.vocab_size, W), "head": (c.vocab_size, W), "final.norm": (W,)}
        if c.pair:
            out["bigram"] = (int(c.pair["buckets"]) + 1, W)
        if c.loop:
            out["loop.in"] = (W, 2 * W)
        for i, b in enumerate(self.blocks):
            p = f"l{i}."
            out.update({p + "norm1": (W,), p + "norm1b": (W,)})
            out.update({p + "mix." + k: v for k, v in b.mixer.weight_shapes(W).items()})
            if b.ff is not None:
                out.update({p + "norm2": (W,), p + "norm2b": (W,)})
                out.update({p + "mlp." + k: v for k, v in b.ff.weight_shapes(W).items()})
        return out

    # ---- cache and state ---------------------------------------------------------------------------------------------
    def cache_block_bytes(self, block_size: int) -> int:
        elem = 4 if self.dtype == torch.float32 else 2
        return sum(b.mixer.cache_row_elems() * b.passes for b in self.blocks) * block_size * elem

    def state_slot_bytes(self) -> int:
        return sum(b.mixer.state_slot_bytes() * b.passes for b in self.blocks) + 8

    def bind_cache(self, num_blocks: int, block_size: int, num_state_slots: int) -> None:
        self.block_size = block_size
        slots = max(num_state_slots, 1)
        for b in self.blocks:
            b.mixer.bind(num_blocks, block_size, slots, b.passes)
        self.prev_tok = torch.zeros(slots, dtype=torch.int64, device=self.device)
        self._bound = True

    def unbind_cache(self) -> None:
        for b in self.blocks:
            b.mixer.unbind()
        self.prev_tok = None
        self._bound = False

    def modules(self):
        return iter(())               # no paged-GQA attention operators of the first library: the cache is bound through bind_cache()

    # ---- forward ------------------------------------------------------------------------------------------------------
    @staticmethod
    def _spans(ctx, n: int) -> mixops.StepSpans:
        if ctx.is_prefill:
            return mixops.StepSpans(ctx.cu_seqlens_q.numel() - 1, int(ctx.max_seqlen_q), ctx.cu_seqlens_q, ctx.cu_seqlens_k, None)
        return mixops.StepSpans(n, 1, None, None, ctx.context_lens)

    def _open_pass(self, x_act: torch.Tensor, x0_act: torch.Tensor) -> torch.Tensor:
        """x <- W_in [x ; x0] as a new fp32 stream (operands in the activation type, the accumulator written as is)."""
        both = torch.cat((x_act, x0_act), -1)
        if self.dtype == torch.float32:
            return F.linear(both, self.loop_in)
        if self._mm_f32_out:
            try:
                return torch.mm(both, self.loop_in.t(), out_dtype=torch.float32)
            except (RuntimeError, TypeError):
                self._mm_f32_out = False
        return F.linear(both, self.loop_in).float()

    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, taps: list | None = None) -> torch.Tensor:
        """-> the fp32 residual stream after the last layer, [tokens, width].  ``taps`` (a list) collects a copy of the stream
        after every layer run."""
        if not self._bound:
            raise RuntimeError("bind_cache() first: this model has no cache-less path")
        ctx, c = get_context(), self.cfg
        n = input_ids.shape[0]
        spans = self._spans(ctx, n)
        x0_act = torch.empty(n, self.hidden, dtype=self.dtype, device=self.device) if c.loop else None
        pair = c.pair or {}
        x = mixops.embed_pair(input_ids, self.embed, c.embed_scale, spans, self.pair_table, int(pair.get("buckets", 0)),
                              int(pair.get("mul_prev", 0)), int(pair.get("mul_cur", 0)), self.prev_tok, ctx.state_slots, copy=x0_act)
        runs = c.runs
        x_act, h = x0_act, None                       # the stream in the activation type (when a pass opens next) / the next mixer's input
        for r, (i, k, opens) in enumerate(runs):
            b = self.blocks[i]
            if opens:
                x = self._open_pass(x_act, x0_act)
                h = None
            if h is None:
                h = b.norm1.open(x)
            y = b.mixer.forward(h, positions, ctx, spans, k)
            nxt = runs[r + 1] if r + 1 < len(runs) else None
            last_norm = b.norm2 if b.ff is not None else b.norm1
            if b.ff is not None:
                y = b.ff.forward(b.norm1.close(x, y, then=b.norm2))
            if nxt is not None and nxt[2]:            # a pass opens next: it reads the stream itself
                x_act = torch.empty(n, self.hidden, dtype=self.dtype, device=self.device)
                last_norm.close(x, y, copy=x_act)
                h = None
            else:
                h = last_norm.close(x, y, then=self.blocks[nxt[0]].norm1 if nxt is not None else None)
            if taps is not None:
                taps.append(x.clone())
        return x

    __call__ = forward

    @torch.inference_mode()
    def last_token_rows(self, hidden: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError("the fused LM head takes bf16 rows; this model normalises selected rows in compute_logits")

    @torch.inference_mode()
    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """fp32 logits of the step's last token per sequence, or of the rows named by ``ctx.logit_rows`` (int32)."""
        ctx = get_context()
        rows = getattr(ctx, "logit_rows", None)
        if rows is None and ctx.is_prefill:
            rows = (ctx.cu_seqlens_q[1:] - 1).to(torch.int32)
        hn = mixops.rmsnorm_rows(hidden, self.final_norm, self.eps, w_offset=1.0, rows_idx=rows)
        if self.dtype == torch.float32:
            return F.linear(hn, self.lm_head)
        if self._mm_f32_out:
            try:
                return torch.mm(hn, self.lm_head.t(), out_dtype=torch.float32)        # bf16 operands, fp32 accumulator written as is
            except (RuntimeError, TypeError):
                self._mm_f32_out = False          # shapes or a library build without that output type: round once to bf16 instead
        return F.linear(hn, self.lm_head).float()
