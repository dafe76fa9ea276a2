"""Fegolorn: a decoder whose layers read a normed stream and gate, norm and scale what a sublayer returns,

    x <- x + ls1 * rms(mixer(h) * sigmoid(R1 h + r1)) * g1b,   h = rms(x) * g1
    x <- x + ls2 * rms(ff(h') * sigmoid(R2 h' + r2)) * g2b,    h' = rms(x) * g2

with ONE number as the weight of every norm, a column vector ``ls`` and a gate matrix ``R`` per sublayer.  The token embedding is
scaled by a constant and joined by a hashed embedding of the (previous token, token) pair.  The mixer of a layer is grouped-query
attention with per-head query/key norms, a banded partial rotation and values that are rotated by their own position and turned
back at the query's (``attention``), or windowed latent attention with an output gate (``latent_attention``).  The feed-forward
is a clamped gated dense block, a mixture of gated experts chosen by the largest router logits with a shared expert, or absent.
A layer may run with another layer's weights (``weights_of``) and a cache of its own.  The logits pass through a tanh soft cap.
config.json (``"architecture": "Fegolorn"``) lists the layers and gives every size and constant.

The residual stream is fp32 in both number formats; projections, caches and branch outputs are bf16 (serving) or fp32; norms,
attention statistics, rotation angles, router logits and the expert sum are fp32 in both.  Like the other models of this
package it is a plain object: named device tensors and a flat list of launches per step, the same for prompt portions, mixed
batches and (captured in CUDA graphs) decode steps.

Cache and state: per layer (also one that borrows its weights) a paged cache, ``[blocks * block_size, kv_heads * (dim + vdim)]``
for attention and ``[blocks * block_size, kv_rank + rot_dim]`` for latent attention, addressed through the engine's block tables
and slot numbers; one state-slot entry per live sequence holds its last token for the pair embedding.  The engine's block
manager hands out pages and slots.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops
from ..layers.latent_attention import GatedWindowLatentAttention
from ..layers.layernorm import GatedScaledSandwich
from ..layers.moe import BiasedTopKExpertsFF, ClampedGluFF
from ..layers.window_attention import RotatedValueAttention
from ..utils.context import get_context

MIXERS = {"attention": RotatedValueAttention, "latent_attention": GatedWindowLatentAttention}
FEED_FORWARDS = {"dense": ClampedGluFF, "moe": BiasedTopKExpertsFF}


class FegolornConfig:
    """The parsed config.json plus the attribute names the engine reads from any model configuration."""
    architectures = ["Fegolorn"]

    def __init__(self, raw: dict, max_position_embeddings: int = 1 << 20):
        self.raw = raw
        self.layers = raw["layers"]
        self.vocab_size = int(raw["vocab"])
        self.hidden_size = int(raw["width"])
        self.norm_eps = float(raw["norm"]["eps"])
        emb = raw.get("embedding") or {}
        self.embed_scale = float(emb.get("scale", 1.0))
        self.pair = emb.get("bigram") or None           # {buckets, mul_prev, mul_cur}
        self.logit_softcap = float(raw.get("logit_softcap") or 0.0)
        self.num_hidden_layers = len(self.layers)
        self.max_position_embeddings = int(raw.get("max_position", max_position_embeddings))
        self.eos_token_id = raw.get("eos")
        # runs: (layer that owns the weights, which of that layer's caches) in execution order; a borrowing layer runs with the owner's
        # entry (sizes and constants), its own entry only has to agree in the mixer type
        self.runs: list[tuple[int, int]] = []
        uses: dict[int, int] = {}
        for i, layer in enumerate(self.layers):
            if layer["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") not in FEED_FORWARDS:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            src = layer.get("weights_of")
            if src is None:
                src = i
            else:
                src = int(src)
                if not 0 <= src < i or self.layers[src].get("weights_of") is not None:
                    raise ValueError(f"layer {i}: weights_of must name an earlier layer with tensors of its own")
                if layer["type"] != self.layers[src]["type"]:
                    raise ValueError(f"layer {i}: its mixer type differs from layer {src}, whose weights it uses")
            self.runs.append((src, uses.get(src, 0)))
            uses[src] = uses.get(src, 0) + 1
        self.copies = uses                               # weight-owning layer -> caches it needs


class _Block:
    __slots__ = ("norm1", "mixer", "norm2", "ff")


class FegolornForCausalLM:
    needs_block_tables = True        # attention always reads keys through the block tables, also in a first portion
    has_recurrent_state = True       # the pair embedding keeps a token per sequence
    supports_prefix_cache = False    # the token before a skipped prefix's end is not kept apart from the state slot

    def __init__(self, hf_config: FegolornConfig, tp_rank: int = 0, tp_size: int = 1, device="cuda", max_position: int | None = None,
                 dtype=torch.bfloat16):
        if tp_size != 1:
            raise NotImplementedError("Fegolorn runs on one GPU (no tensor-parallel sharding of its mixers yet)")
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
        self.final_norm = torch.ones(W, dtype=dtype, device=self.device)        # one number, on every column
        self.blocks: dict[int, _Block] = {}
        tables: dict = {}
        for i, layer in enumerate(c.layers):
            if layer.get("weights_of") is not None:
                continue
            b = _Block()
            b.norm1 = GatedScaledSandwich(W, self.eps, dtype, self.device)
            b.mixer = MIXERS[layer["type"]](W, layer["mixer"], self.eps, dtype, self.device, max_position, extra_rows=W)
            for table, key in (("cos_sin", "rot_key"), ("v_cos_sin", "v_rot_key")):      # layers with one rotation share its table
                if getattr(b.mixer, table, None) is not None:
                    setattr(b.mixer, table, tables.setdefault(getattr(b.mixer, key), getattr(b.mixer, table)))
            mlp = layer.get("mlp")
            b.ff = FEED_FORWARDS[mlp["kind"]](W, mlp, dtype, self.device, extra_rows=W) if mlp is not None else None
            b.norm2 = GatedScaledSandwich(W, self.eps, dtype, self.device) if mlp is not None else None
            self.blocks[i] = b
        self.prev_tok = None              # int64 [slots]: the last token of every live sequence
        self.block_size = 0
        self._bound = False
        self._mm_f32_out = True

    # ---- weights -----------------------------------------------------------------------------------------------------
    def load_hf_tensor(self, name: str, w: torch.Tensor) -> None:
        """Place one checkpoint tensor: ``embed``, ``bigram``, ``head``, ``final.norm``, ``l<i>.norm1|norm1b|norm2|norm2b`` (one number each),
        ``l<i>.ls1|ls2``, ``l<i>.rg1|rg2`` and their ``.b``, ``l<i>.mix.<leaf>``, ``l<i>.mlp.<leaf>``."""
        top = {"embed": self.embed, "head": self.lm_head, "bigram": self.pair_table}
        if name in top:
            if top[name] is None:
                raise KeyError(f"checkpoint tensor {name} has no counterpart in the configuration")
            top[name].copy_(w)
            return
        if name == "final.norm":
            self.final_norm.copy_(w.to(self.device, torch.float32).reshape(-1).expand_as(self.final_norm))
            return
        head, _, rest = name.partition(".")
        if not (head.startswith("l") and head[1:].isdigit()) or int(head[1:]) not in self.blocks:
            raise KeyError(f"unexpected checkpoint tensor {name}")
        b = self.blocks[int(head[1:])]
        norms = {"norm1": (b.norm1, "in"), "norm1b": (b.norm1, "out"), "ls1": (b.norm1, "ls"),
                 "norm2": (b.norm2, "in"), "norm2b": (b.norm2, "out"), "ls2": (b.norm2, "ls")}
        gates = {"rg1": (b.mixer, "w_extra"), "rg1.b": (b.mixer, "b_extra"), "rg2": (b.ff, "w_extra"), "rg2.b": (b.ff, "b_extra")}
        ok = False
        if rest in norms and norms[rest][0] is not None:
            norms[rest][0].load(norms[rest][1], w); ok = True
        elif rest in gates and gates[rest][0] is not None:
            getattr(*gates[rest]).copy_(w); ok = True
        elif rest.startswith("mix."):
            ok = b.mixer.load(rest[4:], w)
        elif rest.startswith("mlp.") and b.ff is not None:
            ok = b.ff.load(rest[4:], w)
        if not ok:
            raise KeyError(f"unexpected checkpoint tensor {name}")

    def weight_shapes(self) -> dict:
        """name -> shape of every checkpoint tensor of this configuration (random initialisation, tests).  The norms' single numbers are
        listed as one-element vectors."""
        c, W = self.cfg, self.hidden
        out = {"embed": (c.vocab_size, W), "head": (c.vocab_size, W), "final.norm": (1,)}
        if c.pair:
            out["bigram"] = (int(c.pair["buckets"]) + 1, W)
        for i, b in self.blocks.items():
            p = f"l{i}."
            out.update({p + "norm1": (1,), p + "norm1b": (1,), p + "ls1": (W,), p + "rg1": (W, W), p + "rg1.b": (W,)})
            out.update({p + "mix." + k: v for k, v in b.mixer.weight_shapes(W).items()})
            if b.ff is not None:
                out.update({p + "norm2": (1,), p + "norm2b": (1,), p + "ls2": (W,), p + "rg2": (W, W), p + "rg2.b": (W,)})
                out.update({p + "mlp." + k: v for k, v in b.ff.weight_shapes(W).items()})
        return out

    # ---- cache and state ---------------------------------------------------------------------------------------------
    def cache_block_bytes(self, block_size: int) -> int:
        elem = 4 if self.dtype == torch.float32 else 2
        return sum(b.mixer.cache_row_elems() * self.cfg.copies[i] for i, b in self.blocks.items()) * block_size * elem

    def state_slot_bytes(self) -> int:
        return 8

    def bind_cache(self, num_blocks: int, block_size: int, num_state_slots: int) -> None:
        self.block_size = block_size
        slots = max(num_state_slots, 1)
        for i, b in self.blocks.items():
            b.mixer.bind(num_blocks, block_size, slots, self.cfg.copies[i])
        self.prev_tok = torch.zeros(slots, dtype=torch.int64, device=self.device)
        self._bound = True

    def unbind_cache(self) -> None:
        for b in self.blocks.values():
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

    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, taps: list | None = None) -> torch.Tensor:
        """-> the fp32 residual stream after the last layer, [tokens, width].  ``taps`` (a list) collects a copy of the stream
        after every layer."""
        if not self._bound:
            raise RuntimeError("bind_cache() first: this model has no cache-less path")
        ctx, c = get_context(), self.cfg
        spans = self._spans(ctx, input_ids.shape[0])
        pair = c.pair or {}
        x = mixops.embed_pair(input_ids, self.embed, c.embed_scale, spans, self.pair_table, int(pair.get("buckets", 0)),
                              int(pair.get("mul_prev", 0)), int(pair.get("mul_cur", 0)), self.prev_tok, ctx.state_slots)
        runs = c.runs
        h = self.blocks[runs[0][0]].norm1.open(x) if runs else None
        for r, (i, inst) in enumerate(runs):
            b = self.blocks[i]
            nxt = self.blocks[runs[r + 1][0]].norm1 if r + 1 < len(runs) else None
            y, gate = b.mixer.forward(h, positions, ctx, spans, inst)
            if b.ff is not None:
                y, gate = b.ff.forward(b.norm1.close(x, y, gate, then=b.norm2))
                h = b.norm2.close(x, y, gate, then=nxt)
            else:
                h = b.norm1.close(x, y, gate, then=nxt)
            if taps is not None:
                taps.append(x.clone())
        return x

    __call__ = forward

    @torch.inference_mode()
    def last_token_rows(self, hidden: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError("the fused LM head takes bf16 rows; this model normalises selected rows in compute_logits")

    @torch.inference_mode()
    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """fp32 logits of the step's last token per sequence, or of the rows named by ``ctx.logit_rows`` (int32), soft-capped."""
        ctx = get_context()
        rows = getattr(ctx, "logit_rows", None)
        if rows is None and ctx.is_prefill:
            rows = (ctx.cu_seqlens_q[1:] - 1).to(torch.int32)
        hn = mixops.rmsnorm_rows(hidden, self.final_norm, self.eps, rows_idx=rows)
        logits = None
        if self.dtype == torch.float32:
            logits = F.linear(hn, self.lm_head)
        elif self._mm_f32_out:
            try:
                logits = torch.mm(hn, self.lm_head.t(), out_dtype=torch.float32)      # bf16 operands, fp32 accumulator written as is
            except (RuntimeError, TypeError):
                self._mm_f32_out = False          # shapes or a library build without that output type: round once to bf16 instead
        if logits is None:
            logits = F.linear(hn, self.lm_head).float()
        if self.cfg.logit_softcap > 0.0:
            mixops.softcap_(logits, self.cfg.logit_softcap)
        return logits
