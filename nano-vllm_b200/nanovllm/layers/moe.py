"""Feed-forward blocks of hybrid decoders: a gated dense block and a routed mixture of small experts.

Dense:   W_down (gelu_tanh(W_gate h) * (W_up h))
Biased:  W_down gelu_tanh(W_up h + b_up) + b_down
Routed:  z = W_router h (fp32), s = sigmoid(z); the `top` experts with the largest s get weight s (not renormalised);
         the weight scales the expert's INPUT:  out = sum_e expert_e(s_e h),  expert(x) = W_down relu(W_up x)^2;
         an optional shared expert of the same form runs for every token, scaled by sigmoid(W_sg h).

Group-routed (``GroupRoutedExpertsFF``):
         z = W_router h (fp32), s = softmax(z) over all router outputs; the choice is made on s + correction, only among the
         experts of the `keep` best of `count` equal groups of neighbours (a group's score: its largest s + correction); the
         weights are the chosen experts' s, divided by their sum + 1e-20, times a constant, and scale the expert's OUTPUT:
         out = sum_e w_e expert_e(h),  expert(x) = W_down (silu(W_gate x) * (W_up x));  the last `identity` router outputs are
         identity experts without tensors (expert(x) = x); an optional ungated shared expert of the same form is added.

Clamped (``ClampedGluFF``):  g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit);  W_down (g sigmoid(alpha g) (u + 1)).

Top-k by logit (``BiasedTopKExpertsFF``): z = W_router h + b_router (fp32); the `top` largest z are chosen and weighted with the
         softmax over the chosen z alone (= the softmax over all, renormalised over the chosen, which is what the group-routed kernel
         computes with one group and no correction); gated SiLU experts and an ungated shared expert as above.

The routed path groups (token, choice) pairs by expert on the device and runs two grouped GEMMs over the grouped rows; the
router (and the shared gate, one more row of the same fp32 GEMM) never leave fp32.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops


class GatedDenseFF:
    def __init__(self, width: int, mlp: dict, dtype, device):
        self.ff = int(mlp["ff"])
        self.w_gate_up = torch.empty(2 * self.ff, width, dtype=dtype, device=device)
        self.w_down = torch.empty(width, self.ff, dtype=dtype, device=device)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "gate":
            self.w_gate_up[:self.ff].copy_(w)
        elif leaf == "up":
            self.w_gate_up[self.ff:].copy_(w)
        elif leaf == "down":
            self.w_down.copy_(w)
        else:
            return False
        return True

    def forward(self, h: torch.Tensor):
        """-> (T tensor, None)"""
        return F.linear(mixops.ff_act(F.linear(h, self.w_gate_up), mixops.FF_GELU_TANH_MUL), self.w_down), None


class BiasedDenseFF:
    """W_down act(W_up h + b_up) + b_down with the tanh form of GELU: an ungated dense block whose projections carry biases
    (added in the GEMM epilogues)."""

    def __init__(self, width: int, mlp: dict, dtype, device):
        self.ff = int(mlp["ff"])
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.w_up, self.b_up = e(self.ff, width), e(self.ff)
        self.w_down, self.b_down = e(width, self.ff), e(width)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        named = {"up": self.w_up, "up.b": self.b_up, "down": self.w_down, "down.b": self.b_down}
        if leaf not in named:
            return False
        named[leaf].copy_(w)
        return True

    def weight_shapes(self, width: int) -> dict:
        return {"up": (self.ff, width), "up.b": (self.ff,), "down": (width, self.ff), "down.b": (width,)}

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return F.linear(mixops.ff_act(F.linear(h, self.w_up, self.b_up), mixops.FF_GELU_TANH), self.w_down, self.b_down)


class RoutedExpertsFF:
    def __init__(self, width: int, mlp: dict, dtype, device):
        self.experts, self.top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
        self.ff = int(mlp["expert"]["ff"])
        shared = mlp.get("shared")
        self.shared_ff = int(shared["ff"]) if shared else 0
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.w_up = e(self.experts, self.ff, width)
        self.w_down = e(self.experts, width, self.ff)
        self.w_router = torch.zeros(self.experts + (1 if shared else 0), width, dtype=torch.float32, device=device)  # + shared gate row
        if shared:
            self.sh_up, self.sh_down = e(self.shared_ff, width), e(width, self.shared_ff)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        parts = leaf.split(".")
        if parts[0].startswith("e") and parts[0][1:].isdigit() and len(parts) == 2:
            k = int(parts[0][1:])
            if parts[1] == "up":
                self.w_up[k].copy_(w)
            elif parts[1] == "down":
                self.w_down[k].copy_(w)
            else:
                return False
        elif leaf == "router":
            self.w_router[:self.experts].copy_(w.float())
        elif leaf == "shared.up" and self.shared_ff:
            self.sh_up.copy_(w)
        elif leaf == "shared.down" and self.shared_ff:
            self.sh_down.copy_(w)
        elif leaf == "shared.sg" and self.shared_ff:
            self.w_router[self.experts].copy_(w.float().view(-1))
        else:
            return False
        return True

    def forward(self, h: torch.Tensor):
        """-> (None, fp32 tensor)"""
        n = h.shape[0]
        logits = F.linear(h.float(), self.w_router)
        idx, wgt = mixops.moe_route(logits, self.experts, self.top)
        sorted_rows, pos_of, tile_expert, num_tiles = mixops.moe_align(idx, self.experts)
        inter = mixops.moe_gemm(h, sorted_rows, tile_expert, num_tiles, self.w_up, wgt=wgt, top=self.top, act=1)
        rows = mixops.moe_gemm(inter, sorted_rows, tile_expert, num_tiles, self.w_down, out_f32=True)
        shared = gate = None
        if self.shared_ff:
            shared = F.linear(mixops.ff_act(F.linear(h, self.sh_up), mixops.FF_RELU2), self.sh_down)
            gate = logits[:, self.experts]
        return None, mixops.moe_combine(rows, pos_of, self.top, n, shared, gate)


class GroupRoutedExpertsFF:
    def __init__(self, width: int, mlp: dict, dtype, device):
        r = mlp["router"]
        self.identity = int(r.get("identity") or 0)
        self.experts, self.top = int(r["experts"]), int(r["top"])          # experts with tensors; identity ones come after them
        self.outputs = self.experts + self.identity
        g = r.get("groups") or {}
        self.groups, self.keep = int(g.get("count") or 1), int(g.get("keep") or 1)
        self.route_scale = float(r.get("scale", 1.0))
        if self.outputs % self.groups or not 0 < self.keep <= self.groups or self.top > self.keep * (self.outputs // self.groups):
            raise ValueError("router groups must divide the router outputs and leave at least `top` experts open")
        self.ff = int(mlp["expert"]["ff"])
        shared = mlp.get("shared")
        self.shared_ff = int(shared["ff"]) if shared else 0
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.w_gate_up = e(max(self.experts, 1), 2 * self.ff, width)        # per expert: gate rows, then up rows
        self.w_down = e(max(self.experts, 1), width, self.ff)
        self.w_router = torch.zeros(self.outputs, width, dtype=torch.float32, device=device)
        self.router_bias = None                                             # fp32 [outputs], added to the router logits
        self.correction = torch.zeros(self.outputs, dtype=torch.float32, device=device)
        if shared:
            self.sh_gate_up, self.sh_down = e(2 * self.shared_ff, width), e(width, self.shared_ff)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        parts = leaf.split(".")
        if parts[0].startswith("e") and parts[0][1:].isdigit() and len(parts) == 2 and int(parts[0][1:]) < self.experts:
            k = int(parts[0][1:])
            if parts[1] == "gate":
                self.w_gate_up[k, :self.ff].copy_(w)
            elif parts[1] == "up":
                self.w_gate_up[k, self.ff:].copy_(w)
            elif parts[1] == "down":
                self.w_down[k].copy_(w)
            else:
                return False
        elif leaf == "router":
            self.w_router.copy_(w.float())
        elif leaf == "correction":
            self.correction.copy_(w.float().view(-1))
        elif leaf == "shared.gate" and self.shared_ff:
            self.sh_gate_up[:self.shared_ff].copy_(w)
        elif leaf == "shared.up" and self.shared_ff:
            self.sh_gate_up[self.shared_ff:].copy_(w)
        elif leaf == "shared.down" and self.shared_ff:
            self.sh_down.copy_(w)
        else:
            return False
        return True

    def weight_shapes(self, width: int) -> dict:
        out = {"router": (self.outputs, width), "correction": (self.outputs,)}
        for k in range(self.experts):
            out.update({f"e{k}.gate": (self.ff, width), f"e{k}.up": (self.ff, width), f"e{k}.down": (width, self.ff)})
        if self.shared_ff:
            out.update({"shared.gate": (self.shared_ff, width), "shared.up": (self.shared_ff, width), "shared.down": (width, self.shared_ff)})
        return out

    def forward(self, h: torch.Tensor, x32: torch.Tensor) -> torch.Tensor:
        """h: the block's input in the activation type, x32: the same rows in fp32 (router input, identity experts) -> fp32."""
        n = h.shape[0]
        logits = F.linear(x32, self.w_router, self.router_bias)
        idx, wgt = mixops.moe_route_grouped(logits, self.outputs, self.top, self.correction, self.groups, self.keep, self.experts,
                                            scale=self.route_scale)
        sorted_rows, pos_of, tile_expert, num_tiles = mixops.moe_align(idx, max(self.experts, 1))
        inter = mixops.moe_gemm(h, sorted_rows, tile_expert, num_tiles, self.w_gate_up, top=self.top, act=2, gather=True)
        rows = mixops.moe_gemm(inter, sorted_rows, tile_expert, num_tiles, self.w_down, out_f32=True)
        shared = None
        if self.shared_ff:
            shared = F.linear(mixops.ff_act(F.linear(h, self.sh_gate_up), mixops.FF_SILU_MUL), self.sh_down)
        return mixops.moe_combine(rows, pos_of, self.top, n, shared, None, wgt=wgt, ident=x32 if self.identity else None)


class BiasedTopKExpertsFF(GroupRoutedExpertsFF):
    """Routed gated-SiLU experts chosen by the largest router logits (weight matrix plus bias, fp32), weighted with the softmax over
    the chosen logits only, plus an optional ungated shared expert.  ``extra_rows`` more rows ride in no projection here: the
    block's gate is a GEMM of its own (``w_extra``, ``b_extra``), since the experts' inputs are gathered per expert."""

    def __init__(self, width: int, mlp: dict, dtype, device, extra_rows: int = 0):
        r = dict(mlp["router"])
        for key in ("identity", "groups", "scale"):
            r.pop(key, None)                                                 # one group, no identity experts, unit scale
        super().__init__(width, {**mlp, "router": r}, dtype, device)
        self.router_bias = torch.zeros(self.outputs, dtype=torch.float32, device=device)
        self.dtype = dtype
        self.w_extra = torch.empty(extra_rows, width, dtype=dtype, device=device) if extra_rows else None
        self.b_extra = torch.zeros(extra_rows, dtype=dtype, device=device) if extra_rows else None

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "router.b":
            self.router_bias.copy_(w.float().view(-1))
            return True
        if leaf == "correction":
            return False
        return super().load(leaf, w)

    def weight_shapes(self, width: int) -> dict:
        out = super().weight_shapes(width)
        del out["correction"]
        out["router.b"] = (self.outputs,)
        return out

    def forward(self, h: torch.Tensor):
        """-> (fp32 [n, width], the extra rows' projection of h or None)."""
        y = super().forward(h, h if h.dtype == torch.float32 else h.float())
        return y, (F.linear(h, self.w_extra, self.b_extra) if self.w_extra is not None else None)


class ClampedGluFF:
    """W_down (g * sigmoid(alpha * g) * (u + 1)) with g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit).  ``[W_gate ; W_up]`` and
    ``extra_rows`` more rows (with a bias) that read the same input are one GEMM; ``forward`` returns the extra columns as a view."""

    def __init__(self, width: int, mlp: dict, dtype, device, extra_rows: int = 0, alpha: float = 1.702):
        self.ff, self.limit, self.alpha = int(mlp["ff"]), float(mlp["limit"]), float(mlp.get("alpha", alpha))
        self.extra = extra_rows
        self.w_in = torch.empty(2 * self.ff + extra_rows, width, dtype=dtype, device=device)
        self.b_in = torch.zeros(2 * self.ff + extra_rows, dtype=dtype, device=device) if extra_rows else None
        self.w_extra = self.w_in[2 * self.ff:] if extra_rows else None
        self.b_extra = self.b_in[2 * self.ff:] if extra_rows else None
        self.w_down = torch.empty(width, self.ff, dtype=dtype, device=device)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "gate":
            self.w_in[:self.ff].copy_(w)
        elif leaf == "up":
            self.w_in[self.ff:2 * self.ff].copy_(w)
        elif leaf == "down":
            self.w_down.copy_(w)
        else:
            return False
        return True

    def weight_shapes(self, width: int) -> dict:
        return {"gate": (self.ff, width), "up": (self.ff, width), "down": (width, self.ff)}

    def forward(self, h: torch.Tensor):
        proj = F.linear(h, self.w_in, self.b_in)
        y = F.linear(mixops.ff_glu_clamped(proj[:, :2 * self.ff], self.limit, self.alpha), self.w_down)
        return y, (proj[:, 2 * self.ff:] if self.extra else None)
