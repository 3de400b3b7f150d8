"""Feed-forwards without a gate, W_down f(W_up h), alone ("act_mlp") or as a mixture of experts
("routed_experts", whose experts may also be gated, W_down (f(W_gate h) * (W_up h)), and whose router may
have a bias): a router scores the experts per token in float32 (sigmoid or softmax), experts lie in
equal groups of neighbours of which only the best ``group_keep`` (by the sum of their ``group_top`` best
scores) can be chosen, the ``top`` best experts of those run for the token, weighted by their scores
(as they are, or divided by their sum), and a shared expert of the same form may run for every token.
The experts' products are grouped matrix products over (token, expert) pairs listed expert by expert on
the device (csrc/moe.cu); nothing of the routing is read by the host.

Further options: ``identity`` router outputs behind the experts stand for the input itself (a chosen one adds
weight * h and runs no product); ``choice_bias``: a number per router output that is added to the scores for
the choice alone (the weights are the scores without it); ``renorm_floor`` joins the sum the chosen scores are
divided by, ``weight_scale`` multiplies the weights; gated experts may use ``clamped_swish`` (gate and up
clamped by ``limit``, g * sigmoid(slope * g) * (up + 1)); the shared expert of gated experts is gated too, with
``shared_limit`` as its clamp.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import FeedForward, op_mark, register
from .spec import TensorSpec


@dataclass(frozen=True)
class ActMLPParams:
    hidden_size: int
    intermediate_size: int
    activation: str = "relu_squared"     # a name of ops.kernels.ACTIVATIONS


@register("ffn", "act_mlp")
class ActMLP(FeedForward):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.act = kernels.ACTIVATIONS[self.params.activation]

    def tensors(self) -> Dict[str, TensorSpec]:
        p = self.params
        return {"up": TensorSpec((p.intermediate_size, p.hidden_size)),
                "down": TensorSpec((p.hidden_size, p.intermediate_size))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_up, self.w_down = tensors["up"], tensors["down"]

    def nbytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_up, self.w_down))

    def run(self, x, ctx, name: str) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        act = rt.workspace.get(name + ".act", (rt.max_tokens, p.intermediate_size), rt.dtype)[:T]
        linear(x, self.w_up, act)
        kernels.bias_act(act, None, self.act)
        op_mark(ctx, "up+act", self.w_up, T)
        out = rt.workspace.get(name + ".out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        linear(act, self.w_down, out)
        op_mark(ctx, "down_proj", self.w_down, T)
        return out

    def forward(self, x, ctx) -> torch.Tensor:
        return self.run(x, ctx, "ffn")


@dataclass(frozen=True)
class RoutedExpertsParams:
    hidden_size: int
    intermediate_size: int               # of one expert
    num_experts: int
    top: int
    groups: int = 1
    group_keep: int = 1
    group_top: int = 2                   # a group is scored by the sum of its so many best experts
    score: str = "sigmoid"               # or "softmax"
    renormalize: bool = False            # divide the chosen weights by their sum
    activation: str = "gelu"
    shared_intermediate_size: int = 0    # 0: no shared expert
    shared_activation: Optional[str] = None
    gated: bool = False                  # experts are W_down (f(W_gate h) * (W_up h)) instead of W_down f(W_up h)
    router_bias: bool = False            # a bias on the router's logits
    identity: int = 0                    # router outputs behind the experts that stand for the input itself
    choice_bias: bool = False            # a number per router output added to the scores for the choice alone
    weight_scale: float = 1.0            # factor on the chosen experts' weights
    renorm_floor: float = 0.0            # renormalize: the chosen scores are divided by their sum + this
    limit: float = 0.0                   # clamped_swish: the clamp of gate and up
    slope: float = 1.0                   # clamped_swish: g * sigmoid(slope * g)
    shared_limit: float = 0.0            # the shared expert's clamp (0: ``limit``)


@register("ffn", "routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        self.outputs = p.num_experts + p.identity          # what the router scores
        if p.identity < 0 or self.outputs % p.groups != 0 or not 1 <= p.group_keep <= p.groups:
            raise ValueError(f"{self.outputs} router outputs do not form {p.groups} equal groups of which {p.group_keep} stay")
        if not 1 <= p.top <= p.group_keep * (self.outputs // p.groups):
            raise ValueError(f"top {p.top} experts cannot be chosen among {p.group_keep} groups of "
                             f"{self.outputs // p.groups}")
        if p.score not in ("sigmoid", "softmax"):
            raise ValueError(f"router score '{p.score}' is not supported (sigmoid, softmax)")
        self.clamped = p.activation == "clamped_swish"
        if self.clamped and not (p.gated and p.limit > 0):
            raise ValueError("routed_experts: clamped_swish goes with gated experts and a positive limit")
        self.act = kernels.ACT_CLAMPED_SWISH if self.clamped else kernels.ACTIVATIONS[p.activation]
        self.shared = None
        if p.shared_intermediate_size > 0 and p.gated:
            from .mlp import GatedMLPParams, SwiGLUMLP
            from .spec import PartSpec
            self.shared = SwiGLUMLP(PartSpec("swiglu_mlp", GatedMLPParams(
                p.hidden_size, p.shared_intermediate_size, activation=p.shared_activation or p.activation,
                limit=p.shared_limit or p.limit, slope=p.slope)), rt)
        elif p.shared_intermediate_size > 0:
            from .spec import PartSpec
            self.shared = ActMLP(PartSpec("act_mlp", ActMLPParams(p.hidden_size, p.shared_intermediate_size,
                                                                  p.shared_activation or p.activation)), rt)

    def tensors(self) -> Dict[str, TensorSpec]:
        p = self.params
        t = {"router": TensorSpec((self.outputs, p.hidden_size))}
        if p.router_bias:
            t["router_bias"] = TensorSpec((self.outputs,))
        if p.choice_bias:
            t["choice_bias"] = TensorSpec((self.outputs,))
        for e in range(p.num_experts):
            if p.gated:
                t[f"gate{e}"] = TensorSpec((p.intermediate_size, p.hidden_size))
            t[f"up{e}"] = TensorSpec((p.intermediate_size, p.hidden_size))
            t[f"down{e}"] = TensorSpec((p.hidden_size, p.intermediate_size))
        if self.shared is not None:
            if p.gated:
                t["shared_gate"] = TensorSpec((p.shared_intermediate_size, p.hidden_size))
            t["shared_up"] = TensorSpec((p.shared_intermediate_size, p.hidden_size))
            t["shared_down"] = TensorSpec((p.hidden_size, p.shared_intermediate_size))
        return t

    def fused(self) -> Dict[str, list]:
        n = self.params.num_experts
        if self.params.gated:      # every expert's gate rows, then its up rows
            return {"up_all": [f"{m}{e}" for e in range(n) for m in ("gate", "up")],
                    "down_all": [f"down{e}" for e in range(n)]}
        return {"up_all": [f"up{e}" for e in range(n)], "down_all": [f"down{e}" for e in range(n)]}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.params

        def stacked(fused_name: str, stem: str) -> torch.Tensor:
            if fused_name in tensors:
                return tensors[fused_name]
            stems = ("gate", "up") if (p.gated and stem == "up") else (stem,)
            ws = [tensors[f"{m}{e}"] for e in range(p.num_experts) for m in stems]
            dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
            return torch.cat([w.to(dt) for w in ws], dim=0).contiguous()

        self.w_up = stacked("up_all", "up")            # [experts * ff, hidden] (gated: [experts * 2 ff, hidden])
        self.b_router = tensors["router_bias"].float().contiguous() if p.router_bias else None
        self.b_choice = tensors["choice_bias"].float().contiguous() if p.choice_bias else None
        self.w_down = stacked("down_all", "down")      # [experts * hidden, ff]
        self.w_router = tensors["router"]
        if self.shared is not None and p.gated:
            self.shared.load({"gate": tensors["shared_gate"], "up": tensors["shared_up"], "down": tensors["shared_down"]})
        elif self.shared is not None:
            self.shared.load({"up": tensors["shared_up"], "down": tensors["shared_down"]})

    def nbytes(self) -> int:
        n = sum(w.numel() * w.element_size() for w in (self.w_up, self.w_down, self.w_router))
        return n + (self.shared.nbytes() if self.shared is not None else 0)

    def forward(self, x, ctx) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        ws = rt.workspace
        pairs = T * p.top
        max_pairs = rt.max_tokens * p.top
        max_tiles = kernels.moe_max_tiles(pairs, max(p.num_experts, 1))
        cap_tiles = kernels.moe_max_tiles(max_pairs, max(p.num_experts, 1))
        choice = ws.get("moe.choice", (max_pairs,), torch.int32)
        weight = ws.get("moe.weight", (max_pairs,), torch.float32)
        order = ws.get("moe.order", (max_pairs,), torch.int32)
        tile_expert = ws.get("moe.tile_expert", (cap_tiles,), torch.int32)
        tile_begin = ws.get("moe.tile_begin", (cap_tiles,), torch.int32)
        tile_rows = ws.get("moe.tile_rows", (cap_tiles,), torch.int32)
        meta = ws.get("moe.meta", (4,), torch.int32)
        # the router's logits as a matrix product with float32 sums and a float32 result, then the choice
        logits = ws.get("moe.logits", (rt.max_tokens, self.outputs), torch.float32)[:T]
        linear(x, self.w_router, logits)
        kernels.moe_route(logits, None, choice, weight, T, p.groups, p.group_keep, p.group_top, p.top,
                          softmax=p.score == "softmax", renorm=p.renormalize, bias=self.b_router,
                          choice_bias=self.b_choice, weight_scale=p.weight_scale, renorm_floor=p.renorm_floor)
        kernels.moe_group(choice, pairs, self.outputs, order, tile_expert, tile_begin, tile_rows, meta,
                          tiled=p.num_experts)
        op_mark(ctx, "route", self.w_router, T)
        if x.dtype != self.w_up.dtype:
            raise kernels.KernelError("routed_experts: expert weights must have the activation type")
        act = ws.get("moe.act", (max_pairs, p.intermediate_size), rt.dtype)[:pairs]
        y = ws.get("moe.y", (max_pairs, p.hidden_size), rt.dtype)[:pairs]
        lists = (order, tile_expert, tile_begin, tile_rows, meta, max_tiles)
        if p.gated:
            gu = ws.get("moe.gate_up", (max_pairs, 2 * p.intermediate_size), rt.dtype)[:pairs]
            kernels.moe_gemm(x, p.top, self.w_up, gu, *lists)
            kernels.gated_act(gu, act, self.act, p.limit, p.slope)
        else:
            kernels.moe_gemm(x, p.top, self.w_up, act, *lists, act=self.act)
        kernels.moe_gemm(act, 1, self.w_down, y, *lists)
        elem = x.element_size()
        mats = 3 if p.gated else 2
        op_mark(ctx, "experts", nbytes=float(min(pairs, p.num_experts) * mats * p.intermediate_size * p.hidden_size * elem
                                             + pairs * (mats * p.intermediate_size + 2 * p.hidden_size) * elem),
                flops=2.0 * mats * pairs * p.intermediate_size * p.hidden_size)
        shared = None
        if self.shared is not None:
            shared = self.shared.run(x, ctx, "moe.shared")
        out = ws.get("ffn.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        if p.identity > 0:
            kernels.moe_combine(y, weight, shared, out, T, p.top, choice=choice, real_experts=p.num_experts, x=x)
        else:
            kernels.moe_combine(y, weight, shared, out, T, p.top)
        op_mark(ctx, "combine", nbytes=float((pairs + 2 * T) * p.hidden_size * elem))
        return out
