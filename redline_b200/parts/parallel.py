"""Two mixers side by side: both read the same input, and the layer's mixer output is
left_scale * left(h) + right_scale * right(h).

Each side stops before its output projection and writes its (scaled) heads into its columns of one
buffer; ONE product with the two output weights laid side by side, [W_o,left | W_o,right], then gives the
sum.  A side is any mixer that has ``inner_size()``, ``forward_inner(x, ctx, cache, state, y, scale)`` and
``out_weight()``.  At most one side keeps a cache and at most one keeps a state; the pair hands the
engine that side's ``cache_spec`` / ``state_spec`` (if both keep a state, a tuple of the two).  Tensor names
of the pair are the sides' own with ``left.`` / ``right.`` in front (``parallel_spec`` builds the ``PartSpec``).

``combine`` "normed": every side keeps its own output projection (with its bias, if it has one, added in
float32 by the kernel that norms), each result is RMS-normed over the model width with a weight of the pair (``left.out`` / ``right.out``), and the
pair's output is left_scale * N(left) + right_scale * N(right) (one kernel, csrc/stream_ops.cu).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, build_part, op_mark, register
from .spec import PartSpec, TensorSpec

SIDES = ("left", "right")


@dataclass(frozen=True)
class ParallelMixersParams:
    hidden_size: int
    left: PartSpec
    right: PartSpec
    left_scale: float = 1.0
    right_scale: float = 1.0
    combine: str = "sum"         # sum: one product over both sides' heads; normed: see above
    eps: float = 1e-6            # of the norms of ``combine`` "normed"


def parallel_spec(hidden_size: int, left: PartSpec, right: PartSpec, left_scale: float = 1.0,
                  right_scale: float = 1.0, combine: str = "sum", eps: float = 1e-6,
                  out_norm_names: Optional[Dict[str, str]] = None) -> PartSpec:
    """``out_norm_names``: checkpoint names of the pair's own ``left.out`` / ``right.out`` (``combine`` "normed")."""
    names = {f"{side}.{k}": v for side, part in zip(SIDES, (left, right)) for k, v in part.names.items()}
    names.update(out_norm_names or {})
    return PartSpec("parallel_mixers", ParallelMixersParams(hidden_size, left, right, left_scale, right_scale,
                                                            combine, eps), names)


@register("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        self.sides = [build_part("mixer", p.left, rt), build_part("mixer", p.right, rt)]
        self.scales = [p.left_scale, p.right_scale]
        for side, m in zip(SIDES, self.sides):
            if not all(hasattr(m, a) for a in ("inner_size", "forward_inner", "out_weight")):
                raise ValueError(f"the {side} mixer '{m.spec.kind}' cannot run beside another one: it has no "
                                 "forward_inner / inner_size / out_weight")
        if sum(m.cache_spec() is not None for m in self.sides) > 1:
            raise ValueError("of two mixers side by side at most one keeps a cache")
        if any(isinstance(m.state_spec(), (tuple, list)) for m in self.sides):
            raise ValueError("a mixer that runs beside another one keeps at most one state")
        if p.combine not in ("sum", "normed"):
            raise ValueError(f"parallel_mixers: combine '{p.combine}' is not known (sum, normed)")
        if p.combine == "sum" and any(getattr(m.params, "out_bias", False) for m in self.sides):
            raise ValueError("parallel_mixers: a bias on a side's output projection needs combine 'normed'")
        self.widths = [m.inner_size() for m in self.sides]
        self.both_states = all(m.state_spec() is not None for m in self.sides)

    # -- what the engine asks of a mixer: answered by the side that has it
    def cache_spec(self):
        return next((m.cache_spec() for m in self.sides if m.cache_spec() is not None), None)

    def state_spec(self):
        if self.both_states:
            return tuple(m.state_spec() for m in self.sides)
        return next((m.state_spec() for m in self.sides if m.state_spec() is not None), None)

    def _state_of(self, i: int, state):
        if self.sides[i].state_spec() is None:
            return None
        return state[i] if self.both_states else state

    def state_in_graphs(self) -> bool:
        return all(m.state_in_graphs() for m in self.sides if m.state_spec() is not None)

    def tiling(self):
        named = {m.tiling() for m in self.sides} - {None}
        if len(named) > 1:
            raise ValueError(f"the two sides want the step's work lists cut in different ways: {sorted(named)}")
        return next(iter(named)) if named else None

    def decode_variant(self, ctx) -> int:
        return self.sides[0].decode_variant(ctx) * 1024 + self.sides[1].decode_variant(ctx)

    # -- tensors
    def tensors(self) -> Dict[str, TensorSpec]:
        t = {f"{side}.{k}": v for side, m in zip(SIDES, self.sides) for k, v in m.tensors().items()}
        if self.params.combine == "normed":
            t.update({f"{side}.out": TensorSpec((self.params.hidden_size,)) for side in SIDES})
        return t

    def fused(self) -> Dict[str, list]:
        return {f"{side}.{k}": [f"{side}.{n}" for n in members]
                for side, m in zip(SIDES, self.sides) for k, members in m.fused().items()}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for side, m in zip(SIDES, self.sides):
            m.load({k[len(side) + 1:]: v for k, v in tensors.items() if k.startswith(side + ".")})
        if self.params.combine == "normed":
            self.w_o = None
            self.out_norms = [tensors["left.out"], tensors["right.out"]]
            return
        ws = [m.out_weight() for m in self.sides]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_o = torch.cat([w.to(dt) for w in ws], dim=1).contiguous()

    def nbytes(self) -> int:
        return sum(m.nbytes() for m in self.sides) + (self.w_o.numel() * self.w_o.element_size() if self.w_o is not None else 0)

    def forward(self, x, ctx, cache, state) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        y = rt.workspace.get("parallel.y", (rt.max_tokens, sum(self.widths)), rt.dtype)[:T]
        normed = p.combine == "normed"
        col = 0
        outs, biases = [], []
        for i, (m, width, scale) in enumerate(zip(self.sides, self.widths, self.scales)):
            heads = y[:, col:col + width]
            m.forward_inner(x, ctx, cache if m.cache_spec() is not None else None, self._state_of(i, state), heads,
                            1.0 if normed else scale)
            col += width
            if normed:         # the side's own output projection
                o = rt.workspace.get(f"parallel.out{i}", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
                linear(heads, m.out_weight(), o)
                op_mark(ctx, "o_proj", m.out_weight(), T)
                outs.append(o)
                biases.append(m.out_bias() if hasattr(m, "out_bias") else None)   # added in the norm's kernel
        out = rt.workspace.get("mixer.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        if normed:
            kernels.pair_norm_mean(outs[0], self.out_norms[0], self.scales[0], outs[1], self.out_norms[1],
                                   self.scales[1], out, p.eps, rows=T, bias_a=biases[0], bias_b=biases[1])
            op_mark(ctx, "pair_norm+mean", nbytes=3.0 * T * p.hidden_size * out.element_size())
            return out
        linear(y, self.w_o, out)
        op_mark(ctx, "o_proj", self.w_o, T)
        return out
