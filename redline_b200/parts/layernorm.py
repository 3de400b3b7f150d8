"""Layer norm with a weight and no bias, y = (x - mean) / sqrt(var + eps) * w with the variance as the
mean of squared deviations, sums in float32; fused with the add to the residual stream like the
RMSNorm part.  ``add_post_norm`` serves blocks that also norm a sublayer's OUTPUT before it is added:
stream += norm_b(delta), then (optionally) the next sublayer's input norm, in one kernel."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels
from .base import Norm, register
from .spec import TensorSpec


@dataclass(frozen=True)
class LayerNormParams:
    size: int
    eps: float


@register("norm", "layernorm")
class LayerNorm(Norm):
    kind = kernels.NORM_LAYER

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.params.size,))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def add_norm(self, residual, delta, out, rows_idx=None, rows=None) -> None:
        if rows_idx is not None and delta is not None:
            # (the kernel norms gathered rows of the stream as it is: what is left to add goes in first)
            kernels.add_residual(residual, delta)
            delta = None
        kernels.sandwich_norm(residual, delta, None, self.weight, out, self.params.eps, self.kind, rows_idx, rows)

    def add_post_norm(self, residual: torch.Tensor, delta: torch.Tensor, next_norm: Optional["LayerNorm"],
                      out: Optional[torch.Tensor], rows: Optional[int] = None) -> bool:
        """residual += self(delta); with ``next_norm`` (a norm of the same kind, eps and weight type) also
        out = next_norm(residual).  False if ``next_norm`` cannot share the kernel (the caller then norms
        by itself)."""
        fuse = (next_norm is not None and out is not None and isinstance(next_norm, LayerNorm)
                and next_norm.kind == self.kind and next_norm.params.eps == self.params.eps
                and next_norm.weight.dtype == self.weight.dtype)
        kernels.sandwich_norm(residual, delta, self.weight, next_norm.weight if fuse else None,
                              out if fuse else None, self.params.eps, self.kind, rows=rows)
        return fuse

    def add_post_cast(self, residual: torch.Tensor, delta: torch.Tensor, out: Optional[torch.Tensor],
                      rows: Optional[int] = None) -> None:
        """residual += self(delta); with ``out`` also out = the new stream rows in out's type, for a sublayer
        that reads the stream itself."""
        kernels.sandwich_norm(residual, delta, self.weight, None, out, self.params.eps, self.kind, rows=rows)


@register("norm", "rmsnorm_sandwich")
class SandwichRMSNorm(LayerNorm):
    """The same interface with an RMS norm (no mean removed), for blocks that norm both sides with it."""

    kind = kernels.NORM_RMS
