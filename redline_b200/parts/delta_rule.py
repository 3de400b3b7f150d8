"""The gated delta rule with one decay per key channel ("channel_delta").

q = W_q h and k = W_k h (qk_heads x dim), v = W_v h (heads x vdim); head h uses the q and k of head
h // (heads / qk_heads).  Each of q, k and v passes a short causal convolution over time per channel and an
activation (SiLU); q and k are then made unit vectors per head, x / sqrt(sum x^2 + unit_floor), and q is
multiplied by ``q_scale`` (dim^(-1/2) unless given).  beta = sigmoid(W_b h), one per head; one decay per head
and key channel, a = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 h) + dt_bias)).  Per head, in this order,

    S <- diag(a) S;   d = beta (v - S^T k);   S <- S + k d^T;   o = S^T q

so the read-out sees the token's own write.  Every head's o is RMS-normed over vdim with one weight of vdim
entries shared by the heads, multiplied by sigmoid(W_g2 (W_g1 h)), and projected by W_o.

The per-request state is S (float32 [heads, dim, vdim]) and the convolution's last taps - 1 inputs
(float32): two pools.  q, k, v and the two low-rank inner projections [a1 | g1] come from one fused product;
the products for beta and the decays have float32 results; unit vectors, beta, decays, the recurrence and
the norm are float32 (csrc/delta_rule.cu, csrc/stream_ops.cu).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, op_mark, register
from .spec import StateSpec, TensorSpec


@dataclass(frozen=True)
class GatedDeltaParams:
    hidden_size: int
    num_heads: int
    num_qk_heads: int
    dim: int
    vdim: int
    conv_taps: int
    decay_rank: int                    # inner size of W_a2 W_a1
    gate_rank: int                     # inner size of W_g2 W_g1
    eps: float = 1e-6                  # of the heads' norm
    unit_floor: float = 1e-6           # under the root of the unit vectors
    q_scale: Optional[float] = None    # None: dim^(-1/2)
    activation: str = "silu"           # behind the convolutions


@register("mixer", "gated_delta")
class GatedDelta(Mixer):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        if p.num_heads % p.num_qk_heads != 0:
            raise ValueError(f"gated_delta: heads {p.num_heads} is no multiple of the q/k heads {p.num_qk_heads}")
        if not 1 <= p.dim <= 256:
            raise ValueError(f"the delta rule's kernels take key sizes up to 256; got {p.dim}")
        if not 1 <= p.conv_taps <= kernels.MAX_CONV_TAPS:
            raise ValueError(f"a short convolution has 1 to {kernels.MAX_CONV_TAPS} taps; got {p.conv_taps}")
        if p.activation not in ("silu", "none"):
            raise ValueError(f"gated_delta: activation '{p.activation}' behind the convolution is not built (silu, none)")
        self.qk_size = p.num_qk_heads * p.dim
        self.v_size = p.num_heads * p.vdim
        self.conv_size = 2 * self.qk_size + self.v_size
        self.proj_size = self.conv_size + p.decay_rank + p.gate_rank
        self.q_scale = p.q_scale if p.q_scale is not None else p.dim ** -0.5
        self.act = kernels.ACT_SILU if p.activation == "silu" else kernels.ACT_NONE

    def state_spec(self):
        p = self.params
        s = StateSpec((p.num_heads * p.dim * p.vdim,), "float32")
        if p.conv_taps > 1:
            return (s, StateSpec(((p.conv_taps - 1) * self.conv_size,), "float32"))
        return s

    def state_in_graphs(self) -> bool:
        return True

    def tensors(self) -> Dict[str, TensorSpec]:
        p = self.params
        W = p.hidden_size
        return {
            "q": TensorSpec((self.qk_size, W)), "k": TensorSpec((self.qk_size, W)), "v": TensorSpec((self.v_size, W)),
            "q_conv": TensorSpec((self.qk_size, p.conv_taps)), "k_conv": TensorSpec((self.qk_size, p.conv_taps)),
            "v_conv": TensorSpec((self.v_size, p.conv_taps)),
            "b": TensorSpec((p.num_heads, W)), "A_log": TensorSpec((p.num_heads,)), "norm": TensorSpec((p.vdim,)),
            "a1": TensorSpec((p.decay_rank, W)), "a2": TensorSpec((p.num_heads * p.dim, p.decay_rank)),
            "dt_bias": TensorSpec((p.num_heads * p.dim,)),
            "g1": TensorSpec((p.gate_rank, W)), "g2": TensorSpec((self.v_size, p.gate_rank)),
            "o": TensorSpec((W, self.v_size)),
        }

    def fused(self) -> Dict[str, list]:
        return {"qkvag": ["q", "k", "v", "a1", "g1"], "qkv_conv": ["q_conv", "k_conv", "v_conv"]}

    @staticmethod
    def _joined(tensors, fused_name, members):
        if fused_name in tensors:
            return tensors[fused_name]
        ws = [tensors[n] for n in members]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        return torch.cat([w.to(dt) for w in ws], dim=0).contiguous()

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_in = self._joined(tensors, "qkvag", ["q", "k", "v", "a1", "g1"])
        self.w_conv = self._joined(tensors, "qkv_conv", ["q_conv", "k_conv", "v_conv"])
        self.w_b, self.w_a2, self.w_g2, self.w_o = tensors["b"], tensors["a2"], tensors["g2"], tensors["o"]
        self.w_norm = tensors["norm"]
        self.a_log = tensors["A_log"].float().contiguous()
        self.dt_bias = tensors["dt_bias"].float().contiguous()

    def nbytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_b, self.w_a2, self.w_g2, self.w_o))

    def inner_size(self) -> int:
        return self.v_size

    def out_weight(self) -> torch.Tensor:
        return self.w_o

    def forward(self, x, ctx, cache, state) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        y = rt.workspace.get("delta.y", (rt.max_tokens, self.v_size), rt.dtype)[:T]
        self.forward_inner(x, ctx, cache, state, y)
        out = rt.workspace.get("mixer.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        linear(y, self.w_o, out)
        op_mark(ctx, "o_proj", self.w_o, T)
        return out

    def forward_inner(self, x, ctx, cache, state, y: torch.Tensor, scale: float = 1.0) -> None:
        """Everything before the output projection: y [T, heads * vdim] <- the normed, gated heads."""
        if scale != 1.0:
            raise ValueError("gated_delta: a scale on the heads is not built")
        p, rt = self.params, self.rt
        T = ctx.T
        ws = rt.workspace
        s_state, conv_state = state if isinstance(state, (tuple, list)) else (state, None)
        proj = ws.get("delta.proj", (rt.max_tokens, self.proj_size), rt.dtype)[:T]
        linear(x, self.w_in, proj)
        op_mark(ctx, "qkvag_proj", self.w_in, T)
        conv = ws.get("delta.conv", (rt.max_tokens, self.conv_size), rt.dtype)[:T]
        if conv_state is None:           # one tap: a weight per channel and the activation
            conv_state = ws.get("delta.no_state", (rt.max_seqs + 1, 1), torch.float32)
        kernels.short_conv(proj, 0, self.w_conv, None, conv, 0, self.act, ctx.seq_of_token, ctx.state_slot,
                           conv_state, T, single=ctx.num_decode == ctx.S == T)
        op_mark(ctx, "conv+act", nbytes=2.0 * T * self.conv_size * proj.element_size())
        H, D = p.num_heads, p.dim
        zb = ws.get("delta.zb", (rt.max_tokens, H), torch.float32)[:T]
        linear(x, self.w_b, zb)
        op_mark(ctx, "beta_proj", self.w_b, T)
        za = ws.get("delta.za", (rt.max_tokens, H * D), torch.float32)[:T]
        linear(proj[:, self.conv_size:self.conv_size + p.decay_rank], self.w_a2, za)
        op_mark(ctx, "decay_proj", self.w_a2, T)
        gate = ws.get("delta.gate", (rt.max_tokens, self.v_size), rt.dtype)[:T]
        linear(proj[:, self.conv_size + p.decay_rank:], self.w_g2, gate)
        op_mark(ctx, "gate_proj", self.w_g2, T)
        q = ws.get("delta.q", (rt.max_tokens, self.qk_size), torch.float32)[:T]
        k = ws.get("delta.k", (rt.max_tokens, self.qk_size), torch.float32)[:T]
        beta = ws.get("delta.beta", (rt.max_tokens, H), torch.float32)[:T]
        decay = ws.get("delta.decay", (rt.max_tokens, H * D), torch.float32)[:T]
        kernels.delta_prep(conv, 0, self.qk_size, p.num_qk_heads, H, D, self.q_scale, p.unit_floor, zb, za,
                           self.dt_bias, self.a_log, q, k, beta, decay, T)
        op_mark(ctx, "unit_qk+beta+decay", nbytes=T * (2.0 * self.qk_size * (4 + conv.element_size()) + 8.0 * H * D))
        o = ws.get("delta.o", (rt.max_tokens, self.v_size), torch.float32)[:T]
        kernels.delta_rule(q, k, conv[:, 2 * self.qk_size:], beta, decay, ctx.seq_of_token, ctx.state_slot, s_state, o,
                           T, ctx.S, H, p.num_qk_heads, D, p.vdim)
        op_mark(ctx, "delta_rule", nbytes=T * (8.0 * self.qk_size + 4.0 * H * D + self.v_size * (4.0 + conv.element_size())),
                flops=6.0 * T * H * D * p.vdim)
        kernels.head_gated_norm(o, gate, self.w_norm, y, T, H, p.vdim, p.eps, dim=D)
        op_mark(ctx, "head_norm+gate", nbytes=T * self.v_size * (4.0 + 2.0 * y.element_size()))
