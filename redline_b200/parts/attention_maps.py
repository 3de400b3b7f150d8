"""Grouped-query causal attention with score maps over the paged cache.

Every head has ``maps`` score maps (queries and keys of ``dim`` each) over the same values of ``vdim``;
two maps are combined as a difference, o = a1 - lambda * a2 (differential attention), one is ordinary
attention.  Scores may be capped, s <- cap * tanh(s / cap); the mask is causal with a sliding window that
keeps the first ``keep_first`` tokens of the sequence visible; a head's output may be divided by its root
mean square and multiplied by ``post_scale``.  q, k and v come from one fused projection [q | k | v] with
optional biases; a position encoding, if the layer has one, is applied to q and k before the cache write.

Further options, each with its constants as parameters: queries and keys RMS-normed with a weight before the
rotation, per head (``head_norm`` "each": one weight of ``dim`` entries for all heads) or over the whole
projection ("whole": weights of heads * dim entries); a rotation of the first entries of every head in
neighbouring pairs (a ``rope_pairs`` position encoding); a sink, one learned number per head that joins the
softmax's denominator without a key or a value; an output gate sigmoid(W_g h) per head or per entry, applied
before the output projection (W_g is then the fourth block of the fused projection); and a blend of the
values with those that an earlier layer of the model computed for the same token (``value_mix`` "keep" in
the layer that provides them, "blend" in those that use them: v <- (1 - lam) v + lam v_first; what is blended
is what is cached).  ``conv_taps``: a short causal convolution over time on every channel of q, k and v
directly behind the projection (and its biases), whose last inputs are the mixer's per-request state;
``out_bias``: a bias on the output projection; a ``rope_halves`` encoding pairs entry i with entry i + half.
``values_are_keys``: there is no value projection, a key head's vector is also its value (one map, vdim = dim;
only the keys are cached and the kernels read them twice); ``distance_slopes``: one number per head, times the
distance between query and key, is taken off every score; ``sink_value``: a constant in place of the learned
sink (0.0 adds a one to every denominator).

The cache holds keys [kv_heads * maps, dim] and values [kv_heads, vdim] per token (a window group that
keeps its first pages); sequences that bring one token go to the partitioned decode kernel, longer
portions to the tiled kernel (csrc/attention_maps.cu); scores, softmax, combination and norm in float32.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import LayerCache, Mixer, build_part, op_mark, register
from .spec import CacheSpec, CacheTensor, PartSpec, StateSpec, TensorSpec


@dataclass(frozen=True)
class MapsAttentionParams:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    dim: int                     # size of a query / key of one map
    vdim: int                    # size of a value
    maps: int = 1                # 2: differential attention
    bias: bool = False           # q, k, v projections have biases
    window: int = 0              # 0: every earlier key
    keep_first: int = 0          # the first tokens stay visible behind the window
    scale: Optional[float] = None
    softcap: float = 0.0         # 0: scores are not capped
    diff: float = 0.0            # maps = 2: lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
    unit_norm: bool = False      # divide a head's output by its root mean square
    post_scale: float = 1.0      # and multiply it by this
    eps: float = 1e-6
    position: Optional[PartSpec] = None
    head_norm: str = "none"      # none | each | whole: RMS norm of q and k with a weight, before the rotation
    sink: bool = False           # a learned number per head in the softmax's denominator (one map)
    gate: str = "none"           # none | head | entry: the output times sigmoid(W_g h)
    value_mix: str = "none"      # none | keep | blend (see above)
    value_mix_key: str = "v"     # layers that share values name the same key
    conv_taps: int = 0           # > 0: a causal convolution over time on every channel of q, k and v, behind the projection
    out_bias: bool = False       # the output projection has a bias
    values_are_keys: bool = False            # no W_v: v = k as projected; only k is cached
    distance_slopes: Optional[tuple] = None  # per head: s_ij <- s_ij - slope_h * (i - j)
    sink_value: Optional[float] = None       # a constant sink for every head (with ``sink`` False)


@register("mixer", "maps_attention")
class MapsAttention(Mixer):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        if p.num_heads % p.num_kv_heads != 0:
            raise ValueError(f"num_heads {p.num_heads} is no multiple of num_kv_heads {p.num_kv_heads}")
        if p.maps not in (1, 2):
            raise ValueError(f"attention with {p.maps} score maps is not supported (1 or 2)")
        if not (1 <= p.dim <= kernels.MAPS_MAX_DIM and 1 <= p.vdim <= kernels.MAPS_MAX_VDIM):
            raise ValueError(f"attention_maps kernels take key sizes up to {kernels.MAPS_MAX_DIM} and value sizes up to "
                             f"{kernels.MAPS_MAX_VDIM}; got dim={p.dim}, vdim={p.vdim}")
        self.position = build_part("position", p.position, rt) if p.position is not None else None
        self.rotary = None           # (cos, sin) of an encoding whose pairs the head kernel rotates
        self.halves = False          # ... entry i with entry i + half instead of its neighbour
        if self.position is not None and self.position.rotary_tables() is not None:
            if getattr(self.position, "pairing", None) not in ("neighbours", "halves"):
                raise ValueError("maps_attention rotates the first entries of a head in neighbouring pairs "
                                 "(rope_pairs) or entry i with entry i + half (rope_halves), or applies a position "
                                 "encoding through its apply()")
            self.halves = self.position.pairing == "halves"
            self.rotary = self.position.rotary_tables()
            if 2 * self.rotary[0].shape[1] > p.dim:
                raise ValueError(f"a rotation of {2 * self.rotary[0].shape[1]} entries does not fit heads of {p.dim}")
        if p.head_norm not in ("none", "each", "whole") or p.gate not in ("none", "head", "entry") \
                or p.value_mix not in ("none", "keep", "blend"):
            raise ValueError(f"maps_attention: head_norm '{p.head_norm}', gate '{p.gate}' or value_mix "
                             f"'{p.value_mix}' is not known")
        if (p.sink or p.sink_value is not None) and p.maps != 1:
            raise ValueError("a sink goes with one score map")
        if p.sink and p.sink_value is not None:
            raise ValueError("a sink is learned or a constant, not both")
        if p.distance_slopes is not None and len(p.distance_slopes) != p.num_heads:
            raise ValueError(f"{len(p.distance_slopes)} distance slopes for {p.num_heads} heads")
        if p.values_are_keys and (p.maps != 1 or p.vdim != p.dim or p.bias or p.conv_taps > 0 or p.position is not None
                                  or p.head_norm != "none" or p.value_mix != "none"):
            raise ValueError("values_are_keys goes with one map, vdim = dim, and no bias, convolution, position "
                             "encoding, head norm or value blend")
        self.scale = p.scale if p.scale is not None else 1.0 / math.sqrt(p.dim)
        self.q_size = p.num_heads * p.maps * p.dim
        self.k_size = p.num_kv_heads * p.maps * p.dim
        self.v_size = 0 if p.values_are_keys else p.num_kv_heads * p.vdim
        self.qkv_size = self.q_size + self.k_size + self.v_size
        self.out_size = p.num_heads * p.vdim
        self.gate_size = {"none": 0, "head": p.num_heads, "entry": self.out_size}[p.gate]
        self.gate_mode = {"none": 0, "head": 1, "entry": 2}[p.gate]
        self.proj_size = self.qkv_size + self.gate_size
        self.lam = 0.0
        self.mix = 0.0
        if p.conv_taps < 0 or p.conv_taps > kernels.MAX_CONV_TAPS:
            raise ValueError(f"a short convolution has up to {kernels.MAX_CONV_TAPS} taps; got {p.conv_taps}")

    def state_spec(self):
        """The convolution's last taps - 1 inputs of every q, k and v channel."""
        p = self.params
        if p.conv_taps > 1:
            return StateSpec(((p.conv_taps - 1) * self.qkv_size,), "float32")
        return None

    def state_in_graphs(self) -> bool:
        return True

    def cache_spec(self) -> CacheSpec:
        p = self.params
        tensors = (CacheTensor("k", (p.num_kv_heads * p.maps, p.dim)),)
        if not p.values_are_keys:
            tensors += (CacheTensor("v", (p.num_kv_heads, p.vdim)),)
        if p.window > 0:
            return CacheSpec("window", tensors, p.window, p.keep_first)
        return CacheSpec("full", tensors)

    def tiling(self):
        return kernels.PREFILL_TILE_ROWS, kernels.DECODE_PARTITION

    def tensors(self) -> Dict[str, TensorSpec]:
        p = self.params
        t = {
            "q": TensorSpec((self.q_size, p.hidden_size)),
            "k": TensorSpec((self.k_size, p.hidden_size)),
            "v": TensorSpec((self.v_size, p.hidden_size)),
            "o": TensorSpec((p.hidden_size, self.out_size)),
            "q_bias": TensorSpec((self.q_size,), optional=not p.bias),
            "k_bias": TensorSpec((self.k_size,), optional=not p.bias),
            "v_bias": TensorSpec((self.v_size,), optional=not p.bias),
        }
        if p.values_are_keys:
            del t["v"], t["v_bias"]
        if p.maps == 2:
            t.update({n: TensorSpec((p.dim,)) for n in ("lq1", "lk1", "lq2", "lk2")})
        if p.head_norm != "none":
            whole = p.head_norm == "whole"
            t["q_norm"] = TensorSpec((self.q_size if whole else p.dim,))
            t["k_norm"] = TensorSpec((self.k_size if whole else p.dim,))
        if p.sink:
            t["sink"] = TensorSpec((p.num_heads,))
        if p.gate != "none":
            t["g"] = TensorSpec((self.gate_size, p.hidden_size))
        if p.value_mix != "none":            # (the layer that provides the values may have the number too: unused)
            t["vmix"] = TensorSpec((), optional=p.value_mix == "keep")
        if p.conv_taps > 0:
            t.update({"q_conv": TensorSpec((self.q_size, p.conv_taps)), "k_conv": TensorSpec((self.k_size, p.conv_taps)),
                      "v_conv": TensorSpec((self.v_size, p.conv_taps))})
        if p.out_bias:
            t["o_bias"] = TensorSpec((p.hidden_size,))
        return t

    def fused(self) -> Dict[str, list]:
        out = {"qkv": ["q", "k"] + ([] if self.params.values_are_keys else ["v"])
               + (["g"] if self.params.gate != "none" else [])}
        if self.params.conv_taps > 0:
            out["qkv_conv"] = ["q_conv", "k_conv", "v_conv"]
        return out

    # -- what a mixer that runs beside another one under a common output projection is asked for
    def inner_size(self) -> int:
        return self.out_size

    def out_weight(self) -> torch.Tensor:
        return self.w_o

    def out_bias(self) -> Optional[torch.Tensor]:
        return self.b_o

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.params
        if "qkv" in tensors:
            self.w_qkv = tensors["qkv"]
        else:
            ws = [tensors[n] for n in self.fused()["qkv"]]
            dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
            self.w_qkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.w_o = tensors["o"]
        self.b_o = tensors["o_bias"].float().contiguous() if p.out_bias else None
        self.w_conv = None
        if p.conv_taps > 0:
            self.w_conv = tensors["qkv_conv"] if "qkv_conv" in tensors else \
                torch.cat([tensors[n] for n in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.b_qkv = None
        if p.bias:
            self.b_qkv = torch.cat([tensors[n].float() for n in ("q_bias", "k_bias", "v_bias")]).contiguous()
        if p.maps == 2:
            # one number for the layer, in float32 like everything around the scores
            lq1, lk1, lq2, lk2 = (tensors[n].float() for n in ("lq1", "lk1", "lq2", "lk2"))
            self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + p.diff)
        self.w_qnorm, self.w_knorm = tensors.get("q_norm"), tensors.get("k_norm")
        self.sink = tensors["sink"].float().contiguous() if p.sink else None
        if p.sink_value is not None:
            self.sink = torch.full((p.num_heads,), float(p.sink_value), dtype=torch.float32, device=self.rt.device)
        self.slopes = None
        if p.distance_slopes is not None:
            self.slopes = torch.tensor([float(x) for x in p.distance_slopes], dtype=torch.float32, device=self.rt.device)
        self.mix = float(tensors["vmix"].float()) if p.value_mix == "blend" else 0.0
        self.norm_mode = {"none": kernels.HEAD_NORM_NONE, "each": kernels.HEAD_NORM_EACH,
                          "whole": kernels.HEAD_NORM_WHOLE}[p.head_norm]
        self.mix_mode = {"none": kernels.VALUE_MIX_NONE, "keep": kernels.VALUE_MIX_KEEP,
                         "blend": kernels.VALUE_MIX_BLEND}[p.value_mix]

    def nbytes(self) -> int:
        return self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()

    def forward(self, x, ctx, cache: Optional[LayerCache], state=None) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        attn = rt.workspace.get("mattn.out", (rt.max_tokens, self.out_size), rt.dtype)[:T]
        self.forward_inner(x, ctx, cache, state, attn)
        out = rt.workspace.get("mixer.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        linear(attn, self.w_o, out)
        if self.b_o is not None:
            kernels.bias_act(out, self.b_o, kernels.ACT_NONE)
        op_mark(ctx, "o_proj", self.w_o, T)
        return out

    def forward_inner(self, x, ctx, cache: Optional[LayerCache], state, attn: torch.Tensor, scale: float = 1.0) -> None:
        """Everything before the output projection: attn [T, heads * vdim] (possibly a view of columns of a
        wider buffer) <- scale * the heads' gated outputs."""
        p, rt = self.params, self.rt
        T = ctx.T
        ws = rt.workspace
        qkv = ws.get("mattn.qkv", (rt.max_tokens, self.proj_size), rt.dtype)[:T]
        linear(x, self.w_qkv, qkv)
        gate_buf = qkv                     # where the gate's columns lie
        if self.w_conv is not None:
            # (the biases are added on the way into the convolution, whose state keeps the biased inputs)
            conv = ws.get("mattn.qkv_conv", (rt.max_tokens, self.proj_size), rt.dtype)[:T]
            if state is None:          # one tap: a weight per channel, nothing carried
                state = ws.get("mattn.no_state", (rt.max_seqs + 1, 1), torch.float32)
            kernels.short_conv(qkv, 0, self.w_conv, self.b_qkv, conv, 0, kernels.ACT_NONE, ctx.seq_of_token,
                               ctx.state_slot, state, T, single=ctx.num_decode == ctx.S == T)
            qkv = conv
        elif self.b_qkv is not None:
            kernels.bias_act(qkv, self.b_qkv, kernels.ACT_NONE, cols=self.qkv_size)
        op_mark(ctx, "qkv_proj", self.w_qkv, T)
        if self.position is not None and self.rotary is None:
            self.position.apply(qkv, p.num_heads * p.maps, p.num_kv_heads * p.maps, p.dim, ctx)
        if self.rotary is not None or self.norm_mode != kernels.HEAD_NORM_NONE or self.mix_mode != kernels.VALUE_MIX_NONE:
            v_first = None
            if self.mix_mode != kernels.VALUE_MIX_NONE:
                # (the layers run one after another within a step: the buffer holds this step's tokens)
                v_first = ws.get("mattn.v_first." + p.value_mix_key, (rt.max_tokens, self.v_size), rt.dtype)
            cos, sin = self.rotary if self.rotary is not None else (None, None)
            g = ctx.groups[cache.group]
            # (the same kernel puts the finished keys and values into the cache)
            kernels.head_prep(qkv, ctx.positions, T, 0, p.num_heads * p.maps, self.q_size, p.num_kv_heads * p.maps, p.dim,
                              ctx.status, self.w_qnorm, self.w_knorm, self.norm_mode, p.eps, cos, sin,
                              self.q_size + self.k_size, self.v_size, v_first, self.mix_mode, self.mix,
                              g.slots if cache.write else None, cache.tensors["k"], cache.tensors["v"], rt.page_size,
                              halves=self.rotary is not None and self.halves)
            op_mark(ctx, "qk_norm+rotate+kv_write", nbytes=(2.0 * self.qkv_size + self.k_size + self.v_size) * T * qkv.element_size())
            stored = True
        else:
            stored = False
        g = ctx.groups[cache.group]
        k_cache = cache.tensors["k"]
        v_cache = k_cache if p.values_are_keys else cache.tensors["v"]
        if cache.write and not stored:
            kernels.cache_store(qkv, self.q_size, p.num_kv_heads * p.maps, p.dim, g.slots, k_cache, rt.page_size,
                                ctx.status, tokens=T)
            if not p.values_are_keys:
                kernels.cache_store(qkv, self.q_size + self.k_size, p.num_kv_heads, p.vdim, g.slots, v_cache,
                                    rt.page_size, ctx.status, tokens=T)
            op_mark(ctx, "kv_write", nbytes=2.0 * T * (self.k_size + self.v_size) * qkv.element_size())
        gate = gate_buf[:, self.qkv_size:] if self.gate_mode else None
        common = (p.num_heads, p.num_kv_heads, p.dim, p.vdim, p.maps, rt.page_size, p.window, p.keep_first,
                  self.scale, p.softcap, self.lam, p.post_scale * scale, p.eps, p.unit_norm, self.sink, gate,
                  self.gate_mode)
        if ctx.num_decode > 0:
            rows = ctx.max_items * p.num_heads * p.maps * ctx.parts_capacity
            part_o = ws.get("mattn.part_o", (rows * p.vdim,), torch.float32)
            part_ml = ws.get("mattn.part_ml", (rows * 2,), torch.float32)
            kernels.maps_attn_decode(qkv, self.proj_size, k_cache, v_cache, g.block_table, ctx.decode_info, part_o,
                                     part_ml, ctx.decode_parts, attn, ctx.num_decode, *common, slopes=self.slopes)
            self._mark(ctx, "attention_decode", "decode")
        if ctx.num_tiles > 0:
            kernels.maps_attn_prefill(qkv, self.proj_size, k_cache, v_cache, g.block_table, ctx.tile_seq, ctx.tile_tok,
                                      ctx.tile_rows, ctx.positions, attn, ctx.num_tiles, kernels.PREFILL_TILE_ROWS,
                                      *common, slopes=self.slopes)
            self._mark(ctx, "attention_prefill", "prefill")

    def _mark(self, ctx, op: str, which: str) -> None:
        if ctx.profiler is None:
            return
        from ..engine.profiler import attention_work
        p = self.params
        elem = 2 if self.rt.dtype == torch.bfloat16 else 4
        window = p.window + p.keep_first if p.window > 0 else 0
        nbytes, flops = attention_work(ctx.host, p.num_heads * p.maps, p.num_kv_heads * p.maps, (p.dim + p.vdim) // 2,
                                       window, elem)[which]
        ctx.profiler.mark(op, nbytes, flops)
