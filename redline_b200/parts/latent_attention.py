"""Causal attention whose keys and values come from one latent vector per token.

Per token the mixer projects its input to queries (per head ``dim`` unrotated and ``rot_dim`` rotated entries)
and to [c' | k_r]: a latent of ``kv_rank`` entries, RMS-normed with a weight into c, and one rotated key part
of ``rot_dim`` entries that all heads share.  Head h's key is [W_uk,h c | k_r], its value W_uv,h c; scores are
scale * q . k over every earlier token, ordinary softmax.  Only [c | k_r] is cached (one row per token, one
"key head" for all query heads), and the keys and values are never formed:

    q_n . (W_uk,h c_j) = (W_uk,h^T q_n) . c_j          sum_j p_j W_uv,h c_j = W_uv,h (sum_j p_j c_j)

so the attention kernels (those of ``maps_attention``: csrc/attention_maps.cu) run over the cached rows with the
query [W_uk,h^T q_n | q_r] and the row's first ``kv_rank`` entries as the value, and W_uv,h is applied to what
they return.  The two per-head products and the kernel between projection and cache (norm, rotation, cache
write) are csrc/latent.cu.  The rotation is a ``rope_halves`` position encoding over the first ``rot_dims``
entries of the rotated part.  Norm, rotation, scores and softmax are float32 in both engine types.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import LayerCache, Mixer, build_part, op_mark, register
from .spec import CacheSpec, CacheTensor, PartSpec, TensorSpec


@dataclass(frozen=True)
class LatentAttentionParams:
    hidden_size: int
    num_heads: int
    dim: int                     # unrotated entries of a head's query and key
    rot_dim: int                 # rotated entries (0: none); the key's are one vector for all heads
    vdim: int                    # size of a head's value
    kv_rank: int                 # size of the cached latent
    scale: float
    eps: float = 1e-6            # of the latent's RMS norm
    position: Optional[PartSpec] = None      # a ``rope_halves`` encoding of the rotated part (needed if rot_dim > 0)


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        self.key_size = p.kv_rank + p.rot_dim          # a cached row, and a head's query for the kernels
        if min(p.num_heads, p.dim, p.vdim, p.kv_rank) <= 0 or p.rot_dim < 0:
            raise ValueError("latent_attention: heads, dim, vdim and kv_rank must be positive")
        if self.key_size > kernels.MAPS_MAX_DIM or p.kv_rank > kernels.MAPS_MAX_VDIM:
            raise ValueError(f"latent_attention: kv_rank + rot_dim is {self.key_size}; the attention kernels take "
                             f"rows of up to {kernels.MAPS_MAX_DIM} entries of which {kernels.MAPS_MAX_VDIM} are the latent")
        self.cos = self.sin = None
        self.rot_dims = 0
        if p.rot_dim > 0:
            if p.position is None:
                raise ValueError("latent_attention: a rotated part needs a position encoding")
            pos = build_part("position", p.position, rt)
            if getattr(pos, "pairing", None) != "halves" or pos.rotary_tables() is None:
                raise ValueError("latent_attention rotates entry i with entry i + half (rope_halves)")
            self.cos, self.sin = pos.rotary_tables()
            self.rot_dims = 2 * self.cos.shape[1]
            if self.rot_dims > p.rot_dim:
                raise ValueError(f"a rotation of {self.rot_dims} entries does not fit a rotated part of {p.rot_dim}")
        self.q_head = p.dim + p.rot_dim
        self.q_size = p.num_heads * self.q_head
        self.proj_size = self.q_size + self.key_size
        self.qa_size = p.num_heads * self.key_size
        self.lat_size = p.num_heads * p.kv_rank
        self.out_size = p.num_heads * p.vdim

    def cache_spec(self) -> CacheSpec:
        return CacheSpec("full", (CacheTensor("k", (1, self.key_size)),))

    def tiling(self):
        return kernels.PREFILL_TILE_ROWS, kernels.DECODE_PARTITION

    def tensors(self) -> Dict[str, TensorSpec]:
        p = self.params
        return {
            "q": TensorSpec((self.q_size, p.hidden_size)),
            "dkv": TensorSpec((self.key_size, p.hidden_size)),
            "dkv_norm": TensorSpec((p.kv_rank,)),
            "uk": TensorSpec((p.num_heads * p.dim, p.kv_rank)),
            "uv": TensorSpec((self.out_size, p.kv_rank)),
            "o": TensorSpec((p.hidden_size, self.out_size)),
        }

    def fused(self) -> Dict[str, list]:
        return {"q_dkv": ["q", "dkv"]}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.params
        if "q_dkv" in tensors:
            self.w_proj = tensors["q_dkv"]
        else:
            ws = [tensors["q"], tensors["dkv"]]
            dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
            self.w_proj = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.w_norm = tensors["dkv_norm"]
        # W_uk,h^T for every head: [heads, kv_rank, dim], the matrix the unrotated query part is multiplied by
        self.w_uk_t = tensors["uk"].view(p.num_heads, p.dim, p.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"].view(p.num_heads, p.vdim, p.kv_rank).contiguous()
        self.w_o = tensors["o"]

    def nbytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_proj, self.w_uk_t, self.w_uv, self.w_o))

    def forward(self, x, ctx, cache: Optional[LayerCache], state=None) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        ws = rt.workspace
        proj = ws.get("latent.proj", (rt.max_tokens, self.proj_size), rt.dtype)[:T]
        linear(x, self.w_proj, proj)
        op_mark(ctx, "q_dkv_proj", self.w_proj, T)
        g = ctx.groups[cache.group]
        k_cache = cache.tensors["k"]
        qa = ws.get("latent.qa", (rt.max_tokens, self.qa_size), rt.dtype)[:T]
        kernels.latent_prep(proj, ctx.positions, T, p.num_heads, p.dim, p.rot_dim, p.kv_rank, self.rot_dims, self.w_norm,
                            p.eps, self.cos, self.sin, qa, g.slots if cache.write else None, k_cache, rt.page_size,
                            ctx.status)
        elem = proj.element_size()
        op_mark(ctx, "latent_norm+rotate+write", nbytes=float(T * (self.proj_size + 2 * self.key_size
                                                                   + p.num_heads * p.rot_dim) * elem))
        kernels.head_linear(proj, 0, self.q_head, self.w_uk_t, qa, 0, self.key_size, tokens=T)
        op_mark(ctx, "q_absorb", nbytes=float(T * p.num_heads * (p.dim + p.kv_rank) * elem + self.w_uk_t.numel() * elem),
                flops=2.0 * T * p.num_heads * p.dim * p.kv_rank)
        lat = ws.get("latent.out", (rt.max_tokens, self.lat_size), rt.dtype)[:T]
        v_stride = self.key_size if p.rot_dim > 0 else 0
        common = (p.num_heads, 1, self.key_size, p.kv_rank, 1, rt.page_size, 0, 0, p.scale, 0.0, 0.0, 1.0, p.eps, False)
        if ctx.num_decode > 0:
            rows = ctx.max_items * p.num_heads * ctx.parts_capacity
            part_o = ws.get("mattn.part_o", (rows * p.kv_rank,), torch.float32)
            part_ml = ws.get("mattn.part_ml", (rows * 2,), torch.float32)
            kernels.maps_attn_decode(qa, self.qa_size, k_cache, k_cache, g.block_table, ctx.decode_info, part_o, part_ml,
                                     ctx.decode_parts, lat, ctx.num_decode, *common, v_stride=v_stride)
            self._mark(ctx, "attention_decode", "decode")
        if ctx.num_tiles > 0:
            kernels.maps_attn_prefill(qa, self.qa_size, k_cache, k_cache, g.block_table, ctx.tile_seq, ctx.tile_tok,
                                      ctx.tile_rows, ctx.positions, lat, ctx.num_tiles, kernels.PREFILL_TILE_ROWS,
                                      *common, v_stride=v_stride)
            self._mark(ctx, "attention_prefill", "prefill")
        heads_v = ws.get("latent.values", (rt.max_tokens, self.out_size), rt.dtype)[:T]
        kernels.head_linear(lat, 0, p.kv_rank, self.w_uv, heads_v, 0, p.vdim, tokens=T)
        op_mark(ctx, "v_up", nbytes=float(T * p.num_heads * (p.vdim + p.kv_rank) * elem + self.w_uv.numel() * elem),
                flops=2.0 * T * p.num_heads * p.vdim * p.kv_rank)
        out = ws.get("mixer.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        linear(heads_v, self.w_o, out)
        op_mark(ctx, "o_proj", self.w_o, T)
        return out

    def _mark(self, ctx, op: str, which: str) -> None:
        if ctx.profiler is None:
            return
        from ..engine.profiler import attention_work
        p = self.params
        elem = 2 if self.rt.dtype == torch.bfloat16 else 4
        nbytes, flops = attention_work(ctx.host, p.num_heads, 1, (self.key_size + p.kv_rank) // 2, 0, elem)[which]
        ctx.profiler.mark(op, nbytes, flops)
