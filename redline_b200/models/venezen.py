"""``Venezen`` laid out as parts: a token embedding multiplied by a constant; pre-norm blocks with layer norms
(a weight, no bias) whose mixer is attention over a cached latent (``latent_attention``: keys and values of all
heads from one latent vector per token, a rotated key part shared by the heads) or grouped attention over a
sliding window whose keys are its values (``maps_attention`` with ``values_are_keys``, a distance bias per head
and a constant sink of 0, which adds a one to every softmax denominator); a dense SiLU-gated feed-forward with
biases, routed experts with clamped gate and up (softmax router over experts and identity experts, a choice
corrected per router output, renormalized and scaled weights, a shared expert), or none; a final layer norm and
the embedding table as the head.  A run of layers may be repeated on the same tensors, every pass with caches
of its own; before every pass but the first the embedding output is added to the stream
(``LayerCall.add_embedding``).  Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``.
"""

from __future__ import annotations

import math
from typing import Iterator, Tuple

import torch

from ..config.model_config import VenezenConfig
from ..config.registry import Architecture, register_architecture
from ..parts.attention_maps import MapsAttentionParams
from ..parts.embedding import EmbeddingParams, HeadParams
from ..parts.latent_attention import LatentAttentionParams
from ..parts.layernorm import LayerNormParams
from ..parts.mlp import GatedMLPParams
from ..parts.moe import RoutedExpertsParams
from ..parts.rope import RotaryHalvesParams
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

# what the design fixes
SWISH_SLOPE = 1.702            # an expert's gate: g * sigmoid(1.702 g)
WEIGHT_FLOOR = 1e-20           # joins the sum the chosen experts' scores are divided by
SINK_SCORE = 0.0               # the windowed attention's sink: exp(0) = 1 in every denominator


def distance_slopes(heads: int) -> Tuple[float, ...]:
    """Head h takes 2^(-8 (h + 1) / heads) per token of distance off its scores."""
    return tuple(2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads))


def venezen_spec(c: VenezenConfig) -> ModelSpec:
    W = c.hidden_size

    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", LayerNormParams(W, c.norm_eps), {"weight": name})

    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "latent_attention":
            names = {n: f"{p}mix.{n}" for n in ("q", "dkv", "uk", "uv", "o")}
            names["dkv_norm"] = p + "mix.dkv.norm"
            position = None
            if m.rot_dim > 0:
                position = PartSpec("rope_halves", RotaryHalvesParams(m.rot.dims, m.rot.base, c.max_position_embeddings))
            mixer = PartSpec("latent_attention", LatentAttentionParams(
                hidden_size=W, num_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank,
                scale=m.scale, eps=c.norm_eps, position=position), names)
        else:
            mixer = PartSpec("maps_attention", MapsAttentionParams(
                hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, maps=1,
                window=m.window, scale=m.scale, eps=c.norm_eps, values_are_keys=True,
                distance_slopes=distance_slopes(m.heads), sink_value=SINK_SCORE),
                {n: f"{p}mix.{n}" for n in ("q", "k", "o")})
        f = layer.mlp
        ffn = None
        if f is not None and f.kind == "dense":
            names = {n: f"{p}mlp.{n}" for n in ("gate", "up", "down")}
            names.update({f"{n}_bias": f"{p}mlp.{n}.b" for n in ("gate", "up", "down")})
            ffn = PartSpec("swiglu_mlp", GatedMLPParams(W, f.ff, bias=True, activation="silu"), names)
        elif f is not None:
            names = {"router": p + "mlp.router", "choice_bias": p + "mlp.correction"}
            for e in range(f.experts):
                for n in ("gate", "up", "down"):
                    names[f"{n}{e}"] = f"{p}mlp.e{e}.{n}"
            if f.shared is not None:
                names.update({f"shared_{n}": f"{p}mlp.shared.{n}" for n in ("gate", "up", "down")})
            ffn = PartSpec("routed_experts", RoutedExpertsParams(
                hidden_size=W, intermediate_size=f.ff, num_experts=f.experts, top=f.top, score="softmax",
                renormalize=True, activation="clamped_swish", gated=True, identity=f.identity, choice_bias=True,
                weight_scale=f.scale, renorm_floor=WEIGHT_FLOOR, limit=f.limit, slope=SWISH_SLOPE,
                shared_intermediate_size=f.shared.ff if f.shared is not None else 0,
                shared_limit=f.shared.limit if f.shared is not None else 0.0), names)
        layers.append(LayerSpec(arrangement="prenorm", mixer_norm=norm(p + "norm1"), mixer=mixer,
                                ffn_norm=norm(p + "norm2") if ffn is not None else None, ffn=ffn))
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab_size, max_positions=c.max_position_embeddings,
        embedding=PartSpec("token_embedding", EmbeddingParams(c.vocab_size, W, c.embedding_scale), {"weight": "embed"}),
        layers=tuple(layers), order=tuple(LayerCall(i, add_embedding=add) for i, add in c.run_order()),
        final_norm=norm("final.norm"), head=PartSpec("lm_head", HeadParams(c.vocab_size, W, True), {}))


def venezen_random_tensors(c: VenezenConfig, seed: int, dtype: torch.dtype) -> Iterator[Tuple[str, tuple, object]]:
    """Yields (name, shape, make) in file order: matrices N(0, 1 / fan_in), the embedding N(0, 1) divided by its
    scale, norm weights 1 + N(0, 0.1^2), biases N(0, 0.1^2), choice corrections N(0, 0.02^2); one seeded
    generator run in order."""
    g = torch.Generator().manual_seed(seed)
    W = c.hidden_size

    def mat(n, k, std=None):
        return (n, k), lambda: (torch.randn(n, k, generator=g) * (std if std is not None else 1.0 / math.sqrt(k))).to(dtype)

    def vec(n, mean, std):
        return (n,), lambda: (mean + std * torch.randn(n, generator=g)).to(dtype)

    def emit(name, shape_make):
        return name, shape_make[0], shape_make[1]

    yield emit("embed", mat(c.vocab_size, W, 1.0 / c.embedding_scale))
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        m = layer.mixer
        yield emit(p + "norm1", vec(W, 1.0, 0.1))
        if layer.type == "latent_attention":
            yield emit(p + "mix.q", mat(m.heads * (m.dim + m.rot_dim), W))
            yield emit(p + "mix.dkv", mat(m.kv_rank + m.rot_dim, W))
            yield emit(p + "mix.dkv.norm", vec(m.kv_rank, 1.0, 0.1))
            yield emit(p + "mix.uk", mat(m.heads * m.dim, m.kv_rank))
            yield emit(p + "mix.uv", mat(m.heads * m.vdim, m.kv_rank))
            yield emit(p + "mix.o", mat(W, m.heads * m.vdim))
        else:
            yield emit(p + "mix.q", mat(m.heads * m.dim, W))
            yield emit(p + "mix.k", mat(m.kv_heads * m.dim, W))
            yield emit(p + "mix.o", mat(W, m.heads * m.vdim))
        f = layer.mlp
        if f is None:
            continue
        yield emit(p + "norm2", vec(W, 1.0, 0.1))
        if f.kind == "dense":
            for n, rows, cols in (("gate", f.ff, W), ("up", f.ff, W), ("down", W, f.ff)):
                yield emit(p + "mlp." + n, mat(rows, cols))
                yield emit(p + "mlp." + n + ".b", vec(rows, 0.0, 0.1))
        else:
            for e in range(f.experts):
                yield emit(f"{p}mlp.e{e}.gate", mat(f.ff, W))
                yield emit(f"{p}mlp.e{e}.up", mat(f.ff, W))
                yield emit(f"{p}mlp.e{e}.down", mat(W, f.ff))
            yield emit(p + "mlp.router", mat(f.experts + f.identity, W))
            yield emit(p + "mlp.correction", vec(f.experts + f.identity, 0.0, 0.02))
            if f.shared is not None:
                yield emit(p + "mlp.shared.gate", mat(f.shared.ff, W))
                yield emit(p + "mlp.shared.up", mat(f.shared.ff, W))
                yield emit(p + "mlp.shared.down", mat(W, f.shared.ff))
    yield emit("final.norm", vec(W, 1.0, 0.1))


register_architecture(Architecture(
    name="Venezen",
    config_from_hf=VenezenConfig.from_hf,
    build_spec=venezen_spec,
    random_tensors=venezen_random_tensors,
))
