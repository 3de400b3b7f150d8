"""``Vizotar`` laid out as parts: a token embedding; "hyper" blocks (pre-norm sublayers on several residual
streams, each sublayer with a ``stream_connection``) whose mixer is a pair side by side (``parallel_mixers``
with ``combine`` "normed": ``maps_attention`` with a window, a sink, short convolutions behind q, k and v,
norms over the whole projection and a ``rope_halves`` rotation with YaRN scaling, beside a ``matrix_memory``)
or the gated delta rule (``gated_delta``); a dense feed-forward with clamped gate and up (``swiglu_mlp`` with
``clamped_swish``) or routed gated experts (``routed_experts``: softmax over the chosen logits, a router
bias), or none; a final RMS norm and the embedding table as the head.  A layer that uses another layer's
tensors is a second entry of the run order for the same ``LayerSpec``, with a cache and states of its own.
Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.*``
(``l<i>.mix.left.*`` / ``l<i>.mix.right.*`` in a pair), ``l<i>.mlp.*`` (``l<i>.mlp.e<k>.*`` per expert),
``final.norm``.
"""

from __future__ import annotations

import math
from typing import Iterator, Tuple

import torch

from ..config.model_config import VizotarAttention, VizotarConfig
from ..config.registry import Architecture, register_architecture
from ..parts.attention_maps import MapsAttentionParams
from ..parts.delta_rule import GatedDeltaParams
from ..parts.embedding import EmbeddingParams, HeadParams
from ..parts.matrix_memory import MatrixMemoryParams
from ..parts.mlp import GatedMLPParams
from ..parts.moe import RoutedExpertsParams
from ..parts.parallel import parallel_spec
from ..parts.rmsnorm import RMSNormParams
from ..parts.rope import RotaryHalvesParams
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..parts.streams import StreamConnectionParams

# constants that the design fixes
MEMORY_DENOMINATOR_FLOOR = 1e-6      # added to the matrix memory's denominator
UNIT_FLOOR = 1e-6                    # under the root of the delta rule's unit vectors
GLU_SLOPE = 1.702                    # of the dense feed-forward's sigmoid
PAIR_WEIGHT = 0.5                    # a pair's output is the mean of its two normed sides


def _left_spec(c: VizotarConfig, a: VizotarAttention, prefix: str) -> PartSpec:
    names = {n: prefix + n for n in ("q", "k", "v", "o", "sink")}
    names.update({"q_bias": prefix + "q.b", "k_bias": prefix + "k.b", "v_bias": prefix + "v.b", "o_bias": prefix + "o.b",
                  "q_norm": prefix + "q.norm", "k_norm": prefix + "k.norm"})
    if a.conv > 0:
        names.update({"q_conv": prefix + "q.conv", "k_conv": prefix + "k.conv", "v_conv": prefix + "v.conv"})
    position = None
    if a.rot is not None:
        s = a.rot.scaling
        position = PartSpec("rope_halves", RotaryHalvesParams(
            a.rot.dims, a.rot.base, c.max_position_embeddings, s.factor if s else 0.0, s.original if s else 0,
            s.fast if s else 32.0, s.slow if s else 1.0))
    return PartSpec("maps_attention", MapsAttentionParams(
        hidden_size=c.hidden_size, num_heads=a.heads, num_kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim, maps=1,
        bias=True, window=a.window, scale=a.scale, eps=c.norm_eps, position=position, head_norm="whole", sink=True,
        conv_taps=a.conv, out_bias=True), names)


def vizotar_spec(c: VizotarConfig) -> ModelSpec:
    W = c.hidden_size

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", RMSNormParams(W, c.norm_eps), {"weight": name})

    def conn(prefix: str) -> PartSpec:
        return PartSpec("stream_connection", StreamConnectionParams(c.streams),
                        {n: prefix + n for n in ("in", "out", "mix")})

    layers, spec_of = [], {}
    for i, layer in enumerate(c.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "parallel":
            r = m.right
            names = {n: f"{p}mix.right.{n}" for n in ("q", "k", "v", "g", "o", "norm", "i", "f")}
            names.update({"i_bias": p + "mix.right.i.b", "f_bias": p + "mix.right.f.b"})
            memory = PartSpec("matrix_memory", MatrixMemoryParams(
                hidden_size=W, num_heads=r.heads, dim=r.dim, vdim=r.vdim, gate_cap=r.gate_cap, eps=c.norm_eps,
                floor=MEMORY_DENOMINATOR_FLOOR), names)
            mixer = parallel_spec(W, _left_spec(c, m.left, p + "mix.left."), memory, PAIR_WEIGHT, PAIR_WEIGHT,
                                  combine="normed", eps=c.norm_eps,
                                  out_norm_names={"left.out": p + "mix.left.out", "right.out": p + "mix.right.out"})
        else:
            names = {n: f"{p}mix.{n}" for n in ("q", "k", "v", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o")}
            names.update({f"{n}_conv": f"{p}mix.{n}.conv" for n in ("q", "k", "v")})
            mixer = PartSpec("gated_delta", GatedDeltaParams(
                hidden_size=W, num_heads=m.heads, num_qk_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, conv_taps=m.conv,
                decay_rank=m.decay_rank, gate_rank=m.gate_rank, eps=c.norm_eps, unit_floor=UNIT_FLOOR), names)
        f = layer.mlp
        ffn = None
        if f is not None and f.kind == "dense":
            ffn = PartSpec("swiglu_mlp", GatedMLPParams(W, f.ff, activation="clamped_swish", limit=f.limit, slope=GLU_SLOPE),
                           {n: f"{p}mlp.{n}" for n in ("gate", "up", "down")})
        elif f is not None:
            names = {"router": p + "mlp.router", "router_bias": p + "mlp.router.b"}
            for e in range(f.experts):
                names.update({f"{n}{e}": f"{p}mlp.e{e}.{n}" for n in ("gate", "up", "down")})
            ffn = PartSpec("routed_experts", RoutedExpertsParams(
                hidden_size=W, intermediate_size=f.ff, num_experts=f.experts, top=f.top, score="softmax",
                renormalize=True, activation="silu", gated=True, router_bias=True), names)
        spec_of[i] = len(layers)
        layers.append(LayerSpec(arrangement="hyper", mixer_norm=norm(p + "norm1"), mixer=mixer,
                                ffn_norm=norm(p + "norm2") if ffn is not None else None, ffn=ffn,
                                mixer_conn=conn(p + "hc1."), ffn_conn=conn(p + "hc2.") if ffn is not None else None))
    order = tuple(LayerCall(spec_of[i if layer.weights_of is None else layer.weights_of])
                  for i, layer in enumerate(c.layers))
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab_size, max_positions=c.max_position_embeddings,
        embedding=PartSpec("token_embedding", EmbeddingParams(c.vocab_size, W), {"weight": "embed"}),
        layers=tuple(layers), order=order, final_norm=norm("final.norm"),
        head=PartSpec("lm_head", HeadParams(c.vocab_size, W, True), {}))


def vizotar_random_tensors(c: VizotarConfig, seed: int, dtype: torch.dtype) -> Iterator[Tuple[str, tuple, object]]:
    """Yields (name, shape, make) in file order: matrices N(0, 1 / fan_in), the embedding N(0, 1), norm weights
    1 + N(0, 0.1^2), convolution taps N(0, 0.5^2), sinks and biases N(0, 1) (the forget gate's around 2), the
    streams' mixing matrices near the identity; one seeded generator run in order."""
    g = torch.Generator().manual_seed(seed)
    W, n = c.hidden_size, c.streams

    def mat(rows, cols, std=None):
        return (rows, cols), lambda: (torch.randn(rows, cols, generator=g) * (std if std is not None else 1.0 / math.sqrt(cols))).to(dtype)

    def vec(size, mean, std):
        return (size,), lambda: (mean + std * torch.randn(size, generator=g)).to(dtype)

    def emit(name, shape_make):
        return name, shape_make[0], shape_make[1]

    def connection(p):
        yield emit(p + "in", vec(n, 1.0 / n, 0.2 / n))
        yield emit(p + "out", vec(n, 1.0, 0.2))
        yield emit(p + "mix", ((n, n), lambda: (torch.eye(n) + 0.15 * torch.randn(n, n, generator=g)).to(dtype)))

    yield emit("embed", mat(c.vocab_size, W, 1.0))
    for i, layer in enumerate(c.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        m = layer.mixer
        yield emit(p + "norm1", vec(W, 1.0, 0.1))
        if layer.type == "parallel":
            a, r = m.left, m.right
            q = p + "mix.left."
            for name, rows in (("q", a.heads * a.dim), ("k", a.kv_heads * a.dim), ("v", a.kv_heads * a.vdim)):
                yield emit(q + name, mat(rows, W))
                yield emit(q + name + ".b", vec(rows, 0.0, 0.3))
                if a.conv > 0:
                    yield emit(q + name + ".conv", mat(rows, a.conv, 0.5))
            yield emit(q + "q.norm", vec(a.heads * a.dim, 1.0, 0.1))
            yield emit(q + "k.norm", vec(a.kv_heads * a.dim, 1.0, 0.1))
            yield emit(q + "sink", vec(a.heads, 0.0, 1.0))
            yield emit(q + "o", mat(W, a.heads * a.vdim))
            yield emit(q + "o.b", vec(W, 0.0, 0.3))
            q = p + "mix.right."
            for name, rows in (("q", r.heads * r.dim), ("k", r.heads * r.dim), ("v", r.heads * r.vdim), ("g", r.heads * r.vdim)):
                yield emit(q + name, mat(rows, W))
            yield emit(q + "o", mat(W, r.heads * r.vdim))
            yield emit(q + "norm", vec(r.heads * r.vdim, 1.0, 0.1))
            yield emit(q + "i", mat(r.heads, W))
            yield emit(q + "i.b", vec(r.heads, 0.0, 1.0))
            yield emit(q + "f", mat(r.heads, W))
            yield emit(q + "f.b", vec(r.heads, 2.0, 1.0))
            yield emit(p + "mix.left.out", vec(W, 1.0, 0.1))
            yield emit(p + "mix.right.out", vec(W, 1.0, 0.1))
        else:
            q = p + "mix."
            for name, rows in (("q", m.kv_heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.heads * m.vdim)):
                yield emit(q + name, mat(rows, W))
                yield emit(q + name + ".conv", mat(rows, m.conv, 0.5))
            yield emit(q + "b", mat(m.heads, W))
            yield emit(q + "A_log", vec(m.heads, -1.0, 0.5))
            yield emit(q + "norm", vec(m.vdim, 1.0, 0.1))
            yield emit(q + "a1", mat(m.decay_rank, W))
            yield emit(q + "a2", mat(m.heads * m.dim, m.decay_rank))
            yield emit(q + "dt_bias", vec(m.heads * m.dim, -1.0, 1.0))
            yield emit(q + "g1", mat(m.gate_rank, W))
            yield emit(q + "g2", mat(m.heads * m.vdim, m.gate_rank))
            yield emit(q + "o", mat(W, m.heads * m.vdim))
        f = layer.mlp
        if f is not None:
            yield emit(p + "norm2", vec(W, 1.0, 0.1))
            if f.kind == "dense":
                yield emit(p + "mlp.gate", mat(f.ff, W))
                yield emit(p + "mlp.up", mat(f.ff, W))
                yield emit(p + "mlp.down", mat(W, f.ff))
            else:
                for e in range(f.experts):
                    yield emit(f"{p}mlp.e{e}.gate", mat(f.ff, W))
                    yield emit(f"{p}mlp.e{e}.up", mat(f.ff, W))
                    yield emit(f"{p}mlp.e{e}.down", mat(W, f.ff))
                yield emit(p + "mlp.router", mat(f.experts, W))
                yield emit(p + "mlp.router.b", vec(f.experts, 0.0, 1.0))
        yield from connection(p + "hc1.")
        if f is not None:
            yield from connection(p + "hc2.")
    yield emit("final.norm", vec(W, 1.0, 0.1))


register_architecture(Architecture(
    name="Vizotar",
    config_from_hf=VizotarConfig.from_hf,
    build_spec=vizotar_spec,
    random_tensors=vizotar_random_tensors,
))
