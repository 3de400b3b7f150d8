"""Typed model configurations read from an architecture's own ``config.json`` keys.

``ModelConfig`` is what the rest of the framework may ask of any architecture;
``LlamaConfig`` holds what ``LlamaForCausalLM`` adds.  Keys, defaults and the
accepted rope-scaling types follow the reference's reading of HF configs
(python/redline/convert.py:86-150) and its validation
(src/core/model_config.cpp:97-116).  No size or constant that ``config.json``
gives is repeated anywhere else in the package.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A ``config.json`` that cannot be used, with the key that is at fault."""


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of rotary embeddings (src/core/model_config.h:26-32)."""

    type: str = "none"  # none | linear | llama3
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @staticmethod
    def from_hf(cfg: Dict[str, Any]) -> Tuple[float, "RopeScaling"]:
        """Returns (rope_theta, scaling) from ``rope_scaling`` / ``rope_parameters``
        and ``rope_theta`` (python/redline/convert.py:86-105)."""
        params = cfg.get("rope_parameters") or {}
        scaling = cfg.get("rope_scaling") or params or None
        theta = float(cfg.get("rope_theta", params.get("rope_theta", 10000.0)))
        if not scaling:
            return theta, RopeScaling()
        rtype = scaling.get("rope_type", scaling.get("type", "default"))
        if rtype in ("default", None, "none"):
            return theta, RopeScaling()
        if rtype == "linear":
            return theta, RopeScaling(type="linear", factor=float(_need(scaling, "factor", "rope_scaling")))
        if rtype == "llama3":
            return theta, RopeScaling(
                type="llama3",
                factor=float(_need(scaling, "factor", "rope_scaling")),
                low_freq_factor=float(scaling.get("low_freq_factor", 1.0)),
                high_freq_factor=float(scaling.get("high_freq_factor", 4.0)),
                original_max_position_embeddings=int(
                    scaling.get("original_max_position_embeddings", 8192)),
            )
        raise ConfigError(f"rope_scaling type '{rtype}' is not supported (none, default, linear, llama3)")

    def to_hf(self) -> Optional[Dict[str, Any]]:
        if self.type == "none":
            return None
        if self.type == "linear":
            return {"rope_type": "linear", "factor": self.factor}
        return {
            "rope_type": "llama3",
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


def _need(d: Dict[str, Any], key: str, where: str = "config.json") -> Any:
    if key not in d or d[key] is None:
        raise ConfigError(f"{where} has no '{key}'")
    return d[key]


@dataclass(frozen=True)
class ModelConfig:
    """What every architecture's configuration gives the engine."""

    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    bos_token_id: int
    eos_token_ids: Tuple[int, ...]

    def to_hf(self) -> Dict[str, Any]:  # pragma: no cover - overridden
        raise NotImplementedError

    def save(self, model_dir: str) -> None:
        os.makedirs(model_dir, exist_ok=True)
        with open(os.path.join(model_dir, "config.json"), "w") as f:
            json.dump(self.to_hf(), f, indent=1)


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    """``LlamaForCausalLM``: pre-norm decoder, RMSNorm, grouped-query attention with
    rotary embeddings, SiLU-gated feed-forward (src/cuda/model/llama.cpp:56-151)."""

    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    attention_bias: bool = False
    mlp_bias: bool = False
    tie_word_embeddings: bool = False

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def gqa_group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @classmethod
    def from_hf(cls, cfg: Dict[str, Any], model_dir: Optional[str] = None) -> "LlamaConfig":
        archs = cfg.get("architectures") or ["LlamaForCausalLM"]
        act = cfg.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act '{act}' is not supported: the feed-forward is SiLU-gated")
        theta, scaling = RopeScaling.from_hf(cfg)
        heads = int(_need(cfg, "num_attention_heads"))
        hidden = int(_need(cfg, "hidden_size"))
        eos = cfg.get("eos_token_id")
        if model_dir is not None:
            gen = os.path.join(model_dir, "generation_config.json")
            if os.path.exists(gen):
                with open(gen) as f:
                    eos = json.load(f).get("eos_token_id", eos)
        if eos is None:
            eos = []
        elif isinstance(eos, int):
            eos = [eos]
        bos = cfg.get("bos_token_id")
        c = cls(
            architecture=archs[0],
            vocab_size=int(_need(cfg, "vocab_size")),
            hidden_size=hidden,
            max_position_embeddings=int(cfg.get("max_position_embeddings", 4096)),
            bos_token_id=int(bos) if bos is not None else -1,
            eos_token_ids=tuple(int(e) for e in eos),
            intermediate_size=int(_need(cfg, "intermediate_size")),
            num_hidden_layers=int(_need(cfg, "num_hidden_layers")),
            num_attention_heads=heads,
            num_key_value_heads=int(cfg.get("num_key_value_heads") or heads),
            head_dim=int(cfg.get("head_dim") or hidden // heads),
            rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-5)),
            rope_theta=theta,
            rope_scaling=scaling,
            attention_bias=bool(cfg.get("attention_bias", False)),
            mlp_bias=bool(cfg.get("mlp_bias", False)),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        )
        c.validate()
        return c

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim must be even for rotary embeddings, got {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.rope_scaling.type != "none" and not self.rope_scaling.factor > 0:
            raise ConfigError("rope_scaling.factor must be positive")
        if self.rope_scaling.type == "llama3" and \
                self.rope_scaling.high_freq_factor == self.rope_scaling.low_freq_factor:
            raise ConfigError("rope_scaling: high_freq_factor must differ from low_freq_factor")

    def to_hf(self) -> Dict[str, Any]:
        eos: Any = list(self.eos_token_ids)
        if len(eos) == 1:
            eos = eos[0]
        elif not eos:
            eos = None
        return {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_hf(),
            "max_position_embeddings": self.max_position_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "tie_word_embeddings": self.tie_word_embeddings,
            "bos_token_id": self.bos_token_id if self.bos_token_id >= 0 else None,
            "eos_token_id": eos,
            "torch_dtype": "bfloat16",
        }


# --------------------------------------------------------------------------- Kapitar

@dataclass(frozen=True)
class KapitarMask:
    size: int                 # a key is visible while the query is less than so many positions ahead of it
    keep_first: int = 0       # ... and the first so many keys of the sequence always are


@dataclass(frozen=True)
class KapitarAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    diff: float
    mask: KapitarMask


@dataclass(frozen=True)
class KapitarLightning:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class KapitarMLP:
    kind: str                 # dense | moe
    ff: int                   # dense: width of the layer; moe: of one expert
    experts: int = 0
    top: int = 0
    groups: int = 1
    groups_keep: int = 1
    shared_ff: int = 0        # 0: no shared expert


@dataclass(frozen=True)
class KapitarLayer:
    type: str                 # attention | lightning
    mixer: Any
    mlp: Optional[KapitarMLP]


@dataclass(frozen=True)
class KapitarConfig(ModelConfig):
    """``Kapitar``: a decoder whose layers norm (layer norm, weight only) the input and the output of every
    sublayer; mixers are differential attention (two capped score maps over shared values, a window that
    keeps the first tokens, no rotation) or linear attention with a per-head decay; feed-forwards are dense
    (squared ReLU) or routed (sigmoid router, groups of experts, a shared expert, erf GELU); the head is the
    embedding table.  Its config.json lists the layers one by one under ``layers``."""

    norm_eps: float = 1e-6
    layers: Tuple[KapitarLayer, ...] = ()
    raw: Optional[Dict[str, Any]] = field(default=None, compare=False, repr=False)

    @classmethod
    def from_hf(cls, cfg: Dict[str, Any], model_dir: Optional[str] = None) -> "KapitarConfig":
        layers: List[KapitarLayer] = []
        for i, entry in enumerate(_need(cfg, "layers")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            m = _need(entry, "mixer", where)
            if kind == "attention":
                mask = _need(m, "mask", where + ".mixer")
                mixer: Any = KapitarAttention(
                    heads=int(_need(m, "heads", where)), kv_heads=int(m.get("kv_heads") or m["heads"]),
                    dim=int(_need(m, "dim", where)), vdim=int(_need(m, "vdim", where)),
                    scale=float(_need(m, "scale", where)), softcap=float(_need(m, "softcap", where)),
                    diff=float(_need(m, "diff", where)),
                    mask=KapitarMask(int(_need(mask, "size", where + ".mixer.mask")), int(mask.get("keep_first", 0))))
            elif kind == "lightning":
                mixer = KapitarLightning(heads=int(_need(m, "heads", where)), dim=int(_need(m, "dim", where)),
                                         vdim=int(_need(m, "vdim", where)),
                                         decay=tuple(float(d) for d in _need(m, "decay", where)))
            else:
                raise ConfigError(f"{where}: mixer type '{kind}' is not supported (attention, lightning)")
            mlp = entry.get("mlp")
            ff: Optional[KapitarMLP] = None
            if mlp is not None:
                mk = _need(mlp, "kind", where + ".mlp")
                if mk == "dense":
                    ff = KapitarMLP("dense", int(_need(mlp, "ff", where + ".mlp")))
                elif mk == "moe":
                    r = _need(mlp, "router", where + ".mlp")
                    groups = r.get("groups") or {}
                    shared = mlp.get("shared") or {}
                    ff = KapitarMLP("moe", int(_need(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert")),
                                    experts=int(_need(r, "experts", where + ".mlp.router")),
                                    top=int(_need(r, "top", where + ".mlp.router")),
                                    groups=int(groups.get("count", 1)), groups_keep=int(groups.get("keep", groups.get("count", 1))),
                                    shared_ff=int(shared.get("ff", 0)))
                else:
                    raise ConfigError(f"{where}.mlp: kind '{mk}' is not supported (dense, moe)")
            layers.append(KapitarLayer(kind, mixer, ff))
        eos = cfg.get("eos_token_id")
        eos = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        bos = cfg.get("bos_token_id")
        c = cls(architecture="Kapitar", vocab_size=int(_need(cfg, "vocab")), hidden_size=int(_need(cfg, "width")),
                max_position_embeddings=int(cfg.get("max_positions", 1 << 30)),
                bos_token_id=int(bos) if bos is not None else -1, eos_token_ids=tuple(int(e) for e in eos),
                norm_eps=float(_need(_need(cfg, "norm"), "eps", "norm")), layers=tuple(layers), raw=dict(cfg))
        c.validate()
        return c

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.heads <= 0 or m.dim <= 0 or m.vdim <= 0:
                raise ConfigError(f"layers[{i}]: heads, dim and vdim must be positive")
            if layer.type == "attention":
                if m.kv_heads <= 0 or m.heads % m.kv_heads != 0:
                    raise ConfigError(f"layers[{i}]: heads ({m.heads}) must be a multiple of kv_heads ({m.kv_heads})")
                if m.mask.size <= 0 or m.mask.keep_first < 0 or not m.softcap > 0:
                    raise ConfigError(f"layers[{i}]: mask.size and softcap must be positive, keep_first not negative")
            elif len(m.decay) != m.heads:
                raise ConfigError(f"layers[{i}]: {m.heads} heads need as many decays, got {len(m.decay)}")
            f = layer.mlp
            if f is not None and f.kind == "moe":
                if f.experts <= 0 or f.groups <= 0 or f.experts % f.groups != 0 or not 1 <= f.groups_keep <= f.groups:
                    raise ConfigError(f"layers[{i}].mlp: {f.experts} experts do not form {f.groups} equal groups "
                                      f"of which {f.groups_keep} stay")
                if not 1 <= f.top <= f.groups_keep * (f.experts // f.groups):
                    raise ConfigError(f"layers[{i}].mlp: top {f.top} experts cannot be chosen")

    def to_hf(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                         "softcap": m.softcap, "diff": m.diff, "mask": {"size": m.mask.size, "keep_first": m.mask.keep_first}}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            f = layer.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.ff},
                       "router": {"experts": f.experts, "top": f.top, "groups": {"count": f.groups, "keep": f.groups_keep}}}
                if f.shared_ff > 0:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        out = {"architecture": "Kapitar", "vocab": self.vocab_size, "width": self.hidden_size,
               "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.bos_token_id >= 0:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


# ------------------------------------------------------------------------------------ Pufevik

@dataclass(frozen=True)
class PufevikRotation:
    base: float
    dims: int                 # the first so many entries of every head are rotated


@dataclass(frozen=True)
class PufevikAttention:
    """Softmax attention of a Pufevik layer.  ``window`` 0: every earlier key (the 'attention' mixer, whose
    queries and keys are normed per head and whose gate is one number per output entry); > 0: a sliding window
    (the left side of a 'parallel' mixer: norms over the whole projection, a sink, one gate per head)."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[PufevikRotation]
    window: int = 0
    v_mix: bool = False


@dataclass(frozen=True)
class PufevikMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class PufevikParallel:
    left: PufevikAttention
    right: PufevikMemory
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class PufevikLayer:
    type: str                 # attention | parallel
    mixer: Any
    ff: int                   # width of the dense feed-forward; 0: the layer has none


@dataclass(frozen=True)
class PufevikConfig(ModelConfig):
    """``Pufevik``: a decoder whose sublayers read the residual stream itself and whose outputs are RMS-normed
    before they are added.  Mixers: gated softmax attention with normed, partly rotated queries and keys and
    values blended with those of the first such layer; or a pair side by side, windowed attention with a sink
    beside a matrix memory with exponential gates.  Feed-forwards are dense and gated (tanh GELU).  The
    embedding is multiplied by a constant; the head has a matrix of its own.  config.json lists the layers one
    by one under ``layers``."""

    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    layers: Tuple[PufevikLayer, ...] = ()
    raw: Optional[Dict[str, Any]] = field(default=None, compare=False, repr=False)

    @staticmethod
    def _attention(m: Dict[str, Any], where: str) -> PufevikAttention:
        rot = m.get("rot")
        mask = m.get("mask") or {}
        heads = int(_need(m, "heads", where))
        return PufevikAttention(
            heads=heads, kv_heads=int(m.get("kv_heads") or heads), dim=int(_need(m, "dim", where)),
            vdim=int(_need(m, "vdim", where)), scale=float(_need(m, "scale", where)),
            rot=PufevikRotation(float(_need(rot, "base", where + ".rot")), int(_need(rot, "dims", where + ".rot")))
            if rot else None,
            window=int(mask.get("size", 0)), v_mix=bool(m.get("v_mix", False)))

    @classmethod
    def from_hf(cls, cfg: Dict[str, Any], model_dir: Optional[str] = None) -> "PufevikConfig":
        layers: List[PufevikLayer] = []
        for i, entry in enumerate(_need(cfg, "layers")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            m = _need(entry, "mixer", where)
            if kind == "attention":
                mixer: Any = cls._attention(m, where + ".mixer")
            elif kind == "parallel":
                r = _need(m, "right", where + ".mixer")
                rw = where + ".mixer.right"
                mixer = PufevikParallel(
                    left=cls._attention(_need(m, "left", where + ".mixer"), where + ".mixer.left"),
                    right=PufevikMemory(int(_need(r, "heads", rw)), int(_need(r, "dim", rw)), int(_need(r, "vdim", rw)),
                                        float(_need(r, "gate_cap", rw))),
                    left_scale=float(_need(m, "left_scale", where + ".mixer")),
                    right_scale=float(_need(m, "right_scale", where + ".mixer")))
            else:
                raise ConfigError(f"{where}: mixer type '{kind}' is not supported (attention, parallel)")
            mlp = entry.get("mlp")
            ff = 0
            if mlp is not None:
                if _need(mlp, "kind", where + ".mlp") != "dense":
                    raise ConfigError(f"{where}.mlp: kind '{mlp['kind']}' is not supported (dense)")
                ff = int(_need(mlp, "ff", where + ".mlp"))
            layers.append(PufevikLayer(kind, mixer, ff))
        eos = cfg.get("eos_token_id")
        eos = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        bos = cfg.get("bos_token_id")
        c = cls(architecture="Pufevik", vocab_size=int(_need(cfg, "vocab")), hidden_size=int(_need(cfg, "width")),
                max_position_embeddings=int(cfg.get("max_positions", 1 << 30)),
                bos_token_id=int(bos) if bos is not None else -1, eos_token_ids=tuple(int(e) for e in eos),
                norm_eps=float(_need(_need(cfg, "norm"), "eps", "norm")),
                embedding_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)), layers=tuple(layers), raw=dict(cfg))
        c.validate()
        return c

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        shared = None
        for i, layer in enumerate(self.layers):
            att = layer.mixer if layer.type == "attention" else layer.mixer.left
            if att.heads <= 0 or att.kv_heads <= 0 or att.heads % att.kv_heads != 0 or att.dim <= 0 or att.vdim <= 0:
                raise ConfigError(f"layers[{i}]: heads must be a positive multiple of kv_heads, dim and vdim positive")
            if att.rot is not None and (att.rot.dims <= 0 or att.rot.dims % 2 != 0 or att.rot.dims > att.dim):
                raise ConfigError(f"layers[{i}]: rot.dims must be even and at most dim")
            if att.window < 0 or layer.ff < 0:
                raise ConfigError(f"layers[{i}]: mask.size and mlp.ff must not be negative")
            if layer.type == "attention" and att.v_mix:
                if shared is not None and shared != (att.kv_heads, att.vdim):
                    raise ConfigError(f"layers[{i}]: layers with v_mix must have values of one shape (kv_heads, vdim)")
                shared = (att.kv_heads, att.vdim)
            if layer.type == "parallel":
                r = layer.mixer.right
                if r.heads <= 0 or r.dim <= 0 or r.vdim <= 0 or not r.gate_cap > 0:
                    raise ConfigError(f"layers[{i}].mixer.right: heads, dim, vdim and gate_cap must be positive")

    def to_hf(self) -> Dict[str, Any]:
        def attention(a: PufevikAttention, parallel: bool) -> Dict[str, Any]:
            out: Dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
            if a.rot is not None:
                out["rot"] = {"base": a.rot.base, "dims": a.rot.dims}
            if parallel:
                out["mask"] = {"size": a.window}
            else:
                out["v_mix"] = a.v_mix
            return out

        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                mixer = attention(m, False)
            else:
                mixer = {"left": attention(m.left, True), "left_scale": m.left_scale,
                         "right": {"heads": m.right.heads, "dim": m.right.dim, "vdim": m.right.vdim,
                                   "gate_cap": m.right.gate_cap},
                         "right_scale": m.right_scale}
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": {"kind": "dense", "ff": layer.ff} if layer.ff > 0 else None})
        out = {"architecture": "Pufevik", "vocab": self.vocab_size, "width": self.hidden_size,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.bos_token_id >= 0:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


# ------------------------------------------------------------------------------------ Vizotar

@dataclass(frozen=True)
class VizotarScaling:
    """YaRN scaling of a rotation's frequencies."""

    factor: float
    original: int
    fast: float
    slow: float


@dataclass(frozen=True)
class VizotarRotation:
    base: float
    dims: int                 # the first so many entries of every head are rotated, entry i with i + dims / 2
    scaling: Optional[VizotarScaling] = None


@dataclass(frozen=True)
class VizotarAttention:
    """The left side of a 'parallel' mixer: windowed softmax attention with a sink."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int               # mask.size; 0: every earlier key
    conv: int                 # taps of the convolution behind q, k and v; 0: none
    rot: Optional[VizotarRotation]


@dataclass(frozen=True)
class VizotarMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class VizotarParallel:
    left: VizotarAttention
    right: VizotarMemory


@dataclass(frozen=True)
class VizotarDelta:
    """A 'channel_delta' mixer.  The inner sizes of its two low-rank projections are not in config.json: they are
    the checkpoint's tensor shapes (``decay_rank`` / ``gate_rank`` may be given for a model without a file)."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int
    gate_rank: int


@dataclass(frozen=True)
class VizotarMLP:
    kind: str                 # dense | moe
    ff: int                   # dense: width of the layer; moe: of one expert
    limit: float = 0.0        # dense: the clamp of gate and up
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class VizotarLayer:
    type: str                 # parallel | channel_delta
    mixer: Any
    mlp: Optional[VizotarMLP]
    weights_of: Optional[int] = None     # the layer whose tensors this one uses (caches and states are its own)


def _safetensors_shapes(model_dir: Optional[str]) -> Dict[str, Tuple[int, ...]]:
    """Tensor name -> shape from the header of ``model.safetensors`` (empty if there is no such file)."""
    if not model_dir:
        return {}
    path = os.path.join(model_dir, "model.safetensors")
    try:
        with open(path, "rb") as f:
            n = int.from_bytes(f.read(8), "little")
            if not 0 < n < (1 << 30):
                return {}
            header = json.loads(f.read(n))
    except (OSError, ValueError):
        return {}
    return {k: tuple(v["shape"]) for k, v in header.items() if k != "__metadata__" and isinstance(v, dict)}


@dataclass(frozen=True)
class VizotarConfig(ModelConfig):
    """``Vizotar``: pre-norm sublayers on ``streams`` residual streams (hyper-connections).  Mixers: a pair side by
    side (windowed attention with a sink, short convolutions behind q, k and v, norms over the whole projection
    and a partly rotated head with YaRN scaling, beside a matrix memory with exponential gates; each side's
    output RMS-normed, then their mean), or the gated delta rule with a decay per key channel.  Feed-forwards:
    dense with clamped gate and up, or routed experts (softmax over the chosen logits).  A layer may use
    another layer's tensors.  The head is the embedding table.  config.json lists the layers under ``layers``."""

    norm_eps: float = 1e-6
    streams: int = 1
    layers: Tuple[VizotarLayer, ...] = ()
    raw: Optional[Dict[str, Any]] = field(default=None, compare=False, repr=False)

    @staticmethod
    def _attention(m: Dict[str, Any], where: str) -> VizotarAttention:
        rot = m.get("rot")
        r = None
        if rot:
            sc = rot.get("scaling")
            w = where + ".rot.scaling"
            r = VizotarRotation(float(_need(rot, "base", where + ".rot")), int(_need(rot, "dims", where + ".rot")),
                                VizotarScaling(float(_need(sc, "factor", w)), int(_need(sc, "original", w)),
                                               float(_need(sc, "fast", w)), float(_need(sc, "slow", w))) if sc else None)
        heads = int(_need(m, "heads", where))
        return VizotarAttention(heads=heads, kv_heads=int(m.get("kv_heads") or heads), dim=int(_need(m, "dim", where)),
                                vdim=int(_need(m, "vdim", where)), scale=float(_need(m, "scale", where)),
                                window=int((m.get("mask") or {}).get("size", 0)), conv=int(m.get("conv") or 0), rot=r)

    @classmethod
    def from_hf(cls, cfg: Dict[str, Any], model_dir: Optional[str] = None) -> "VizotarConfig":
        shapes = _safetensors_shapes(model_dir)
        entries = _need(cfg, "layers")
        layers: List[VizotarLayer] = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            m = _need(entry, "mixer", where)
            src = entry.get("weights_of")
            if src is not None and not (isinstance(src, int) and 0 <= src < i and entries[src].get("weights_of") is None):
                raise ConfigError(f"{where}: weights_of must name an earlier layer that has tensors of its own")
            if kind == "parallel":
                r = _need(m, "right", where + ".mixer")
                rw = where + ".mixer.right"
                mixer: Any = VizotarParallel(
                    left=cls._attention(_need(m, "left", where + ".mixer"), where + ".mixer.left"),
                    right=VizotarMemory(int(_need(r, "heads", rw)), int(_need(r, "dim", rw)), int(_need(r, "vdim", rw)),
                                        float(_need(r, "gate_cap", rw))))
            elif kind == "channel_delta":
                heads = int(_need(m, "heads", where + ".mixer"))
                p = f"l{i if src is None else src}.mix."
                ranks = []
                for key, name in (("decay_rank", "a1"), ("gate_rank", "g1")):
                    if p + name in shapes:
                        ranks.append(int(shapes[p + name][0]))
                    elif m.get(key) is not None:
                        ranks.append(int(m[key]))
                    else:
                        raise ConfigError(f"{where}.mixer: the inner size of '{name}' is neither a tensor shape of the "
                                          f"checkpoint nor given as '{key}'")
                mixer = VizotarDelta(heads=heads, kv_heads=int(m.get("kv_heads") or heads),
                                     dim=int(_need(m, "dim", where + ".mixer")), vdim=int(_need(m, "vdim", where + ".mixer")),
                                     conv=int(_need(m, "conv", where + ".mixer")), decay_rank=ranks[0], gate_rank=ranks[1])
            else:
                raise ConfigError(f"{where}: mixer type '{kind}' is not supported (parallel, channel_delta)")
            mlp = entry.get("mlp")
            ff: Optional[VizotarMLP] = None
            if mlp is not None:
                mk = _need(mlp, "kind", where + ".mlp")
                if mk == "dense":
                    ff = VizotarMLP("dense", int(_need(mlp, "ff", where + ".mlp")), limit=float(_need(mlp, "limit", where + ".mlp")))
                elif mk == "moe":
                    r = _need(mlp, "router", where + ".mlp")
                    ff = VizotarMLP("moe", int(_need(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert")),
                                    experts=int(_need(r, "experts", where + ".mlp.router")),
                                    top=int(_need(r, "top", where + ".mlp.router")))
                else:
                    raise ConfigError(f"{where}.mlp: kind '{mk}' is not supported (dense, moe)")
            layers.append(VizotarLayer(kind, mixer, ff, src))
        eos = cfg.get("eos_token_id")
        eos = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        bos = cfg.get("bos_token_id")
        c = cls(architecture="Vizotar", vocab_size=int(_need(cfg, "vocab")), hidden_size=int(_need(cfg, "width")),
                max_position_embeddings=int(cfg.get("max_positions", 1 << 30)),
                bos_token_id=int(bos) if bos is not None else -1, eos_token_ids=tuple(int(e) for e in eos),
                norm_eps=float(_need(_need(cfg, "norm"), "eps", "norm")), streams=int(cfg.get("streams", 1)),
                layers=tuple(layers), raw=dict(cfg))
        c.validate()
        return c

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if not 1 <= self.streams <= 8:
            raise ConfigError(f"streams must lie between 1 and 8, got {self.streams}")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.weights_of is not None and (self.layers[layer.weights_of].type != layer.type
                                                 or self.layers[layer.weights_of].mixer != m
                                                 or self.layers[layer.weights_of].mlp != layer.mlp):
                raise ConfigError(f"layers[{i}]: a layer that uses another one's tensors has the same mixer and mlp entries")
            if layer.type == "parallel":
                a, r = m.left, m.right
                if a.heads <= 0 or a.kv_heads <= 0 or a.heads % a.kv_heads != 0 or a.dim <= 0 or a.vdim <= 0:
                    raise ConfigError(f"layers[{i}].mixer.left: heads must be a positive multiple of kv_heads, dim and vdim positive")
                if a.rot is not None and (a.rot.dims <= 0 or a.rot.dims % 2 != 0 or a.rot.dims > a.dim):
                    raise ConfigError(f"layers[{i}].mixer.left: rot.dims must be even and at most dim")
                if a.rot is not None and a.rot.scaling is not None and not (
                        a.rot.scaling.factor > 0 and a.rot.scaling.original > 0 and a.rot.scaling.fast > 0
                        and a.rot.scaling.slow > 0 and a.rot.base > 1):
                    raise ConfigError(f"layers[{i}].mixer.left: rot.scaling needs positive factor, original, fast and slow")
                if a.window < 0 or not 0 <= a.conv <= 8:
                    raise ConfigError(f"layers[{i}].mixer.left: mask.size must not be negative, conv at most 8")
                if r.heads <= 0 or r.dim <= 0 or r.vdim <= 0 or not r.gate_cap > 0:
                    raise ConfigError(f"layers[{i}].mixer.right: heads, dim, vdim and gate_cap must be positive")
            else:
                if m.heads <= 0 or m.kv_heads <= 0 or m.heads % m.kv_heads != 0 or m.dim <= 0 or m.vdim <= 0:
                    raise ConfigError(f"layers[{i}].mixer: heads must be a positive multiple of kv_heads, dim and vdim positive")
                if not 1 <= m.conv <= 8 or m.decay_rank <= 0 or m.gate_rank <= 0:
                    raise ConfigError(f"layers[{i}].mixer: conv must lie between 1 and 8, the inner sizes be positive")
            f = layer.mlp
            if f is not None and (f.ff <= 0 or (f.kind == "dense" and not f.limit > 0)
                                  or (f.kind == "moe" and not 1 <= f.top <= f.experts)):
                raise ConfigError(f"layers[{i}].mlp: ff and limit must be positive, top between 1 and experts")

    def to_hf(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "parallel":
                a, r = m.left, m.right
                left: Dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim,
                                        "scale": a.scale, "mask": {"size": a.window}, "conv": a.conv}
                if a.rot is not None:
                    left["rot"] = {"base": a.rot.base, "dims": a.rot.dims}
                    if a.rot.scaling is not None:
                        s = a.rot.scaling
                        left["rot"]["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
                mixer = {"left": left, "right": {"heads": r.heads, "dim": r.dim, "vdim": r.vdim, "gate_cap": r.gate_cap}}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv,
                         "decay_rank": m.decay_rank, "gate_rank": m.gate_rank}
            f = layer.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff, "limit": f.limit}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.ff}, "router": {"experts": f.experts, "top": f.top}}
            entry = {"type": layer.type, "mixer": mixer, "mlp": mlp}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            layers.append(entry)
        out = {"architecture": "Vizotar", "vocab": self.vocab_size, "width": self.hidden_size, "streams": self.streams,
               "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.bos_token_id >= 0:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


# ------------------------------------------------------------------------------------------------ Venezen

@dataclass(frozen=True)
class VenezenRotation:
    base: float
    dims: int                 # the first so many entries of the rotated part turn, entry i with i + dims / 2


@dataclass(frozen=True)
class VenezenLatent:
    """A 'latent_attention' mixer: keys and values of all heads come from one cached latent vector per token."""

    heads: int
    dim: int                  # unrotated entries of a head's query and key
    rot_dim: int              # rotated entries (the key's are one vector for all heads)
    vdim: int
    kv_rank: int              # size of the latent
    scale: float
    rot: VenezenRotation


@dataclass(frozen=True)
class VenezenWindowed:
    """An 'attention' mixer: grouped heads over a sliding window, the keys serving as values."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int               # mask.size; 0: every earlier key


@dataclass(frozen=True)
class VenezenShared:
    ff: int
    limit: float


@dataclass(frozen=True)
class VenezenMLP:
    kind: str                 # dense | moe
    ff: int                   # dense: width of the layer; moe: of one expert
    limit: float = 0.0        # moe: the clamp of an expert's gate and up
    experts: int = 0
    identity: int = 0         # router outputs behind the experts that stand for the input itself
    top: int = 0
    scale: float = 1.0        # factor on the chosen experts' weights
    shared: Optional[VenezenShared] = None


@dataclass(frozen=True)
class VenezenLayer:
    type: str                 # latent_attention | attention
    mixer: Any
    mlp: Optional[VenezenMLP]


@dataclass(frozen=True)
class VenezenLoop:
    """Layers ``start`` .. ``stop`` - 1 run ``times`` times in a row on the same tensors."""

    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class VenezenConfig(ModelConfig):
    """``Venezen``: pre-norm layers (layer norm with a weight) on one float32 stream fed by a scaled embedding.
    Mixers: attention over a cached latent with a partly rotated key shared by all heads, or grouped attention
    over a window whose keys are its values, with a distance bias per head and a one in the softmax's
    denominator.  Feed-forwards: dense SiLU-gated with biases, or routed experts with clamped gate and up, a
    choice corrected per expert, identity experts and a shared expert.  A run of layers may be repeated; the
    head is the embedding table.  config.json lists the layers under ``layers``."""

    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    layers: Tuple[VenezenLayer, ...] = ()
    loop: Optional[VenezenLoop] = None

    @classmethod
    def from_hf(cls, cfg: Dict[str, Any], model_dir: Optional[str] = None) -> "VenezenConfig":
        layers: List[VenezenLayer] = []
        for i, entry in enumerate(_need(cfg, "layers")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            m = _need(entry, "mixer", where)
            mw = where + ".mixer"
            if kind == "latent_attention":
                rot = _need(m, "rot", mw)
                mixer: Any = VenezenLatent(
                    heads=int(_need(m, "heads", mw)), dim=int(_need(m, "dim", mw)), rot_dim=int(_need(m, "rot_dim", mw)),
                    vdim=int(_need(m, "vdim", mw)), kv_rank=int(_need(m, "kv_rank", mw)), scale=float(_need(m, "scale", mw)),
                    rot=VenezenRotation(float(_need(rot, "base", mw + ".rot")), int(_need(rot, "dims", mw + ".rot"))))
            elif kind == "attention":
                heads = int(_need(m, "heads", mw))
                mixer = VenezenWindowed(
                    heads=heads, kv_heads=int(m.get("kv_heads") or heads), dim=int(_need(m, "dim", mw)),
                    vdim=int(_need(m, "vdim", mw)), scale=float(_need(m, "scale", mw)),
                    window=int((m.get("mask") or {}).get("size", 0)))
            else:
                raise ConfigError(f"{where}: mixer type '{kind}' is not supported (latent_attention, attention)")
            mlp = entry.get("mlp")
            ff: Optional[VenezenMLP] = None
            if mlp is not None:
                fw = where + ".mlp"
                mk = _need(mlp, "kind", fw)
                if mk == "dense":
                    ff = VenezenMLP("dense", int(_need(mlp, "ff", fw)))
                elif mk == "moe":
                    r = _need(mlp, "router", fw)
                    e = _need(mlp, "expert", fw)
                    sh = mlp.get("shared")
                    ff = VenezenMLP(
                        "moe", int(_need(e, "ff", fw + ".expert")), limit=float(_need(e, "limit", fw + ".expert")),
                        experts=int(_need(r, "experts", fw + ".router")), identity=int(r.get("identity") or 0),
                        top=int(_need(r, "top", fw + ".router")), scale=float(r.get("scale", 1.0)),
                        shared=VenezenShared(int(_need(sh, "ff", fw + ".shared")), float(_need(sh, "limit", fw + ".shared")))
                        if sh else None)
                else:
                    raise ConfigError(f"{fw}: kind '{mk}' is not supported (dense, moe)")
            layers.append(VenezenLayer(kind, mixer, ff))
        lp = cfg.get("loop")
        loop = None
        if lp:
            loop = VenezenLoop(int(_need(lp, "start", "loop")), int(_need(lp, "stop", "loop")), int(_need(lp, "times", "loop")))
        eos = cfg.get("eos_token_id")
        eos = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        bos = cfg.get("bos_token_id")
        c = cls(architecture="Venezen", vocab_size=int(_need(cfg, "vocab")), hidden_size=int(_need(cfg, "width")),
                max_position_embeddings=int(cfg.get("max_positions", 1 << 30)),
                bos_token_id=int(bos) if bos is not None else -1, eos_token_ids=tuple(int(e) for e in eos),
                norm_eps=float(_need(_need(cfg, "norm"), "eps", "norm")),
                embedding_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                layers=tuple(layers), loop=loop)
        c.validate()
        return c

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            mw = f"layers[{i}].mixer"
            if layer.type == "latent_attention":
                if min(m.heads, m.dim, m.vdim, m.kv_rank) <= 0 or m.rot_dim < 0:
                    raise ConfigError(f"{mw}: heads, dim, vdim and kv_rank must be positive")
                if m.rot_dim > 0 and (m.rot.dims <= 0 or m.rot.dims % 2 != 0 or m.rot.dims > m.rot_dim or not m.rot.base > 0):
                    raise ConfigError(f"{mw}: rot.dims must be even and at most rot_dim, rot.base positive")
            else:
                if m.heads <= 0 or m.kv_heads <= 0 or m.heads % m.kv_heads != 0 or m.dim <= 0:
                    raise ConfigError(f"{mw}: heads must be a positive multiple of kv_heads, dim positive")
                if m.vdim != m.dim:
                    raise ConfigError(f"{mw}: the keys are the values, so vdim must equal dim")
                if m.window < 0:
                    raise ConfigError(f"{mw}: mask.size must not be negative")
            f = layer.mlp
            fw = f"layers[{i}].mlp"
            if f is not None and f.ff <= 0:
                raise ConfigError(f"{fw}: ff must be positive")
            if f is not None and f.kind == "moe":
                if f.experts < 0 or f.identity < 0 or not 1 <= f.top <= f.experts + f.identity or not f.limit > 0:
                    raise ConfigError(f"{fw}: top must lie between 1 and experts + identity, limit be positive")
                if f.shared is not None and (f.shared.ff <= 0 or not f.shared.limit > 0):
                    raise ConfigError(f"{fw}.shared: ff and limit must be positive")
        lp = self.loop
        if lp is not None and not (0 <= lp.start < lp.stop <= len(self.layers) and lp.times >= 1):
            raise ConfigError("loop: 0 <= start < stop <= number of layers, times at least 1")

    def run_order(self) -> List[Tuple[int, bool]]:
        """(layer, whether the embedding output is added to the stream right before it) in the order of a pass."""
        n = len(self.layers)
        lp = self.loop
        if lp is None:
            return [(i, False) for i in range(n)]
        order = [(i, False) for i in range(lp.start)]
        for rep in range(lp.times):
            order += [(i, rep > 0 and i == lp.start) for i in range(lp.start, lp.stop)]
        return order + [(i, False) for i in range(lp.stop, n)]

    def to_hf(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "latent_attention":
                mixer: Dict[str, Any] = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                                         "kv_rank": m.kv_rank, "scale": m.scale,
                                         "rot": {"base": m.rot.base, "dims": m.rot.dims}}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                         "mask": {"size": m.window}}
            f = layer.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.ff, "limit": f.limit},
                       "router": {"experts": f.experts, "identity": f.identity, "top": f.top, "scale": f.scale}}
                if f.shared is not None:
                    mlp["shared"] = {"ff": f.shared.ff, "limit": f.shared.limit}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        out: Dict[str, Any] = {"architecture": "Venezen", "vocab": self.vocab_size, "width": self.hidden_size,
                               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                               "layers": layers}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.bos_token_id >= 0:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
