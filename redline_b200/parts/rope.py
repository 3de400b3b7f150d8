"""Rotary position encoding: inverse frequencies with none / linear / llama3
scaling in double precision, angle = float32(pos) * float32(inv_freq) formed in
float32, pairs (i, i + D/2) rotated (reference: src/core/model_config.cpp:126-169,
src/cuda/kernels/rope_kv.cu:26-51).  ``NoPosition`` is the encoding that does
nothing."""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch

from ..config.model_config import RopeScaling
from .base import PositionEncoding, register


@dataclass(frozen=True)
class RotaryParams:
    head_dim: int
    theta: float
    scaling: RopeScaling
    max_positions: int


def rope_inv_freq(head_dim: int, theta: float, scaling: RopeScaling) -> List[float]:
    half = head_dim // 2
    inv = [theta ** (-(2.0 * i) / head_dim) for i in range(half)]
    if scaling.type == "linear":
        return [f / scaling.factor for f in inv]
    if scaling.type == "llama3":
        orig = float(scaling.original_max_position_embeddings)
        long_wave = orig / scaling.low_freq_factor    # longer than this: fully scaled
        short_wave = orig / scaling.high_freq_factor  # shorter than this: untouched
        span = scaling.high_freq_factor - scaling.low_freq_factor
        scaled = []
        for f in inv:
            wave = 2.0 * math.pi / f
            if wave < short_wave:
                scaled.append(f)
            elif wave > long_wave:
                scaled.append(f / scaling.factor)
            else:
                t = (orig / wave - scaling.low_freq_factor) / span
                scaled.append((1.0 - t) * f / scaling.factor + t * f)
        return scaled
    return inv


def rope_tables(params: RotaryParams, num_positions: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos, sin [num_positions, D/2] float32 on the CPU."""
    inv = np.asarray(rope_inv_freq(params.head_dim, params.theta, params.scaling), dtype=np.float64)
    angle = np.arange(num_positions, dtype=np.float32)[:, None] * inv.astype(np.float32)[None, :]
    angle = angle.astype(np.float32).astype(np.float64)
    return (torch.from_numpy(np.cos(angle).astype(np.float32)),
            torch.from_numpy(np.sin(angle).astype(np.float32)))


@register("position", "rope")
class RotaryPosition(PositionEncoding):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        n = min(self.params.max_positions, rt.max_seq_len) if rt.max_seq_len > 0 else self.params.max_positions
        cos, sin = rope_tables(self.params, max(n, 1))
        self.cos = cos.to(rt.device)
        self.sin = sin.to(rt.device)

    def rotary_tables(self):
        return self.cos, self.sin

    def nbytes(self) -> int:
        return 2 * self.cos.numel() * 4


@register("position", "none")
class NoPosition(PositionEncoding):
    pass


@dataclass(frozen=True)
class RotaryPairsParams:
    dims: int              # how many entries of a head are rotated: the first ``dims`` (an even number)
    base: float
    max_positions: int


_pair_tables = {}          # tables shared by the parts that ask for the same ones


@register("position", "rope_pairs")
class RotaryPairs(PositionEncoding):
    """Rotation of neighbouring pairs: entries (2i, 2i+1), i < dims / 2, of a head turn by the angle
    pos * base^(-2i / dims); the entries from ``dims`` on stay as they are.  The tables hold the cosines and
    sines [positions, dims / 2] in float32 of angles formed in double precision; the mixer applies them."""

    pairing = "neighbours"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        if p.dims <= 0 or p.dims % 2 != 0:
            raise ValueError(f"rope_pairs rotates an even number of entries, got {p.dims}")
        n = max(min(p.max_positions, rt.max_seq_len) if rt.max_seq_len > 0 else p.max_positions, 1)
        key = (p.dims, float(p.base), n, str(rt.device))
        if key not in _pair_tables:
            freq = np.asarray([float(p.base) ** (-2.0 * i / p.dims) for i in range(p.dims // 2)], dtype=np.float64)
            angle = np.arange(n, dtype=np.float64)[:, None] * freq[None, :]
            _pair_tables[key] = (torch.from_numpy(np.cos(angle).astype(np.float32)).to(rt.device),
                                 torch.from_numpy(np.sin(angle).astype(np.float32)).to(rt.device))
        self.cos, self.sin = _pair_tables[key]

    def rotary_tables(self):
        return self.cos, self.sin

    def nbytes(self) -> int:
        return 2 * self.cos.numel() * 4


@dataclass(frozen=True)
class RotaryHalvesParams:
    """Rotation of the first ``dims`` entries of a head, entry i paired with entry i + dims / 2, with optional
    YaRN scaling of the frequencies (``factor`` 0 or 1: none)."""

    dims: int
    base: float
    max_positions: int
    factor: float = 0.0        # YaRN: how far the context is stretched
    original: int = 0          # the context length the frequencies were made for
    fast: float = 32.0         # pairs that turn at least so often within ``original`` keep their frequency
    slow: float = 1.0          # pairs that turn at most so often are divided by ``factor``


def yarn_frequencies(p: RotaryHalvesParams) -> Tuple[List[float], float]:
    """(frequency of every pair, factor on cos and sin).  With f_i = base^(-2i/dims) and
    index(turns) = dims ln(original / (2 pi turns)) / (2 ln base): lo = max(floor(index(fast)), 0),
    hi = min(ceil(index(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); pair i turns at
    f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are multiplied by 0.1 ln(factor) + 1."""
    half = p.dims // 2
    f = [float(p.base) ** (-2.0 * i / p.dims) for i in range(half)]
    if not p.factor or p.factor == 1.0:
        return f, 1.0

    def index(turns: float) -> float:
        return p.dims * math.log(p.original / (2.0 * math.pi * turns)) / (2.0 * math.log(p.base))

    lo = max(math.floor(index(p.fast)), 0)
    hi = min(math.ceil(index(p.slow)), p.dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / p.factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(p.factor) + 1.0


_half_tables = {}


@register("position", "rope_halves")
class RotaryHalves(PositionEncoding):
    """Tables [positions, dims / 2] of cos and sin (float32 of angles formed in double precision, the YaRN
    factor multiplied in); the mixer's kernel pairs entry i with entry i + dims / 2."""

    pairing = "halves"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        if p.dims <= 0 or p.dims % 2 != 0:
            raise ValueError(f"rope_halves rotates an even number of entries, got {p.dims}")
        if p.factor and p.factor != 1.0 and (p.factor < 0 or p.original <= 0 or p.fast <= 0 or p.slow <= 0 or p.base <= 1):
            raise ValueError("rope_halves: a scaling needs positive factor, original, fast and slow and a base above 1")
        n = max(min(p.max_positions, rt.max_seq_len) if rt.max_seq_len > 0 else p.max_positions, 1)
        key = (p, n, str(rt.device))
        if key not in _half_tables:
            freq, mag = yarn_frequencies(p)
            angle = np.arange(n, dtype=np.float64)[:, None] * np.asarray(freq, dtype=np.float64)[None, :]
            _half_tables[key] = (torch.from_numpy((np.cos(angle) * mag).astype(np.float32)).to(rt.device),
                                 torch.from_numpy((np.sin(angle) * mag).astype(np.float32)).to(rt.device))
        self.cos, self.sin = _half_tables[key]

    def rotary_tables(self):
        return self.cos, self.sin

    def nbytes(self) -> int:
        return 2 * self.cos.numel() * 4
