"""Helpers of the Venezen GPU tests: model folders, engines, comparisons with the plain implementation."""

from __future__ import annotations

import os
from typing import Dict, Optional, Sequence

import numpy as np
import torch

import plain_venezen as P
from gpu_utils import F32_REL, rel_max


def make_model(tmp, cfg: dict, seed: int, sharpen: float = 2.0, patch=None):
    """Writes a model folder with seeded weights; returns (folder, weights as float32 values bfloat16 holds)."""
    w = P.random_weights(cfg, seed, sharpen)
    if patch is not None:
        patch(w)
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    d = os.path.join(str(tmp), f"venezen_{seed}_{abs(hash(str(cfg))) % 10**8}")
    P.write_model_dir(d, cfg, w)
    return d, w


def engine_for(model_dir: str, dtype: str, **kw):
    from redline_b200.engine.engine import Engine
    opts = dict(dtype=dtype, kv_cache_tokens=1024, max_seq_len=1024, max_num_seqs=4, max_num_batched_tokens=512,
                max_logit_rows=512, cuda_graphs=False, async_scheduling=False)
    opts.update(kw)
    return Engine(model_dir, **opts)


def oracle(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], rounded: Optional[torch.dtype] = None) -> np.ndarray:
    P.STORE_DTYPE = rounded
    try:
        return P.forward(cfg, w, list(tokens)).numpy()
    finally:
        P.STORE_DTYPE = None


class Reference:
    """The plain implementation's logits of a sequence: exact (float64), and for a 16-bit engine also with
    everything rounded that such an engine stores in 16 bits.  ``noise32`` (made when first asked for) is
    what the plain implementation run in float32 differs by from itself in float64, per row and relative to
    the largest logit: how much a row amplifies rounding."""

    def __init__(self, cfg: dict, w, tokens: Sequence[int], dtype: str):
        self.cfg, self.w, self.tokens = cfg, w, list(tokens)
        self.exact = oracle(cfg, w, tokens)
        self.rounded = oracle(cfg, w, tokens, torch.bfloat16) if dtype != "float32" else None
        self.main = self.exact if self.rounded is None else self.rounded
        self._noise32 = None

    @property
    def noise32(self) -> np.ndarray:
        if self._noise32 is None:
            P.F64 = torch.float32
            try:
                low = P.forward(self.cfg, self.w, self.tokens).double().numpy()
            finally:
                P.F64 = torch.float64
            self._noise32 = np.abs(low - self.exact).max(axis=1) / (np.abs(self.exact).max() + 1e-30)
        return self._noise32


def row_rms(d: np.ndarray) -> np.ndarray:
    d = d - d.mean(axis=-1, keepdims=True)
    return np.sqrt((d * d).mean(axis=-1))


# A 16-bit engine against the exact logits: a row may be off by up to this many times what rounding alone
# does to the plain implementation on the same sequence (its worst calm row).  Faults of logic (a key one
# position off, a lost state, a sink left out) are tens of times larger and show in every row behind them,
# and the 32-bit runs hold them to 1e-4.
#
# A model may have positions that amplify rounding far beyond their neighbours (a router's choice that two
# outputs almost tie for, a softmax between near-equal scores behind sharp weights).  Such rows are told from the
# plain implementation itself, which run in float32 differs there from its float64 self by more than SENSITIVE
# times the median row; they are left out of the 16-bit comparison (there may be few), and in the 32-bit
# comparison they get 3 times their own float32 noise.  Of the other rows of a 16-bit run at most 1 in 100 (one,
# from 50 rows on) may exceed the limit, none by more than 8 times.
BF16_NOISE_FACTOR = 3.0
SENSITIVE = 8.0
MOST_SENSITIVE_ROWS = 0.08

_model_noise: Dict[int, float] = {}


def model_noise(cfg: dict, w) -> float:
    """What rounding alone does to the plain implementation's logits on a 64-token sequence of this model
    (the row at the 90th percentile): the floor under the level of a short sequence, whose own rows are a poor
    estimate."""
    key = id(w)
    if key not in _model_noise:
        toks = np.random.RandomState(0).randint(0, cfg["vocab"], size=64).tolist()
        _model_noise[key] = float(np.percentile(row_rms(oracle(cfg, w, toks, torch.bfloat16) - oracle(cfg, w, toks)), 90))
    return _model_noise[key]


def check(got: np.ndarray, cfg: dict, w, tokens: Sequence[int], dtype: str, rows=None, ref: Optional[Reference] = None) -> float:
    """float32: every row's largest difference from the exact logits below 1e-4 of the largest logit (3 times
    the row's own float32 noise where that is more).  bfloat16: every calm row's error (root mean square, mean
    removed) against the exact logits within BF16_NOISE_FACTOR times the rounding error of the plain
    implementation itself (see above)."""
    rows = list(range(len(tokens))) if rows is None else list(rows)
    ref = ref or Reference(cfg, w, tokens, dtype)
    if dtype == "float32":
        want = ref.exact[rows]
        err = np.abs(got - want).max(axis=1) / (np.abs(ref.exact).max() + 1e-30)
        if (err >= F32_REL).any():
            limit = np.maximum(F32_REL, 3.0 * ref.noise32[rows])
            worst = int((err / limit).argmax())
            assert err[worst] < limit[worst], (f"float32 logits differ: row {rows[worst]} by {err[worst]:.3e} of the largest "
                                               f"logit; the plain implementation's own float32 noise there is "
                                               f"{ref.noise32[rows[worst]]:.3e}")
        return float(err.max())
    sens = ref.noise32
    calm_all = sens <= SENSITIVE * np.median(sens)
    assert (~calm_all).sum() <= max(1, MOST_SENSITIVE_ROWS * len(sens)), "too many rows amplify rounding: a poor test sequence"
    own = row_rms(ref.rounded - ref.exact)
    level = max(float(own[calm_all].max()) if calm_all.any() else 0.0, model_noise(cfg, w))
    err = row_rms(got - ref.exact[rows])
    calm = calm_all[rows]
    over = calm & (err > BF16_NOISE_FACTOR * level)
    far = calm & (err > 8 * BF16_NOISE_FACTOR * level)
    allowed = 0 if calm.sum() < 50 else max(1, int(calm.sum()) // 100)
    worst = int(np.where(calm, err, 0.0).argmax())
    assert not far.any() and over.sum() <= allowed, (
        f"bfloat16 logits differ: {int(over.sum())} calm rows of {int(calm.sum())} are over the limit, row {rows[worst]} "
        f"by {err[worst]:.3e}; rounding alone gives {level:.3e}")
    return float(err[worst] / level)
