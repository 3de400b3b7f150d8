"""Plain, slow implementation of the Vizotar decoder: the oracle of its tests.

Whole sequences, no cache, no batching, float64, one function per mechanism.  It shares no code with
``redline_b200``: it reads the configuration dictionary itself, draws its own random weights and writes
its own safetensors file.

The model in this file's notation (W applied as W x; N(x, w) = x / sqrt(mean(x^2) + eps) * w):

  embedding   e = table[token]; the n = ``streams`` streams X_1 .. X_n all start as e
  sublayer    (mixer, then feed-forward, each with tensors in, out [n] and mix [n, n]):
              u = sum_s in[s] X_s;  y = sublayer(N(u, norm));  X_t <- sum_s mix[s, t] X_s + out[t] y  (all t at once)
  a layer with ``weights_of: j`` uses layer j's tensors and keeps caches and states of its own
  parallel    0.5 * (N(left(h), left.out) + N(right(h), right.out))
    left      q, k, v projections with biases; a causal convolution over time on every channel of each
              (taps weights, the last one on the current token, zeros before the sequence); q and k RMS-normed
              over the whole projection with weights; the first rot.dims entries of every head rotated, entry i
              paired with i + dims/2, by the angle pos * f_i, frequencies blended between f_i and f_i / factor by a
              ramp over the pair index, cos and sin times 0.1 ln(factor) + 1; s = scale q.k inside a sliding
              window; exp(sink_h) joins the softmax's denominator; output projection with a bias
    right     matrix memory with exponential gates: q = W_q h / sqrt(dim), k, v; i = cap tanh((W_i h + b_i)/cap),
              f = logsigmoid(cap tanh((W_f h + b_f)/cap)); m_t = max(f + m_(t-1), i), m_0 = 0;
              S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T, n_t likewise with k;
              o = S_t^T q / (max(|n_t.q|, exp(-m_t)) + 1e-6); o divided by its root mean square per head, times a
              weight over all heads, times sigmoid(W_g h); output projection
  channel_delta   q, k (kv_heads x dim), v (heads x vdim): projection, causal convolution, SiLU; q and k made unit
              vectors per head (x / sqrt(sum x^2 + 1e-6)), q times dim^(-1/2); beta = sigmoid(W_b h) per head;
              decay per head and key channel a = exp(-exp(A_log_h) softplus(W_a2 W_a1 h + dt_bias));
              S <- diag(a) S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T q;
              o RMS-normed per head with one weight of vdim, times sigmoid(W_g2 W_g1 h); output projection
  dense ff    g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))
  routed ff   logits W_r h + b_r; the ``top`` largest are chosen, weights = softmax over the chosen logits;
              sum of weight * W_down (silu(W_gate h) * (W_up h)) over the chosen experts
  output      logits = table N(sum of the streams, final.norm)
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

F64 = torch.float64
DENOMINATOR_FLOOR = 1e-6        # added to the matrix memory's denominator
UNIT_FLOOR = 1e-6               # under the root of the delta rule's unit vectors
GLU_SLOPE = 1.702               # of the dense feed-forward's sigmoid

# When set to a 16-bit type, what a 16-bit engine stores in that type is rounded here as well (the
# sublayers' inputs, projections, convolutions and activations, cached keys and values, sublayer outputs);
# the streams, scores, states, gates of the recurrences and the norms' arithmetic stay double.
STORE_DTYPE: Optional[torch.dtype] = None


def stored(x: torch.Tensor) -> torch.Tensor:
    return x if STORE_DTYPE is None else x.to(STORE_DTYPE).to(F64)


# ------------------------------------------------------------------ small pieces

def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -(torch.clamp(-z, min=0.0) + torch.log1p(torch.exp(-z.abs())))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) + torch.log1p(torch.exp(-z.abs()))


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the sequence."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def scaled_frequencies(rot: dict) -> (List[float], float):
    """The rotation's frequencies per pair index and the factor on cos and sin."""
    dims, base = rot["dims"], float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def index_of(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_halves(x: torch.Tensor, rot: dict, first: int = 0) -> torch.Tensor:
    """x [T, heads, size]: entry i < dims/2 of every head is paired with entry i + dims/2."""
    T = x.shape[0]
    dims = rot["dims"]
    half = dims // 2
    freq, mag = scaled_frequencies(rot)
    out = x.clone()
    pos = torch.arange(first, first + T, dtype=F64)
    for i in range(half):
        a = pos * freq[i]
        c, s = (torch.cos(a) * mag)[:, None], (torch.sin(a) * mag)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def window_sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int,
                          sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, DV] -> [T, H, DV].  Token i sees j when 0 <= i - j < window (every
    earlier token if window <= 0); ``sink`` [H] adds exp(sink_h) to head h's denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = 0 if window <= 0 else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            mx = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - mx)
            den = e.sum() if sink is None else e.sum() + torch.exp(sink[h] - mx)
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def matrix_memory(q, k, v, ig, fg):
    """q, k [T, D], v [T, DV], ig, fg [T] (logarithms of the gates) -> o [T, DV]; state from zero, m_0 = 0."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=q.dtype)
    n = torch.zeros(D, dtype=q.dtype)
    m = torch.zeros((), dtype=q.dtype)
    out = []
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a, b = torch.exp(fg[t] + m - m_new), torch.exp(ig[t] - m_new)
        S = a * S + b * torch.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        den = torch.maximum((n @ q[t]).abs(), torch.exp(-m)) + DENOMINATOR_FLOOR
        out.append((S.T @ q[t]) / den)
    return torch.stack(out)


def gated_delta(q, k, v, beta, decay):
    """q, k [T, D] (unit vectors, q scaled), v [T, DV], beta [T], decay [T, D] -> o [T, DV]; S from zero."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = decay[t][:, None] * S
        d = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], d)
        out.append(S.T @ q[t])
    return torch.stack(out)


# ------------------------------------------------------------------ mixers

def left_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, D, DV = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    proj = {}
    for n in ("q", "k", "v"):
        u = stored(h @ w[p + n].T + w[p + n + ".b"])
        proj[n] = stored(causal_conv(u, w[p + n + ".conv"])) if m.get("conv") else u
    q = rms_norm(proj["q"], w[p + "q.norm"], eps).view(T, H, D)
    k = rms_norm(proj["k"], w[p + "k.norm"], eps).view(T, G, D)
    v = proj["v"].view(T, G, DV)
    if m.get("rot"):
        q, k = rotate_halves(q, m["rot"]), rotate_halves(k, m["rot"])
    q, k = stored(q), stored(k)
    o = window_sink_attention(q, k, v, m["scale"], (m.get("mask") or {}).get("size", 0), w[p + "sink"])
    return stored(stored(o.reshape(T, H * DV)) @ w[p + "o"].T + w[p + "o.b"])


def right_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    cap = m["gate_cap"]
    q = stored(h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = stored(h @ w[p + "k"].T).view(T, H, D)
    v = stored(h @ w[p + "v"].T).view(T, H, DV)
    ig = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    fg = log_sigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    o = torch.stack([matrix_memory(q[:, x], k[:, x], v[:, x], ig[:, x], fg[:, x]) for x in range(H)], dim=1)
    o = rms_norm(o, None, eps).reshape(T, H * DV) * w[p + "norm"] * sigmoid(stored(h @ w[p + "g"].T))
    return stored(stored(o) @ w[p + "o"].T)


def parallel_mixer(h, w, p, m, eps):
    a = rms_norm(left_mixer(h, w, p + "left.", m["left"], eps), w[p + "left.out"], eps)
    b = rms_norm(right_mixer(h, w, p + "right.", m["right"], eps), w[p + "right.out"], eps)
    return 0.5 * (a + b)


def channel_delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, D, DV = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]

    def branch(n):
        return stored(silu(stored(causal_conv(stored(h @ w[p + n].T), w[p + n + ".conv"]))))

    q, k, v = branch("q").view(T, G, D), branch("k").view(T, G, D), branch("v").view(T, H, DV)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + UNIT_FLOOR) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + UNIT_FLOOR)
    beta = sigmoid(h @ w[p + "b"].T)                                                   # [T, H]
    dt = softplus(stored(h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, D)
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * dt)
    per = H // G
    o = torch.stack([gated_delta(q[:, x // per], k[:, x // per], v[:, x], beta[:, x], decay[:, x]) for x in range(H)], dim=1)
    gate = sigmoid(stored(stored(h @ w[p + "g1"].T) @ w[p + "g2"].T)).view(T, H, DV)
    o = rms_norm(o, w[p + "norm"], eps) * gate
    return stored(stored(o.reshape(T, H * DV)) @ w[p + "o"].T)


# ------------------------------------------------------------------ feed-forwards

def dense_ff(h, w, p, f):
    limit = f["limit"]
    g = torch.clamp(stored(h @ w[p + "gate"].T), max=limit)
    u = torch.clamp(stored(h @ w[p + "up"].T), min=-limit, max=limit)
    return stored(stored(g * sigmoid(GLU_SLOPE * g) * (u + 1.0)) @ w[p + "down"].T)


def route(h, w, p, f):
    """(chosen experts [T, top], their weights [T, top])."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    top = f["router"]["top"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def routed_ff(h, w, p, f):
    idx, wt = route(h, w, p, f)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = f"{p}e{int(idx[t, j])}."
            a = stored(silu(stored(w[e + "gate"] @ h[t])) * stored(w[e + "up"] @ h[t]))
            out[t] += wt[t, j] * stored(w[e + "down"] @ a)
    return stored(out)


# ------------------------------------------------------------------ the model

def weights_layer(cfg: dict, i: int) -> int:
    j = cfg["layers"][i].get("weights_of")
    return i if j is None else int(j)


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[list] = None
            ) -> torch.Tensor:
    """Logits [tokens, vocab] of one whole sequence.  ``layers_out`` receives the sum of the streams after
    every layer."""
    w = {k: v.to(F64) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    n = int(cfg.get("streams", 1))
    e = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    X = [e.clone() for _ in range(n)]

    def sublayer(X, hc, norm, fn):
        u = sum(w[hc + "in"][s] * X[s] for s in range(n))
        y = fn(stored(rms_norm(u, w[norm], eps)))
        return [sum(w[hc + "mix"][s, t] * X[s] for s in range(n)) + w[hc + "out"][t] * y for t in range(n)]

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{weights_layer(cfg, i)}."
        m = layer["mixer"]
        if layer["type"] == "parallel":
            X = sublayer(X, p + "hc1.", p + "norm1", lambda h: parallel_mixer(h, w, p + "mix.", m, eps))
        elif layer["type"] == "channel_delta":
            X = sublayer(X, p + "hc1.", p + "norm1", lambda h: channel_delta_mixer(h, w, p + "mix.", m, eps))
        else:
            raise ValueError(f"layer type {layer['type']}")
        f = layer.get("mlp")
        if f is not None:
            fn = dense_ff if f["kind"] == "dense" else routed_ff
            X = sublayer(X, p + "hc2.", p + "norm2", lambda h: fn(h, w, p + "mlp.", f))
        if layers_out is not None:
            layers_out.append(sum(X))
    return stored(rms_norm(sum(X), w["final.norm"], eps)) @ w["embed"].T


# ------------------------------------------------------------------ weights and files

def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W = cfg["width"]
    n = int(cfg.get("streams", 1))
    out: Dict[str, tuple] = {"embed": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p = f"l{i}."
        m = layer["mixer"]
        out[p + "norm1"] = (W,)
        if layer["type"] == "parallel":
            l, r = m["left"], m["right"]
            H, G, D, DV = l["heads"], l.get("kv_heads") or l["heads"], l["dim"], l["vdim"]
            q = p + "mix.left."
            for name, rows in (("q", H * D), ("k", G * D), ("v", G * DV)):
                out[q + name] = (rows, W)
                out[q + name + ".b"] = (rows,)
                if l.get("conv"):
                    out[q + name + ".conv"] = (rows, l["conv"])
            out.update({q + "q.norm": (H * D,), q + "k.norm": (G * D,), q + "sink": (H,), q + "o": (W, H * DV),
                        q + "o.b": (W,)})
            H, D, DV = r["heads"], r["dim"], r["vdim"]
            q = p + "mix.right."
            out.update({q + "q": (H * D, W), q + "k": (H * D, W), q + "v": (H * DV, W), q + "g": (H * DV, W),
                        q + "o": (W, H * DV), q + "norm": (H * DV,), q + "i": (H, W), q + "i.b": (H,),
                        q + "f": (H, W), q + "f.b": (H,)})
            out.update({p + "mix.left.out": (W,), p + "mix.right.out": (W,)})
        else:
            H, G, D, DV = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
            q = p + "mix."
            rank_a, rank_g = m.get("_rank_a", 8), m.get("_rank_g", 8)
            for name, rows in (("q", G * D), ("k", G * D), ("v", H * DV)):
                out[q + name] = (rows, W)
                out[q + name + ".conv"] = (rows, m["conv"])
            out.update({q + "b": (H, W), q + "A_log": (H,), q + "norm": (DV,), q + "a1": (rank_a, W),
                        q + "a2": (H * D, rank_a), q + "dt_bias": (H * D,), q + "g1": (rank_g, W),
                        q + "g2": (H * DV, rank_g), q + "o": (W, H * DV)})
        f = layer.get("mlp")
        if f is not None:
            out[p + "norm2"] = (W,)
            if f["kind"] == "dense":
                out.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
            else:
                ff = f["expert"]["ff"]
                for e in range(f["router"]["experts"]):
                    out.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
                out.update({p + "mlp.router": (f["router"]["experts"], W), p + "mlp.router.b": (f["router"]["experts"],)})
        for q in ("hc1.",) + (("hc2.",) if f is not None else ()):
            out.update({p + q + "in": (n,), p + q + "out": (n,), p + q + "mix": (n, n)})
    out["final.norm"] = (W,)
    return out


def random_weights(cfg: dict, seed: int, sharpen: float = 2.0) -> Dict[str, torch.Tensor]:
    """Seeded weights as the float32 values that bfloat16 holds.  Matrices N(0, 1 / fan_in); the norms of queries
    and keys ``sharpen`` times larger so that attention is not flat; the streams' mixing matrices near the
    identity, their read-in weights near 1 / streams and their write-out weights near 1."""
    g = torch.Generator().manual_seed(seed)
    n = int(cfg.get("streams", 1))
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        r = lambda: torch.randn(shape, generator=g)
        if name.endswith(("q.norm", "k.norm")):
            t = math.sqrt(sharpen) * (1.0 + 0.1 * r())
        elif last in ("norm1", "norm2", "norm") or name.endswith(("final.norm", "left.out", "right.out")):
            t = 1.0 + 0.1 * r()
        elif last == "conv":
            t = r() * 0.5
        elif last == "sink":
            t = r()
        elif name.endswith(("i.b", "router.b")):
            t = r()
        elif name.endswith("f.b"):
            t = 2.0 + r()
        elif last == "b" and len(shape) == 1:
            t = 0.3 * r()
        elif last == "A_log":
            t = -1.0 + 0.5 * r()
        elif last == "dt_bias":
            t = -1.0 + r()
        elif last == "in":
            t = (1.0 + 0.2 * r()) / n
        elif last == "out":
            t = 1.0 + 0.2 * r()
        elif last == "mix":
            t = torch.eye(n) + 0.15 * r()
        elif name == "embed":
            t = r()
        else:
            t = r() / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).float()
    return out


def write_model_dir(path: str, cfg: dict, weights: Dict[str, torch.Tensor], dtype=torch.bfloat16) -> None:
    """config.json and model.safetensors (8-byte length, JSON header, raw data), written by hand."""
    os.makedirs(path, exist_ok=True)
    clean = json.loads(json.dumps(cfg))
    for layer in clean["layers"]:
        for key in [k for k in layer["mixer"] if k.startswith("_")]:
            del layer["mixer"][key]
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(clean, f)
    code = {torch.bfloat16: "BF16", torch.float32: "F32"}[dtype]
    header, blobs, off = {}, [], 0
    for name, t in weights.items():
        raw = t.to(dtype).contiguous()
        data = raw.reshape(-1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": code, "shape": list(t.shape), "data_offsets": [off, off + len(data)]}
        blobs.append(data)
        off += len(data)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def read_model_dir(path: str):
    """(cfg, weights as float32) of a folder written by ``write_model_dir`` or any file of that format."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        buf = bytearray(data[a:b])
        if e["dtype"] == "BF16":
            t = torch.frombuffer(buf, dtype=torch.bfloat16).float()
        elif e["dtype"] == "F32":
            t = torch.frombuffer(buf, dtype=torch.float32).clone()
        elif e["dtype"] == "I32":
            t = torch.frombuffer(buf, dtype=torch.int32).clone()
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = t.reshape(e["shape"])
    return cfg, out
