"""A plain, slow implementation of the Venezen decoder, one function per mechanism, in float64 on whole
sequences (every token sees the full score matrix; no cache, no portions).  It shares no code with the
package: it reads the configuration dictionary itself, makes its own random weights and writes and reads
its own safetensors files.  The GPU tests hold the engine to it.

Notation.  A linear map W is stored [out, in] and applied as W x.  x_t is the residual stream at token t
(position t, counted from 0).

    x_t = s_E * E[token_t]                                    (e_t, kept for the loop below)
    layer:  x += mixer(LN_1(x));  x += ff(LN_2(x))           LN(u) = (u - mean u) / sqrt(var u + eps) * w
    run order: layers [0, a), then layers [a, b) `times` times on the same tensors, then layers [b, L);
               before every pass over [a, b) but the first, x_t += e_t
    logits = E LN_f(x)

    latent attention (H heads):  q = W_q h laid out per head as [n | r] (n: `dim` entries, r: `rot_dim`);
        [c' | k_r] = W_dkv h;  c = c' / rms(c') * w_c;  q_r and k_r rotated by the position (k_r is one vector
        for all heads);  per head k_n = W_uk c, v = W_uv c;  s_ij = scale (q_n,i . k_n,j + q_r,i . k_r,j),
        j <= i;  softmax;  W_o on the joined heads.
    rotation of the first d entries of a vector, entry i with entry i + d/2: angle p * base^(-2i/d).
    windowed attention (H heads, G key heads, head h reads key head h // (H/G)):  q = W_q h, k = W_k h, the
        values ARE the keys;  s_ij = scale q_i . k_j - m_h (i - j) for 0 <= i - j < size,
        m_h = 2^(-8 (h + 1) / H);  weights exp(s_ij) / (1 + sum_j exp(s_ij));  W_o on the joined heads.
    dense feed-forward:  W_d (silu(W_g h + b_g) * (W_u h + b_u)) + b_d.
    expert:  g = min(W_g h, l), u = clamp(W_u h, -l, l), W_d (g sigmoid(1.702 g) (u + 1)).
    routed feed-forward with n experts and i identity experts:  z = W_r h (n + i numbers), s = softmax(z);
        the `top` largest of s + correction are chosen;  their weights are s / (sum of the chosen s + 1e-20)
        * router scale;  a chosen index >= n stands for the identity (its output is h);  the result is the
        weighted sum plus a shared expert (same form, its own width and limit) that every token runs.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

F64 = torch.float64
STORE_DTYPE: Optional[torch.dtype] = None     # set to torch.bfloat16: round what a 16-bit engine stores in 16 bits

SWISH_SLOPE = 1.702
WEIGHT_FLOOR = 1e-20


def stored(x: torch.Tensor) -> torch.Tensor:
    if STORE_DTYPE is None:
        return x
    return x.to(STORE_DTYPE).to(F64)


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def rotate_halves(x: torch.Tensor, base: float, dims: int, positions: Sequence[int]) -> torch.Tensor:
    """x [T, ..., n]: the first ``dims`` entries of the last axis turned by the token's position, entry i
    with entry i + dims/2; the rest unchanged."""
    half = dims // 2
    out = x.clone()
    if half == 0:
        return out
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = torch.tensor(list(positions), dtype=torch.float64)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).to(x.dtype).view(shape), torch.sin(ang).to(x.dtype).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def causal_softmax(s: torch.Tensor) -> torch.Tensor:
    """s [T, T]: row i over j <= i."""
    T = s.shape[0]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, -math.inf)
    s = s - s.max(-1, keepdim=True).values
    e = torch.exp(s)
    return e / e.sum(-1, keepdim=True)


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                     positions: Sequence[int]) -> torch.Tensor:
    T = h.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    q = stored(h @ w[p + "q"].T).view(T, H, dn + dr)
    ckr = stored(h @ w[p + "dkv"].T)
    c = stored(rms_norm(ckr[:, :rank], w[p + "dkv.norm"], eps))
    kr = stored(rotate_halves(ckr[:, rank:], rot["base"], rot["dims"], positions))
    qn = q[:, :, :dn]
    qr = stored(rotate_halves(q[:, :, dn:], rot["base"], rot["dims"], positions))
    kn = stored(c @ w[p + "uk"].T).view(T, H, dn)
    v = stored(c @ w[p + "uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * m["scale"]
        out[:, hd] = causal_softmax(s) @ v[:, hd]
    return stored(stored(out.reshape(T, H * dv)) @ w[p + "o"].T)


def head_slopes(heads: int) -> List[float]:
    return [2.0 ** (-8.0 * (hd + 1) / heads) for hd in range(heads)]


def biased_window_weights(s: torch.Tensor, slope: float, size: int) -> torch.Tensor:
    """s [T, T] scaled scores -> the weights of a row over its window, with the distance taken off and a
    one added to the denominator."""
    T = s.shape[0]
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    dist = (i - j).to(F64)
    seen = (dist >= 0) & ((dist < size) if size > 0 else (dist >= 0))          # size 0: no window
    s = (s - slope * dist).masked_fill(~seen, -math.inf)
    mx = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)          # the added one is exp(0)
    e = torch.exp(s - mx)
    return e / (torch.exp(-mx) + e.sum(-1, keepdim=True))


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    assert m["vdim"] == d, "the values are the keys"
    q = stored(h @ w[p + "q"].T).view(T, H, d)
    k = stored(h @ w[p + "k"].T).view(T, G, d)
    slopes = head_slopes(H)
    out = torch.zeros(T, H, d, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        a = biased_window_weights(q[:, hd] @ k[:, g].T * m["scale"], slopes[hd], (m.get("mask") or {}).get("size", 0))
        out[:, hd] = a @ k[:, g]
    return stored(stored(out.reshape(T, H * d)) @ w[p + "o"].T)


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    g = stored(h @ w[p + "gate"].T + w[p + "gate.b"])
    u = stored(h @ w[p + "up"].T + w[p + "up.b"])
    return stored(stored(g * sigmoid(g) * u) @ w[p + "down"].T + w[p + "down.b"])


def clamped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(stored(h @ gate.T), max=limit)
    u = torch.clamp(stored(h @ up.T), min=-limit, max=limit)
    return stored(stored(g * sigmoid(SWISH_SLOPE * g) * (u + 1.0)) @ down.T)


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (chosen indices [T, top], their weights [T, top]); an index >= experts is an identity expert."""
    r = f["router"]
    z = h @ w[p + "router"].T
    s = torch.softmax(z, dim=-1)
    pick = torch.topk(s + w[p + "correction"], r["top"], dim=-1).indices
    chosen = torch.gather(s, 1, pick)
    return pick, chosen / (chosen.sum(-1, keepdim=True) + WEIGHT_FLOOR) * r["scale"]


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    r = f["router"]
    pick, weight = route(h, w, p, f)
    out = torch.zeros_like(h)
    for e in range(r["experts"] + r["identity"]):
        hit = pick == e                                   # [T, top]: which tokens chose output e, and where
        rows = hit.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        if e >= r["experts"]:
            y = h[rows]
        else:
            y = clamped_expert(h[rows], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], f["expert"]["limit"])
        out[rows] += (weight[rows] * hit[rows]).sum(-1, keepdim=True) * y
    if f.get("shared") is not None:
        out = out + clamped_expert(h, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"], f["shared"]["limit"])
    return stored(out)


def run_order(cfg: dict) -> List[Tuple[int, bool]]:
    """(layer, whether the embedding output is added before it) in the order the layers run."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if loop is None:
        return [(i, False) for i in range(L)]
    a, b, n = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for rep in range(n):
        order += [(i, rep > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, L)]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[list] = None,
            first_pos: int = 0) -> torch.Tensor:
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    positions = [first_pos + t for t in range(len(tokens))]
    e = w["embed"][list(tokens)] * cfg["embedding"]["scale"]
    x = e.clone()
    for i, add in run_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        if add:
            x = x + e
        h = stored(layer_norm(x, w[p + "norm1"], eps))
        if layer["type"] == "latent_attention":
            x = x + latent_attention(h, w, p + "mix.", layer["mixer"], eps, positions)
        elif layer["type"] == "attention":
            x = x + window_attention(h, w, p + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        f = layer.get("mlp")
        if f is not None:
            h = stored(layer_norm(x, w[p + "norm2"], eps))
            x = x + (dense_ff(h, w, p + "mlp.") if f["kind"] == "dense" else routed_ff(h, w, p + "mlp.", f))
        if layers_out is not None:
            layers_out.append(x.clone())
    return stored(layer_norm(x, w["final.norm"], eps)) @ w["embed"].T


# ---------------------------------------------------------------------------------------- files and weights

def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W = cfg["width"]
    out: Dict[str, tuple] = {"embed": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        out[p + "norm1"] = (W,)
        if layer["type"] == "latent_attention":
            H = m["heads"]
            out[p + "mix.q"] = (H * (m["dim"] + m["rot_dim"]), W)
            out[p + "mix.dkv"] = (m["kv_rank"] + m["rot_dim"], W)
            out[p + "mix.dkv.norm"] = (m["kv_rank"],)
            out[p + "mix.uk"] = (H * m["dim"], m["kv_rank"])
            out[p + "mix.uv"] = (H * m["vdim"], m["kv_rank"])
            out[p + "mix.o"] = (W, H * m["vdim"])
        else:
            out[p + "mix.q"] = (m["heads"] * m["dim"], W)
            out[p + "mix.k"] = (m["kv_heads"] * m["dim"], W)
            out[p + "mix.o"] = (W, m["heads"] * m["vdim"])
        f = layer.get("mlp")
        if f is None:
            continue
        out[p + "norm2"] = (W,)
        if f["kind"] == "dense":
            for n, shape in (("gate", (f["ff"], W)), ("up", (f["ff"], W)), ("down", (W, f["ff"]))):
                out[p + "mlp." + n] = shape
                out[p + "mlp." + n + ".b"] = (shape[0],)
        else:
            r = f["router"]
            for e in range(r["experts"]):
                out[f"{p}mlp.e{e}.gate"] = (f["expert"]["ff"], W)
                out[f"{p}mlp.e{e}.up"] = (f["expert"]["ff"], W)
                out[f"{p}mlp.e{e}.down"] = (W, f["expert"]["ff"])
            out[p + "mlp.router"] = (r["experts"] + r["identity"], W)
            out[p + "mlp.correction"] = (r["experts"] + r["identity"],)
            if f.get("shared") is not None:
                out[p + "mlp.shared.gate"] = (f["shared"]["ff"], W)
                out[p + "mlp.shared.up"] = (f["shared"]["ff"], W)
                out[p + "mlp.shared.down"] = (W, f["shared"]["ff"])
    out["final.norm"] = (W,)
    return out


def random_weights(cfg: dict, seed: int, sharpen: float = 2.0) -> Dict[str, torch.Tensor]:
    """Seeded weights as the float32 values that bfloat16 holds.  Matrices N(0, 1/fan_in) (queries and keys
    times ``sharpen``, so that attention is not flat), the embedding N(0, 1) / scale, norm weights around 1,
    biases and corrections small."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[1] if "." in name else name
        if name == "embed":
            t = torch.randn(shape, generator=g) / cfg["embedding"]["scale"]
        elif len(shape) == 1 and leaf.endswith(".b"):
            t = 0.1 * torch.randn(shape, generator=g)
        elif leaf == "mlp.correction":
            t = 0.02 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if leaf in ("mix.q", "mix.k", "mix.dkv", "mix.uk"):
                t = t * sharpen
            if leaf == "mlp.router":
                t = t * 2.0
        out[name] = t.to(torch.bfloat16).float()
    return out


def write_model_dir(path: str, cfg: dict, weights: Dict[str, torch.Tensor], dtype=torch.bfloat16) -> None:
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name, t in weights.items():
        if t.is_floating_point():
            t = t.to(dtype).contiguous()
            code = {torch.bfloat16: "BF16", torch.float32: "F32"}[dtype]
            raw = t.view(torch.int16 if dtype == torch.bfloat16 else torch.int32).numpy().tobytes()
        else:
            t = t.to(torch.int32).contiguous()
            code, raw = "I32", t.numpy().tobytes()
        header[name] = {"dtype": code, "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)


def read_model_dir(path: str):
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = np.frombuffer(data[lo:hi], dtype={"BF16": np.uint16, "F32": np.float32, "I32": np.int32}[info["dtype"]])
        if info["dtype"] == "BF16":
            t = torch.from_numpy((raw.astype(np.uint32) << 16).view(np.float32).copy())
        else:
            t = torch.from_numpy(raw.copy())
        out[name] = t.view(info["shape"])
    return cfg, out
