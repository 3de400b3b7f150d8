"""Small Vizotar configurations for the tests (as config.json dictionaries).  Sizes differ from layer to layer
and include what a model may happen to make equal or 1: one stream, heads = kv heads, key size = value size, a
rotation of the whole head and of two entries, a window of one token, one tap, one expert chosen or all of
them, a layer without a feed-forward.  A key that starts with an underscore is for the tests' weight
generator only and is not written to config.json (the inner sizes of the low-rank projections are tensor
shapes)."""

import copy
import random


def rotation(dims, base=10000.0, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        factor, original, fast, slow = scaling
        r["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return r


def left(heads, kv_heads, dim, vdim, size, conv, rot, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if size:
        m["mask"] = {"size": size}
    if conv:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = rot
    return m


def right(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def pair(l, r):
    return {"left": l, "right": r}


def delta(heads, kv_heads, dim, vdim, conv, rank_a=6, rank_g=5):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "_rank_a": rank_a, "_rank_g": rank_g}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(layers, vocab=160, width=96, streams=3, eps=1e-5):
    out = []
    for entry in layers:
        kind, mixer, mlp = entry[:3]
        e = {"type": kind, "mixer": mixer, "mlp": mlp}
        if len(entry) > 3:
            e["weights_of"] = entry[3]
        out.append(e)
    return {"architecture": "Vizotar", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps},
            "layers": out}


_PAIR = pair(left(4, 2, 16, 24, 20, 3, rotation(8, 10000.0, (8.0, 64, 16.0, 2.0)), scale=0.3), right(3, 8, 16, 10.0))
_DELTA = delta(4, 2, 24, 12, 4)

# every mechanism; the third layer runs on the first one's tensors
MIX = model([("parallel", _PAIR, dense(80, 2.5)),
             ("channel_delta", _DELTA, moe(6, 2, 40)),
             ("parallel", copy.deepcopy(_PAIR), dense(80, 2.5), 0),
             ("channel_delta", delta(2, 2, 16, 16, 2, rank_a=3, rank_g=8), None),
             ("channel_delta", copy.deepcopy(_DELTA), moe(6, 2, 40), 1)])

# the same without a router's close calls (every expert is chosen): for 16-bit engines
CALM = model([("parallel", _PAIR, dense(80, 2.5)),
              ("channel_delta", _DELTA, moe(3, 3, 40)),
              ("parallel", copy.deepcopy(_PAIR), dense(80, 2.5), 0),
              ("channel_delta", delta(2, 2, 16, 16, 2, rank_a=3, rank_g=8), None)])

# sizes that are multiples of neither 8 nor 16, one stream, one tap, one expert chosen, a rotation of the whole
# head without scaling, full attention in one pair
ODD = model([("channel_delta", delta(3, 3, 13, 20, 1, rank_a=5, rank_g=7), moe(5, 1, 28)),
             ("parallel", pair(left(3, 3, 20, 12, 0, 2, rotation(20, 5000.0)), right(2, 10, 6, 4.0)), dense(52, 0.7)),
             ("parallel", pair(left(2, 1, 10, 14, 1, 0, rotation(2, 100.0, (2.0, 16, 4.0, 1.0))), right(1, 13, 13, 30.0)), None)],
            vocab=130, width=100, streams=1)
ODD_CALM = model([("channel_delta", delta(3, 3, 13, 20, 1, rank_a=5, rank_g=7), moe(2, 2, 28)),
                  ("parallel", pair(left(3, 3, 20, 12, 0, 2, rotation(20, 5000.0)), right(2, 10, 6, 4.0)), dense(52, 0.7)),
                  ("parallel", pair(left(2, 1, 10, 14, 1, 0, rotation(2, 100.0, (2.0, 16, 4.0, 1.0))), right(1, 13, 13, 30.0)), None)],
                 vocab=130, width=100, streams=1)

# pairs only, delta layers only
PAIRS = model([("parallel", _PAIR, None), ("parallel", pair(left(2, 2, 32, 32, 7, 4, None), right(2, 16, 8, 15.0)), dense(64, 1.0))],
              streams=2)
DELTAS = model([("channel_delta", _DELTA, dense(64, 1.5)), ("channel_delta", delta(1, 1, 64, 40, 3), None)], streams=4)

ALL = {"mix": MIX, "calm": CALM, "odd": ODD, "odd_calm": ODD_CALM, "pairs": PAIRS, "deltas": DELTAS}


def one_windowed_layer(size, heads=2, kv_heads=1, dim=32, vdim=32, rot_dims=8, conv=0, streams=2):
    """One pair (the tests switch its memory side off through the side's output norm) with a window."""
    return model([("parallel", pair(left(heads, kv_heads, dim, vdim, size, conv, rotation(rot_dims, 200000.0, (4.0, 32, 8.0, 1.0))),
                                    right(1, 8, 8, 10.0)), None)], vocab=48, width=64, streams=streams)


def clone(cfg):
    return copy.deepcopy(cfg)


def random_config(seed, calm=False):
    """Layers of either kind in any order with sizes, windows, taps and constants drawn at random; a layer may
    run on an earlier layer's tensors."""
    r = random.Random(seed)
    layers = []
    for i in range(r.randint(2, 5)):
        own = [j for j, e in enumerate(layers) if len(e) == 3]
        if own and r.random() < 0.25:
            j = r.choice(own)
            layers.append((layers[j][0], copy.deepcopy(layers[j][1]), copy.deepcopy(layers[j][2]), j))
            continue
        if r.random() < 0.5:
            kv = r.choice([1, 2, 3])
            dim = r.choice([8, 16, 24, 40, 64])
            rot = None if r.random() < 0.2 else rotation(
                r.choice([d for d in (2, 4, 8, 16, 24, 40, 64) if d <= dim]), r.choice([100.0, 10000.0, 1e6]),
                None if r.random() < 0.4 else (r.choice([2.0, 4.0, 16.0]), r.choice([32, 128, 1024]), r.choice([8.0, 32.0]), r.choice([1.0, 2.0])))
            mixer = pair(left(kv * r.choice([1, 2]), kv, dim, r.choice([8, 16, 32, 48]), r.choice([0, 1, 5, 33, 64, 200]),
                              r.choice([0, 1, 2, 3, 4]), rot, scale=r.choice([None, 0.2, 1.0])),
                         right(r.choice([1, 2, 4]), r.choice([8, 16, 32]), r.choice([8, 24, 64]), r.choice([5.0, 15.0])))
            kind = "parallel"
        else:
            kv = r.choice([1, 2])
            mixer = delta(kv * r.choice([1, 2, 3]), kv, r.choice([8, 16, 32, 48]), r.choice([8, 16, 40, 64]),
                          r.choice([1, 2, 3, 4]), rank_a=r.choice([2, 8, 16]), rank_g=r.choice([4, 8]))
            kind = "channel_delta"
        f = r.random()
        experts = r.choice([2, 4, 7])
        mlp = None if f < 0.2 else (dense(r.choice([32, 72, 128]), r.choice([0.5, 1.0, 7.0])) if f < 0.6 else
                                    moe(experts, experts if calm else r.randint(1, experts), r.choice([16, 40])))
        layers.append((kind, mixer, mlp))
    return model(layers, vocab=r.choice([100, 256]), width=r.choice([64, 96, 128]), streams=r.choice([1, 2, 4, 5]),
                 eps=r.choice([1e-6, 1e-5]))
