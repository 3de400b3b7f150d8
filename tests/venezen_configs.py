"""Small Venezen configurations for the tests (as config.json dictionaries).  Sizes differ from layer to layer
and include what a model may happen to make equal or 1: heads = key heads, a rotation of fewer entries than the
rotated part holds, a window of one token, one expert chosen or all of them, no identity expert, no shared
expert, a layer without a feed-forward, a repeated run that starts at the first layer, one that is the whole
model, one that runs once, and no repetition at all."""

import copy
import random


def latent(heads, dim, rot_dim, vdim, rank, rot_dims=None, base=10000.0, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
            "rot": {"base": base, "dims": rot_dims if rot_dims is not None else rot_dim},
            "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}


def windowed(heads, kv_heads, dim, size, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale if scale is not None else dim ** -0.5}
    if size:
        m["mask"] = {"size": size}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff, limit, scale=1.0, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
         "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared is not None:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return f


def model(layers, loop=None, vocab=160, width=96, eps=1e-5, embed_scale=4.0):
    out = {"architecture": "Venezen", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale},
           "norm": {"eps": eps}, "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


def _mix(calm):
    def routed(experts, identity, top, ff, limit, scale, shared):
        return moe(experts, identity, experts + identity if calm else top, ff, limit, scale, shared)
    return model([
        ("latent_attention", latent(3, 16, 8, 24, 40, base=10000.0, scale=0.2), dense(80)),
        ("attention", windowed(4, 2, 16, 20, scale=0.25), routed(6, 2, 3, 40, 1.5, 1.5, (24, 2.5))),
        ("latent_attention", latent(2, 24, 16, 16, 32, rot_dims=8, base=500.0), routed(4, 1, 2, 32, 0.8, 2.0, None)),
        ("attention", windowed(2, 2, 32, 33), None),
        ("latent_attention", latent(4, 8, 8, 8, 24), dense(48)),
    ], loop=(1, 3, 3))


# every mechanism; layers 1 and 2 run three times
MIX = _mix(False)
# the same with routers that choose every output (no close calls): for 16-bit engines
CALM = _mix(True)

# sizes that are multiples of neither 8 nor 16; the repeated run starts at the first layer; a window of one
# token; one expert chosen, no identity experts, no shared expert; three query heads on one key head
def _odd(calm):
    return model([
        ("latent_attention", latent(3, 10, 6, 12, 20, rot_dims=2, base=100.0), moe(5, 0, 5 if calm else 1, 28, 0.7)),
        ("attention", windowed(3, 1, 20, 1), dense(52)),
        ("attention", windowed(2, 2, 13, 0, scale=0.4), moe(2, 3, 5 if calm else 2, 12, 3.0, 0.5, (20, 1.0))),
    ], loop=(0, 2, 2), vocab=130, width=100, embed_scale=1.0)


ODD, ODD_CALM = _odd(False), _odd(True)

# one kind of mixer only; no repetition; a run that is the whole model; a run that runs once
LATENTS = model([("latent_attention", latent(4, 16, 16, 16, 48, scale=0.3), None),
                 ("latent_attention", latent(1, 32, 32, 64, 64, rot_dims=32), dense(64))], loop=(0, 2, 2))
WINDOWS = model([("attention", windowed(4, 1, 32, 7), dense(64)), ("attention", windowed(6, 3, 16, 64), None)],
                loop=(1, 2, 1), embed_scale=8.0)
PLAIN = model([("attention", windowed(2, 2, 16, 40), dense(32)), ("latent_attention", latent(2, 16, 0, 16, 32), dense(32))])

ALL = {"mix": MIX, "calm": CALM, "odd": ODD, "odd_calm": ODD_CALM, "latents": LATENTS, "windows": WINDOWS, "plain": PLAIN}


def one_windowed_layer(size, heads=2, kv_heads=1, dim=32):
    return model([("attention", windowed(heads, kv_heads, dim, size), None)], vocab=48, width=64)


def one_latent_layer(heads=2, dim=16, rot_dim=8, vdim=16, rank=32):
    return model([("latent_attention", latent(heads, dim, rot_dim, vdim, rank, base=200000.0), None)], vocab=48, width=64)


def clone(cfg):
    return copy.deepcopy(cfg)


def random_config(seed, calm=False):
    """Layers of either kind in any order with sizes, windows and constants drawn at random, and a repeated run
    drawn at random too."""
    r = random.Random(seed)
    layers = []
    n = r.randint(2, 5)
    for i in range(n):
        if r.random() < 0.5:
            rot_dim = r.choice([0, 2, 8, 16, 24])
            mixer = latent(r.choice([1, 2, 3, 5]), r.choice([8, 16, 24, 40]), rot_dim, r.choice([8, 16, 40]),
                           r.choice([16, 24, 48, 72]), rot_dims=r.choice([d for d in (2, 8, 16, 24) if d <= rot_dim] or [2]),
                           base=r.choice([100.0, 10000.0, 5e5]), scale=r.choice([None, 0.15, 0.5]))
            kind = "latent_attention"
        else:
            kv = r.choice([1, 2, 3])
            mixer = windowed(kv * r.choice([1, 2, 4]), kv, r.choice([8, 16, 24, 48, 64]), r.choice([0, 1, 5, 33, 64, 200]),
                             scale=r.choice([None, 0.2, 0.6]))
            kind = "attention"
        f = r.random()
        experts, identity = r.choice([2, 4, 7]), r.choice([0, 1, 3])
        mlp = None if f < 0.2 else (dense(r.choice([32, 72, 128])) if f < 0.55 else
                                    moe(experts, identity, experts + identity if calm else r.randint(1, experts + identity),
                                        r.choice([16, 40]), r.choice([0.5, 1.0, 7.0]), r.choice([1.0, 2.5]),
                                        None if r.random() < 0.4 else (r.choice([16, 48]), r.choice([1.0, 2.0]))))
        layers.append((kind, mixer, mlp))
    loop = None
    if r.random() < 0.75:
        a = r.randint(0, n - 1)
        loop = (a, r.randint(a + 1, n), r.choice([1, 2, 3]))
    return model(layers, loop=loop, vocab=r.choice([100, 256]), width=r.choice([64, 96, 128]), eps=r.choice([1e-6, 1e-5]),
                 embed_scale=r.choice([1.0, 3.0, 12.0]))
