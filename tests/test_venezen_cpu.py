"""Venezen without a GPU: its configuration (keys, errors, round trip, the run order of a repeated run), the
tensor names the model expects against the plain implementation's own list, cache groups per layer run, the
random-weights writer, and the plain implementation against closed forms of its own mechanisms."""

import copy
import json
import math
import os

import pytest
import torch

import plain_venezen as P
import venezen_configs as C


def test_configuration_round_trip_and_registry(tmp_path):
    from redline_b200.config.model_config import VenezenConfig
    from redline_b200.config.registry import config_from_dict, load_config
    for name, cfg in C.ALL.items():
        c = config_from_dict(cfg)
        assert isinstance(c, VenezenConfig) and c.architecture == "Venezen"
        assert c.vocab_size == cfg["vocab"] and c.hidden_size == cfg["width"] and c.norm_eps == cfg["norm"]["eps"]
        assert c.embedding_scale == cfg["embedding"]["scale"] and len(c.layers) == len(cfg["layers"])
        assert config_from_dict(c.to_hf()) == c, name
        c.save(str(tmp_path / name))
        assert load_config(str(tmp_path / name)) == c
        assert c.run_order() == P.run_order(cfg)
    m = config_from_dict(C.MIX)
    a = m.layers[0].mixer
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.scale, a.rot.dims, a.rot.base) == (3, 16, 8, 24, 40, 0.2, 8, 10000.0)
    assert m.layers[2].mixer.rot.dims == 8 and m.layers[2].mixer.rot_dim == 16
    b = m.layers[1].mixer
    assert (b.heads, b.kv_heads, b.dim, b.vdim, b.window, b.scale) == (4, 2, 16, 16, 20, 0.25)
    f = m.layers[1].mlp
    assert (f.experts, f.identity, f.top, f.ff, f.limit, f.scale, f.shared.ff, f.shared.limit) == (6, 2, 3, 40, 1.5, 1.5, 24, 2.5)
    assert m.layers[2].mlp.shared is None and m.layers[3].mlp is None and m.layers[0].mlp.kind == "dense"
    assert (m.loop.start, m.loop.stop, m.loop.times) == (1, 3, 3)
    assert [i for i, _ in m.run_order()] == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert [add for _, add in m.run_order()] == [False, False, False, True, False, True, False, False, False]
    o = config_from_dict(C.ODD)
    assert [x for x in o.run_order()] == [(0, False), (1, False), (0, True), (1, False), (2, False)]
    assert o.layers[2].mixer.window == 0 and o.layers[0].mlp.identity == 0
    assert config_from_dict(C.PLAIN).loop is None and config_from_dict(C.PLAIN).layers[1].mixer.rot_dim == 0
    # what config.json leaves out does not exist
    bare = copy.deepcopy(C.WINDOWS)
    del bare["embedding"], bare["loop"]
    c = config_from_dict(bare)
    assert c.embedding_scale == 1.0 and c.loop is None and [i for i, _ in c.run_order()] == [0, 1]


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"].pop("rot"), "rot"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 10), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("vdim", 8), "vdim"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "sparse"), "sparse"),
    (lambda c: c["layers"][1].__setitem__("type", "recurrent"), "recurrent"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c["loop"].__setitem__("times", 0), "loop"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].__setitem__("eps", 0.0), "eps"),
])
def test_configuration_errors_name_the_key(edit, word):
    from redline_b200.config.model_config import ConfigError
    from redline_b200.config.registry import config_from_dict
    cfg = copy.deepcopy(C.MIX)
    edit(cfg)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


def _model(cfg):
    from redline_b200.config.registry import config_from_dict, model_spec
    from redline_b200.engine.model import DecoderModel
    from redline_b200.parts.base import Runtime
    rt = Runtime(device=torch.device("cpu"), dtype=torch.float32, max_tokens=8, max_seqs=2, max_seq_len=64, page_size=16)
    return DecoderModel(model_spec(config_from_dict(cfg)), rt)


@pytest.mark.parametrize("name", list(C.ALL))
def test_expected_tensors_are_the_plain_implementations(name):
    model = _model(C.ALL[name])
    exp = {n: tuple(s.shape) for n, s in model.expected_tensors().items()}
    assert exp == P.tensor_shapes(C.ALL[name])


def test_cache_groups_follow_the_layer_runs():
    """Nine runs on five sets of tensors: every run owns a cache; the latent layers cache one row of latent and
    rotated key part, the windowed ones their keys only."""
    model = _model(C.MIX)
    assert len(model.blocks) == 5
    assert [(c.layer, c.add_embedding) for c in model.spec.order] == P.run_order(C.MIX)
    assert all(c.cache_of is None for c in model.spec.order)
    groups = {(g.spec.kind, g.spec.window, tuple(t.shape for t in g.spec.tensors)): g.owners for g in model.cache_groups()}
    by_owner = {o: key for key, owners in groups.items() for o in owners}
    assert sorted(by_owner) == list(range(9))
    assert by_owner[0] == ("full", 0, ((1, 48),)) and by_owner[2] == by_owner[4] == by_owner[6] == ("full", 0, ((1, 48),))
    assert by_owner[1] == by_owner[3] == by_owner[5] == ("window", 20, ((2, 16),))
    assert by_owner[7] == ("window", 33, ((2, 32),)) and by_owner[8] == ("full", 0, ((1, 32),))
    assert model.state_specs() == {}
    # no rotated part: the cached row is the latent alone; a window of 0 is full attention
    kinds = sorted((g.spec.kind, g.spec.window, g.spec.tensors[0].shape) for g in _model(C.PLAIN).cache_groups())
    assert kinds == [("full", 0, (1, 32)), ("window", 40, (2, 16))]
    assert ("full", 0, (2, 13)) in [(g.spec.kind, g.spec.window, g.spec.tensors[0].shape) for g in _model(C.ODD).cache_groups()]


def test_random_weights_writer(tmp_path):
    from redline_b200.config.registry import config_from_dict
    from redline_b200.weights.random_init import write_random_model
    from redline_b200.weights.safetensors_io import CheckpointReader
    d = write_random_model(str(tmp_path / "m"), config_from_dict(C.MIX), seed=3)
    r = CheckpointReader(d)
    assert {n: tuple(r.info(n)[1]) for n in r.names()} == P.tensor_shapes(C.MIX)
    assert json.load(open(os.path.join(d, "config.json")))["architecture"] == "Venezen"
    w = {n: r.tensor(n).float() for n in r.names()}
    cfg2, w2 = P.read_model_dir(d)                # the plain reader reads the framework's file
    assert all(torch.equal(w[n], w2[n]) for n in w)
    assert torch.isfinite(P.forward(cfg2, w, [1, 5, 9, 2])).all()


# ------------------------------------------------------------------ the plain implementation itself

def test_plain_window_distance_and_the_added_one():
    """Equal scores: inside the window the weights are e^(-m d) / (1 + sum), outside they are zero, and a row's
    weights add up to less than one."""
    T, size, slope = 9, 4, 0.25
    a = P.biased_window_weights(torch.zeros(T, T, dtype=torch.float64), slope, size)
    for i in range(T):
        seen = [j for j in range(T) if 0 <= i - j < size]
        den = 1.0 + sum(math.exp(-slope * (i - j)) for j in seen)
        for j in range(T):
            want = math.exp(-slope * (i - j)) / den if j in seen else 0.0
            assert abs(float(a[i, j]) - want) < 1e-12
        assert float(a[i].sum()) < 1.0
    # very negative scores: the added one takes everything
    a = P.biased_window_weights(torch.full((3, 3), -50.0, dtype=torch.float64), 0.0, 3)
    assert float(a.sum()) < 1e-20
    # very large scores: it takes nothing, and the largest score does not overflow
    a = P.biased_window_weights(torch.full((3, 3), 800.0, dtype=torch.float64), 0.0, 3)
    assert abs(float(a[2].sum()) - 1.0) < 1e-12
    assert P.head_slopes(4) == [2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8]
    assert abs(P.head_slopes(3)[0] - 2.0 ** (-8 / 3)) < 1e-15


def test_plain_windowed_attention_groups_heads_and_reads_keys_as_values():
    g = torch.Generator().manual_seed(1)
    T, W = 7, 12
    m = C.windowed(4, 2, 6, 3, scale=0.5)
    w = {"q": torch.randn(24, W, generator=g, dtype=torch.float64), "k": torch.randn(12, W, generator=g, dtype=torch.float64),
         "o": torch.eye(24, dtype=torch.float64)}
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    out = P.window_attention(h, w, "", m).view(T, 4, 6)
    k = (h @ w["k"].T).view(T, 2, 6)
    q = (h @ w["q"].T).view(T, 4, 6)
    i = 5
    for hd in range(4):
        kv = hd // 2
        e = [math.exp(float(q[i, hd] @ k[j, kv]) * 0.5 - P.head_slopes(4)[hd] * (i - j)) for j in (3, 4, 5)]
        want = sum(x * k[j, kv] for x, j in zip(e, (3, 4, 5))) / (1.0 + sum(e))
        assert torch.allclose(out[i, hd], want, atol=1e-12)


def test_plain_rotation_pairs_halves_and_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1, 10, generator=g, dtype=torch.float64)
    y = P.rotate_halves(x, 100.0, 6, [3])
    for i in range(3):
        a = 3 * 100.0 ** (-2.0 * i / 6)
        assert abs(float(y[0, i]) - (float(x[0, i]) * math.cos(a) - float(x[0, i + 3]) * math.sin(a))) < 1e-12
        assert abs(float(y[0, i + 3]) - (float(x[0, i + 3]) * math.cos(a) + float(x[0, i]) * math.sin(a))) < 1e-12
    assert torch.equal(y[0, 6:], x[0, 6:])
    q, k = torch.randn(1, 8, generator=g, dtype=torch.float64), torch.randn(1, 8, generator=g, dtype=torch.float64)
    d1 = float(P.rotate_halves(q, 50.0, 8, [9])[0] @ P.rotate_halves(k, 50.0, 8, [4])[0])
    d2 = float(P.rotate_halves(q, 50.0, 8, [25])[0] @ P.rotate_halves(k, 50.0, 8, [20])[0])
    assert abs(d1 - d2) < 1e-10


def test_plain_latent_attention_against_keys_and_values_written_out():
    """The mixer against per-head keys and values formed token by token, and the identity that lets an engine
    attend over the latents themselves: q_n . (W_uk c) = (W_uk^T q_n) . c."""
    g = torch.Generator().manual_seed(3)
    T, W = 6, 20
    m = C.latent(2, 4, 4, 3, 5, rot_dims=2, base=30.0, scale=0.7)
    w = {n: torch.randn(s, generator=g, dtype=torch.float64) for n, s in
         (("q", (16, W)), ("dkv", (9, W)), ("dkv.norm", (5,)), ("uk", (8, 5)), ("uv", (6, 5)))}
    w["o"] = torch.eye(6, dtype=torch.float64)
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    pos = list(range(T))
    out = P.latent_attention(h, w, "", m, 1e-5, pos).view(T, 2, 3)
    ckr = h @ w["dkv"].T
    c = ckr[:, :5] / torch.sqrt((ckr[:, :5] ** 2).mean(-1, keepdim=True) + 1e-5) * w["dkv.norm"]
    kr = P.rotate_halves(ckr[:, 5:], 30.0, 2, pos)
    q = (h @ w["q"].T).view(T, 2, 8)
    i = 4
    for hd in range(2):
        qr = P.rotate_halves(q[:, hd, 4:], 30.0, 2, pos)
        uk, uv = w["uk"][hd * 4:(hd + 1) * 4], w["uv"][hd * 3:(hd + 1) * 3]
        s = torch.stack([(q[i, hd, :4] @ (uk @ c[j]) + qr[i] @ kr[j]) * 0.7 for j in range(i + 1)])
        absorbed = torch.stack([((uk.T @ q[i, hd, :4]) @ c[j] + qr[i] @ kr[j]) * 0.7 for j in range(i + 1)])
        assert torch.allclose(s, absorbed, atol=1e-12)
        p = torch.softmax(s, 0)
        want = sum(p[j] * (uv @ c[j]) for j in range(i + 1))
        assert torch.allclose(out[i, hd], want, atol=1e-12)
        assert torch.allclose(want, uv @ sum(p[j] * c[j] for j in range(i + 1)), atol=1e-12)


def test_plain_router_and_feed_forwards():
    W = 6
    f = C.moe(3, 2, 2, 4, 1.0, scale=2.5, shared=(4, 2.0))
    w = {"router": torch.zeros(5, W, dtype=torch.float64), "correction": torch.tensor([0.0, 0.3, 0.0, 0.0, 0.2], dtype=torch.float64)}
    w["router"][:, 0] = torch.tensor([2.0, 0.0, 1.0, 0.5, 0.0], dtype=torch.float64)
    h = torch.zeros(2, W, dtype=torch.float64)
    h[:, 0] = 1.0
    h[1, 1] = 3.0
    pick, weight = P.route(h, w, "", f)
    s = torch.softmax(torch.tensor([2.0, 0.0, 1.0, 0.5, 0.0], dtype=torch.float64), 0)
    # the correction lifts output 1 over outputs 2 and 3 for the choice; the weights are the scores without it
    assert pick[0].tolist() == [0, 1]
    assert torch.allclose(weight[0], torch.stack([s[0], s[1]]) / (s[0] + s[1]) * 2.5, atol=1e-12)
    # an identity expert chosen: its output is the input
    w["correction"] = torch.tensor([0.0, 0.0, 0.0, 0.0, 5.0], dtype=torch.float64)
    g = torch.Generator().manual_seed(4)
    for e in range(3):
        for n, shape in (("gate", (4, W)), ("up", (4, W)), ("down", (W, 4))):
            w[f"e{e}.{n}"] = torch.randn(shape, generator=g, dtype=torch.float64)
    for n, shape in (("gate", (4, W)), ("up", (4, W)), ("down", (W, 4))):
        w["shared." + n] = torch.zeros(shape, dtype=torch.float64)
    pick, weight = P.route(h, w, "", f)
    assert pick[0].tolist() == [4, 0]
    out = P.routed_ff(h, w, "", f)
    want = weight[0, 0] * h[0] + weight[0, 1] * P.clamped_expert(h[:1], w["e0.gate"], w["e0.up"], w["e0.down"], 1.0)[0]
    assert torch.allclose(out[0], want, atol=1e-12)
    # the clamp: a gate above the limit counts as the limit, an up below -limit as -limit
    one = torch.ones(1, 1, dtype=torch.float64)
    y = P.clamped_expert(one, one * 9.0, one * -9.0, one, 2.0)
    assert abs(float(y) - 2.0 / (1.0 + math.exp(-1.702 * 2.0)) * (-2.0 + 1.0)) < 1e-12
    d = {"gate": torch.eye(2, dtype=torch.float64), "gate.b": torch.tensor([1.0, 0.0], dtype=torch.float64),
         "up": torch.eye(2, dtype=torch.float64) * 2, "up.b": torch.tensor([0.0, 1.0], dtype=torch.float64),
         "down": torch.eye(2, dtype=torch.float64), "down.b": torch.tensor([0.5, 0.5], dtype=torch.float64)}
    x = torch.tensor([[1.0, -1.0]], dtype=torch.float64)
    silu = lambda z: z / (1.0 + math.exp(-z))      # noqa: E731
    assert torch.allclose(P.dense_ff(x, d, ""), torch.tensor([[silu(2.0) * 2.0 + 0.5, silu(-1.0) * -1.0 + 0.5]], dtype=torch.float64))


def test_plain_repeated_run_feeds_the_embedding_in_again():
    """A model whose layers add nothing (output matrices zero): after a run repeated n times the stream is
    (1 + n - 1) times the embedding output, so the logits are those of the embedding alone."""
    cfg = C.clone(C.WINDOWS)
    cfg["loop"] = {"start": 0, "stop": 2, "times": 3}
    w = P.random_weights(cfg, 5)
    for n in w:
        if n.endswith(("mix.o", "mlp.down", "mlp.down.b")):
            w[n] = w[n] * 0.0
    layers = []
    P.forward(cfg, w, [3, 4, 5], layers)
    e = w["embed"][[3, 4, 5]].double() * cfg["embedding"]["scale"]
    assert len(layers) == 6
    for i, x in enumerate(layers):
        assert torch.allclose(x, e * (1 + i // 2), atol=1e-12)


def test_the_comparison_model_of_the_bench():
    """`bench.py --compare-design venezen`: one layer of every pairing of mixer and feed-forward, beside a model
    of as many layers, the same width, heads, window and experts."""
    from redline_b200.apps import design_bench as D
    from redline_b200.config.registry import config_from_dict, model_spec
    sizes, make, beside, make_beside = D.DESIGNS["venezen"]
    assert beside == "kapitar"
    for s in sizes.values():
        v, k = config_from_dict(make(s)), config_from_dict(make_beside(s))
        assert [(l.type, l.mlp.kind) for l in v.layers] == [("latent_attention", "dense"), ("attention", "moe"),
                                                           ("latent_attention", "moe"), ("attention", "dense")]
        assert (v.hidden_size, v.vocab_size, len(model_spec(v).order)) == (k.hidden_size, k.vocab_size, len(model_spec(k).order))
        assert v.layers[1].mixer.window == k.layers[0].mixer.mask.size and v.layers[1].mlp.experts == k.layers[1].mlp.experts
        assert v.layers[0].mixer.kv_rank + v.layers[0].mixer.rot_dim <= 256
