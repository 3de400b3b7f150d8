"""Vizotar without a GPU: its configuration (keys, errors, round trip, inner sizes taken from tensor shapes),
the tensor names the model expects against the plain implementation's own list, cache groups and states per
layer run (a layer on another layer's tensors has its own), the random-weights writer, and the plain
implementation against closed forms of its own mechanisms."""

import copy
import json
import math
import os

import pytest
import torch

import plain_vizotar as P
import vizotar_configs as C


def with_ranks(cfg):
    """The configuration as a model without a file gives it: the low-rank projections' inner sizes as keys."""
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        m = layer["mixer"]
        if "_rank_a" in m:
            m["decay_rank"], m["gate_rank"] = m.pop("_rank_a"), m.pop("_rank_g")
    return cfg


def test_configuration_round_trip_and_registry(tmp_path):
    from redline_b200.config.model_config import VizotarConfig
    from redline_b200.config.registry import config_from_dict, load_config
    for name, cfg in C.ALL.items():
        c = config_from_dict(with_ranks(cfg))
        assert isinstance(c, VizotarConfig) and c.architecture == "Vizotar"
        assert c.vocab_size == cfg["vocab"] and c.hidden_size == cfg["width"] and c.norm_eps == cfg["norm"]["eps"]
        assert c.streams == cfg["streams"] and len(c.layers) == len(cfg["layers"])
        assert config_from_dict(c.to_hf()) == c, name
        c.save(str(tmp_path / name))
        assert load_config(str(tmp_path / name)) == c
    m = config_from_dict(with_ranks(C.MIX))
    left = m.layers[0].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.window, left.conv, left.scale) == (4, 2, 16, 24, 20, 3, 0.3)
    assert left.rot.dims == 8 and left.rot.scaling.factor == 8.0 and left.rot.scaling.original == 64
    assert m.layers[0].mixer.right.gate_cap == 10.0 and m.layers[0].mlp.limit == 2.5
    assert m.layers[2].weights_of == 0 and m.layers[4].weights_of == 1 and m.layers[3].mlp is None
    assert (m.layers[1].mlp.experts, m.layers[1].mlp.top, m.layers[1].mlp.ff) == (6, 2, 40)
    assert (m.layers[3].mixer.decay_rank, m.layers[3].mixer.gate_rank) == (3, 8)
    o = config_from_dict(with_ranks(C.ODD))
    assert o.layers[1].mixer.left.window == 0 and o.layers[2].mixer.left.conv == 0 and o.layers[1].mixer.left.rot.scaling is None


def test_inner_sizes_come_from_the_file(tmp_path):
    """config.json does not hold the low-rank projections' inner sizes: the checkpoint's shapes do."""
    from redline_b200.config.model_config import ConfigError
    from redline_b200.config.registry import config_from_dict, load_config
    d = str(tmp_path / "m")
    P.write_model_dir(d, C.MIX, P.random_weights(C.MIX, 1))
    assert "decay_rank" not in json.dumps(json.load(open(os.path.join(d, "config.json"))))
    c = load_config(d)
    assert [(l.mixer.decay_rank, l.mixer.gate_rank) for l in c.layers if l.type == "channel_delta"] == [(6, 5), (3, 8), (6, 5)]
    bare = json.load(open(os.path.join(d, "config.json")))
    with pytest.raises(ConfigError, match="a1"):
        config_from_dict(bare)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "conv"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 7), "top"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "glu"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 3), "weights_of"),
    (lambda c: c["layers"][4].__setitem__("weights_of", 2), "weights_of"),
    (lambda c: c["layers"][2]["mixer"]["left"].__setitem__("dim", 32), "same"),
    (lambda c: c.__setitem__("streams", 9), "streams"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].__setitem__("eps", 0.0), "eps"),
])
def test_configuration_errors_name_the_key(edit, word):
    from redline_b200.config.model_config import ConfigError
    from redline_b200.config.registry import config_from_dict
    cfg = with_ranks(C.MIX)
    edit(cfg)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


def _model(cfg):
    from redline_b200.config.registry import config_from_dict, model_spec
    from redline_b200.engine.model import DecoderModel
    from redline_b200.parts.base import Runtime
    rt = Runtime(device=torch.device("cpu"), dtype=torch.float32, max_tokens=8, max_seqs=2, max_seq_len=64, page_size=16)
    return DecoderModel(model_spec(config_from_dict(with_ranks(cfg))), rt)


@pytest.mark.parametrize("name", list(C.ALL))
def test_expected_tensors_are_the_plain_implementations(name):
    model = _model(C.ALL[name])
    exp = {n: tuple(s.shape) for n, s in model.expected_tensors().items()}
    assert exp == P.tensor_shapes(C.ALL[name])


def test_cache_groups_and_states_follow_the_layer_runs():
    """Five runs on three sets of tensors: every run has a cache or a state of its own."""
    model = _model(C.MIX)
    assert len(model.blocks) == 3 and [c.layer for c in model.spec.order] == [0, 1, 0, 2, 1]
    groups = model.cache_groups()
    owners = sorted(o for g in groups for o in g.owners)
    assert owners == [0, 2]
    for g in groups:
        assert g.spec.kind == "window" and g.spec.window == 20
        assert [t.shape for t in g.spec.tensors] == [(2, 16), (2, 24)]
    states = model.state_specs()
    assert sorted(states) == [0, 1, 2, 3, 4]

    def sizes(i):
        s = states[i]
        return sorted(math.prod(x.shape) for x in (s if isinstance(s, (tuple, list)) else (s,)))

    # a pair: the memory's S and n [heads, dim, vdim + 1] with a stabiliser per head, and the attention's
    # convolution inputs (taps - 1 rows of q, k and v)
    assert sizes(0) == sizes(2) == sorted([3 * 8 * 17 + 3, 2 * (4 * 16 + 2 * 16 + 2 * 24)])
    # the delta rule: S [heads, dim, vdim] and taps - 1 rows of q, k and v
    assert sizes(1) == sizes(4) == sorted([4 * 24 * 12, 3 * (2 * 2 * 24 + 4 * 12)])
    assert sizes(3) == sorted([2 * 16 * 16, 1 * (2 * 2 * 16 + 2 * 16)])
    # one tap, no convolution on the pair's attention: states of the recurrences only
    odd = _model(C.ODD).state_specs()
    assert [len(s) if isinstance(s, (tuple, list)) else 1 for s in (odd[0], odd[2])] == [1, 1]
    kinds = sorted((g.spec.kind, g.spec.window) for g in _model(C.ODD).cache_groups())
    assert kinds == [("full", 0), ("window", 1)]


def test_random_weights_writer(tmp_path):
    from redline_b200.config.registry import config_from_dict
    from redline_b200.weights.random_init import write_random_model
    from redline_b200.weights.safetensors_io import CheckpointReader
    d = write_random_model(str(tmp_path / "m"), config_from_dict(with_ranks(C.MIX)), seed=3)
    r = CheckpointReader(d)
    assert {n: tuple(r.info(n)[1]) for n in r.names()} == P.tensor_shapes(C.MIX)
    assert json.load(open(os.path.join(d, "config.json")))["architecture"] == "Vizotar"
    w = {n: r.tensor(n).float() for n in r.names()}
    cfg2, w2 = P.read_model_dir(d)                # the plain reader reads the framework's file
    assert all(torch.equal(w[n], w2[n]) for n in w)
    assert torch.isfinite(P.forward(cfg2, w, [1, 5, 9, 2])).all()


# ------------------------------------------------------------------ the plain implementation itself

def test_plain_delta_rule_stores_and_replaces():
    """With beta = 1 and no decay a unit key reads back exactly the value last written under it, whatever was
    there; an orthogonal key's value is untouched; with decay a the old content of channel c fades by a_c."""
    D, DV = 4, 3
    e = torch.eye(D, dtype=P.F64)
    v = torch.tensor([[1.0, 2.0, 3.0], [-1.0, 0.5, 4.0], [7.0, 7.0, 7.0], [0.0, 0.0, 0.0]], dtype=P.F64)
    k = torch.stack([e[0], e[1], e[0], e[2]])
    q = torch.stack([e[0], e[0], e[0], e[1]])
    one, ones = torch.ones(4, dtype=P.F64), torch.ones(4, D, dtype=P.F64)
    o = P.gated_delta(q, k, v, one, ones)
    assert torch.allclose(o[0], v[0]) and torch.allclose(o[1], v[0]) and torch.allclose(o[2], v[2]) and torch.allclose(o[3], v[1])
    # beta = 0.25 moves a quarter of the way from the old value to the new one
    o = P.gated_delta(q[:3], k[:3], v[:3], torch.tensor([1.0, 1.0, 0.25], dtype=P.F64), ones[:3])
    assert torch.allclose(o[2], 0.75 * v[0] + 0.25 * v[2])
    # decay acts on the rows of S by key channel, before the token's own write
    decay = torch.ones(3, D, dtype=P.F64)
    decay[1, 0] = 0.5
    decay[2, 1] = 0.1
    o = P.gated_delta(torch.stack([e[0], e[0], e[0] + e[1]]), torch.stack([e[0], e[1], e[2]]), v[:3], one[:3], decay)
    assert torch.allclose(o[1], 0.5 * v[0]) and torch.allclose(o[2], 0.5 * v[0] + 0.1 * v[1])


def test_plain_delta_rule_against_its_unrolled_form():
    g = torch.Generator().manual_seed(3)
    T, D, DV = 9, 5, 4
    q, k = torch.randn(T, D, generator=g, dtype=P.F64), torch.randn(T, D, generator=g, dtype=P.F64)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(T, DV, generator=g, dtype=P.F64)
    beta = torch.rand(T, generator=g, dtype=P.F64)
    decay = torch.rand(T, D, generator=g, dtype=P.F64)
    got = P.gated_delta(q, k, v, beta, decay)
    # S_t = (I - beta_t k_t k_t^T) diag(a_t) S_(t-1) + beta_t k_t v_t^T
    S = torch.zeros(D, DV, dtype=P.F64)
    for t in range(T):
        S = (torch.eye(D, dtype=P.F64) - beta[t] * torch.outer(k[t], k[t])) @ (torch.diag(decay[t]) @ S) + beta[t] * torch.outer(k[t], v[t])
        assert torch.allclose(got[t], S.T @ q[t], atol=1e-12)


def test_plain_memory_is_the_gated_sum_and_starts_its_stabiliser_at_zero():
    g = torch.Generator().manual_seed(0)
    T, D, DV = 11, 4, 6
    q, k = torch.randn(T, D, generator=g, dtype=P.F64), torch.randn(T, D, generator=g, dtype=P.F64)
    v = torch.randn(T, DV, generator=g, dtype=P.F64)
    ig = torch.randn(T, generator=g, dtype=P.F64)
    fg = P.log_sigmoid(torch.randn(T, generator=g, dtype=P.F64) + 2.0)
    got = P.matrix_memory(q, k, v, ig, fg)
    m = 0.0
    for t in range(T):
        m = max(float(fg[t]) + m, float(ig[t]))
        num, den = torch.zeros(DV, dtype=P.F64), 0.0
        for s in range(t + 1):
            wgt = math.exp(float(ig[s] + fg[s + 1:t + 1].sum()) - m)
            num += wgt * float(k[s] @ q[t]) * v[s]
            den += wgt * float(k[s] @ q[t])
        assert torch.allclose(got[t], num / (max(abs(den), math.exp(-m)) + P.DENOMINATOR_FLOOR), atol=1e-12), t
    # a first token with a very negative input gate: m stays 0, the floor of the denominator is 1
    first = P.matrix_memory(q[:1], k[:1], v[:1], torch.tensor([-9.0], dtype=P.F64), fg[:1])
    kq = math.exp(-9.0) * float(k[0] @ q[0])
    assert torch.allclose(first[0], kq * v[0] / (max(abs(kq), 1.0) + P.DENOMINATOR_FLOOR), atol=1e-15)


def test_plain_convolution_is_a_causal_correlation():
    g = torch.Generator().manual_seed(4)
    u, w = torch.randn(12, 5, generator=g, dtype=P.F64), torch.randn(5, 4, generator=g, dtype=P.F64)
    got = P.causal_conv(u, w)
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (3, 0)), w[:, None, :], groups=5)[0].T
    assert torch.allclose(got, want, atol=1e-13)
    assert torch.allclose(got[0], w[:, 3] * u[0])                   # the last tap is the current token's
    assert torch.allclose(P.causal_conv(u, w[:, 3:]), u * w[:, 3])  # one tap: a weight per channel


def test_plain_sink_window_and_groups():
    q = torch.zeros(5, 2, 4, dtype=P.F64)
    k = torch.zeros(5, 1, 4, dtype=P.F64)
    v = torch.arange(5, dtype=P.F64).view(5, 1, 1).expand(5, 1, 3).contiguous()
    o = P.window_sink_attention(q, k, v, 1.0, 0, None)
    assert torch.allclose(o[4, 0], torch.full((3,), 2.0, dtype=P.F64))
    o = P.window_sink_attention(q, k, v, 1.0, 2, None)
    assert torch.allclose(o[4, 1], torch.full((3,), 3.5, dtype=P.F64)) and torch.allclose(o[0, 0], torch.zeros(3, dtype=P.F64))
    sink = torch.tensor([0.0, math.log(2.0)], dtype=P.F64)
    o = P.window_sink_attention(q, k, v, 1.0, 2, sink)
    assert torch.allclose(o[4, 0], torch.full((3,), 7.0 / 3.0, dtype=P.F64))      # weights 1/3, 1/3 and the sink's 1/3
    assert torch.allclose(o[4, 1], torch.full((3,), 7.0 / 4.0, dtype=P.F64))      # a sink that counts twice
    # the scale multiplies the scores and not the sink
    q1 = torch.ones(1, 1, 4, dtype=P.F64)
    o = P.window_sink_attention(q1, q1.clone(), torch.ones(1, 1, 1, dtype=P.F64), 0.25, 0, torch.tensor([1.0], dtype=P.F64))
    assert torch.allclose(o[0, 0], torch.tensor([0.5], dtype=P.F64))              # e^(4 * 0.25) against e^1
    # window of one token: itself only
    o = P.window_sink_attention(q, k, v, 1.0, 1, None)
    assert torch.allclose(o[:, 0, 0], torch.arange(5, dtype=P.F64))


def test_plain_rotation_frequencies():
    plain = {"base": 10000.0, "dims": 8}
    f, mag = P.scaled_frequencies(plain)
    assert mag == 1.0 and f == [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 256, "fast": 32.0, "slow": 1.0}}
    f, mag = P.scaled_frequencies(rot)
    f0 = [10000.0 ** (-2.0 * i / 16) for i in range(8)]
    assert mag == 0.1 * math.log(4.0) + 1.0
    # pairs that turn more than 'fast' times within the original length keep their frequency; those that
    # turn less than 'slow' times are slowed by the factor; between them the blend grows with the index
    turns = [256 * x / (2 * math.pi) for x in f0]
    ratio = [a / b for a, b in zip(f, f0)]
    for i in range(8):
        if turns[i] > 32.0 * 10000.0 ** (2.0 / 16):
            assert ratio[i] == 1.0
        if turns[i] < 1.0 / 10000.0 ** (2.0 / 16):
            assert abs(ratio[i] - 0.25) < 1e-15
    assert all(a >= b for a, b in zip(ratio, ratio[1:])) and ratio[0] == 1.0 and abs(ratio[-1] - 0.25) < 1e-15
    assert any(0.25 < r < 1.0 for r in ratio)


def test_plain_rotation_pairs_halves_and_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(2)
    rot = {"base": 100.0, "dims": 8}
    x = torch.randn(1, 1, 12, generator=g, dtype=P.F64).expand(9, 1, 12).contiguous()
    y = torch.randn(1, 1, 12, generator=g, dtype=P.F64).expand(9, 1, 12).contiguous()
    rx, ry = P.rotate_halves(x, rot), P.rotate_halves(y, rot)
    assert torch.equal(rx[:, :, 8:], x[:, :, 8:]) and torch.allclose(rx[0], x[0])
    dots = torch.einsum("ihd,jhd->ij", rx, ry)
    for d in range(1, 5):
        assert torch.allclose(dots.diagonal(d), dots.diagonal(d)[0].expand(9 - d), atol=1e-12)
    e = torch.zeros(4, 1, 12, dtype=P.F64)
    e[:, 0, 1] = 1.0                                        # entry 1 is paired with entry 1 + 4
    r = P.rotate_halves(e, rot)
    a = torch.arange(4, dtype=P.F64) * 100.0 ** (-2.0 / 8)
    assert torch.allclose(r[:, 0, 1], torch.cos(a)) and torch.allclose(r[:, 0, 5], torch.sin(a))
    assert torch.allclose(P.rotate_halves(x[3:5], rot, first=3), rx[3:5])
    # scaling multiplies cos and sin alike: the rotated part grows by the magnitude
    sc = {"base": 100.0, "dims": 8, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    rs = P.rotate_halves(x, sc)
    mag = 0.1 * math.log(2.0) + 1.0
    assert torch.allclose(rs[:, :, :8].norm(dim=-1), mag * x[:, :, :8].norm(dim=-1))


def test_plain_feed_forwards():
    z = torch.tensor([[-3.0, 0.5, 4.0]], dtype=P.F64)
    w = {"gate": torch.eye(3), "up": torch.eye(3), "down": torch.eye(3)}
    w = {k: v.to(P.F64) for k, v in w.items()}
    got = P.dense_ff(z, w, "", {"limit": 2.0})
    gate = torch.tensor([-3.0, 0.5, 2.0], dtype=P.F64)          # clamped from above only
    up = torch.tensor([-2.0, 0.5, 2.0], dtype=P.F64)            # clamped on both sides
    assert torch.allclose(got[0], gate * P.sigmoid(P.GLU_SLOPE * gate) * (up + 1.0))
    # the router: softmax over the chosen logits only, the bias counts in the choice
    w = {"router": torch.eye(4, dtype=P.F64), "router.b": torch.tensor([0.0, 0.0, 5.0, 0.0], dtype=P.F64)}
    idx, wt = P.route(torch.tensor([[2.0, 1.0, -3.5, 0.0]], dtype=P.F64), w, "", {"router": {"experts": 4, "top": 2}})
    assert idx[0].tolist() == [0, 2] and torch.allclose(wt[0], torch.softmax(torch.tensor([2.0, 1.5], dtype=P.F64), 0))
    idx, wt = P.route(torch.tensor([[2.0, 1.0, -3.5, 0.0]], dtype=P.F64), w, "", {"router": {"experts": 4, "top": 1}})
    assert idx[0].tolist() == [0] and wt[0].tolist() == [1.0]


def test_plain_streams_with_one_stream_are_the_residual_sum():
    """One stream with in = out = mix = 1 is the pre-norm residual layer; several streams that start equal stay a
    weighted sum of the same sublayer outputs."""
    cfg = C.clone(C.DELTAS)
    cfg["streams"] = 1
    w = {k: v.double() for k, v in P.random_weights(cfg, 5).items()}
    for n in w:
        if ".hc" in n:
            w[n] = torch.ones_like(w[n])
    toks = [3, 9, 4, 4, 11, 0, 7]
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(toks)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + P.channel_delta_mixer(P.rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        if layer["mlp"] is not None:
            x = x + P.dense_ff(P.rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
    want = P.rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    outs = []
    got = P.forward(cfg, w, toks, outs)
    assert torch.allclose(got, want, atol=1e-10) and torch.allclose(outs[-1], x, atol=1e-10)
    # a layer on another layer's tensors: the same weights, a state of its own
    twice = C.clone(cfg)
    twice["layers"] = [twice["layers"][1], dict(copy.deepcopy(twice["layers"][1]), weights_of=0)]
    w2 = {n.replace("l1.", "l0."): t for n, t in w.items() if not n.startswith("l0.")}
    x = w2["embed"][torch.tensor(toks)]
    for _ in range(2):
        x = x + P.channel_delta_mixer(P.rms_norm(x, w2["l0.norm1"], eps), w2, "l0.mix.", twice["layers"][0]["mixer"], eps)
    assert torch.allclose(P.forward(twice, w2, toks), P.rms_norm(x, w2["final.norm"], eps) @ w2["embed"].T, atol=1e-10)


def test_the_comparison_models_of_the_bench_parse():
    """`bench.py --compare-design`: every design's model and the one beside it build at every size, with as
    many layers, the same width and vocabulary."""
    from redline_b200.apps import design_bench as D
    from redline_b200.config.registry import config_from_dict, model_spec
    for design, (sizes, make, beside, make_beside) in D.DESIGNS.items():
        for s in sizes.values():
            a, b = config_from_dict(make(s)), config_from_dict(make_beside(s))
            sa, sb = model_spec(a), model_spec(b)
            assert (sa.hidden_size, sa.vocab_size, len(sa.order)) == (sb.hidden_size, sb.vocab_size, len(sb.order)), design
    v = config_from_dict(D.vizotar_config(D.VIZOTAR_SIZES["s"]))
    assert [l.type for l in v.layers] == ["parallel", "channel_delta", "parallel", "channel_delta"]
    assert [l.mlp.kind for l in v.layers] == ["dense", "moe", "moe", "dense"] and v.streams == 4
    m = v.layers[1].mlp
    assert m.top * m.ff == v.layers[0].mlp.ff          # the chosen experts together are as wide as the dense one
