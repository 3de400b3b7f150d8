"""Venezen through the engine against the plain implementation (tests/plain_venezen.py): whole prompts,
prefill against token-by-token decoding, portions down to two tokens, unequal requests in one batch against
each alone with pages used again, a key just inside and just outside a window (in prompts, at the cut of a
portion and in decoding, also at page borders), a far key among hundreds under the latent attention, the one
in the softmax's denominator, the first tokens of a sequence, long decoding, models of one kind of layer only,
sizes that are multiples of neither 8 nor 16, repeated runs of every shape, configurations drawn at random,
greedy generation through the scheduler, and the trace replay program."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_venezen as P
import venezen_configs as C
from gpu_utils import random_tokens, rel_max
from venezen_utils import Reference, check, engine_for, make_model, oracle
from test_replay_gpu import mixed_schedule

pytestmark = pytest.mark.gpu

# (a 16-bit engine gets the models whose routers choose every output: no close calls)
CASES = [("mix", "float32"), ("calm", "bfloat16"), ("latents", "bfloat16"), ("windows", "float32"), ("plain", "bfloat16")]


class Models(dict):
    def __missing__(self, key):
        name, dtype = key
        self[key] = make_model(self.tmp, C.ALL[name], seed=3 + list(C.ALL).index(name) + (0 if dtype == "float32" else 10),
                               sharpen=2.0)
        return self[key]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    m = Models()
    m.tmp = tmp_path_factory.mktemp("venezen")
    return m


@pytest.fixture(scope="module")
def engines(models):
    cache = {}

    def get(name, dtype, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in cache:
            cache[key] = engine_for(models[name, dtype][0], dtype, **kw)
        return cache[key]

    yield get
    cache.clear()


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole(name, dtype, models, engines):
    eng, (_, w) = engines(name, dtype), models[name, dtype]
    toks = random_tokens(C.ALL[name]["vocab"], 150, 1)
    out = eng.step_tokens([("w", toks, list(range(len(toks))))]).cpu().numpy()
    eng.close_request("w")
    check(out, C.ALL[name], w, toks, dtype)
    eng.runner.cache.check_invariants()


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_against_decoding_token_by_token(name, dtype, models, engines):
    eng, (_, w) = engines(name, dtype), models[name, dtype]
    toks = random_tokens(C.ALL[name]["vocab"], 120, 2)
    ref = Reference(C.ALL[name], w, toks, dtype)
    n0 = 70
    outs = [eng.step_tokens([("d", toks[:n0], [n0 - 1])]).cpu().numpy()]
    for i in range(n0, len(toks)):
        outs.append(eng.step_tokens([("d", toks[i:i + 1], [0])]).cpu().numpy())
    eng.close_request("d")
    check(np.concatenate(outs), C.ALL[name], w, toks, dtype, rows=range(n0 - 1, len(toks)), ref=ref)
    # and everything one token at a time, from the first
    outs = [eng.step_tokens([("e", toks[i:i + 1], [0])]).cpu().numpy() for i in range(60)]
    eng.close_request("e")
    check(np.concatenate(outs), C.ALL[name], w, toks, dtype, rows=range(60), ref=ref)


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_changing_size(name, dtype, models, engines):
    eng, (_, w) = engines(name, dtype), models[name, dtype]
    toks = random_tokens(C.ALL[name]["vocab"], 180, 3)
    sizes = [17, 5, 2, 31, 2, 1, 33, 2, 16, 3, 7, 2, 64]
    outs, i = [], 0
    for s in sizes:
        s = min(s, len(toks) - i)
        if s <= 0:
            break
        outs.append(eng.step_tokens([("p", toks[i:i + s], list(range(s)))]).cpu().numpy())
        i += s
    eng.close_request("p")
    assert i == len(toks)
    check(np.concatenate(outs), C.ALL[name], w, toks, dtype)


@pytest.mark.parametrize("name,dtype", [("mix", "float32"), ("calm", "bfloat16"), ("windows", "bfloat16")])
def test_unequal_requests_together_with_pages_used_again(name, dtype, models, engines):
    lengths = [129, 70, 40, 97, 33, 150, 64, 5, 2]
    pool = 384
    eng, (_, w) = engines(name, dtype, kv_cache_tokens=pool, max_num_seqs=4), models[name, dtype]
    toks = {i: random_tokens(C.ALL[name]["vocab"], n, 100 + i) for i, n in enumerate(lengths)}
    got = {i: [] for i in toks}
    pages_seen = {}
    reused = False
    for entries, ends in mixed_schedule(lengths, pool, seed=11):
        batch = [(f"r{i}", toks[i][s:s + n], list(range(n))) for i, s, n in entries]
        out = eng.step_tokens(batch).cpu().numpy()
        r = 0
        for i, s, n in entries:
            got[i].append(out[r:r + n])
            r += n
            rc = eng.runner.cache.get(f"r{i}")
            for table in rc.tables:
                for p in table:
                    if p and pages_seen.setdefault(p, i) != i:
                        reused = True
        for i in ends:
            eng.close_request(f"r{i}")
        eng.runner.cache.check_invariants()
    assert reused, "the pool was so large that no page was handed out twice"
    assert eng.runner.cache.num_open() == 0
    for i in toks:
        check(np.concatenate(got[i]), C.ALL[name], w, toks[i], dtype)


@pytest.mark.parametrize("name,dtype", [("mix", "float32"), ("calm", "bfloat16")])
def test_long_decoding(name, dtype, models, engines):
    """Single tokens for hundreds of steps: the windows pass over decoded tokens and their pages go back, the
    latent layers' contexts grow over several partitions of keys."""
    eng, (_, w) = engines(name, dtype), models[name, dtype]
    toks = random_tokens(C.ALL[name]["vocab"], 420, 9)
    eng.step_tokens([("l", toks[:50], [])])
    free_before = [eng.runner.cache.num_free_pages(g) for g in range(len(eng.runner.cache.groups))]
    outs, rows = [], []
    for i in range(50, len(toks)):
        want = [0] if (i % 37 == 0 or i in (127, 128, 129, 255, 256, 257, 383, 384, 385, 419)) else []
        o = eng.step_tokens([("l", toks[i:i + 1], want)])
        if want:
            outs.append(o.cpu().numpy())
            rows.append(i)
    free_after = [eng.runner.cache.num_free_pages(g) for g in range(len(eng.runner.cache.groups))]
    windows = [g.window for g in eng.runner.cache.groups]
    assert any(w_ and w_ < 100 and a >= b - 3 for w_, a, b in zip(windows, free_after, free_before)), \
        "a short window's pages were not given back while decoding"
    eng.close_request("l")
    check(np.concatenate(outs), C.ALL[name], w, toks, dtype, rows=rows)


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens_of_a_sequence(name, dtype, models, engines):
    eng, (_, w) = engines(name, dtype), models[name, dtype]
    toks = random_tokens(C.ALL[name]["vocab"], 6, 4)
    outs = [eng.step_tokens([("f", toks[i:i + 1], [0])]).cpu().numpy() for i in range(3)]
    outs.append(eng.step_tokens([("f", toks[3:6], [0, 1, 2])]).cpu().numpy())
    eng.close_request("f")
    check(np.concatenate(outs), C.ALL[name], w, toks, dtype)
    one = eng.step_tokens([("g", toks[:1], [0, 0])]).cpu().numpy()
    eng.close_request("g")
    assert np.array_equal(one[0], one[1])
    check(one[:1], C.ALL[name], w, toks[:1], dtype)
    two = eng.step_tokens([("h", toks[:2], [1])]).cpu().numpy()
    eng.close_request("h")
    check(two, C.ALL[name], w, toks[:2], dtype, rows=[1])


# ---------------------------------------------------------------------------- what a position sees

def sharper(factor):
    """Queries and keys (and what the latent keys come from) multiplied, so that attention picks a key."""
    def patch(w):
        for n in list(w):
            if n.endswith(("mix.q", "mix.k", "mix.uk")):
                w[n] = w[n] * factor
    return patch


def standout_model(tmp, cfg, seeds, factor, make_tokens, row, least=0.05):
    """A one-layer model and two tokens (A, B) such that in a sequence of A's with one B the logits at ``row``
    differ from those of A's alone by more than ``least`` of the largest: whether B is seen decides them."""
    V = cfg["vocab"]
    for seed in seeds:
        d, w = make_model(tmp, cfg, seed, patch=sharper(factor))
        for A, B in ((seed % V, (seed * 7 + 3) % V), ((seed * 5 + 1) % V, (seed * 11 + 2) % V)):
            if A == B:
                continue
            with_b, alone = make_tokens(A, B), make_tokens(A, A)
            if rel_max(oracle(cfg, w, with_b)[row], oracle(cfg, w, alone)[row]) > least:
                return d, w, A, B
    raise AssertionError("no seed gave a key that stands out")


@pytest.fixture(scope="module")
def edge_model(tmp_path_factory):
    """One windowed layer (window 24, pages of 16) whose weights make one key stand out: sequences are all
    token A but for one B, so whether B is visible decides the logits."""
    size = 24
    cfg = C.one_windowed_layer(size=size)

    def toks(A, B):
        t = [A] * (size + 9)
        t[5] = B
        return t
    d, w, A, B = standout_model(tmp_path_factory.mktemp("edge"), cfg, range(40, 80), 4.0, toks, 5 + size - 1)
    return cfg, d, w, A, B


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_at_the_edges_of_the_window(dtype, edge_model):
    cfg, d, w, A, B = edge_model
    size = 24
    eng = engine_for(d, dtype)
    rounded = None if dtype == "float32" else torch.bfloat16
    for j in (0, 1, 5, 15, 16, 17, 31, 32, 40):          # where B stands: the first tokens, around page borders
        n = j + size + 4
        toks = [A] * n
        toks[j] = B
        ref = Reference(cfg, w, toks, dtype)
        base = oracle(cfg, w, [A] * n, rounded)
        inside, outside = j + size - 1, j + size
        # the construction holds: B decides the logits where the window shows it, and only there
        assert rel_max(ref.main[inside], base[inside]) > 0.02
        assert rel_max(ref.main[outside], base[outside]) < 1e-9
        rows = [max(j, 1) - 1, j, inside - 1, inside, outside, n - 1]
        out = eng.step_tokens([("w", toks, rows)]).cpu().numpy()
        eng.close_request("w")
        check(out, cfg, w, toks, dtype, rows=rows, ref=ref)
        # with portions cut at the edge: ..inside | outside.., and two tokens around it
        cuts = [inside - 1, 2, n - inside - 1]
        outs, i = [], 0
        for s in cuts:
            outs.append(eng.step_tokens([("c", toks[i:i + s], list(range(s)))]).cpu().numpy())
            i += s
        eng.close_request("c")
        check(np.concatenate(outs), cfg, w, toks, dtype, ref=ref)
        # decoding over the edge token by token
        n0 = max(j + 1, 2)
        outs = [eng.step_tokens([("d", toks[:n0], [n0 - 1])]).cpu().numpy()]
        for i in range(n0, n):
            outs.append(eng.step_tokens([("d", toks[i:i + 1], [0])]).cpu().numpy())
        eng.close_request("d")
        check(np.concatenate(outs), cfg, w, toks, dtype, rows=range(n0 - 1, n), ref=ref)
        eng.runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_one_in_the_denominator_and_the_distance_count(dtype, tmp_path):
    """A windowed layer with flat scores (queries and keys shrunk): the added one then takes a large share of
    every row and the distance bias orders the rest, so leaving either out would change every logit."""
    cfg = C.one_windowed_layer(size=12, heads=4, kv_heads=2, dim=16)

    def patch(w):
        for n in list(w):
            if n.endswith(("mix.q", "mix.k")):
                w[n] = w[n] * (0.02 if n.endswith("mix.q") else 1.0)
            if n.endswith("mix.o"):
                w[n] = w[n] * 4.0
    d, w = make_model(tmp_path, cfg, 91, patch=patch)
    toks = random_tokens(cfg["vocab"], 60, 12)
    ref = Reference(cfg, w, toks, dtype)
    # the plain implementation without the one, and without the bias: both far from the model
    m = cfg["layers"][0]["mixer"]
    h = P.layer_norm(w["embed"][toks].double() * cfg["embedding"]["scale"], w["l0.norm1"].double(), cfg["norm"]["eps"])
    k = (h @ w["l0.mix.k"].double().T).view(len(toks), 2, 16)
    q = (h @ w["l0.mix.q"].double().T).view(len(toks), 4, 16)
    s = q[:, 0] @ k[:, 0].T * m["scale"]
    a = P.biased_window_weights(s, P.head_slopes(4)[0], 12)
    assert float(a[30].sum()) < 0.95                               # the one takes its share
    assert float(a[30, 30] / a[30, 19]) > 10.0                     # the distance orders the keys
    eng = engine_for(d, dtype)
    outs = [eng.step_tokens([("s", toks[:41], list(range(41)))]).cpu().numpy()]
    for i in range(41, len(toks)):
        outs.append(eng.step_tokens([("s", toks[i:i + 1], [0])]).cpu().numpy())
    eng.close_request("s")
    check(np.concatenate(outs), cfg, w, toks, dtype, ref=ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(dtype, tmp_path):
    """One latent attention layer: one key near the start must reach queries 700 tokens later, in a prompt's
    tiles and over the partitions of a decoding token's context."""
    cfg = C.one_latent_layer()
    n = 700

    def toks_of(A, B):
        t = [A] * n
        t[1] = B
        return t
    d, w, A, B = standout_model(tmp_path, cfg, range(60, 100), 6.0, toks_of, n - 1)
    toks = toks_of(A, B)
    ref = Reference(cfg, w, toks, dtype)
    eng = engine_for(d, dtype, max_num_batched_tokens=1024)
    rows = [0, 1, 2, 127, 128, 129, 511, 512, 640, 698, 699]
    out = eng.step_tokens([("w", toks, rows)]).cpu().numpy()
    eng.close_request("w")
    check(out, cfg, w, toks, dtype, rows=rows, ref=ref)
    outs = [eng.step_tokens([("d", toks[:660], [659])]).cpu().numpy()]
    for i in range(660, n):
        outs.append(eng.step_tokens([("d", toks[i:i + 1], [0])]).cpu().numpy())
    eng.close_request("d")
    check(np.concatenate(outs), cfg, w, toks, dtype, rows=range(659, n), ref=ref)


# ---------------------------------------------------------------------------- other shapes of model

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_no_multiples_of_8(dtype, models, engines):
    """Width 100, a cached row of 26 entries, heads of 10 + 6 and 12, a rotation of two entries, keys of 20 and
    13, a window of one token, one expert chosen: no 16-byte pieces, no tensor-core tiles; a prompt in portions,
    then single tokens."""
    name = "odd" if dtype == "float32" else "odd_calm"
    eng, (_, w) = engines(name, dtype), models[name, dtype]
    cfg = C.ALL[name]
    toks = random_tokens(cfg["vocab"], 90, 21)
    ref = Reference(cfg, w, toks, dtype)
    outs, i = [], 0
    for s in (40, 2, 17, 1, 1, 29):
        outs.append(eng.step_tokens([("o", toks[i:i + s], list(range(s)))]).cpu().numpy())
        i += s
    eng.close_request("o")
    check(np.concatenate(outs), cfg, w, toks, dtype, ref=ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_and_what_it_leaves(dtype, models, engines):
    name = "mix" if dtype == "float32" else "calm"
    eng, (_, w) = engines(name, dtype), models[name, dtype]
    cfg = C.ALL[name]
    toks = random_tokens(cfg["vocab"], 430, 5)
    ref = Reference(cfg, w, toks, dtype)
    out = eng.step_tokens([("w", toks, list(range(len(toks))))]).cpu().numpy()
    eng.close_request("w")
    check(out, cfg, w, toks, dtype, ref=ref)
    outs, i = [], 0
    for s in (300, 2, 1, 1, 100, 26):
        outs.append(eng.step_tokens([("p", toks[i:i + s], list(range(s)))]).cpu().numpy())
        i += s
    eng.close_request("p")
    check(np.concatenate(outs), cfg, w, toks, dtype, ref=ref)


def test_every_pass_of_a_repeated_run_has_its_own_cache(tmp_path):
    """Three passes over the same two layers: were a pass to read or write another pass's cache, decoding
    would differ from the prompt run at once.  The residual stream after every layer run is compared too."""
    cfg = C.clone(C.MIX)
    d, w = make_model(tmp_path, cfg, 17)
    eng = engine_for(d, "float32")
    toks = random_tokens(cfg["vocab"], 40, 6)
    snaps = []
    blocks = eng.runner.model.blocks
    for blk in blocks:
        def wrapped(residual, pending, ctx, cache, state, _o=blk.forward):
            out = _o(residual, pending, ctx, cache, state)
            snaps.append((residual.clone() + (out.float() if out is not None else 0)).cpu().double())
            return out
        blk.forward = wrapped
    eng.step_tokens([("a", toks, [])])
    eng.close_request("a")
    for blk in blocks:
        del blk.forward
    layers = []
    P.forward(cfg, w, toks, layers)
    assert len(snaps) == len(layers) == 9
    for got, want in zip(snaps, layers):
        assert float((got - want).abs().max() / want.abs().max()) < 1e-5
    outs = [eng.step_tokens([("b", toks[:25], [24])]).cpu().numpy()]
    for i in range(25, 40):
        outs.append(eng.step_tokens([("b", toks[i:i + 1], [0])]).cpu().numpy())
    eng.close_request("b")
    check(np.concatenate(outs), cfg, w, toks, "float32", rows=range(24, 40))


@pytest.mark.parametrize("seed", [1, 2, 5, 8, 11, 14])
def test_configurations_drawn_at_random(seed, tmp_path):
    """Other layer orders, head counts, sizes, windows, repeated runs and constants: a prompt in portions with
    single tokens between them, then whole, in both engine types."""
    for dtype in ("float32", "bfloat16"):
        cfg = C.random_config(seed, calm=dtype != "float32")
        toks = random_tokens(cfg["vocab"], 330, seed)
        d, w = make_model(tmp_path, cfg, seed + (0 if dtype == "float32" else 100), sharpen=1.5)
        eng = engine_for(d, dtype)
        ref = Reference(cfg, w, toks, dtype)
        outs, i = [], 0
        for s in (130, 2, 1, 70, 1, 1, 1, 3, 121):
            outs.append(eng.step_tokens([("p", toks[i:i + s], list(range(s)))]).cpu().numpy())
            i += s
        eng.close_request("p")
        check(np.concatenate(outs), cfg, w, toks, dtype, ref=ref)
        whole = eng.step_tokens([("w", toks, list(range(len(toks))))]).cpu().numpy()
        eng.close_request("w")
        check(whole, cfg, w, toks, dtype, ref=ref)
        del eng


def test_decoding_as_cuda_graphs(models):
    """Single-token steps padded and replayed as CUDA graphs."""
    for name in ("mix", "latents"):
        cfg = C.ALL[name]
        d, w = models[name, "float32"]
        eng = engine_for(d, "float32", cuda_graphs=True)
        toks = random_tokens(cfg["vocab"], 90, 6)
        before = eng.runner.num_graph_steps
        outs = [eng.step_tokens([("d", toks[:50], [49])], graphs=True).cpu().numpy()]
        for i in range(50, len(toks)):
            outs.append(eng.step_tokens([("d", toks[i:i + 1], [0])], graphs=True).cpu().numpy())
        eng.close_request("d")
        assert eng.runner.num_graph_steps - before == 40
        check(np.concatenate(outs), cfg, w, toks, "float32", rows=range(49, len(toks)))


# ---------------------------------------------------------------------------- generation and programs

@pytest.mark.parametrize("name,dtype,opts", [
    ("mix", "float32", dict(async_scheduling=True, cuda_graphs=True, max_num_batched_tokens=48)),
    ("mix", "float32", dict(async_scheduling=False, cuda_graphs=False, max_num_batched_tokens=48)),
    ("windows", "float32", dict(async_scheduling=True, cuda_graphs=True, max_num_batched_tokens=64)),
    ("calm", "bfloat16", dict(async_scheduling=False, max_num_batched_tokens=32)),
])
def test_greedy_generation_through_the_scheduler(name, dtype, opts, models):
    """The framework's own entry point: requests of unequal length admitted by the scheduler, prompts in
    portions under a small token budget, decoding beside them; every generated token is the oracle's arg
    max given the tokens before it (or within the dtype's margin of it)."""
    from redline_b200.runtime import Engine
    d, w = models[name, dtype]
    cfg = C.ALL[name]
    prompts = [random_tokens(cfg["vocab"], n, 30 + i) for i, n in enumerate((5, 70, 33, 1, 18, 90))]
    eng = Engine(d, dtype=dtype, max_seqs=4, max_seq_len=256, kv_cache_tokens=512, **opts)
    outs = eng.generate(prompts, max_new_tokens=12, ignore_eos=True)
    margin = 1e-3 if dtype == "float32" else 0.25
    assert (eng._engine.runner.num_graph_steps > 0) == bool(opts.get("cuda_graphs", True))
    for p, o in zip(prompts, outs):
        assert len(o["output_ids"]) == 12
        seq = p + o["output_ids"]
        ref = oracle(cfg, w, seq[:-1], None if dtype == "float32" else torch.bfloat16)
        for i, tok in enumerate(o["output_ids"]):
            row = ref[len(p) - 1 + i]
            assert row[tok] >= row.max() - margin, (name, dtype, i, tok, int(row.argmax()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, models, tmp_path):
    name = "mix" if dtype == "float32" else "calm"
    model_dir, w = models[name, dtype]
    cfg = C.ALL[name]
    V = cfg["vocab"]
    a, b = random_tokens(V, 70, 11), random_tokens(V, 45, 12)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[40:42], "want": [1]},
                                {"id": "b", "tokens": b[:45], "want": [44]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[42:43], "want": []}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": a[43:70], "want": [26]},
                                {"id": "c", "tokens": b[:2], "want": [1, 0]}], "end": ["a", "c"]},
    ]
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_dir,
                           "--dtype", dtype, "--out", str(out), "--max-tokens", "256"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                          timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    assert not (out / "2.f32").exists()
    f = {i: np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V) for i in (0, 1, 3)}
    check(np.concatenate([f[0], f[1][:1], f[3][:1]]), cfg, w, a, dtype, rows=[0, 39, 41, 69])
    check(f[1][1:], cfg, w, b, dtype, rows=[44])
    check(f[3][1:], cfg, w, b[:2], dtype, rows=[1, 0])


def test_command_line_with_random_weights(tmp_path):
    """`bin/redline_generate --random-weights`: the framework writes a seeded Venezen model from a config.json,
    generates greedily, and the plain implementation, reading that folder, agrees with every token."""
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(C.MIX))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "redline_generate"), "--random-weights", str(cfg_path),
                        "--weights-seed", "5", "--model", str(tmp_path / "rand"), "--dtype", "float32", "--prompt-ids",
                        "1,2,3,50,9", "--prompt-ids", "7", "--max-new-tokens", "8", "--ignore-eos", "--max-seq-len", "64",
                        "--kv-cache-tokens", "256", "--max-seqs", "2"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(x) for x in r.stdout.splitlines() if x.startswith("{")]
    assert [x["id"] for x in lines] == [0, 1] and all(len(x["output_ids"]) == 8 for x in lines)
    cfg, w = P.read_model_dir(str(tmp_path / "rand"))
    for prompt, line in zip(([1, 2, 3, 50, 9], [7]), lines):
        seq = prompt + line["output_ids"]
        ref = oracle(cfg, w, seq[:-1])
        for i, tok in enumerate(line["output_ids"]):
            row = ref[len(prompt) - 1 + i]
            assert row[tok] >= row.max() - 1e-3, (i, tok, int(row.argmax()))
