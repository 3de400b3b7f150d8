"""The kernels that came with Venezen, each against a float64 restatement: the per-head products (CUDA cores and
tensor cores), the kernel between a latent attention's projection and its cache (norm, rotation, cache write),
attention whose values are the leading entries of its keys with a distance bias and a constant sink (prompt
portions on tensor cores and CUDA cores, single tokens over partitions) over shuffled pages, and the router with
a choice bias, identity experts and scaled weights."""

import math

import pytest
import torch

import plain_venezen as P

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel(a, b):
    return float((a.double().cpu() - b.double().cpu()).abs().max() / (b.double().abs().max() + 1e-30))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,N,K", [(1, 3, 40, 16), (37, 2, 24, 48), (150, 5, 130, 20), (70, 1, 7, 13), (129, 4, 64, 192)])
def test_per_head_products(dtype, T, H, N, K):
    """y[t, h] = W_h x[t, h] with heads laid out at strides of their own inside wider rows."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(T + N)
    xh, yh = K + 6, N + 2                      # a head's stride in the rows of x and of y
    x = torch.randn(T, 4 + H * xh, generator=g).to(dtype)
    w = (torch.randn(H, N, K, generator=g) / math.sqrt(K)).to(dtype)
    want = torch.einsum("thk,hnk->thn", torch.stack([x[:, 4 + h * xh:4 + h * xh + K] for h in range(H)], 1).double(), w.double())
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    for impl in (0, 1):
        y = torch.full((T, 2 + H * yh), float("nan"), dtype=dtype, device=DEV)
        kernels.head_linear(x.to(DEV), 4, xh, w.to(DEV), y, 2, yh, impl=impl)
        got = torch.stack([y[:, 2 + h * yh:2 + h * yh + N] for h in range(H)], 1)
        assert rel(got, want) < tol, impl
        # nothing but the heads' outputs is written
        mask = torch.ones_like(y, dtype=torch.bool)
        for h in range(H):
            mask[:, 2 + h * yh:2 + h * yh + N] = False
        assert torch.isnan(y[mask]).all()
    # a row's result does not depend on what else is in the launch
    if T > 20:
        a = torch.zeros((T, 2 + H * yh), dtype=dtype, device=DEV)
        b = torch.zeros((T, 2 + H * yh), dtype=dtype, device=DEV)
        kernels.head_linear(x.to(DEV), 4, xh, w.to(DEV), a, 2, yh)
        kernels.head_linear(x[17:20].contiguous().to(DEV), 4, xh, w.to(DEV), b, 2, yh, tokens=3)
        assert torch.equal(a[17:20], b[:3])


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("H,dn,dr,rank,rot", [(3, 16, 8, 40, 8), (2, 10, 6, 20, 2), (1, 32, 32, 64, 32), (4, 8, 16, 24, 8), (2, 16, 0, 32, 0)])
def test_latent_between_projection_and_cache(dtype, tol, H, dn, dr, rank, rot):
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(H * rank + dr)
    T, ps, eps, base = 21, 16, 1e-5, 300.0
    key = rank + dr
    proj = torch.randn(T, H * (dn + dr) + key, generator=g).to(dtype)
    nw = (1.0 + 0.2 * torch.randn(rank, generator=g)).to(dtype)
    pos = torch.randint(0, 200, (T,), generator=g).to(torch.int32)
    slots = torch.randperm(5 * ps, generator=g)[:T].to(torch.int32)
    slots[3] = -1                                       # a token without a slot writes nothing
    cos = sin = None
    if dr > 0:
        ang = torch.arange(200, dtype=torch.float64)[:, None] * torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)],
                                                                             dtype=torch.float64)[None, :]
        cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    cache = torch.full((5, 1, ps, key), float("nan"), dtype=dtype, device=DEV)
    qa = torch.full((T, H * key), float("nan"), dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.latent_prep(proj.to(DEV), pos.to(DEV), T, H, dn, dr, rank, rot, nw.to(DEV), eps, cos, sin, qa, slots.to(DEV), cache,
                        ps, status)
    assert int(status.item()) == 0
    p64 = proj.double()
    craw = p64[:, H * (dn + dr):]
    c = P.rms_norm(craw[:, :rank], nw.double(), eps)
    flat = cache.view(5 * ps, key)
    for t in range(T):
        kr = P.rotate_halves(craw[t:t + 1, rank:], base, rot, [int(pos[t])])[0] if dr > 0 else craw[t, rank:]
        if int(slots[t]) >= 0:
            assert rel(flat[int(slots[t])], torch.cat([c[t], kr])) < tol
        for h in range(H):
            if dr > 0:
                q = p64[t:t + 1, h * (dn + dr) + dn:(h + 1) * (dn + dr)]
                assert rel(qa[t, h * key + rank:(h + 1) * key], P.rotate_halves(q, base, rot, [int(pos[t])])[0]) < tol
            assert torch.isnan(qa[t, h * key:h * key + rank]).all()          # the unrotated part is the product's to fill
    written = torch.zeros(5 * ps, dtype=torch.bool)
    written[slots[slots >= 0].long()] = True
    assert torch.isnan(flat[~written]).all()
    if dr > 0:
        kernels.latent_prep(proj.to(DEV), torch.full((T,), 500, dtype=torch.int32, device=DEV), T, H, dn, dr, rank, rot,
                            nw.to(DEV), eps, cos, sin, qa, None, cache, ps, status)
        assert int(status.item()) == 2


def plain_attention(q, k, v, scale, size, slopes, sink):
    """q [L, H, D], k [L, G, D], v [L, G, DV] (float64) -> [L, H, DV]: causal, window ``size`` (0: none), the
    distance bias of ``slopes`` and exp(sink) in the denominator (None: neither)."""
    L, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(L, H, v.shape[2], dtype=torch.float64)
    i = torch.arange(L).view(L, 1)
    j = torch.arange(L).view(1, L)
    seen = (j <= i) & ((i - j < size) if size > 0 else torch.ones(L, L, dtype=torch.bool))
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * scale
        if slopes is not None:
            s = s - slopes[h] * (i - j).double()
        s = s.masked_fill(~seen, -math.inf)
        mx = s.max(-1, keepdim=True).values
        if sink is not None:
            mx = torch.clamp(mx, min=sink)
        e = torch.exp(s - mx)
        den = e.sum(-1, keepdim=True) + (torch.exp(sink - mx) if sink is not None else 0.0)
        out[:, h] = (e / den) @ v[:, g]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,DV,size,biased", [
    (4, 2, 32, 32, 24, True),        # the keys are the values
    (3, 1, 20, 20, 1, True),         # ... at sizes the tensor cores do not take, a window of one token
    (6, 3, 16, 16, 130, True),
    (8, 1, 80, 64, 0, False),        # one key head for all query heads, the value the keys' first 64 entries
    (3, 1, 26, 20, 0, False),
    (2, 1, 160, 128, 0, False),
    (5, 1, 48, 48, 0, False),        # no rotated part: the whole row is the value
    (2, 1, 320, 288, 0, False),      # rows longer than the tensor-core kernel takes
])
def test_attention_over_keys_that_are_the_values(dtype, H, G, D, DV, size, biased):
    """A portion of 150 tokens after 70 cached ones and, in the same cache, single tokens at several contexts,
    over pages handed out in a shuffled order; cache rows that no query may read hold NaN.  There is one cache:
    the kernels read a value as the first DV entries of a key row."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(H * D + DV + size)
    ps, L, p0 = 16, 220, 70
    n = L - p0
    scale = 0.3
    q = torch.randn(L, H, D, generator=g).to(dtype)
    k = torch.randn(L, G, D, generator=g).to(dtype)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]) if biased else None
    sink = 0.0 if biased else None
    pages = (L + ps - 1) // ps
    perm = (torch.randperm(pages + 3, generator=g) + 1)[:pages].to(torch.int32)
    kc = torch.full((pages + 4, G, ps, D), float("nan"), dtype=dtype)
    for j in range(L):
        kc[perm[j // ps], :, j % ps] = k[j]
    if size > 0:
        for j in range(0, max(0, p0 - size + 1)):
            kc[perm[j // ps], :, j % ps] = float("nan")
    kc = kc.to(DEV)
    table = torch.zeros(1, pages + 2, dtype=torch.int32)
    table[0, :pages] = perm
    table = table.to(DEV)
    want = plain_attention(q.double(), k.double(), k.double()[:, :, :DV], scale, size, slopes, sink)[p0:].reshape(n, -1)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    buf = q[p0:].reshape(n, -1).contiguous().to(DEV)
    sl = slopes.to(DEV) if biased else None
    sk = torch.zeros(H, device=DEV) if biased else None
    stride = D if DV != D else 0
    positions = torch.arange(p0, L, dtype=torch.int32, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)      # noqa: E731
    tile_seq, tile_tok, tile_rows = i32([0, 0]), i32([0, 128]), i32([128, n - 128])
    impls = [1] + ([2] if dtype == torch.bfloat16 and D % 16 == 0 and DV % 16 == 0 and D <= 256 else [])
    for impl in impls:
        out = torch.full((n, H * DV), float("nan"), dtype=dtype, device=DEV)
        kernels.maps_attn_prefill(buf, buf.stride(0), kc, kc, table, tile_seq, tile_tok, tile_rows, positions, out, 2,
                                  128, H, G, D, DV, 1, ps, size, 0, scale, 0.0, 0.0, 1.0, 1e-5, False, sk, None, 0,
                                  impl=impl, slopes=sl, v_stride=stride)
        assert rel(out, want) < tol, impl
    ends = [p0 + 1, 128, 129, 130, L]
    rows = [e - 1 - p0 for e in ends]
    items = i32([[r, 0, e, 0] for r, e in zip(rows, ends)])
    parts = (L + 127) // 128
    part_o = torch.full((len(ends) * H * parts * DV,), float("nan"), device=DEV)
    part_ml = torch.full((len(ends) * H * parts * 2,), float("nan"), device=DEV)
    out = torch.zeros((n, H * DV), dtype=dtype, device=DEV)
    kernels.maps_attn_decode(buf, buf.stride(0), kc, kc, table, items, part_o, part_ml, parts, out, len(ends), H, G, D, DV,
                             1, ps, size, 0, scale, 0.0, 0.0, 1.0, 1e-5, False, sk, None, 0, slopes=sl, v_stride=stride)
    assert rel(out[rows], want[rows]) < tol


def test_the_distance_bias_and_the_added_one_show():
    """Equal keys and zero queries: without the bias and the sink every weight would be 1 / keys; with them a
    head's output is the value times sum(e^(-m d)) / (1 + sum(e^(-m d)))."""
    from redline_b200.ops import kernels
    H, D, L, ps, size = 2, 16, 40, 16, 12
    q = torch.zeros(L, H * D, device=DEV)
    row = torch.arange(1, D + 1, dtype=torch.float32)
    kc = torch.zeros(4, 1, ps, D, device=DEV)
    kc[1:4] = row.to(DEV)
    table = torch.tensor([[1, 2, 3, 0]], dtype=torch.int32, device=DEV)
    slopes = torch.tensor([0.5, 0.03125], device=DEV)
    sk = torch.zeros(H, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)      # noqa: E731
    out = torch.zeros(L, H * D, device=DEV)
    kernels.maps_attn_prefill(q, H * D, kc, kc, table, i32([0]), i32([0]), i32([L]), torch.arange(L, dtype=torch.int32, device=DEV),
                              out, 1, 128, H, 1, D, D, 1, ps, size, 0, 1.0, 0.0, 0.0, 1.0, 1e-5, False, sk, None, 0, slopes=slopes)
    for i in (0, 5, 11, 12, 39):
        for h, m in enumerate((0.5, 0.03125)):
            e = sum(math.exp(-m * d) for d in range(min(i + 1, size)))
            assert rel(out[i, h * D:(h + 1) * D], row.double() * e / (1.0 + e)) < 1e-5


@pytest.mark.parametrize("E,I,top,renorm", [(6, 2, 3, True), (5, 0, 1, True), (2, 3, 5, True), (40, 3, 4, False)])
def test_router_with_a_choice_bias_identity_outputs_and_scaled_weights(E, I, top, renorm):
    """Softmax over experts and identity outputs; the choice by score + bias, the weights the scores themselves,
    divided by their sum + floor and multiplied by a constant; rows whose choice is a close call are left out."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(E + top)
    T, n = 300, E + I
    z = 2.0 * torch.randn(T, n, generator=g)
    bias = 0.05 * torch.randn(n, generator=g)
    s = torch.softmax(z.double(), -1)
    ranked = torch.sort(s + bias.double(), -1, descending=True)
    pick = ranked.indices[:, :top]
    clear = torch.ones(T, dtype=torch.bool) if top == n else (ranked.values[:, top - 1] - ranked.values[:, top]) > 1e-5
    chosen = torch.gather(s, 1, pick)
    want = (chosen / (chosen.sum(-1, keepdim=True) + 1e-20) if renorm else chosen) * 2.5
    choice = torch.zeros(T * top, dtype=torch.int32, device=DEV)
    weight = torch.zeros(T * top, dtype=torch.float32, device=DEV)
    kernels.moe_route(z.to(DEV), None, choice, weight, T, 1, 1, 1, top, softmax=True, renorm=renorm,
                      choice_bias=bias.to(DEV), weight_scale=2.5, renorm_floor=1e-20)
    got = choice.view(T, top).cpu().long()
    assert clear.sum() > T // 2
    assert torch.equal(got[clear], pick[clear])
    assert rel(weight.view(T, top)[clear], want[clear]) < 1e-5
    # the pairs of identity outputs get no tiles, and their term of the weighted sum is the input row
    order = torch.zeros(T * top, dtype=torch.int32, device=DEV)
    tiles = kernels.moe_max_tiles(T * top, n)
    te, tb, tr = (torch.zeros(tiles, dtype=torch.int32, device=DEV) for _ in range(3))
    meta = torch.zeros(4, dtype=torch.int32, device=DEV)
    kernels.moe_group(choice, T * top, n, order, te, tb, tr, meta, tiled=E)
    nt = int(meta[0])
    assert int(tr[:nt].sum()) == int((got < E).sum()) and (te[:nt] < E).all()
    listed = torch.cat([order[int(b):int(b) + int(r)] for b, r in zip(tb[:nt].tolist(), tr[:nt].tolist())]) if nt else order[:0]
    assert (choice[listed.long()] < E).all()
    W = 24
    x = torch.randn(T, W, generator=g).to(DEV)
    y = torch.randn(T * top, W, generator=g).to(DEV)
    out = torch.zeros(T, W, device=DEV)
    kernels.moe_combine(y, weight, None, out, T, top, choice=choice, real_experts=E, x=x)
    terms = torch.where((choice.view(T, top, 1) >= E), x.view(T, 1, W).expand(T, top, W), y.view(T, top, W))
    assert rel(out, (weight.view(T, top, 1).double() * terms.double()).sum(1)) < 1e-5
