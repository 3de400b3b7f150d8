"""Vizotar's kernels alone, each against the plain implementation's function of the same mechanism
(tests/plain_vizotar.py) or a float64 restatement here: the delta rule's recurrence from states that earlier
tokens left (unequal sequences in slots out of order, long sequences and single tokens, key sizes that are no
multiples of 4, values in both activation types, foreign slots untouched), what it is fed (unit vectors, beta,
decays), the per-head norm with gate, the short convolution with its carried inputs (portions of every length
around the number of taps, large steps that walk several tokens per thread, single-token steps), the streams'
boundary kernel in all its modes, and the normed mean of a pair with biases."""

import numpy as np
import pytest
import torch

import plain_vizotar as P

pytestmark = pytest.mark.gpu

F64 = torch.float64


def dev():
    return torch.device("cuda:0")


def seq_index(lengths):
    return torch.tensor([i for i, n in enumerate(lengths) for _ in range(n)], dtype=torch.int32, device=dev())


def close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max()) + 1e-30
    err = float((got - want).abs().max()) / scale
    assert err < tol, f"differs by {err:.3e} of the largest entry"


# ---------------------------------------------------------------------------- the delta rule

def plain_delta_from(S, q, k, v, beta, decay):
    """The plain recurrence from a given state; returns (o, S)."""
    out = []
    for t in range(q.shape[0]):
        S = decay[t][:, None] * S
        d = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], d)
        out.append(S.T @ q[t])
    return torch.stack(out), S


@pytest.mark.parametrize("D,DV,H,HQ,lengths,act", [
    (16, 24, 4, 2, (40, 1, 3, 17), torch.float32),        # mixed: the few-groups layout
    (16, 24, 4, 2, (70,), torch.bfloat16),                # long: the many-groups layout
    (13, 20, 3, 3, (33, 2), torch.float32),               # rows beyond D stay zero; plain 4-byte copies
    (13, 7, 3, 1, (90,), torch.bfloat16),                 # odd value size: values staged by plain loads
    (64, 40, 2, 1, (1, 1, 1), torch.bfloat16),            # single tokens
    (128, 72, 2, 2, (150, 9), torch.float32),             # 16 row groups over a long sequence, 4 over the mix
    (24, 16, 2, 2, (8, 16, 9), torch.float32),            # exactly one and two staged batches, and one token more
    (256, 24, 1, 1, (40, 3), torch.float32),              # the largest key size: four tokens staged at a time
    (256, 16, 2, 1, (80,), torch.bfloat16),
    (48, 40, 6, 2, (5, 64, 2), torch.bfloat16),           # three heads to a q/k head
])
def test_recurrence_from_states_in_shuffled_slots(D, DV, H, HQ, lengths, act):
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(D * 100 + DV)
    T, S_n = sum(lengths), len(lengths)
    slots = S_n + 3
    q = torch.nn.functional.normalize(torch.randn(T, HQ, D, generator=g, dtype=F64), dim=-1) * D ** -0.5
    k = torch.nn.functional.normalize(torch.randn(T, HQ, D, generator=g, dtype=F64), dim=-1)
    v = torch.randn(T, H, DV, generator=g, dtype=F64).to(act).to(F64)
    beta = torch.rand(T, H, generator=g, dtype=F64)
    decay = 0.5 + 0.5 * torch.rand(T, H, D, generator=g, dtype=F64)
    state = torch.randn(slots, H, D, DV, generator=g, dtype=F64) * 0.3
    order = torch.randperm(slots, generator=g)[:S_n].tolist()
    # two calls: the first half of every sequence, then the rest from what the first call left
    cuts = [max(1, n // 2) if n > 1 else 1 for n in lengths]
    st = state.float().reshape(slots, -1).contiguous().to(dev())
    want_o = torch.zeros(T, H, DV, dtype=F64)
    want_state = state.clone()
    starts = np.concatenate([[0], np.cumsum(lengths)]).tolist()
    for s, n in enumerate(lengths):
        a = starts[s]
        for h in range(H):
            hq = h // (H // HQ)
            o, S = plain_delta_from(want_state[order[s], h], q[a:a + n, hq], k[a:a + n, hq], v[a:a + n, h], beta[a:a + n, h],
                                    decay[a:a + n, h])
            want_o[a:a + n, h] = o
            want_state[order[s], h] = S
    got_o = torch.zeros(T, H * DV, device=dev())
    for part in (0, 1):
        rows, lens = [], []
        for s, n in enumerate(lengths):
            lo, hi = (0, cuts[s]) if part == 0 else (cuts[s], n)
            lens.append(hi - lo)
            rows.extend(range(starts[s] + lo, starts[s] + hi))
        keep = [i for i, n in enumerate(lens) if n > 0]
        if not keep:
            continue
        idx = torch.tensor(rows)
        qq = q[idx].reshape(len(rows), -1).float().contiguous().to(dev())
        kk = k[idx].reshape(len(rows), -1).float().contiguous().to(dev())
        # the values are columns of a wider buffer, as in the mixer
        wide = torch.zeros(len(rows), H * DV + 6, dtype=act, device=dev())
        wide[:, 2:2 + H * DV] = v[idx].reshape(len(rows), -1).to(act).to(dev())
        bb = beta[idx].float().contiguous().to(dev())
        dd = decay[idx].reshape(len(rows), -1).float().contiguous().to(dev())
        out = torch.full((len(rows), H * DV), float("nan"), device=dev())
        kernels.delta_rule(qq, kk, wide[:, 2:2 + H * DV], bb, dd, seq_index([lens[i] for i in keep]),
                           torch.tensor([order[i] for i in keep], dtype=torch.int32, device=dev()), st, out,
                           len(rows), len(keep), H, HQ, D, DV)
        got_o[idx.to(dev())] = out
    torch.cuda.synchronize()
    close(got_o.reshape(T, H, DV), want_o, 2e-5)
    close(st.reshape(slots, H, D, DV), want_state, 2e-5)
    untouched = [s for s in range(slots) if s not in order]
    assert torch.equal(st.reshape(slots, H, D, DV)[untouched].cpu(), state.float()[untouched])


def test_what_the_recurrence_is_fed_and_the_heads_norm():
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(5)
    T, H, HQ, D, DV = 37, 6, 3, 20, 12
    for act in (torch.float32, torch.bfloat16):
        x = torch.randn(T, 2 * HQ * D + 9, generator=g).to(act)
        zb, za = torch.randn(T, H, generator=g), 3.0 * torch.randn(T, H * D, generator=g)
        dt, a_log = torch.randn(H * D, generator=g), torch.randn(H, generator=g)
        q = torch.empty(T, HQ * D, device=dev())
        k, beta, decay = torch.empty_like(q), torch.empty(T, H, device=dev()), torch.empty(T, H * D, device=dev())
        kernels.delta_prep(x.to(dev()), 4, 4 + HQ * D, HQ, H, D, 0.37, 1e-6, zb.to(dev()), za.to(dev()), dt.to(dev()),
                           a_log.to(dev()), q, k, beta, decay, T)
        xd = x.double()
        xq, xk = xd[:, 4:4 + HQ * D].reshape(T, HQ, D), xd[:, 4 + HQ * D:4 + 2 * HQ * D].reshape(T, HQ, D)
        close(q.reshape(T, HQ, D), 0.37 * xq / torch.sqrt((xq * xq).sum(-1, keepdim=True) + 1e-6), 1e-5)
        close(k.reshape(T, HQ, D), xk / torch.sqrt((xk * xk).sum(-1, keepdim=True) + 1e-6), 1e-5)
        close(beta, P.sigmoid(zb.double()), 1e-6)
        want = torch.exp(-torch.exp(a_log.double())[:, None] * P.softplus(za.double() + dt.double()).reshape(T, H, D))
        close(decay.reshape(T, H, D), want, 1e-5)
        o = torch.randn(T, H * DV, generator=g)
        gate = torch.randn(T, H * DV + 3, generator=g).to(act)
        w = (1.0 + 0.1 * torch.randn(DV, generator=g)).to(act)
        y = torch.empty(T, H * DV + 5, dtype=act, device=dev())
        kernels.head_gated_norm(o.to(dev()), gate.to(dev())[:, 3:], w.to(dev()), y[:, 1:1 + H * DV], T, H, DV, 1e-5, dim=D)
        od = o.double().reshape(T, H, DV)
        want = od / torch.sqrt((od * od).mean(-1, keepdim=True) + 1e-5) * w.double() \
            * P.sigmoid(gate.double()[:, 3:].reshape(T, H, DV))
        close(y[:, 1:1 + H * DV].reshape(T, H, DV), want, 1e-5 if act == torch.float32 else 1e-2)


# ---------------------------------------------------------------------------- the short convolution

@pytest.mark.parametrize("taps,channels,act_silu,dtype", [
    (4, 70, False, torch.float32), (3, 33, True, torch.float32), (2, 256, True, torch.bfloat16), (1, 48, True, torch.float32),
    (8, 20, False, torch.float32),
])
def test_convolution_over_portions_of_every_length(taps, channels, act_silu, dtype):
    """Three sequences fed in portions of 1 .. taps + 2 tokens (and one long one), interleaved in steps with
    slots out of order; single-token steps take the one-launch path."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(taps * 7 + channels)
    lengths = (41, 29, 57)
    us = [torch.randn(n, channels, generator=g).to(dtype).double() for n in lengths]
    w = (0.5 * torch.randn(channels, taps, generator=g)).to(dtype)
    bias = torch.randn(channels, generator=g)
    want = []
    for u in us:
        y = P.causal_conv(u + bias.double(), w.double())
        want.append(P.silu(y) if act_silu else y)
    slots = [4, 0, 2]
    state = torch.zeros(6, max(taps - 1, 1) * channels, device=dev())
    state[1] = 7.0                                                  # a foreign slot
    done = [0, 0, 0]
    got = [torch.zeros(n, channels, dtype=F64) for n in lengths]
    rng = np.random.RandomState(taps)
    step = 0
    while any(d < n for d, n in zip(done, lengths)):
        live = [s for s in range(3) if done[s] < lengths[s]]
        single = step % 3 == 2
        lens = [1 if single else min(int(rng.randint(1, taps + 3)) if step % 5 else 19, lengths[s] - done[s]) for s in live]
        x = torch.cat([us[s][done[s]:done[s] + n] for s, n in zip(live, lens)]).to(dtype)
        wide = torch.zeros(x.shape[0], channels + 10, dtype=dtype, device=dev())
        wide[:, 3:3 + channels] = x.to(dev())
        y = torch.empty(x.shape[0], channels + 4, dtype=dtype, device=dev())
        kernels.short_conv(wide, 3, w.to(dev()), bias.to(dev()), y, 2, kernels.ACT_SILU if act_silu else kernels.ACT_NONE,
                           seq_index(lens), torch.tensor([slots[s] for s in live], dtype=torch.int32, device=dev()), state,
                           x.shape[0], single=single)
        at = 0
        for s, n in zip(live, lens):
            got[s][done[s]:done[s] + n] = y[at:at + n, 2:2 + channels].double().cpu()
            done[s] += n
            at += n
        step += 1
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for a, b in zip(got, want):
        close(a, b, tol)
    assert float(state[1].min()) == 7.0 and float(state[1].max()) == 7.0
    if taps > 1:                                                    # the slots hold the last inputs, bias added, oldest first
        for s in range(3):
            tail = (us[s] + bias.double())[-(taps - 1):]
            close(state[slots[s], :(taps - 1) * channels].reshape(taps - 1, channels)[-tail.shape[0]:], tail, 1e-6)


def test_convolution_of_a_large_step():
    """Thousands of tokens: a thread walks several of them; a second sequence begins in the middle of a tile."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(3)
    taps, channels, lengths = 4, 512, (1029, 1, 1030)
    us = [torch.randn(n, channels, generator=g) for n in lengths]
    w = 0.5 * torch.randn(channels, taps, generator=g)
    prev = [torch.randn(taps - 1, channels, generator=g) for _ in lengths]          # what earlier steps left
    state = torch.zeros(4, (taps - 1) * channels, device=dev())
    for s in range(3):
        state[s + 1] = prev[s].reshape(-1).to(dev())
    x = torch.cat(us).to(dev())
    y = torch.empty_like(x)
    kernels.short_conv(x, 0, w.to(dev()), None, y, 0, kernels.ACT_NONE, seq_index(lengths),
                       torch.tensor([1, 2, 3], dtype=torch.int32, device=dev()), state, x.shape[0])
    at = 0
    for s, n in enumerate(lengths):
        full = P.causal_conv(torch.cat([prev[s], us[s]]).double(), w.double())[taps - 1:]
        close(y[at:at + n], full, 1e-5)
        close(state[s + 1].reshape(taps - 1, channels), torch.cat([prev[s], us[s]])[-(taps - 1):], 1e-6)
        at += n


# ---------------------------------------------------------------------------- streams and pairs

@pytest.mark.parametrize("n,width,dtype", [(1, 100, torch.float32), (4, 320, torch.bfloat16), (3, 1000, torch.float32),
                                           (8, 64, torch.bfloat16), (5, 4100, torch.float32)])
def test_streams_boundary_in_all_its_modes(n, width, dtype):
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(n * 31 + width)
    T = 19
    emb = torch.randn(T, width, generator=g)
    mix = torch.eye(n) + 0.2 * torch.randn(n, n, generator=g)
    out_w, read_in = torch.randn(n, generator=g), torch.randn(n, generator=g)
    norm_w = (1.0 + 0.1 * torch.randn(width, generator=g)).to(dtype)
    streams = torch.full((T + 2, n, width), float("nan"), device=dev())
    x = torch.empty(T, width + 8, dtype=dtype, device=dev())
    # every stream starts as the embedding; the first sublayer's input
    kernels.streams_step(streams, T, init=emb.to(dev()), read_in=read_in.to(dev()), norm_w=norm_w.to(dev()), eps=1e-5,
                         normed=x[:, 8:])
    X = emb.double()[:, None, :].repeat(1, n, 1)
    close(streams[:T], X, 1e-7)
    close(x[:, 8:], P.rms_norm((read_in.double()[None, :, None] * X).sum(1), norm_w.double(), 1e-5),
          1e-5 if dtype == torch.float32 else 1e-2)
    # a sublayer's output written back, the next input formed, and the sum of the streams
    y = torch.randn(T, width + 2, generator=g).to(dtype)
    total = torch.empty(T, width, device=dev())
    kernels.streams_step(streams, T, y=y.to(dev())[:, 2:], mix=mix.to(dev()), out_w=out_w.to(dev()), read_in=read_in.to(dev()),
                         norm_w=norm_w.to(dev()), eps=1e-5, normed=x[:, 8:], total=total)
    X = torch.einsum("st,bsw->btw", mix.double(), X) + out_w.double()[None, :, None] * y.double()[:, None, 2:]
    close(streams[:T], X, 1e-5)
    close(total, X.sum(1), 1e-5)
    close(x[:, 8:], P.rms_norm((read_in.double()[None, :, None] * X).sum(1), norm_w.double(), 1e-5),
          1e-5 if dtype == torch.float32 else 1e-2)
    assert torch.isnan(streams[T:]).all()                           # rows beyond the step's tokens are not touched
    # the last boundary: write back and sum only
    kernels.streams_step(streams, T, y=y.to(dev())[:, 2:], mix=mix.to(dev()), out_w=out_w.to(dev()), total=total)
    X = torch.einsum("st,bsw->btw", mix.double(), X) + out_w.double()[None, :, None] * y.double()[:, None, 2:]
    close(total, X.sum(1), 1e-5)


@pytest.mark.parametrize("width,dtype,biases", [(100, torch.float32, (True, False)), (1024, torch.bfloat16, (True, True)),
                                                (2050, torch.float32, (False, False))])
def test_normed_mean_of_a_pair(width, dtype, biases):
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(width)
    T = 23
    a, b = torch.randn(T, width + 4, generator=g).to(dtype), (3.0 * torch.randn(T, width, generator=g)).to(dtype)
    wa, wb = (1.0 + 0.1 * torch.randn(width, generator=g)).to(dtype), (1.0 + 0.1 * torch.randn(width, generator=g)).to(dtype)
    ba, bb = [torch.randn(width, generator=g) if on else None for on in biases]
    out = torch.empty(T, width, dtype=dtype, device=dev())
    kernels.pair_norm_mean(a.to(dev())[:, 4:], wa.to(dev()), 0.5, b.to(dev()), wb.to(dev()), 0.25, out, 1e-6, rows=T,
                           bias_a=ba.to(dev()) if ba is not None else None, bias_b=bb.to(dev()) if bb is not None else None)
    xa = a.double()[:, 4:] + (ba.double() if ba is not None else 0.0)
    xb = b.double() + (bb.double() if bb is not None else 0.0)
    want = 0.5 * P.rms_norm(xa, wa.double(), 1e-6) + 0.25 * P.rms_norm(xb, wb.double(), 1e-6)
    close(out, want, 1e-5 if dtype == torch.float32 else 1e-2)
