"""Each kernel of the Kotisun parts alone against the plain functions, on inputs made so that a fault shows: a residual in
streams with a mix that is not symmetric; attention whose one key scores far above all others, placed at the first
position, on both sides of block borders, far back, and just inside and just outside the window; a recurrence fed in
two steps of odd and even lengths from NaN-poisoned neighbours' states."""
import pytest
import torch

import plain_kotisun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(t, dtype=torch.float32):
    return t.to(device=DEV, dtype=dtype).contiguous()


def close(got, want, tol, what=""):
    got, want = got.double().cpu(), want.double()
    assert torch.isfinite(got).all(), what
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err < tol, (what, err)


@pytest.mark.parametrize("S,d", [(1, 40), (3, 64), (4, 100), (7, 33), (16, 8)])
def test_streams_read_write_embed(S, d):
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(S)
    T, V = 9, 50
    table = torch.randn(V, d, generator=g)
    toks = torch.randint(0, V, (T,), generator=g)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = torch.full((T, S * d), float("nan"), device=DEV)
    ops.embed_streams(dev(table, torch.bfloat16), dev(toks, torch.int32), x, S, 1.75, err)
    want0 = (table.bfloat16().double()[toks] * 1.75)
    close(x.view(T, S, d), want0[:, None, :].expand(T, S, d), 1e-6, "embed")
    xs = torch.randn(T, S, d, generator=g).double()
    a, b, m, w = (torch.randn(n, generator=g).double() for n in (S, S, S * S, d))
    m = m.view(S, S)
    y = torch.randn(T, d, generator=g).double()
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 6e-3)):
        out = torch.empty(T, d, dtype=dtype, device=DEV)
        ops.streams_read_norm(dev(xs.view(T, S * d)), S, dev(a), dev(w), 1e-5, out)
        close(out, plain.rms_norm(torch.einsum("s,tsd->td", a, xs), w, 1e-5), tol, "read")
    rows = torch.tensor([5, 0, 5, 8], dtype=torch.int32)
    out = torch.empty(4, d, device=DEV)
    ops.streams_read_norm(dev(xs.view(T, S * d)), S, None, dev(w), 1e-5, out, dev(rows, torch.int32))
    close(out, plain.rms_norm(xs.sum(1)[rows.long()], w, 1e-5), 1e-5, "sum of the streams, gathered rows")
    xd = dev(xs.view(T, S * d))
    ops.streams_write(xd, S, dev(m), dev(b), dev(y), T - 1)
    want = torch.einsum("sj,tsd->tjd", m, xs) + b[None, :, None] * y[:, None, :]
    close(xd.view(T, S, d)[:T - 1], want[:T - 1], 1e-5, "write")
    close(xd.view(T, S, d)[T - 1], xs[T - 1], 1e-7, "rows beyond the step stay")
    a2, w2 = torch.randn(S, generator=g).double(), torch.randn(d, generator=g).double()
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 6e-3)):
        xd, h = dev(xs.view(T, S * d)), torch.full((T, d), float("nan"), dtype=dtype, device=DEV)
        ops.streams_write_read(xd, S, dev(m), dev(b), dev(y), dev(a2), dev(w2), 1e-5, h, T - 1)
        close(xd.view(T, S, d)[:T - 1], want[:T - 1], 1e-5, "write of write_read")
        close(h[:T - 1], plain.rms_norm(torch.einsum("j,tjd->td", a2, want), w2, 1e-5)[:T - 1], tol, "read of write_read")
        close(xd.view(T, S, d)[T - 1], xs[T - 1], 1e-7, "rows beyond the step stay")
    lg = torch.randn(5, 37, generator=g) * 40
    ld = dev(lg)
    ops.softcap(ld, 4, 30.0)
    close(ld[:4], 30.0 * torch.tanh(lg[:4].double() / 30.0), 1e-6, "softcap")
    assert torch.equal(ld[4].cpu(), lg[4])


class PagedKV:
    """A paged cache with a permuted block table and NaN in every place that nothing wrote."""

    def __init__(self, n_slots, max_len, G, dk, dv, dtype):
        self.bt = 64
        self.max_blocks = (max_len + 63) // 64
        nb = n_slots * self.max_blocks + 3
        self.k = torch.full((nb, G, 64, dk), float("nan"), dtype=dtype, device=DEV)
        self.v = torch.full((nb, G, 64, dv), float("nan"), dtype=dtype, device=DEV)
        perm = torch.randperm(nb, generator=torch.Generator().manual_seed(1))[:n_slots * self.max_blocks]
        self.table = dev(perm.view(n_slots, self.max_blocks), torch.int32)


def run_attention(q, k, v, positions, slot_of, lens, G, scale, window, rot, dtype, out_scale=1.0, tail=None, splits=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] unrotated, for tokens at (slot_of[t], positions[t]): all appended to the
    cache, then attended.  tail None: every token is a query of one prompt step, by the kernel that takes a warp per token
    and head.  tail = n: the last n tokens of every sequence are the step's new tokens (a later portion of a prompt; n = 1:
    a decode step, its contexts cut into `splits` parts), by the kernel that the step function chooses."""
    import types
    from vlrf_b200.csrc import ops
    from vlrf_b200.parts.context import Workspace
    T, H, dk = q.shape
    dv = v.shape[2]
    cache = PagedKV(max(slot_of) + 1, max(lens), G, dk, dv, dtype)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1)
    wide = torch.full((T, proj.shape[1] + 5), float("nan"))
    wide[:, 3:3 + proj.shape[1]] = proj                       # the rows lie inside wider rows
    wide = dev(wide)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    qo = torch.full((T, H * dk), float("nan"), dtype=dtype, device=DEV)
    freq = None
    if rot:
        base, dims, factor = rot
        freq = dev(torch.tensor([base ** (-2.0 * i / dims) / factor for i in range(dims // 2)], dtype=torch.float64))
    tok_slot, tok_pos = dev(torch.tensor(slot_of), torch.int32), dev(torch.tensor(positions), torch.int32)
    ops.qkv_rope_append(wide[:, 3:3 + proj.shape[1]], 0, H * dk, H * dk + G * dk, freq, rot[1] if rot else 0, qo, cache.k, cache.v,
                        cache.table, tok_slot, tok_pos, T, H, G, dk, dv, True, err)
    pad = 8                                                    # (the tensor-core kernel wants rows on 4-byte boundaries)
    if tail is None:
        out = torch.full((T, H * dv + 2 * pad), float("nan"), dtype=dtype, device=DEV)
        ops.attention_window(qo, cache.k, cache.v, cache.table, tok_slot, tok_pos, out[:, pad:pad + H * dv], T, H, G, dk, dv, scale,
                             window, out_scale, err)
        keep = list(range(T))
    else:
        keep, seq_start, seq_pos0, start = [], [0], [], 0
        for n in lens:
            m = min(tail, n)
            keep += list(range(start + n - m, start + n))
            seq_start.append(seq_start[-1] + m); seq_pos0.append(n - m)
            start += n
        idx = torch.tensor(keep)
        ctx = types.SimpleNamespace(
            n_tokens=len(keep), n_seqs=len(lens), max_new=min(tail, max(lens)), max_context=max(lens), ws=Workspace(DEV), dev_err=err,
            tok_slot=dev(torch.tensor(slot_of)[idx], torch.int32), tok_pos=dev(torch.tensor(positions)[idx], torch.int32),
            seq_slot=dev(torch.tensor(list(range(len(lens)))), torch.int32), seq_start=dev(torch.tensor(seq_start), torch.int32),
            seq_pos0=dev(torch.tensor(seq_pos0), torch.int32))
        out = torch.full((len(keep), H * dv + 2 * pad), float("nan"), dtype=dtype, device=DEV)
        import os
        if splits:
            os.environ["VLRF_B200_DECODE_SPLITS"] = str(splits)
        try:
            ops.attention_window_step(qo[idx.to(DEV)].contiguous(), cache.k, cache.v, cache.table, out[:, pad:pad + H * dv], ctx, H, G, dk, dv,
                                      scale, window, out_scale)
        finally:
            os.environ.pop("VLRF_B200_DECODE_SPLITS", None)
    assert int(err.item()) == 0
    assert torch.isnan(out[:, :pad].float()).all() and torch.isnan(out[:, pad + H * dv:].float()).all()
    return out[:, pad:pad + H * dv].view(len(keep), H, dv), keep


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,G,dk,dv,window,rot", [
    (4, 2, 16, 24, 40, (10000.0, 8, 2.0)), (2, 2, 32, 32, 64, (500.0, 32, 1.0)), (6, 1, 8, 16, 0, None), (3, 3, 24, 8, 65, (3e4, 12, 8.0)),
    (3, 1, 12, 20, 1, (3000.0, 6, 1.3)), (5, 5, 80, 48, 130, (250.0, 16, 4.0)), (16, 1, 64, 128, 100, (1e4, 64, 1.0)),
    (8, 2, 128, 104, 0, (1e4, 32, 1.0)), (34, 2, 40, 40, 70, None)])
def test_attention_with_a_key_that_stands_out(H, G, dk, dv, window, rot, dtype, tol):
    """Sequences of 1, 2, 64, 65, 129 and 200 tokens in one step.  For the LAST query of every sequence the oldest key its
    window lets it see is made to score far above the rest, and the key just before that one, which it must not see,
    higher still; without a window the first key of the sequence stands out.  As one prompt step, as a later portion of
    70 and of 3 tokens, and as a decode step whose contexts are whole, cut in 2 and cut in 5."""
    g = torch.Generator().manual_seed(dk + dv)
    lens = [1, 2, 64, 65, 129, 200]
    slot_of, positions = [], []
    for s, n in enumerate(lens):
        slot_of += [s] * n
        positions += list(range(n))
    T = len(slot_of)
    rd = lambda *shape: torch.randn(*shape, generator=g).bfloat16().double()   # noqa: E731
    q, k, v = rd(T, H, dk), rd(T, G, dk), rd(T, G, dv)
    start = 0
    for s, n in enumerate(lens):
        last = start + n - 1
        inside = max(0, n - window) if window else 0               # the oldest key the last query sees
        for hk in range(G):
            # (unrotated entries only, so the rotation cannot undo it) matched to the first query head that reads the key
            h = hk * (H // G)
            lo = rot[1] if rot else 0
            if lo < dk:
                unit = q[last, h, lo:] / max(1e-3, float(q[last, h, lo:].norm()))
                k[start + inside, hk, lo:] = (6.0 * unit).bfloat16().double()
                if inside > 0:
                    k[start + inside - 1, hk, lo:] = (9.0 * unit).bfloat16().double()     # just outside: louder still
        start += n
    pos = torch.tensor(positions)
    rq = plain.rotate_scaled(q, pos, *rot) if rot else q
    rk = plain.rotate_scaled(k, pos, *rot) if rot else k
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    start = 0
    for n in lens:
        want[start:start + n] = plain.window_attention(rq[start:start + n], rk[start:start + n], v[start:start + n], 0.3, window)
        start += n
    for tail, splits in ((None, None), (70, None), (3, None), (1, 1), (1, 2), (1, 5)):
        if tail is None and (H // G > 16 or max(dk, dv) > 256):
            continue
        got, keep = run_attention(q.float(), k.float(), v.float(), positions, slot_of, lens, G, 0.3, window, rot, dtype, 0.6, tail, splits)
        close(got, 0.6 * want[torch.tensor(keep)], tol, f"attention, tail {tail}, {splits} parts")


@pytest.mark.parametrize("Hs,P,N,G,taps,ng", [(4, 8, 16, 2, 4, 2), (2, 24, 8, 1, 2, 1), (3, 16, 24, 3, 3, 3), (5, 6, 10, 5, 5, 3),
                                              (1, 32, 16, 1, 1, 1), (2, 64, 128, 1, 4, 8), (8, 80, 48, 2, 4, 4)])
def test_recurrence_in_steps_of_every_parity(Hs, P, N, G, taps, ng):
    """Three sequences in slots 4, 0 and 2 of six (the others full of NaN, and a padding row in every step): a first step of
    5, 8 and 1 tokens, then single tokens, then a step of 2, 3 and 6 — against the plain functions over the whole."""
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(Hs * 100 + P)
    inner, channels = Hs * P, Hs * P + 2 * G * N
    width = 2 * inner + 2 * G * N + Hs
    lens = [5 + 3 + 2, 8 + 3 + 3, 1 + 3 + 6]
    slots = [4, 0, 2]
    cuts = [[5, 1, 1, 1, 2], [8, 1, 1, 1, 3], [1, 1, 1, 1, 6]]
    proj = [torch.randn(n, width, generator=g).double() for n in lens]
    conv_w, conv_b = torch.randn(channels, taps, generator=g).double() * 0.5, torch.randn(channels, generator=g).double() * 0.3
    dt_bias, a_log, D = torch.randn(Hs, generator=g).double(), torch.randn(Hs, generator=g).double() - 1.0, torch.randn(Hs, generator=g).double()
    norm_w = torch.randn(inner, generator=g).double()
    want = []
    for pr in proj:
        z, xbc, dt = pr[:, :inner], pr[:, inner:inner + channels], pr[:, inner + channels:]
        xbc = plain.silu(plain.causal_conv(xbc, conv_w, conv_b))
        n = pr.shape[0]
        y = plain.selective_scan(xbc[:, :inner].reshape(n, Hs, P), xbc[:, inner:inner + G * N].reshape(n, G, N),
                                 xbc[:, inner + G * N:].reshape(n, G, N), plain.softplus(dt + dt_bias), a_log, D).reshape(n, inner)
        want.append(0.9 * plain.group_rms_norm(y * plain.silu(z), norm_w, ng, 1e-5))
    state_row = Hs * N * P + (taps - 1) * channels
    state = torch.full((6, 2, state_row), float("nan"), device=DEV)
    for s in slots:
        state[s].zero_()
    got = [[] for _ in lens]
    at = [0, 0, 0]
    for step in range(5):
        rows, seq_slot, seq_start, seq_pos0 = [], [], [0], []
        for i in (1, 0, 2):                                            # the step lists the sequences in another order
            n = cuts[i][step]
            rows.append(proj[i][at[i]:at[i] + n])
            seq_slot.append(slots[i]); seq_pos0.append(at[i]); seq_start.append(seq_start[-1] + n)
            if i == 0:                                                  # a padding row between two sequences
                rows.append(torch.full((1, width), float("nan"), dtype=torch.float64))
                seq_slot.append(-1); seq_pos0.append(0); seq_start.append(seq_start[-1] + 1)
        pr = dev(torch.cat(rows))
        T = pr.shape[0]
        ss, st, sp = (dev(torch.tensor(v), torch.int32) for v in (seq_slot, seq_start, seq_pos0))
        xbc = torch.full((T, channels), float("nan"), device=DEV)
        ops.ssd_conv(pr, inner, dev(conv_w), dev(conv_b), state, Hs * N * P, ss, st, sp, xbc, len(seq_slot), max(c[step] for c in cuts))
        y = torch.full((T, inner), float("nan"), device=DEV)
        ops.ssd_scan(xbc, pr, inner + channels, dev(dt_bias), dev(a_log), dev(D), state, ss, st, sp, y, len(seq_slot), Hs, G, N, P)
        out = torch.full((T, inner + 3), float("nan"), device=DEV)
        ops.ssd_gate_norm(y, pr, 0, dev(norm_w), ng, 1e-5, 0.9, out[:, 2:2 + inner], T)
        r = 0
        for i in (1, 0, 2):
            n = cuts[i][step]
            got[i].append(out[r:r + n, 2:2 + inner].cpu())
            at[i] += n
            r += n + (1 if i == 0 else 0)
    for i in range(3):
        close(torch.cat(got[i]), want[i], 3e-5, f"sequence {i}")
    assert torch.isnan(state[[1, 3, 5]]).all()
