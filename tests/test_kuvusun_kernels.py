"""Each mechanism of the Kuvusun design alone: the kernel against the plain function on inputs of its own — norms in
groups, the cache row of a token (latent norm and rotation), the queries' rows, products per head and per group, the
router, and attention over rows of latents with a key made to stand out far away, at block borders and at the ends."""
import math

import pytest
import torch

import plain_kuvusun as plain

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]


def tol(dt):
    return 2e-5 if dt == torch.float32 else 1.2e-2


def close(got, want, t, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert math.isfinite(err) and err <= t, f"{what}: error {err:.3e} above {t:.1e}"


def dev(t, dt=None):
    return t.to("cuda", dt if dt is not None else t.dtype).contiguous()


@pytest.mark.parametrize("d,groups", [(96, 3), (100, 5), (128, 1), (64, 64), (2048, 8)])
def test_rms_norm_in_groups(d, groups):
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(d + groups)
    y = torch.randn(9, d, generator=g, dtype=torch.float64) * torch.linspace(0.01, 30, d, dtype=torch.float64)
    w = 1 + 0.3 * torch.randn(d, generator=g, dtype=torch.float64)
    want = plain.group_rms_norm(y, w, groups, 1e-5)
    yd, wd = dev(y, torch.float32), dev(w, torch.float32)
    out = torch.zeros(9, d, device="cuda")
    ops.group_rmsnorm(yd, wd, 1e-5, groups, out)
    close(out, want, 2e-6, "replace")
    base = torch.randn(9, d, generator=g, dtype=torch.float64)
    acc = dev(base, torch.float32)
    also = torch.zeros(9, d, dtype=torch.bfloat16, device="cuda")
    ops.group_rmsnorm(yd, wd, 1e-5, groups, acc, accumulate=True, also=also)
    close(acc, base + want, 2e-6, "accumulate")
    assert torch.equal(also, acc.to(torch.bfloat16)), "the second output is the rounding of the first"
    rows = torch.tensor([7, 0, 7, 3], dtype=torch.int32, device="cuda")
    half = torch.zeros(4, d, dtype=torch.bfloat16, device="cuda")
    ops.group_rmsnorm(yd, wd, 1e-5, groups, half, rows)
    close(half, want[[7, 0, 7, 3]], 8e-3, "gathered rows in bfloat16")
    ops.group_rmsnorm(yd, wd, 1e-5, groups, yd)
    close(yd, want, 2e-6, "in place")
    # eps stands inside the root: a part of zeros stays finite and zero
    z = torch.zeros(1, d, device="cuda")
    ops.group_rmsnorm(z, wd, 1e-5, groups, z)
    assert torch.equal(z, torch.zeros_like(z))


def test_gates_with_float32_inputs_and_ranges_of_wider_rows():
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    wide = torch.randn(7, 50, generator=g, dtype=torch.float64) * 3
    b = torch.randn(7, 20, generator=g, dtype=torch.float64)
    w32 = dev(wide, torch.float32)
    for gate, f in (("silu", lambda x: x * torch.sigmoid(x)), ("sigmoid", torch.sigmoid)):
        out = torch.zeros(7, 20, dtype=torch.bfloat16, device="cuda")
        ops.gate_mul(w32[:, 3:23], w32[:, 23:43], out, gate, 7, 20)                    # float32, float32 → bfloat16
        close(out, f(wide[:, 3:23]) * wide[:, 23:43], 5e-3, gate)
        bb = dev(b, torch.bfloat16)
        ops.gate_mul(w32[:, 3:23], bb, bb, gate, 7, 20)                                # float32, bfloat16 → in place
        close(bb, f(wide[:, 3:23]) * dev(b, torch.bfloat16).double().cpu(), 5e-3, gate + " in place")
        o32 = torch.zeros(7, 20, device="cuda")
        ops.gate_mul(w32[:, 3:23], w32[:, 23:43], o32, gate, 7, 20)
        close(o32, f(wide[:, 3:23]) * wide[:, 23:43], 1e-6, gate + " float32")
        h16 = dev(wide, torch.bfloat16)
        o16 = torch.zeros(7, 16, dtype=torch.bfloat16, device="cuda")
        ops.gate_mul(h16[:, 8:24], h16[:, 24:40], o16, gate, 7, 16)                    # all bfloat16, eight a thread
        close(o16, f(h16[:, 8:24].double().cpu()) * h16[:, 24:40].double().cpu(), 5e-3, gate + " bfloat16")


def paged(n_blocks, order, row_w, dt):
    """A latent cache of NaN and a block table that maps slot 1's blocks to `order`."""
    cache = torch.full((n_blocks, 64, row_w), float("nan"), dtype=dt, device="cuda")
    table = torch.full((3, 32), -1, dtype=torch.int32)
    table[1, :len(order)] = torch.tensor(order, dtype=torch.int32)
    return cache, table.cuda()


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("C,R,dims,base", [(40, 8, 8, 10000.0), (36, 6, 6, 3000.0), (64, 0, 0, 1.0), (24, 16, 8, 500.0)])
def test_a_tokens_cache_row_is_the_normed_latent_and_the_rotated_key_part(C, R, dims, base, dt):
    from vlrf_b200.csrc import ops
    from vlrf_b200.parts import RotaryPositions
    g = torch.Generator().manual_seed(C + R)
    positions = [0, 1, 2, 63, 64, 65, 127, 128, 700, 1023]
    proj = torch.randn(len(positions), C + R + 3, generator=g, dtype=torch.float64) * 3
    w = 1 + 0.2 * torch.randn(C, generator=g, dtype=torch.float64)
    order = [5, 2, 9, 0, 7, 1, 3, 4, 6, 8, 10, 11, 12, 13, 14, 15]
    cache, table = paged(16, order, C + R, dt)
    rot = RotaryPositions(base, dims, "cuda") if R > 0 else None
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    slot = torch.ones(len(positions), dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.latent_append(dev(proj, torch.float32), C, R, dev(w, torch.float32), 1e-5, rot.inv_freq if rot else None, dims, cache,
                      table, slot, pos, len(positions), err)
    assert int(err.item()) == 0
    c = plain.rms_norm(proj[:, :C], w, 1e-5)
    for i, p in enumerate(positions):
        row = cache[order[p // 64], p % 64]
        close(row[:C], c[i], 1e-6 if dt == torch.float32 else 5e-3, f"latent at {p}")
        if R > 0:
            r = plain.rotate(proj[i:i + 1, C:C + R], torch.tensor([p]), base, dims)[0]
            close(row[C:], r, 3e-5 if dt == torch.float32 else 5e-3, f"rotated part at {p}")     # angle of up to 1023 rad in float32
    written = torch.zeros(16, 64, dtype=torch.bool)
    for p in positions:
        written[order[p // 64], p % 64] = True
    assert torch.isnan(cache.float().cpu()[~written]).all(), "a row that belongs to no token was written"
    # a token whose block is not mapped is skipped and reported
    ops.latent_append(dev(proj, torch.float32), C, R, dev(w, torch.float32), 1e-5, rot.inv_freq if rot else None, dims, cache,
                      table, slot, pos + 1024, len(positions), err)
    assert int(err.item()) == 4
    err.zero_()


@pytest.mark.parametrize("dt", DT)
def test_query_rows_split_and_rotate(dt):
    from vlrf_b200.csrc import ops
    from vlrf_b200.parts import RotaryPositions
    H, dim, R, C, dims, base = 3, 12, 10, 20, 6, 777.0
    g = torch.Generator().manual_seed(1)
    q = torch.randn(5, H * (dim + R), generator=g, dtype=torch.float64)
    positions = torch.tensor([0, 3, 64, 500, 129])
    rot = RotaryPositions(base, dims, "cuda")
    qn = torch.zeros(5, H * dim, dtype=dt, device="cuda")
    qp = torch.zeros(5, H * (C + R), dtype=dt, device="cuda")
    ops.latent_q_rows(dev(q, torch.float32), H, dim, R, rot.inv_freq, dims, dev(positions, torch.int32), qn, qp, C, 5)
    q3 = q.view(5, H, dim + R)
    close(qn.view(5, H, dim), q3[..., :dim], 1e-6 if dt == torch.float32 else 5e-3, "unrotated parts")
    close(qp.view(5, H, C + R)[..., C:], plain.rotate(q3[..., dim:], positions, base, dims), 2e-5 if dt == torch.float32 else 5e-3, "rotated parts")
    assert float(qp.view(5, H, C + R)[..., :C].abs().max()) == 0.0


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,H,N,K", [(1, 3, 40, 16), (70, 5, 24, 36), (130, 2, 129, 64), (9, 1, 7, 5)])
def test_products_per_head(M, H, N, K, dt):
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(M + N)
    x = dev(torch.randn(M, H, K + 3, generator=g), dt)        # heads inside wider rows
    w = dev(torch.randn(H, N, K, generator=g) / math.sqrt(K), dt)
    out = torch.full((M, H, N + 2), 7.0, dtype=dt, device="cuda")
    ops.linear_heads(x[:, :, 1:K + 1], w, out[:, :, 2:], M)
    want = torch.einsum("mhk,hnk->mhn", x[:, :, 1:K + 1].double(), w.double())
    close(out[:, :, 2:], want, tol(dt), "heads")
    assert float((out[:, :, :2].float() - 7.0).abs().max()) == 0.0, "columns outside the heads' outputs were written"
    if dt == torch.bfloat16:
        out32 = torch.zeros(M, H, N, device="cuda")
        ops.linear_heads(x[:, :, 1:K + 1], w, out32, M)
        close(out32, want, 1e-5, "float32 result of bfloat16 operands")


@pytest.mark.parametrize("dt", DT)
def test_products_per_group(dt):
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    counts = [0, 5, 130, 0, 64, 1, 0]
    G, N, K = len(counts), 50, 44
    P = sum(counts)
    x = dev(torch.randn(P + 9, K, generator=g), dt)            # rows beyond the last group belong to nobody
    w = dev(torch.randn(G, N, K, generator=g) / math.sqrt(K), dt)
    offsets = torch.tensor([sum(counts[:i]) for i in range(G + 1)], dtype=torch.int32, device="cuda")
    out = torch.full((P + 9, N), 5.0, dtype=torch.float32, device="cuda")
    ops.linear_grouped(x, w, out, offsets, P + 9)
    at = 0
    for e, n in enumerate(counts):
        if n:
            close(out[at:at + n], x[at:at + n].double() @ w[e].double().T, 1e-5, f"group {e}")
        at += n
    assert float((out[P:] - 5.0).abs().max()) == 0.0


@pytest.mark.parametrize("M,H,N,K", [(300, 5, 72, 64), (70, 3, 512, 32), (1, 16, 40, 128), (129, 2, 130, 200), (64, 20, 24, 24),
                                     (4100, 30, 16, 16)])
def test_products_per_head_on_the_tensor_cores(M, H, N, K):
    """Shapes that the tcgen05 kernel takes (rows and heads on 16-byte boundaries): heads narrower than the 64 columns
    a copy brings (the neighbour's columns arrive and must count for nothing), row tiles with tails, column tails."""
    from vlrf_b200.csrc import library, ops
    g = torch.Generator().manual_seed(M + K)
    x = dev(torch.randn(M, H, K, generator=g), torch.bfloat16)
    w = dev(torch.randn(H, N, K, generator=g) / math.sqrt(K), torch.bfloat16)
    want = torch.einsum("mhk,hnk->mhn", x.double(), w.double())
    wide = (N + 15) // 8 * 8                                   # heads' outputs inside wider rows, on 16-byte boundaries
    assert library().vlrf_gemm_tcgen05_groups_takes(M, H, N, K, H * K, K, H * wide, wide, 0)
    for odt, t in ((torch.bfloat16, 1.2e-2), (torch.float32, 1e-5)):
        out = torch.full((M, H, wide), 7.0, dtype=odt, device="cuda")
        ops.linear_heads(x, w, out[:, :, :N], M)
        close(out[:, :, :N], want, t, f"heads, {odt}")
        assert float((out[:, :, N:].float() - 7.0).abs().max()) == 0.0, "columns outside the heads' outputs were written"
    assert ops.device_errors() == 0


@pytest.mark.parametrize("counts,N,K", [([0, 5, 130, 0, 64, 1, 0, 300], 200, 96), ([128, 128], 48, 64), ([0, 0, 3], 136, 256),
                                        ([7] * 40, 64, 32)])
def test_products_per_group_on_the_tensor_cores(counts, N, K):
    from vlrf_b200.csrc import library, ops
    g = torch.Generator().manual_seed(N + K)
    G, P = len(counts), sum(counts)
    x = dev(torch.randn(P + 9, K, generator=g), torch.bfloat16)
    x[P:] = float("nan")                                       # rows of no group are read but must count for nothing
    w = dev(torch.randn(G, N, K, generator=g) / math.sqrt(K), torch.bfloat16)
    offsets = torch.tensor([sum(counts[:i]) for i in range(G + 1)], dtype=torch.int32, device="cuda")
    assert library().vlrf_gemm_tcgen05_groups_takes(P + 9, G, N, K, K, 0, N, 0, 1)
    for odt, t in ((torch.float32, 1e-5), (torch.bfloat16, 1.2e-2)):
        out = torch.full((P + 9, N), 5.0, dtype=odt, device="cuda")
        ops.linear_grouped(x, w, out, offsets, P + 9)
        at = 0
        for e, n in enumerate(counts):
            if n:
                close(out[at:at + n], x[at:at + n].double() @ w[e].double().T, t, f"group {e}, {odt}")
            at += n
        assert float((out[P:].float() - 5.0).abs().max()) == 0.0
    assert ops.device_errors() == 0


def test_router_chooses_weighs_and_sorts():
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(8)
    T, E, top, width = 37, 11, 3, 20
    z = torch.randn(T, E + 1, generator=g, dtype=torch.float64) * 2
    z[4, :E] = 1.5                       # all equal: the lowest indices win
    z[5, 2] = z[5, 7] = z[5, 9] = 9.0    # a tie among the chosen
    z[6, 3] = float("nan")               # never chosen before a number
    slot = torch.zeros(T, dtype=torch.int32)
    slot[10] = -1                        # a padding row chooses nothing
    zd = dev(z, torch.float32)
    ids = torch.zeros(T, top, dtype=torch.int32, device="cuda"); rank = torch.zeros_like(ids); row_of = torch.zeros_like(ids)
    wts = torch.zeros(T, top, device="cuda"); gate = torch.zeros(T, 1, device="cuda")
    counts = torch.zeros(E, dtype=torch.int32, device="cuda"); offsets = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    ops.moe_route(zd, E, top, True, slot.cuda(), ids, wts, rank, gate, counts, T)
    z_plain = z[:, :E].clone()
    z_plain[6, 3] = -1e30
    want_ids, want_w = plain.route(z_plain, top)
    live = [t for t in range(T) if t != 10]
    assert ids.cpu()[live].tolist() == want_ids[live].tolist()
    assert ids.cpu()[4].tolist() == [0, 1, 2] and ids.cpu()[5].tolist() == [2, 7, 9] and ids.cpu()[10].tolist() == [-1] * top
    close(wts[live], want_w[live], 1e-6, "weights")
    close(gate[:, 0][live], torch.sigmoid(z[live, E]), 1e-6, "shared gate")
    n_of = torch.bincount(want_ids[live].flatten(), minlength=E)
    assert counts.cpu().tolist() == n_of.tolist()
    ops.moe_plan(counts, offsets, E)
    assert offsets.cpu().tolist() == [int(n_of[:e].sum()) for e in range(E + 1)] and int(counts.abs().sum()) == 0
    h = dev(torch.randn(T, width, generator=g), torch.float32)
    rows = torch.full((T * top, width), float("nan"), device="cuda")
    ops.moe_gather(h, ids, rank, offsets, rows, row_of, T, top)
    r = row_of.cpu()
    assert sorted(r[live].flatten().tolist()) == list(range(len(live) * top)), "the pairs' rows are a permutation"
    assert r[10].tolist() == [-1] * top
    off = offsets.cpu()
    for t in live:
        for j in range(top):
            e = int(want_ids[t, j])
            assert off[e] <= r[t, j] < off[e + 1] and torch.equal(rows[int(r[t, j])], h[t])
    # the weighted sum of the experts' rows, the shared expert through its gate, and the residual
    eo = dev(torch.randn(T * top, width, generator=g), torch.float32)
    so = dev(torch.randn(T, width, generator=g), torch.float32)
    y = torch.zeros(T, width, device="cuda")
    ops.moe_combine(eo, row_of, wts, top, so, gate, y, T)
    want = torch.stack([sum(want_w[t, j] * eo[int(r[t, j])].double().cpu() for j in range(top)) + torch.sigmoid(z[t, E]) * so[t].double().cpu()
                        for t in live])
    close(y[live], want, 1e-6, "combine")
    y2 = torch.ones(T, width, device="cuda")
    ops.moe_combine(eo, row_of, wts, top, None, None, y2, T, residual=y2)
    close(y2[live], want - torch.stack([torch.sigmoid(z[t, E]) * so[t].double().cpu() for t in live]) + 1.0, 1e-6, "combine onto a residual")


def plain_rows_attention(q, rows, C, scale, pos, window=0):
    """q [H, C + R], rows [n, C + R] → per head Σ_j p_j rows[j, :C] over the visible j ≤ pos."""
    first = max(0, pos - window + 1) if window > 0 else 0
    s = (q.double() @ rows[first:pos + 1].double().T) * scale
    return torch.softmax(s, -1) @ rows[first:pos + 1, :C].double()


def step_tables(positions, runs, splits=None):
    """What a step hands to the attention kernels besides each token's slot and position: its sequence tables.
    `runs`: how many consecutive tokens each sequence of the step brings (all of slot 1)."""
    import types
    from vlrf_b200.parts.context import Workspace
    starts = [0]
    for n in runs:
        starts.append(starts[-1] + n)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return types.SimpleNamespace(max_new=max(runs), n_seqs=len(runs), seq_slot=t([1] * len(runs)), seq_start=t(starts),
                                 seq_pos0=t([positions[a] for a in starts[:-1]]), max_context=max(positions) + 1,
                                 ws=Workspace("cuda"))


@pytest.mark.parametrize("C,R,H", [(64, 0, 2), (512, 64, 2), (32, 16, 9), (96, 16, 20), (256, 32, 16)])
@pytest.mark.parametrize("splits", [None, 1, 3, 16])
def test_tensor_core_attention_over_latent_rows(C, R, H, splits, monkeypatch):
    """The tensor-core kernel against the plain attention: a prompt's portion (consecutive tokens of one sequence that
    begin in the middle of a block and cross borders, with more and fewer tokens than a CTA takes), and single tokens
    whose contexts are cut into parts (more parts than some contexts have tiles).  One key per head stands out."""
    from vlrf_b200.csrc import ops
    if splits is not None:
        monkeypatch.setenv("VLRF_B200_DECODE_SPLITS", str(splits))
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(C + H)
    n, D, scale = 700, C + R, 0.37
    rows = torch.randn(n, D, generator=g).to(dt)
    order = [5, 2, 9, 0, 7, 1, 3, 4, 6, 8, 10]
    cache, table = paged(12, order, D, dt)
    for b in range(11):
        cache[order[b], :min(64, n - 64 * b)] = rows[64 * b:64 * b + 64].cuda()
    if splits is None:
        positions, runs = list(range(59, 59 + 75)) + list(range(0, 3)) + [690], [75, 3, 1]       # portions of a prompt
    else:
        positions = [699, 0, 31, 32, 63, 64, 65, 300, 1, 127]                                  # single tokens
        runs = [1] * len(positions)
    stars = [(7 * i + 3) % (p + 1) if i % 3 else p - min(p, i % 5) for i, p in enumerate(positions)]
    qp = torch.zeros(len(positions), H * D, dtype=dt)
    for i, (pos, star) in enumerate(zip(positions, stars)):
        for h in range(H):
            k = rows[(star + 11 * h) % (pos + 1)].float()
            qp[i, h * D:(h + 1) * D] = (k * (30.0 / (scale * float(k @ k)))).to(dt) + (0.05 * torch.randn(D, generator=g)).to(dt)
    ctx = step_tables(positions, runs)
    assert ops.attention_latent_kind(dt, C, R)["decode"] == "mma.sync"
    pos_t = torch.tensor(positions, dtype=torch.int32, device="cuda")
    slot = torch.ones(len(positions), dtype=torch.int32, device="cuda")
    out = torch.full((len(positions), H * C), float("nan"), dtype=dt, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.attention_latent(qp.cuda(), cache, C, R, table, slot, pos_t, out, len(positions), H, scale, 0, err, ctx=ctx)
    assert int(err.item()) == 0
    general = torch.zeros_like(out)
    ops.attention_latent(qp.cuda(), cache, C, R, table, slot, pos_t, general, len(positions), H, scale, 0, err)
    for i, pos in enumerate(positions):
        want = plain_rows_attention(qp[i].view(H, D), rows, C, scale, pos)
        close(out[i].view(H, C), want, 1.2e-2, f"token {i} at {pos}")
        close(out[i].view(H, C), general[i].view(H, C), 1.2e-2, f"token {i} at {pos} against the general kernel")
    if splits is None:        # a window, whose edge falls inside a tile for some tokens and on its border for others
        for window in (33, 64):
            ops.attention_latent(qp.cuda(), cache, C, R, table, slot, pos_t, out, len(positions), H, scale, window, err, ctx=ctx)
            for i, pos in enumerate(positions):
                close(out[i].view(H, C), plain_rows_attention(qp[i].view(H, D), rows, C, scale, pos, window), 1.2e-2, f"window {window}, token at {pos}")
    # padding sequences give zeros
    ctx.seq_slot[0] = -1
    ops.attention_latent(qp.cuda(), cache, C, R, table, slot, pos_t, out, len(positions), H, scale, 0, err, ctx=ctx)
    assert float(out[:runs[0]].float().abs().max()) == 0.0 and int(err.item()) == 0


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("C,R,H", [(40, 8, 3), (36, 6, 5), (64, 0, 2), (512, 64, 2), (24, 16, 9)])
def test_attention_over_latent_rows_finds_a_key_that_stands_out(C, R, H, dt):
    """Among hundreds of rows one is made to score far above the rest: at the start, at both sides of block borders,
    far back, and at the query's own position; the head's output must be that row.  The block table is a permutation
    and unmapped blocks hold NaN."""
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(C + H)
    n = 700
    D = C + R
    rows = torch.randn(n, D, generator=g).to(dt)
    order = [5, 2, 9, 0, 7, 1, 3, 4, 6, 8, 10]
    cache, table = paged(12, order, D, dt)
    for b in range(11):
        cache[order[b], :min(64, n - 64 * b)] = rows[64 * b:64 * b + 64].cuda()
    scale = 0.37
    queries = [(699, 0), (699, 63), (699, 64), (699, 3), (699, 699), (640, 639), (64, 64), (63, 0), (128, 127), (0, 0), (1, 0), (300, 191)]
    qp = torch.zeros(len(queries), H * D, dtype=dt)
    for i, (pos, star) in enumerate(queries):
        for h in range(H):
            k = rows[(star + h) % (pos + 1)].float()                 # every head its own key
            qp[i, h * D:(h + 1) * D] = (k * (30.0 / (scale * float(k @ k)))).to(dt) + (0.05 * torch.randn(D, generator=g)).to(dt)
    pos_t = torch.tensor([p for p, _ in queries], dtype=torch.int32, device="cuda")
    slot = torch.ones(len(queries), dtype=torch.int32, device="cuda")
    out = torch.full((len(queries), H * C), float("nan"), dtype=dt, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.attention_latent(qp.cuda(), cache, C, R, table, slot, pos_t, out, len(queries), H, scale, 0, err)
    assert int(err.item()) == 0
    for i, (pos, star) in enumerate(queries):
        want = plain_rows_attention(qp[i].view(H, D), rows, C, scale, pos)
        close(out[i].view(H, C), want, 1e-5 if dt == torch.float32 else 1e-2, f"query at {pos}, key at {star}")
        for h in range(H):                                            # and the output is that key's latent
            k = rows[(star + h) % (pos + 1), :C].double()
            assert float((want[h] - k).abs().max()) < 0.2 * float(k.abs().max())
    # windows: a key just inside is found, one just outside is not
    for window, star, inside in ((100, 600, True), (100, 599, False), (64, 636, True), (64, 635, False)):
        q1 = torch.zeros(1, H * D, dtype=dt)
        k = rows[star].float()
        q1[0] = ((k * (30.0 / (scale * float(k @ k)))).to(dt)).repeat(H)
        o1 = torch.zeros(1, H * C, dtype=dt, device="cuda")
        ops.attention_latent(q1.cuda(), cache, C, R, table, slot[:1], pos_t[:1], o1, 1, H, scale, window, err)
        want = plain_rows_attention(q1[0].view(H, D), rows, C, scale, 699, window)
        close(o1.view(H, C), want, 1e-5 if dt == torch.float32 else 1e-2, f"window {window}, key at {star}")
        hit = float((want[0] - rows[star, :C].double()).abs().max()) < 0.2 * float(rows[star, :C].abs().max())
        assert hit == inside
    # padding rows give zeros; an unmapped block is reported, not read
    slot2 = torch.tensor([-1, 1], dtype=torch.int32, device="cuda")
    o2 = torch.full((2, H * C), 3.0, dtype=dt, device="cuda")
    ops.attention_latent(qp[:2].cuda(), cache, C, R, table, slot2, torch.tensor([5, 705], dtype=torch.int32, device="cuda"), o2, 2, H,
                         scale, 0, err)
    assert float(o2[0].abs().max()) == 0.0 and int(err.item()) == 4
    err.zero_()


@pytest.mark.parametrize("dim,R,vdim,H", [(32, 32, 32, 3), (16, 16, 24, 2), (64, 32, 64, 2), (128, 64, 128, 2), (64, 0, 48, 2), (96, 32, 8, 1),
                                          (192, 64, 128, 1)])
def test_prompt_attention_over_plain_rows(dim, R, vdim, H):
    """Sequences of 1 to 200 tokens that begin at position 0, keys in two parts (per head, and one shared by the heads);
    per query and head one key is made to stand out: the first, the query's own, the last of the tile before, far back."""
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(dim + R + vdim)
    lens = [1, 70, 64, 200, 33, 65]
    T = sum(lens)
    starts = [sum(lens[:i]) for i in range(len(lens) + 1)]
    bf = torch.bfloat16
    kn = torch.randn(T, H, dim, generator=g).to(bf)
    kr = torch.randn(T, R, generator=g).to(bf) if R else None
    v = torch.randn(T, H, vdim, generator=g).to(bf)
    scale = 0.29
    qn = torch.zeros(T, H, dim, dtype=bf)
    qr = torch.zeros(T, H, R, dtype=bf) if R else None
    for si, n in enumerate(lens):
        for i in range(n):
            for h in range(H):
                star = [0, i, max(0, (i // 32) * 32 - 1), (i * 7 + h) % (i + 1)][(i + h) % 4]
                key = torch.cat([kn[starts[si] + star, h].float()] + ([kr[starts[si] + star].float()] if R else []))
                q = key * (25.0 / (scale * float(key @ key))) + 0.05 * torch.randn(dim + R, generator=g)
                qn[starts[si] + i, h] = q[:dim].to(bf)
                if R:
                    qr[starts[si] + i, h] = q[dim:].to(bf)
    assert ops.attention_rows_takes(bf, dim, R, vdim, H)
    out = torch.full((T, H * vdim), float("nan"), dtype=bf, device="cuda")
    ops.attention_rows(qn.view(T, -1).cuda(), qr.view(T, -1).cuda() if R else None, kn.view(T, -1).cuda(), kr.cuda() if R else None,
                       v.view(T, -1).cuda(), torch.tensor(starts, dtype=torch.int32, device="cuda"), out, len(lens), max(lens), H, dim, R, vdim, scale)
    got = out.view(T, H, vdim).double().cpu()
    assert torch.isfinite(got).all()
    for si, n in enumerate(lens):
        a, b = starts[si], starts[si] + n
        sc = torch.einsum("ihd,jhd->hij", qn[a:b].double(), kn[a:b].double())
        if R:
            sc = sc + torch.einsum("ihd,jd->hij", qr[a:b].double(), kr[a:b].double())
        want = plain.causal_softmax_attention(sc * scale, v[a:b].double())
        close(got[a:b], want, 1.2e-2, f"sequence of {n}")


def test_cache_rows_of_a_step_as_plain_matrices():
    from vlrf_b200.csrc import ops
    C, R = 40, 8
    order = [3, 0, 2, 1]
    for dt in DT:
        cache, table = paged(4, order, C + R, dt)
        rows = torch.randn(256, C + R).to(dt)
        for b in range(4):
            cache[order[b]] = rows[64 * b:64 * b + 64].cuda()
        pos = [0, 63, 64, 200, 255, 5]
        slot = torch.tensor([1, 1, 1, 1, 1, -1], dtype=torch.int32, device="cuda")
        oc = torch.full((6, C), 9.0, dtype=dt, device="cuda"); orr = torch.full((6, R), 9.0, dtype=dt, device="cuda")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.latent_gather(cache, C, R, table, slot, torch.tensor(pos, dtype=torch.int32, device="cuda"), oc, orr, 6, err)
        assert int(err.item()) == 0
        assert torch.equal(oc[:5].cpu(), rows[pos[:5], :C]) and torch.equal(orr[:5].cpu(), rows[pos[:5], C:])
        assert float(oc[5].float().abs().max()) == 0.0 and float(orr[5].float().abs().max()) == 0.0
