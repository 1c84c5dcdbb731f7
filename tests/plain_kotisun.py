"""A plain, slow implementation of the Kotisun design in float64, one function per mechanism, written from the
design's equations and sharing no code with the package (it reads model folders with the tests' own reader).

Kotisun: a decoder whose residual is carried in several streams (hyper-connections), whose mixer runs a windowed
softmax attention and a selective state-space recurrence side by side on the same input, with a gated feed-forward,
a range of layers that is run several times in a row with the same weights, and logits squashed by a tanh.

Notation: T tokens, width d.  Linear weights are [out, in] and applied as x · Wᵀ.
"""
from __future__ import annotations

import math

import torch

from plain_gpt2 import read_model_dir  # noqa: F401  (the tests' own reader of config.json + model.safetensors)


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def group_rms_norm(x, w, groups, eps):
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(shape) * w


def silu(x):
    return x / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def rotate_scaled(v, positions, base, dims, factor):
    """v [T, heads, n]: of the first `dims` entries of a head, entry i pairs with entry i + dims/2; the pair (a, b) at
    position p becomes (a cos t − b sin t, b cos t + a sin t), t = p · base^(−2i/dims) / factor."""
    half = dims // 2
    out = v.clone()
    for i in range(half):
        f = float(base) ** (-2.0 * i / dims) / float(factor)
        t = (positions.to(torch.float64) * f)[:, None]
        a, b = v[..., i], v[..., i + half]
        out[..., i] = a * torch.cos(t) - b * torch.sin(t)
        out[..., i + half] = b * torch.cos(t) + a * torch.sin(t)
    return out


def window_attention(q, k, v, scale, window):
    """q [T, H, n], k [T, G, n], v [T, G, m] → [T, H, m].  Query head h reads key/value head h // (H/G); query i sees
    keys j with 0 ≤ i − j < window (window None or 0: every j ≤ i); softmax over the visible keys."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(T):
        lo = 0 if not window else max(0, i - window + 1)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            p = torch.softmax(s, dim=0)
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def attention_branch(h, w, p, m, positions):
    """The softmax branch: projections with biases, rotation of queries and keys, windowed attention, W_o."""
    T = h.shape[0]
    H, G, n, nv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, n)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, n)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, nv)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_scaled(q, positions, rot["base"], rot["dims"], factor)
        k = rotate_scaled(k, positions, rot["base"], rot["dims"], factor)
    window = (m.get("mask") or {}).get("size")
    o = window_attention(q, k, v, m["scale"], window)
    return o.reshape(T, H * nv) @ w[p + "o"].T


def causal_conv(u, taps_w, bias):
    """u [T, channels]; taps_w [channels, taps], the last column multiplies the current token, zeros before the start."""
    T, C = u.shape
    K = taps_w.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u])
    out = torch.zeros_like(u)
    for j in range(K):
        out = out + padded[j:j + T] * taps_w[:, j]
    return out + bias


def selective_scan(x, B, C, dt, a_log, D):
    """x [T, Hs, P], B and C [T, Gs, N], dt [T, Hs] (already positive).  Per head (group h // (Hs/Gs)):
    S ← exp(−exp(a_log)·dt)·S + dt·B xᵀ (S is N × P, zero at the start); y = Sᵀ C + D x."""
    T, Hs, P = x.shape
    Gs, N = B.shape[1], B.shape[2]
    y = torch.zeros_like(x)
    for h in range(Hs):
        g = h // (Hs // Gs)
        S = torch.zeros(N, P, dtype=x.dtype)
        for t in range(T):
            decay = math.exp(-math.exp(float(a_log[h])) * float(dt[t, h]))
            S = decay * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * x[t, h]
    return y


def recurrent_branch(h, w, p, m, eps):
    """The state-space branch: one input projection cut into gate, values, B, C and step sizes; a short causal
    convolution with silu over values, B and C; the scan; gate, norm in groups, W_o."""
    T = h.shape[0]
    Hs, P, N, Gs = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hs * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * Gs * N], proj[:, 2 * inner + 2 * Gs * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, Hs, P)
    B = xbc[:, inner:inner + Gs * N].reshape(T, Gs, N)
    C = xbc[:, inner + Gs * N:].reshape(T, Gs, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = selective_scan(x, B, C, dt, w[p + "A_log"], w[p + "D"]).reshape(T, inner)
    y = group_rms_norm(y * silu(z), w[p + "norm"], m["norm_groups"], eps)
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps, positions):
    return (m["left_scale"] * attention_branch(h, w, p + "left.", m["left"], positions)
            + m["right_scale"] * recurrent_branch(h, w, p + "right.", m["right"], eps))


def gated_mlp(h, w, p):
    return (torch.relu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def hyper_sublayer(xs, w, p, norm_w, eps, fn):
    """xs [S, T, d]: the sublayer reads u = Σ_s in[s]·x_s through its norm; every stream then becomes
    x_t ← Σ_s mix[s, t]·x_s + out[t]·y, all from the old streams."""
    u = torch.einsum("s,std->td", w[p + "in"], xs)
    y = fn(rms_norm(u, norm_w, eps))
    return torch.einsum("sj,std->jtd", w[p + "mix"], xs) + w[p + "out"][:, None, None] * y[None]


def schedule(cfg):
    """The order in which layers run: layers start … stop−1 `times` times in a row, the others once."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, k = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n))


def forward(cfg, w, ids, keep_layers=False):
    """Logits at every position [T, vocab] (and, on request, the summed streams after every layer run)."""
    w = {k: v.to(torch.float64) for k, v in w.items()}
    T = len(ids)
    eps = cfg["norm"]["eps"]
    positions = torch.arange(T)
    x0 = w["embed"][torch.tensor(ids)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    S = cfg.get("streams")
    xs = x0[None].repeat(S or 1, 1, 1)
    after = []
    for i in schedule(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        mix = lambda hh: parallel_mixer(hh, w, p + "mix.", layer["mixer"], eps, positions)   # noqa: E731
        ff = lambda hh: gated_mlp(hh, w, p + "mlp.")                                          # noqa: E731
        if S:
            xs = hyper_sublayer(xs, w, p + "hc1.", w[p + "norm1"], eps, mix)
            if layer.get("mlp"):
                xs = hyper_sublayer(xs, w, p + "hc2.", w[p + "norm2"], eps, ff)
        else:
            xs = xs + mix(rms_norm(xs[0], w[p + "norm1"], eps))[None]
            if layer.get("mlp"):
                xs = xs + ff(rms_norm(xs[0], w[p + "norm2"], eps))[None]
        after.append(xs.sum(0))
    logits = rms_norm(xs.sum(0), w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if keep_layers else logits


def logits_all_positions(cfg, w, ids):
    return forward(cfg, w, ids)


def greedy_generate(cfg, w, prompt, n_new):
    """The n_new tokens that taking the largest logit generates (the first maximal index), recomputing everything."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        t = int(torch.argmax(forward(cfg, w, ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
