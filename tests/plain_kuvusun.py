"""A plain, slow implementation of the Kuvusun design in float64, one function per mechanism, written from the
design's equations and sharing no code with the package (it reads model folders with the tests' own reader).

Notation: T tokens, width d.  Linear weights are [out, in] and applied as x · Wᵀ.
"""
from __future__ import annotations

import math

import torch

from plain_gpt2 import read_model_dir  # noqa: F401  (the tests' own reader of config.json + model.safetensors)


def group_rms_norm(x, w, groups, eps):
    """Each of `groups` equal consecutive parts of the last axis divided by sqrt(mean(part²) + eps); then · w."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(shape) * w


def rms_norm(x, w, eps):
    return group_rms_norm(x, w, 1, eps)


def rotate(v, positions, base, dims):
    """v [T, …, n]: of the first `dims` entries, entry i pairs with entry i + dims/2; the pair (a, b) at position p
    becomes (a cos t − b sin t, b cos t + a sin t), t = p · base^(−2i/dims).  Entries beyond dims pass."""
    half = dims // 2
    out = v.clone()
    for i in range(half):
        f = float(base) ** (-2.0 * i / dims)
        t = positions.to(torch.float64) * f
        while t.dim() < v.dim() - 1:
            t = t.unsqueeze(-1)
        a, b = v[..., i], v[..., i + half]
        out[..., i] = a * torch.cos(t) - b * torch.sin(t)
        out[..., i + half] = b * torch.cos(t) + a * torch.sin(t)
    return out


def causal_softmax_attention(scores, values):
    """scores [H, T, T] (query, key), values [T, H, n] → [T, H, n]; query i sees keys j ≤ i."""
    T = scores.shape[1]
    out = torch.zeros(T, values.shape[1], values.shape[2], dtype=scores.dtype)
    for i in range(T):
        p = torch.softmax(scores[:, i, :i + 1], dim=-1)                    # [H, i+1]
        out[i] = torch.einsum("hj,jhn->hn", p, values[:i + 1])
    return out


def latent_rows(h, w, prefix, m, eps, positions):
    """What a layer with a cache of its own keeps per token: the normed latent c [T, kv_rank] and, with a rotated
    part, the rotated shared key part r [T, rot_dim] (else None)."""
    proj = h @ w[prefix + "dkv"].T
    c = rms_norm(proj[:, :m["kv_rank"]], w[prefix + "dkv.norm"], eps)
    r = None
    if m.get("rot_dim", 0) > 0:
        r = rotate(proj[:, m["kv_rank"]:], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, r


def latent_attention(h, w, prefix, m, eps, positions, rows):
    """The mixer.  `rows` = (c, r) of the layer whose cache is read (its own or another's)."""
    T, H, dim, vdim = h.shape[0], m["heads"], m["dim"], m["vdim"]
    R = m.get("rot_dim", 0)
    if "q_rank" in m:
        cq = rms_norm(h @ w[prefix + "dq"].T, w[prefix + "dq.norm"], eps)
        q = (cq @ w[prefix + "uq"].T).reshape(T, H, dim + R)
    else:
        q = (h @ w[prefix + "q"].T).reshape(T, H, dim + R)
    c, r = rows
    k = (c @ w[prefix + "uk"].T).reshape(T, H, dim)
    v = (c @ w[prefix + "uv"].T).reshape(T, H, vdim)
    scores = torch.einsum("ihd,jhd->hij", q[..., :dim], k)
    if R > 0:
        qr = rotate(q[..., dim:], positions, m["rot"]["base"], m["rot"]["dims"])
        scores = scores + torch.einsum("ihd,jd->hij", qr, r)
    merged = causal_softmax_attention(scores * m["scale"], v).reshape(T, H * vdim)
    if prefix + "g" in w:
        merged = merged * torch.sigmoid(h @ w[prefix + "g"].T)
    return merged @ w[prefix + "o"].T


def dense_ff(h, w, prefix):
    return (torch.relu(h @ w[prefix + "up"].T) ** 2) @ w[prefix + "down"].T


def gated_expert(h, w, prefix):
    g = h @ w[prefix + "gate"].T
    return ((g * torch.sigmoid(g)) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(z, top):
    """The `top` largest logits per row (ties: lower index) and the softmax over them alone."""
    idx = torch.zeros(z.shape[0], top, dtype=torch.long)
    for t in range(z.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-float(z[t, e]), e))
        idx[t] = torch.tensor(order[:top])
    val = torch.gather(z, 1, idx)
    return idx, torch.softmax(val, dim=-1)


def routed_ff(h, w, prefix, ml, margins=None):
    z = h @ w[prefix + "router"].T + w[prefix + "router.b"]
    idx, wt = route(z, ml["router"]["top"])
    if margins is not None:          # by how much the last chosen logit beats the first one left out, per token,
        top = ml["router"]["top"]    # over the size of the token's logits (an error of rounding grows with them)
        s = torch.sort(z, dim=-1, descending=True).values
        size = z.abs().max(dim=-1).values.clamp_min(1.0)
        margins.append((s[:, top - 1] - s[:, top]) / size if top < z.shape[1] else torch.full((z.shape[0],), float("inf"), dtype=z.dtype))
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            y[t] += wt[t, j] * gated_expert(h[t:t + 1], w, prefix + f"e{int(idx[t, j])}.")[0]
    if ml.get("shared") is not None:
        y = y + gated_expert(h, w, prefix + "shared.") * torch.sigmoid(h @ w[prefix + "shared.sg"].T)
    return y


def hidden_all_positions(cfg, w, ids, per_layer=None, margins=None):
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    positions = torch.arange(len(ids))
    x = group_rms_norm(w["embed"][torch.tensor(ids)], w["embed.norm"], groups, eps)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        src = m.get("kv_from")
        if src is None:
            kept[i] = latent_rows(x, w, p + "mix.", m, eps, positions)
            src = i
        x = x + group_rms_norm(latent_attention(x, w, p + "mix.", m, eps, positions, kept[src]), w[p + "norm1"], groups, eps)
        ml = layer.get("mlp")
        if ml is not None:
            y = dense_ff(x, w, p + "mlp.") if ml["kind"] == "dense" else routed_ff(x, w, p + "mlp.", ml, margins)
            x = x + group_rms_norm(y, w[p + "norm2"], groups, eps)
        if per_layer is not None:
            per_layer.append(x.clone())
    return x


def logits_all_positions(cfg, w, ids):
    x = hidden_all_positions(cfg, w, ids)
    return group_rms_norm(x, w["final.norm"], cfg["norm"]["groups"], cfg["norm"]["eps"]) @ w["embed"].T


def decided_prefix(cfg, w, ids, least=0.05):
    """How many leading positions of a request are free of close calls of any router: up to the first token whose
    last chosen logit beats the first one left out by less than `least` of the size of its logits.  An implementation that rounds differently
    may choose other experts there, and everything after may attend that token."""
    margins = []
    hidden_all_positions(cfg, w, ids, margins=margins)
    n = len(ids)
    for m in margins:
        close = (m < least).nonzero()
        if close.numel():
            n = min(n, int(close[0]))
    return n


def greedy_generate(cfg, w, prompt, max_new_tokens):
    ids = list(prompt)
    for _ in range(max_new_tokens):
        ids.append(int(torch.argmax(logits_all_positions(cfg, w, ids)[-1])))
    return ids[len(prompt):]
