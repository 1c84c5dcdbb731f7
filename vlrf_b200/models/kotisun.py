"""Kotisun: a decoder whose layers run windowed softmax attention and a state-space recurrence side by side, over a
residual carried in several streams, with a range of layers that is run several times.

Tensors (all linear weights [out, in]): `embed` [vocab, width]; per layer i `l<i>.norm1`, `l<i>.norm2`; the attention
branch `l<i>.mix.left.q / .k / .v` with biases `.q.b / .k.b / .v.b` and `.o`; the recurrent branch `l<i>.mix.right.in`,
`.conv` [channels, taps], `.conv.b`, `.dt_bias`, `.A_log`, `.D`, `.norm`, `.o`; the feed-forward `l<i>.mlp.gate / .up /
.down`; with streams, `l<i>.hc1.in / .out / .mix` and `l<i>.hc2.*` (read coefficients, write coefficients, and the
[from, to] mix of the streams for the mixer and for the feed-forward); `final.norm`; `head` [vocab, width].

  x = embed[token] · embedding.scale, copied into every stream
  per scheduled layer: sublayer 1 is the parallel mixer, sublayer 2 the gated feed-forward (relu gate), each read and
  written through the streams (parts/block.py, "hyper_connection"); without streams, x += sublayer(norm(x))
  logits = cap · tanh(head · norm(Σ streams) / cap)

A layer inside the loop appears several times in the schedule; every appearance has a cache and state of its own.
"""
from __future__ import annotations

import torch

from ..config.kotisun import KotisunConfig
from ..engine.model import BuildOptions, DecoderModel, LayerCall
from ..parts import LMHead, TokenEmbedding, get_part
from ..registry import Architecture, register_architecture
from ..weights.spec import CheckedWeights, TensorSpec, place

#: positions a sequence may reach: the design has no position table, so this only sizes the block tables
MAX_POSITIONS = 1 << 17


def weight_spec(cfg: KotisunConfig) -> list[TensorSpec]:
    d, S = cfg.width, cfg.streams
    specs = [TensorSpec("embed", (cfg.vocab, d))]
    for i, lc in enumerate(cfg.layer_configs):
        p = f"l{i}."
        a, r = lc.left, lc.right
        inner, channels = r.heads * r.vdim, r.heads * r.vdim + 2 * r.groups * r.state
        specs += [TensorSpec(p + "norm1", (d,), "vector"), TensorSpec(p + "norm2", (d,), "vector", optional=lc.ff is None)]
        q = p + "mix.left."
        specs += [TensorSpec(q + "q", (a.heads * a.dim, d)), TensorSpec(q + "q.b", (a.heads * a.dim,), "vector"),
                  TensorSpec(q + "k", (a.kv_heads * a.dim, d)), TensorSpec(q + "k.b", (a.kv_heads * a.dim,), "vector"),
                  TensorSpec(q + "v", (a.kv_heads * a.vdim, d)), TensorSpec(q + "v.b", (a.kv_heads * a.vdim,), "vector"),
                  TensorSpec(q + "o", (d, a.heads * a.vdim))]
        q = p + "mix.right."
        specs += [TensorSpec(q + "in", (2 * inner + 2 * r.groups * r.state + r.heads, d)),
                  TensorSpec(q + "conv", (channels, r.conv), "vector"), TensorSpec(q + "conv.b", (channels,), "vector"),
                  TensorSpec(q + "dt_bias", (r.heads,), "vector"), TensorSpec(q + "A_log", (r.heads,), "vector"),
                  TensorSpec(q + "D", (r.heads,), "vector"), TensorSpec(q + "norm", (inner,), "vector"),
                  TensorSpec(q + "o", (d, inner))]
        if lc.ff is not None:
            specs += [TensorSpec(p + "mlp.gate", (lc.ff, d)), TensorSpec(p + "mlp.up", (lc.ff, d)), TensorSpec(p + "mlp.down", (d, lc.ff))]
        if S is not None:
            for hc in ("hc1.",) + (("hc2.",) if lc.ff is not None else ()):
                specs += [TensorSpec(p + hc + "in", (S,), "vector"), TensorSpec(p + hc + "out", (S,), "vector"),
                          TensorSpec(p + hc + "mix", (S, S), "vector")]
            if lc.ff is None:
                specs += [TensorSpec(p + "hc2." + n, sh, "vector", optional=True) for n, sh in (("in", (S,)), ("out", (S,)), ("mix", (S, S)))]
    specs += [TensorSpec("final.norm", (d,), "vector"), TensorSpec("head", (cfg.vocab, d))]
    return specs


def random_weights(cfg: KotisunConfig, gen: torch.Generator) -> dict:
    """Matrices N(0, 1/in), norm weights 1 + N(0, 0.1), biases N(0, 0.3); the streams' coefficients near a plain
    residual (reads near 1/streams, writes near 1, a mix near the identity) with noise, so that no term is hidden; the
    recurrence's step bias and decay rates spread so that some heads forget within a few tokens and others keep
    hundreds; the embedding N(0, 1) and the head N(0, 1/width)."""
    S = cfg.streams
    out = {}
    for spec in weight_spec(cfg):
        if spec.optional:                  # (tensors of a feed-forward that the layer does not have)
            continue
        name, shape = spec.name, spec.shape
        t = torch.randn(shape, generator=gen, dtype=torch.float32)
        if name.endswith(".hc1.in") or name.endswith(".hc2.in"):
            t = 1.0 / S + 0.2 * t
        elif name.endswith(".hc1.out") or name.endswith(".hc2.out"):
            t = 1.0 + 0.3 * t
        elif name.endswith(".mix") and len(shape) == 2 and shape[0] == shape[1] == (S or -1) and ".hc" in name:
            t = torch.eye(S) + 0.15 * t
        elif name.endswith(".dt_bias"):
            t = -2.0 + 1.5 * torch.rand(shape, generator=gen)
        elif name.endswith(".A_log"):
            t = torch.log(0.05 + 3.0 * torch.rand(shape, generator=gen))
        elif name.endswith(".D"):
            t = 1.0 + 0.3 * t
        elif name.endswith(".conv"):
            t = t / float(shape[-1]) ** 0.5
        elif name.endswith(".b"):
            t = 0.3 * t
        elif spec.kind == "vector":
            t = 1.0 + 0.1 * t
        elif name == "embed":
            pass
        else:
            t = t / float(shape[-1]) ** 0.5
        out[name] = t
    return out


def build(cfg: KotisunConfig, weights: CheckedWeights, options: BuildOptions) -> DecoderModel:
    dt, dev = options.dtype, options.device

    def matrix(name):
        return place(weights[name], "matrix", dt, dev)

    def vector(name):
        return place(weights[name], "vector", dt, dev)

    S = cfg.streams
    stream_norm = get_part("norm", "stream_rmsnorm")
    plain_norm = get_part("norm", "group_rmsnorm")
    rotations, layers = {}, []
    for i, lc in enumerate(cfg.layer_configs):
        p = f"l{i}."
        a, r = lc.left, lc.right
        rotary = None
        if a.rot_dims > 0:
            rk = (a.rot_base, a.rot_dims, a.rot_factor)
            if rk not in rotations:
                rotations[rk] = get_part("position", "rotary")(a.rot_base, a.rot_dims, dev, scaling_factor=a.rot_factor)
            rotary = rotations[rk]
        q = p + "mix.left."
        left = get_part("mixer", "window_attention")(
            matrix(q + "q"), matrix(q + "k"), matrix(q + "v"), matrix(q + "o"), n_heads=a.heads, n_kv_heads=a.kv_heads, dim=a.dim,
            vdim=a.vdim, scale=a.scale, b_q=vector(q + "q.b"), b_k=vector(q + "k.b"), b_v=vector(q + "v.b"), window=a.window,
            rotary=rotary)
        q = p + "mix.right."
        right = get_part("mixer", "state_space")(
            matrix(q + "in"), vector(q + "conv"), vector(q + "conv.b"), vector(q + "dt_bias"), vector(q + "A_log"), vector(q + "D"),
            vector(q + "norm"), matrix(q + "o"), n_heads=r.heads, vdim=r.vdim, n_state=r.state, n_groups=r.groups,
            norm_groups=r.norm_groups, eps=cfg.norm_eps)
        mixer = get_part("mixer", "parallel")(left, right, left_scale=lc.left_scale, right_scale=lc.right_scale)
        ffn = None
        if lc.ff is not None:
            ffn = get_part("feed_forward", "gated_mlp")(matrix(p + "mlp.gate"), matrix(p + "mlp.up"), matrix(p + "mlp.down"),
                                                        activation="relu")
        if S is None:
            layers.append(get_part("block", "pre_norm")(plain_norm(vector(p + "norm1"), cfg.norm_eps, 1), mixer,
                                                        plain_norm(vector(p + "norm2"), cfg.norm_eps, 1) if ffn is not None else None, ffn))
        else:
            layers.append(get_part("block", "hyper_connection")(
                stream_norm(vector(p + "norm1"), cfg.norm_eps, S, vector(p + "hc1.in")), mixer,
                stream_norm(vector(p + "norm2"), cfg.norm_eps, S, vector(p + "hc2.in")) if ffn is not None else None, ffn,
                streams=S, mix1=vector(p + "hc1.mix"), out1=vector(p + "hc1.out"),
                mix2=vector(p + "hc2.mix") if ffn is not None else None, out2=vector(p + "hc2.out") if ffn is not None else None))
    embedding = TokenEmbedding(matrix("embed"), None, scale=cfg.embedding_scale, streams=S or 1)
    return DecoderModel(config=cfg, embedding=embedding, layers=layers, schedule=[LayerCall(i) for i in cfg.layer_order],
                        final_norm=stream_norm(vector("final.norm"), cfg.norm_eps, S or 1), head=LMHead(matrix("head"), cfg.logit_softcap),
                        options=options, max_seq_len=MAX_POSITIONS)


KOTISUN = register_architecture(Architecture(
    name="Kotisun", config_cls=KotisunConfig, weight_spec=weight_spec, random_weights=random_weights, build=build))
