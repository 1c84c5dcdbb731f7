"""Kuvusun: a decoder of latent-attention layers with dense or routed feed-forwards.

Tensors (all linear weights [out, in]): `embed` [vocab, width] and `embed.norm`; per layer i `l<i>.norm1`, `l<i>.norm2`,
the mixer's `l<i>.mix.*` and the feed-forward's `l<i>.mlp.*`; `final.norm`.  The head is the embedding table.

  mixer "latent_attention"     mix.dq, mix.dq.norm, mix.uq (queries through a latent), mix.dkv, mix.dkv.norm, mix.uk,
                               mix.uv, mix.o
  mixer "latent_attention_2"   mix.q, mix.dkv ([kv_rank + rot_dim, width]; absent with kv_from), mix.dkv.norm, mix.uk,
                               mix.uv, mix.g (sigmoid gate on the merged heads), mix.o
  mlp "dense"                  mlp.up, mlp.down (activation relu²)
  mlp "moe"                    mlp.router, mlp.router.b, mlp.e<k>.gate / .up / .down, and with a shared expert
                               mlp.shared.gate / .up / .down / .sg

The embedding and the last hidden rows go through the model's norm (RMS norm in groups); every layer is
x += norm1(mixer(x)); x += norm2(ffn(x)), the norm on the sublayer's output.  A layer with `kv_from` reads that
layer's cache rows and writes none.
"""
from __future__ import annotations

import torch

from ..config.kuvusun import KuvusunConfig
from ..engine.model import BuildOptions, DecoderModel, LayerCall
from ..parts import LMHead, TokenEmbedding, get_part
from ..registry import Architecture, register_architecture
from ..weights.spec import CheckedWeights, TensorSpec, place

#: positions a sequence may reach: the design has no position table, so this only sizes the block tables
MAX_POSITIONS = 1 << 17


def weight_spec(cfg: KuvusunConfig) -> list[TensorSpec]:
    d = cfg.width
    specs = [TensorSpec("embed", (cfg.vocab, d)), TensorSpec("embed.norm", (d,), "vector")]
    for i, (m, ml) in enumerate(zip(cfg.mixers, cfg.mlps)):
        p = f"l{i}."
        specs.append(TensorSpec(p + "norm1", (d,), "vector"))
        specs.append(TensorSpec(p + "norm2", (d,), "vector", optional=ml is None))
        per_q = m.dim + m.rot_dim
        if m.q_rank is not None:
            specs += [TensorSpec(p + "mix.dq", (m.q_rank, d)), TensorSpec(p + "mix.dq.norm", (m.q_rank,), "vector"),
                      TensorSpec(p + "mix.uq", (m.heads * per_q, m.q_rank))]
        else:
            specs.append(TensorSpec(p + "mix.q", (m.heads * per_q, d)))
        if m.kv_from is None:
            specs += [TensorSpec(p + "mix.dkv", (m.kv_rank + m.rot_dim, d)), TensorSpec(p + "mix.dkv.norm", (m.kv_rank,), "vector")]
        specs += [TensorSpec(p + "mix.uk", (m.heads * m.dim, m.kv_rank)), TensorSpec(p + "mix.uv", (m.heads * m.vdim, m.kv_rank))]
        if m.gated:
            specs.append(TensorSpec(p + "mix.g", (m.heads * m.vdim, d)))
        specs.append(TensorSpec(p + "mix.o", (d, m.heads * m.vdim)))
        if ml is None:
            continue
        if ml.kind == "dense":
            specs += [TensorSpec(p + "mlp.up", (ml.ff, d)), TensorSpec(p + "mlp.down", (d, ml.ff))]
        else:
            specs += [TensorSpec(p + "mlp.router", (ml.experts, d)), TensorSpec(p + "mlp.router.b", (ml.experts,), "vector")]
            for e in range(ml.experts):
                q = p + f"mlp.e{e}."
                specs += [TensorSpec(q + "gate", (ml.ff, d)), TensorSpec(q + "up", (ml.ff, d)), TensorSpec(q + "down", (d, ml.ff))]
            if ml.shared_ff is not None:
                q = p + "mlp.shared."
                specs += [TensorSpec(q + "gate", (ml.shared_ff, d)), TensorSpec(q + "up", (ml.shared_ff, d)),
                          TensorSpec(q + "down", (d, ml.shared_ff)), TensorSpec(q + "sg", (1, d))]
    specs.append(TensorSpec("final.norm", (d,), "vector"))
    return specs


def random_weights(cfg: KuvusunConfig, gen: torch.Generator) -> dict:
    """Matrices N(0, 1/in) (so that every product keeps the scale of its input), norm weights 1 + N(0, 0.1), router
    biases N(0, 0.1): no term of a formula is hidden by a zero or a one.  The norm behind the embedding is drawn ten
    times smaller: with the embedding as head a token's own embedding otherwise dominates its logits, and a random
    model does nothing but repeat its last token whatever its layers compute."""
    out = {}
    for spec in weight_spec(cfg):
        t = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        if spec.kind == "vector":
            t = 0.1 * t if spec.name.endswith("router.b") else 1.0 + 0.1 * t
            if spec.name == "embed.norm":
                t = 0.1 * t
        elif spec.name == "embed":
            pass
        else:
            t = t / float(spec.shape[-1]) ** 0.5
        out[spec.name] = t
    return out


def build(cfg: KuvusunConfig, weights: CheckedWeights, options: BuildOptions) -> DecoderModel:
    dt, dev = options.dtype, options.device

    def matrix(name):
        return place(weights[name], "matrix", dt, dev)

    def vector(name):
        return place(weights[name], "vector", dt, dev)

    norm_cls = get_part("norm", "group_rmsnorm")

    def model_norm(name):
        return norm_cls(vector(name), cfg.norm_eps, cfg.norm_groups)

    embed = matrix("embed")
    embedding = TokenEmbedding(embed, None, norm=model_norm("embed.norm"))
    mixer_cls, block_cls = get_part("mixer", "latent_attention"), get_part("block", "sublayer_norm")
    layers, schedule, rotations = [], [], {}
    for i, (m, ml) in enumerate(zip(cfg.mixers, cfg.mlps)):
        p = f"l{i}."
        rotary = None
        if m.rot_dim > 0:
            rk = (m.rot_base, m.rot_dims)
            if rk not in rotations:
                rotations[rk] = get_part("position", "rotary")(m.rot_base, m.rot_dims, dev)
            rotary = rotations[rk]
        own = m.kv_from is None
        mixer = mixer_cls(
            n_heads=m.heads, dim=m.dim, vdim=m.vdim, kv_rank=m.kv_rank, rot_dim=m.rot_dim, scale=m.scale, eps=cfg.norm_eps,
            w_q=matrix(p + "mix.q") if m.q_rank is None else None,
            w_dq=matrix(p + "mix.dq") if m.q_rank is not None else None,
            dq_norm=vector(p + "mix.dq.norm") if m.q_rank is not None else None,
            w_uq=matrix(p + "mix.uq") if m.q_rank is not None else None,
            w_dkv=matrix(p + "mix.dkv") if own else None, dkv_norm=vector(p + "mix.dkv.norm") if own else None,
            w_uk=matrix(p + "mix.uk"), w_uv=matrix(p + "mix.uv"), w_gate=matrix(p + "mix.g") if m.gated else None,
            w_out=matrix(p + "mix.o"), rotary=rotary)
        ffn = norm2 = None
        if ml is not None:
            norm2 = model_norm(p + "norm2")
            if ml.kind == "dense":
                ffn = get_part("feed_forward", "dense_mlp")(matrix(p + "mlp.up"), None, matrix(p + "mlp.down"), None,
                                                            activation="relu2")
            else:
                def stack(what):
                    return torch.stack([matrix(p + f"mlp.e{e}.{what}") for e in range(ml.experts)]).contiguous()
                shared = None
                if ml.shared_ff is not None:
                    q = p + "mlp.shared."
                    shared = (matrix(q + "gate"), matrix(q + "up"), matrix(q + "down"), matrix(q + "sg"))
                ffn = get_part("feed_forward", "routed_experts")(
                    matrix(p + "mlp.router"), vector(p + "mlp.router.b"), stack("gate"), stack("up"), stack("down"),
                    top=ml.top, shared=shared)
        layers.append(block_cls(model_norm(p + "norm1"), mixer, norm2, ffn))
        schedule.append(LayerCall(i, reads_cache_of=m.kv_from))
    return DecoderModel(config=cfg, embedding=embedding, layers=layers, schedule=schedule,
                        final_norm=model_norm("final.norm"), head=LMHead(embed), options=options,
                        max_seq_len=MAX_POSITIONS)


KUVUSUN = register_architecture(Architecture(
    name="Kuvusun", config_cls=KuvusunConfig, weight_spec=weight_spec, random_weights=random_weights, build=build))
