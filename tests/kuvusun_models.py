"""Small Kuvusun configurations for the tests: every size differs from layer to layer and between the models, and
what a configuration could make equal by accident (query/key size and value size, rotated size, an expert's inner
size and the shared expert's, top = 1, top = all experts, one norm group) is covered somewhere."""
import json
from pathlib import Path

import torch


def _att1(heads, dim, vdim, kv_rank, q_rank, scale):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}}


def _att2(heads, dim, vdim, kv_rank, rot_dim, base, scale, kv_from=None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "rot_dim": rot_dim,
         "rot": {"base": base, "dims": rot_dims or rot_dim}, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention_2", "mixer": m}


def _moe(ff, experts, top, shared_ff=None):
    ml = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff is not None:
        ml["shared"] = {"ff": shared_ff}
    return ml


def _layer(att, mlp):
    return dict(att, mlp=mlp)


#: rotated layers first, a layer that reads the cache of a layer two before it, a layer without feed-forward, experts
#: without a shared one and with top = all
KUV_A = {"architecture": "Kuvusun", "vocab": 301, "width": 96, "norm": {"eps": 1e-5, "groups": 3}, "layers": [
    _layer(_att2(3, 16, 24, 40, 8, 10000.0, 0.2), _moe(48, 5, 2, 80)),
    _layer(_att1(4, 24, 16, 56, 72, 0.15), {"kind": "dense", "ff": 136}),
    _layer(_att2(5, 8, 16, 40, 8, 10000.0, 0.3, kv_from=0), None),
    _layer(_att2(2, 32, 8, 24, 16, 500.0, 0.18), _moe(40, 4, 4)),
]}
#: one norm group, one head, top = 1, the unrotated-only mixer twice with different sizes
KUV_B = {"architecture": "Kuvusun", "vocab": 257, "width": 128, "norm": {"eps": 1e-6, "groups": 1}, "layers": [
    _layer(_att1(1, 64, 32, 64, 48, 0.11), _moe(64, 8, 1, 32)),
    _layer(_att1(6, 16, 8, 96, 40, 0.25), {"kind": "dense", "ff": 200}),
    _layer(_att2(4, 16, 32, 72, 24, 1000.0, 0.16), {"kind": "dense", "ff": 72}),
    _layer(_att2(2, 24, 16, 72, 24, 1000.0, 0.2, kv_from=2), _moe(24, 3, 2, 24)),
]}
#: sizes that are no multiples of 8 (tails in every product, rows that no vector load fits)
KUV_ODD = {"architecture": "Kuvusun", "vocab": 199, "width": 100, "norm": {"eps": 1e-5, "groups": 5}, "layers": [
    _layer(_att2(3, 12, 20, 36, 6, 3000.0, 0.21), _moe(28, 6, 3, 44)),
    _layer(_att1(2, 20, 12, 52, 30, 0.19), {"kind": "dense", "ff": 90}),
]}
#: attention made sharp (the query projections are drawn larger, see `write_model`), so that a wrong key, scale or
#: mask edge moves the logits by far more than rounding does
#: (no routed experts: every position can be held against the plain implementation in bfloat16 too)
KUV_SHARP = {"architecture": "Kuvusun", "vocab": 311, "width": 64, "norm": {"eps": 1e-5, "groups": 2}, "layers": [
    _layer(_att2(2, 16, 16, 32, 16, 10000.0, 0.25), {"kind": "dense", "ff": 96}),
    _layer(_att1(2, 32, 24, 48, 40, 0.18), None),
    _layer(_att2(4, 8, 8, 32, 16, 10000.0, 0.3, kv_from=0), {"kind": "dense", "ff": 64}),
]}
SHARP_FACTOR = 2.0
MODELS = {"kuv_a": KUV_A, "kuv_b": KUV_B, "kuv_odd": KUV_ODD, "kuv_sharp": KUV_SHARP}


def write_model(cfg: dict, seed: int, out_dir, sharp: float = 1.0, embedding: float = 1.0) -> None:
    """The package's random draw for the configuration, the matrices that make queries multiplied by `sharp` and the
    weight of the norm behind the embedding by `embedding` (with a tied head a token's own embedding otherwise
    dominates its logits, and every model just repeats its last token)."""
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.registry import parse_config
    from vlrf_b200.weights import write_safetensors
    arch, parsed = parse_config(cfg)
    tensors = arch.random_weights(parsed, torch.Generator().manual_seed(seed))
    for name in tensors:
        if name.endswith("mix.q") or name.endswith("mix.uq"):
            tensors[name] = tensors[name] * sharp
        if name == "embed.norm":
            tensors[name] = tensors[name] * embedding
        if name.endswith("router.b"):
            tensors[name] = tensors[name] * 10.0          # fewer close calls between experts (see the plain decided_prefix)
    Path(out_dir).mkdir(parents=True, exist_ok=True)
    (Path(out_dir) / "config.json").write_text(json.dumps(cfg, indent=2))
    write_safetensors(Path(out_dir) / "model.safetensors",
                      {k: (v.to(torch.bfloat16) if v.is_floating_point() else v) for k, v in tensors.items()})
