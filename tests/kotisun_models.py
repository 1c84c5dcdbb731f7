"""Small Kotisun configurations for the tests: every size differs from layer to layer and between the models, and what a
configuration could make equal or 1 by accident (query/key size and value size, heads and key/value heads, groups and
heads, one norm group, one stream, one tap, a rotation of the whole head, a window of one token, a window that ends on a
block border, a loop that runs once) is covered somewhere, as is every key that may be absent."""
import json
from pathlib import Path

import torch


def _left(heads, kv_heads, dim, vdim, scale, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        base, dims, factor = rot
        m["rot"] = {"base": base, "dims": dims}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    return m


def _right(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _layer(left, right, ls, rs, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


#: three streams, a loop over two layers, a layer without feed-forward, a window inside a block and one across a border,
#: a layer without window and rotation, heads = kv_heads, dim = vdim, groups = heads, a rotation of the whole head
KOT_A = {"architecture": "Kotisun", "vocab": 263, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "streams": 3,
         "loop": {"start": 1, "stop": 3, "times": 2}, "logit_softcap": 20.0, "layers": [
    _layer(_left(4, 2, 16, 24, 0.25, 40, (10000.0, 8, 2.0)), _right(4, 8, 16, 2, 4, 2), 0.7, 1.1, 96),
    _layer(_left(2, 2, 32, 32, 0.2, 70, (500.0, 32, None)), _right(2, 24, 8, 1, 2, 1), 1.3, 0.5, None),
    _layer(_left(6, 1, 8, 16, 0.3), _right(3, 16, 24, 3, 3, 3), 0.9, 0.8, 72),
    _layer(_left(3, 3, 24, 8, 0.22, 130, (30000.0, 12, 8.0)), _right(6, 8, 8, 2, 4, 6), 0.4, 1.2, 40),
]}
#: one stream, no loop, no soft cap, no embedding scale; windows of 1, 64 and 65 tokens; one tap; one head
KOT_B = {"architecture": "Kotisun", "vocab": 197, "width": 96, "norm": {"eps": 1e-6}, "streams": 1, "layers": [
    _layer(_left(1, 1, 48, 16, 0.15, 64, (1000.0, 48, 1.5)), _right(1, 32, 16, 1, 1, 1), 1.0, 1.0, 128),
    _layer(_left(4, 4, 16, 40, 0.3, 1, (1000.0, 4, None)), _right(8, 8, 4, 4, 4, 2), 0.5, 0.5, 64),
    _layer(_left(6, 3, 16, 8, 0.28, 65, (77.0, 16, 3.0)), _right(2, 40, 32, 2, 6, 5), 0.8, 1.4, None),
]}
#: no streams at all (the plain residual sum), a loop that covers every layer and one that runs once is in KOT_ODD
KOT_PLAIN = {"architecture": "Kotisun", "vocab": 211, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
             "loop": {"start": 0, "stop": 2, "times": 3}, "logit_softcap": 25.0, "layers": [
    _layer(_left(2, 1, 24, 16, 0.2, 33, (10000.0, 24, 4.0)), _right(3, 16, 8, 1, 3, 1), 0.6, 0.9, 80),
    _layer(_left(3, 3, 16, 24, 0.25, 100, (10000.0, 8, 4.0)), _right(2, 24, 16, 2, 4, 4), 1.0, 0.7, 56),
]}
#: sizes that are no multiples of 8, five streams, a loop that runs once
KOT_ODD = {"architecture": "Kotisun", "vocab": 149, "width": 100, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.7}, "streams": 5,
           "loop": {"start": 1, "stop": 2, "times": 1}, "logit_softcap": 50.0, "layers": [
    _layer(_left(3, 1, 12, 20, 0.21, 37, (3000.0, 6, 1.3)), _right(5, 6, 10, 5, 5, 3), 0.65, 0.95, 90),
    _layer(_left(2, 2, 20, 12, 0.19, 7, (3000.0, 10, None)), _right(2, 14, 6, 1, 2, 7), 1.05, 0.75, 44),
]}
#: attention made sharp and a recurrence that keeps its state for hundreds of tokens (see `write_model`), so that a wrong
#: key, a window's edge one token off or a lost state moves the logits far beyond rounding
KOT_SHARP = {"architecture": "Kotisun", "vocab": 223, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5}, "streams": 2,
             "loop": {"start": 0, "stop": 1, "times": 2}, "logit_softcap": 30.0, "layers": [
    _layer(_left(4, 2, 16, 16, 0.25, 48, (10000.0, 16, 2.0)), _right(4, 16, 16, 2, 4, 2), 1.0, 1.0, 96),
    _layer(_left(2, 1, 32, 24, 0.18, 66, (10000.0, 8, None)), _right(2, 16, 32, 1, 3, 1), 0.8, 1.2, 64),
]}
SHARP_FACTOR = 4.0
MODELS = {"kot_a": KOT_A, "kot_b": KOT_B, "kot_plain": KOT_PLAIN, "kot_odd": KOT_ODD, "kot_sharp": KOT_SHARP}


def write_model(cfg: dict, seed: int, out_dir, sharp: float = 1.0) -> None:
    """The package's random draw for the configuration; with `sharp` > 1 the query matrices are multiplied by it and the
    recurrence's decay rates made small (a state that lasts)."""
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.registry import parse_config
    from vlrf_b200.weights import write_safetensors
    arch, parsed = parse_config(cfg)
    tensors = arch.random_weights(parsed, torch.Generator().manual_seed(seed))
    if sharp != 1.0:
        for name in tensors:
            if name.endswith("mix.left.q"):
                tensors[name] = tensors[name] * sharp
            if name.endswith("A_log"):
                tensors[name] = tensors[name] - 3.0
    Path(out_dir).mkdir(parents=True, exist_ok=True)
    (Path(out_dir) / "config.json").write_text(json.dumps(cfg, indent=2))
    write_safetensors(Path(out_dir) / "model.safetensors",
                      {k: (v.to(torch.bfloat16) if v.is_floating_point() else v) for k, v in tensors.items()})
