"""Kotisun configurations drawn at random (every size, count, window, constant and the order of layers from a seeded
generator; keys that may be absent are absent now and then) through the engine against the plain implementation: whole,
the last tokens one by one, and an unequal batch.  What the hand-made models happen not to combine shows here.

The 32-bit comparison is the sharp one.  A drawn model can be badly conditioned (rounding every product's operands to
bfloat16 in the plain implementation alone moves one of these models' logits by 6 % of their scale), so the bfloat16
bound here is wide: it is there to show a kernel of the bfloat16 path that a size sends wrong, not to grade rounding."""
import random

import pytest
import torch

import plain_kotisun as plain
from conftest import random_ids, record_error
from engine_drives import drive_batches, drive_tail_one_by_one, drive_whole
from kotisun_models import write_model
from test_kotisun import compare, poison_states

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    r = random.Random(seed)
    width = r.choice([32, 40, 48, 64, 72, 96, 100, 128, 160])
    cfg = {"architecture": "Kotisun", "vocab": r.choice([97, 128, 200, 333]), "width": width, "norm": {"eps": r.choice([1e-5, 1e-6])}}
    if r.random() < 0.8:
        cfg["embedding"] = {"scale": r.choice([0.7, 1.0, 2.5, 4.0])}
    if r.random() < 0.85:
        cfg["streams"] = r.choice([1, 2, 3, 4, 6])
    if r.random() < 0.7:
        cfg["logit_softcap"] = r.choice([15.0, 30.0, 50.0])
    n_layers = r.choice([1, 2, 3, 4])
    layers = []
    for _ in range(n_layers):
        kv = r.choice([1, 2, 3, 4])
        heads = kv * r.choice([1, 1, 2, 3, 6])
        dim, vdim = r.choice([8, 16, 24, 32, 40, 64, 80, 96, 128, 12]), r.choice([8, 16, 24, 32, 48, 64, 80, 104, 128, 20])
        left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": round(dim ** -0.5 * r.choice([0.8, 1.0, 1.5]), 4)}
        if r.random() < 0.85:
            left["mask"] = {"size": r.choice([1, 2, 5, 17, 31, 32, 33, 63, 64, 65, 90, 128, 129, 200])}
        if r.random() < 0.85:
            dims = r.choice([d for d in (2, 4, 8, 16, 32, 64, dim) if d <= dim and d % 2 == 0])
            left["rot"] = {"base": r.choice([100.0, 10000.0, 250000.0]), "dims": dims}
            if r.random() < 0.7:
                left["rot"]["scaling"] = {"factor": r.choice([1.0, 2.0, 4.0, 8.0])}
        groups = r.choice([1, 2, 3])
        r_heads = groups * r.choice([1, 2, 3])
        r_vdim = r.choice([4, 6, 8, 16, 24, 32, 40, 48, 64, 80])
        inner = r_heads * r_vdim
        right = {"heads": r_heads, "vdim": r_vdim, "state": r.choice([4, 6, 8, 16, 24, 32, 48, 64, 72, 128, 136]), "groups": groups,
                 "conv": r.choice([1, 2, 3, 4, 4, 6]), "norm_groups": r.choice([g for g in (1, 2, 3, 4, 6, 8) if inner % g == 0])}
        layers.append({"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": r.choice([0.4, 0.6, 1.0, 1.3]),
                                                      "right_scale": r.choice([0.5, 0.9, 1.0, 1.2])},
                       "mlp": {"kind": "dense", "ff": r.choice([24, 64, 100, 136, 256])} if r.random() < 0.85 else None})
    cfg["layers"] = layers
    if r.random() < 0.7:
        a = r.randrange(0, n_layers)
        b = r.randrange(a, n_layers + 1)
        cfg["loop"] = {"start": a, "stop": b, "times": r.choice([1, 2, 3])}
    return cfg


@pytest.mark.parametrize("seed", range(16))
def test_a_random_model_whole_decoded_and_batched(tmp_path, seed):
    from vlrf_b200.engine import Engine, load_model
    cfg = draw_config(1000 + seed)
    write_model(cfg, seed, tmp_path)
    pc, w = plain.read_model_dir(tmp_path)
    reqs = [random_ids(cfg["vocab"], n, 31 * seed + i) for i, n in enumerate((1 + seed % 3, 70 + 3 * seed, 137))]
    want = [plain.logits_all_positions(pc, w, ids) for ids in reqs]
    for dtype in ("float32", "bfloat16"):
        eng = Engine(load_model(tmp_path, dtype), max_tokens=512)
        poison_states(eng)
        name, tol = f"random {seed}", None if dtype == "float32" else 0.15
        compare(drive_whole(eng, reqs), want, dtype, "whole", name, tol)
        compare(drive_tail_one_by_one(eng, reqs, 40), want, dtype, "prefix + 40 single tokens", name, tol)
        poison_states(eng)
        compare(drive_batches(eng, reqs, 3, [1, 33, 100]), want, dtype, "unequal batch", name, tol)
        assert eng.cache.slots.n_held == 0
