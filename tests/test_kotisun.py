"""Kotisun through the engine against the plain implementation: whole requests, the last tokens one by one, prompts in
portions down to two tokens, unequal batches with reused slots, blocks and states, the first tokens, long decoding past
every window, and greedy generation through the package's entry point — in 32-bit and in bfloat16, on five small models
whose sizes all differ."""
import pytest
import torch

import plain_kotisun as plain
from conftest import random_ids, record_error
from engine_drives import drive_batches, drive_portions, drive_tail_one_by_one, drive_whole, poison
from kotisun_models import MODELS, SHARP_FACTOR, write_model

pytestmark = pytest.mark.gpu

#: largest absolute logit error over the largest absolute logit of the plain implementation
TOL = {"float32": 1e-4, "bfloat16": 6e-2}
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"kot_a": [1 + 12, 41 + 12, 64 + 12, 131 + 12, 150], "kot_b": [3 + 10, 63 + 10, 129 + 10, 180],
           "kot_plain": [2 + 8, 34 + 8, 100 + 8, 130], "kot_odd": [7 + 9, 38 + 9, 90], "kot_sharp": [5 + 16, 49 + 16, 127 + 16, 220]}
DECODE = {"kot_a": 12, "kot_b": 10, "kot_plain": 8, "kot_odd": 9, "kot_sharp": 16}
NAMES = list(MODELS)


def poison_states(engine):
    """NaN in every state of a slot that no sequence holds: a slot that is taken must be zeroed, not trusted."""
    poison(engine)
    for g in engine.cache._groups:
        if hasattr(g, "state"):
            for s in range(engine.cache.n_slots):
                if not engine.cache.slots.is_held(s):
                    g.state[:, s].fill_(float("nan"))


@pytest.fixture(scope="module")
def kot_dirs(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(MODELS.items()):
        d = tmp_path_factory.mktemp(name)
        write_model(cfg, 60 + i, d, sharp=SHARP_FACTOR if name == "kot_sharp" else 1.0)
        out[name] = d
    return out


@pytest.fixture(scope="module")
def truth(kot_dirs):
    out = {}
    for name, d in kot_dirs.items():
        cfg, w = plain.read_model_dir(d)
        reqs = [random_ids(cfg["vocab"], n, 21 + i) for i, n in enumerate(LENGTHS[name])]
        out[name] = (cfg, w, reqs, [plain.logits_all_positions(cfg, w, ids) for ids in reqs])
    return out


def make_engine(kot_dirs, name, dtype, max_tokens):
    from vlrf_b200.engine import Engine, load_model
    eng = Engine(load_model(kot_dirs[name], dtype), max_tokens=max_tokens)
    poison_states(eng)
    return eng


def compare(got, want, dtype, what, model, tol=None):
    tol = TOL[dtype] if tol is None else tol
    worst = 0.0
    for i, (g, t) in enumerate(zip(got, want)):
        assert g.shape == t.shape, f"{what}: request {i} has shape {tuple(g.shape)}, expected {tuple(t.shape)}"
        assert torch.isfinite(g).all(), f"{what}: request {i} has non-finite logits (something unwritten was read)"
        err = (g.double() - t).abs().max(dim=1).values / float(t.abs().max())
        bad = (err > tol).nonzero()
        assert bad.numel() == 0, (f"{what} ({model}, {dtype}): request {i} (length {len(t)}) first differs at position "
                                  f"{int(bad[0])} with error {float(err[bad[0]]):.3e} of the logit scale")
        worst = max(worst, float(err.max()))
    record_error("kotisun " + what, model, dtype, worst)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(kot_dirs, truth, name, dtype):
    _, _, reqs, want = truth[name]
    eng = make_engine(kot_dirs, name, dtype, 320)
    compare(drive_whole(eng, reqs), want, dtype, "whole", name)
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_tokens_one_by_one(kot_dirs, truth, name, dtype):
    _, _, reqs, want = truth[name]
    eng = make_engine(kot_dirs, name, dtype, 320)
    compare(drive_tail_one_by_one(eng, reqs, 32), want, dtype, "prefix + 32 single tokens", name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("portion", [2, 3, 7, 64, 65])
def test_prompts_in_portions(kot_dirs, truth, portion, dtype):
    """Portions of an even and of an odd number of tokens (the state's two copies), shorter than the convolution's reach,
    and ending on and just behind a block border."""
    for name in ("kot_a", "kot_b", "kot_sharp"):
        _, _, reqs, want = truth[name]
        eng = make_engine(kot_dirs, name, dtype, 320)
        compare(drive_portions(eng, reqs[1:], portion), want[1:], dtype, f"portions of {portion}", name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_with_reused_slots_blocks_and_states(kot_dirs, truth, name, dtype):
    _, _, reqs, want = truth[name]
    prompt_lens = [max(1, len(r) - DECODE[name]) for r in reqs]
    batch = 3
    order = list(reversed(range(len(reqs))))

    def need_of(rs):
        return max(sum((len(r) + 63) // 64 * 64 for r in rs[b:b + batch]) for b in range(0, len(rs), batch))

    eng = make_engine(kot_dirs, name, dtype, max(need_of(reqs), need_of([reqs[i] for i in order])))
    compare(drive_batches(eng, reqs, batch, prompt_lens), want, dtype, "unequal batches", name)
    assert eng.cache.slots.n_held == 0
    poison_states(eng)           # what the second pass reads it must have written (or zeroed) itself
    got = drive_batches(eng, [reqs[i] for i in order], batch, [prompt_lens[i] for i in order])
    compare(got, [want[i] for i in order], dtype, "unequal batches, reused cache", name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens(kot_dirs, truth, name, dtype):
    cfg, w, _, _ = truth[name]
    reqs = [random_ids(cfg["vocab"], n, 70 + n) for n in (1, 2, 3, 1)]
    want = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    eng = make_engine(kot_dirs, name, dtype, 256)
    compare(drive_whole(eng, reqs), want, dtype, "first tokens, whole", name)
    compare(drive_batches(eng, reqs, 4, [1, 1, 1, 1]), want, dtype, "first tokens, batch", name)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_one_token(kot_dirs, truth, dtype):
    """Every token decoded alone: past every window, over block borders, with blocks behind the windows given back."""
    for name in ("kot_a", "kot_sharp"):
        cfg, w, _, _ = truth[name]
        ids = random_ids(cfg["vocab"], 200, 5)
        want = plain.logits_all_positions(cfg, w, ids)
        eng = make_engine(kot_dirs, name, dtype, 256)
        compare(drive_tail_one_by_one(eng, [ids], tail=len(ids) - 1), [want], dtype, "decoding 200 positions", name)


def test_a_batch_of_seventy_sequences(kot_dirs, truth):
    """More rows in a decode step than the few-row products take."""
    cfg, w, _, _ = truth["kot_odd"]
    reqs = [random_ids(cfg["vocab"], 4 + (i * 7) % 30, 300 + i) for i in range(70)]
    want = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    for dtype in DTYPES:
        eng = make_engine(kot_dirs, "kot_odd", dtype, 70 * 64)
        compare(drive_batches(eng, reqs, 70, [max(1, len(r) - 3) for r in reqs]), want, dtype, "seventy sequences", "kot_odd")


@pytest.mark.parametrize("name", ["kot_a", "kot_sharp"])
def test_greedy_generation_through_the_entry_point(kot_dirs, truth, name):
    """Seven requests over three rows: requests wait, take over rows (and states) of those that ended, and decode in the
    replayed session beside padding rows; every request gets what it gets alone from the plain implementation (32-bit,
    so that no argmax rests on rounding)."""
    from vlrf_b200.api import Model
    from vlrf_b200.sampling.params import SamplingParams
    cfg, w, _, _ = truth[name]
    prompts = [random_ids(cfg["vocab"], n, 900 + n) for n in (3, 20, 1, 66, 9, 33, 5)]
    new = [6, 3, 9, 4, 7, 2, 8]
    model = Model.load(kot_dirs[name], "float32", max_tokens=3 * 128, n_slots=3)
    params = [SamplingParams(max_new_tokens=n, do_sample=False) for n in new]
    results = model.generate_ids(prompts, params)
    want = [plain.greedy_generate(cfg, w, p, n) for p, n in zip(prompts, new)]
    assert [r.new_tokens for r in results] == want
    assert len({t for ts in want for t in ts}) > 10, "the model just repeats itself: the test would show nothing"
    assert model.engine.cache.slots.n_held == 0
    model.engine.cache.check()


def test_trace_replay_of_a_batch_of_unequal_requests(kot_dirs, truth, tmp_path):
    """`bin/trace_run` on a Kotisun folder: nine requests of 1 to 70 tokens start together in one step, go on one token a
    step and end one after another.  32-bit, every wanted position."""
    from test_trace_run import Replay, read
    cfg, w, _, _ = truth["kot_a"]
    V = cfg["vocab"]
    reqs = {f"q{i}": random_ids(V, n, 500 + i) for i, n in enumerate([1, 2, 3, 5, 13, 34, 70, 4, 1])}
    want = {k: plain.logits_all_positions(cfg, w, ids) for k, ids in reqs.items()}
    fed = {k: max(1, len(ids) - 4) for k, ids in reqs.items()}
    rp = Replay(kot_dirs["kot_a"], "float32", tmp_path / "out", sum(len(v) for v in reqs.values()))
    f = rp.send([{"id": k, "tokens": ids[:fed[k]], "want": [fed[k] - 1]} for k, ids in reqs.items()],
                end=[k for k, ids in reqs.items() if fed[k] == len(ids)])
    got = read(f, V)
    for r, k in enumerate(reqs):
        assert float((got[r].double() - want[k][fed[k] - 1]).abs().max() / want[k].abs().max()) < TOL["float32"], (k, "prompt")
    live = [k for k, ids in reqs.items() if fed[k] < len(ids)]
    while live:
        f = rp.send([{"id": k, "tokens": [reqs[k][fed[k]]], "want": [0]} for k in live],
                    end=[k for k in live if fed[k] + 1 == len(reqs[k])])
        got = read(f, V)
        for r, k in enumerate(live):
            assert float((got[r].double() - want[k][fed[k]]).abs().max() / want[k].abs().max()) < TOL["float32"], (k, fed[k])
            fed[k] += 1
        live = [k for k in live if fed[k] < len(reqs[k])]
    rp.close()
