"""Kotisun without a GPU: its configuration, its tensor list, its layer schedule, the cache's tuple needs, and the plain
implementation's own mechanisms."""
import copy

import pytest
import torch

import plain_kotisun as plain
from kotisun_models import KOT_A, KOT_B, KOT_PLAIN, KOT_SHARP, MODELS, SHARP_FACTOR, write_model


def test_config_json_selects_the_architecture_and_reads_every_layer():
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.registry import parse_config
    arch, cfg = parse_config(KOT_A)
    assert arch.name == "Kotisun" and cfg.n_layer == 4 and cfg.streams == 3 and cfg.embedding_scale == 2.0
    assert cfg.layer_order == [0, 1, 2, 1, 2, 3] == plain.schedule(KOT_A)
    a = [lc.left for lc in cfg.layer_configs]
    assert [x.window for x in a] == [40, 70, 0, 130] and [x.rot_dims for x in a] == [8, 32, 0, 12]
    assert a[0].rot_factor == 2.0 and a[1].rot_factor == 1.0 and a[3].rot_base == 30000.0
    assert [lc.ff for lc in cfg.layer_configs] == [96, None, 72, 40]
    assert cfg.layer_configs[2].right.groups == 3 and cfg.layer_configs[1].right.conv == 2
    assert cfg.to_dict() == KOT_A
    _, b = parse_config(KOT_B)
    assert b.embedding_scale == 1.0 and b.logit_softcap is None and b.layer_order == [0, 1, 2] and b.streams == 1
    _, c = parse_config(KOT_PLAIN)
    assert c.streams is None and c.layer_order == [0, 1, 0, 1, 0, 1]


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "rot"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), "mask"),
    (lambda c: c["layers"][0].update(type="serial"), "type"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(groups=3), "groups"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_configurations_that_describe_no_model_are_refused(edit, text):
    from vlrf_b200.config.base import ConfigError
    from vlrf_b200.registry import parse_config
    cfg = copy.deepcopy(KOT_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        parse_config(cfg)


def test_tensor_list_follows_the_layers(tmp_path):
    from vlrf_b200.registry import parse_config
    from vlrf_b200.weights.model_dir import open_model_dir
    arch, cfg = parse_config(KOT_A)
    names = {s.name: s for s in arch.weight_spec(cfg)}
    assert tuple(names["l0.mix.left.q"].shape) == (64, 64) and tuple(names["l0.mix.left.k"].shape) == (32, 64)
    assert tuple(names["l0.mix.left.v.b"].shape) == (48,) and tuple(names["l0.mix.left.o"].shape) == (64, 96)
    assert tuple(names["l0.mix.right.in"].shape) == (2 * 32 + 2 * 2 * 16 + 4, 64) and tuple(names["l0.mix.right.conv"].shape) == (96, 4)
    assert tuple(names["l2.mix.right.norm"].shape) == (48,) and tuple(names["l0.hc1.mix"].shape) == (3, 3)
    assert "l1.mlp.up" not in names and names["l1.norm2"].optional and "head" in names and "final.norm" in names
    write_model(KOT_A, 3, tmp_path)
    arch2, _, checked = open_model_dir(tmp_path)
    assert arch2.name == "Kotisun" and set(checked.tensors) == {n for n, s in names.items() if not s.optional}
    arch3, cfg3 = parse_config(KOT_PLAIN)
    assert not any(".hc" in s.name for s in arch3.weight_spec(cfg3))


def test_a_checkpoint_that_lacks_or_adds_tensors_is_refused_in_one_error(tmp_path):
    from vlrf_b200.weights import WeightError, read_safetensors, write_safetensors
    from vlrf_b200.weights.model_dir import open_model_dir
    write_model(KOT_B, 4, tmp_path)
    t = dict(read_safetensors(tmp_path / "model.safetensors"))
    del t["l1.mix.right.dt_bias"]
    t["l2.mlp.gate"] = torch.zeros(8, 96, dtype=torch.bfloat16)       # layer 2 has no feed-forward
    write_safetensors(tmp_path / "model.safetensors", t)
    with pytest.raises(WeightError) as e:
        open_model_dir(tmp_path)
    assert "l1.mix.right.dt_bias" in str(e.value) and "l2.mlp.gate" in str(e.value)


def test_a_mixer_that_keeps_two_things_gets_a_view_of_each():
    from vlrf_b200.cache import KVNeed, SequenceCache, StateNeed
    both = (KVNeed(2, 16, "window", 70, v_dim=24), StateNeed((2, 50), torch.float32))
    other = (KVNeed(1, 8, "full", 0, v_dim=12), StateNeed((2, 50), torch.float32))
    c = SequenceCache([both, None, other, both], max_tokens=256, max_seq_len=512, dtype=torch.float32, device="cpu")
    v0, v2, v3 = c.view(0), c.view(2), c.view(3)
    assert len(v0.parts) == 2 and tuple(v0.parts[0].k.shape) == (4, 2, 64, 16) and tuple(v0.parts[0].v.shape) == (4, 2, 64, 24)
    assert tuple(v2.parts[0].v.shape) == (4, 1, 64, 12) and tuple(v0.parts[1].state.shape) == (4, 2, 50)
    assert v0.parts[0].k.data_ptr() != v3.parts[0].k.data_ptr() and v0.parts[1].state.data_ptr() != v2.parts[1].state.data_ptr()
    assert len(c._groups) == 3                                   # two key/value groups, and one for the three states
    a = c.acquire()
    v0.parts[1].state[a].fill_(7.0)
    c.reserve(a, 200); c.advance(a, 200)
    c.check()
    assert sum(int(b >= 0) for b in c._where[(0, 0)][0].table_host[a]) == 2     # the window let the first blocks go
    c.release(a)
    assert c.acquire() == a and float(v0.parts[1].state[a].abs().max()) == 0.0  # a slot that is used again starts at zero
    c.check()


def test_plain_window_attention_sees_exactly_the_window():
    T, w = 12, 4
    q = torch.zeros(T, 1, 2, dtype=torch.float64); q[:, 0, 0] = 50.0
    k = torch.zeros(T, 1, 2, dtype=torch.float64); k[3, 0, 0] = 1.0        # key 3 stands out
    v = torch.arange(T, dtype=torch.float64).reshape(T, 1, 1)
    out = plain.window_attention(q, k, v, 1.0, w)[:, 0, 0]
    assert abs(float(out[6]) - 3.0) < 1e-9 and abs(float(out[3]) - 3.0) < 1e-9    # 6 − 3 < 4: seen
    assert abs(float(out[7]) - 5.5) < 1e-9                                        # 7 − 3 = 4: not seen (mean of 4 … 7)
    full = plain.window_attention(q, k, v, 1.0, None)[:, 0, 0]
    assert abs(float(full[11]) - 3.0) < 1e-9


def test_plain_scan_carries_its_state_and_the_convolution_its_inputs():
    g = torch.Generator().manual_seed(0)
    T, Hs, P, G, N = 9, 4, 3, 2, 5
    x, B, C = (torch.randn(s, generator=g, dtype=torch.float64) for s in ((T, Hs, P), (T, G, N), (T, G, N)))
    dt = torch.rand(T, Hs, generator=g, dtype=torch.float64)
    a_log, D = torch.randn(Hs, generator=g, dtype=torch.float64), torch.randn(Hs, generator=g, dtype=torch.float64)
    y = plain.selective_scan(x, B, C, dt, a_log, D)
    # written out for one head and the last token: Σ_j exp(−e^a Σ_{j<i≤t} dt_i) dt_j (C_t · B_j) x_j + D x_t
    h, t, grp = 3, T - 1, 1
    want = D[h] * x[t, h]
    for j in range(T):
        decay = torch.exp(-torch.exp(a_log[h]) * dt[j + 1:t + 1, h].sum())
        want = want + decay * dt[j, h] * (C[t, grp] @ B[j, grp]) * x[j, h]
    assert torch.allclose(y[t, h], want)
    u = torch.randn(7, 3, generator=g, dtype=torch.float64)
    w, b = torch.randn(3, 4, generator=g, dtype=torch.float64), torch.randn(3, generator=g, dtype=torch.float64)
    out = plain.causal_conv(u, w, b)
    assert torch.allclose(out[0], u[0] * w[:, 3] + b) and torch.allclose(out[2], u[0] * w[:, 1] + u[1] * w[:, 2] + u[2] * w[:, 3] + b)


def test_plain_rotation_is_a_slowed_rotation_by_position():
    v = torch.randn(4, 2, 10, dtype=torch.float64)
    pos = torch.tensor([0, 1, 8, 1000])
    r = plain.rotate_scaled(v, pos, 10000.0, 6, 4.0)
    assert torch.equal(r[0], v[0]) and torch.equal(r[..., 6:], v[..., 6:])
    assert torch.allclose((r[..., :6] ** 2).sum(-1), (v[..., :6] ** 2).sum(-1))
    c, s = torch.cos(torch.tensor(2.0, dtype=torch.float64)), torch.sin(torch.tensor(2.0, dtype=torch.float64))
    assert torch.allclose(r[2, :, 0], v[2, :, 0] * c - v[2, :, 3] * s)      # position 8 at a quarter of the speed: 2 radians


def test_every_test_model_has_a_registered_architecture():
    from vlrf_b200.registry import parse_config
    for cfg in MODELS.values():
        parse_config(cfg)


def test_the_sharp_model_depends_on_its_window_and_on_far_tokens(tmp_path):
    """Windows one token narrower, and another token far outside every window (which only the recurrence's state can
    carry), move the last logits by fifty and by ten times the 32-bit comparisons' bound or more: the engine tests on this
    model would show a window's edge one token off, or a lost state."""
    from conftest import random_ids
    write_model(KOT_SHARP, 64, tmp_path, sharp=SHARP_FACTOR)
    cfg, w = plain.read_model_dir(tmp_path)
    ids = random_ids(cfg["vocab"], 220, 24)
    want = plain.logits_all_positions(cfg, w, ids)
    narrowed = copy.deepcopy(cfg)
    for layer in narrowed["layers"]:
        layer["mixer"]["left"]["mask"]["size"] -= 1
    moved = plain.logits_all_positions(narrowed, w, ids)[-1]
    assert float((moved - want[-1]).abs().max() / want.abs().max()) > 5e-3
    far = list(ids)
    far[5] = (far[5] + 1) % cfg["vocab"]
    moved = plain.logits_all_positions(cfg, w, far)[-1]
    assert float((moved - want[-1]).abs().max() / want.abs().max()) > 1e-3
