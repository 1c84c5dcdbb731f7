"""Kuvusun without a GPU: its configuration, its tensor list, its registry entry and the cache's rows of latents."""
import copy

import pytest
import torch

import plain_kuvusun as plain
from kuvusun_models import KUV_A, KUV_B, MODELS, write_model


def test_config_json_selects_the_architecture_and_reads_every_layer():
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.registry import parse_config
    arch, cfg = parse_config(KUV_A)
    assert arch.name == "Kuvusun" and cfg.n_layer == 4
    assert [m.kv_from for m in cfg.mixers] == [None, None, 0, None]
    assert cfg.mixers[1].q_rank == 72 and cfg.mixers[1].rot_dim == 0 and not cfg.mixers[1].gated
    assert cfg.mixers[0].rot_dim == 8 and cfg.mixers[0].gated and cfg.mixers[3].rot_base == 500.0
    assert cfg.mlps[2] is None and cfg.mlps[1].kind == "dense" and cfg.mlps[0].shared_ff == 80 and cfg.mlps[3].shared_ff is None
    assert cfg.to_dict() == KUV_A


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "differ"),            # layer 1 keeps rows of another width
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_configurations_that_describe_no_model_are_refused(edit, text):
    from vlrf_b200.config.base import ConfigError
    from vlrf_b200.registry import parse_config
    cfg = copy.deepcopy(KUV_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        parse_config(cfg)


def test_tensor_list_follows_the_layers(tmp_path):
    from vlrf_b200.registry import parse_config
    from vlrf_b200.weights.model_dir import open_model_dir
    arch, cfg = parse_config(KUV_A)
    names = {s.name: s for s in arch.weight_spec(cfg)}
    assert "l2.mix.dkv" not in names and "l0.mix.dkv" in names and tuple(names["l0.mix.dkv"].shape) == (48, 96)
    assert "l1.mix.g" not in names and "l0.mix.g" in names and "l1.mix.dq.norm" in names and "l0.mix.q" in names
    assert "l3.mlp.shared.sg" not in names and tuple(names["l0.mlp.shared.sg"].shape) == (1, 96)
    assert "l2.mlp.up" not in names and names["l2.norm2"].optional and "l3.mlp.e3.down" in names and "l3.mlp.e4.down" not in names
    write_model(KUV_A, 3, tmp_path)
    arch2, cfg2, checked = open_model_dir(tmp_path)
    assert arch2.name == "Kuvusun" and set(checked.tensors) == set(names)


def test_a_checkpoint_that_lacks_or_adds_tensors_is_refused_in_one_error(tmp_path):
    from vlrf_b200.weights import WeightError, read_safetensors, write_safetensors
    from vlrf_b200.weights.model_dir import open_model_dir
    write_model(KUV_B, 4, tmp_path)
    t = dict(read_safetensors(tmp_path / "model.safetensors"))
    del t["l3.mlp.router.b"]
    t["l3.mix.dkv"] = torch.zeros(96, 128, dtype=torch.bfloat16)       # layer 3 reads layer 2's cache: it has none
    write_safetensors(tmp_path / "model.safetensors", t)
    with pytest.raises(WeightError) as e:
        open_model_dir(tmp_path)
    assert "l3.mlp.router.b" in str(e.value) and "l3.mix.dkv" in str(e.value)


def test_cache_rows_of_latents_are_paged_like_keys_and_values():
    from vlrf_b200.cache import KVNeed, LatentNeed, SequenceCache
    needs = [LatentNeed(48), KVNeed(2, 16), None, LatentNeed(48), LatentNeed(40)]
    c = SequenceCache(needs, max_tokens=256, max_seq_len=512, dtype=torch.float32, device="cpu")
    v0, v3, v4, v1 = c.view(0), c.view(3), c.view(4), c.view(1)
    assert tuple(v0.rows.shape) == (4, 64, 48) and tuple(v4.rows.shape) == (4, 64, 40) and v0.k is None and v1.rows is None
    assert v0.rows.data_ptr() != v3.rows.data_ptr() and v0.block_table is v3.block_table
    a, b = c.acquire(), c.acquire()
    c.reserve(a, 130); c.advance(a, 130); c.reserve(b, 64); c.advance(b, 64)
    c.check()
    assert c.live_kv_bytes([a, b]) == (130 + 64) * (4 * (48 + 48 + 40) + 2 * 2 * 16 * 4)
    with pytest.raises(Exception):
        c.reserve(b, 129)              # three blocks of four are held by a, one by b
    c.release(a)
    c.reserve(b, 129); c.advance(b, 65)
    c.check()
    c.release(b)
    c.check()


def test_plain_router_prefers_the_lower_index_on_ties():
    idx, w = plain.route(torch.tensor([[1.0, 3.0, 3.0, 0.5, 3.0]], dtype=torch.float64), 2)
    assert idx.tolist() == [[1, 2]] and torch.allclose(w, torch.tensor([[0.5, 0.5]], dtype=torch.float64))


def test_plain_rotation_is_a_rotation_by_position():
    v = torch.randn(5, 3, 12, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    r = plain.rotate(v, pos, 10000.0, 8)
    assert torch.equal(r[0], v[0]) and torch.equal(r[..., 8:], v[..., 8:])
    assert torch.allclose((r[..., :8] ** 2).sum(-1), (v[..., :8] ** 2).sum(-1))
    # entry 0 pairs with entry 4 at frequency 1: position 1 turns the pair by one radian
    assert torch.allclose(r[1, :, 0], v[1, :, 0] * torch.cos(torch.tensor(1.0)) - v[1, :, 4] * torch.sin(torch.tensor(1.0)))


def test_every_test_model_has_a_registered_architecture():
    from vlrf_b200.registry import parse_config
    for cfg in MODELS.values():
        parse_config(cfg)
