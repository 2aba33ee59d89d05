"""Fasesun on the host: its configuration, the list of blocks and the schedule built from it, and the cache's paged rows."""
import copy

import pytest
import torch

import fasesun_models as fm
import plain_fasesun
from tau_rs_b200.cache import SequenceCache
from tau_rs_b200.config import FasesunConfig, InvalidConfig
from tau_rs_b200.config.metadata import metadata_from_json
from tau_rs_b200.config.registry import architecture_for, spec_from_config_json
from tau_rs_b200.parts import CacheNeed, DecoderModel


def test_the_short_spelling_of_the_architecture_is_read():
    metadata = metadata_from_json(fm.MIXED)
    assert (metadata.architecture, metadata.model_type, metadata.declared_dtype) == ("Fasesun", "fasesun", None)
    assert architecture_for(fm.MIXED).storage_dtype == "bfloat16"


@pytest.mark.parametrize("cfg", [fm.MIXED, fm.ODD, fm.PEAKY, fm.RAGGED])
def test_layer_runs_follow_the_loop(cfg):
    config = FasesunConfig.from_json(cfg)
    assert list(config.layer_runs()) == list(plain_fasesun.layer_runs(cfg))


def test_loop_edges():
    four = [fm.lightning(), fm.mlstm(), fm.lightning(), fm.mlstm()]
    assert FasesunConfig.from_json(fm.config(four, loop=(0, 4, 2))).layer_runs() == (0, 1, 2, 3, 0, 1, 2, 3)
    assert FasesunConfig.from_json(fm.config(four, loop=(2, 2, 5))).layer_runs() == (0, 1, 2, 3)
    assert FasesunConfig.from_json(fm.config(four, loop=(3, 4, 3))).layer_runs() == (0, 1, 2, 3, 3, 3)
    assert FasesunConfig.from_json(fm.config(four, loop=(1, 2, 1))).layer_runs() == (0, 1, 2, 3)


def test_every_run_has_a_cache_layer_of_its_own_and_like_mixers_share_a_group():
    spec = spec_from_config_json(fm.MIXED)
    assert [entry.layer for entry in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    seen = set()
    for entry in spec.schedule:
        assert (entry.cache_group, entry.cache_layer) not in seen
        seen.add((entry.cache_group, entry.cache_layer))
    groups = DecoderModel(spec, torch.float32, "cpu").cache_groups()
    kinds = sorted((need.kind, layers) for need, layers in groups.values())
    assert kinds == [("rows", 1), ("rows", 3), ("state", 1), ("state", 3)]
    assert spec.residual_dtype == "float32" and spec.tie_head


def test_the_model_asks_for_exactly_the_tensors_of_the_design():
    for cfg in (fm.MIXED, fm.ODD):
        wanted = DecoderModel.tensor_specs_of(spec_from_config_json(cfg))
        made = fm.weights(cfg, 0)
        assert set(wanted) == set(made)
        for name, spec in wanted.items():
            assert tuple(spec.shape) == tuple(made[name].shape), name


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="mamba"), "type must be one of"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=32), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c.update(loop={"start": 3, "stop": 2, "times": 2}), "loop"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][2]["mixer"].pop("gate_cap"), "gate_cap"),
])
def test_bad_configurations_are_refused_by_name(change, message):
    cfg = copy.deepcopy(fm.MIXED)
    change(cfg)
    with pytest.raises(InvalidConfig, match=message):
        FasesunConfig.from_json(cfg)


def test_paged_rows_are_taken_given_back_and_taken_again():
    groups = {"latent": (CacheNeed("rows", row_width=24), 2), "memory": (CacheNeed("state", state_shape=(5,)), 3)}
    cache = SequenceCache(groups, max_tokens=64 * 4, max_sequence_tokens=1 << 20, dtype=torch.float32, device="cpu")
    assert cache.kv["latent"].keys.shape == (2, 4, 64, 24) and cache.kv["latent"].values is None
    assert cache.bytes_per_token() == 2 * 24 * 4
    first = cache.open()
    cache.reserve(first, 130)
    cache.advance(first, 130)
    assert len(cache.kv["latent"].held[first]) == 3
    cache.states["memory"].state[:, first] = 7.0
    second = cache.open()
    cache.reserve(second, 64)
    cache.advance(second, 64)
    with pytest.raises(Exception):
        cache.reserve(second, 65)
    cache.check()
    pages = list(cache.kv["latent"].held[first])
    cache.close(first)
    third = cache.open()
    assert third == first and float(cache.states["memory"].state[:, third].abs().sum()) == 0.0
    cache.reserve(third, 100)
    assert set(cache.kv["latent"].held[third]) <= set(pages)
    view = cache.layer_view("latent", 1)
    assert view.rows.shape == (4, 64, 24) and view.group == "latent"
    cache.check()
