"""Bisudra on the host: its configuration, the blocks and schedule built from it, what its cache keeps, and the plain statement
against itself (a window that covers everything, prompts cut in two by hand)."""
import copy

import pytest
import torch

import bisudra_models as bm
import plain_bisudra as plain
from tau_rs_b200.cache import SequenceCache
from tau_rs_b200.config import BisudraConfig, InvalidConfig
from tau_rs_b200.config.metadata import metadata_from_json
from tau_rs_b200.config.registry import architecture_for, spec_from_config_json
from tau_rs_b200.parts import DecoderModel


def test_the_architecture_is_registered_and_stores_bfloat16():
    metadata = metadata_from_json(bm.MIXED)
    assert (metadata.architecture, metadata.model_type, metadata.declared_dtype) == ("Bisudra", "bisudra", None)
    assert architecture_for(bm.MIXED).storage_dtype == "bfloat16"


def test_every_size_and_constant_is_read_from_the_configuration():
    config = BisudraConfig.from_json(bm.MIXED)
    assert (config.vocab, config.width, config.taps, config.side_dim, config.eps) == (211, 96, 3, 10, 1e-5)
    second = config.layers[1]
    assert (second.mixer.heads, second.mixer.kv_heads, second.mixer.dim, second.mixer.vdim, second.mixer.window) == (6, 3, 8, 40, 70)
    assert (second.mixer.diff, second.mixer.rot_dims, second.mixer.rot_base) == (0.6, 8, 5000.0)
    assert (second.mlp.kind, second.mlp.experts, second.mlp.top, second.mlp.expert_ff) == ("moe", 6, 2, 40)
    assert config.layers[0].mlp.kind == "dense" and config.layers[0].mlp.ff == 72 and config.layers[2].mlp is None


def test_blocks_schedule_and_cache_groups():
    spec = spec_from_config_json(bm.MIXED)
    assert spec.residual_dtype == "float32" and spec.tie_head and spec.keeps_results
    assert [block.depth_mix for block in spec.blocks] == [2, 3, 4, 5]
    assert [block.token_side.offset for block in spec.blocks] == [0, 10, 20, 30]
    assert all(block.input_taps == 3 and block.residual_gate for block in spec.blocks)
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].feed_forward_norm is None
    seen = set()
    for index, entry in enumerate(spec.schedule):
        assert (entry.cache_group, entry.cache_layer) not in seen and entry.extra_cache == (("taps", "taps", index),)
        seen.add((entry.cache_group, entry.cache_layer))
    groups = DecoderModel(spec, torch.float32, "cpu").cache_groups()
    assert groups["taps"][0].kind == "state" and groups["taps"][0].state_shape == (2, 96) and groups["taps"][1] == 4
    rows = sorted((need.row_width, need.window, layers) for name, (need, layers) in groups.items() if need.kind == "rows")
    assert rows == sorted([(2 * (2 * 16 + 24), 37, 1), (2 * (2 * 24 + 16), 130, 1), (3 * (2 * 8 + 40), 70, 1)])
    # Where the wider of a key and a value is a multiple of 16, every map is an ordinary head of that width: 2 key/value heads per group.
    assert [(need.n_kv_heads, need.head_dim, need.window, layers) for need, layers in groups.values() if need.kind == "kv"] == [(2, 32, 64, 1)]


def test_one_tap_keeps_no_state():
    spec = spec_from_config_json(bm.ONE_TAP)
    assert all(entry.extra_cache == () for entry in spec.schedule)
    assert all(need.kind in ("rows", "kv") for need, _ in DecoderModel(spec, torch.float32, "cpu").cache_groups().values())


def test_the_model_asks_for_exactly_the_tensors_of_the_design():
    for cfg in (bm.MIXED, bm.ODD, bm.ONE_TAP):
        wanted = DecoderModel.tensor_specs_of(spec_from_config_json(cfg))
        made = bm.weights(cfg, 0)
        assert set(wanted) == set(made)
        for name, spec in wanted.items():
            assert tuple(spec.shape) == tuple(made[name].shape), name


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="mamba"), "type must be one of"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), "'mask'"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c.pop("canon"), "'canon'"),
    (lambda c: c["token_side"].update(dim=0), "'dim'"),
    (lambda c: c.update(width=-3), "'width'"),
])
def test_a_bad_configuration_is_refused_by_name(change, message):
    raw = copy.deepcopy(bm.MIXED)
    change(raw)
    with pytest.raises(InvalidConfig, match=message):
        BisudraConfig.from_json(raw)


def test_a_window_cache_holds_a_few_pages_however_long_the_sequence():
    model = DecoderModel(spec_from_config_json(bm.EDGY), torch.float32, "cpu")
    cache = SequenceCache(model.cache_groups(), 64 * 6, 1 << 20, torch.float32, "cpu")
    slot = cache.open()
    for length in range(1, 900, 7):
        cache.reserve(slot, length)
        cache.advance(slot, length)
        cache.check()
        assert all(len(group.held[slot]) <= 3 for group in cache.kv.values())
    assert cache.states["taps"].state.shape == (2, cache.n_slots, 3, 64)
    cache.close(slot)
    cache.check()


def test_the_plain_statement_against_itself():
    """The window: with one as long as the sequence every position sees everything before it, and the first `window` positions of
    a short window equal those; the convolution: zeros stand before the start."""
    torch.manual_seed(0)
    q, k, v = torch.randn(50, 8, dtype=plain.F), torch.randn(50, 8, dtype=plain.F), torch.randn(50, 5, dtype=plain.F)
    full = plain.windowed_softmax_attention(q, k, v, 0.4, 50)
    short = plain.windowed_softmax_attention(q, k, v, 0.4, 7)
    assert torch.allclose(full[:7], short[:7]) and not torch.allclose(full[7], short[7])
    only_self = plain.windowed_softmax_attention(q, k, v, 0.4, 1)
    assert torch.allclose(only_self, v)
    h, w = torch.randn(9, 4, dtype=plain.F), torch.randn(4, 3, dtype=plain.F)
    taps = plain.causal_taps(h, w)
    assert torch.allclose(taps[0], w[:, 2] * h[0]) and torch.allclose(taps[5], w[:, 0] * h[3] + w[:, 1] * h[4] + w[:, 2] * h[5])
    x = torch.randn(3, 6, 8, dtype=plain.F)
    turned = plain.rotate_pairs(x, 4, 100.0)
    assert torch.allclose(turned[0], x[0]) and torch.allclose(turned[..., 4:], x[..., 4:])
    assert torch.allclose(turned[..., :4].norm(dim=-1), x[..., :4].norm(dim=-1))
