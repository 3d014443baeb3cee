"""Configuration, tensor list and cache bookkeeping of the Zofadra design (no GPU needed)."""

from __future__ import annotations

import copy

import pytest

import plain_zofadra as pz
from forge_engine_b200.cache import CacheManager, CacheNeeds, PagedKVSpec, StateSpec
from forge_engine_b200.config import read_model_config
from forge_engine_b200.config.specs import join_name, local_name
from forge_engine_b200.errors import ConfigError

LAYERS = [pz.latent_layer(), pz.attention_layer(window=6, dim=16, vdim=24), pz.lightning_layer(),
          pz.latent_layer(kv_from=0, ff=None)]


def test_registry_reads_the_architecture_and_lists_every_tensor():
    cfg = pz.config(LAYERS, streams=3)
    arch, typed, spec = read_model_config(cfg)
    assert arch.name == "Zofadra" and typed.streams == 3
    assert spec.residual_streams == 3 and spec.embedding_scale == 2.0
    assert [run.cache_of for run in spec.schedule] == [None, None, None, 0]
    expected = arch.expected_tensors(spec)
    assert {name: tuple(info.shape) for name, info in expected.items()} == pz.tensor_shapes(cfg)


def test_optional_keys_have_defaults_and_no_streams_means_no_mixing_tensors():
    cfg = pz.config(LAYERS, streams=None, residual_mult=None, scale=None)
    arch, typed, spec = read_model_config(cfg)
    assert typed.streams is None and typed.residual_mult == 1.0 and typed.embedding_scale == 1.0
    assert spec.residual_streams == 1
    assert not [name for name in arch.expected_tensors(spec) if ".hc" in name]
    assert set(arch.expected_tensors(spec)) == set(pz.tensor_shapes(cfg))


@pytest.mark.parametrize("damage, message", [
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "no latent"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=8), "kv_rank"),
    (lambda c: c["layers"][0].update(type="mamba"), "known"),
    (lambda c: c["layers"][2]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "even"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "dense"),
])
def test_configuration_errors_name_the_key(damage, message):
    cfg = copy.deepcopy(pz.config(LAYERS))
    damage(cfg)
    with pytest.raises(ConfigError, match=message):
        read_model_config(cfg)


def test_names_with_an_empty_local_part():
    class Spec:
        rename = (("weight", ""),)

    assert local_name(Spec, "weight") == "" and local_name(Spec, "bias") == "bias"
    assert join_name("l0.norm1", "") == "l0.norm1" and join_name("l0.mix", "q") == "l0.mix.q"


def test_cache_groups_for_latents_values_of_another_size_and_states():
    needs = [
        CacheNeeds(kv=PagedKVSpec(1, 40, None, 0)),                # a latent: one vector per token
        CacheNeeds(kv=PagedKVSpec(2, 16, 6, 24)),                  # windowed, values wider than keys
        CacheNeeds(state=StateSpec((2, 16, 8))),
        CacheNeeds(kv=PagedKVSpec(1, 40, None, 0)),                # reads run 0's
        CacheNeeds(kv=PagedKVSpec(2, 16, 6, 24)),                  # same geometry as run 1: same group
    ]
    import torch

    cache = CacheManager(needs, page_size=4, num_pages=10, max_requests=2, dtype=torch.float32, device="cpu",
                         shares={3: 0})
    assert len(cache.groups) == 2 and cache.groups[1].units == [1, 4]
    latent, nothing = cache.kv_of_run(0)
    assert nothing is None and latent.shape == (11, 1, 4, 40)
    assert cache.view(3).owns is False and cache.view(3).kv[0].data_ptr() == latent.data_ptr()
    keys1, values1 = cache.kv_of_run(1)
    keys4, values4 = cache.kv_of_run(4)
    assert keys1.shape == (11, 2, 4, 16) and values1.shape == (11, 2, 4, 24)
    spans = sorted((t.data_ptr(), t.data_ptr() + t.numel() * 4) for t in (keys1, values1, keys4, values4))
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))     # the four planes do not overlap
    assert cache.bytes_per_token() == 4 * (40 + 2 * 2 * (16 + 24))
    assert cache.state_of_run(2).shape == (3, 2, 16, 8)


def test_window_pages_are_released_and_slots_reused():
    needs = [CacheNeeds(kv=PagedKVSpec(1, 8, None, 0)), CacheNeeds(kv=PagedKVSpec(1, 8, 6)),
             CacheNeeds(state=StateSpec((2,)))]
    cache = CacheManager(needs, page_size=4, num_pages=8, max_requests=2)
    first = cache.begin_request("a")
    cache.reserve("a", 30)
    cache.advance("a", 30)
    assert cache.leased_pages()[0] == 8 and cache.leased_pages()[1] == 2    # the window holds pages 6 and 7 only
    cache.end_request("a")
    second = cache.begin_request("b")
    assert second.slot == first.slot and cache.leased_pages() == [0, 0]
    cache.check_consistency()
