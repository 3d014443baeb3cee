"""The Tekilorn configuration reader, the schedule of looped layers, the checkpoint's tensor
list, and the cache manager's bookkeeping for windows that keep their first tokens (no GPU)."""

from __future__ import annotations

import copy

import pytest

import plain_tekilorn as pt
from forge_engine_b200.cache.manager import CacheManager, CacheNeeds, PagedKVSpec
from forge_engine_b200.config import read_model_config
from forge_engine_b200.errors import ConfigError


def example():
    return pt.config([pt.differential_layer(), pt.window_layer(mlp=pt.routed()), pt.window_layer(mlp=None, window=None),
                      pt.differential_layer(softcap=None, q_temp=None)], loop=(1, 3, 3))


def test_registry_finds_the_architecture_and_reads_every_constant():
    arch, cfg, spec = read_model_config(example())
    assert arch.name == "Tekilorn" and spec.vocab_size == 97 and spec.hidden_size == 64
    first, second, third, fourth = (layer.mixer for layer in spec.layers)
    assert first.differential.offset == 0.25 and first.softcap == 20.0 and first.query_temperature == (0.4, 8)
    assert first.window is None and first.position.kind == "none" and not first.head_gate
    assert second.window == 9 and second.keep_first == 3 and second.head_gate and second.differential is None
    assert second.position.interleaved and second.position.rotary_dim == 8 and second.position.theta == 100.0
    assert third.window is None and third.keep_first == 0
    assert fourth.softcap is None and fourth.query_temperature is None
    routed = spec.layers[1].ffn
    assert (routed.experts, routed.top, routed.score, routed.weight_on, routed.renormalise) == (5, 2, "sigmoid", "input", False)
    assert routed.expert.limit == 1.25 and routed.shared.limit == 2.0 and routed.shared_gate
    assert spec.layers[2].ffn is None and spec.layers[2].post_norm is None
    assert spec.layers[0].ffn.activation == "clamped_swish" and spec.layers[0].ffn.slope == 1.702


def test_looped_layers_become_runs_with_caches_of_their_own():
    _, cfg, spec = read_model_config(example())
    assert [run.layer for run in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [run.shift for run in spec.schedule] == [None, ("loop.step", 0), None, ("loop.step", 1), None,
                                                    ("loop.step", 2), None, None]
    assert all(run.cache_of is None for run in spec.schedule)
    raw = example()
    del raw["loop"]
    _, _, plain_spec = read_model_config(raw)
    assert [run.layer for run in plain_spec.schedule] == [0, 1, 2, 3] and not plain_spec.extra_tensors
    assert [(layer, t) for layer, t in cfg.runs()] == pt.layer_order(example())


def test_expected_tensors_are_the_checkpoints():
    for raw in (example(), pt.config([pt.window_layer(mlp=pt.routed(shared_ff=None))])):
        arch, _, spec = read_model_config(raw)
        expected = arch.expected_tensors(spec)
        shapes = pt.tensor_shapes(raw)
        assert set(expected) == set(shapes)
        assert all(tuple(expected[name].shape) == tuple(shapes[name]) for name in shapes)


@pytest.mark.parametrize("path, value", (
    (("layers", 0, "type"), "attention_3"),
    (("layers", 0, "mixer", "heads"), 3),
    (("layers", 0, "mixer", "softcap"), 0.0),
    (("layers", 1, "mixer", "rot", "dims"), 7),
    (("layers", 1, "mixer", "rot", "dims"), 18),
    (("layers", 1, "mlp", "router", "top"), 6),
    (("layers", 1, "mlp", "kind"), "sparse"),
    (("layers", 0, "mlp", "limit"), -1.0),
    (("loop", "stop"), 9),
    (("loop", "times"), 0),
    (("norm", "eps"), 0.0),
))
def test_bad_values_are_refused(path, value):
    raw = copy.deepcopy(example())
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        read_model_config(raw)


def test_pages_of_kept_first_tokens_are_never_given_back():
    spec = PagedKVSpec(2, 16, window=6, v_head_dim=None, keep_first=5)
    plain = PagedKVSpec(2, 16, window=6)
    cache = CacheManager([CacheNeeds(kv=spec), CacheNeeds(kv=plain)], page_size=4, num_pages=40, max_requests=2)
    assert spec.kept_pages(4) == 2 and plain.kept_pages(4) == 0 and PagedKVSpec(1, 8, None, None, 9).kept_pages(4) == 0
    cache.begin_request("a")
    length = 0
    for count in (3, 9, 1, 1, 20, 1, 7):
        cache.reserve("a", length + count)
        length += count
        cache.advance("a", length)
        cache.check_consistency()
        kept, windowed = cache.request("a").tables
        first_needed = max(0, length - 6 + 1) // 4
        assert all(page >= 0 for page in kept.pages[:2])                       # positions 0..4 stay
        assert all(page < 0 for page in kept.pages[2:first_needed])
        assert all(page >= 0 for page in kept.pages[max(2, first_needed):])
        assert all(page < 0 for page in windowed.pages[:first_needed])
        assert len(kept.live_pages()) == len(windowed.live_pages()) + min(2, first_needed)
    assert cache.worst_case_pages(100, 8)[0] == cache.worst_case_pages(100, 8)[1] + 2
    cache.end_request("a")
    assert cache.leased_pages() == [0, 0]
