"""Legelix on the host: reading config.json, the model spec it turns into, the tensors it declares, the
frequency table of its rotation, and the cache manager's handling of chunked attention."""

import copy
import json

import pytest
import torch

from legelix_models import CONFIGS, DECAY_RANK, make_weights
from plain_legelix import plain_rotary_frequencies


def test_the_registry_finds_the_design_by_its_own_key():
    from zephyr_b200.config import LegelixConfig, resolve_architecture

    assert resolve_architecture(CONFIGS["P"]).config_class is LegelixConfig
    config = LegelixConfig.from_dict(CONFIGS["Q"])
    assert LegelixConfig.from_dict(config.to_dict()) == config
    assert json.loads(json.dumps(config.to_dict())) == CONFIGS["Q"]


@pytest.mark.parametrize("name", list(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    from zephyr_b200.config import LegelixConfig
    from zephyr_b200.parts import expected_weights
    from zephyr_b200.weights.loader import shape_fits

    config = CONFIGS[name]
    weights = make_weights(config, DECAY_RANK[name], seed=1)
    declared = expected_weights(LegelixConfig.from_dict(config).to_model_spec())
    assert set(declared) == set(weights)
    for tensor_name, decl in declared.items():
        assert shape_fits(tuple(weights[tensor_name].shape), decl.shape), tensor_name
    # the one size no key gives: any inner size of the decay projection fits, and random weights need it named
    open_sizes = [n for n, d in declared.items() if -1 in d.shape]
    assert all(n.endswith((".a1", ".a2")) for n in open_sizes) and open_sizes
    named = expected_weights(LegelixConfig(**{**LegelixConfig.from_dict(config).__dict__, "decay_rank": 6}).to_model_spec())
    assert all(-1 not in d.shape for d in named.values())


def test_stores_of_every_layer():
    from zephyr_b200.cache import PagedCacheSpec, StateCacheSpec
    from zephyr_b200.config import LegelixConfig
    from zephyr_b200.parts import cache_specs

    spec = LegelixConfig.from_dict(CONFIGS["Q"]).to_model_spec()
    stores = cache_specs(spec)
    # parallel (pages + state), gla (state), parallel (pages + state)
    assert [type(s) for s in stores] == [PagedCacheSpec, StateCacheSpec, StateCacheSpec, PagedCacheSpec, StateCacheSpec]
    assert stores[0] == PagedCacheSpec(3, key_dim=24, value_dim=40, window=0, chunk=10)
    assert stores[1].shape == (3 * 24 * 40 + 3 * (3 * 40 + 2 * 3 * 24),)       # state, and three inputs of every channel
    assert stores[2].shape == (3 * 80 * 40,)
    assert spec.run_order[0].caches == (0, 1) and spec.run_order[1].caches == (2,) and spec.run_order[2].caches == (3, 4)
    assert spec.layers[0].feed_forward is not None and spec.input.params["float32_stream"]


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=15), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(tau=0), "tau"),
    (lambda c: c.update(vocab=0), "vocab"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "dense"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(change, message):
    from zephyr_b200.config import ConfigError, LegelixConfig

    config = copy.deepcopy(CONFIGS["P"])
    change(config)
    with pytest.raises(ConfigError, match=message):
        LegelixConfig.from_dict(config)


@pytest.mark.parametrize("rot", [{"base": 10000.0, "dims": 16}, {"base": 500.0, "dims": 24, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
                                 {"base": 50.0, "dims": 64, "scaling": {"factor": 3.0, "low": 2.0, "high": 16.0, "original": 512}}])
def test_rotation_frequencies(rot):
    from zephyr_b200.config import PositionSpec
    from zephyr_b200.parts import RopePairs

    part = RopePairs(PositionSpec("rope_pairs", head_dim=64, max_positions=128, params=rot), torch.float32, "cpu")
    freqs, dims = part.as_pair_frequencies()
    expected = plain_rotary_frequencies(rot)
    assert dims == rot["dims"] and freqs.dtype == torch.float32
    assert torch.allclose(freqs.double(), expected, rtol=1e-7, atol=0)
    if "scaling" in rot:      # all three regimes occur: kept, blended, divided
        plain = plain_rotary_frequencies({"base": rot["base"], "dims": rot["dims"]})
        ratio = (expected / plain).tolist()
        factor = rot["scaling"]["factor"]
        assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / factor) < 1e-12 and any(1 / factor < r < 1.0 for r in ratio)


def test_chunked_groups_give_pages_back_at_chunk_edges():
    from zephyr_b200.cache import CacheManager, PagedCacheSpec, StateCacheSpec

    manager = CacheManager([PagedCacheSpec(2, 8, 4, chunk=24), StateCacheSpec((5,)), PagedCacheSpec(2, 8, 4)], page_size=8,
                           num_pages=12, max_requests=2)
    assert len(manager.groups) == 2 and manager.groups[0].chunk == 24
    assert manager.add_request("a")
    for computed in range(1, 80):
        assert manager.ensure_capacity("a", computed)
        manager.commit("a", computed)
        manager.check_invariants()
        chunked, full = manager.block_table("a", 0), manager.block_table("a", 1)
        start = computed // 24 * 24                   # the first position a later query may read
        for block, page in enumerate(chunked):
            assert (page == 0) == ((block + 1) * 8 <= start), (computed, block)
        assert all(page != 0 for page in full)
    # 79 positions: the chunk from 72 on lives in one page; the full group holds ten
    assert manager.num_free_pages(0) == 11 - 1 and manager.num_free_pages(1) == 11 - 10
    manager.free_request("a")
    manager.check_invariants()
    assert manager.num_free_pages(0) == manager.num_free_pages(1) == 11


def test_random_model_from_the_command_line(tmp_path):
    """``random-model`` writes a Legelix folder whose decay projection has the inner size asked for, and
    the folder reads back as the same configuration with every declared tensor present."""
    from zephyr_b200.cli import main
    from zephyr_b200.config import load_model_config
    from zephyr_b200.parts import expected_weights
    from zephyr_b200.weights import Checkpoint
    from zephyr_b200.weights.loader import check_store

    source = tmp_path / "config.json"
    source.write_text(json.dumps(CONFIGS["P"]))
    assert main(["random-model", "--config", str(source), "--out", str(tmp_path / "model"), "--decay-rank", "6", "--seed", "3"]) == 0
    config = load_model_config(tmp_path / "model")
    assert config.to_dict() == CONFIGS["P"]
    store = Checkpoint(tmp_path / "model")
    check_store(store, expected_weights(config.to_model_spec()))
    assert tuple(store.shape("l0.mix.a1")) == (6, 64) and tuple(store.shape("l0.mix.a2")) == (32, 6)
