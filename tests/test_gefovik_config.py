"""Gefovik on the host: reading config.json, the model spec it turns into, the tensors it declares, the
stores of its layers (a latent layer keeps keys only), the plain routing rule, and ``random-model``."""

import copy
import json

import pytest
import torch

from gefovik_models import CONFIGS, make_weights
from plain_gefovik import F64, query_temperature, routing


def test_the_registry_finds_the_design_by_its_own_key():
    from zephyr_b200.config import GefovikConfig, resolve_architecture

    assert resolve_architecture(CONFIGS["A"]).config_class is GefovikConfig
    config = GefovikConfig.from_dict(CONFIGS["B"])
    assert GefovikConfig.from_dict(config.to_dict()) == config
    assert json.loads(json.dumps(config.to_dict())) == CONFIGS["B"]


@pytest.mark.parametrize("name", list(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    from zephyr_b200.config import GefovikConfig
    from zephyr_b200.parts import expected_weights

    weights = make_weights(CONFIGS[name], seed=1)
    declared = expected_weights(GefovikConfig.from_dict(CONFIGS[name]).to_model_spec())
    assert set(declared) == set(weights)
    for tensor_name, decl in declared.items():
        assert tuple(weights[tensor_name].shape) == decl.shape, tensor_name


def test_the_spec_names_every_mechanism_with_its_constants():
    from zephyr_b200.cache import PagedCacheSpec
    from zephyr_b200.config import GefovikConfig
    from zephyr_b200.parts import cache_specs

    spec = GefovikConfig.from_dict(CONFIGS["A"]).to_model_spec()
    stores = cache_specs(spec)
    # a latent layer keeps one "head" of its latent's width and nothing for the values
    assert stores[0] == PagedCacheSpec(1, key_dim=48, keys_only=True) and stores[0].stored_per_position == 48
    assert stores[1] == PagedCacheSpec(2, key_dim=32) and stores[1].stored_per_position == 2 * 64
    assert stores[3] == PagedCacheSpec(1, key_dim=16)
    assert spec.input.params["scale"] == 0.7 and spec.input.params["float32_stream"]
    assert spec.output.params["weight"] == "embed"                              # the head is the table itself
    assert [layer.block for layer in spec.layers] == ["outnorm_residual"] * 4
    assert all(norm.bias is None for layer in spec.layers for norm in layer.norms.values())
    attention = spec.layers[1].mixer.params
    assert attention["values_from_keys"] and attention["unit_qk_norm"] and attention["softcap"] == 4.0
    assert attention["q_temp"] == {"coef": 0.25, "every": 16} and "v_proj" not in attention
    routed = spec.layers[1].feed_forward
    assert routed.kind == "routed" and (routed.params["experts"], routed.params["identity"], routed.params["top"]) == (5, 2, 3)
    assert spec.layers[0].feed_forward.params["activation"] == "relu" and routed.params["activation"] == "silu"
    assert spec.layers[2].feed_forward is None and set(spec.layers[2].norms) == {"mixer_out"}
    # no bound and no multiplier where the configuration gives none
    plain = GefovikConfig.from_dict(CONFIGS["B"]).to_model_spec().layers[0].mixer.params
    assert plain["softcap"] == 0.0 and plain["q_temp"] is None


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=48), "vdim must equal dim"),
    (lambda c: c["layers"][1]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=8), "router.top"),
    (lambda c: c["layers"][0].update(mlp={"kind": "conv", "ff": 8}), "dense or a moe"),
    (lambda c: c.update(vocab=0), "vocab"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(change, message):
    from zephyr_b200.config import ConfigError, GefovikConfig

    config = copy.deepcopy(CONFIGS["A"])
    change(config)
    with pytest.raises(ConfigError, match=message):
        GefovikConfig.from_dict(config)


def test_keys_only_pages_are_half_as_large():
    from zephyr_b200.cache import PagedCacheSpec
    from zephyr_b200.cache.storage import paged_cache_bytes_per_page

    both = paged_cache_bytes_per_page(PagedCacheSpec(1, key_dim=48), 16, torch.bfloat16)
    keys = paged_cache_bytes_per_page(PagedCacheSpec(1, key_dim=48, keys_only=True), 16, torch.bfloat16)
    assert both == 2 * keys == 2 * 16 * 48 * 2
    assert PagedCacheSpec(1, key_dim=48).group_key != PagedCacheSpec(1, key_dim=48, keys_only=True).group_key


def test_the_plain_routing_rule():
    """The correction moves the choice and not the weight; ties go to the lower index; weights are the
    softmax scores over ALL outputs, not renormalised."""
    z = torch.tensor([[2.0, 1.0, 0.0, -1.0], [0.0, 0.0, 0.0, 0.0]], dtype=F64)
    none = torch.zeros(4, dtype=F64)
    chosen, weights, margins = routing(z, none, 2)
    s = torch.softmax(z, -1)
    assert chosen == [[0, 1], [0, 1]] and weights[0] == [float(s[0, 0]), float(s[0, 1])]
    assert abs(sum(weights[0]) - 1.0) > 0.05 and margins[1] == 0.0
    shifted = torch.tensor([0.0, 0.0, 0.0, 1.0], dtype=F64)
    chosen, weights, _ = routing(z, shifted, 2)
    assert chosen[0] == [3, 0] and weights[0] == [float(s[0, 3]), float(s[0, 0])]
    # the multiplier on the queries: 1 until position every - 1, then a step at every multiple
    temp = query_temperature(torch.arange(12), 0.5, 4)
    assert temp[:3].tolist() == [1.0, 1.0, 1.0] and temp[3] == temp[6] == 1.0 + 0.5 * torch.log(torch.tensor(2.0, dtype=F64))
    assert temp[7] == temp[10] > temp[6] and temp[11] > temp[10]


def test_random_model_from_the_command_line(tmp_path):
    from zephyr_b200.cli import main
    from zephyr_b200.config import load_model_config
    from zephyr_b200.parts import expected_weights
    from zephyr_b200.weights import Checkpoint
    from zephyr_b200.weights.loader import check_store

    source = tmp_path / "config.json"
    source.write_text(json.dumps(CONFIGS["C"]))
    assert main(["random-model", "--config", str(source), "--out", str(tmp_path / "model"), "--seed", "3"]) == 0
    config = load_model_config(tmp_path / "model")
    assert config.to_dict() == CONFIGS["C"]
    store = Checkpoint(tmp_path / "model")
    check_store(store, expected_weights(config.to_model_spec()))
    assert tuple(store.shape("l0.mix.uk")) == (8 * 32, 128) and tuple(store.shape("l0.mlp.router")) == (12, 128)
