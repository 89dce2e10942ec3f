"""Gefovik configurations drawn at random (sizes that are no multiples of anything in particular, every
optional piece present or absent, layers in any order and number), each replayed in a mixed trace and in
portions against the plain implementation: what a particular choice of sizes would hide, another one
shows."""

import random

import pytest

from gefovik_models import attention, dense, latent, moe, write_model
from replay_util import collect, random_tokens, trace_mixed, trace_portions
from test_gefovik_gpu import DTYPES, FIXED_CHOICE, assert_rows_match, replay

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 136, 50, 256, 33])

    def feed_forward():
        kind = rng.random()
        if kind < 0.2:
            return None
        if kind < 0.55:
            # not a handful of units: behind its norm a ReLU-gated layer whose few gates are all but closed is a
            # step function of them (the norm blows the one that is barely open up to unit size)
            return dense(rng.choice([48, 100, 36, 44, 256]))
        experts, identity = rng.randint(1, 12), rng.choice([0, 0, 1, 2, 5])
        return moe(experts, identity, rng.randint(1, min(experts + identity, 6)), rng.choice([8, 24, 30, 64, 13]))

    layers = []
    for _ in range(rng.randint(1, 6)):
        if rng.random() < 0.4:
            layers.append(latent(rng.choice([1, 2, 3, 5, 8, 18]), rng.choice([4, 8, 16, 24, 32, 7]), rng.choice([4, 8, 20, 32, 64]),
                                 rng.choice([8, 16, 32, 40, 64, 96, 128, 130, 27]), rng.uniform(0.05, 0.6), feed_forward()))
            continue
        kv_heads = rng.choice([1, 2, 3, 4])
        layers.append(attention(kv_heads * rng.choice([1, 2, 4, 5]), kv_heads, rng.choice([8, 16, 24, 32, 64, 96, 128, 10]),
                                rng.uniform(0.05, 1.2), feed_forward(),
                                softcap=rng.choice([None, 0.5, 3.0, 20.0, 50.0]),
                                q_temp=rng.choice([None, (0.35, 48), (1.5, 1), (0.1, 7), (0.8, 100)])))
    return {"architecture": "Gefovik", "vocab": rng.randint(50, 300), "width": width,
            "embedding": {"scale": rng.choice([0.25, 0.5, 1.0, 3.0])}, "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}


@pytest.mark.parametrize("seed,dtype", [(s, "float32") for s in range(10)] + [(s, "bfloat16") for s in (100, 101, 102, 103)])
def test_a_configuration_drawn_at_random(tmp_path, cuda_device, seed, dtype):
    config = draw_config(seed)
    folder = write_model(tmp_path / "model", config, seed=seed, dtype=DTYPES[dtype], fixed_choice=FIXED_CHOICE[dtype])
    rng = random.Random(seed + 1)
    requests = {f"r{i}": random_tokens(config["vocab"], rng.randint(1, 170), seed=seed * 10 + i) for i in range(6)}
    for build in (trace_mixed, trace_portions):
        steps = build(requests)
        rows = collect(steps, replay(folder, dtype, steps, page_size=rng.choice([16, 32])))
        assert_rows_match(rows, requests, folder, dtype, f"seed {seed} {build.__name__}")
