"""Legelix configurations drawn at random (sizes that are no multiples of anything in particular, every
optional piece present or absent, layers in any order), each replayed in a mixed trace against the plain
implementation: what a particular choice of sizes would hide, another one shows."""

import random

import pytest
import torch

from legelix_models import attention, gla, mamba, parallel, write_model
from replay_util import collect, random_tokens, trace_mixed, trace_portions
from test_legelix_gpu import DTYPES, assert_rows_match, replay

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> tuple[dict, int]:
    rng = random.Random(seed)
    width = rng.choice([40, 72, 100, 136, 50])
    layers = []
    for _ in range(rng.randint(2, 4)):
        ff = rng.choice([None, 48, 100, 36])
        if rng.random() < 0.45:
            layers.append(gla(rng.choice([1, 2, 3]), rng.choice([8, 20, 32, 48]), rng.choice([8, 24, 36, 70]),
                              rng.uniform(1.0, 32.0), ff))
            continue
        kv_heads, dim = rng.choice([1, 2, 3]), rng.choice([8, 16, 24, 32, 64])
        rot = None
        if rng.random() < 0.8:
            rot = {"base": rng.choice([100.0, 10000.0, 500000.0]), "dims": rng.choice([d for d in (2, 4, 8, 16, 24, 32, 64) if d <= dim])}
            if rng.random() < 0.5:
                rot["scaling"] = {"factor": rng.choice([2.0, 8.0]), "low": 1.0, "high": rng.choice([2.0, 4.0]),
                                  "original": rng.choice([16, 64, 256])}
        left = attention(kv_heads * rng.choice([1, 2, 4]), kv_heads, dim, rng.choice([dim, dim, 6, 16, 40]),
                         rng.uniform(0.05, 0.5), chunk=rng.choice([None, 7, 16, 50, 128]), rot=rot)
        heads = rng.choice([1, 2, 4, 6])
        vdim = rng.choice([4, 8, 20, 32])
        inner = heads * vdim
        right = mamba(heads, vdim, rng.choice([4, 16, 40]), rng.choice([g for g in (1, 2, 3, 4, 6) if heads % g == 0]),
                      rng.choice([1, 2, 3, 4]),
                      # a unit norm over a handful of values is a sign function: parts of eight values and more
                      rng.choice([n for n in (1, 2, 4) if inner % n == 0 and inner // n >= 8] or [1]))
        layers.append(parallel(left, right, rng.uniform(0.3, 1.5), rng.uniform(0.3, 1.5), ff))
    config = {"architecture": "Legelix", "vocab": rng.randint(50, 300), "width": width,
              "residual_mult": rng.choice([0.25, 0.5, 1.0]), "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    return config, rng.choice([3, 8, 17])


@pytest.mark.parametrize("seed,dtype", [(s, "float32") for s in range(8)] + [(s, "bfloat16") for s in (100, 101, 102)])
def test_a_configuration_drawn_at_random(tmp_path, cuda_device, seed, dtype):
    config, rank = draw_config(seed)
    folder = write_model(tmp_path / "model", config, rank, seed=seed, dtype=DTYPES[dtype])
    rng = random.Random(seed + 1)
    requests = {f"r{i}": random_tokens(config["vocab"], rng.randint(1, 170), seed=seed * 10 + i) for i in range(6)}
    for build in (trace_mixed, trace_portions):
        steps = build(requests)
        rows = collect(steps, replay(folder, dtype, steps, page_size=16))
        assert_rows_match(rows, requests, folder, dtype, f"seed {seed} {build.__name__}")
