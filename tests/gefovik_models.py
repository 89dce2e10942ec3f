"""Small Gefovik configurations and weights for the tests: sizes that differ from one another in every way
the design allows (head counts and group ratios, key widths that take the tensor-core attention kernels
and widths that do not, latent sizes likewise, value sizes unlike the key sizes, with and without a bound
on the scores and a query multiplier, an embedding multiplier of one, routed layers that take one, some
or all of their outputs, with and without identity experts, a layer without a feed-forward, widths and
inner sizes that are no multiples of eight)."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def latent(heads, dim, vdim, rank, scale, mlp):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale},
            "mlp": mlp}


def attention(heads, kv_heads, dim, scale, mlp, softcap=None, q_temp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if softcap is not None:
        mixer["softcap"] = softcap
    if q_temp is not None:
        mixer["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


CONFIGS = {
    # A: latent and head sizes that only the general attention kernel takes, beside a layer on the fast
    # ones; a routed layer with identity experts; a layer without a feed-forward; a single key/value head
    "A": {"architecture": "Gefovik", "vocab": 97, "width": 64, "embedding": {"scale": 0.7}, "norm": {"eps": 1e-5}, "layers": [
        latent(3, 16, 24, 48, 0.3, dense(80)),
        attention(4, 2, 32, 0.6, moe(5, 2, 3, 40), softcap=4.0, q_temp=(0.25, 16)),
        latent(2, 8, 40, 20, 0.5, None),
        attention(6, 1, 16, 0.9, moe(3, 0, 1, 56), softcap=2.5, q_temp=(1.0, 5))]},
    # B: an embedding multiplier of one, a width that is no power of two, no bound and no multiplier in one
    # attention layer, a router that takes ALL its outputs, an inner size that is no multiple of eight,
    # one key/value head per query head
    "B": {"architecture": "Gefovik", "vocab": 131, "width": 96, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "layers": [
        attention(3, 3, 64, 0.4, dense(50)),
        latent(4, 24, 8, 64, 0.25, moe(4, 1, 5, 36)),
        attention(2, 1, 96, 0.5, moe(6, 3, 2, 20), softcap=25.0, q_temp=(0.4, 48)),
        latent(5, 32, 32, 96, 0.2, dense(72))]},
    # C: pages of 32, eight heads on a latent of 128, a bound small enough to flatten most scores, a
    # multiplier that changes every third position
    "C": {"architecture": "Gefovik", "vocab": 64, "width": 128, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6}, "layers": [
        latent(8, 32, 16, 128, 0.15, moe(9, 3, 2, 24)),
        attention(8, 2, 96, 0.7, dense(160), softcap=1.5, q_temp=(0.5, 3)),
        attention(4, 4, 32, 1.0, None, q_temp=(2.0, 40))]},
}
PAGE_SIZE = {"A": 16, "B": 16, "C": 32}


def make_weights(config: dict, seed: int, fixed_choice: bool = False) -> dict[str, torch.Tensor]:
    """Float32 tensors by name, from distributions that keep every mechanism alive: scales around one,
    sinks that take a real share, gates on both sides of one half, corrections that move some choices.
    With ``fixed_choice`` the corrections lie 1.5 apart, further than two scores can: every token then takes
    the same outputs (with its own weights), and no rounding of a layer's input can flip a choice."""
    g = torch.Generator().manual_seed(seed)
    width = config["width"]

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(*shape, generator=g) * std + mean

    def linear(out, inp, gain=1.0):
        return normal(out, inp, std=gain * inp ** -0.5)

    W = {"embed": normal(config["vocab"], width), "final.norm": normal(width, std=0.1, mean=1.0)}
    for index, layer in enumerate(config["layers"]):
        L, m = f"l{index}", layer["mixer"]
        W[f"{L}.norm1"] = normal(width, std=0.1, mean=1.0)
        if layer["type"] == "latent_attention":
            hd, hv, rank = m["heads"] * m["dim"], m["heads"] * m["vdim"], m["kv_rank"]
            W.update({f"{L}.mix.q": linear(hd, width), f"{L}.mix.dkv": linear(rank, width),
                      f"{L}.mix.dkv.norm": normal(rank, std=0.2, mean=1.0), f"{L}.mix.uk": linear(hd, rank, 2.0),
                      f"{L}.mix.uv": linear(hv, rank), f"{L}.mix.sink": normal(m["heads"], std=1.5),
                      f"{L}.mix.g": linear(m["heads"], width, 1.5), f"{L}.mix.o": linear(width, hv)})
        else:
            W.update({f"{L}.mix.q": linear(m["heads"] * m["dim"], width), f"{L}.mix.k": linear(m["kv_heads"] * m["dim"], width),
                      f"{L}.mix.o": linear(width, m["heads"] * m["dim"])})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        W[f"{L}.norm2"] = normal(width, std=0.1, mean=1.0)
        if mlp["kind"] == "dense":
            W.update({f"{L}.mlp.gate": linear(mlp["ff"], width), f"{L}.mlp.up": linear(mlp["ff"], width),
                      f"{L}.mlp.down": linear(width, mlp["ff"])})
        else:
            ff, r = mlp["expert"]["ff"], mlp["router"]
            outputs = r["experts"] + r["identity"]
            W[f"{L}.mlp.router"] = linear(outputs, width, 1.0 / (config["embedding"]["scale"] * (1 + index) ** 0.5))
            W[f"{L}.mlp.correction"] = normal(outputs, std=0.1)
            if fixed_choice:
                W[f"{L}.mlp.correction"] = torch.randperm(outputs, generator=g).float() * 1.5
            for e in range(r["experts"]):
                W.update({f"{L}.mlp.e{e}.gate": linear(ff, width), f"{L}.mlp.e{e}.up": linear(ff, width),
                          f"{L}.mlp.e{e}.down": linear(width, ff)})
    return W


def write_model(folder: Path, config: dict, seed: int, dtype: torch.dtype, fixed_choice: bool = False) -> Path:
    """config.json and model.safetensors in ``dtype``.  The plain implementation reads the stored
    (rounded) values back, so both sides start from the same numbers."""
    from zephyr_b200.weights.safetensors_io import save_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    save_safetensors(folder / "model.safetensors",
                     {name: t.to(dtype).contiguous() for name, t in make_weights(config, seed, fixed_choice).items()})
    return folder


def read_model(folder: Path) -> tuple[dict, dict[str, torch.Tensor]]:
    from zephyr_b200.weights import Checkpoint

    store = Checkpoint(folder)
    return json.loads((Path(folder) / "config.json").read_text()), {name: store.read(name) for name in store.names()}
