"""Small Legelix configurations and weights for the tests: sizes that differ from one another in every
way the design allows (head counts and group ratios, key and value widths that are unequal and not
powers of two, rotation on part of a head and on all of it, with and without frequency scaling, with
and without a chunked mask, chunks smaller and larger than a page, one to four convolution taps,
one or several norm parts, a layer without a feed-forward, multipliers other than one half)."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def gla(heads, dim, vdim, tau, ff):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def parallel(left, right, left_scale, right_scale, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def attention(heads, kv_heads, dim, vdim, scale, chunk=None, rot=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        out["mask"] = {"size": chunk}
    if rot:
        out["rot"] = rot
    return out


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}

CONFIGS = {
    # P: narrow, every kind of layer, a layer without a feed-forward, chunks of 24 (a page and a half)
    "P": {"architecture": "Legelix", "vocab": 97, "width": 64, "residual_mult": 0.7, "norm": {"eps": 1e-5}, "layers": [
        gla(2, 16, 24, 8.0, 96),
        parallel(attention(4, 2, 32, 16, 0.2, chunk=24, rot={"base": 10000.0, "dims": 16}),
                 mamba(4, 16, 16, 1, 3, 1), 1.3, 0.6, 96),
        gla(2, 16, 24, 8.0, None),
        parallel(attention(4, 2, 32, 16, 0.2, chunk=24, rot={"base": 10000.0, "dims": 16}),
                 mamba(4, 16, 16, 1, 3, 1), 1.3, 0.6, 80)]},
    # Q: widths that are no powers of two, one key/value head per query head, rotation on the whole head
    # with scaled frequencies, a chunk smaller than a page, four taps, three norm parts, groups = heads
    "Q": {"architecture": "Legelix", "vocab": 131, "width": 96, "residual_mult": 1.0, "norm": {"eps": 1e-6}, "layers": [
        parallel(attention(3, 3, 24, 40, 0.35, chunk=10, rot={"base": 500.0, "dims": 24, "scaling": SCALING}),
                 mamba(3, 40, 24, 3, 4, 3), 0.8, 1.1, 72),
        gla(3, 80, 40, 2.0, 72),
        parallel(attention(3, 3, 24, 40, 0.35, chunk=10, rot={"base": 500.0, "dims": 24, "scaling": SCALING}),
                 mamba(3, 40, 24, 3, 4, 3), 0.8, 1.1, 72)]},
    # R: one key/value head for all query heads, no mask and no rotation at all, two taps, a single head
    # in the recurrent layers, a key width of 144 channels (five warps, the last one partly empty)
    "R": {"architecture": "Legelix", "vocab": 64, "width": 128, "residual_mult": 0.25, "norm": {"eps": 1e-6}, "layers": [
        gla(1, 144, 48, 32.0, 160),
        parallel(attention(4, 1, 16, 16, 0.25), mamba(1, 64, 32, 1, 2, 2), 1.0, 1.0, 160),
        parallel(attention(8, 2, 16, 48, 0.25, chunk=64, rot={"base": 100.0, "dims": 8}),
                 mamba(8, 16, 48, 4, 1, 4), 0.5, 2.0, None)]},
    # S: keys and values of one width (32, then 64): in bfloat16 these layers take the split-context
    # decode kernel and the tensor-core prompt kernel, which mask chunks and count sinks themselves
    "S": {"architecture": "Legelix", "vocab": 80, "width": 64, "residual_mult": 0.5, "norm": {"eps": 1e-6}, "layers": [
        parallel(attention(4, 2, 32, 32, 0.18, chunk=40, rot={"base": 300.0, "dims": 32, "scaling": SCALING}),
                 mamba(2, 32, 16, 2, 4, 1), 1.2, 0.9, 96),
        gla(1, 32, 64, 16.0, 96),
        parallel(attention(2, 2, 64, 64, 0.125, chunk=72, rot={"base": 10000.0, "dims": 16}),
                 mamba(2, 32, 16, 1, 4, 2), 0.7, 1.0, 96)]},
}
PAGE_SIZE = {"P": 16, "Q": 16, "R": 32, "S": 16}
DECAY_RANK = {"P": 8, "Q": 5, "R": 16, "S": 4}


def make_weights(config: dict, rank: int, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors by name, from distributions that keep every mechanism alive: scales around one,
    shifts and sinks that matter, decays spread between fast and slow."""
    g = torch.Generator().manual_seed(seed)
    width = config["width"]

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(*shape, generator=g) * std + mean

    def linear(out, inp):
        return normal(out, inp, std=inp ** -0.5)

    W = {"embed": normal(config["vocab"], width), "head": linear(config["vocab"], width),
         "final.norm": normal(width, std=0.1, mean=1.0), "final.norm.b": normal(width, std=0.1)}
    for index, layer in enumerate(config["layers"]):
        L, m = f"l{index}", layer["mixer"]
        names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer["mlp"] else [])
        for name in names:
            W[f"{L}.{name}"] = normal(width, std=0.1, mean=1.0)
            W[f"{L}.{name}.b"] = normal(width, std=0.1)
        if layer["type"] == "gla":
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            W.update({f"{L}.mix.q": linear(hd, width), f"{L}.mix.k": linear(hd, width), f"{L}.mix.v": linear(hv, width),
                      f"{L}.mix.g": linear(hv, width), f"{L}.mix.o": linear(width, hv),
                      f"{L}.mix.norm": normal(m["vdim"], std=0.1, mean=1.0), f"{L}.mix.a1": linear(rank, width),
                      f"{L}.mix.a2": linear(hd, rank) * 2.0, f"{L}.mix.a2.b": normal(hd, std=1.0, mean=2.0)})
        else:
            a, r = m["left"], m["right"]
            P = f"{L}.mix.left"
            W.update({f"{P}.q": linear(a["heads"] * a["dim"], width), f"{P}.q.b": normal(a["heads"] * a["dim"], std=0.3),
                      f"{P}.k": linear(a["kv_heads"] * a["dim"], width), f"{P}.k.b": normal(a["kv_heads"] * a["dim"], std=0.3),
                      f"{P}.v": linear(a["kv_heads"] * a["vdim"], width), f"{P}.v.b": normal(a["kv_heads"] * a["vdim"], std=0.3),
                      f"{P}.q.norm": normal(a["dim"], std=0.2, mean=1.0), f"{P}.k.norm": normal(a["dim"], std=0.2, mean=1.0),
                      f"{P}.sink": normal(a["heads"], std=1.5),
                      f"{P}.o": linear(width, a["heads"] * a["vdim"]), f"{P}.o.b": normal(width, std=0.3)})
            P = f"{L}.mix.right"
            inner = r["heads"] * r["vdim"]
            channels = inner + 2 * r["groups"] * r["state"]
            W.update({f"{P}.in": linear(2 * inner + 2 * r["groups"] * r["state"] + r["heads"], width),
                      f"{P}.conv": normal(channels, r["conv"], std=0.5), f"{P}.conv.b": normal(channels, std=0.2),
                      f"{P}.dt_bias": normal(r["heads"], std=1.0, mean=-1.0), f"{P}.A_log": normal(r["heads"], std=0.7),
                      f"{P}.D": normal(r["heads"], std=0.5, mean=1.0), f"{P}.norm": normal(inner, std=0.1, mean=1.0),
                      f"{P}.o": linear(width, inner)})
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            W.update({f"{L}.mlp.gate": linear(ff, width), f"{L}.mlp.up": linear(ff, width), f"{L}.mlp.down": linear(width, ff)})
    return W


def write_model(folder: Path, config: dict, rank: int, seed: int, dtype: torch.dtype) -> Path:
    """config.json and model.safetensors in ``dtype``.  The plain implementation reads the stored
    (rounded) values back, so both sides start from the same numbers."""
    from zephyr_b200.weights.safetensors_io import save_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    save_safetensors(folder / "model.safetensors",
                     {name: t.to(dtype).contiguous() for name, t in make_weights(config, rank, seed).items()})
    return folder


def read_model(folder: Path) -> tuple[dict, dict[str, torch.Tensor]]:
    from zephyr_b200.weights import Checkpoint

    store = Checkpoint(folder)
    return json.loads((Path(folder) / "config.json").read_text()), {name: store.read(name) for name in store.names()}
