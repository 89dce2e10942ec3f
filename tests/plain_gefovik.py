"""A plain, slow Gefovik in float64: one function per mechanism, written from the design's equations
and sharing nothing with the package.  Weights come as a dict of torch tensors by checkpoint name; the
configuration is the design's own ``config.json`` dictionary.

The layer: x <- x + LN1(mixer(x)); x <- x + LN2(ff(x)), LN being a layer norm with a scale and no shift;
the parts read x itself.  Mixers: ``latent_attention`` (queries against keys and values that are two
linear maps of one normed low-rank latent, a learned sink in the softmax's denominator, a sigmoid gate per
head) and ``attention`` (grouped heads, the values are the keys as projected, unit-RMS queries and keys, a
query multiplier that grows with the logarithm of the position, capped scores).  Feed-forwards: a gated
dense one with relu, and a routed one with silu experts, a correction that only moves the choice, and
identity experts.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm_scale(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef * ln(floor((p + 1) / every) + 1) for every position p."""
    steps = torch.div(positions + 1, every, rounding_mode="floor").to(F64)
    return 1.0 + coef * torch.log(steps + 1.0)


def causal_softmax(scores: torch.Tensor, sink: torch.Tensor | None = None) -> torch.Tensor:
    """scores [H, T, T] -> weights [H, T, T]; key j counts for query i only if j <= i.  ``sink`` [H]: one
    more term exp(sink_h) in the denominator."""
    T = scores.shape[-1]
    visible = torch.ones(T, T, dtype=torch.bool).tril()
    scores = scores.masked_fill(~visible, -math.inf)
    top = scores.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.view(-1, 1, 1))
    e = torch.exp(scores - top)
    total = e.sum(-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink.view(-1, 1, 1) - top)
    return e / total


def latent_attention(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[f"{prefix}.q"].T).view(T, H, d)
    latent = unit_rms(h @ w[f"{prefix}.dkv"].T, eps) * w[f"{prefix}.dkv.norm"]
    k = (latent @ w[f"{prefix}.uk"].T).view(T, H, d)
    v = (latent @ w[f"{prefix}.uv"].T).view(T, H, dv)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    p = causal_softmax(scores, w[f"{prefix}.sink"])
    o = torch.einsum("hij,jhd->ihd", p, v)
    gate = torch.sigmoid(h @ w[f"{prefix}.g"].T)               # [T, H]
    o = o * gate.unsqueeze(-1)
    return o.reshape(T, H * dv) @ w[f"{prefix}.o"].T


def capped_attention(h: torch.Tensor, w: dict, prefix: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[f"{prefix}.q"].T).view(T, H, d)
    k = (h @ w[f"{prefix}.k"].T).view(T, G, d)
    v = k                                                      # the values are the keys as projected
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    temp = m.get("q_temp")
    if temp is not None:
        q = q * query_temperature(torch.arange(T), temp["coef"], temp["every"]).view(T, 1, 1)
    per = H // G
    k_of = k.repeat_interleave(per, dim=1)
    v_of = v.repeat_interleave(per, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k_of) * m["scale"]
    cap = m.get("softcap")
    if cap:
        scores = cap * torch.tanh(scores / cap)
    p = causal_softmax(scores)
    o = torch.einsum("hij,jhd->ihd", p, v_of)
    return o.reshape(T, H * d) @ w[f"{prefix}.o"].T


def dense_ff(h: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    return (torch.relu(h @ w[f"{prefix}.gate"].T) * (h @ w[f"{prefix}.up"].T)) @ w[f"{prefix}.down"].T


def routing(z: torch.Tensor, correction: torch.Tensor, top: int):
    """Router logits z [T, outputs] -> (chosen outputs [T][top], their weights, the margin of every token's
    choice: how far the last chosen output's choice score lies above the best one left out)."""
    s = torch.softmax(z, dim=-1)
    choice = s + correction
    chosen, weights, margins = [], [], []
    for t in range(z.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-float(choice[t, e]), e))
        chosen.append(order[:top])
        weights.append([float(s[t, e]) for e in order[:top]])
        margins.append(float(choice[t, order[top - 1]] - choice[t, order[top]]) if top < z.shape[1] else float("inf"))
    return chosen, weights, margins


def routed_ff(h: torch.Tensor, w: dict, prefix: str, mlp: dict, margins: list | None = None) -> torch.Tensor:
    r = mlp["router"]
    real, top = r["experts"], r["top"]
    chosen, weights, gaps = routing(h @ w[f"{prefix}.router"].T, w[f"{prefix}.correction"], top)
    if margins is not None:
        margins.append(gaps)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t], weights[t]):
            if e >= real:
                y = h[t]
            else:
                p = f"{prefix}.e{e}"
                gate = h[t] @ w[f"{p}.gate"].T
                y = (gate * torch.sigmoid(gate) * (h[t] @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T
            out[t] += weight * y
    return out


def forward(config: dict, weights: dict, tokens: list[int], layer_outputs: list | None = None,
            margins: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence, float64.  ``layer_outputs`` collects the stream after each layer,
    ``margins`` one list per routed layer with every token's routing margin."""
    w = {name: t.to(F64) for name, t in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens)] * config.get("embedding", {}).get("scale", 1.0)
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            mixed = latent_attention(x, w, f"l{i}.mix", m, eps)
        else:
            mixed = capped_attention(x, w, f"l{i}.mix", m, eps)
        x = x + layer_norm_scale(mixed, w[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, w, f"l{i}.mlp") if mlp["kind"] == "dense" else routed_ff(x, w, f"l{i}.mlp", mlp, margins)
            x = x + layer_norm_scale(y, w[f"l{i}.norm2"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return layer_norm_scale(x, w["final.norm"], eps) @ w["embed"].T
