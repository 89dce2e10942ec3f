"""A plain, slow Legelix in float64: one function per mechanism, written from the equations, sharing
nothing with the package.  It takes the configuration as the dictionary of config.json and the
tensors as a dictionary by name, runs one whole sequence token by token where a mechanism is
recurrent, and returns the logits of every position (and the residual stream after every layer).

Notation: h [T, width] is a sublayer's input, positions count from 0.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def f64(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu").to(F64)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def plain_layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w + b


def plain_unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


# ----------------------------------------------------------------------------- gated linear attention
def plain_gla(h: torch.Tensor, W: dict, p: dict, eps: float) -> torch.Tensor:
    """S_t = diag(a_t) S_{t-1} + k_t v_t^T per head (S is [dim, vdim]), o_t = S_t^T q_t, with
    a_t = sigmoid(z_t)^(1/tau); o is unit-RMS'd per head, scaled, gated by silu(W_g h), projected."""
    T = h.shape[0]
    H, D, V, tau = p["heads"], p["dim"], p["vdim"], float(p["tau"])
    q = (h @ W["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ W["k"].T).view(T, H, D)
    v = (h @ W["v"].T).view(T, H, V)
    z = (h @ W["a1"].T) @ W["a2"].T + W["a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=F64)
    out = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = plain_unit_rms(out, eps) * W["norm"]
    gate = silu(h @ W["g"].T)
    return (out.reshape(T, H * V) * gate) @ W["o"].T


# ----------------------------------------------------------------------------- rotary positions
def plain_rotary_frequencies(rot: dict) -> torch.Tensor:
    dims = rot["dims"]
    f = torch.tensor([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f.tolist():
            wavelength = 2.0 * math.pi / fi
            if wavelength < orig / high:
                out.append(fi)
            elif wavelength > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wavelength - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=F64)
    return f


def plain_rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, dims: int) -> torch.Tensor:
    """x [T, heads, dim]: dimensions 2i and 2i+1 (i < dims/2) turn by positions * freqs[i]."""
    angle = positions.to(F64)[:, None] * freqs[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, w = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


# ----------------------------------------------------------------------------- chunked attention with a sink
def plain_attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, size: int | None,
                         sinks: torch.Tensor | None, start: int = 0) -> torch.Tensor:
    """q [T, H, D] at positions start..start+T-1 over k [start+T, G, D], v [start+T, G, V]: causal, only
    within a position's own chunk of ``size`` (chunks counted from position 0), softmax with one more
    term exp(sink_h) in the denominator that has no key and no value.  Returns [T, H, V]."""
    T, H, _ = q.shape
    G, V = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, V, dtype=F64)
    i = torch.arange(start, start + T)[:, None]
    j = torch.arange(k.shape[0])[None, :]
    seen = j <= i
    if size:
        seen = seen & ((i // size) == (j // size))
    for head in range(H):
        g = head // (H // G)
        score = ((q[:, head] @ k[:, g].T) * scale).masked_fill(~seen, float("-inf"))
        top = score.max(dim=-1, keepdim=True).values
        if sinks is not None:
            top = torch.maximum(top, sinks[head])
        e = torch.exp(score - top)
        denominator = e.sum(dim=-1, keepdim=True)
        if sinks is not None:
            denominator = denominator + torch.exp(sinks[head] - top)
        out[:, head] = (e / denominator) @ v[:, g]
    return out


def plain_chunked_sink_attention(h: torch.Tensor, W: dict, p: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = (h @ W["q"].T + W["q.b"]).view(T, H, D)
    k = (h @ W["k"].T + W["k.b"]).view(T, G, D)
    v = (h @ W["v"].T + W["v.b"]).view(T, G, V)
    q = plain_unit_rms(q, eps) * W["q.norm"]
    k = plain_unit_rms(k, eps) * W["k.norm"]
    rot = p.get("rot")
    positions = torch.arange(T)
    if rot:
        freqs = plain_rotary_frequencies(rot)
        q = plain_rotate(q, positions, freqs, rot["dims"])
        k = plain_rotate(k, positions, freqs, rot["dims"])
    size = p["mask"]["size"] if p.get("mask") else None
    out = plain_attention_core(q, k, v, float(p["scale"]), size, W["sink"])
    return out.reshape(T, H * V) @ W["o"].T + W["o.b"]


# ----------------------------------------------------------------------------- Mamba-2
def plain_mamba2(h: torch.Tensor, W: dict, p: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, P, N, G, taps, parts = p["heads"], p["vdim"], p["state"], p["groups"], p["conv"], p["norm_groups"]
    inner = H * P
    proj = h @ W["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    channels = xbc.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, channels, dtype=F64), xbc], dim=0)
    conv = torch.zeros(T, channels, dtype=F64)
    for j in range(taps):            # column taps-1 weighs the current token, column 0 the oldest
        conv += padded[j:j + T] * W["conv"][:, j]
    xbc = silu(conv + W["conv.b"])
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W["dt_bias"])
    decay = torch.exp(-torch.exp(W["A_log"]) * dt)           # [T, H]
    S = torch.zeros(H, N, P, dtype=F64)
    y = torch.zeros(T, H, P, dtype=F64)
    group_of = [head // (H // G) for head in range(H)]
    for t in range(T):
        Bt, Ct = B[t][group_of], C[t][group_of]              # [H, N]
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * Bt[:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, Ct) + W["D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    y = plain_unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


def plain_parallel(h: torch.Tensor, W: dict, p: dict, eps: float) -> torch.Tensor:
    left = plain_chunked_sink_attention(h, _under(W, "left."), p["left"], eps)
    right = plain_mamba2(h, _under(W, "right."), p["right"], eps)
    return float(p["left_scale"]) * left + float(p["right_scale"]) * right


def plain_dense_ff(h: torch.Tensor, W: dict) -> torch.Tensor:
    return (silu(h @ W["gate"].T) * (h @ W["up"].T)) @ W["down"].T


def _under(W: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t for name, t in W.items() if name.startswith(prefix)}


MIXERS = {"gla": plain_gla, "parallel": plain_parallel}


def plain_legelix(config: dict, tensors: dict, tokens: list[int]):
    """Logits [T, vocab] and the residual stream after every layer [layers, T, width]."""
    W = {name: f64(t) for name, t in tensors.items()}
    eps, m = float(config["norm"]["eps"]), float(config["residual_mult"])
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    after = []
    for index, layer in enumerate(config["layers"]):
        L = _under(W, f"l{index}.")
        mixed = MIXERS[layer["type"]](plain_layer_norm(x, L["norm1"], L["norm1.b"], eps), _under(L, "mix."),
                                      layer["mixer"], eps)
        x = x + m * plain_layer_norm(mixed, L["norm1b"], L["norm1b.b"], eps)
        if layer.get("mlp") is not None:
            fed = plain_dense_ff(plain_layer_norm(x, L["norm2"], L["norm2.b"], eps), _under(L, "mlp."))
            x = x + m * plain_layer_norm(fed, L["norm2b"], L["norm2b.b"], eps)
        after.append(x.clone())
    logits = plain_layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    return logits, torch.stack(after)
