"""Typed configuration of Legelix, a decoder whose layers alternate token mixers of different kinds.

config.json names the design under ``architecture`` and lists its layers under ``layers``; each entry
gives ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (a dense gated
feed-forward ``{"kind": "dense", "ff": n}``, or null for a layer without one).  Model-wide keys:
``vocab``, ``width``, ``residual_mult``, ``norm.eps``.  Mixer types:

  * ``gla``: gated linear attention; ``heads``, ``dim`` (key channels per head), ``vdim`` (value
    channels per head), ``tau`` (temperature of the decay).  The inner size of the decay's low-rank
    projection is not a key: the checkpoint's tensor gives it.
  * ``parallel``: two mixers over the same input, ``left_scale * left + right_scale * right``.
    ``left`` is attention with grouped key/value heads (``heads``, ``kv_heads``, ``dim``, ``vdim``),
    biases, per-head RMS norm of q and k, rotation of adjacent pairs on the first ``rot.dims``
    dimensions (``rot.base``, optional ``rot.scaling`` = factor / low / high / original), a score
    ``scale``, a chunked mask (``mask.size``) and a learned sink per head.  ``right`` is Mamba-2
    (``heads``, ``vdim``, ``state``, ``groups``, ``conv`` taps, ``norm_groups``).

Every layer is norm -> part -> norm -> scaled sum into a float32 residual stream (the
``sandwich_residual`` block) with layer norms that have scale and shift.  Tensor names: ``embed``,
``l<i>.norm1|norm1b|norm2|norm2b`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``,
``final.norm`` (+ ``.b``), ``head``.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Mapping

from .errors import ConfigError
from .spec import (FeedForwardSpec, InputSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, OutputSpec, PositionSpec)

# The design names no longest sequence; the engine's own ``max_seq_len`` bounds a run.
MAX_POSITIONS = 1 << 17


def _int(table: Mapping[str, Any], key: str, where: str) -> int:
    value = table.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"{where}: '{key}' must be a positive integer, got {value!r}")
    return value


def _number(table: Mapping[str, Any], key: str, where: str) -> float:
    value = table.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(float(value)):
        raise ConfigError(f"{where}: '{key}' must be a finite number, got {value!r}")
    return float(value)


def _table(table: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = table.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where}: '{key}' must be a JSON object")
    return value


@dataclass
class LegelixConfig:
    vocab: int
    width: int
    layers: tuple[Mapping[str, Any], ...]
    norm_eps: float
    residual_mult: float
    # For random-weight models only: the inner size of the gated linear attention's decay projection,
    # which a checkpoint's tensor gives and no configuration key names.
    decay_rank: int | None = field(default=None, compare=False)

    architecture = "Legelix"
    model_type = "legelix"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, config: Mapping[str, Any], where: str = "config.json") -> "LegelixConfig":
        if not isinstance(config, Mapping):
            raise ConfigError(f"{where}: the configuration must be a JSON object")
        if config.get("architecture", cls.architecture) != cls.architecture:
            raise ConfigError(f"{where}: not a {cls.architecture} configuration")
        layers = config.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        result = cls(vocab=_int(config, "vocab", where), width=_int(config, "width", where),
                     layers=tuple(copy.deepcopy(layers)), norm_eps=_number(_table(config, "norm", where), "eps", where),
                     residual_mult=_number(config, "residual_mult", where))
        result.validate(where)
        return result

    def validate(self, where: str = "config") -> None:
        if not self.norm_eps > 0.0:
            raise ConfigError(f"{where}: norm.eps must be positive")
        for index, layer in enumerate(self.layers):
            at = f"{where}: layers[{index}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"{at} must be a JSON object")
            kind, mixer = layer.get("type"), _table(layer, "mixer", at)
            if kind == "gla":
                for key in ("heads", "dim", "vdim"):
                    _int(mixer, key, at)
                if not _number(mixer, "tau", at) > 0.0:
                    raise ConfigError(f"{at}: tau must be positive")
            elif kind == "parallel":
                left, right = _table(mixer, "left", at), _table(mixer, "right", at)
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _int(left, key, at)
                if left["heads"] % left["kv_heads"] != 0:
                    raise ConfigError(f"{at}: heads must be a multiple of kv_heads")
                _number(left, "scale", at)
                if left.get("mask") is not None:
                    _int(_table(left, "mask", at), "size", at)
                if left.get("rot") is not None:
                    rot = _table(left, "rot", at)
                    if _int(rot, "dims", at) % 2 != 0 or rot["dims"] > left["dim"] or not _number(rot, "base", at) > 0.0:
                        raise ConfigError(f"{at}: rot.dims must be even and at most dim, rot.base positive")
                    if rot.get("scaling") is not None:
                        for key in ("factor", "low", "high", "original"):
                            _number(_table(rot, "scaling", at), key, at)
                for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                    _int(right, key, at)
                _number(mixer, "left_scale", at)
                _number(mixer, "right_scale", at)
            else:
                raise ConfigError(f"{at}: unknown layer type {kind!r}; known: gla, parallel")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"{at}: 'mlp' must be null or a dense feed-forward")
                _int(mlp, "ff", at)

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)),
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab,
                "width": self.width}

    # --------------------------------------------------------------- model spec
    def _gla(self, prefix: str, m: Mapping[str, Any]) -> MixerSpec:
        return MixerSpec("gla", {
            "hidden_size": self.width, "heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
            "tau": float(m["tau"]), "norm_eps": self.norm_eps, "decay_rank": self.decay_rank,
            "q": f"{prefix}.q", "k": f"{prefix}.k", "v": f"{prefix}.v", "g": f"{prefix}.g", "o": f"{prefix}.o",
            "norm": f"{prefix}.norm", "a1": f"{prefix}.a1", "a2": f"{prefix}.a2", "a2_bias": f"{prefix}.a2.b"})

    def _attention(self, prefix: str, m: Mapping[str, Any]) -> MixerSpec:
        rot = m.get("rot")
        position = None
        if rot is not None:
            position = PositionSpec("rope_pairs", head_dim=m["dim"], max_positions=MAX_POSITIONS, params={
                "base": float(rot["base"]), "dims": rot["dims"],
                "scaling": dict(rot["scaling"]) if rot.get("scaling") is not None else None})
        return MixerSpec("attention", {
            "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "window": 0, "chunk": m["mask"]["size"] if m.get("mask") is not None else 0,
            "scale": float(m["scale"]), "qk_norm_eps": self.norm_eps,
            "q_proj": f"{prefix}.q", "k_proj": f"{prefix}.k", "v_proj": f"{prefix}.v", "o_proj": f"{prefix}.o",
            "q_bias": f"{prefix}.q.b", "k_bias": f"{prefix}.k.b", "v_bias": f"{prefix}.v.b", "o_bias": f"{prefix}.o.b",
            "q_norm": f"{prefix}.q.norm", "k_norm": f"{prefix}.k.norm", "sinks": f"{prefix}.sink"}, position)

    def _mamba2(self, prefix: str, m: Mapping[str, Any]) -> MixerSpec:
        return MixerSpec("mamba2", {
            "hidden_size": self.width, "heads": m["heads"], "value_dim": m["vdim"], "state": m["state"],
            "groups": m["groups"], "conv": m["conv"], "norm_groups": m["norm_groups"], "norm_eps": self.norm_eps,
            "in": f"{prefix}.in", "conv_weight": f"{prefix}.conv", "conv_bias": f"{prefix}.conv.b",
            "dt_bias": f"{prefix}.dt_bias", "a_log": f"{prefix}.A_log", "skip": f"{prefix}.D",
            "norm": f"{prefix}.norm", "o": f"{prefix}.o"})

    def _norm(self, name: str) -> NormSpec:
        return NormSpec("layernorm", self.width, self.norm_eps, name, bias=f"{name}.b")

    def to_model_spec(self) -> ModelSpec:
        from ..parts.model import run_order_for

        layers = []
        for index, layer in enumerate(self.layers):
            prefix, m = f"l{index}", layer["mixer"]
            if layer["type"] == "gla":
                mixer = self._gla(f"{prefix}.mix", m)
            else:
                mixer = MixerSpec("parallel", {"branches": (
                    (self._attention(f"{prefix}.mix.left", m["left"]), float(m["left_scale"])),
                    (self._mamba2(f"{prefix}.mix.right", m["right"]), float(m["right_scale"])))})
            norms = {"mixer": self._norm(f"{prefix}.norm1"), "mixer_out": self._norm(f"{prefix}.norm1b")}
            feed_forward = None
            if layer.get("mlp") is not None:
                feed_forward = FeedForwardSpec("swiglu", {
                    "hidden_size": self.width, "intermediate_size": layer["mlp"]["ff"],
                    "gate_proj": f"{prefix}.mlp.gate", "up_proj": f"{prefix}.mlp.up", "down_proj": f"{prefix}.mlp.down"})
                norms["feed_forward"] = self._norm(f"{prefix}.norm2")
                norms["feed_forward_out"] = self._norm(f"{prefix}.norm2b")
            layers.append(LayerSpec("sandwich_residual", mixer, feed_forward, norms,
                                    block_params={"residual_mult": self.residual_mult}))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_seq_len=MAX_POSITIONS,
            input=InputSpec("embedding", {"weight": "embed", "vocab_size": self.vocab, "hidden_size": self.width,
                                          "float32_stream": True}),
            layers=tuple(layers), run_order=run_order_for(layers),
            output=OutputSpec("norm_head", {"norm": self._norm("final.norm"), "weight": "head",
                                            "vocab_size": self.vocab, "hidden_size": self.width}))
        spec.validate()
        return spec
