"""Typed configuration of Gefovik, a decoder whose layers norm what their parts put out, not what they read.

config.json names the design under ``architecture`` and lists its layers under ``layers``; each entry
gives ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (the feed-forward, or null
for a layer without one).  Model-wide keys: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``.

Mixer types:

  * ``latent_attention``: ``heads``, ``dim`` (query/key size per head), ``vdim`` (value size per head),
    ``kv_rank`` (size of the latent every position keeps), ``scale``.  Keys and values are linear maps
    of the normed latent; a learned sink per head joins the softmax's denominator; a sigmoid gate per
    head multiplies the head's output.  No position encoding.
  * ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim`` (= ``dim``: the values are the keys as
    projected), ``scale``, and optionally ``softcap`` and ``q_temp`` = {``coef``, ``every``}.  Queries
    and keys are brought to unit root mean square per head (no scales); the queries are then multiplied
    by 1 + coef * ln(floor((p + 1) / every) + 1) at position p; scaled scores are bounded by
    softcap * tanh(score / softcap).  No position encoding.

Feed-forwards (``mlp.kind``): ``dense`` (``ff``; gated, ReLU on the gate) and ``moe`` (``expert.ff``;
``router.experts`` gated SiLU experts and ``router.identity`` identity experts, of which a token takes
``router.top``; the choice is by softmax score plus a learned correction, the weight is the score).

Every layer is x <- x + LN(mixer(x)), x <- x + LN(ff(x)) on a float32 residual stream (the
``outnorm_residual`` block), LN being a layer norm with a scale and no shift.  The head is the embedding
table itself (without the multiplier).  Tensor names: ``embed``, ``l<i>.norm1|norm2``,
``l<i>.mix.q|dkv|dkv.norm|uk|uv|sink|g|o`` or ``l<i>.mix.q|k|o``, ``l<i>.mlp.gate|up|down`` or
``l<i>.mlp.router|correction|e<j>.gate|up|down``, ``final.norm``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .errors import ConfigError
from .legelix import MAX_POSITIONS, _int, _number, _table
from .spec import FeedForwardSpec, InputSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, OutputSpec


@dataclass
class GefovikConfig:
    vocab: int
    width: int
    layers: tuple[Mapping[str, Any], ...]
    norm_eps: float
    embedding_scale: float

    architecture = "Gefovik"
    model_type = "gefovik"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, config: Mapping[str, Any], where: str = "config.json") -> "GefovikConfig":
        if not isinstance(config, Mapping):
            raise ConfigError(f"{where}: the configuration must be a JSON object")
        if config.get("architecture", cls.architecture) != cls.architecture:
            raise ConfigError(f"{where}: not a {cls.architecture} configuration")
        layers = config.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        scale = 1.0
        if config.get("embedding") is not None:
            scale = _number(_table(config, "embedding", where), "scale", where)
        result = cls(vocab=_int(config, "vocab", where), width=_int(config, "width", where),
                     layers=tuple(copy.deepcopy(layers)), norm_eps=_number(_table(config, "norm", where), "eps", where),
                     embedding_scale=scale)
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
            if kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "kv_rank"):
                    _int(mixer, key, at)
                _number(mixer, "scale", at)
            elif kind == "attention":
                for key in ("heads", "kv_heads", "dim"):
                    _int(mixer, key, at)
                if mixer["heads"] % mixer["kv_heads"] != 0:
                    raise ConfigError(f"{at}: heads must be a multiple of kv_heads")
                if mixer.get("vdim", mixer["dim"]) != mixer["dim"]:
                    raise ConfigError(f"{at}: the values are the keys, so vdim must equal dim")
                _number(mixer, "scale", at)
                if mixer.get("softcap") is not None and not _number(mixer, "softcap", at) >= 0.0:
                    raise ConfigError(f"{at}: softcap must not be negative")
                if mixer.get("q_temp") is not None:
                    temp = _table(mixer, "q_temp", at)
                    _number(temp, "coef", at)
                    _int(temp, "every", at)
            else:
                raise ConfigError(f"{at}: unknown layer type {kind!r}; known: attention, latent_attention")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"{at}: 'mlp' must be null, a dense or a moe feed-forward")
            if mlp["kind"] == "dense":
                _int(mlp, "ff", at)
            else:
                _int(_table(mlp, "expert", at), "ff", at)
                router = _table(mlp, "router", at)
                experts, top = _int(router, "experts", at), _int(router, "top", at)
                identity = router.get("identity") or 0
                if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
                    raise ConfigError(f"{at}: router.identity must be a non-negative integer")
                if top > experts + identity:
                    raise ConfigError(f"{at}: router.top exceeds the number of router outputs")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
                "width": self.width}

    # --------------------------------------------------------------- model spec
    def _latent_attention(self, prefix: str, m: Mapping[str, Any]) -> MixerSpec:
        return MixerSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
            "rank": m["kv_rank"], "scale": float(m["scale"]), "norm_eps": self.norm_eps,
            "q_proj": f"{prefix}.q", "latent_proj": f"{prefix}.dkv", "latent_norm": f"{prefix}.dkv.norm",
            "k_up": f"{prefix}.uk", "v_up": f"{prefix}.uv", "sinks": f"{prefix}.sink", "gate": f"{prefix}.g",
            "o_proj": f"{prefix}.o"})

    def _attention(self, prefix: str, m: Mapping[str, Any]) -> MixerSpec:
        temp = m.get("q_temp")
        if temp is not None and float(temp["coef"]) == 0.0:
            temp = None
        return MixerSpec("attention", {
            "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["dim"], "window": 0, "chunk": 0, "scale": float(m["scale"]), "qk_norm_eps": self.norm_eps,
            "unit_qk_norm": True, "values_from_keys": True, "softcap": float(m.get("softcap") or 0.0),
            "q_temp": {"coef": float(temp["coef"]), "every": int(temp["every"])} if temp is not None else None,
            "q_proj": f"{prefix}.q", "k_proj": f"{prefix}.k", "o_proj": f"{prefix}.o"}, None)

    def _feed_forward(self, prefix: str, mlp: Mapping[str, Any]) -> FeedForwardSpec:
        if mlp["kind"] == "dense":
            return FeedForwardSpec("gated", {
                "hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "relu",
                "gate_proj": f"{prefix}.gate", "up_proj": f"{prefix}.up", "down_proj": f"{prefix}.down"})
        router = mlp["router"]
        return FeedForwardSpec("routed", {
            "hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"], "activation": "silu",
            "experts": router["experts"], "identity": router.get("identity") or 0, "top": router["top"],
            "router": f"{prefix}.router", "correction": f"{prefix}.correction",
            "expert_names": tuple((f"{prefix}.e{j}.gate", f"{prefix}.e{j}.up", f"{prefix}.e{j}.down")
                                  for j in range(router["experts"]))})

    def _norm(self, name: str) -> NormSpec:
        return NormSpec("layernorm", self.width, self.norm_eps, name, bias=None)

    def to_model_spec(self) -> ModelSpec:
        from ..parts.model import run_order_for

        layers = []
        for index, layer in enumerate(self.layers):
            prefix, m = f"l{index}", layer["mixer"]
            if layer["type"] == "latent_attention":
                mixer = self._latent_attention(f"{prefix}.mix", m)
            else:
                mixer = self._attention(f"{prefix}.mix", m)
            norms = {"mixer_out": self._norm(f"{prefix}.norm1")}
            feed_forward = None
            if layer.get("mlp") is not None:
                feed_forward = self._feed_forward(f"{prefix}.mlp", layer["mlp"])
                norms["feed_forward_out"] = self._norm(f"{prefix}.norm2")
            layers.append(LayerSpec("outnorm_residual", mixer, feed_forward, norms))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_seq_len=MAX_POSITIONS,
            input=InputSpec("embedding", {"weight": "embed", "vocab_size": self.vocab, "hidden_size": self.width,
                                          "float32_stream": True, "scale": self.embedding_scale,
                                          "rounded_copy": True}),
            layers=tuple(layers), run_order=run_order_for(layers),
            output=OutputSpec("norm_head", {"norm": self._norm("final.norm"), "weight": "embed",
                                            "vocab_size": self.vocab, "hidden_size": self.width}))
        spec.validate()
        return spec
