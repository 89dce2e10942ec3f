"""Latent attention as a mixer: keys and values of all heads are two linear maps of one small latent per
position, and only the latent is cached.

    q = Wq h                                   [heads, dim]
    c = rmsnorm(Wc h) * w_c                    [rank]        (the latent; the one thing a position keeps)
    k_j = Wuk c_j,  v_j = Wuv c_j              per head: [dim], [vdim]
    score_ij = scale * (q_i . k_j),  causal;   softmax, with exp(sink_h) in the denominator where the
                                               spec names sinks (a term without key or value)
    o_i = sum_j p_ij v_j,  times sigmoid(Wg h)_h where the spec names a gate;  out = Wo concat(o)

There is no position encoding.  The part works in the latent space, which is what makes caching c alone
enough: q_i . (Wuk_h c_j) = (Wuk_h^T q_i) . c_j and sum_j p_ij Wuv_h c_j = Wuv_h (sum_j p_ij c_j).  So the
queries are carried into the latent space head by head (``ops.head_linear`` with the transposed key
maps), the attention runs with ONE key/value head of width ``rank`` whose keys are its values (a cache
that keeps keys only), and the result is carried out by the value maps, with the gate in the same
kernel.  Scores, softmax and the latent's norm are float32.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..cache import PagedCacheSpec
from ..config.errors import ConfigError
from ..config.spec import LayerCall, MixerSpec
from ..kernels import ops
from ..weights.loader import ROLE_LINEAR, ROLE_NORM, ROLE_ZERO, WeightDecl
from .base import Mixer, StepContext, register_mixer


class LatentAttention(Mixer):
    graph_safe = True
    takes_out_dtype = True

    def __init__(self, spec: MixerSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device | str):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.hd, self.vd, self.rank = int(p["num_heads"]), int(p["head_dim"]), int(p["value_dim"]), int(p["rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["norm_eps"])
        self.dtype = dtype
        if min(self.nh, self.hd, self.vd, self.rank) <= 0:
            raise ConfigError("latent attention needs positive head count, head sizes and rank")
        if self.rank > 512:
            raise ConfigError(f"latent attention takes a latent size of at most 512, not {self.rank}")
        nh, hd, vd, rank = self.nh, self.hd, self.vd, self.rank
        gate = weights[p["gate"]] if p.get("gate") else None
        # One product for everything that reads the layer's input: queries, the latent, the gates.
        rows = [weights[p["q_proj"]], weights[p["latent_proj"]]] + ([gate] if gate is not None else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.has_gate = gate is not None
        self.latent_norm = weights[p["latent_norm"]].float().contiguous()
        # Per head [rank, dim]: the key map transposed, so that it carries a query into the latent space.
        self.w_q_to_latent = weights[p["k_up"]].view(nh, hd, rank).transpose(1, 2).contiguous()
        self.w_latent_to_v = weights[p["v_up"]].view(nh, vd, rank).contiguous()
        self.w_o = weights[p["o_proj"]]
        self.sinks = weights[p["sinks"]].float().contiguous() if p.get("sinks") else None
        self.tile_tokens = ops.attention_tile_tokens(nh)
        # In bfloat16 the split-context decode kernel and the tensor-core prompt kernel take the latent
        # as one key/value head whose keys are its values, where they take its width and head count.
        self.fast_decode = ops.paged_decode_supported(nh, 1, rank, dtype)
        self.fast_prefill = ops.paged_prefill_supported(nh, 1, rank, dtype)
        self.prefill_tile_tokens = ops.paged_prefill_tile_tokens()

    @staticmethod
    def weight_decls(spec: MixerSpec) -> dict[str, WeightDecl]:
        p = spec.params
        hidden, nh, hd, vd, rank = (int(p[k]) for k in ("hidden_size", "num_heads", "head_dim", "value_dim", "rank"))
        decls = {
            p["q_proj"]: WeightDecl((nh * hd, hidden), ROLE_LINEAR),
            p["latent_proj"]: WeightDecl((rank, hidden), ROLE_LINEAR),
            p["latent_norm"]: WeightDecl((rank,), ROLE_NORM),
            p["k_up"]: WeightDecl((nh * hd, rank), ROLE_LINEAR),
            p["v_up"]: WeightDecl((nh * vd, rank), ROLE_LINEAR),
            p["o_proj"]: WeightDecl((hidden, nh * vd), ROLE_LINEAR),
        }
        if p.get("gate"):
            decls[p["gate"]] = WeightDecl((nh, hidden), ROLE_LINEAR)
        if p.get("sinks"):
            decls[p["sinks"]] = WeightDecl((nh,), ROLE_ZERO)
        return decls

    def weights_read(self) -> list[torch.Tensor]:
        return [self.w_in, self.w_q_to_latent, self.w_latent_to_v, self.w_o, self.latent_norm]

    @staticmethod
    def cache_spec(spec: MixerSpec) -> PagedCacheSpec:
        return PagedCacheSpec(1, key_dim=int(spec.params["rank"]), keys_only=True)

    @staticmethod
    def tile_requests(spec: MixerSpec) -> list[tuple[int, str]]:
        tokens = ops.attention_tile_tokens(int(spec.params["num_heads"]))
        return [(tokens, "all"), (tokens, "multi"), (tokens, "single"), (ops.paged_prefill_tile_tokens(), "multi")]

    def forward(self, x: torch.Tensor, ctx: StepContext, call: LayerCall,
                out_dtype: torch.dtype | None = None) -> torch.Tensor:
        nh, hd, rank = self.nh, self.hd, self.rank
        table = ctx.block_table(call.cache)
        cache = ctx.caches[call.cache]
        projected = ops.linear(x, self.w_in, out_dtype=torch.float32)          # [T, nh*hd + rank (+ nh)]
        if call.writes_cache:
            # The latent's norm and its place in the pages, one kernel; nothing else is kept of a position.
            ops.qkv_pairs(projected[:, nh * hd: nh * hd + rank], 0, 1, rank, 0, None, None, self.latent_norm, self.eps,
                          None, 0, ctx.positions, ctx.token_row, cache, table, ctx.status, self.dtype)
        q_latent = ops.head_linear(projected[:, : nh * hd], self.w_q_to_latent)  # [T, nh * rank], the model's type
        attended = self.attend(q_latent, ctx, cache, table)
        gate = projected[:, nh * hd + rank:] if self.has_gate else None
        heads_out = ops.head_linear(attended, self.w_latent_to_v, gate=gate)     # [T, nh * vd]
        return ops.linear(heads_out, self.w_o, out_dtype=out_dtype)

    def attend(self, q: torch.Tensor, ctx: StepContext, cache: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        """Attention of the latent-space queries [T, heads * rank] over the cached latents: rows with one
        new token on the split-context kernel, rows with several on the tensor-core prompt kernel, where
        those take this shape and type; whatever is left on the general kernel."""
        out = torch.empty_like(q)
        common = (self.nh, 1, self.rank, 0, self.scale, ctx.status)
        decode_done = self.fast_decode and ctx.num_decode_rows > 0
        if decode_done:
            ops.paged_decode(q, cache, table, ctx.decode_rows, ctx.row_q_start, ctx.row_ctx, ctx.max_decode_context,
                             *common, out=out, sinks=self.sinks, keys_only=True)
        prefill_done = False
        if self.fast_prefill:
            tile_row, tile_q0 = ctx.tiles[(self.prefill_tile_tokens, "multi")]
            prefill_done = True
            if tile_row.numel() > 0:
                ops.paged_prefill(q, cache, table, tile_row, tile_q0, ctx.row_q_start, ctx.row_q_len, ctx.row_ctx,
                                  *common, out=out, sinks=self.sinks, keys_only=True)
        if decode_done and prefill_done:
            return out
        which = "multi" if decode_done else ("single" if prefill_done else "all")
        tile_row, tile_q0 = ctx.tiles[(self.tile_tokens, which)]
        if tile_row.numel() > 0:
            ops.paged_attention(q, cache, table, tile_row, tile_q0, self.tile_tokens, ctx.row_q_start, ctx.row_q_len,
                                ctx.row_ctx, *common, out=out, sinks=self.sinks, shared_kv=True)
        return out


register_mixer("latent_attention", LatentAttention)
