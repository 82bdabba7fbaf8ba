"""Typed configuration of LFM2 (Lfm2ForCausalLM), read from its config.json keys.

The reference reads the same facts from a model file's metadata
(imparo-model/src/lfm2/plan.rs:34-46 sizes and constants, :47-52 taps >= 2,
:54-63 head size = width / heads, :65-80 per-layer mixer kind and one GQA ratio,
:82-84 optional sliding window on the attention blocks, :163-169 tied head).
Nothing here is a model size: every number comes from config.json.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional, Tuple

from .base import ConfigError, KeyReader

LAYER_KINDS = ("conv", "full_attention", "sliding_attention")


@dataclass(frozen=True)
class Lfm2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    layer_types: Tuple[str, ...]
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    conv_L_cache: int
    conv_bias: bool
    block_ff_dim: int
    block_auto_adjust_ff_dim: bool
    block_ffn_dim_multiplier: Optional[float]
    block_multiple_of: int
    rope_theta: float
    norm_eps: float
    tie_embedding: bool
    max_position_embeddings: int
    sliding_window: Optional[int]
    layer_schedule: Optional[Tuple[Tuple[int, Optional[int]], ...]]
    eos_token_ids: Tuple[int, ...]

    @property
    def ff_dim(self) -> int:
        """Feed-forward width.  With block_auto_adjust_ff_dim: int(2F/3), times the
        multiplier when given, rounded up to block_multiple_of; else block_ff_dim as is.
        (The reference reads the final width directly, plan.rs:36.)"""
        f = self.block_ff_dim
        if self.block_auto_adjust_ff_dim:
            f = int(2 * f / 3)
            if self.block_ffn_dim_multiplier is not None:
                f = int(self.block_ffn_dim_multiplier * f)
            m = self.block_multiple_of
            f = m * ((f + m - 1) // m)
        return f

    def to_json_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = asdict(self)
        d["layer_types"] = list(self.layer_types)
        d.pop("eos_token_ids")
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.layer_schedule is None:
            d.pop("layer_schedule")
        else:
            d["layer_schedule"] = [list(e) for e in self.layer_schedule]
        for k in ("sliding_window", "block_ffn_dim_multiplier"):
            if d[k] is None:
                d.pop(k)
        d["architectures"] = ["Lfm2ForCausalLM"]
        d["model_type"] = "lfm2"
        return d


def parse_lfm2_config(values: dict) -> Lfm2Config:
    r = KeyReader(values)
    n_layers = r.integer("num_hidden_layers", minimum=1)
    layer_types = r.strings("layer_types", default=None)
    if layer_types is None:
        full = r.integers("full_attn_idxs", default=None)
        if full is None:
            raise ConfigError("config.json: missing required key 'layer_types' (also accepted: full_attn_idxs)")
        layer_types = tuple("full_attention" if i in set(full) else "conv" for i in range(n_layers))
    if len(layer_types) != n_layers:
        raise ConfigError(f"config.json: layer_types has {len(layer_types)} entries but num_hidden_layers is {n_layers}")
    for i, k in enumerate(layer_types):
        if k not in LAYER_KINDS:
            raise ConfigError(f"config.json: layer_types[{i}] is '{k}'; known kinds: {', '.join(LAYER_KINDS)}")

    hidden = r.integer("hidden_size", minimum=1)
    heads = r.integer("num_attention_heads", minimum=1)
    kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)
    head_dim = r.integer("head_dim", default=None)
    if head_dim is None:
        if hidden % heads != 0:
            raise ConfigError(f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads {heads}")
        head_dim = hidden // heads
    if heads % kv_heads != 0:
        raise ConfigError(f"config.json: num_key_value_heads {kv_heads} does not divide num_attention_heads {heads}")
    if head_dim < 2 or head_dim % 2 != 0:
        raise ConfigError(f"config.json: head size {head_dim} must be even (rotation pairs dimension i with i + head/2)")
    taps = r.integer("conv_L_cache", minimum=2)     # a 1-tap conv carries no state (plan.rs:47-52)

    window = r.integer("sliding_window", default=None)
    if "sliding_attention" in layer_types and (window is None or window < 1):
        raise ConfigError("config.json: layer_types names 'sliding_attention' but 'sliding_window' is missing or < 1")

    sched = values.get("layer_schedule")
    schedule = None
    if sched is not None:
        try:
            schedule = tuple((int(e[0]), None if e[1] is None else int(e[1])) if isinstance(e, (list, tuple))
                             else (int(e), None) for e in sched)
        except (TypeError, ValueError, IndexError):
            raise ConfigError("config.json: layer_schedule must be a list of layer indices or [layer, cache_from] pairs") from None

    eos = r.integers("eos_token_id", default=())
    return Lfm2Config(
        vocab_size=r.integer("vocab_size", minimum=1),
        hidden_size=hidden,
        num_hidden_layers=n_layers,
        layer_types=tuple(layer_types),
        num_attention_heads=heads,
        num_key_value_heads=kv_heads,
        head_dim=head_dim,
        conv_L_cache=taps,
        conv_bias=r.boolean("conv_bias", default=False),
        block_ff_dim=r.integer("block_ff_dim", "intermediate_size", minimum=1),
        block_auto_adjust_ff_dim=_auto_adjust(r),
        block_ffn_dim_multiplier=r.number("block_ffn_dim_multiplier", default=None),
        block_multiple_of=r.integer("block_multiple_of", default=256, minimum=1),
        rope_theta=_rope_theta(r),
        norm_eps=r.number("norm_eps", "rms_norm_eps", default=1e-5),
        tie_embedding=r.boolean("tie_embedding", "tie_word_embeddings", default=True),
        max_position_embeddings=r.integer("max_position_embeddings", default=128000, minimum=1),
        sliding_window=window,
        layer_schedule=schedule,
        eos_token_ids=tuple(eos or ()),
    )


def _auto_adjust(r: KeyReader) -> bool:
    """block_auto_adjust_ff_dim has no default here: the feed-forward width follows from it, writers
    of config.json do not agree on what an absent key means, and a guess would show up only as
    wrong-shape weights (or, with random weights, as another model).  The key must be there."""
    v = r.raw("block_auto_adjust_ff_dim")
    if v is None:
        raise ConfigError("config.json: missing required key 'block_auto_adjust_ff_dim' (true: the feed-forward width is "
                          "block_ff_dim * 2/3, times block_ffn_dim_multiplier, rounded up to block_multiple_of; "
                          "false: block_ff_dim as it is)")
    return r.boolean("block_auto_adjust_ff_dim")


def _rope_theta(r: KeyReader) -> float:
    rp = r.raw("rope_parameters")
    if isinstance(rp, dict) and "rope_theta" in rp and "rope_theta" not in r.values:
        return float(rp["rope_theta"])
    return r.number("rope_theta", default=10000.0)
