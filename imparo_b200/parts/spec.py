"""Data that describes a model before any weight exists.

A model is described the way the reference's plan describes one: per layer a mixer
kind with its geometry and a feed-forward kind, plus embedding and output plans
(imparo-model/src/lib.rs:90-141 Attention, :296-326 Ffn, :380-385 LayerPlan,
:401-417 EmbedPlan/OutputPlan, :446-467 ModelPlan).  Here every part is a
(kind, parameters) pair resolved through the part registry, and the order in which
layers run is a list of its own: an entry may name a layer a second time, or read
the cache an earlier entry wrote (the reference's LayerPlan.kv_source).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: which registered kind, and its sizes and constants."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged (block) and which parts they are.

    prefix is the layer's tensor-name prefix, e.g. "model.layers.3.".
    """
    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block: str = "prenorm_residual"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  cache_from names an EARLIER entry of the schedule whose
    cache this run reads instead of owning one (it then writes nothing there)."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()
    # (stored name, name the model reads): tensors a file may carry as a copy of another one (a tied head
    # written out beside the embedding table); the loader accepts them when they equal the original
    duplicate_tensors: Tuple[Tuple[str, str], ...] = ()

    def __post_init__(self):
        n = len(self.layers)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ValueError(f"schedule entry {i} names layer {e.layer}; the model has {n} layers")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ValueError(f"schedule entry {i}: cache_from must name an earlier entry, found {e.cache_from}")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {i}: cache_from names entry {e.cache_from}, which owns no cache")


# ---------------------------------------------------------------------------
# what a part asks of the cache manager
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class PagedKV:
    """Keys and values that grow with the sequence, kept in pages.

    window=None keeps every position; window=w keeps the last w positions a query
    can still see, and pages wholly behind that are given back.
    (imparo-kv/src/state.rs:16-21 StateKind::{Full, Window})"""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    @property
    def width(self) -> int:
        return self.n_kv_heads * self.head_dim


@dataclass(frozen=True)
class SlotState:
    """State of fixed size per request, zeroed when a request gets its slot
    (imparo-model/src/lib.rs:205-219 recurrent_layout; :1951-1972 reset at position 0).
    Always kept in 32-bit."""
    shape: Tuple[int, ...]


# ---------------------------------------------------------------------------
# weights a part asks of the loader
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class WeightSpec:
    """One tensor of the model file.

    role: "matrix" (bfloat16 in the bfloat16 path, 32-bit in the 32-bit path),
          "vector" (always 32-bit: norm weights, conv taps, biases),
          "int_table" (int32).
    shapes: accepted shapes; the first is the one the random-weights mode writes.
    init: ("normal", std) | ("one_plus_uniform", half_width) | ("ones",) | ("zeros",)
    """
    name: str
    shapes: Tuple[Tuple[int, ...], ...]
    role: str = "matrix"
    init: Tuple = ("normal", 0.02)
    optional: bool = False
