"""Interfaces of the parts a model is put together from, and the registry of part kinds.

A part knows its own sizes and constants (given as parameters) and nothing about the
model it is in.  Kinds:

  "mixer"        forward(x, batch, caches, residual)  adds its output into residual
  "feed_forward" forward(x, batch, residual)          adds its output into residual
  "norm"         forward(x, out=None, rows=None)      -> normed activations
  "position"     tables / apply for queries and keys
  "block"        forward(x, batch, caches, only_rows) arranges norm, mixer, feed-forward
  "embedding"    forward(batch)                       -> the 32-bit residual stream [tokens, width]
  "head"         forward(h)                           -> 32-bit logits

x is the normed input in the activation dtype (bfloat16, or float32 in the 32-bit
path); residual is the 32-bit residual stream [tokens, width].  batch is the step's
StepBatch.  caches is a tuple with one bound view per entry of the part's
cache_specs().

Every part declares the tensors it reads (weight_specs) and receives them already on
the device in the right dtype (bind).  Adding a kind is register_part(kind, name, cls);
nothing else in the framework changes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .spec import PartSpec, WeightSpec


@dataclass
class Runtime:
    """Engine-wide facts handed to every part when it is built."""
    precision: str                      # "bfloat16" | "float32"
    device: torch.device
    status: Optional[torch.Tensor] = None       # int32[4] device word kernels report bad indices into
    workspace: "Workspace" = None
    # Stage probe (the reference's IMPARO_PROBE_LAYER / IMPARO_GPU_PROBE, imparo-model/src/cpu_support.rs:26-46,
    # gpu_support.rs:202): when probe_entry names a schedule entry, that entry's block hands named
    # intermediates (whole tensors) to probe(name, tensor), so that two engines can be compared stage by stage.
    probe_entry: Optional[int] = None
    probe: Optional[object] = None
    probe_now: bool = False                     # set by the model while the probed entry runs
    # the launchers' bookkeeping and scratch of this engine (kernels/ops.py LaunchState); None: the module's default
    launch_state: Optional[object] = None

    @property
    def act_dtype(self) -> torch.dtype:
        return torch.bfloat16 if self.precision == "bfloat16" else torch.float32

    @property
    def matrix_dtype(self) -> torch.dtype:
        return self.act_dtype


class Workspace:
    """Activation scratch by tag.  A tag's buffer only ever grows (outside graph capture),
    so addresses are stable from step to step and never depend on which requests a step
    carries (the reference sizes activation buffers once per batch width,
    imparo-model/src/gpu_support.rs:557-715)."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}      # (tag, dtype, shape) -> view handed out before
        self.generation = 0      # bumped whenever a buffer moves: captured graphs of older generations are stale
        # the most tokens and the most wanted (or one-token) rows a step of this engine holds, when known: a buffer
        # whose first dimension is one of them is made for the most at once instead of growing step by step
        self.most = {"tokens": 0, "rows": 0, "context": 0}

    def expect(self, tokens: int = 0, rows: int = 0, context: int = 0) -> None:
        """tokens / rows: the most a step holds; context: the most positions a request reaches."""
        self.most["tokens"] = max(self.most["tokens"], int(tokens))
        self.most["rows"] = max(self.most["rows"], int(rows))
        self.most["context"] = max(self.most["context"], int(context))

    def get(self, tag: str, shape: Sequence[int], dtype: torch.dtype, first: Optional[str] = None,
            reserve: int = 0) -> torch.Tensor:
        """first: what the first dimension counts ("tokens" | "rows"), if it is one of the step's totals;
        reserve: elements to make room for at least (for buffers whose size follows no single dimension)."""
        shape = tuple(shape)
        seen = self._views.get((tag, dtype, shape))
        if seen is not None:
            return seen
        n = 1
        for s in shape:
            n *= int(s)
        key = (tag, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"workspace buffer '{tag}' would grow during graph capture")
            grown = max(n, 1, int(reserve))
            if first is not None and shape and shape[0] <= self.most.get(first, 0):
                grown = max(grown, n // max(int(shape[0]), 1) * self.most[first])
            # small buffers grow by doubling: every move makes captured graphs stale, and a serving loop
            # meets slightly larger shapes for a long while
            if buf is not None and grown * buf.element_size() <= (64 << 20):
                grown = max(grown, 2 * buf.numel())
            moved = buf is not None
            buf = torch.empty(grown, dtype=dtype, device=self.device)
            self._bufs[key] = buf
            if moved:                 # a buffer that did not exist is in no captured graph
                self.generation += 1
            self._views = {k: v for k, v in self._views.items() if k[:2] != key}
        view = buf[:n].view(*shape)
        if len(self._views) < 4096:
            self._views[(tag, dtype, shape)] = view
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


class Part:
    """Base of every part.  params are the PartSpec's parameters; prefix is the tensor-name
    prefix of the layer (or "" for model-level parts)."""

    # True when forward() takes everything that varies from step to step (tokens, positions,
    # tables, slots) from the batch's DEVICE arrays, so a step of single tokens can be captured
    # once and replayed.  A part that reads batch.host in forward() must set this to False.
    graph_safe = True
    # True when the part's LAST write to the residual is ops.linear(..., residual, accumulate=True)
    # (ops.add_bias after it is fine): that add may then stay split partials that the next norm folds in
    # (ops.allow_deferred_add).  A part that writes the residual any other way keeps False.
    adds_with_linear = False

    def __init__(self, params: dict, prefix: str, rt: Runtime):
        self.params = dict(params)
        self.prefix = prefix
        self.rt = rt

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """tensors: full tensor name -> device tensor, for the names of weight_specs()
        (optional ones absent when the file has none)."""

    def cache_specs(self) -> Tuple:
        return ()


class Block(Part):
    """Base of the "block" kind: how a layer's parts are arranged.  The model calls
    forward(x, batch, caches, only_rows=None) (x: the 32-bit stream, updated in place) and reads one declared fact:

    picks_rows: True when forward(only_rows=(rows, n)) is implemented: as the model's last block it may then
        run whatever follows its mixer on the n wanted rows only and return their stream [n, width]."""
    picks_rows = False

    def forward(self, x, batch, caches, only_rows=None):
        raise NotImplementedError


_PARTS: Dict[Tuple[str, str], type] = {}


def register_part(kind: str, name: str, cls: type, replace: bool = False) -> None:
    key = (kind, name)
    if key in _PARTS and not replace:
        raise ValueError(f"{kind} part '{name}' is already registered")
    _PARTS[key] = cls


def make_part(kind: str, spec: PartSpec, prefix: str, rt: Runtime) -> Part:
    _ensure_builtin()
    try:
        cls = _PARTS[(kind, spec.kind)]
    except KeyError:
        known = sorted(n for k, n in _PARTS if k == kind)
        raise ValueError(f"unknown {kind} part '{spec.kind}'; known: {', '.join(known)}") from None
    return cls(spec.params, prefix, rt)


def known_parts(kind: str) -> Tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(n for k, n in _PARTS if k == kind))


def _ensure_builtin() -> None:
    from . import builtin  # noqa: F401  (registers the built-in parts on import)
