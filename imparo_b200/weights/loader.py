"""Loads a model's tensors by name from model.safetensors and checks them against what
the model's parts declare.

Like the reference's resolver, a tensor is found by name and a failure names the tensor
(imparo-model/src/cpu_support.rs:97-175: missing by name, unsupported dtype by name,
"refusing to load rather than silently misread").  Here every problem of a file is
collected into ONE error: missing tensors, unexpected tensors, wrong shapes, unreadable
dtypes.

dtypes kept: "matrix" tensors become bfloat16 in the bfloat16 path and float32 in the
32-bit path; "vector" tensors (norm weights, conv taps, biases) are always float32;
"int_table" tensors are int32.
"""
from __future__ import annotations

import os
from typing import Dict, Iterable, List

import torch

from ..parts.spec import WeightSpec
from .safetensors_io import SafetensorsFile

_FLOAT_STORED = {"F32", "BF16", "F16", "F64"}
_INT_STORED = {"I32", "I64", "I16", "I8", "U8"}


class WeightError(ValueError):
    """The model file does not hold what the model needs; the message lists everything."""

    def __init__(self, path, missing=(), unexpected=(), wrong_shape=(), bad_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.bad_dtype = list(bad_dtype)
        lines = [f"{path}: the tensors do not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, found, expected in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(found)}, expected " + " or ".join(str(list(s)) for s in expected))
        for name, dt, why in self.bad_dtype:
            lines.append(f"  unreadable dtype: {name} is {dt} ({why})")
        super().__init__("\n".join(lines))


def _aliases(name: str) -> List[str]:
    """A tensor may be stored with or without the "model." prefix."""
    out = [name]
    if name.startswith("model."):
        out.append(name[len("model."):])
    else:
        out.append("model." + name)
    return out


def target_dtype(role: str, precision: str) -> torch.dtype:
    if role == "matrix":
        return torch.bfloat16 if precision == "bfloat16" else torch.float32
    if role == "vector":
        return torch.float32
    if role == "int_table":
        return torch.int32
    raise ValueError(f"unknown tensor role '{role}'")


def load_weights(folder: str, specs: Iterable[WeightSpec], precision: str, device,
                 duplicates: Dict[str, str] = None) -> Dict[str, torch.Tensor]:
    """-> {spec name: device tensor}.  Raises WeightError listing every mismatch.

    duplicates: {stored name: spec name} for tensors a file may carry although the model reads them
    under another name (a tied head written out beside the embedding table).  Such a tensor is not
    "unexpected" when it equals the one it duplicates; when it differs, it is reported as a wrong
    tensor, since the model would silently ignore it."""
    path = os.path.join(folder, "model.safetensors")
    if not os.path.isfile(path):
        if os.path.isfile(path + ".index.json"):
            raise FileNotFoundError(f"{folder}: the checkpoint is sharded (model.safetensors.index.json); sharded checkpoints "
                                    "are not read: merge the shards into one model.safetensors")
        raise FileNotFoundError(f"{folder}: no model.safetensors in this model folder")
    specs = list(specs)
    missing, wrong, bad = [], [], []
    out: Dict[str, torch.Tensor] = {}
    with SafetensorsFile(path) as f:
        stored = set(f.names())
        used = set()
        for w in specs:
            found = next((a for a in _aliases(w.name) if a in stored), None)
            if found is None:
                if not w.optional:
                    missing.append(w.name)
                continue
            used.add(found)
            dt, shape = f.info(found)
            if shape not in tuple(tuple(s) for s in w.shapes):
                wrong.append((w.name, shape, w.shapes))
                continue
            if w.role == "int_table":
                if dt not in _INT_STORED:
                    bad.append((w.name, dt, "an integer table is expected"))
                    continue
            elif dt not in _FLOAT_STORED:
                bad.append((w.name, dt, "float32, bfloat16 or float16 is expected"))
                continue
            t = f.tensor(found)
            out[w.name] = t.to(device=device, dtype=target_dtype(w.role, precision)).contiguous()
        for dup, name in (duplicates or {}).items():
            found = next((a for a in _aliases(dup) if a in stored and a not in used), None)
            orig = next((a for a in _aliases(name) if a in used), None)
            if found is None or orig is None:
                continue
            used.add(found)
            if f.info(found) != f.info(orig) or not torch.equal(f.tensor(found), f.tensor(orig)):
                bad.append((dup, f.info(found)[0], f"the model reads {name} in its place and the two differ"))
        unexpected = sorted(stored - used)
    if missing or unexpected or wrong or bad:
        raise WeightError(path, missing, unexpected, wrong, bad)
    return out
