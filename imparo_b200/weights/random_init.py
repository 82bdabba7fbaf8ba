"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no such mode (its tests build plans in code and never weights,
imparo-model/src/lfm2/workflow_gpu.rs:2204-2261).  Distributions: matrices and the
embedding N(0, matrix_std); conv taps N(0, conv_std); biases N(0, matrix_std); norm weights
1 + U(-norm_jitter, norm_jitter) (norm_jitter 0 gives exactly 1).  One generator, seeded
once, drawn from in the order the model declares its tensors, always in float32 and
rounded to the stored dtype afterwards.
"""
from __future__ import annotations

import json
import os
from typing import Union

import torch

from ..config.registry import load_config
from ..parts.base import Runtime, Workspace
from ..parts.model import Model
from .safetensors_io import write_safetensors


def model_on_cpu(config: Union[dict, str]):
    """(architecture, typed config, Model with no weights) — for listing tensors."""
    arch, cfg = load_config(config)
    rt = Runtime(precision="float32", device=torch.device("cpu"), workspace=Workspace("cpu"))
    return arch, cfg, Model(arch.model_spec(cfg), rt)


def draw_random_tensors(specs, seed: int, dtype: str = "bfloat16", device="cpu", matrix_std: float = 0.02,
                        conv_std: float = 0.2, norm_jitter: float = 0.1):
    """name -> tensor on device, drawn in the order of specs from one generator seeded once."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    tensors = {}
    for w in specs:
        shape = tuple(w.shapes[0])
        kind = w.init[0]
        if kind == "skip":
            continue
        if kind == "norm":
            t = 1.0 + (torch.rand(shape, generator=gen, dtype=torch.float32, device=device) * 2.0 - 1.0) * float(norm_jitter)
        elif kind == "conv_taps":
            t = torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * float(conv_std)
        elif kind == "bias":
            t = torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * float(matrix_std)
        elif kind == "normal":
            t = torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * float(w.init[1] if len(w.init) > 1 else matrix_std)
        elif kind == "ones":
            t = torch.ones(shape, dtype=torch.float32, device=device)
        elif kind == "zeros":
            t = torch.zeros(shape, dtype=torch.float32, device=device)
        else:
            raise ValueError(f"tensor '{w.name}': unknown init '{kind}'")
        if w.role == "matrix" and dtype == "bfloat16":
            t = t.to(torch.bfloat16)
        elif w.role == "int_table":
            t = t.to(torch.int32)
        tensors[w.name] = t
    return tensors


def write_random_model(folder: str, config: dict, seed: int, dtype: str = "bfloat16", matrix_std: float = 0.02,
                       conv_std: float = 0.2, norm_jitter: float = 0.1) -> str:
    """config is a config.json dictionary of a registered architecture.  dtype is the stored
    dtype of matrices ("bfloat16" or "float32"); vectors are stored in float32."""
    if dtype not in ("bfloat16", "float32"):
        raise ValueError("dtype must be 'bfloat16' or 'float32'")
    arch, cfg, model = model_on_cpu(config)
    tensors = draw_random_tensors(model.weight_specs(), seed, dtype, "cpu", matrix_std, conv_std, norm_jitter)
    os.makedirs(folder, exist_ok=True)
    out_cfg = dict(config)
    out_cfg.setdefault("architectures", [arch.name])
    out_cfg["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(out_cfg, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      {"format": "pt", "seed": str(seed), "generator": "imparo_b200.random_init"})
    return folder
