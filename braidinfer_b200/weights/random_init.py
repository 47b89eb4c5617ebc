"""The random-weights mode: write a model folder (config.json, model.safetensors)
from a configuration and a seed.

Tensors are drawn on the CPU from one seeded generator in the order the model lists
them: matrices and the embedding N(0, 0.02), norm weights 1 + N(0, 0.02), drawn in
float32 and stored in bfloat16.  The same configuration and seed give the same bytes.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Optional

import torch

from ..models.decoder import DecoderModel
from ..models.registry import architecture_for
from ..parts.runtime import Runtime
from ..parts.spec import ModelSpec, TensorSpec
from .safetensors_io import save_file


def tensor_specs_of(spec: ModelSpec) -> "Mapping[str, TensorSpec]":
    """The tensors a model description needs (no device involved)."""
    rt = Runtime(act_dtype=torch.bfloat16, device=torch.device("cpu"), kernels=None)
    return DecoderModel(spec, rt).tensor_specs()


def draw_tensors(specs: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                 skip_optional: bool = False) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for name, ts in specs.items():
        if ts.optional and skip_optional:
            continue
        if ts.integer:
            raise ValueError(f"the random-weights mode cannot draw the integer table {name}")
        x = torch.randn(ts.shape, generator=g, dtype=torch.float32) * ts.std
        if ts.init == "one_plus_normal":
            x = x + 1.0
        elif ts.init != "normal":
            raise ValueError(f"unknown init {ts.init!r} for {name}")
        out[name] = x.to(dtype)
    return out


def write_random_model(config_dict: Mapping, folder: str, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Write `folder`/config.json and `folder`/model.safetensors for the architecture that
    `config_dict` names.  Returns the folder."""
    arch = architecture_for(config_dict)
    cfg = arch.config_from_dict(config_dict)
    spec = arch.build_spec(cfg)
    specs = tensor_specs_of(spec)
    tensors = draw_tensors(specs, seed, dtype)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(config_dict), f, indent=2)
    save_file(tensors, os.path.join(folder, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    return folder
