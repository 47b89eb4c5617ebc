"""Helpers shared by the GPU tests."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

import plain_mistral as P
from tiny import CONFIGS, SEEDS, TOL_BF16, TOL_F32, config_of, make_folder, read_weights

TOL = {"float32": TOL_F32, "bfloat16": TOL_BF16}


def sharpen(folder: str, gain: float = 6.0) -> str:
    """Scale every query and key projection so that attention is peaked: a missing or
    misplaced key then moves the logits by far more than any tolerance."""
    from braidinfer_b200.weights import open_model_folder, save_file
    tensors = {n: f.tensor(k).clone() for n, (f, k) in open_model_folder(folder).items()}
    for n in tensors:
        if n.endswith("q_proj.weight") or n.endswith("k_proj.weight"):
            tensors[n] = (tensors[n].float() * gain).to(tensors[n].dtype)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return folder


class Oracle:
    """Plain logits of whole sequences for one model folder, computed once per sequence."""

    def __init__(self, folder: str) -> None:
        self.cfg = config_of(folder)
        self.w = read_weights(folder)
        self._memo: Dict[Tuple[int, ...], torch.Tensor] = {}

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = P.forward_logits(self.w, self.cfg, list(tokens), torch.float64)
        return self._memo[key]


def engine(folder: str, dtype: str, **kw):
    from braidinfer_b200.engine import Engine
    kw.setdefault("max_tokens", 64 * 16)
    kw.setdefault("verbose", False)
    return Engine.from_folder(folder, dtype=dtype, **kw)


def max_err(got: torch.Tensor, want: torch.Tensor) -> float:
    return (got.double().cpu() - want.double()).abs().max().item()
