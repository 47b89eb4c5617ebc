"""Loading a model's tensors by name.

What is asked for comes from the parts (`DecoderModel.tensor_specs`); what is there
comes from the folder.  The two are compared before anything is copied, and every
difference that stops the load is reported in one error: missing tensors, wrong
shapes, wrong kinds of element (the reference reports them one at a time and panics
on a size mismatch, crates/braidinfer-runtime/src/weights.rs:229-236, :301-307).
Tensors that the folder holds and no part asks for (older exports store
``...rotary_emb.inv_freq``, for one) do not stop it: they are listed in one
`UnexpectedTensorsWarning` and in the error, if there is one; `strict=True` makes
them an error of their own.

Names: the parts ask for the names Mistral model folders use.  A folder that stores the same
tensors under one more prefix (a model wrapped into a larger one: ``language_model.model.layers.0...``)
is found by the reference through the text before ``layers.0.`` in any tensor name
(crates/braidinfer-runtime/src/model/model_load.rs:219-239); here the same discovery runs when
asked-for names are missing: if every one of them is there under one common prefix, that prefix
is used.

Element types: floating tensors stored in 16 bits are kept in bfloat16, a tensor
stored in 32 bits stays float32, integer tables become int32.  A float32 run widens
everything floating to float32 (exactly; bfloat16 -> float32 loses nothing).  A
float16 tensor in a bfloat16 run is rounded to bfloat16 (8 mantissa bits for its
11), which one `RoundedWeightsWarning` per load says.
"""
from __future__ import annotations

import warnings
from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..parts.spec import TensorSpec
from .safetensors_io import open_model_folder


class WeightsError(ValueError):
    """The folder's tensors do not fit the model.  Attributes list what is wrong."""

    def __init__(self, folder: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: List[Tuple[str, str]] = ()) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"{folder}: the stored tensors do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong element type ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {dt}" for n, dt in self.wrong_dtype))
        super().__init__("\n".join(lines))


class UnexpectedTensorsWarning(UserWarning):
    """The folder holds tensors that no part of the model asks for; they were not loaded."""


class RoundedWeightsWarning(UserWarning):
    """Tensors stored in float16 were rounded to bfloat16 for a bfloat16 run."""


def target_dtype(stored: torch.dtype, spec: TensorSpec, run_dtype: torch.dtype) -> torch.dtype:
    if spec.integer or not stored.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def discover_prefix(found_names, specs: Mapping[str, TensorSpec]) -> str:
    """The prefix P under which most of the asked-for, non-optional names are stored as P + name,
    or "" when no prefix holds more of them than the names as they are.  Candidates are the texts
    before an asked-for first-layer name inside a stored name (model_load.rs:219-239 takes the
    text before "layers.0."; a candidate with "mtp" in it, a draft head, comes last there and here)."""
    names = set(found_names)
    required = [n for n, s in specs.items() if not s.optional]
    anchors = [n for n in required if "layers.0." in n] or required[:1]
    candidates = []
    for stored in found_names:
        for a in anchors:
            if stored.endswith(a) and len(stored) > len(a):
                p = stored[:-len(a)]
                if p not in candidates:
                    candidates.append(p)
    candidates.sort(key=lambda p: ("mtp" in p, len(p)))
    best, best_hits = "", sum(n in names for n in required)
    for p in candidates:
        hits = sum(p + n in names for n in required)
        if hits > best_hits:
            best, best_hits = p, hits
    return best


def load_tensors(folder: str, specs: Mapping[str, TensorSpec], run_dtype: torch.dtype,
                 device, strict: bool = False) -> Dict[str, torch.Tensor]:
    """Check the folder against `specs`, then copy every asked-for tensor to `device`.
    `strict`: tensors nobody asks for are an error instead of a warning."""
    found = open_model_folder(folder)
    if any(n not in found and not s.optional for n, s in specs.items()):
        prefix = discover_prefix(list(found), specs)
        if prefix:                       # the same tensors under one more prefix: look them up there
            found = {(n[len(prefix):] if n.startswith(prefix) else n): v for n, v in found.items()}
    missing = [n for n, s in specs.items() if n not in found and not s.optional]
    unexpected = [n for n in found if n not in specs]
    wrong_shape, wrong_dtype = [], []
    for n, s in specs.items():
        if n not in found:
            continue
        f, key = found[n]
        dt, shape = f.info(key)
        if tuple(shape) != tuple(s.shape):
            wrong_shape.append((n, tuple(shape), tuple(s.shape)))
        if s.integer == dt.is_floating_point:
            wrong_dtype.append((n, str(dt)))
    if missing or wrong_shape or wrong_dtype or (strict and unexpected):
        raise WeightsError(folder, missing, unexpected, wrong_shape, wrong_dtype)
    if unexpected:
        warnings.warn(f"{folder}: {len(unexpected)} stored tensors are asked for by no part of the model and were "
                      f"not loaded: " + ", ".join(unexpected), UnexpectedTensorsWarning, stacklevel=2)
    rounded: List[str] = []
    out: Dict[str, torch.Tensor] = {}
    for n, s in specs.items():
        if n not in found:
            continue
        f, key = found[n]
        t = f.tensor(key)
        want = target_dtype(t.dtype, s, run_dtype)
        if t.dtype == want:
            out[n] = t.to(device, copy=True)
        else:
            # convert on the device: the host copy stays a view of the mapped file
            if t.dtype == torch.float16 and want == torch.bfloat16:
                rounded.append(n)
            out[n] = t.to(device).to(want)
    if rounded:
        warnings.warn(f"{folder}: {len(rounded)} tensors stored in float16 were rounded to bfloat16 "
                      f"(first: {rounded[0]}); run with dtype float32 to keep every stored bit",
                      RoundedWeightsWarning, stacklevel=2)
    return out
