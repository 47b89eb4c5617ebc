"""What every part needs to run: the element type of activations, the device and
the kernel library.  The residual stream and the logits are float32 in every mode."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch


@dataclass
class Runtime:
    act_dtype: torch.dtype                 # torch.bfloat16 or torch.float32
    device: torch.device
    kernels: Any                           # braidinfer_b200.csrc.api.Kernels
    # "auto": tensor-core kernels where they apply; "plain": the simple kernels only
    # (tests compare the two).
    gemm_backend: str = "auto"
    attention_backend: str = "auto"
    # Let products of a few tokens leave their partial sums to the next norm or to the
    # rotary encoding, which add them up in their own kernel (fewer launches per step).
    fuse_reduce: bool = True
    # In steps of up to 128 tokens, let an RMSNorm leave its scale to the product that reads its output
    # (csrc/rowscale.cuh), so that the kernel before it works on parts of rows instead of whole rows.
    scaled_norm: bool = True

    @property
    def is_f32(self) -> bool:
        return self.act_dtype == torch.float32

    def empty(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(*shape, dtype=dtype or self.act_dtype, device=self.device)
