"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, plain w
(reference: kernels/megakernel_ops.hip:862-904; `1 + w` is another model family's rule,
crates/braidinfer-runtime/src/config.rs:552).  Reads the float32 residual stream, writes
the run's element type; the sum of squares and the scale are float32."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import NORMS, Norm
from .linear import ROW_SCALE_MAX_ROWS
from .spec import TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: width, eps, name (tensor name under the prefix)."""

    accepts_deferred = True      # adds a deferred residual sum in the same kernel as the norm

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.name = prefix + params["name"]
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.width,), init="one_plus_normal")}

    def load(self, tensors) -> None:
        self.weight = tensors[self.name]

    def forward(self, x: torch.Tensor, ctx=None, row_index: Optional[torch.Tensor] = None,
                rows: Optional[int] = None, reader_takes_row_scale: bool = False) -> torch.Tensor:
        n = rows if rows is not None else x.shape[0]
        out = self.rt.empty(n, self.width)
        d = ctx.take_deferred(x) if ctx is not None else None
        if (reader_takes_row_scale and self.rt.scaled_norm and ctx is not None and row_index is None and out.dtype == torch.bfloat16
                and n <= ROW_SCALE_MAX_ROWS and self.width % 4 == 0 and self.rt.gemm_backend == "auto"):
            # a step of few tokens: x is completed, `out` = x * weight, and the scale is left to the reader.
            # The kernel works on 512 columns of a row per CTA instead of on whole rows.
            if d is not None and d[1] != "residual":
                raise RuntimeError("a norm can only complete a deferred residual sum")
            ctx.set_row_scale(out, self.rt.kernels.streamk_reduce_prep(d[0] if d is not None else None, x, self.weight,
                                                                       out, self.eps))
            return out
        if d is not None:
            handle, kind = d
            if kind != "residual":
                raise RuntimeError("a norm can only complete a deferred residual sum")
            self.rt.kernels.streamk_reduce_norm(handle, x, self.weight, out, self.eps, row_index=row_index)
        else:
            self.rt.kernels.rmsnorm(x, self.weight, out, self.eps, row_index=row_index)
        return out
