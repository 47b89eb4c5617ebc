"""SwiGLU feed-forward: down( silu(gate x) * (up x) ), added to the residual
(reference: crates/braidinfer-runtime/src/megakernel/compile_layers.rs:373-386;
kernels/megakernel_ops.hip:1474-1545 gate/up with silu as x / (1 + exp(-x)),
:1559-1602 down with the residual).  Gate and up are one stacked product; on the
tensor-core path the activation is its epilogue."""
from __future__ import annotations

from typing import Dict

from .base import FEED_FORWARDS, FeedForward
from .linear import Linear
from .spec import TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size, tensor names gate_proj, up_proj, down_proj."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.gate_up = Linear(runtime, [prefix + p.get("gate_proj", "mlp.gate_proj.weight"),
                                        prefix + p.get("up_proj", "mlp.up_proj.weight")],
                              [self.inter, self.inter], self.hidden, gate_up=True)
        self.down = Linear(runtime, [prefix + p.get("down_proj", "mlp.down_proj.weight")], [self.hidden], self.inter)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.gate_up.tensor_specs())
        d.update(self.down.tensor_specs())
        return d

    def load(self, tensors) -> None:
        self.gate_up.load(tensors)
        self.down.load(tensors)

    def takes_row_scale(self) -> bool:
        return self.gate_up.takes_row_scale()

    def forward(self, x, residual, ctx):
        act = self.gate_up.forward(x, swiglu=True, in_scale=ctx.take_row_scale(x) if ctx is not None else None)
        return self.down.forward(act, residual=residual, defer_to=ctx)
