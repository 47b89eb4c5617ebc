"""Token embedding and output head.

Embedding: h[t, :] = float(E[token_t, :]), no scale (reference:
kernels/megakernel_ops.hip:1757-1768).  Head: logits = W h in float32
(kernels/megakernel_ops.hip:1783-1835); W is lm_head.weight, or the embedding table
when the model ties them (crates/braidinfer-runtime/src/model/model_load.rs:388-398).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import EMBEDDINGS, HEADS, Embedding, Head
from .linear import Linear
from .spec import TensorSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    """params: vocab_size, hidden_size, name."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = prefix + params.get("name", "model.embed_tokens.weight")
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.vocab, self.hidden))}

    def load(self, tensors) -> None:
        self.weight = tensors[self.name]

    def forward(self, token_ids: torch.Tensor, rows: int) -> torch.Tensor:
        h = torch.empty((rows, self.hidden), dtype=torch.float32, device=self.rt.device)
        self.rt.kernels.embed(self.weight, token_ids, h)
        return h


@HEADS.register("linear_head")
class LinearHead(Head):
    """params: vocab_size, hidden_size, name, tied (use the embedding table)."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        # None: tied exactly when the model folder stores no head tensor.
        self.tied = params.get("tied", False)
        self.name = prefix + params.get("name", "lm_head.weight")
        self.linear = Linear(runtime, [self.name], [self.vocab], self.hidden)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        if self.tied:
            return {}
        specs = self.linear.tensor_specs()
        if self.tied is None:
            specs = {n: TensorSpec(ts.shape, optional=True) for n, ts in specs.items()}
        return specs

    def load(self, tensors) -> None:
        if self.tied is None:
            self.tied = self.name not in tensors
        if not self.tied:
            self.linear.load(tensors)

    def tie(self, embedding_weight: torch.Tensor) -> None:
        self.linear.share(embedding_weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear.forward(x, out_dtype=torch.float32)
