"""A decoder put together from a `ModelSpec`: embedding, layers (blocks of parts),
the schedule in which they run, final norm and output head.  It knows parts only
through their interfaces and registries; nothing here is specific to one
architecture."""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS
from ..parts.spec import CacheRequest, ModelSpec, TensorSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime) -> None:
        spec.validate()
        self.spec = spec
        self.rt = runtime
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding.params, "", runtime)
        self.blocks = []
        for ls in spec.layers:
            mixer = MIXERS.get(ls.mixer.kind)(ls.mixer.params, ls.prefix, runtime)
            mixer_norm = NORMS.get(ls.mixer_norm.kind)(ls.mixer_norm.params, ls.prefix, runtime)
            ffn = ffn_norm = None
            if ls.feed_forward is not None:
                ffn = FEED_FORWARDS.get(ls.feed_forward.kind)(ls.feed_forward.params, ls.prefix, runtime)
                ffn_norm = NORMS.get(ls.feed_forward_norm.kind)(ls.feed_forward_norm.params, ls.prefix, runtime)
            self.blocks.append(BLOCKS.get(ls.block)(mixer, mixer_norm, ffn, ffn_norm))
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm.params, "", runtime)
        self.head = HEADS.get(spec.head.kind)(spec.head.params, "", runtime)

    # ------------------------------------------------------------------ weights
    def all_parts(self):
        yield self.embedding
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm
        yield self.head

    def tensor_specs(self) -> "OrderedDict[str, TensorSpec]":
        """Every tensor the model reads, in a fixed order (the random-weights mode
        draws them in this order)."""
        specs: "OrderedDict[str, TensorSpec]" = OrderedDict()
        for part in self.all_parts():
            for name, ts in part.tensor_specs().items():
                if name in specs and specs[name].shape != ts.shape:
                    raise ValueError(f"tensor {name} is asked for with two shapes: {specs[name].shape} and {ts.shape}")
                specs[name] = ts
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for part in self.all_parts():
            part.load(tensors)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.weight)

    # ------------------------------------------------------------------ cache plan
    def cache_plan(self) -> List[Tuple[Optional[CacheRequest], Optional[int], int]]:
        """Per schedule entry: what its mixer wants kept, whose cache it reads, state bytes."""
        plan = []
        for e in self.spec.schedule:
            mixer = self.blocks[e.layer].mixer
            plan.append((mixer.cache_request(), e.cache_of, int(mixer.state_bytes())))
        return plan

    # ------------------------------------------------------------------ one step
    def forward(self, ctx, cache, tap=None) -> Optional[torch.Tensor]:
        """Run the step's tokens through the schedule; return float32 logits
        [wanted rows, vocab] (None when nothing is wanted).  `tap(i, h)`, if given, is shown
        the float32 residual stream [rows, width] after the embedding (i = 0) and after
        schedule entry i - 1 (sums that a part left deferred are completed first)."""
        h = self.embedding.forward(ctx.token_ids, ctx.rows)
        if tap is not None:
            tap(0, h)
        for e, entry in enumerate(self.spec.schedule):
            view = cache.layer_view(e)
            if view is not None:
                view.page_table = ctx.page_tables[view.group]
            h = self.blocks[entry.layer].forward(h, ctx, view, cache.state_view(e))
            if tap is not None:
                tap(e + 1, ctx.resolve(h))
        if ctx.n_want == 0:
            ctx.drop_deferred()
            return None
        if not self.final_norm.accepts_deferred:
            ctx.resolve(h)
        x = self.final_norm.forward(h, ctx, row_index=ctx.want_rows, rows=ctx.n_want)
        return self.head.forward(x)
