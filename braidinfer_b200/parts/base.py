"""Interfaces of the parts a layer is made of, and the registries that map a
part's name to its class.

A part gets its sizes and constants as parameters, the prefix of its tensor
names, and the runtime (dtype, device, kernels).  It never learns which model
it belongs to.  A new part is a subclass registered under a new name; the
model description (`PartSpec.kind`) then picks it layer by layer.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Type

import torch

from .spec import CacheRequest, PartSpec, TensorSpec


class Part:
    """Common base: tensors in, nothing else assumed."""

    # A part whose forward reads the step's host-side fields, or otherwise does work that
    # a CUDA graph cannot replay, sets this to False; the engine then launches every
    # step kernel by kernel.
    graph_safe = True

    # A part that can finish a deferred sum inside its own kernel (see StepContext.deferred)
    # says so here; every other part is handed tensors that are already complete.
    accepts_deferred = False

    def takes_row_scale(self) -> bool:
        """A mixer or feed-forward that looks up `ctx.take_row_scale(x)` for its input and applies the
        scale it finds (see StepContext.row_scales) answers True; only then is it ever handed rows whose
        norm is not complete."""
        return False

    def __init__(self, params: dict, prefix: str, runtime) -> None:
        self.params = dict(params)
        self.prefix = prefix
        self.rt = runtime

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        """Full tensor names (prefix included) that the part needs, with shapes."""
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take the device tensors named by `tensor_specs` (already in run dtype)."""


class Norm(Part):
    def forward(self, x: torch.Tensor, ctx, row_index: Optional[torch.Tensor] = None,
                rows: Optional[int] = None) -> torch.Tensor:
        """x: residual stream [rows, width] float32 -> normalised rows in the run dtype.

        As a layer's norm it is called with (x, ctx) and returns every row.  As the model's
        final norm it is called with `row_index` (int32 on the device) and `rows`: it then
        returns the `rows` rows x[row_index[i]] only, normalised, and leaves x as it is.

        A norm with `accepts_deferred` is also passed `reader_takes_row_scale=` by the block: if
        true, it may return its rows without their scale and register the scale with
        `ctx.set_row_scale(out, scale)` for the reader to apply (StepContext.row_scales)."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Holds the constants of a position encoding.  A mixer that keeps keys and values hands
    it the step's stacked q, k, v rows; it encodes queries and keys and stores keys and
    values, so that a cached key is encoded exactly once."""

    def encode_and_store(self, qkv: torch.Tensor, nqh: int, nkh: int, ctx, cache) -> None:
        """qkv: [rows, (nqh + 2 nkh) * head_dim] in the run dtype, query heads first, then key
        heads, then value heads.  Encode the query and key heads in place using
        `ctx.positions`, then write each row's keys and values into `cache` (a LayerCache)
        at its position; `cache` None or read-only: no write.  Rows with ctx.token_seq < 0
        are padding.  `ctx.take_deferred(qkv)` tells whether qkv still waits for a deferred
        sum; only a part with `accepts_deferred` is ever handed such a tensor."""
        raise NotImplementedError


class Mixer(Part):
    """Mixes information across the tokens of a sequence (attention, or a
    recurrence with state)."""

    def cache_request(self) -> Optional[CacheRequest]:
        """Keys/values the mixer wants kept, or None."""
        return None

    def state_bytes(self) -> int:
        """Bytes of fixed-size state per sequence (zeroed when a slot is taken)."""
        return 0

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache, state) -> torch.Tensor:
        """x: normed tokens [rows, width] (run dtype); residual: [rows, width] float32.

        Returns residual + mix(x) as float32 (it may write into `residual`).  A built-in
        mixer may leave the last sum to the next norm (`ctx.defer`, see
        StepContext.deferred); whoever needs the value at once calls `ctx.resolve(t)`.
        `cache` is this run's `LayerCache` view or None; `state` is a uint8
        tensor [slots, state_bytes] for this layer or None.  Rows are the
        step's tokens packed sequence after sequence, padded rows last.
        """
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> torch.Tensor:
        """Returns residual + f(x), float32, rows independent of one another."""
        raise NotImplementedError


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor, rows: int) -> torch.Tensor:
        """token_ids [rows] int32 on the device -> the residual stream [rows, width], float32."""
        raise NotImplementedError


class Head(Part):
    """The output head.  If it has an attribute `tied` that is true after `load`, the model
    calls `tie(embedding.weight)` so that it can use the embedding table."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [wanted rows, width] (the final norm's output) -> logits [wanted rows, vocab], float32."""
        raise NotImplementedError


class Block:
    """The arrangement of a layer's parts.  `forward(h, ctx, cache, state) -> h` runs them on
    the float32 residual stream; `cache` and `state` are the mixer's (see Mixer.forward).
    h may arrive with a deferred sum pending (`ctx.deferred`): hand it only to a part with
    `accepts_deferred`, else call `ctx.resolve(h)` first."""

    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: Optional[FeedForward],
                 feed_forward_norm: Optional[Norm]) -> None:
        self.mixer = mixer
        self.mixer_norm = mixer_norm
        self.feed_forward = feed_forward
        self.feed_forward_norm = feed_forward_norm

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
                if p is not None]

    def forward(self, h: torch.Tensor, ctx, cache, state) -> torch.Tensor:
        raise NotImplementedError


class Registry:
    """Name -> class, with a clear error that lists what is known."""

    def __init__(self, what: str) -> None:
        self.what = what
        self._items: Dict[str, type] = {}

    def register(self, name: str, cls: Optional[type] = None):
        def put(c):
            self._items[name] = c
            return c
        return put(cls) if cls is not None else put

    def unregister(self, name: str) -> None:
        self._items.pop(name, None)

    def get(self, name: str) -> type:
        if name not in self._items:
            raise KeyError(f"unknown {self.what} '{name}'; known: {sorted(self._items)}")
        return self._items[name]

    def names(self):
        return sorted(self._items)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
