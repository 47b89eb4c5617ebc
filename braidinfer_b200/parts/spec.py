"""Data that describes a model: which parts each layer is made of, and the
order in which layers run.  A description holds names and numbers only; the
parts themselves are built from it by `braidinfer_b200.models.decoder`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: the name it is registered under and its sizes and constants."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (block) of a mixer, a feed-forward and norms.

    `prefix` is put before every tensor name the layer's parts ask for.
    """
    block: str
    prefix: str
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `cache_of` names an earlier schedule entry whose
    cache this run reads instead of keeping its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, the order they run in, final norm, head."""
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_position: int = 0                      # longest sequence the model is meant for (0: not stated)
    eos_token_ids: Tuple[int, ...] = ()        # tokens that end a sequence unless the caller names others
    bos_token_id: Optional[int] = None         # put before a text prompt by the command line

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, which does not exist")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(
                        f"schedule entry {i} reads the cache of entry {e.cache_of}, "
                        f"which must be an earlier entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(
                        f"schedule entry {i} reads the cache of entry {e.cache_of}, "
                        f"which has no cache of its own")


@dataclass(frozen=True)
class TensorSpec:
    """A tensor that a part needs from the model folder.

    `init` tells the random-weights mode how to draw it: "normal" is N(0, std),
    "one_plus_normal" is 1 + N(0, std).  `integer` marks index tables, which are
    kept as int32 whatever the run's dtype.
    """
    shape: Tuple[int, ...]
    init: str = "normal"
    std: float = 0.02
    integer: bool = False
    optional: bool = False


@dataclass(frozen=True)
class CacheRequest:
    """What a mixer needs kept for each sequence between steps.

    kind "full": keys and values of every past token; "window": of the last
    `window` tokens only.  Layers whose requests are equal share one group of
    storage.
    """
    kind: str
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self) -> Tuple:
        return (self.kind, self.num_kv_heads, self.head_dim, self.window)
