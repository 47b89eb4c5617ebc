"""Rotary position encoding, fused with the write of keys and values into the cache.

inv_freq[p] = theta^(-2p/rd) (reference: crates/braidinfer-runtime/src/weights.rs:743-751);
each pair (a, b) of a head becomes (a cos - b sin, a sin + b cos) with angle
pos * inv_freq[p] (kernels/megakernel_ops.hip:2019-2030).  The pair is (x[2p], x[2p+1])
for pairing "adjacent", as in that kernel, or (x[p], x[p + rd/2]) for "half".  Keys are
rotated once, before they are stored; attention never rotates a cached key again.
Angles, sine and cosine are float32.
"""
from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, PositionEncoding


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding(PositionEncoding):
    """params: head_dim, theta, rope_dim (default head_dim), pairing ("half" | "adjacent")."""

    accepts_deferred = True      # adds a deferred q/k/v product in the same kernel as the rotation
    # ... in steps of up to this many rows.  That kernel runs a small CTA per row and head, which saves a
    # launch in a chain of few rows and loses to reduce kernel + rotation kernel beyond (8 layers of the 7B
    # sizes: 1.036 against 1.043 ms at 64 rows, 1.125 against 1.118 at 80, 1.56 against 1.42 at 256).
    FUSED_REDUCE_MAX_ROWS = 64

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        self.head_dim = int(params["head_dim"])
        self.rope_dim = int(params.get("rope_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.pairing = params.get("pairing", "half")
        if self.pairing not in ("half", "adjacent"):
            raise ValueError(f"rope pairing must be 'half' or 'adjacent', got {self.pairing!r}")
        if self.rope_dim % 2 or not (0 <= self.rope_dim <= self.head_dim):
            raise ValueError(f"rope_dim={self.rope_dim} must be even and within head_dim={self.head_dim}")
        p = torch.arange(self.rope_dim // 2, dtype=torch.float64)
        inv = 1.0 / (self.theta ** (2.0 * p / self.rope_dim))
        self.inv_freq = inv.to(torch.float32).to(runtime.device)

    def encode_and_store(self, qkv: torch.Tensor, nqh: int, nkh: int, ctx, cache) -> None:
        """Rotate the query and key heads of qkv [rows, (nqh + 2 nkh) * hd] in place and
        write keys and values into `cache` (a LayerCache, or None / read-only: no write)."""
        writable = cache is not None and not cache.read_only
        if qkv.shape[0] > self.FUSED_REDUCE_MAX_ROWS:
            ctx.resolve(qkv)
        d = ctx.take_deferred(qkv)
        if d is not None:
            handle, kind = d
            if kind != "store" or qkv.dtype != torch.bfloat16:
                raise RuntimeError("the rotary encoding can only complete a deferred bfloat16 product")
            self.rt.kernels.streamk_reduce_rope_kv(
                handle, qkv, self.inv_freq, ctx.positions, ctx.token_seq,
                cache.page_table if writable else None, cache.storage if writable else None,
                nqh, nkh, self.head_dim, self.rope_dim, self.pairing == "adjacent",
                cache.page_size if cache is not None else 1)
            return
        self.rt.kernels.rope_kv_write(
            qkv, self.inv_freq, ctx.positions, ctx.token_seq,
            cache.page_table if writable else None, cache.storage if writable else None,
            nqh, nkh, self.head_dim, self.rope_dim, self.pairing == "adjacent",
            cache.page_size if cache is not None else 1)


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(RotaryEncoding):
    """No position information in queries and keys: they pass through as the projections made
    them, and keys and values are stored.  (The rotation of zero elements: the same kernels.)
    params: head_dim."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__({"head_dim": params["head_dim"], "theta": 1.0, "rope_dim": 0}, prefix, runtime)
