"""Grouped-query attention with an optional sliding window.

norm'd tokens -> q, k, v (one stacked product) -> position encoding, keys and values
into the cache -> attention over the cache -> output projection added to the residual
(reference: crates/braidinfer-runtime/src/megakernel/compile_attention.rs:79-126, 275-351;
softmax in kernels/megakernel_ops.hip:2310-2342).  Head h reads kv head h // g.  Key j is
visible to the query at position p iff j <= p and (no window or p - j < window); the
reference has no window (crates/braidinfer-runtime/src/config.rs:416).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .base import MIXERS, POSITION_ENCODINGS, Mixer
from .linear import Linear
from .spec import CacheRequest, PartSpec, TensorSpec


@MIXERS.register("gqa_attention")
class GQAAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, window (int | None),
    position_encoding (PartSpec), and tensor names q_proj, k_proj, v_proj, o_proj."""

    def __init__(self, params, prefix, runtime) -> None:
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nqh = int(p["num_heads"])
        self.nkh = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.window = p.get("window")
        if self.nqh % self.nkh:
            raise ValueError(f"{self.nqh} query heads do not divide into {self.nkh} kv heads")
        pe: PartSpec = p["position_encoding"]
        self.pe = POSITION_ENCODINGS.get(pe.kind)(pe.params, prefix, runtime)
        self.qkv = Linear(runtime, [prefix + p.get("q_proj", "self_attn.q_proj.weight"),
                                    prefix + p.get("k_proj", "self_attn.k_proj.weight"),
                                    prefix + p.get("v_proj", "self_attn.v_proj.weight")],
                          [self.nqh * self.hd, self.nkh * self.hd, self.nkh * self.hd], self.hidden)
        self.o = Linear(runtime, [prefix + p.get("o_proj", "self_attn.o_proj.weight")], [self.hidden],
                        self.nqh * self.hd)
        self.scale = 1.0 / math.sqrt(self.hd)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = dict(self.qkv.tensor_specs())
        d.update(self.o.tensor_specs())
        d.update(self.pe.tensor_specs())
        return d

    def load(self, tensors) -> None:
        self.qkv.load(tensors)
        self.o.load(tensors)
        self.pe.load(tensors)

    def cache_request(self) -> Optional[CacheRequest]:
        kind = "window" if self.window else "full"
        return CacheRequest(kind, self.nkh, self.hd, self.window)

    def takes_row_scale(self) -> bool:
        return self.qkv.takes_row_scale()

    def forward(self, x, residual, ctx, cache, state):
        if cache is None:
            raise RuntimeError("gqa_attention needs a cache view")
        rt = self.rt
        fused = self.pe.accepts_deferred
        qkv = self.qkv.forward(x, defer_to=ctx if fused else None, in_scale=ctx.take_row_scale(x))
        self.pe.encode_and_store(qkv, self.nqh, self.nkh, ctx, cache)
        rows = x.shape[0]
        out = rt.empty(rows, self.nqh * self.hd)
        self._attend(qkv, out, ctx, cache)
        return self.o.forward(out, residual=residual, defer_to=ctx)

    def _attend(self, qkv, out, ctx, cache) -> None:
        """Pick the attention kernel for this step.  float32 runs, and runs that ask for
        the plain kernels, use the one-warp-per-query kernel for everything.  bfloat16
        runs use the tcgen05 kernel for prompts (head sizes 64 and 128; "mma" as the
        backend keeps them on the mma.sync kernel, which also serves every other head
        size), and the mma.sync kernel with the context sliced for steps of few tokens,
        so that a handful of sequences still fills the machine."""
        K = self.rt.kernels
        plain = (self.rt.is_f32 or self.rt.attention_backend == "plain" or not K.attn_mma_supports(self.hd))
        if plain:
            K.attn_simple(qkv, out, cache.storage, cache.page_table, ctx.positions, ctx.token_seq,
                          self.nqh, self.nkh, self.hd, cache.page_size, self.window, self.scale)
            return
        few = ctx.max_q_len <= 8
        if not few and self.rt.attention_backend == "auto" and K.attn_tc_supports(self.hd):
            K.attn_tc(qkv, out, cache.storage, cache.page_table, ctx.q_start, ctx.q_len, ctx.kv_before,
                      ctx.n_seqs, ctx.max_q_len, self.nqh, self.nkh, self.hd, self.window, self.scale)
            return
        n_splits = 1
        if few:
            g = self.nqh // self.nkh
            ctas = ctx.n_seqs * self.nkh * -(-g // 16)
            span = min(ctx.max_kv_len, self.window) if self.window else ctx.max_kv_len
            tiles = max(1, -(-span // 32))
            # one wave of CTAs over the device, and at least four key tiles a slice
            n_splits = max(1, min(K.attn_decode_slots(self.hd) // ctas, tiles // 4, 64))
        K.attn_mma(qkv, out, cache.storage, cache.page_table, ctx.q_start, ctx.q_len, ctx.kv_before, ctx.token_seq,
                   ctx.n_seqs, ctx.max_q_len, self.nqh, self.nkh, self.hd, self.window, self.scale,
                   n_splits=n_splits, few_tokens=few)
