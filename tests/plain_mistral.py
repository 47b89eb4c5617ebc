"""Plain, slow implementation of the Mistral decoder, for the tests only.

It rests on the reference's formulas, not on running the reference: the
reference is Rust + HIP for AMD GPUs and can be neither compiled nor imported
on this machine (no cargo, rustc, hipcc or ROCm), so nothing here was compared
with its output.  Each function cites the reference file and lines that state
its formula.  Whole sequences, no cache, one function per part, torch CPU
tensors only, and no import from the package under test.

Two things are this library's own and have no reference line: the sliding
window mask (the reference never reads ``sliding_window``,
crates/braidinfer-runtime/src/config.rs:416) and the half-split rotary
pairing (the reference rotates adjacent pairs only).  Both are pinned by
hand-worked numbers in tests/test_plain.py.

The configuration is read here too (`PlainConfig`), from config.json's keys
with the defaults of crates/braidinfer-runtime/src/config.rs:227-268, so that a
wrong default or a wrong per-layer window in the package shows as a difference
instead of being wrong on both sides.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- configuration
class PlainConfig:
    """The sizes and constants the formulas below need, read from config.json's keys.

    Defaults: kv heads = heads (config.rs:236-246), head_dim = hidden / heads (:247),
    eps 1e-5 (:249-252), theta 10000 (:253-260), rotated part = head_dim *
    partial_rotary_factor with factor 1 (:261-268).  ``sliding_window``,
    ``layer_types`` and ``rope_pairing`` are this library's own keys.
    """

    def __init__(self, d: Dict) -> None:
        self.num_hidden_layers = int(d["num_hidden_layers"])
        self.hidden_size = int(d["hidden_size"])
        self.num_attention_heads = int(d["num_attention_heads"])
        kv = d.get("num_key_value_heads")
        self.num_key_value_heads = int(kv) if kv is not None else self.num_attention_heads
        hd = d.get("head_dim")
        self.head_dim = int(hd) if hd is not None else self.hidden_size // self.num_attention_heads
        self.intermediate_size = int(d["intermediate_size"])
        self.vocab_size = int(d["vocab_size"])
        eps = d.get("rms_norm_eps")
        self.rms_norm_eps = float(eps) if eps is not None else 1e-5
        theta = d.get("rope_theta")
        self.rope_theta = float(theta) if theta is not None else 10000.0
        factor = d.get("partial_rotary_factor")
        self.rope_dim = int(self.head_dim * (float(factor) if factor is not None else 1.0))
        self.rope_pairing = d.get("rope_pairing") or "half"
        self.sliding_window = d.get("sliding_window")
        self.layer_types = d.get("layer_types")

    @classmethod
    def from_folder(cls, folder: str) -> "PlainConfig":
        with open(os.path.join(folder, "config.json")) as f:
            return cls(json.load(f))

    def layer_window(self, layer: int) -> Optional[int]:
        """None: the layer sees every earlier key.  With ``layer_types``, only layers named
        "sliding_attention" are windowed; without it every layer is, when a window is set."""
        if self.sliding_window is None:
            return None
        if self.layer_types is not None and self.layer_types[layer] != "sliding_attention":
            return None
        return int(self.sliding_window)


# --------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, tokens: Sequence[int], dtype=torch.float32) -> torch.Tensor:
    """h[t,:] = float(E[token_t,:]), no scale.  kernels/megakernel_ops.hip:1757-1768."""
    idx = torch.as_tensor(list(tokens), dtype=torch.long)
    return table.to(dtype)[idx]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y_i = x_i * rsqrt(mean(x^2) + eps) * w_i, plain w.

    kernels/megakernel_ops.hip:862-904; CPU oracle
    crates/braidinfer-runtime/tests/op_rmsnorm_test.rs:34-50.
    """
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * torch.rsqrt(ms + eps) * w.to(x.dtype)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = W x with W[out,in] row-major, no bias.

    kernels/megakernel_ops.hip:168-216; oracle
    crates/braidinfer-runtime/tests/linear_proj_test.rs:13-23.
    """
    return x @ w.to(x.dtype).t()


def inv_freq(rope_dim: int, theta: float, dtype=torch.float32) -> torch.Tensor:
    """inv_freq[p] = theta^(-2p/rd).  crates/braidinfer-runtime/src/weights.rs:743-751."""
    p = torch.arange(rope_dim // 2, dtype=torch.float64)
    return (1.0 / (float(theta) ** (2.0 * p / rope_dim))).to(dtype)


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float, pairing: str = "half",
         rope_dim: Optional[int] = None) -> torch.Tensor:
    """Rotate the first `rope_dim` elements (default: all) of each head of x[T, heads, hd] by
    angle pos*inv_freq[p]; elements from rope_dim on pass through.

    (a, b) <- (a cos - b sin, a sin + b cos); kernels/megakernel_ops.hip:2019-2030
    (its loop runs over rope_dim / 2 pairs and leaves the rest of the head alone),
    oracle crates/braidinfer-runtime/tests/mrope_test.rs:25-59, where the pair is
    (x[2p], x[2p+1]) ("adjacent").  "half" pairs (x[p], x[p+rd/2]) instead.
    """
    T, H, hd = x.shape
    rd = hd if rope_dim is None else int(rope_dim)
    f = inv_freq(rd, theta, dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]          # [T, rd/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if pairing == "adjacent":
        a, b = x[..., 0:rd:2], x[..., 1:rd:2]
        out[..., 0:rd:2] = a * c - b * s
        out[..., 1:rd:2] = a * s + b * c
    elif pairing == "half":
        a, b = x[..., : rd // 2], x[..., rd // 2:rd]
        out[..., : rd // 2] = a * c - b * s
        out[..., rd // 2:rd] = a * s + b * c
    else:
        raise ValueError(pairing)
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int]) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    q[T, nqh, hd], k/v[T, nkh, hd].  Head h reads kv head h // g; score
    (q.k) * rsqrt(hd); softmax over visible keys; kernels/megakernel_ops.hip:2192-2194
    and :2310-2342 (online form of the same softmax).  Key j is visible to query
    i iff j <= i (the reference's seq_len = p+1,
    crates/braidinfer-runtime/src/megakernel/compile_attention.rs:285) and, with a
    window w, i - j < w.
    """
    T, nqh, hd = q.shape
    nkh = k.shape[1]
    g = nqh // nkh
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & ((i - j) < window)
    out = torch.empty_like(q)
    for h in range(nqh):
        kv = h // g
        s = (q[:, h, :] @ k[:, kv, :].t()) * (1.0 / math.sqrt(hd))
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kv, :]
    return out


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """down( gate/(1+exp(-gate)) * up ).  kernels/megakernel_ops.hip:1474-1545, 1559-1602."""
    gate = linear(x, w_gate)
    up = linear(x, w_up)
    act = gate / (1.0 + torch.exp(-gate)) * up
    return linear(act, w_down)


# --------------------------------------------------------------------------- model
def attention_block(h, weights: Dict[str, torch.Tensor], prefix: str, cfg, layer: int,
                    positions, kv_override=None, return_kv=False):
    """norm -> q,k,v -> rope(q,k) -> attention -> o; the caller adds the residual.

    crates/braidinfer-runtime/src/megakernel/compile_attention.rs:79-90 (norm, projections),
    :229-240 (rotation), :333-351 (output projection).
    """
    T = h.shape[0]
    nqh, nkh, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    n = rmsnorm(h, weights[prefix + "input_layernorm.weight"], cfg.rms_norm_eps)
    q = linear(n, weights[prefix + "self_attn.q_proj.weight"]).view(T, nqh, hd)
    rd = getattr(cfg, "rope_dim", None)
    q = rope(q, positions, cfg.rope_theta, cfg.rope_pairing, rd)
    if kv_override is None:
        k = linear(n, weights[prefix + "self_attn.k_proj.weight"]).view(T, nkh, hd)
        v = linear(n, weights[prefix + "self_attn.v_proj.weight"]).view(T, nkh, hd)
        k = rope(k, positions, cfg.rope_theta, cfg.rope_pairing, rd)
    else:
        k, v = kv_override
    a = attention(q, k, v, cfg.layer_window(layer)).reshape(T, nqh * hd)
    o = linear(a, weights[prefix + "self_attn.o_proj.weight"])
    return (o, (k, v)) if return_kv else o


def decoder_layer(h, weights, layer: int, cfg, positions):
    """h + attn(norm(h)), then h + ffn(norm(h)).

    crates/braidinfer-runtime/src/megakernel/megakernel_compile.rs:115-236 (layer order);
    crates/braidinfer-runtime/src/megakernel/compile_layers.rs:373-386 (feed-forward).
    """
    prefix = f"model.layers.{layer}."
    h = h + attention_block(h, weights, prefix, cfg, layer, positions)
    n = rmsnorm(h, weights[prefix + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
    h = h + swiglu(n, weights[prefix + "mlp.gate_proj.weight"],
                   weights[prefix + "mlp.up_proj.weight"],
                   weights[prefix + "mlp.down_proj.weight"])
    return h


def forward_logits(weights: Dict[str, torch.Tensor], cfg, tokens: Sequence[int],
                   dtype=torch.float32, schedule: Optional[List] = None, hidden: Optional[List] = None) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence.

    Embedding, the layers in order, final norm, output head
    (crates/braidinfer-runtime/src/megakernel/megakernel_compile.rs:238-259); the head
    is the embedding table when no lm_head.weight is stored
    (crates/braidinfer-runtime/src/model/model_load.rs:388-398).

    ``schedule`` (this library's own) lists (layer, cache_of) pairs: the order in
    which layers run; ``cache_of`` names an earlier schedule entry whose keys and
    values the entry reads instead of making its own.  ``hidden``, a list, receives the
    residual stream [T, width] after the embedding and after every run of a layer.
    """
    w = {k: v.to(dtype) for k, v in weights.items()}
    T = len(tokens)
    positions = torch.arange(T)
    h = embedding(w["model.embed_tokens.weight"], tokens, dtype)
    if hidden is not None:
        hidden.append(h)
    if schedule is None:
        for layer in range(cfg.num_hidden_layers):
            h = decoder_layer(h, w, layer, cfg, positions)
            if hidden is not None:
                hidden.append(h)
    else:
        kept = []
        for layer, cache_of in schedule:
            prefix = f"model.layers.{layer}."
            override = kept[cache_of] if cache_of is not None else None
            o, kv = attention_block(h, w, prefix, cfg, layer, positions,
                                    kv_override=override, return_kv=True)
            kept.append(kv)
            h = h + o
            n = rmsnorm(h, w[prefix + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
            h = h + swiglu(n, w[prefix + "mlp.gate_proj.weight"], w[prefix + "mlp.up_proj.weight"],
                           w[prefix + "mlp.down_proj.weight"])
            if hidden is not None:
                hidden.append(h)
    h = rmsnorm(h, w["model.norm.weight"], cfg.rms_norm_eps)
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return linear(h, head)


# --------------------------------------------------------------------------- sampling
def argmax_lowest(logits: torch.Tensor) -> int:
    """Index of the largest logit; the lowest index wins a tie (this library's rule;
    the reference's max_by keeps the last, crates/braidinfer-runtime/src/generate.rs:493-500)."""
    m = logits.max()
    return int(torch.nonzero(logits == m)[0].item())


def sample(logits: torch.Tensor, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
           min_p: float = 0.0, repetition_penalty: float = 1.0, logit_bias=None,
           history: Sequence[int] = (), u: float = 0.0) -> int:
    """One draw as crates/braidinfer-runtime/src/sampling.rs:49-171 makes it.

    Order: bias (:57-65), repetition penalty (:68-79), temperature with 0 => argmax
    (:82-87), top-k (:90-104), min-p (:107-118), top-p (:121-151), softmax (:154-159),
    inverse CDF with the given uniform ``u``: first i with u <= cumsum (:162-170).
    """
    x = logits.to(torch.float32).clone()
    n = x.numel()
    if logit_bias:
        for tok, delta in logit_bias:
            if 0 <= tok < n:
                x[tok] += delta
    if repetition_penalty != 1.0:
        for tok in history:
            if 0 <= tok < n:
                x[tok] = x[tok] / repetition_penalty if x[tok] > 0 else x[tok] * repetition_penalty
    if temperature == 0.0:
        return argmax_lowest(x)
    x = x / temperature
    if 0 < top_k < n:
        order = torch.argsort(x, descending=True, stable=True)
        x[order[top_k:]] = float("-inf")
    if min_p > 0.0:
        mx = x.max()
        drop = (x > float("-inf")) & (torch.exp(x - mx) < min_p)
        x[drop] = float("-inf")
    if top_p < 1.0:
        order = torch.argsort(x, descending=True, stable=True)
        order = order[x[order] > float("-inf")]
        p = torch.exp(x[order] - x[order[0]])
        p = p / p.sum()
        c = torch.cumsum(p, 0)
        hit = torch.nonzero(c >= top_p)
        cut = int(hit[0].item()) + 1 if hit.numel() else order.numel()
        x[order[cut:]] = float("-inf")
    p = torch.exp(x - x.max())
    p = p / p.sum()
    c = torch.cumsum(p, 0)
    hit = torch.nonzero(c >= u)
    return int(hit[0].item()) if hit.numel() else argmax_lowest(p)
