"""Typed configuration of the dense Mistral decoder, read from config.json keys.

Every size and constant of the model comes from here; no kernel or part holds
a model size of its own.  Key names, alias keys and fallbacks follow the reference
parser (crates/braidinfer-runtime/src/config.rs:193-277): ``num_hidden_layers`` may
be spelled ``n_layer`` or ``num_transformer_layers`` (:214-223), ``hidden_size``
``n_embd`` or ``d_model`` (:208-213), ``vocab_size`` ``n_vocab`` (:224-226),
``num_attention_heads`` ``n_head`` (:227-235); ``num_key_value_heads`` (or
``num_kv_heads``) falls back to the head count (:236-246), ``head_dim`` to
hidden/heads (:247), ``rms_norm_eps`` (or ``norm_eps``, ``layer_norm_epsilon``) to
1e-5 (:249-252), ``rope_theta`` (or ``rope_freq_constant``,
``rope_parameters.rope_theta``) to 10000 (:253-260), ``partial_rotary_factor`` (also
under ``rope_parameters``) to 1 (:261-268), ``max_position_embeddings`` (or
``max_context_length``, ``rope_max_length``) to 2048 (:269-272),
``tie_word_embeddings`` may be spelled ``share_input_output_layers`` (:275-277).
``sliding_window`` is read here although the reference ignores it
(config.rs:416 maps ``sliding_attention`` to plain attention).

A key that asks for arithmetic this model does not do (another activation, scaled
rotary frequencies, biases) is refused with an error that names key and value; it
never runs silently with other math.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError

ROPE_PAIRINGS = ("half", "adjacent")
LAYER_TYPES = ("full_attention", "sliding_attention")


def _require_int(d: Mapping[str, Any], key: str, *, minimum: int = 1) -> int:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, got {v}")
    return v


def _opt_int(d: Mapping[str, Any], key: str, default: Optional[int], *, minimum: int = 1) -> Optional[int]:
    v = d.get(key, None)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer or null, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, got {v}")
    return v


def _first(d: Mapping[str, Any], *keys: str):
    """(key, value) of the first of `keys` that config.json holds with a value, else (keys[0], None)."""
    for k in keys:
        if d.get(k) is not None:
            return k, d[k]
    return keys[0], None


def _refuse_unsupported(d: Mapping[str, Any]) -> None:
    """Keys whose value would change the arithmetic in a way no part here computes."""
    act = d.get("hidden_act", d.get("hidden_activation"))
    if act is not None and act != "silu":
        raise ConfigError(f"config.json: 'hidden_act' is {act!r}; the feed-forward here computes silu(gate) * up only")
    scaling = d.get("rope_scaling")
    if scaling is not None:
        kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, Mapping) else scaling
        if kind not in (None, "default"):
            raise ConfigError(f"config.json: 'rope_scaling' is {scaling!r}; scaled rotary frequencies are not computed "
                              "here (only the plain theta^(-2p/d) ones)")
    rp = d.get("rope_parameters")
    if isinstance(rp, Mapping):
        kind = rp.get("rope_type", rp.get("type"))
        if kind not in (None, "default"):
            raise ConfigError(f"config.json: 'rope_parameters.rope_type' is {kind!r}; only the default rotary "
                              "encoding is computed here")
    for key in ("attention_bias", "mlp_bias"):
        v = d.get(key)
        if v not in (None, False):
            raise ConfigError(f"config.json: '{key}' is {v!r}; the projections here have no bias")


def _opt_float(d: Mapping[str, Any], key: str, default: float) -> float:
    v = d.get(key, None)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class MistralConfig:
    """All sizes and options of a Mistral decoder (``MistralForCausalLM``)."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    sliding_window: Optional[int] = None
    # How many elements of a head are rotated (head_dim * partial_rotary_factor); the rest pass through.
    rope_dim: Optional[int] = None
    # None: decided at load time by whether lm_head.weight is stored.
    tie_word_embeddings: Optional[bool] = None
    max_position_embeddings: int = 2048
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[Tuple[int, ...]] = None
    # "half" pairs element p with p + head_dim/2 (the layout Mistral model
    # folders are stored for); "adjacent" pairs (2p, 2p+1) as the reference's
    # rotation kernel does (kernels/megakernel_ops.hip:2019-2030).
    rope_pairing: str = "half"
    # Per-layer attention kind; None means every layer uses `sliding_window`
    # when it is set and full attention otherwise.
    layer_types: Optional[Tuple[str, ...]] = None
    architectures: Tuple[str, ...] = ("MistralForCausalLM",)
    model_type: str = "mistral"
    torch_dtype: str = "bfloat16"

    architecture_name = "MistralForCausalLM"

    def __post_init__(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim must be even for rotary pairs, got {self.head_dim}")
        if self.rope_dim is None:
            object.__setattr__(self, "rope_dim", self.head_dim)
        if self.rope_dim % 2 or not (0 < self.rope_dim <= self.head_dim):
            raise ConfigError(f"rope_dim must be even and within head_dim={self.head_dim}, got {self.rope_dim}")
        if self.rope_pairing not in ROPE_PAIRINGS:
            raise ConfigError(f"rope_pairing must be one of {ROPE_PAIRINGS}, got {self.rope_pairing!r}")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(
                    f"layer_types has {len(self.layer_types)} entries for "
                    f"{self.num_hidden_layers} layers")
            for t in self.layer_types:
                if t not in LAYER_TYPES:
                    raise ConfigError(f"layer_types entry {t!r} is not one of {LAYER_TYPES}")
            if "sliding_attention" in self.layer_types and self.sliding_window is None:
                raise ConfigError("layer_types names sliding_attention but sliding_window is null")

    # ------------------------------------------------------------------ derived
    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> Optional[int]:
        """Window of one layer's attention, or None when it sees every key."""
        if self.sliding_window is None:
            return None
        if self.layer_types is None:
            return self.sliding_window
        return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None

    # ------------------------------------------------------------------ io
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MistralConfig":
        _refuse_unsupported(d)
        alias = lambda *keys: {keys[0]: _first(d, *keys)[1]}    # {primary key: the value found under any spelling}
        hidden = _require_int(alias("hidden_size", "n_embd", "d_model"), "hidden_size")
        heads = _require_int(alias("num_attention_heads", "n_head"), "num_attention_heads")
        kv_heads = _opt_int(alias("num_key_value_heads", "num_kv_heads"), "num_key_value_heads", heads)
        head_dim = _opt_int(d, "head_dim", None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"config.json: head_dim is absent and hidden_size ({hidden}) is not a "
                    f"multiple of num_attention_heads ({heads})")
            head_dim = hidden // heads
        rp = d.get("rope_parameters") if isinstance(d.get("rope_parameters"), Mapping) else {}
        rope_theta = _first(d, "rope_theta", "rope_freq_constant")[1]
        if rope_theta is None:
            rope_theta = rp.get("rope_theta")
        factor = d.get("partial_rotary_factor")
        if factor is None:
            factor = rp.get("partial_rotary_factor")
        factor = _opt_float({"partial_rotary_factor": factor}, "partial_rotary_factor", 1.0)
        if not (0.0 < factor <= 1.0):
            raise ConfigError(f"config.json: 'partial_rotary_factor' must be in (0, 1], got {factor}")
        rope_dim = int(head_dim * factor)                   # truncation, as config.rs:268 does
        if rope_dim % 2 or rope_dim <= 0:
            raise ConfigError(f"config.json: 'partial_rotary_factor' {factor} of head_dim {head_dim} gives "
                              f"{rope_dim} rotated elements; they must be a positive even number")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_t = None
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_t = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_t = tuple(int(e) for e in eos)
        else:
            raise ConfigError(f"config.json: 'eos_token_id' must be an int or a list of ints, got {eos!r}")
        tie = _first(d, "tie_word_embeddings", "share_input_output_layers")[1]
        if tie is not None and not isinstance(tie, bool):
            raise ConfigError(f"config.json: 'tie_word_embeddings' must be a boolean, got {tie!r}")
        lt = d.get("layer_types")
        if lt is not None:
            if not isinstance(lt, (list, tuple)) or not all(isinstance(t, str) for t in lt):
                raise ConfigError("config.json: 'layer_types' must be a list of strings")
            lt = tuple(lt)
        archs = d.get("architectures") or ["MistralForCausalLM"]
        return cls(
            vocab_size=_require_int(alias("vocab_size", "n_vocab"), "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_require_int(d, "intermediate_size"),
            num_hidden_layers=_require_int(alias("num_hidden_layers", "n_layer", "num_transformer_layers"),
                                           "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=_opt_float(alias("rms_norm_eps", "norm_eps", "layer_norm_epsilon"), "rms_norm_eps", 1e-5),
            rope_theta=_opt_float({"rope_theta": rope_theta}, "rope_theta", 10000.0),
            sliding_window=_opt_int(d, "sliding_window", None),
            rope_dim=rope_dim,
            tie_word_embeddings=tie,
            max_position_embeddings=_opt_int(alias("max_position_embeddings", "max_context_length", "rope_max_length"),
                                             "max_position_embeddings", 2048),
            bos_token_id=_opt_int(d, "bos_token_id", None, minimum=0),
            eos_token_id=eos_t,
            rope_pairing=d.get("rope_pairing", "half"),
            layer_types=lt,
            architectures=tuple(archs),
            model_type=str(d.get("model_type", "mistral")),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        if self.eos_token_id is not None:
            d["eos_token_id"] = list(self.eos_token_id) if len(self.eos_token_id) != 1 else self.eos_token_id[0]
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        else:
            d.pop("layer_types")
        if self.tie_word_embeddings is None:
            d.pop("tie_word_embeddings")
        if self.rope_pairing == "half":
            d.pop("rope_pairing")
        rope_dim = d.pop("rope_dim")
        if rope_dim != self.head_dim:
            d["partial_rotary_factor"] = rope_dim / self.head_dim
        return d
