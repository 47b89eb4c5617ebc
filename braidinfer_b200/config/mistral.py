"""Typed configuration of the dense Mistral decoder, read from config.json keys.

Every size and constant of the model comes from here; no kernel or part holds
a model size of its own.  Key names and fallbacks follow the reference parser
(crates/braidinfer-runtime/src/config.rs:193-277): ``num_key_value_heads``
falls back to the head count (:236-246), ``head_dim`` to hidden/heads (:247),
``rms_norm_eps`` to 1e-5 (:249-252), ``rope_theta`` to 10000 (:253-260).
``sliding_window`` is read here although the reference ignores it
(config.rs:416 maps ``sliding_attention`` to plain attention).
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
        hidden = _require_int(d, "hidden_size")
        heads = _require_int(d, "num_attention_heads")
        kv_heads = _opt_int(d, "num_key_value_heads", heads)
        head_dim = _opt_int(d, "head_dim", None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"config.json: head_dim is absent and hidden_size ({hidden}) is not a "
                    f"multiple of num_attention_heads ({heads})")
            head_dim = hidden // heads
        rope_theta = d.get("rope_theta")
        if rope_theta is None and isinstance(d.get("rope_parameters"), Mapping):
            rope_theta = d["rope_parameters"].get("rope_theta")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_t = None
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_t = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_t = tuple(int(e) for e in eos)
        else:
            raise ConfigError(f"config.json: 'eos_token_id' must be an int or a list of ints, got {eos!r}")
        tie = d.get("tie_word_embeddings")
        if tie is not None and not isinstance(tie, bool):
            raise ConfigError(f"config.json: 'tie_word_embeddings' must be a boolean, got {tie!r}")
        lt = d.get("layer_types")
        if lt is not None:
            if not isinstance(lt, (list, tuple)) or not all(isinstance(t, str) for t in lt):
                raise ConfigError("config.json: 'layer_types' must be a list of strings")
            lt = tuple(lt)
        archs = d.get("architectures") or ["MistralForCausalLM"]
        return cls(
            vocab_size=_require_int(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_require_int(d, "intermediate_size"),
            num_hidden_layers=_require_int(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=_opt_float(d, "rms_norm_eps", 1e-5),
            rope_theta=_opt_float({"rope_theta": rope_theta}, "rope_theta", 10000.0),
            sliding_window=_opt_int(d, "sliding_window", None),
            tie_word_embeddings=tie,
            max_position_embeddings=_opt_int(d, "max_position_embeddings", 2048),
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
        return d
