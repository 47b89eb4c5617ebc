"""Named configurations, as config.json dictionaries: two tiny ones for tests and the
sizes that measurements are quoted on.  These are inputs to the same path a model
folder's config.json takes; no code elsewhere holds any of these numbers."""
from __future__ import annotations

from typing import Dict


def _mistral(**kw) -> Dict:
    d = {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "torch_dtype": "bfloat16",
         "tie_word_embeddings": False, "hidden_act": "silu"}
    d.update(kw)
    return d


PRESETS: Dict[str, Dict] = {
    "tiny_a": _mistral(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=16, intermediate_size=176, vocab_size=256, rope_theta=10000.0,
                       rms_norm_eps=1e-5, sliding_window=None, max_position_embeddings=4096),
    "tiny_b": _mistral(num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=2,
                       head_dim=32, intermediate_size=256, vocab_size=384, rope_theta=1e6,
                       rms_norm_eps=1e-6, sliding_window=8, max_position_embeddings=4096),
    "mistral_7b_v03": _mistral(num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                               num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=32768,
                               rope_theta=1e6, rms_norm_eps=1e-5, sliding_window=None,
                               max_position_embeddings=32768),
    "mistral_7b_v01": _mistral(num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                               num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=32000,
                               rope_theta=10000.0, rms_norm_eps=1e-5, sliding_window=4096,
                               max_position_embeddings=32768),
    "mistral_nemo_12b": _mistral(num_hidden_layers=40, hidden_size=5120, num_attention_heads=32,
                                 num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=131072,
                                 rope_theta=1e6, rms_norm_eps=1e-5, sliding_window=None,
                                 max_position_embeddings=131072),
}


def preset(name: str) -> Dict:
    if name not in PRESETS:
        raise KeyError(f"unknown preset '{name}'; known: {sorted(PRESETS)}")
    return dict(PRESETS[name])
