"""The tests' own small configurations (as config.json dictionaries) and helpers.

A and B differ in every size and option: layers, width, head counts and group size,
head_dim (B's is not width / heads), intermediate size, vocabulary, theta, eps, window.
C adds per-layer attention kinds (two cache groups), a tied head and adjacent rotary
pairs, with sizes that are no power of two.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

TINY_A: Dict = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral", "torch_dtype": "bfloat16",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "sliding_window": None, "tie_word_embeddings": False,
    "max_position_embeddings": 4096, "eos_token_id": 2, "bos_token_id": 1,
}

TINY_B: Dict = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral", "torch_dtype": "bfloat16",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 384, "rope_theta": 1e6,
    "rms_norm_eps": 1e-6, "sliding_window": 8, "tie_word_embeddings": False,
    "max_position_embeddings": 2048,
}

TINY_C: Dict = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral", "torch_dtype": "bfloat16",
    "num_hidden_layers": 4, "hidden_size": 120, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 331, "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6, "sliding_window": 70, "tie_word_embeddings": True,
    "layer_types": ["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
    "rope_pairing": "adjacent", "max_position_embeddings": 1024,
}

SEEDS = {"A": 0, "B": 7, "C": 3}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}

# Tolerances on logits (absolute; logits of these models are of order 0.5).
TOL_F32 = 2e-5
TOL_BF16 = 1.5e-2


def make_folder(tmp_path, name: str, **override) -> str:
    """Write a random model folder for configuration `name` and return its path."""
    from braidinfer_b200.weights import write_random_model
    d = dict(CONFIGS[name])
    d.update(override)
    folder = os.path.join(str(tmp_path), f"tiny_{name}")
    write_random_model(d, folder, SEEDS[name])
    return folder


def read_weights(folder: str) -> Dict[str, torch.Tensor]:
    """The folder's tensors as float64 CPU tensors, read with the tests' own few lines."""
    import struct
    path = os.path.join(folder, "model.safetensors")
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + b:8 + n + en]), dtype=kinds[e["dtype"]]).reshape(e["shape"])
        out[name] = t.to(torch.float64)
    return out


def config_of(folder: str):
    """The folder's configuration as the plain implementation reads it (its own few lines,
    nothing of the package under test)."""
    from plain_mistral import PlainConfig
    return PlainConfig.from_folder(folder)


def random_prompts(vocab: int, lengths: List[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
