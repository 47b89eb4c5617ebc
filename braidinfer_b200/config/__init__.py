"""Typed configurations read from config.json."""
from .errors import ConfigError, UnknownArchitectureError
from .mistral import MistralConfig
from .presets import PRESETS, preset


def read_config_json(folder: str) -> dict:
    import json
    import os
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json")
    with open(path) as f:
        try:
            d = json.load(f)
        except Exception as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: must hold a JSON object")
    return d
