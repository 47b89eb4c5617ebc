"""Architectures: how a configuration becomes a description of parts, and the
registry from config.json's architecture name to that recipe."""
from .registry import ARCHITECTURES, Architecture, architecture_for, register_architecture
from . import mistral  # noqa: F401  (registration)
from .decoder import DecoderModel
