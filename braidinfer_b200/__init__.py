"""braidinfer_b200: a small, whole generation library for the dense Mistral decoder on
one NVIDIA B200 (sm_100a): config and registry, weights, parts, cache, step function,
generation loop, sampling, command line, trace replay, hand-written CUDA kernels."""
__version__ = "0.1.0"

from .api import Model, load                                  # noqa: E402
from .engine.generate import Completion, GenerationStats     # noqa: E402
from .sampling import SamplingParams                          # noqa: E402

__all__ = ["Model", "load", "Completion", "GenerationStats", "SamplingParams"]
