"""The engine: step function, generation loop, entry points."""
from .engine import Engine, parse_dtype
from .step import StepContext, StepPacker
