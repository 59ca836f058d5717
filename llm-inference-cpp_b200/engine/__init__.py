"""The engine: step function, generation loop, trace replay."""
from .batch import SequenceStep, StepError  # noqa: F401
from .loader import load_model, parse_dtype, random_model  # noqa: F401
from .model import Model  # noqa: F401
