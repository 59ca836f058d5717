"""Weights: the safetensors file, binding by tensor name, and seeded random models."""
from .binding import WeightBindingError, check_tensors, load_tensors  # noqa: F401
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors  # noqa: F401
