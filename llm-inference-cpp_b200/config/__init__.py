"""Typed configurations and the registry from architecture name to model recipe."""
from .llama import ConfigError, LlamaConfig  # noqa: F401
from .registry import (Architecture, get_architecture, parse_config, read_model_config,  # noqa: F401
                       register_architecture, registered_architectures)
