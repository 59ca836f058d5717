"""A small B200-native model library with generation of its own, for the Llama / SmolLM2
dense decoder: from a model folder (or a configuration and a seed) to generated tokens on
one GPU, on hand-written sm_100a kernels.

Python entry points::

    model = load(model_dir, dtype="bfloat16")            # or random(config_dict, seed, dtype)
    cache = model.new_cache(max_tokens)
    logits = model.step(cache, [SequenceStep(slot, tokens, want)])
    outputs = generate(model, prompts, max_new=32, sampling=SamplingParams(temperature=0.8, seed=1))
"""
from . import models  # noqa: F401  (registers the architectures)
from .cache import CacheError, SequenceCache  # noqa: F401
from .config import ConfigError, LlamaConfig, parse_config, register_architecture  # noqa: F401
from .engine import Model, SequenceStep, StepError, load_model, random_model  # noqa: F401
from .engine.generate import generate  # noqa: F401
from .parts import register_part  # noqa: F401
from .sampling import SamplingParams  # noqa: F401
from .weights import WeightBindingError  # noqa: F401
from .weights.random_weights import write_random_model  # noqa: F401

load = load_model
random = random_model
