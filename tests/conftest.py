"""Shared fixtures: the two tiny configurations and model folders made in temporary folders."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    """A GPU test that does not come back (a warp stuck in a kernel) ends after five minutes instead of holding the
    device until someone kills the run — where the timeout plugin is installed."""
    if not config.pluginmanager.hasplugin("timeout"):
        return
    for item in items:
        if item.get_closest_marker("gpu") is not None and item.get_closest_marker("timeout") is None:
            item.add_marker(pytest.mark.timeout(300, method="thread"))


# Two tiny configurations of the architecture that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 128, "hidden_act": "silu",
    "eos_token_id": 3,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 3, "hidden_size": 120, "num_attention_heads": 5,
    "num_key_value_heads": 1, "head_dim": 24, "intermediate_size": 320, "vocab_size": 384, "rope_theta": 100000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256, "hidden_act": "silu",
    "attention_bias": True, "eos_token_id": [7, 11],
}
# A third one for the replay tests: long enough context for hundreds of keys, head size 32.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 200, "vocab_size": 500, "rope_theta": 50000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 1024, "hidden_act": "silu",
}
# And one whose sizes fit no fast kernel: rows of 72 bytes (no 16-byte alignment), head size 12, an odd vocabulary.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 36, "num_attention_heads": 3,
    "num_key_value_heads": 3, "head_dim": 12, "intermediate_size": 50, "vocab_size": 77, "rope_theta": 300.0,
    "rms_norm_eps": 1e-4, "tie_word_embeddings": False, "max_position_embeddings": 200, "hidden_act": "silu",
    "attention_bias": True,
}
TINY_CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """(config name, storage type) -> model folder with seeded random weights, made on demand."""
    import torch
    from llmi_b200 import write_random_model
    made = {}

    def get(name: str, storage: str = "F32", seed: int = 1234):
        key = (name, storage, seed)
        if key not in made:
            d = tmp_path_factory.mktemp(f"tiny_{name}_{storage}_{seed}")
            write_random_model(str(d), TINY_CONFIGS[name], seed,
                               {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16}[storage])
            made[key] = str(d)
        return made[key]
    return get
