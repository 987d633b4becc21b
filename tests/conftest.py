"""Shared test fixtures: the two tiny configurations and the ``gpu`` marker."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny configurations of the architecture that differ in every size and option.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "torch_dtype": "bfloat16",
    "hidden_act": "silu", "use_cache": True, "tie_word_embeddings": True,
    "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 256,
    "max_position_embeddings": 512, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "bos_token_id": 1, "eos_token_id": 2, "attention_bias": False, "use_sliding_window": False,
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "torch_dtype": "bfloat16",
    "hidden_act": "silu", "use_cache": True, "tie_word_embeddings": False,
    "hidden_size": 96, "intermediate_size": 224, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 32, "vocab_size": 384,
    "max_position_embeddings": 1024, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "bos_token_id": 5, "eos_token_id": 7, "attention_bias": False,
    # layers 1 and 2 see only the last 24 keys: a second cache group with a window
    "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 1,
}
# Two more with the head sizes that the TMA-fed, tcgen05 and cluster kernels take (64 and 128), small otherwise:
# C has a windowed layer, a hidden size that the few-rows product takes and an intermediate size that it refuses;
# D has one query head per kv head.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "torch_dtype": "bfloat16",
    "hidden_act": "silu", "use_cache": True, "tie_word_embeddings": False,
    "hidden_size": 160, "intermediate_size": 272, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 1000,
    "max_position_embeddings": 2048, "rope_theta": 50000.0, "rms_norm_eps": 1e-6,
    "bos_token_id": 3, "eos_token_id": 4, "attention_bias": False,
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 1,
}
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "torch_dtype": "bfloat16",
    "hidden_act": "silu", "use_cache": True, "tie_word_embeddings": True,
    "hidden_size": 96, "intermediate_size": 160, "num_hidden_layers": 2,
    "num_attention_heads": 2, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 300,
    "max_position_embeddings": 1024, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "bos_token_id": 0, "eos_token_id": 1, "attention_bias": False, "use_sliding_window": False,
}
# sigma and seed of the random weights (the benchmark definition's tiny configurations: 0.02 / seed 0 and 0.05 / seed 1)
TINY_INIT = {"A": (0.02, 0), "B": (0.05, 1), "C": (0.06, 2), "D": (0.08, 3)}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


@pytest.fixture(scope="session")
def tiny_configs():
    return TINY


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, written by the random-weights mode."""
    from pih_b200.config import config_from_dict
    from pih_b200.weights import write_random_model
    out = {}
    for name, raw in TINY.items():
        sigma, seed = TINY_INIT[name]
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(str(d), config_from_dict(raw), seed=seed, sigma=sigma)
        out[name] = str(d)
    return out


def load_plain_weights(model_dir):
    """Read a model folder for the plain implementation (own parser use is fine: it is data)."""
    import json
    from pih_b200.weights.safetensors_io import SafetensorsFile
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with SafetensorsFile(os.path.join(model_dir, "model.safetensors")) as sf:
        w = {n: sf.read_tensor(n).to(torch.float64) for n in sf.names()}
    return cfg, w
