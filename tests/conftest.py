"""Shared fixtures: tiny configurations, model folders in a temporary directory, markers."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# Two tiny Llamas that differ in every size and option, and a third whose widths share
# no factor with the others (query width != hidden size, head size 48).
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 172, "vocab_size": 256, "rope_theta": 10000.0,
    "rope_scaling": None, "max_position_embeddings": 128, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256, "vocab_size": 512, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
}
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 80, "num_hidden_layers": 1, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 48, "intermediate_size": 200, "vocab_size": 301, "rope_theta": 2500.0,
    "rope_scaling": None, "max_position_embeddings": 512, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
}
# head size 64 and 16-byte rows everywhere: the tensor-core kernels (tcgen05 products, flash
# attention) run on this one; A, B and C mostly take the generic kernels.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 192, "num_hidden_layers": 2, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 328, "vocab_size": 424, "rope_theta": 100000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 2.0,
                     "original_max_position_embeddings": 32},
    "max_position_embeddings": 1024, "rms_norm_eps": 2e-5, "tie_word_embeddings": True,
}
# Not tiny: wide enough for the kernels that only many tokens and many tiles reach (CTA-pair
# products cut across several CTAs, tcgen05 attention over several items, split key ranges).
MID_E = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 1024, "num_hidden_layers": 2, "num_attention_heads": 8,
    "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 2816, "vocab_size": 1500, "rope_theta": 500000.0,
    "rope_scaling": None, "max_position_embeddings": 2048, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}
# One KV head under 32 query heads: a decoded token has 32 packed rows, more than the 16-row
# tile of the tensor-core attention kernel holds.
TINY_G = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 160, "num_hidden_layers": 1, "num_attention_heads": 32,
    "num_key_value_heads": 1, "head_dim": 64, "intermediate_size": 224, "vocab_size": 333, "rope_theta": 30000.0,
    "rope_scaling": None, "max_position_embeddings": 512, "rms_norm_eps": 4e-6, "tie_word_embeddings": False,
}
TINY = {"A": (TINY_A, 0, "float32"), "B": (TINY_B, 1, "bfloat16"), "C": (TINY_C, 2, "float32"),
        "D": (TINY_D, 3, "bfloat16")}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_sessionfinish(session, exitstatus):
    """FERRUM_TEST_STATS=file: write the worst 16-bit error ratios the session saw (the
    tolerance in helpers.py is set from them)."""
    path = os.environ.get("FERRUM_TEST_STATS")
    if path:
        import json
        import helpers
        with open(path, "w") as f:
            json.dump(dict(sorted(helpers.STATS.items(), key=lambda kv: -kv[1])), f, indent=1)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder with config.json + model.safetensors, written by the random-weights mode."""
    from ferrum_b200.weights import write_random_model
    out = {}
    for name, (cfg, seed, dtype) in list(TINY.items()) + [("E", (MID_E, 5, "bfloat16")), ("G", (TINY_G, 6, "bfloat16"))]:
        d = tmp_path_factory.mktemp("tiny_" + name)
        write_random_model(cfg, str(d), seed, dtype=dtype)
        out[name] = str(d)
    return out


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda")
