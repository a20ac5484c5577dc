"""Shared fixtures: two tiny Llama configurations that differ in every size and option,
random weights for them, and helpers that run the plain implementation.

Tiny A: 2 layers, hidden 64, 4 heads over 2 kv heads (grouped), head size 16, feed-forward 176,
        vocabulary 256, theta 10000 without scaling, eps 1e-5, 128 positions, tied classifier,
        float32 weights, norm weights 1.
Tiny B: 3 layers, hidden 144, 6 heads over 6 kv heads, head size 24, feed-forward 384,
        vocabulary 512, theta 500000 with llama3 scaling (8, 1, 4, 64), eps 1e-6, 256 positions,
        own classifier, bfloat16 weights, norm weights 1 + N(0, 0.1).
"""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 64,
    "intermediate_size": 176,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "vocab_size": 256,
    "max_position_embeddings": 128,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "rope_scaling": None,
    "tie_word_embeddings": True,
    "torch_dtype": "float32",
    "eos_token_id": 2,
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 144,
    "intermediate_size": 384,
    "num_hidden_layers": 3,
    "num_attention_heads": 6,
    "num_key_value_heads": 6,
    "head_dim": 24,
    "vocab_size": 512,
    "max_position_embeddings": 256,
    "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64,
    },
    "tie_word_embeddings": False,
    "torch_dtype": "bfloat16",
    "eos_token_id": [3, 5],
}

TINY = {"A": (TINY_A, 0, 0.0), "B": (TINY_B, 1, 0.1)}  # name -> (config, seed, norm jitter)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def read_weights(model_dir):
    """Tensors of a model folder, read with the third-party safetensors package so that the
    plain implementation does not depend on the library's own reader."""
    from safetensors import safe_open

    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k)
    return out


@pytest.fixture(scope="session")
def tiny_dirs(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (made once per session, in a temp folder)."""
    from rusty_llama_b200 import write_random_model

    dirs = {}
    for name, (cfg, seed, jitter) in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(str(d), cfg, seed, norm_jitter=jitter)
        dirs[name] = str(d)
    return dirs


@pytest.fixture(scope="session")
def tiny_weights(tiny_dirs):
    return {name: read_weights(d) for name, d in tiny_dirs.items()}


def rounded_weights(weights, dtype_name):
    """The weights as the engine holds them in a run of `dtype_name`, widened to float32:
    a bfloat16 run rounds matrices to bfloat16 (and vectors unless stored in 32-bit)."""
    out = {}
    for k, t in weights.items():
        if dtype_name == "bfloat16":
            if t.dim() >= 2 or t.dtype != torch.float32:
                t = t.to(torch.bfloat16)
        out[k] = t.to(torch.float32)
    return out
