"""Shared fixtures: tiny Llama configurations that differ in every size and
option, written as model folders (random weights) into a temporary folder.

tiny-A: 2 layers, hidden 64, 4 heads / 2 kv heads, head_dim 16, intermediate
176, vocab 256, theta 1e4 without scaling, eps 1e-5, tied head, pages of 16.
tiny-B: 3 layers, hidden 96, 3 heads / 1 kv head, head_dim 32, intermediate
256 -> 272 would be a power-of-two neighbour, so 264 is used, vocab 384 -> 389
(no power of two, odd), theta 5e5 with llama3 scaling (factor 4, low 1, high 4,
original 32: its 16 frequencies hit all three branches), eps 1e-6, untied
head, pages of 8.
tiny-B0: tiny-B with intermediate 256, vocab 384 and 256 positions (powers of
two and multiples of 128, which take other tile paths than 264 and 389).
tiny-C: head_dim 64 (the size the tcgen05 attention kernel takes), 2 layers,
hidden 256, 4 heads / 2 kv heads, intermediate 200,
vocab 311, theta 1e6, eps 1e-5, untied head, pages of 16, contexts of several
128-key tiles.
"""
from __future__ import annotations

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


# the checkpoint names of the Llama family, for specs that tests write by hand (a spec names its tensors)
ATT_NAMES = dict(tensor_prefix="self_attn.", tensor_names={"q": "q_proj.weight", "k": "k_proj.weight",
                                                            "v": "v_proj.weight", "o": "o_proj.weight"})
MLP_NAMES = dict(tensor_prefix="mlp.", tensor_names={"gate": "gate_proj.weight", "up": "up_proj.weight",
                                                      "down": "down_proj.weight"})

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0,
    "rope_scaling": None, "max_position_embeddings": 128, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "hidden_act": "silu", "torch_dtype": "float32",
    "bos_token_id": 1, "eos_token_id": 2,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 264, "vocab_size": 389, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
    "max_position_embeddings": 512, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "float32", "bos_token_id": 0, "eos_token_id": [3, 7],
}
# tiny-B with the sizes that are powers of two or multiples of 128 (intermediate 256, vocabulary 384,
# 256 positions): other tile paths of the kernels than tiny-B's odd sizes reach
TINY_B0 = dict(TINY_B, intermediate_size=256, vocab_size=384, max_position_embeddings=256)
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 200, "vocab_size": 311, "rope_theta": 1000000.0,
    "rope_scaling": None, "max_position_embeddings": 640, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "float32",
    "bos_token_id": 1, "eos_token_id": 2,
}
# a head size that is a multiple of 16 but no power of two, as many kv heads as heads, partial rotation, one layer
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 1, "hidden_size": 144, "num_attention_heads": 3, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 120, "vocab_size": 203, "rope_theta": 20000.0,
    "rope_scaling": None, "max_position_embeddings": 256, "rms_norm_eps": 2e-5,
    "tie_word_embeddings": True, "hidden_act": "silu", "torch_dtype": "float32",
    "bos_token_id": 1, "eos_token_id": 2,
}
TINY = {"A": (TINY_A, 0, 16), "B": (TINY_B, 2, 8), "C": (TINY_C, 5, 16), "D": (TINY_D, 9, 4),
        "B0": (TINY_B0, 2, 8)}   # name -> (config, weight seed, page size)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (float32 storage)."""
    from rllm_b200.engine.loading import write_random_model
    out = {}
    for name, (cfg, seed, _) in TINY.items():
        d = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        write_random_model(d, cfg, seed, "float32")
        out[name] = d
    return out


def has_cuda() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if has_cuda():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
