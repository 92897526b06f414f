import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


TINY_A = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "num_experts": 4, "num_experts_per_tok": 2,
    "moe_intermediate_size": 32, "shared_expert_intermediate_size": 64,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "norm_topk_prob": True, "vocab_size": 256,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "use_sliding_window": False,
    "tie_word_embeddings": False, "torch_dtype": "float32",
}

TINY_B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "num_experts": 8, "num_experts_per_tok": 3,
    "moe_intermediate_size": 48, "shared_expert_intermediate_size": 80,
    "intermediate_size": 128, "decoder_sparse_step": 2, "mlp_only_layers": [0],
    "norm_topk_prob": False, "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "use_sliding_window": True, "sliding_window": 8, "max_window_layers": 1,
    "tie_word_embeddings": True, "torch_dtype": "float32",
}


# Tiny B with the sliding layers listed in config.json, and listed differently from what
# the max_window_layers rule would derive: the window is on layers 0 and 2.
TINY_B_LISTED = dict(TINY_B, layer_types=["sliding_attention", "full_attention",
                                          "sliding_attention"])


@pytest.fixture
def tiny_a():
    return dict(TINY_A)


@pytest.fixture
def tiny_b():
    return dict(TINY_B)
