import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


TINY_LLAMA = dict(architectures=["LlamaForCausalLM"], hidden_size=256, intermediate_size=688, num_hidden_layers=4,
                  num_attention_heads=8, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, rope_theta=1e6,
                  vocab_size=32000, max_position_embeddings=512, tie_word_embeddings=False)


@pytest.fixture
def tiny_llama_cfg():
    return dict(TINY_LLAMA)
