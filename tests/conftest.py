import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA GPU (B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_llama_config():
    from transformers import LlamaConfig
    return LlamaConfig(hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=4, vocab_size=32000, rms_norm_eps=1e-6, rope_theta=10000.0,
                       max_position_embeddings=512, tie_word_embeddings=False)


@pytest.fixture(scope="session")
def tiny_llama_dir(tmp_path_factory, tiny_llama_config):
    """fp32 tiny Llama checkpoint, weights N(0, 0.02), seed 0."""
    import torch
    from transformers import LlamaForCausalLM
    torch.manual_seed(0)
    model = LlamaForCausalLM(tiny_llama_config)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() > 1:
                p.normal_(0.0, 0.02)
    d = tmp_path_factory.mktemp("tiny_llama")
    model.save_pretrained(d)
    return str(d)
