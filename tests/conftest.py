import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU and the compiled kernel library")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny configurations of the architecture that differ in every size and option: layers, hidden, heads, groups,
# head size, width of q against hidden, intermediate, vocabulary (neither a power of two in B), theta, eps, tied or
# untied head, norm weights, a sliding-window layer, page size.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=512,
              torch_dtype="float32", hidden_act="silu")
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
              num_attention_heads=6, num_key_value_heads=1, head_dim=32, intermediate_size=272, vocab_size=387,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=1024,
              torch_dtype="bfloat16", hidden_act="silu", sliding_window=40,
              layer_types=["full_attention", "sliding_attention", "full_attention"], eos_token_id=[5, 7])
# A third one with sizes no fast path serves: a width that is no multiple of 8 (no 16-byte vectors, no TMA strides), a
# head size of 48 (no tensor-core attention: the 32-bit kernel runs in bfloat16 too), one query head per key/value head.
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=44,
              num_attention_heads=3, num_key_value_heads=3, head_dim=48, intermediate_size=100, vocab_size=131,
              rope_theta=50000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=300,
              torch_dtype="float32", hidden_act="silu", sliding_window=24, use_sliding_window=True, max_window_layers=1)
# A fourth one that the tensor-core attention kernels serve in bfloat16 (head size 64, pages of 16 rows: the copy-engine
# decode kernel and the tcgen05 prefill kernel) with a sliding-window layer, so that those kernels meet block tables whose
# leading pages a window has passed and given back.
TINY_D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=120,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=200, vocab_size=301,
              rope_theta=100000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=2048,
              torch_dtype="bfloat16", hidden_act="silu", sliding_window=48, layer_types=["sliding_attention", "full_attention"])
TINY = {"C": dict(config=TINY_C, seed=2, std=0.1, norm_std=0.05, page_size=4),
        "D": dict(config=TINY_D, seed=3, std=0.07, norm_std=0.1, page_size=16),
        "A": dict(config=TINY_A, seed=0, std=0.08, norm_std=0.0, page_size=16),
        "B": dict(config=TINY_B, seed=1, std=0.06, norm_std=0.1, page_size=8)}


@pytest.fixture(scope="session")
def tiny_model_dirs(tmp_path_factory):
    """Model folders of the two tiny configurations, written once per session into a temporary folder."""
    from roost_b200.weights.random_init import write_random_model
    out = {}
    for name, t in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(d, t["config"], seed=t["seed"], std=t["std"], norm_std=t["norm_std"])
        out[name] = d
    return out


@pytest.fixture(scope="session")
def kernels():
    from roost_b200.kernels import library
    return library.load()
