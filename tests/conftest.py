import os
import sys

import pytest
import torch

os.environ.setdefault("VAPI_VALIDATE", "1")      # every batch of every test is checked on the host

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny LFM2 configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 192, "block_auto_adjust_ff_dim": False,
    "num_hidden_layers": 4, "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "conv_L_cache": 3, "conv_bias": False, "rope_theta": 10000.0, "norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 128 + 256, "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 509, "hidden_size": 96, "intermediate_size": 384, "block_auto_adjust_ff_dim": True,
    "block_ffn_dim_multiplier": 1.5, "block_multiple_of": 64,
    "num_hidden_layers": 6,
    "layer_types": ["conv", "conv", "full_attention", "conv", "full_attention", "conv"],
    "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 32,
    "conv_L_cache": 4, "conv_bias": True, "rope_parameters": {"rope_theta": 1000000.0}, "norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 512, "eos_token_id": [3, 5],
}
# The two tiny configurations exactly as the benchmark description words them (the two above differ
# from it in head size, vocabulary and length limit so that they also reach other kernel paths)
TINY_A0 = dict(TINY_A, max_position_embeddings=128)
TINY_B0 = dict(TINY_B, vocab_size=512, head_dim=16, max_position_embeddings=256)

# A third shape: heads that do not fill the hidden size, 3:1 groups, a longer conv
TINY_C = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 300, "hidden_size": 80, "intermediate_size": 144,
    "num_hidden_layers": 3, "layer_types": ["full_attention", "conv", "full_attention"],
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 48,
    "conv_L_cache": 5, "conv_bias": False, "rope_theta": 50000.0, "norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 640,
}


# A fourth: head size 64 and widths that are multiples of 32, the shapes the serving kernels
# want (tensor-core attention, the weight-streaming and tcgen05 products), still tiny
TINY_D = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 1003, "hidden_size": 256, "intermediate_size": 640, "block_auto_adjust_ff_dim": False,
    "num_hidden_layers": 4, "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "conv_L_cache": 3, "conv_bias": False, "rope_theta": 1000000.0, "norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 512, "eos_token_id": 2,
}

# A fifth: head size 128 (the other head size of the bfloat16 flash kernel), an attention layer
# first, one kv head, a conv of two taps with bias
TINY_E = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 777, "hidden_size": 192, "intermediate_size": 448, "block_auto_adjust_ff_dim": False,
    "num_hidden_layers": 3, "layer_types": ["full_attention", "conv", "full_attention"],
    "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 128,
    "conv_L_cache": 2, "conv_bias": True, "rope_theta": 10000.0, "norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 512, "eos_token_id": 3,
}


def serving_width_config(sizes: str, layers=("conv", "full_attention", "conv"), vocab: int = 4096) -> dict:
    """A few layers with the widths of the 1.2B model (hidden 2048, 32 heads over 8 kv heads of 64,
    feed-forward 8192) or of the 700M model (hidden 1536, 24 heads, feed-forward 6912: three query
    heads per kv head, widths that are no power of two): the shapes the serving kernels are tuned for."""
    hidden, heads, inter = {"1.2b": (2048, 32, 12288), "700m": (1536, 24, 10240)}[sizes]
    return {
        "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "vocab_size": vocab, "hidden_size": hidden,
        "intermediate_size": inter, "block_auto_adjust_ff_dim": True, "block_ffn_dim_multiplier": 1.0,
        "block_multiple_of": 256, "num_hidden_layers": len(layers), "layer_types": list(layers),
        "num_attention_heads": heads, "num_key_value_heads": 8, "head_dim": 64, "conv_L_cache": 3, "conv_bias": False,
        "rope_theta": 1000000.0, "norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 1024,
    }


@pytest.fixture(scope="session")
def tiny_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, float32 weights (perturbed norm weights so a
    dropped norm weight shows)."""
    from vapi_b200.weights import write_random_model
    out = {}
    for name, cfg, seed in (("A", TINY_A, 0), ("B", TINY_B, 2), ("C", TINY_C, 4), ("D", TINY_D, 6),
                            ("E", TINY_E, 8), ("A0", TINY_A0, 0), ("B0", TINY_B0, 2)):
        d = tmp_path_factory.mktemp(f"tiny{name}")
        # std 0.2 / perturbed norms as the reference's golden generator uses
        # (tools/gen_lfm2_goldens.py:27-49): activations large enough that faults show.
        # (A and A0 as worded: N(0, 0.02) with norm weights of one; B0 as worded: N(0, 0.02))
        write_random_model(str(d), cfg, seed, std={"A": 0.02, "A0": 0.02, "B0": 0.02, "D": 0.1, "E": 0.1}.get(name, 0.2),
                           norm_init="perturbed" if name not in ("A", "A0") else "ones", dtype=torch.float32)
        out[name] = str(d)
    return out


@pytest.fixture()
def plain_kernels(monkeypatch):
    """Stand the plain restatements in for the CUDA kernels so that host-side logic can run
    on a CPU.  Test-only: the package itself refuses CPU tensors."""
    import plain_ops
    from vapi_b200 import ops
    for name in plain_ops.ALL:
        monkeypatch.setattr(ops, name, getattr(plain_ops, name))
    return plain_ops
