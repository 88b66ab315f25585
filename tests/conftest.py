"""Shared fixtures: the tiny configurations, model folders with random weights, GPU marker."""
from __future__ import annotations

import os
import sys

import pytest
import torch

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


# Two tiny configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 4, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "intermediate_size_mlp": 256,
    "num_local_experts": 4, "num_experts_per_tok": 1, "interleave_moe_layer_step": 1,
    "rope_theta": 10000.0, "rope_scaling": None, "no_rope_layers": [3], "attention_chunk_size": 16,
    "use_qk_norm": True, "qk_norm_eps": 1e-6, "attn_temperature_tuning": True, "floor_scale": 8,
    "attn_scale": 0.1, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}
TINY_A_INIT = {"seed": 0, "std": 0.02, "norm_std": 0.1}

TINY_B = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 384, "hidden_size": 96, "num_hidden_layers": 6, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 64, "intermediate_size_mlp": 192,
    "num_local_experts": 8, "num_experts_per_tok": 1, "interleave_moe_layer_step": 2,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 16},
    "no_rope_layers": [2, 5], "attention_chunk_size": 32, "use_qk_norm": False,
    "attn_temperature_tuning": False, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
}
TINY_B_INIT = {"seed": 1, "std": 0.05, "norm_std": 0.0}

# A third one with sizes that are no power of two anywhere, tied embeddings, biased attention projections and
# the flag form of no_rope_layers: hidden 88, 6 heads in 3 groups, head size 48, vocabulary 301.
TINY_C = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 301, "hidden_size": 88, "num_hidden_layers": 3, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 48, "intermediate_size": 40, "intermediate_size_mlp": 104,
    "num_local_experts": 3, "num_experts_per_tok": 1, "moe_layers": [0, 2], "interleave_moe_layer_step": 1,
    "rope_theta": 1000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                     "original_max_position_embeddings": 24},
    "no_rope_layers": [1, 0, 1], "attention_chunk_size": 24, "use_qk_norm": True, "qk_norm_eps": 1e-5,
    "attn_temperature_tuning": True, "floor_scale": 5, "attn_scale": 0.25, "rms_norm_eps": 1e-4,
    "tie_word_embeddings": True, "attention_bias": True,
}
TINY_C_INIT = {"seed": 2, "std": 0.08, "norm_std": 0.2}

# A fourth with head size 64, which (with pages of 16 or more positions) takes the kernels that
# fetch keys and values by TMA; 5 query heads share each kv head as in the large models.
TINY_D = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 200, "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 10,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 48, "intermediate_size_mlp": 96,
    "num_local_experts": 2, "num_experts_per_tok": 1, "interleave_moe_layer_step": 2,
    "rope_theta": 20000.0, "rope_scaling": None, "no_rope_layers": [1], "attention_chunk_size": 48,
    "use_qk_norm": True, "attn_temperature_tuning": True, "floor_scale": 20, "attn_scale": 0.2,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}
TINY_D_INIT = {"seed": 3, "std": 0.04, "norm_std": 0.1}

# The shapes of the large models in small: head size 128 with five query heads to a kv head, pages of 64
# positions, a chunk of 512, the Scout rope scaling, and a prompt long enough (1400 rows in one step) for the
# kernels that only large steps reach: attention tiles of 128 rows on tcgen05, the persistent grouped product,
# two weight tiles per CTA in the down product.
LARGE_SHAPES = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 1000, "hidden_size": 640, "num_hidden_layers": 4, "num_attention_heads": 10,
    "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 384, "intermediate_size_mlp": 512,
    "num_local_experts": 4, "num_experts_per_tok": 1, "interleave_moe_layer_step": 1,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192},
    "no_rope_layers": [3], "attention_chunk_size": 512, "use_qk_norm": True, "attn_temperature_tuning": True,
    "floor_scale": 512, "attn_scale": 0.1, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}


# The layer widths of the large models themselves, two layers deep: a dense SwiGLU layer of Maverick's width
# with chunked RoPE attention, then a mixture layer with global attention; few experts and a small vocabulary
# keep it at 2 GB.
REAL_WIDTHS = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 2048, "hidden_size": 5120, "num_hidden_layers": 2, "num_attention_heads": 40,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 8192, "intermediate_size_mlp": 16384,
    "num_local_experts": 4, "num_experts_per_tok": 1, "interleave_moe_layer_step": 2,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192},
    "no_rope_layers": [1], "attention_chunk_size": 512, "use_qk_norm": True, "attn_temperature_tuning": True,
    "floor_scale": 512, "attn_scale": 0.1, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}


# The mixtures of the large models at reduced width: 16 experts on every layer (Scout's count), and dense layers
# alternating with layers of 128 experts (Maverick's arrangement); head size 128 in groups of five, pages of 64.
EXPERTS_16 = dict(LARGE_SHAPES, num_hidden_layers=2, num_local_experts=16, intermediate_size=256, no_rope_layers=[1],
                  interleave_moe_layer_step=1)
EXPERTS_128 = dict(LARGE_SHAPES, num_hidden_layers=2, num_local_experts=128, intermediate_size=128,
                   intermediate_size_mlp=768, no_rope_layers=[1], interleave_moe_layer_step=2)

# The benchmark's own attention constants at a small width: chunks of 8192 positions, the temperature factor
# stepping at 8192, the Scout rope scaling; a chunked rotary layer with a dense feed-forward, then a global layer
# with 16 experts.  A request of 8300 tokens crosses the chunk's edge.
CHUNK_EDGE = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 500, "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 2,
    "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 64, "intermediate_size_mlp": 128,
    "num_local_experts": 16, "num_experts_per_tok": 1, "interleave_moe_layer_step": 2,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192},
    "no_rope_layers": [1], "attention_chunk_size": 8192, "use_qk_norm": True, "attn_temperature_tuning": True,
    "floor_scale": 8192, "attn_scale": 0.1, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}


TINY = {"A": (TINY_A, TINY_A_INIT), "B": (TINY_B, TINY_B_INIT), "C": (TINY_C, TINY_C_INIT), "D": (TINY_D, TINY_D_INIT)}


def make_model_dir(tmp_path_factory, name: str, store_dtype: str = "bfloat16") -> str:
    from sharpinference_b200.weights import write_random_model
    cfg, init = TINY[name]
    out = str(tmp_path_factory.mktemp(f"tiny_{name}_{store_dtype}"))
    write_random_model(dict(cfg), out, init["seed"], std=init["std"], norm_std=init["norm_std"],
                       store_dtype=store_dtype)
    return out


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders (bfloat16 weights) of the tiny configurations, made once per session."""
    return {name: make_model_dir(tmp_path_factory, name) for name in TINY}
