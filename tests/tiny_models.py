"""Two tiny LFM2 configurations that differ in every size and option, and helpers that write
them as model folders with random weights into a temporary place."""
from __future__ import annotations

import copy

TINY_A = {
    "model_type": "lfm2", "architectures": ["Lfm2ForCausalLM"], "vocab_size": 512, "hidden_size": 64,
    "num_hidden_layers": 4, "num_attention_heads": 4, "num_key_value_heads": 2,
    "max_position_embeddings": 256, "norm_eps": 1e-5, "conv_L_cache": 3, "rope_theta": 10000.0,
    "layer_types": ["conv", "conv", "full_attention", "conv"], "tie_word_embeddings": True,
    "block_ff_dim": 192, "block_auto_adjust_ff_dim": False, "conv_bias": False,
    "bos_token_id": 1, "eos_token_id": 7, "pad_token_id": 0,
}

TINY_B = {
    "model_type": "lfm2", "vocab_size": 1000, "hidden_size": 96, "num_hidden_layers": 6,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "max_position_embeddings": 512, "norm_eps": 1e-6, "conv_L_cache": 4, "rope_theta": 1000000.0,
    "layer_types": ["full_attention", "conv", "conv", "full_attention", "conv", "full_attention"],
    "tie_word_embeddings": False, "intermediate_size": 256,
    "bos_token_id": 1, "eos_token_id": [7, 9], "pad_token_id": 0,
}

# sizes that are no power of two anywhere, head size 48, 5 query heads on 5 kv heads (no grouping),
# a two-tap kernel, layers named only by full_attn_idxs
TINY_C = {
    "model_type": "lfm2", "vocab_size": 777, "hidden_size": 80, "num_hidden_layers": 3,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48,
    "max_position_embeddings": 384, "norm_eps": 3e-6, "conv_L_cache": 2, "rope_theta": 50000.0,
    "full_attn_idxs": [1], "tie_word_embeddings": True, "intermediate_size": 136,
    "bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0,
}

# the head size of the full models (64), which selects the tcgen05 kernels for prompt portions: six query heads
# on two kv heads, two attention layers beside one conv layer
TINY_D = {
    "model_type": "lfm2", "vocab_size": 600, "hidden_size": 192, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64,
    "max_position_embeddings": 512, "norm_eps": 1e-5, "conv_L_cache": 3, "rope_theta": 1000000.0,
    "layer_types": ["full_attention", "conv", "full_attention"], "tie_word_embeddings": True,
    "intermediate_size": 320, "bos_token_id": 1, "eos_token_id": 7, "pad_token_id": 0,
}

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3)}


def write_tiny(tmp_path, name: str, dtype=None) -> str:
    import torch
    from celeg_b200.weights import write_random_model
    raw, seed = CONFIGS[name]
    folder = str(tmp_path / f"tiny_{name}")
    write_random_model(folder, copy.deepcopy(raw), seed, dtype or torch.bfloat16)
    return folder
