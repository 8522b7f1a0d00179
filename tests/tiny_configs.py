"""The two tiny StarCoder2 configurations of the tests, differing in every size and option,
and helpers that write them as model folders with seeded random weights."""

from __future__ import annotations

import torch

from matricxon_b200.config.registry import config_from_dict
from matricxon_b200.weights.random_init import RandomInit, random_tensors, write_random_model

TINY_A = {
    "model_type": "starcoder2", "architectures": ["Starcoder2ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 256, "vocab_size": 512, "rope_theta": 10000.0,
    "sliding_window": 32, "max_position_embeddings": 128, "norm_epsilon": 1e-5,
    "use_bias": True, "tie_word_embeddings": True, "hidden_act": "gelu_pytorch_tanh",
}
INIT_A = RandomInit(weight_std=0.02, bias_std=0.02, norm_weight_std=0.02, norm_bias_std=0.02)
SEED_A = 0

TINY_B = {
    "model_type": "starcoder2", "architectures": ["Starcoder2ForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 352, "vocab_size": 1000, "rope_theta": 100000.0,
    "sliding_window": 24, "max_position_embeddings": 256, "norm_epsilon": 1e-6,
    "use_bias": False, "tie_word_embeddings": False, "hidden_act": "gelu_pytorch_tanh",
}
INIT_B = RandomInit(weight_std=0.02, bias_std=0.0, norm_weight_std=0.0, norm_bias_std=0.0)
SEED_B = 1

TINY = {"A": (TINY_A, INIT_A, SEED_A), "B": (TINY_B, INIT_B, SEED_B)}


def tiny_config(name: str):
    return config_from_dict(dict(TINY[name][0]))


def tiny_tensors(name: str, store_dtype=torch.float32, weight_scale: float = 1.0):
    raw, init, seed = TINY[name]
    if weight_scale != 1.0:
        init = RandomInit(init.weight_std * weight_scale, init.bias_std, init.norm_weight_std,
                          init.norm_bias_std)
    return random_tensors(config_from_dict(dict(raw)), seed, init, store_dtype)


def write_tiny_model(folder, name: str, store_dtype=torch.float32, weight_scale: float = 1.0):
    raw, init, seed = TINY[name]
    if weight_scale != 1.0:
        init = RandomInit(init.weight_std * weight_scale, init.bias_std, init.norm_weight_std,
                          init.norm_bias_std)
    return write_random_model(folder, config_from_dict(dict(raw)), seed, init, store_dtype)


def random_ids(count: int, vocab: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()
