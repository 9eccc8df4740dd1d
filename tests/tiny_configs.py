"""Tiny configurations of the architecture for the tests; they differ in every size and
option.  A and B are the two tiny configurations the benchmark description names; C adds a
window on the upper layers (two cache groups), an odd vocabulary, a head size that is not
hidden / heads, a single kv head, no q/k/v bias, no shared expert and a dense layer named
by ``mlp_only_layers``."""
import copy
import os

import torch

TINY_A = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 4,
    "head_dim": 16, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 256, "decoder_sparse_step": 1, "num_experts": 8, "num_experts_per_tok": 2,
    "norm_topk_prob": False, "moe_intermediate_size": 32, "shared_expert_intermediate_size": 64,
    "intermediate_size": 96, "qkv_bias": True, "tie_word_embeddings": False, "use_sliding_window": False,
    "mlp_only_layers": [], "hidden_act": "silu", "eos_token_id": -1,
}

TINY_B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 32, "vocab_size": 512, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "max_position_embeddings": 512, "decoder_sparse_step": 2, "num_experts": 12, "num_experts_per_tok": 3,
    "norm_topk_prob": True, "moe_intermediate_size": 48, "shared_expert_intermediate_size": 128,
    "intermediate_size": 256, "qkv_bias": True, "tie_word_embeddings": True, "use_sliding_window": False,
    "mlp_only_layers": [], "hidden_act": "silu", "eos_token_id": -1,
}

TINY_C = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 4, "hidden_size": 120, "num_attention_heads": 5, "num_key_value_heads": 1,
    "head_dim": 48, "vocab_size": 331, "rope_theta": 500000.0, "rms_norm_eps": 3e-6,
    "max_position_embeddings": 640, "decoder_sparse_step": 1, "num_experts": 5, "num_experts_per_tok": 2,
    "norm_topk_prob": True, "moe_intermediate_size": 40, "shared_expert_intermediate_size": 0,
    "intermediate_size": 136, "qkv_bias": False, "tie_word_embeddings": False, "use_sliding_window": True,
    "sliding_window": 24, "max_window_layers": 2, "mlp_only_layers": [1], "hidden_act": "silu",
    "eos_token_id": -1,
}

# Head size 128 (the size of the tcgen05 attention kernel), otherwise small; used by the tests that run
# long portions through the engine with pages of 64 tokens.
TINY_D = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 128, "vocab_size": 211, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 1024, "decoder_sparse_step": 1, "num_experts": 6, "num_experts_per_tok": 2,
    "norm_topk_prob": False, "moe_intermediate_size": 24, "shared_expert_intermediate_size": 48,
    "intermediate_size": 64, "qkv_bias": True, "tie_word_embeddings": True, "use_sliding_window": False,
    "mlp_only_layers": [], "hidden_act": "silu", "eos_token_id": -1,
}

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
SEEDS = {"A": 0, "B": 1, "C": 5, "D": 9}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def make_model_dir(tmp_path, name: str, store_dtype=torch.bfloat16, seed=None, raw=None) -> str:
    """Write the random-weights folder of a tiny configuration into a temporary folder."""
    from locus_b200.weights.loader import write_random_model
    import locus_b200.models  # noqa: F401  (registers the architecture)

    d = os.path.join(str(tmp_path), f"tiny_{name}_{str(store_dtype).split('.')[-1]}")
    write_random_model(raw if raw is not None else config(name), SEEDS.get(name, 7) if seed is None else seed,
                       d, store_dtype)
    return d


def random_tokens(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
