"""Tiny configurations of the architecture for the tests.  A and B differ in every size and
option; C adds an execution order that names layers twice and a position that reads another
position's cache, with sizes that are multiples of neither 16 (width) nor a power of two."""
import copy

TINY_A = {
    "architectures": ["FlintForCausalLM"],
    "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "vocab_size": 256, "n_routed_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 32,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": False, "scoring_func": "softmax",
    "norm_topk_prob": True, "qk_norm": False, "attn_sinks": False, "kv_page_size": 4,
}

TINY_B = {
    "architectures": ["FlintForCausalLM"],
    "hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32,
    "vocab_size": 384, "n_routed_experts": 16, "num_experts_per_tok": 4, "moe_intermediate_size": 48,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": True, "scoring_func": "sigmoid",
    "norm_topk_prob": False, "qk_norm": True, "attn_sinks": True,
    "sliding_window": 9, "sliding_window_pattern": [True, False, True], "rope_pattern": [True, False, True],
    "n_shared_experts": 1, "shared_expert_intermediate_size": 96,
    "first_k_dense_replace": 1, "intermediate_size": 80, "kv_page_size": 8,
}

TINY_C = {
    "architectures": ["FlintForCausalLM"],
    "hidden_size": 72, "num_hidden_layers": 2, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 48,
    "vocab_size": 250, "n_routed_experts": 6, "num_experts_per_tok": 3, "moe_intermediate_size": 40,
    "rms_norm_eps": 3e-6, "rope_theta": 25000.0, "tie_word_embeddings": False, "scoring_func": "sigmoid",
    "norm_topk_prob": True, "qk_norm": True, "attn_sinks": False,
    "sliding_window": 21, "sliding_window_pattern": [False, True], "rope_pattern": [True, True],
    "layer_order": [0, 1, 0, 1], "kv_source": [None, None, 0, None], "kv_page_size": 16,
}

# the head size and widths at which the bfloat16 path runs its tcgen05 / TMA kernels (not among the fixtures' names:
# one test replays it)
SMALL_D = {
    "architectures": ["FlintForCausalLM"],
    "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128,
    "vocab_size": 1000, "n_routed_experts": 16, "num_experts_per_tok": 4, "moe_intermediate_size": 128,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": False, "scoring_func": "softmax",
    "norm_topk_prob": True, "qk_norm": True, "attn_sinks": True, "kv_page_size": 16,
}

# the same with every option the other way: a window on two of three layers, groups of 8 query heads, sigmoid scores
# without renormalisation, a shared expert, a dense first layer, tied embeddings, pages of 32, no power of two in sight
SMALL_E = {
    "architectures": ["FlintForCausalLM"],
    "hidden_size": 384, "num_hidden_layers": 3, "num_attention_heads": 16, "num_key_value_heads": 2, "head_dim": 128,
    "vocab_size": 777, "n_routed_experts": 24, "num_experts_per_tok": 6, "moe_intermediate_size": 192,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": True, "scoring_func": "sigmoid",
    "norm_topk_prob": False, "qk_norm": False, "attn_sinks": False,
    "sliding_window": 500, "sliding_window_pattern": [True, False, True], "rope_pattern": [True, False, True],
    "n_shared_experts": 1, "shared_expert_intermediate_size": 256,
    "first_k_dense_replace": 1, "intermediate_size": 320, "kv_page_size": 32,
}

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": SMALL_D, "E": SMALL_E}
# norm weights: ones for A (as its description says), 1 + noise for the others so that a missing
# multiplication by the weight shows
NORM_INIT = {"A": "ones", "B": "random", "C": "random", "D": "random", "E": "random"}


def get(name):
    return copy.deepcopy(ALL[name])
