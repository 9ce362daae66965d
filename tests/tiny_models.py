"""The small configurations the tests run on, and helpers to write them as model
folders.  They differ in every size and option: head counts and grouping, head
size, widths that are no power of two, depth, vocabulary, eps, rotary base and
scaling, tied or untied head, weight scale."""

import os
import tempfile

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 176, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
    "max_position_embeddings": 128, "tie_word_embeddings": True, "hidden_act": "silu",
    "eos_token_id": 255,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 1000, "hidden_size": 192, "intermediate_size": 512, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 32,
    "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "max_position_embeddings": 256, "tie_word_embeddings": False, "hidden_act": "silu",
    "eos_token_id": [998, 999],
}
# head size 48 (a multiple of 16 that is no power of two), no grouping, width that
# is not heads * head size
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 777, "hidden_size": 208, "intermediate_size": 336, "num_hidden_layers": 2,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48,
    "rms_norm_eps": 3e-5, "rope_theta": 100000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 2.0, "original_max_position_embeddings": 32},
    "max_position_embeddings": 192, "tie_word_embeddings": False, "hidden_act": "silu",
}

# head size 64, feed-forward width a multiple of 64: the sizes at which the bfloat16 engine
# takes its tensor-core kernels (flash attention, cluster decode attention, tcgen05 products
# with the SwiGLU epilogue)
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 515, "hidden_size": 256, "intermediate_size": 384, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
    "max_position_embeddings": 320, "tie_word_embeddings": True, "hidden_act": "silu",
}
# head size 128, groups of three query heads, width that is not heads * head size
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 300, "hidden_size": 160, "intermediate_size": 200, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128,
    "rms_norm_eps": 2e-6, "rope_theta": 50000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 2.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 128},
    "max_position_embeddings": 320, "tie_word_embeddings": False, "hidden_act": "silu",
}

CONFIGS = {"tiny_a": (TINY_A, 0, 0.02), "tiny_b": (TINY_B, 1, 0.05), "tiny_c": (TINY_C, 2, 0.08),
           "tiny_d": (TINY_D, 3, 0.05), "tiny_e": (TINY_E, 4, 0.06)}

_made = {}


def model_dir(name, storage="float32"):
    """Writes (once per process) the named tiny model with random weights into a
    temporary folder and returns the path."""
    key = (name, storage)
    if key not in _made:
        from kv_cache_optimization_for_llm_b200.weights import write_random_model
        cfg, seed, std = CONFIGS[name]
        d = tempfile.mkdtemp(prefix=f"kvb200_{name}_{storage}_")
        write_random_model(d, cfg, seed, std, storage_dtype=storage)
        _made[key] = d
    return _made[key]
