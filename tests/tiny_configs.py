"""The tiny configurations the tests use: they differ in every size and option.

  TINY_LLAMA   model_type llama: 2 layers, D 64, 4 heads / 2 kv heads, head 16, I 128, V 256, theta 1e4 with llama3
               scaling whose original length (32) puts the scaled, the blended and the untouched band all inside 128
               positions, eps 1e-5, no bias, own output matrix, norm weights 1
  TINY_QWEN2   model_type qwen2: 3 layers, D 96, 3 heads / 1 kv head, head 32, I 256, V 384, theta 1e6 plain, eps 1e-6,
               q/k/v bias, tied embeddings, norm weights 1 + noise
  TINY_WINDOW  model_type qwen2 with a sliding window of 12 on layers 0 and 2 of 3 (layer 1 sees every key): 5 heads /
               5 kv heads, head 48 (no power of two), D 80, I 176, V 509 (a prime), linear rope scaling
"""
import copy

TINY_LLAMA = {
    "model_type": "llama", "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 256, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "max_position_embeddings": 128, "tie_word_embeddings": False, "hidden_act": "silu",
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
}
TINY_QWEN2 = {
    "model_type": "qwen2", "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "vocab_size": 384, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "max_position_embeddings": 256, "tie_word_embeddings": True, "hidden_act": "silu",
}
TINY_WINDOW = {
    "model_type": "qwen2", "hidden_size": 80, "intermediate_size": 176, "num_hidden_layers": 3,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48, "vocab_size": 509, "rms_norm_eps": 3e-6,
    "rope_theta": 50000.0, "max_position_embeddings": 512, "tie_word_embeddings": False, "hidden_act": "silu",
    "rope_scaling": {"rope_type": "linear", "factor": 2.0},
    "use_sliding_window": True, "sliding_window": 12,
    "layer_types": ["sliding_attention", "full_attention", "sliding_attention"],
}
# head sizes the tensor-core attention kernels take (64 and 128), with the groups of Qwen2.5-0.5B (7) and Llama-3.1 (4)
TINY_HD64 = {
    "model_type": "qwen2", "hidden_size": 136, "intermediate_size": 264, "num_hidden_layers": 2,
    "num_attention_heads": 14, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 331, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "max_position_embeddings": 1024, "tie_word_embeddings": True, "hidden_act": "silu",
    "use_sliding_window": True, "sliding_window": 150, "layer_types": ["full_attention", "sliding_attention"],
}
TINY_HD128 = {
    "model_type": "llama", "hidden_size": 256, "intermediate_size": 384, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 128, "vocab_size": 300, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0, "max_position_embeddings": 1024, "tie_word_embeddings": False, "hidden_act": "silu",
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
}
CONFIGS = {"tiny_llama": (TINY_LLAMA, dict(seed=0, norm_noise=False, page_size=4)),
           "tiny_qwen2": (TINY_QWEN2, dict(seed=7, norm_noise=True, page_size=8)),
           "tiny_window": (TINY_WINDOW, dict(seed=11, norm_noise=True, page_size=4)),
           "tiny_hd64": (TINY_HD64, dict(seed=13, norm_noise=True, page_size=16)),
           "tiny_hd128": (TINY_HD128, dict(seed=17, norm_noise=False, page_size=16))}


def get(name: str):
    c, o = CONFIGS[name]
    return copy.deepcopy(c), dict(o)
