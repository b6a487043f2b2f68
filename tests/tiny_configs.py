"""The two tiny configurations the tests use.  They differ in every size and option: layers,
width, heads and key/value groups (2:1 grouped against a single shared head), head size,
feed-forward width (176 is no multiple of 64), vocabulary, rope base, norm eps, context, and
tied against untied output embeddings."""

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 64, "intermediate_size": 176, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "vocab_size": 256, "max_position_embeddings": 128, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "vocab_size": 384, "max_position_embeddings": 256, "rope_theta": 500000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "hidden_act": "silu",
}

# A third one for longer sequences: head size 48 (a step of 16 that is no power of two),
# width that is no power of two, vocabulary that is no multiple of 8, context 1024.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 120, "intermediate_size": 200, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48,
    "vocab_size": 331, "max_position_embeddings": 1024, "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "hidden_act": "silu",
}

# A fourth one with the head size of the large models (128) and as many key/value heads as query
# heads, for sequences of many cache pages.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 256, "intermediate_size": 344, "num_hidden_layers": 2,
    "num_attention_heads": 2, "num_key_value_heads": 2, "head_dim": 128,
    "vocab_size": 1000, "max_position_embeddings": 2048, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
}

# Head sizes the other four do not have: 80 (a step of 16 between the kernels' instantiations for 64
# and 128, padded inside them) with five query heads on one key/value head, and 256 (the largest
# allowed; prefill attention then runs on the mma.sync kernel), widths and vocabularies that are
# no powers of two.
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 200, "intermediate_size": 312, "num_hidden_layers": 2,
    "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 80,
    "vocab_size": 515, "max_position_embeddings": 512, "rope_theta": 20000.0,
    "rms_norm_eps": 2e-6, "tie_word_embeddings": True, "hidden_act": "silu",
}

TINY_F = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 264, "intermediate_size": 400, "num_hidden_layers": 1,
    "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 256,
    "vocab_size": 777, "max_position_embeddings": 640, "rope_theta": 300000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
}
