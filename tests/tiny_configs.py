"""The two tiny configurations of the architecture that the tests use.  They differ in every
size and option: head counts and group size (2 vs 3), head size (16 vs 32; 4*16 = hidden vs
6*32 != hidden), widths that are no power of two, number of layers, vocabulary, the norms' eps,
the rotary base, tied vs untied head and the longest context."""

TINY_A = {
    "arch": "transformer",
    "vocab_size": 256,
    "hidden_size": 64,
    "intermediate_size": 192,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0,
    "tie_word_embeddings": True,
    "initializer_range": 0.02,
    "max_position_embeddings": 128,
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "vocab_size": 384,
    "hidden_size": 80,
    "intermediate_size": 224,
    "num_hidden_layers": 3,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 32,
    "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0,
    "tie_word_embeddings": False,
    "initializer_range": 0.02,
    "max_position_embeddings": 256,
}

# A third small model whose head size (64) is one the bfloat16 tensor-core attention kernels take,
# so that the engine's fast paths run in the replay tests too (group of 4, untied, another eps).
TINY_C = {
    "arch": "transformer",
    "vocab_size": 320,
    "hidden_size": 96,
    "intermediate_size": 160,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 1,
    "head_dim": 64,
    "rms_norm_eps": 3e-6,
    "rope_theta": 100000.0,
    "tie_word_embeddings": False,
    "initializer_range": 0.02,
    "max_position_embeddings": 512,
}
