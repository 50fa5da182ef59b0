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

# The tiny_c model with room for sequences beyond 12,288 tokens, where decode attention cuts a sequence into more
# pieces than a cluster holds and merges them through scratch memory and a second kernel.
TINY_LONG = {**TINY_C, "max_position_embeddings": 12928}

# The layer sizes of the three benchmark configurations (Qwen3-0.6B, 4B and 8B sizes) with few layers and a small
# vocabulary, so that the plain implementation stays fast: at these sizes the engine takes the kernels that the
# benchmark times (head size 128: tcgen05 prefill attention; the q|k|v product with its fused output stage; the
# persistent, paired and library products; the few-token and swap-AB products of decode).
REAL_06B = {
    "arch": "transformer", "vocab_size": 3000, "hidden_size": 1024, "intermediate_size": 3072, "num_hidden_layers": 2,
    "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": True, "initializer_range": 0.02, "max_position_embeddings": 2048,
}
REAL_4B = {
    "arch": "transformer", "vocab_size": 2200, "hidden_size": 2560, "intermediate_size": 9728, "num_hidden_layers": 1,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": True, "initializer_range": 0.02, "max_position_embeddings": 2048,
}
REAL_8B = {
    "architectures": ["Qwen3ForCausalLM"], "vocab_size": 2500, "hidden_size": 4096, "intermediate_size": 12288,
    "num_hidden_layers": 1, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "tie_word_embeddings": False, "initializer_range": 0.02, "max_position_embeddings": 2048,
}
