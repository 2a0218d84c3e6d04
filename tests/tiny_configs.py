"""Small Qwen2 configurations for the tests; they differ in every size and option."""

from __future__ import annotations


def _base(**overrides):
    config = dict(
        architectures=["Qwen2ForCausalLM"],
        model_type="qwen2",
        hidden_act="silu",
        max_position_embeddings=4096,
        use_sliding_window=False,
    )
    config.update(overrides)
    return config


# 2 layers, 4 q heads on 2 kv heads of 16, tied head, theta 1e4, eps 1e-6 (page 4 in the tests)
TINY_A = _base(
    hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    intermediate_size=176, vocab_size=512, rope_theta=10000.0, rms_norm_eps=1e-6,
    attention_bias=True, tie_word_embeddings=True, eos_token_id=511,
)

# 3 layers, 2 q heads on 1 kv head of 64, head of its own, theta 1e6, eps 1e-5 (page 8)
TINY_B = _base(
    hidden_size=128, num_hidden_layers=3, num_attention_heads=2, num_key_value_heads=1,
    intermediate_size=320, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-5,
    attention_bias=True, tie_word_embeddings=False, eos_token_id=999,
)

# 1 layer, width 96 with an explicit head size of 32 (3 heads, no grouping), odd vocabulary,
# no biases, theta 5e5 (page 16)
TINY_C = _base(
    hidden_size=96, num_hidden_layers=1, num_attention_heads=3, num_key_value_heads=3,
    head_dim=32, intermediate_size=208, vocab_size=331, rope_theta=500000.0, rms_norm_eps=1e-5,
    attention_bias=False, tie_word_embeddings=True, eos_token_id=330,
)

# 2 layers, 8 q heads on 1 kv head of 128 (the production head size and grouping), page 16
TINY_D = _base(
    hidden_size=1024, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=1,
    intermediate_size=408, vocab_size=777, rope_theta=1000000.0, rms_norm_eps=1e-6,
    attention_bias=True, tie_word_embeddings=True, eos_token_id=776,
)

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
PAGE_SIZE = {"A": 4, "B": 8, "C": 16, "D": 16}
SEED = {"A": 11, "B": 22, "C": 33, "D": 44}
