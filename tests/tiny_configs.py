"""Tiny Qwen2 configurations for tests.  They differ in every size and option:
layers, width, head counts and groups, head size (given / derived), intermediate
size, vocabulary, rope theta, norm eps, tied / untied head, eos as int / list,
and a key window on some layers (tiny C only; Azimml/shrike itself never windows)."""

TINY_A = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2",
    hidden_size=64, intermediate_size=128, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256,
    rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True,
    max_position_embeddings=4096, eos_token_id=[255], torch_dtype="float32",
)

TINY_B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2",
    hidden_size=192, intermediate_size=320, num_hidden_layers=3,
    num_attention_heads=6, num_key_value_heads=3, vocab_size=384,
    rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False,
    max_position_embeddings=4096, eos_token_id=383, torch_dtype="float32",
)

# Width 240 = 5 heads of 48: nothing is a power of two; one kv head (multi-query),
# vocabulary 331 (odd, prime), a window of 24 keys on layers 1.. (layer 0 sees all).
TINY_C = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2",
    hidden_size=240, intermediate_size=176, num_hidden_layers=4,
    num_attention_heads=5, num_key_value_heads=1, vocab_size=331,
    rms_norm_eps=3e-6, rope_theta=50000.0, tie_word_embeddings=False,
    use_sliding_window=True, sliding_window=24, max_window_layers=1,
    max_position_embeddings=4096, eos_token_id=330, torch_dtype="float32",
)

# Heads of 64: the head size (with 128) that the tensor-core attention kernel for portions and the
# page-wise single-token kernel serve, so that a replay goes through them; width 384,
# six query heads on two kv heads, vocabulary 509 (prime), untied.
TINY_D = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2",
    hidden_size=384, intermediate_size=416, num_hidden_layers=2,
    num_attention_heads=6, num_key_value_heads=2, head_dim=64, vocab_size=509,
    rms_norm_eps=2e-6, rope_theta=300000.0, tie_word_embeddings=False,
    max_position_embeddings=4096, eos_token_id=[508, 507], torch_dtype="float32",
)

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3}
PAGE_SIZES = {"A": 16, "B": 8, "C": 16, "D": 16}


def windows_of(raw: dict) -> dict:
    """layer -> window, as the Qwen2 reader of the package interprets the keys."""
    if not raw.get("use_sliding_window"):
        return {}
    first = raw.get("max_window_layers", raw["num_hidden_layers"])
    return {layer: raw["sliding_window"] for layer in range(first, raw["num_hidden_layers"])}
