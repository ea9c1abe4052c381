"""The tiny configurations the tests run on.  They differ in every size and option: layer count,
widths, grouped vs multi-query heads, q width equal / unequal to the hidden size, head size, theta,
eps, tying, an odd vocabulary, the window.  A and B are the ones the golden outputs of the reference's
CPU model exist for; C adds windowed layers mixed with full ones, which the reference does not have; D has
the head size (64) that puts prompt portions on the tcgen05 attention kernel in bfloat16; E has head size 128 with
four query heads per key/value head - the kernel specialisations of the large Qwen3 shapes - a q width (1024) far
from the hidden size, and a long context."""
from pulse_infer_b200.config import Qwen3Config

TINY_A = Qwen3Config(
    architecture="Qwen3ForCausalLM", hidden_size=64, intermediate_size=128, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256, max_position_embeddings=128,
    rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True, torch_dtype="bfloat16", eos_token_ids=(0,))

TINY_B = Qwen3Config(
    architecture="Qwen3ForCausalLM", hidden_size=96, intermediate_size=224, num_hidden_layers=3,
    num_attention_heads=8, num_key_value_heads=1, head_dim=32, vocab_size=515, max_position_embeddings=256,
    rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False, torch_dtype="bfloat16", eos_token_ids=(1, 2))

TINY_C = Qwen3Config(
    architecture="Qwen3ForCausalLM", hidden_size=80, intermediate_size=176, num_hidden_layers=4,
    num_attention_heads=6, num_key_value_heads=2, head_dim=48, vocab_size=301, max_position_embeddings=512,
    rms_norm_eps=3e-6, rope_theta=50000.0, tie_word_embeddings=False, torch_dtype="bfloat16", eos_token_ids=(7,),
    layer_types=("full_attention", "sliding_attention", "sliding_attention", "full_attention"), sliding_window=24)

TINY_D = Qwen3Config(
    architecture="Qwen3ForCausalLM", hidden_size=112, intermediate_size=208, num_hidden_layers=2,
    num_attention_heads=6, num_key_value_heads=3, head_dim=64, vocab_size=333, max_position_embeddings=1024,
    rms_norm_eps=2e-6, rope_theta=20000.0, tie_word_embeddings=True, torch_dtype="bfloat16", eos_token_ids=(3,),
    layer_types=("sliding_attention", "full_attention"), sliding_window=150)

TINY_E = Qwen3Config(
    architecture="Qwen3ForCausalLM", hidden_size=320, intermediate_size=712, num_hidden_layers=2,
    num_attention_heads=8, num_key_value_heads=2, head_dim=128, vocab_size=2077, max_position_embeddings=4096,
    rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, torch_dtype="bfloat16", eos_token_ids=(5,))

SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}

# Random weights give every key about the same score, so a key that a kernel skips or reads twice moves the output
# by little.  The folder of E therefore has its per-head query norm weights scaled: scores spread out, a few keys
# (anywhere in the context) carry most of the weight, and a wrong far key shows in the logits.
QUERY_NORM_SCALE = {"E": (2.0, 1.5)}       # per layer
