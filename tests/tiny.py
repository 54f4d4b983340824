"""The tiny configurations the tests use: they differ in every size and option."""
import json
import os

import torch

# 2 layers, width 64, 4 heads over 2 kv heads (group 2), head size 16 = width/heads,
# tied output head, theta 1e4, eps 1e-6
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=192, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
    max_position_embeddings=128, tie_word_embeddings=True, hidden_act="silu", attention_bias=False,
    use_sliding_window=False, sliding_window=None, eos_token_id=7)
TINY_A_INIT = dict(seed=0, std_matrix=0.02, std_embedding=0.02, std_gain=0.1)

# 3 layers, width 96, 6 heads over 2 kv heads (group 3), head size 32 != width/heads,
# separate output head, odd vocabulary, theta 1e6, eps 1e-5, gains stored in 32-bit
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
    intermediate_size=160, vocab_size=389, rope_theta=1000000.0, rms_norm_eps=1e-5,
    max_position_embeddings=256, tie_word_embeddings=False, hidden_act="silu", attention_bias=False,
    use_sliding_window=False, sliding_window=None, eos_token_id=[11, 12])
TINY_B_INIT = dict(seed=2, std_matrix=0.03, std_embedding=0.05, std_gain=0.2, gain_dtype=torch.float32)

# 4 layers, width 80 (no power of two), 5 heads over 1 kv head (group 5), head size 48,
# layers 2 and 3 see a window of 24 keys
TINY_W = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=4, hidden_size=80, num_attention_heads=5, num_key_value_heads=1, head_dim=48,
    intermediate_size=112, vocab_size=301, rope_theta=50000.0, rms_norm_eps=1e-5,
    max_position_embeddings=512, tie_word_embeddings=True, hidden_act="silu", attention_bias=False,
    use_sliding_window=True, sliding_window=24, max_window_layers=2)
TINY_W_INIT = dict(seed=5, std_matrix=0.05, std_embedding=0.05, std_gain=0.1)

# sizes for which the fast bfloat16 kernels apply: head size 64 and 128, widths multiple of 8
TINY_F = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
    intermediate_size=384, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-6,
    max_position_embeddings=4096, tie_word_embeddings=True, hidden_act="silu", attention_bias=False,
    use_sliding_window=False, sliding_window=None)
TINY_F_INIT = dict(seed=9, std_matrix=0.04, std_embedding=0.04, std_gain=0.1)

# head size 64 with three kv heads, windows of 40 keys in the upper two layers, widths that are
# multiples of 32: the sizes the fused layer kernel takes, with options F does not have
TINY_S = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=192, num_attention_heads=6, num_key_value_heads=3, head_dim=64,
    intermediate_size=224, vocab_size=517, rope_theta=10000.0, rms_norm_eps=1e-5,
    max_position_embeddings=1024, tie_word_embeddings=False, hidden_act="silu", attention_bias=False,
    use_sliding_window=True, sliding_window=40, max_window_layers=1)
TINY_S_INIT = dict(seed=13, std_matrix=0.05, std_embedding=0.05, std_gain=0.1)

# head size 128 with windows of 70 keys in the upper layer, group 3, widths that are no powers of two: the tcgen05
# prompt attention's window path at engine level
TINY_G = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=160, num_attention_heads=6, num_key_value_heads=2, head_dim=128,
    intermediate_size=224, vocab_size=611, rope_theta=500000.0, rms_norm_eps=1e-6,
    max_position_embeddings=2048, tie_word_embeddings=True, hidden_act="silu", attention_bias=False,
    use_sliding_window=True, sliding_window=70, max_window_layers=1)
TINY_G_INIT = dict(seed=17, std_matrix=0.05, std_embedding=0.05, std_gain=0.1)

# widths that are no multiples of 8 (100, 90, vocabulary 257) and head size 80: in bfloat16 too, every product and the
# attention run on the plain kernels, which take every size
TINY_O = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=100, num_attention_heads=3, num_key_value_heads=3, head_dim=80,
    intermediate_size=90, vocab_size=257, rope_theta=20000.0, rms_norm_eps=3e-6,
    max_position_embeddings=512, tie_word_embeddings=False, hidden_act="silu", attention_bias=False,
    use_sliding_window=False, sliding_window=None)
TINY_O_INIT = dict(seed=21, std_matrix=0.05, std_embedding=0.05, std_gain=0.1)

CONFIGS = {"O": (TINY_O, TINY_O_INIT), "A": (TINY_A, TINY_A_INIT), "B": (TINY_B, TINY_B_INIT), "W": (TINY_W, TINY_W_INIT),
           "F": (TINY_F, TINY_F_INIT), "S": (TINY_S, TINY_S_INIT), "G": (TINY_G, TINY_G_INIT)}


def make_folder(name: str, out_dir: str) -> str:
    """Write config.json and model.safetensors of tiny configuration ``name`` into ``out_dir``."""
    from synaptix_b200.config import Qwen3Config
    from synaptix_b200.weights import write_model_folder
    cfg_dict, init = CONFIGS[name]
    cfg = Qwen3Config.from_dict(cfg_dict)
    init = dict(init)
    seed = init.pop("seed")
    write_model_folder(cfg, out_dir, seed, **init)
    # write the dict as given, so that keys the typed config does not echo are kept
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg_dict, f, indent=1)
    return out_dir


def random_tokens(vocab: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()

# the benchmark model's layer sizes (Qwen3-4B: width 2560, 32 heads over 8 kv heads of size 128,
# feed-forward 9728) with 2 layers and a shorter, odd vocabulary: the kernels run at the sizes and
# through the code paths of the real model, and the plain implementation still finishes in seconds
WIDE = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    intermediate_size=9728, vocab_size=32003, rope_theta=1000000.0, rms_norm_eps=1e-6,
    max_position_embeddings=40960, tie_word_embeddings=True, hidden_act="silu", attention_bias=False,
    use_sliding_window=False, sliding_window=None)
WIDE_INIT = dict(seed=11, std_matrix=0.02, std_embedding=0.02, std_gain=0.05)
CONFIGS["WIDE"] = (WIDE, WIDE_INIT)
