"""Two tiny Qwen3 configurations that differ in every size and option, and helpers that
write them to temporary model folders with random weights."""

from __future__ import annotations

from pathlib import Path

import torch

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "hidden_act": "silu",
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 4096,
    "tie_word_embeddings": True,
}
TINY_A_PAGE = 16

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 384, "hidden_size": 80, "intermediate_size": 176, "num_hidden_layers": 3,
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 32, "hidden_act": "silu",
    "rms_norm_eps": 1e-5, "rope_theta": 1000000.0, "max_position_embeddings": 2048,
    "tie_word_embeddings": False,
}
TINY_B_PAGE = 8

# A third one for the kernels' odd corners: MHA, head_dim 48, an odd vocabulary and width.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 301, "hidden_size": 72, "intermediate_size": 100, "num_hidden_layers": 2,
    "num_attention_heads": 3, "num_key_value_heads": 3, "head_dim": 48, "hidden_act": "silu",
    "rms_norm_eps": 1e-6, "rope_theta": 50000.0, "max_position_embeddings": 1024,
    "tie_word_embeddings": False,
}
TINY_C_PAGE = 32

# Real layer widths with few layers: the sizes at which the tensor-core kernels take over. At the
# Qwen3-8B widths another set of kernels runs than at the 0.6B ones (library products for decode
# rows, tcgen05 for the narrow outputs, separate norms, four query heads per kv head).
REAL_0_6B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936, "hidden_size": 1024,
    "intermediate_size": 3072, "num_hidden_layers": 2, "num_attention_heads": 16, "num_key_value_heads": 8,
    "head_dim": 128, "hidden_act": "silu", "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "max_position_embeddings": 4096, "tie_word_embeddings": True,
}
REAL_8B = {**REAL_0_6B, "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 1,
           "num_attention_heads": 32, "num_key_value_heads": 8, "tie_word_embeddings": False}

TINIES = {"A": (TINY_A, TINY_A_PAGE, 0), "B": (TINY_B, TINY_B_PAGE, 1), "C": (TINY_C, TINY_C_PAGE, 2)}


def write_tiny(folder: Path, which: str, dtype: torch.dtype = torch.float32, std_scale: float = 8.0) -> Path:
    """Write tiny model ``which`` ("A", "B" or "C") with the framework's random-weights mode.
    The spread is 8x the serving default so that logits differ visibly between tokens."""
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model
    import tinyserve_b200.architectures  # noqa: F401

    d, _, seed = TINIES[which]
    return write_random_model(folder, config_from_dict(d), seed, dtype, std_scale=std_scale)


def random_prompt(length: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()
