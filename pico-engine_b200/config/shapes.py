"""config.json contents of the shapes the benchmarks and tests name: the two tiny test
configurations and the Qwen2.5 sizes (weights for them are drawn at random)."""
from __future__ import annotations

_QWEN2 = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", "torch_dtype": "bfloat16"}

SHAPES = {
    "tiny-a": {**_QWEN2, "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
               "head_dim": 16, "intermediate_size": 160, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
               "max_position_embeddings": 128, "tie_word_embeddings": True, "use_sliding_window": False},
    "tiny-b": {**_QWEN2, "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
               "head_dim": 32, "intermediate_size": 352, "vocab_size": 512, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
               "max_position_embeddings": 256, "tie_word_embeddings": False, "use_sliding_window": True,
               "sliding_window": 32, "max_window_layers": 1},
    "qwen2.5-0.5b": {**_QWEN2, "num_hidden_layers": 24, "hidden_size": 896, "num_attention_heads": 14,
                     "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 4864, "vocab_size": 151936,
                     "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 32768,
                     "tie_word_embeddings": True, "use_sliding_window": False},
    "qwen2.5-7b": {**_QWEN2, "num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28,
                   "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944, "vocab_size": 152064,
                   "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 32768,
                   "tie_word_embeddings": False, "use_sliding_window": False},
    "qwen2.5-14b": {**_QWEN2, "num_hidden_layers": 48, "hidden_size": 5120, "num_attention_heads": 40,
                    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 13824, "vocab_size": 152064,
                    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 32768,
                    "tie_word_embeddings": False, "use_sliding_window": False},
}


def shape(name: str) -> dict:
    try:
        return dict(SHAPES[name.lower()])
    except KeyError:
        raise KeyError(f"unknown shape {name!r}; known: {', '.join(sorted(SHAPES))}") from None
