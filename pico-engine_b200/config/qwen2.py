"""Typed configuration of the dense Qwen2 decoder, read from its own config.json keys.

pico-engine reads the same quantities from GGUF metadata without defaults
(src/pico_engine/engine.py:26-47: block_count, embedding_length, attention.head_count,
attention.head_count_kv, attention.layer_norm_rms_epsilon, rope.freq_base,
feed_forward_length, context_length); a missing size is an error here too.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional, Tuple

from .registry import register_architecture
from .specs import (ConfigError, GQAAttentionSpec, LayerSpec, ModelPlan, RMSNormSpec, RotaryHalfSpec,
                    ScheduleEntry, SwiGLUSpec)

_REQUIRED = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
             "intermediate_size", "rope_theta", "rms_norm_eps", "max_position_embeddings")


def _as_int(d: dict, key: str) -> int:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"{key} must be an integer, found {v!r}")
    if v <= 0:
        raise ConfigError(f"{key} must be positive, found {v}")
    return v


def _as_float(d: dict, key: str) -> float:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{key} must be a number, found {v!r}")
    if not v > 0:
        raise ConfigError(f"{key} must be positive, found {v}")
    return float(v)


def _token_ids(v, key: str) -> Tuple[int, ...]:
    if v is None:
        return ()
    if isinstance(v, int) and not isinstance(v, bool):
        return (v,)
    if isinstance(v, (list, tuple)) and all(isinstance(t, int) and not isinstance(t, bool) for t in v):
        return tuple(v)
    raise ConfigError(f"{key} must be an integer or a list of integers, found {v!r}")


@dataclass(frozen=True)
class Qwen2Config:
    ARCHITECTURE = "Qwen2ForCausalLM"

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float
    rms_norm_eps: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Tuple[int, ...] = ()

    # ---------------------------------------------------------------- reading and writing

    @classmethod
    def from_dict(cls, d: dict) -> "Qwen2Config":
        missing = [k for k in _REQUIRED if k not in d or d[k] is None]
        if missing:
            raise ConfigError("config.json lacks " + ", ".join(missing))
        hidden = _as_int(d, "hidden_size")
        heads = _as_int(d, "num_attention_heads")
        if d.get("head_dim") is not None:
            head_dim = _as_int(d, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError(f"head_dim is not given and hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads}")
            head_dim = hidden // heads
        scaling = d.get("rope_scaling")
        if scaling not in (None, {}) and not (isinstance(scaling, dict) and
                                              scaling.get("rope_type", scaling.get("type")) == "default"):
            raise ConfigError(f"rope_scaling {scaling!r} is not supported: positions are rotated unscaled")
        use_window = bool(d.get("use_sliding_window", False))
        window = d.get("sliding_window")
        if use_window:
            if window is None:
                raise ConfigError("use_sliding_window is true but sliding_window is not given")
            window = _as_int(d, "sliding_window")
        elif window is not None:
            window = _as_int(d, "sliding_window")
        mwl = d.get("max_window_layers")
        if mwl is not None and (isinstance(mwl, bool) or not isinstance(mwl, int) or mwl < 0):
            raise ConfigError(f"max_window_layers must be a non-negative integer, found {mwl!r}")
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        cfg = cls(
            vocab_size=_as_int(d, "vocab_size"), hidden_size=hidden,
            num_hidden_layers=_as_int(d, "num_hidden_layers"), num_attention_heads=heads,
            num_key_value_heads=_as_int(d, "num_key_value_heads"), head_dim=head_dim,
            intermediate_size=_as_int(d, "intermediate_size"), rope_theta=_as_float(d, "rope_theta"),
            rms_norm_eps=_as_float(d, "rms_norm_eps"),
            max_position_embeddings=_as_int(d, "max_position_embeddings"),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            use_sliding_window=use_window, sliding_window=window, max_window_layers=mwl,
            hidden_act=str(d.get("hidden_act", "silu")), torch_dtype=str(dtype),
            bos_token_id=d.get("bos_token_id"), eos_token_id=_token_ids(d.get("eos_token_id"), "eos_token_id"))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.ARCHITECTURE]
        d["model_type"] = "qwen2"
        eos = d.pop("eos_token_id")
        d["eos_token_id"] = None if not eos else (eos[0] if len(eos) == 1 else list(eos))
        return {k: v for k, v in d.items() if v is not None}

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotate-half position encoding")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (silu only)")
        if self.use_sliding_window and not self.sliding_window:
            raise ConfigError("use_sliding_window needs a positive sliding_window")

    # ---------------------------------------------------------------- the plan

    def window_of(self, layer: int) -> Optional[int]:
        """Layers with index >= max_window_layers see a window when use_sliding_window is set."""
        if not self.use_sliding_window:
            return None
        first = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
        return self.sliding_window if layer >= first else None

    def plan(self) -> ModelPlan:
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            layers.append(LayerSpec(
                mixer=GQAAttentionSpec(
                    hidden=self.hidden_size, n_heads=self.num_attention_heads,
                    n_kv_heads=self.num_key_value_heads, head_dim=self.head_dim, qkv_bias=True,
                    window=self.window_of(i), scale=self.head_dim ** -0.5,
                    position=RotaryHalfSpec(head_dim=self.head_dim, theta=self.rope_theta),
                    prefix=p + "self_attn."),
                mixer_norm=RMSNormSpec(self.hidden_size, self.rms_norm_eps, p + "input_layernorm.weight"),
                feed_forward=SwiGLUSpec(hidden=self.hidden_size, intermediate=self.intermediate_size,
                                        prefix=p + "mlp."),
                feed_forward_norm=RMSNormSpec(self.hidden_size, self.rms_norm_eps,
                                              p + "post_attention_layernorm.weight"),
                arrangement="pre_norm"))
        plan = ModelPlan(
            architecture=self.ARCHITECTURE, vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            embedding="model.embed_tokens.weight", layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=RMSNormSpec(self.hidden_size, self.rms_norm_eps, "model.norm.weight"),
            head=None if self.tie_word_embeddings else "lm_head.weight",
            max_positions=self.max_position_embeddings, stop_token_ids=self.eos_token_id,
            ignorable_tensors=("lm_head.weight",) if self.tie_word_embeddings else ())
        plan.validate()
        return plan


register_architecture(Qwen2Config.ARCHITECTURE, Qwen2Config)
