"""Descriptions of the parts a model is put together from.

A model is described by data only: a :class:`ModelPlan` holds one :class:`LayerSpec` per
layer (each naming its mixer, feed-forward and norms with all their sizes and constants)
and a schedule, the list of layer executions in running order.  Nothing in here computes;
``parts`` turns specs into objects that do.

A new kind of part is a new frozen dataclass deriving from :class:`PartSpec`, registered
with its implementation in ``parts.registry``; nothing in this file has to change for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A configuration that cannot be built, with the offending key in the message."""


@dataclass(frozen=True)
class PartSpec:
    """Base of all part descriptions.  Concrete specs are frozen dataclasses."""


# ------------------------------------------------------------------ norms

@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    """y = x * rsqrt(mean(x^2) + eps) * weight  (pico-engine src/pico_engine/kernels.py:19-23)."""
    size: int
    eps: float
    weight: str                      # tensor name


# ------------------------------------------------------------------ position encodings

@dataclass(frozen=True)
class RotaryHalfSpec(PartSpec):
    """Rotate-half rotary encoding: element j pairs with j + head_dim/2, angle
    pos * theta^(-2j/head_dim)  (pico-engine src/pico_engine/model.py:75-79, kernels.py:42-47)."""
    head_dim: int
    theta: float


@dataclass(frozen=True)
class NoPositionSpec(PartSpec):
    """Queries and keys are used as projected."""


# ------------------------------------------------------------------ mixers

@dataclass(frozen=True)
class GQAAttentionSpec(PartSpec):
    """Softmax attention with grouped key/value heads over the key/value cache
    (pico-engine src/pico_engine/model.py:175-213).

    ``window`` None: every earlier key is visible; an integer w: query p sees key j iff
    0 <= p - j < w.  Tensor names are ``prefix + name + ".weight"/".bias"``.
    """
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    qkv_bias: bool
    window: Optional[int]
    scale: float
    position: PartSpec
    prefix: str
    q_name: str = "q_proj"
    k_name: str = "k_proj"
    v_name: str = "v_proj"
    o_name: str = "o_proj"


# ------------------------------------------------------------------ feed-forwards

@dataclass(frozen=True)
class SwiGLUSpec(PartSpec):
    """down(silu(gate(x)) * up(x)), no biases  (pico-engine src/pico_engine/model.py:222-235)."""
    hidden: int
    intermediate: int
    prefix: str
    gate_name: str = "gate_proj"
    up_name: str = "up_proj"
    down_name: str = "down_proj"


# ------------------------------------------------------------------ layers and the model

@dataclass(frozen=True)
class LayerSpec:
    """One block: which parts it has and how they are arranged around the residual stream.

    ``arrangement`` names an entry of ``parts.registry.ARRANGEMENTS``; "pre_norm" is
    x += mixer(norm(x)); x += ffn(norm(x))  (pico-engine src/pico_engine/model.py:167-237).
    Every part is optional: a block without a feed-forward is a mixer-only block (pico-engine's
    recurrent layers are such, src/pico_engine/model.py:389-406), one without a mixer a feed-forward-only
    block, and a half without a norm takes the residual stream as it is.
    """
    mixer: Optional[PartSpec]
    mixer_norm: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  Each entry owns a cache of its own unless ``cache_of``
    names an earlier entry of the schedule, whose cache it then reads without writing."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: str                                   # tensor name of the [vocab, hidden] table
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: Optional[str]                              # tensor name of [vocab, hidden]; None: tied to the embedding
    max_positions: int
    stop_token_ids: Tuple[int, ...] = ()
    ignorable_tensors: Tuple[str, ...] = field(default_factory=tuple)   # names a checkpoint may carry unused

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for e, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"schedule[{e}] names layer {entry.layer}, but there are {len(self.layers)} layers")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < e:
                    raise ConfigError(f"schedule[{e}].cache_of={entry.cache_of} must name an earlier entry")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule[{e}].cache_of={entry.cache_of} names an entry that owns no cache")
