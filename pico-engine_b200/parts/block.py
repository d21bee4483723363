"""A layer: its four parts and the arrangement that runs them around the residual stream."""
from __future__ import annotations

from ..config.specs import ConfigError, LayerSpec
from .base import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, build_part, register_arrangement


class Layer:
    def __init__(self, spec: LayerSpec, dtype, device):
        self.spec = spec
        self.mixer = build_part(MIXERS, "mixer", spec.mixer, dtype, device)
        self.mixer_norm = build_part(NORMS, "norm", spec.mixer_norm, dtype, device)
        self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", spec.feed_forward, dtype, device)
        self.feed_forward_norm = build_part(NORMS, "norm", spec.feed_forward_norm, dtype, device)
        try:
            self._run = ARRANGEMENTS[spec.arrangement]
        except KeyError:
            raise ConfigError(f"unknown arrangement {spec.arrangement!r}; known: {', '.join(sorted(ARRANGEMENTS))}") from None

    def parts(self):
        return (self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm)

    def run(self, x, ctx, entry: int, cache_entry: int, owns_cache: bool) -> None:
        self._run(self, x, ctx, entry, cache_entry, owns_cache)


@register_arrangement("pre_norm")
def pre_norm(layer: Layer, x, ctx, entry, cache_entry, owns_cache) -> None:
    """x += mixer(norm(x)); x += feed_forward(norm(x))  (pico-engine src/pico_engine/model.py:167-237)."""
    if not layer.mixer.takes_pending:
        ctx.settle(x)
    layer.mixer.add_to(x, layer.mixer_norm, ctx, entry, cache_entry, owns_cache)
    if not layer.feed_forward.takes_pending:
        ctx.settle(x)
    layer.feed_forward.add_to(x, layer.feed_forward_norm, ctx)
