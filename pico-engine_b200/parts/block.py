"""A layer: the parts it has (a mixer, a feed-forward, a norm before each; any of them may be
absent) and the arrangement that runs them around the residual stream."""
from __future__ import annotations

from ..config.specs import ConfigError, LayerSpec
from .base import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, Norm, build_part, register_arrangement


class PassThrough(Norm):
    """Stands where a half of a block has no norm: the residual stream as it is, in the step's dtype."""

    def __init__(self, dtype, device):
        super().__init__(None, dtype, device)

    def forward(self, x, out_dtype, rows_index=None):
        rows = x if rows_index is None else x.index_select(0, rows_index.long())
        return rows.to(out_dtype)


class Layer:
    def __init__(self, spec: LayerSpec, dtype, device):
        self.spec = spec
        if spec.mixer is None and spec.feed_forward is None:
            raise ConfigError("a layer needs a mixer or a feed-forward")

        def build(table, kind, part_spec):
            return None if part_spec is None else build_part(table, kind, part_spec, dtype, device)
        self.mixer = build(MIXERS, "mixer", spec.mixer)
        self.feed_forward = build(FEED_FORWARDS, "feed-forward", spec.feed_forward)
        self.mixer_norm = build(NORMS, "norm", spec.mixer_norm) or PassThrough(dtype, device)
        self.feed_forward_norm = build(NORMS, "norm", spec.feed_forward_norm) or PassThrough(dtype, device)
        try:
            self._run = ARRANGEMENTS[spec.arrangement]
        except KeyError:
            raise ConfigError(f"unknown arrangement {spec.arrangement!r}; known: {', '.join(sorted(ARRANGEMENTS))}") from None

    def parts(self):
        """The parts that are there (a stand-in for an absent norm has no tensors and is left out)."""
        return tuple(p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm)
                     if p is not None and not isinstance(p, PassThrough))

    def run(self, x, ctx, entry: int, cache_entry: int, owns_cache: bool) -> None:
        self._run(self, x, ctx, entry, cache_entry, owns_cache)


@register_arrangement("pre_norm")
def pre_norm(layer: Layer, x, ctx, entry, cache_entry, owns_cache) -> None:
    """x += mixer(norm(x)); x += feed_forward(norm(x))  (pico-engine src/pico_engine/model.py:167-237)."""
    if layer.mixer is not None:
        if not layer.mixer.takes_pending:
            ctx.settle(x)
        layer.mixer.add_to(x, layer.mixer_norm, ctx, entry, cache_entry, owns_cache)
    if layer.feed_forward is not None:
        if not layer.feed_forward.takes_pending:
            ctx.settle(x)
        layer.feed_forward.add_to(x, layer.feed_forward_norm, ctx)
