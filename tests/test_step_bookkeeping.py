"""Host-side bookkeeping of a step (CPU): the residual sum that a part may leave pending for the next norm
(who settles it, and when), and how a step's tokens are cut into runs for the prefill attention kernels.

The kernels are replaced by torch arithmetic; what is tested is the bookkeeping of
``StepContext.defer_add / settle / normed``, of the ``pre_norm`` arrangement and of ``prefill_tiles``.
"""
import pytest
import torch

import pico_engine.ops.kernels as kernels
from pico_engine.parts import base
from pico_engine.parts.block import pre_norm


def context():
    z = torch.zeros(0, dtype=torch.int32)
    return base.StepContext(T=3, B=1, dtype=torch.float32, device=torch.device("cpu"), tok_pos=z, tok_row=z, slots=z, row_first=z, row_lens=z,
                            slot_ids=[0], lens=[3], starts=[0], one_token_each=False, cache=None)


class CountingNorm(base.Norm):
    """Doubles its input; counts which of its two entry points ran."""

    def __init__(self):
        self.plain = self.fused = 0

    def forward(self, x, out_dtype, rows_index=None):
        self.plain += 1
        return 2 * x

    def add_forward(self, x, y, out_dtype):
        self.fused += 1
        x += y
        return 2 * x


class Knowing(base.FeedForward):
    """A part that copes with a pending sum and leaves its own pending."""
    takes_pending = True

    def __init__(self):
        pass

    def add_to(self, x, norm, ctx):
        h = ctx.normed(x, norm)
        ctx.defer_add(x, h + 1)


class Plain(base.Mixer):
    """A part that knows nothing of pending sums: it reads x directly."""

    def __init__(self):
        self.saw = None

    def add_to(self, x, norm, ctx, entry, cache_entry, owns_cache):
        self.saw = x.clone()
        x += 10


class Layer:
    def __init__(self, mixer, feed_forward):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = CountingNorm(), CountingNorm()


def test_pending_sum_is_added_by_the_next_norm_or_settled_before_a_part_that_reads_x(monkeypatch):
    adds = []

    def residual_add(x, y):
        adds.append(1)
        x += y
        return x

    monkeypatch.setattr(kernels, "residual_add", residual_add)
    ctx, x = context(), torch.ones(3, 4)

    # a knowing part: norm(1) = 2, pending 3
    ff = Knowing()
    norm = CountingNorm()
    ff.add_to(x, norm, ctx)
    assert ctx.pending is not None and torch.equal(x, torch.ones(3, 4)) and (norm.plain, norm.fused) == (1, 0)
    # the next knowing part's norm adds it in the same pass: x = 4, norm = 8, pending 9
    ff.add_to(x, norm, ctx)
    assert torch.equal(x, torch.full((3, 4), 4.0)) and (norm.plain, norm.fused) == (1, 1) and not adds
    assert torch.equal(ctx.pending, torch.full((3, 4), 9.0))

    # a layer whose mixer reads x itself: the arrangement settles first (x = 13), the mixer sees the settled stream
    layer = Layer(Plain(), Knowing())
    pre_norm(layer, x, ctx, 0, 0, True)
    assert len(adds) == 1 and torch.equal(layer.mixer.saw, torch.full((3, 4), 13.0))
    # mixer: x = 23; feed-forward: norm 46, pending 47
    assert torch.equal(x, torch.full((3, 4), 23.0)) and torch.equal(ctx.pending, torch.full((3, 4), 47.0))
    assert (layer.feed_forward_norm.plain, layer.feed_forward_norm.fused) == (1, 0)

    # the end of the layers: what is pending is added, once
    ctx.settle(x)
    ctx.settle(x)
    assert len(adds) == 2 and ctx.pending is None and torch.equal(x, torch.full((3, 4), 70.0))


def test_a_second_deferred_sum_settles_the_first(monkeypatch):
    monkeypatch.setattr(kernels, "residual_add", lambda x, y: x.add_(y))
    ctx, x = context(), torch.zeros(2, 2)
    ctx.defer_add(x, torch.ones(2, 2))
    ctx.defer_add(x, torch.full((2, 2), 5.0))
    assert torch.equal(x, torch.ones(2, 2)) and torch.equal(ctx.pending, torch.full((2, 2), 5.0))


def test_the_default_norm_adds_then_norms(monkeypatch):
    monkeypatch.setattr(kernels, "residual_add", lambda x, y: x.add_(y))

    class OnlyForward(base.Norm):
        def __init__(self):
            pass

        def forward(self, x, out_dtype, rows_index=None):
            return x * 3

    x = torch.ones(2, 2)
    h = OnlyForward().add_forward(x, torch.ones(2, 2), torch.float32)
    assert torch.equal(x, torch.full((2, 2), 2.0)) and torch.equal(h, torch.full((2, 2), 6.0))


def test_prefill_tiles_cut_runs_per_sequence_and_put_the_longest_first():
    """The host side of the prefill attention kernels: runs of at most `tile` tokens of one sequence,
    every packed token in exactly one run, the runs that see the most keys first."""
    lens, starts = [130, 1, 64, 300], [0, 500, 37, 10]
    for tile in (kernels.PREFILL_TILE, kernels.PREFILL_TILE_TCGEN05):
        rows = kernels.prefill_tiles(lens, starts, "cpu", tile).tolist()
        seen = []
        first = [sum(lens[:b]) for b in range(len(lens))]
        for b, tok0, n, pos0 in rows:
            assert 1 <= n <= tile and pos0 - starts[b] == tok0 - first[b] and 0 <= tok0 - first[b] < lens[b]
            assert (tok0 - first[b]) % tile == 0 and tok0 - first[b] + n <= lens[b]
            seen.extend(range(tok0, tok0 + n))
        assert sorted(seen) == list(range(sum(lens)))
        ends = [pos0 + n for _, _, n, pos0 in rows]
        assert ends == sorted(ends, reverse=True)


# ---------------------------------------------------------------------------- the description of a padded step

def _stepper(max_tokens=1024, max_seqs=8, window=32):
    import types
    from pico_engine.cache import Cache, CacheNeeds, KVNeed
    from pico_engine.engine.step import Stepper
    needs = [CacheNeeds(kv=KVNeed(2, 16, None)), CacheNeeds(kv=KVNeed(2, 16, window))]
    cache = Cache(needs, max_tokens, max_seqs, torch.float32, "cpu", allocate=False)
    model = types.SimpleNamespace(plan=types.SimpleNamespace(vocab_size=100), dtype=torch.float32)
    return Stepper(model, cache, 512), cache


def test_prompt_graph_sizes_and_padding():
    from pico_engine.engine.graph import GraphedPrompt, prompt_sizes
    assert prompt_sizes(1, 2048) == (3, 2048) and prompt_sizes(1, 5) == (3, 128) and prompt_sizes(5, 129) == (10, 256)
    for rows, tokens in [(1, 2048), (1, 5), (3, 27), (8, 8000), (64, 100), (5, 125), (2, 1)]:
        B, T = prompt_sizes(rows, tokens)
        pad = GraphedPrompt.padding(rows, tokens, B, T)
        assert len(pad) == B - rows and sum(pad) == T - tokens and all(0 <= n <= 64 for n in pad)
        assert pad == sorted(pad, reverse=True)                    # rows without a token come last
    with pytest.raises(ValueError):
        GraphedPrompt.padding(1, 10, 2, 256)


def test_a_padded_step_is_described_with_idle_rows_and_a_fixed_number_of_runs():
    """What a captured prompt step uploads: the live rows as they are, idle rows at the first positions of the idle
    page (an idle row may bring no token at all), a logits row for every row, and the list of attention runs filled up
    to a fixed length with the cheapest run there is, listed again."""
    from pico_engine.engine.step import StepError
    st, cache = _stepper()
    a, b = cache.open(), cache.open()
    cache.reserve(a, 70); cache.advance(a, 70)                      # a continues at position 70, b starts
    idle = cache.idle_slot
    lay, host, starts = st.describe([a, b, idle, idle, idle], [130, 5, 64, 57, 0], None,
                                    [[1] * 130, [2] * 5, [0] * 64, [0] * 57, []], widths=[8, 8], n_tiles=(9, 7))
    assert (lay.T, lay.B, lay.W) == (256, 5, 5) and starts == [70, 0, 0, 0, 0]
    assert host[lay.pos: lay.pos + 256].tolist() == list(range(70, 200)) + list(range(5)) + list(range(64)) + list(range(57))
    assert host[lay.row: lay.row + 256].tolist() == [0] * 130 + [1] * 5 + [2] * 64 + [3] * 57
    assert host[lay.first: lay.first + 6].tolist() == [0, 130, 135, 199, 256, 256]
    assert host[lay.lens: lay.lens + 5].tolist() == [130, 5, 64, 57, 0]
    assert host[lay.want: lay.want + 5].tolist() == [129, 134, 198, 255, 0]       # the empty row's logits are token 0's
    t64 = host[lay.tiles[0]: lay.tiles[0] + 4 * 9].reshape(9, 4).tolist()
    t128 = host[lay.tiles[1]: lay.tiles[1] + 4 * 7].reshape(7, 4).tolist()
    assert t64[:3] == [[0, 128, 2, 198], [0, 64, 64, 134], [0, 0, 64, 70]]       # the runs that see the most keys first
    assert sorted(t64[3:6]) == sorted([[1, 130, 5, 0], [2, 135, 64, 0], [3, 199, 57, 0]])
    assert t64[6:] == [[1, 130, 1, 0]] * 3                                      # filled up with the first token of row b
    assert t128[:2] == [[0, 128, 2, 198], [0, 0, 128, 70]] and t128[5:] == [[1, 130, 1, 0]] * 2
    tables = host[lay.tables[0]: lay.tables[0] + 5 * 8].reshape(5, 8)
    assert tables[2, 0] == cache.idle_page and tables[4, 0] == cache.idle_page and (tables[2:, 1:] == -1).all()
    assert cache.length(a) == 70 and len(cache.groups[0].table[a]) == 4         # pages reserved, nothing advanced yet
    with pytest.raises(StepError, match="idle"):
        st.describe([idle], [65], None, None)
    with pytest.raises(StepError, match="attention runs"):
        st.describe([b], [200], None, None, n_tiles=(2, 1))
    with pytest.raises(StepError, match="brings no token"):
        st.describe([b], [0], None, None)
