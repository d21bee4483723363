"""The generation loop's decisions, driven with a scripted backend (CPU)."""
import pytest

from pico_engine.engine.generate import GenerationError, Request, generate, held_tokens, plan_batches


class Scripted:
    """Chooses, for request r at its step s, the token script[r][s]; records everything."""

    def __init__(self, script, slots=8):
        self.script, self.free, self.open_slots = script, list(range(slots)), {}
        self.calls, self.slot_log = [], []

    def open(self):
        s = self.free.pop(0)
        self.open_slots[s] = 0
        self.slot_log.append(("open", s))
        return s

    def close(self, slot):
        assert slot in self.open_slots, "closed twice"
        del self.open_slots[slot]
        self.free.append(slot); self.free.sort()
        self.slot_log.append(("close", slot))

    def prefill(self, slots, prompts, requests):
        self.calls.append(("prefill", list(requests), [len(p) for p in prompts]))
        for s, p in zip(slots, prompts):
            self.open_slots[s] += len(p)
        return [self.script[r][0] for r in requests]

    def decode(self, slots, tokens, requests, steps):
        self.calls.append(("decode", list(requests), list(tokens), list(steps)))
        for s in slots:
            self.open_slots[s] += 1
        return [self.script[r][st] for r, st in zip(requests, steps)]


def test_unequal_prompts_stop_tokens_and_early_ends():
    script = {0: [5, 6, 99, 7], 1: [99], 2: [1, 2, 3, 4, 5, 6]}
    be = Scripted(script)
    reqs = generate(be, [[1, 2, 3], [4], [5, 6, 7, 8, 9]], 4, stop_token_ids=[99], max_batch=8, max_tokens=4096)
    assert [r.output for r in reqs] == [[5, 6], [], [1, 2, 3, 4]]          # the stop token is not returned
    assert [r.finish_reason for r in reqs] == ["stop", "stop", "length"]
    assert be.calls[0] == ("prefill", [0, 1, 2], [3, 1, 5])
    assert be.calls[1] == ("decode", [0, 2], [5, 1], [1, 1])                # request 1 ended at once
    assert be.calls[2] == ("decode", [0, 2], [6, 2], [2, 2])
    assert be.calls[3] == ("decode", [2], [3], [3])                         # the stop token was not fed back
    assert len(be.calls) == 4                                               # and no step follows the last token
    assert not be.open_slots and be.free == list(range(8))


def test_batches_follow_one_another_and_use_slots_again():
    be = Scripted({i: [i + 10] * 3 for i in range(5)}, slots=2)
    reqs = generate(be, [[1]] * 5, 2, stop_token_ids=[], max_batch=2, max_tokens=4096)
    assert [r.output for r in reqs] == [[i + 10] * 2 for i in range(5)]
    assert [c[1] for c in be.calls if c[0] == "prefill"] == [[0, 1], [2, 3], [4]]
    opened = [s for what, s in be.slot_log if what == "open"]
    assert opened == [0, 1, 0, 1, 0]


def test_token_budget_cuts_batches():
    reqs = [Request(i, [0] * n, m) for i, (n, m) in enumerate([(60, 5), (10, 1), (100, 30), (1, 1)])]
    assert [held_tokens(r) for r in reqs] == [64, 64, 192, 64]
    assert [[r.index for r in b] for b in plan_batches(reqs, 8, 256)] == [[0, 1], [2, 3]]
    assert [[r.index for r in b] for b in plan_batches(reqs, 1, 4096)] == [[0], [1], [2], [3]]
    with pytest.raises(GenerationError, match="request 2"):
        plan_batches(reqs, 8, 128)


def test_empty_prompts_zero_budgets_and_bad_arguments():
    be = Scripted({1: [3, 3, 3]})
    reqs = generate(be, [[], [1, 2], [7]], [5, 2, 0], stop_token_ids=[], max_batch=4, max_tokens=1024)
    assert [r.output for r in reqs] == [[], [3, 3], []]
    assert [r.finish_reason for r in reqs] == ["empty", "length", "length"]
    assert be.calls[0] == ("prefill", [1], [2])                              # the others never reach the device
    with pytest.raises(GenerationError):
        generate(be, [[1]], [1, 2], [], 4, 1024)
    with pytest.raises(GenerationError):
        generate(be, [[1]], -1, [], 4, 1024)


def test_slots_are_given_back_after_a_failure():
    class Failing(Scripted):
        def decode(self, *a):
            raise RuntimeError("device lost")
    be = Failing({0: [1, 1], 1: [2, 2]})
    with pytest.raises(RuntimeError, match="device lost"):
        generate(be, [[1], [2]], 3, [], 4, 1024)
    assert not be.open_slots


# ---------------------------------------------------------------------------- one step ahead

class ScriptedAhead(Scripted):
    """The same scripted choices through decode_begin / decode_end.  A row may take its token from the
    step begun just before (``sources``); the backend checks that such a step exists and is still
    unread, resolves the token itself, and records what ran."""

    pipelined = True

    def __init__(self, script, slots=8):
        super().__init__(script, slots)
        self.begun = []            # steps begun and not yet read: (requests, chosen)
        self.last_begun = None
        self.most_in_flight = 0

    def decode_begin(self, slots, tokens, sources, requests, steps):
        resolved = []
        for tok, src in zip(tokens, sources):
            if src >= 0:
                assert self.last_begun is not None, "a source without a step before"
                resolved.append(self.last_begun[1][src])
            else:
                resolved.append(tok)
        for s in slots:
            assert s in self.open_slots, "a step on a slot that was given back"
            self.open_slots[s] += 1
        chosen = [self.script[r][st] for r, st in zip(requests, steps)]
        self.calls.append(("decode", list(requests), resolved, list(steps)))
        handle = (list(requests), chosen, list(slots))
        self.begun.append(handle)
        self.last_begun = handle
        self.most_in_flight = max(self.most_in_flight, len(self.begun))
        return handle

    def decode_end(self, handle):
        assert self.begun and self.begun[0] is handle, "steps are read in the order they were begun"
        self.begun.pop(0)
        return handle[1]

    def close(self, slot):
        assert all(slot not in h[2] for h in self.begun), "a slot given back while a step on it is in flight"
        super().close(slot)


def test_one_step_ahead_gives_the_same_tokens_and_feeds_no_stop_token_to_a_live_request():
    script = {0: [5, 6, 99, 7, 8], 1: [99], 2: [1, 2, 3, 4, 5, 6], 3: [9, 9, 9, 99, 1]}
    prompts, budget = [[1, 2, 3], [4], [5, 6, 7, 8, 9], [1]], [4, 4, 4, 6]
    plain = generate(Scripted(script), prompts, budget, stop_token_ids=[99], max_batch=8, max_tokens=4096)
    be = ScriptedAhead(script)
    ahead = generate(be, prompts, budget, stop_token_ids=[99], max_batch=8, max_tokens=4096)
    assert [r.output for r in ahead] == [r.output for r in plain] == [[5, 6], [], [1, 2, 3, 4], [9, 9, 9]]
    assert [r.finish_reason for r in ahead] == [r.finish_reason for r in plain]
    assert be.most_in_flight == 2                                           # the loop does run ahead
    assert not be.open_slots and be.free == list(range(8)) and not be.begun
    # every step that counts fed each request the token it chose before; rows that ran for a request
    # that had already stopped are the only extra ones
    fed = {}
    for _, requests, tokens, steps in (c for c in be.calls if c[0] == "decode"):
        for r, t, s in zip(requests, tokens, steps):
            fed[(r, s)] = t
    for r in ahead:
        for s in range(1, len(r.output)):
            assert fed[(r.index, s)] == r.output[s - 1]
    extra = [k for k in fed if k[1] > len(ahead[k[0]].output)]
    assert all(ahead[r].finish_reason == "stop" and s == len(ahead[r].output) + 1 for r, s in extra)
    # no step is begun for a request that reaches its length with the token in flight
    assert (2, 4) not in fed and (2, 3) in fed


def test_one_step_ahead_batches_and_failures():
    be = ScriptedAhead({i: [i + 10] * 4 for i in range(5)}, slots=2)
    reqs = generate(be, [[1]] * 5, 3, stop_token_ids=[], max_batch=2, max_tokens=4096)
    assert [r.output for r in reqs] == [[i + 10] * 3 for i in range(5)]
    assert [s for what, s in be.slot_log if what == "open"] == [0, 1, 0, 1, 0]
    assert not be.begun and not be.open_slots

    class Failing(ScriptedAhead):
        def decode_end(self, handle):
            out = super().decode_end(handle)
            if len([c for c in self.calls if c[0] == "decode"]) >= 2:
                raise RuntimeError("device lost")
            return out

    be = Failing({0: [1] * 9, 1: [2] * 9})
    with pytest.raises(RuntimeError, match="device lost"):
        generate(be, [[1], [2]], 8, stop_token_ids=[], max_batch=2, max_tokens=4096)
    assert not be.open_slots and not be.begun                               # nothing stays held or in flight


def test_prompts_are_cut_into_steps_of_a_token_budget():
    from pico_engine.engine.generate import GenerationError, cut_prompts
    assert cut_prompts([5, 9, 13], 100) == [[(0, 0, 5), (1, 0, 9), (2, 0, 13)]]
    steps = cut_prompts([5, 9, 13], 8)
    assert steps == [[(0, 0, 5), (1, 0, 3)], [(1, 3, 6), (2, 0, 2)], [(2, 2, 8)], [(2, 10, 3)]]
    for lengths, budget in (([70, 1, 64, 200], 64), ([3], 1), ([128, 128], 128), ([1, 1, 1], 2)):
        steps = cut_prompts(lengths, budget)
        assert all(0 < sum(n for _, _, n in st) <= budget for st in steps)
        assert all(sum(n for _, _, n in st) == budget for st in steps[:-1])          # every step but the last is full
        seen = {}
        for k, st in enumerate(steps):
            assert len({r for r, _, _ in st}) == len(st)                                # a row comes once in a step
            for r, at, n in st:
                assert at == seen.get(r, (0, k))[0] and k - seen.get(r, (0, k))[1] <= 1 # pieces follow on, in consecutive steps
                seen[r] = (at + n, k)
        assert [seen[r][0] for r in range(len(lengths))] == lengths
    with pytest.raises(GenerationError):
        cut_prompts([3], 0)
