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
