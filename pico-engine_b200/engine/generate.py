"""The generation loop: batches of unequal prompts, stop tokens, sequences that end before
their neighbours, and as many batches one after another as there are requests.

The loop decides; a *backend* computes.  The backend opens and closes sequences, runs the
prompts of a batch as one step and then one token per live sequence, and returns the chosen
next token of every row as host integers.  (Tests drive the loop with a scripted backend.)

pico-engine's loop handles one sequence (src/pico_engine/engine.py:308-337): sample, stop
*before* appending the stop token (engine.py:331-332), append, decode.  Its last iteration
runs a decode step whose logits nobody reads (engine.py:335); this loop does not.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, List, Protocol, Sequence

PAGE = 64


@dataclass
class Request:
    index: int                      # position among the requests of one call; names the sampling stream
    prompt: List[int]
    max_new_tokens: int
    output: List[int] = field(default_factory=list)
    finish_reason: str = ""         # "stop", "length" or "empty"


class Backend(Protocol):
    def open(self) -> int: ...
    def close(self, slot: int) -> None: ...
    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]], requests: Sequence[int]) -> List[int]: ...
    def decode(self, slots: Sequence[int], tokens: Sequence[int], requests: Sequence[int],
               steps: Sequence[int]) -> List[int]: ...
    # A backend may also be ``pipelined`` (an attribute that is true) and then has
    #   decode_begin(slots, tokens, sources, requests, steps) -> handle
    #   decode_end(handle) -> List[int]
    # where sources[j] >= 0 names the row of the step begun just before whose chosen token is
    # row j's input (tokens[j] is then ignored), and optionally decode_idle().


class GenerationError(ValueError):
    pass


def held_tokens(r: Request) -> int:
    """What a request can hold in the cache at most, in whole pages."""
    n = len(r.prompt) + max(r.max_new_tokens - 1, 0)       # the last chosen token is never fed back
    return (n + PAGE - 1) // PAGE * PAGE


def plan_batches(requests: Sequence[Request], max_batch: int, max_tokens: int) -> List[List[Request]]:
    """Requests in their order, cut into batches of at most ``max_batch`` sequences whose
    largest possible cache holdings fit ``max_tokens`` together."""
    if max_batch < 1:
        raise GenerationError("max_batch must be at least 1")
    batches: List[List[Request]] = []
    cur: List[Request] = []
    held = 0
    for r in requests:
        need = held_tokens(r)
        if need > max_tokens:
            raise GenerationError(f"request {r.index} can hold {need} tokens, the cache has room for {max_tokens}")
        if cur and (len(cur) == max_batch or held + need > max_tokens):
            batches.append(cur)
            cur, held = [], 0
        cur.append(r)
        held += need
    if cur:
        batches.append(cur)
    return batches


def cut_prompts(lengths: Sequence[int], tokens_per_step: int) -> List[List[tuple]]:
    """The prompts of a batch cut into steps of at most ``tokens_per_step`` tokens: ``[[(row, first token, tokens), ...],
    ...]``.  Rows are taken in order; a prompt that does not fit what is left of a step goes on in the next one, so
    every row's pieces come in consecutive steps and its last piece ends in the step whose logits choose its first
    token.  A batch that fits one step is one step."""
    if tokens_per_step < 1:
        raise GenerationError("a step must take at least one token")
    steps, cur, room = [], [], tokens_per_step
    for row, n in enumerate(lengths):
        at = 0
        while at < n:
            if room == 0:
                steps.append(cur)
                cur, room = [], tokens_per_step
            take = min(n - at, room)
            cur.append((row, at, take))
            at += take
            room -= take
    if cur:
        steps.append(cur)
    return steps


def _settle(rows: Sequence[Request], chosen: Sequence[int], stop: frozenset) -> None:
    """Give every row of a step its chosen token: a stop token ends the request (and is neither
    returned nor fed back), the token that fills ``max_new_tokens`` ends it too.  Rows of
    requests that had ended before the step was read were computed in vain and are skipped."""
    if len(chosen) != len(rows):
        raise GenerationError(f"the backend chose {len(chosen)} tokens for {len(rows)} sequences")
    for r, tok in zip(rows, chosen):
        if r.finish_reason:
            continue
        if tok in stop:
            r.finish_reason = "stop"
        else:
            r.output.append(int(tok))
            if len(r.output) >= r.max_new_tokens:
                r.finish_reason = "length"


def run_batch(backend: Backend, batch: Sequence[Request], stop_token_ids: Iterable[int]) -> None:
    """Generate for the requests of one batch, which start together.  A request ends when a
    stop token is chosen (which is neither returned nor fed back) or when it has its
    ``max_new_tokens``; its slot is given back at once and the others go on.

    A backend that is ``pipelined`` (``decode_begin`` / ``decode_end``) is driven one step ahead:
    the next step is launched before the tokens of the step in flight have been read, for the
    requests that cannot end by length with those tokens; such a row takes its token from the
    step in flight.  If a stop token then shows that a request has ended, the row that ran for it
    is dropped and its slot is given back when that step has been read.  The tokens returned
    are the same either way."""
    stop = frozenset(stop_token_ids)
    active = [r for r in batch if r.max_new_tokens > 0]
    for r in batch:
        if r.max_new_tokens <= 0:
            r.finish_reason = "length"
    if not active:
        return
    slot_of = {r.index: backend.open() for r in active}
    try:
        chosen = backend.prefill([slot_of[r.index] for r in active], [r.prompt for r in active],
                                 [r.index for r in active])
        if getattr(backend, "pipelined", False):
            _decode_ahead(backend, active, chosen, slot_of, stop)
            return
        while True:
            _settle(active, chosen, stop)
            for r in active:
                if r.finish_reason:
                    backend.close(slot_of.pop(r.index))
            active = [r for r in active if not r.finish_reason]
            if not active:
                return
            chosen = backend.decode([slot_of[r.index] for r in active], [r.output[-1] for r in active],
                                    [r.index for r in active], [len(r.output) for r in active])
    finally:
        for slot in slot_of.values():          # only after an error: nothing stays held
            backend.close(slot)


def _decode_ahead(backend, rows: List[Request], chosen: Sequence[int], slot_of: dict, stop: frozenset) -> None:
    """The decode loop of ``run_batch`` for a pipelined backend.  ``chosen`` are the tokens of
    ``rows``; ``flight`` is the step launched before they were read (None: none)."""
    flight = None                              # (handle, its rows)
    unread = []                                # handles of the steps launched and not read, oldest first
    try:
        while True:
            _settle(rows, chosen, stop)
            flying = {r.index for r in flight[1]} if flight else set()
            for r in rows:                     # ended, and no launched step still writes its cache
                if r.finish_reason and r.index in slot_of and r.index not in flying:
                    backend.close(slot_of.pop(r.index))
            if flight is None:
                rows = [r for r in rows if not r.finish_reason]
                if not rows:
                    return
                flight = (backend.decode_begin([slot_of[r.index] for r in rows], [r.output[-1] for r in rows],
                                               [-1] * len(rows), [r.index for r in rows], [len(r.output) for r in rows]),
                          rows)
                unread.append(flight[0])
            # the step after the one in flight, for those whom its token cannot bring to their length
            ahead_rows = flight[1]
            nxt = [r for r in ahead_rows if not r.finish_reason and len(r.output) + 1 < r.max_new_tokens]
            after = None
            if nxt:
                place = {r.index: j for j, r in enumerate(ahead_rows)}
                after = (backend.decode_begin([slot_of[r.index] for r in nxt], [0] * len(nxt),
                                              [place[r.index] for r in nxt], [r.index for r in nxt],
                                              [len(r.output) + 1 for r in nxt]), nxt)
                unread.append(after[0])
            handle = unread.pop(0)
            chosen, rows = backend.decode_end(handle), ahead_rows
            flight = after
    finally:
        for handle in unread:                  # an error: let what was launched end before its slots are given back
            try:
                backend.decode_end(handle)
            except Exception:                  # noqa: BLE001
                pass
        idle = getattr(backend, "decode_idle", None)
        if idle:
            idle()


def generate(backend: Backend, prompts: Sequence[Sequence[int]], max_new_tokens, stop_token_ids: Iterable[int],
             max_batch: int, max_tokens: int) -> List[Request]:
    """``max_new_tokens`` is one number or one per prompt.  An empty prompt yields nothing
    (pico-engine returns ("", []) for it, src/pico_engine/engine.py:313-314)."""
    if isinstance(max_new_tokens, int):
        max_new_tokens = [max_new_tokens] * len(prompts)
    if len(max_new_tokens) != len(prompts):
        raise GenerationError("max_new_tokens must be one number or one per prompt")
    if any(m < 0 for m in max_new_tokens):
        raise GenerationError("max_new_tokens must be non-negative")
    requests = [Request(i, [int(t) for t in p], int(m)) for i, (p, m) in enumerate(zip(prompts, max_new_tokens))]
    runnable = []
    for r in requests:
        if not r.prompt:
            r.finish_reason = "empty"
        else:
            runnable.append(r)
    for batch in plan_batches(runnable, max_batch, max_tokens):
        run_batch(backend, batch, stop_token_ids)
    return requests
