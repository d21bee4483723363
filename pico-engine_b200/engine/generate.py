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


def run_batch(backend: Backend, batch: Sequence[Request], stop_token_ids: Iterable[int]) -> None:
    """Generate for the requests of one batch, which start together.  A request ends when a
    stop token is chosen (which is neither returned nor fed back) or when it has its
    ``max_new_tokens``; its slot is given back at once and the others go on."""
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
        while True:
            if len(chosen) != len(active):
                raise GenerationError(f"the backend chose {len(chosen)} tokens for {len(active)} sequences")
            still: List[Request] = []
            for r, tok in zip(active, chosen):
                if tok in stop:
                    r.finish_reason = "stop"
                else:
                    r.output.append(int(tok))
                    if len(r.output) >= r.max_new_tokens:
                        r.finish_reason = "length"
                if r.finish_reason:
                    backend.close(slot_of.pop(r.index))
                else:
                    still.append(r)
            active = still
            if not active:
                return
            chosen = backend.decode([slot_of[r.index] for r in active], [r.output[-1] for r in active],
                                    [r.index for r in active], [len(r.output) for r in active])
    finally:
        for slot in slot_of.values():          # only after an error: nothing stays held
            backend.close(slot)


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
