"""Traces for the replay tests: the same requests cut into steps in three ways, run either in
this process through the library's step function or through ``bin/trace_run``."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def whole(requests: dict) -> list:
    """Each request alone, its whole token list in one step, every position wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def tail(requests: dict, n_tail: int = 32) -> list:
    """Each request alone: all but the last ``n_tail`` tokens in one step, then one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - n_tail)
        steps.append({"entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for p in range(head, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def batched(requests: dict, batch_size: int, prompt_fraction: float = 0.5) -> list:
    """Batches of ``batch_size`` requests that start together: the first part of each request
    in one step, then one token each; shorter requests end earlier; one batch after another."""
    steps = []
    ids = list(requests)
    for b0 in range(0, len(ids), batch_size):
        group = ids[b0:b0 + batch_size]
        heads = {r: max(1, int(len(requests[r]) * prompt_fraction)) for r in group}
        steps.append({"entries": [{"id": r, "tokens": requests[r][:heads[r]], "want": list(range(heads[r]))} for r in group],
                      "end": [r for r in group if heads[r] == len(requests[r])]})
        at = dict(heads)
        live = [r for r in group if at[r] < len(requests[r])]
        while live:
            entries = [{"id": r, "tokens": [requests[r][at[r]]], "want": [0]} for r in live]
            for r in live:
                at[r] += 1
            done = [r for r in live if at[r] == len(requests[r])]
            steps.append({"entries": entries, "end": done})
            live = [r for r in live if r not in done]
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def scheduled(requests: dict, plan: dict) -> list:
    """The general cut.  ``plan[id] = (first step, [tokens brought in each of its steps])``: a request
    joins at its first step and brings the listed numbers of tokens in consecutive steps, so one
    step can carry a fresh prompt, a later piece of another prompt and single tokens side by side.
    Every position is wanted."""
    at = {r: 0 for r in requests}
    last = max(first + len(cuts) for first, cuts in plan.values())
    steps = []
    for k in range(last):
        entries, done = [], []
        for r, (first, cuts) in plan.items():
            if first <= k < first + len(cuts):
                n = cuts[k - first]
                entries.append({"id": r, "tokens": requests[r][at[r]:at[r] + n], "want": list(range(n))})
                at[r] += n
                if k == first + len(cuts) - 1:
                    done.append(r)
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": done})
    assert all(at[r] == len(requests[r]) for r in requests), "the plan does not cover every token"
    return steps


def pieces(requests: dict, fractions=(0.45, 0.35, 0.2)) -> list:
    """All requests start together and bring their prompts in pieces of unequal size (the later
    pieces start inside the sequence and have several tokens)."""
    plan = {}
    for i, (r, toks) in enumerate(requests.items()):
        n = len(toks)
        fr = fractions[i % len(fractions):] + fractions[:i % len(fractions)]      # every request is cut elsewhere
        cuts, left = [], n
        for f in fr[:-1]:
            c = min(left, max(1, int(n * f)))
            if c:
                cuts.append(c)
                left -= c
        if left:
            cuts.append(left)
        plan[r] = (0, cuts)
    return scheduled(requests, plan)


def mixed(requests: dict) -> list:
    """Steps that carry a whole prompt, a piece of one and single tokens side by side: request i
    joins at step i, brings most of its tokens in one or two pieces and the rest one by one."""
    plan = {}
    for i, (r, toks) in enumerate(requests.items()):
        n = len(toks)
        singles = min(n - 1, 2 + i)
        head = n - singles
        cuts = [head] if head < 4 or i % 2 == 0 else [head - head // 3, head // 3]
        plan[r] = (i, cuts + [1] * singles)
    return scheduled(requests, plan)


def max_tokens_of(steps: list) -> int:
    """The most tokens live requests hold at any time, each rounded up to 64."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + 63) // 64 * 64 for n in held.values()))
        for r in s["end"]:
            held.pop(r, None)
    return peak


def collect(steps: list, read_step) -> dict:
    """{(request id, position): logits row} from ``read_step(step) -> array [wanted, vocab]``."""
    out, at = {}, {}
    for s in steps:
        rows = None
        k = 0
        for e in s["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                if rows is None:
                    rows = read_step(s["step"])
                out[(e["id"], base + w)] = rows[k]
                k += 1
            at[e["id"]] = base + len(e["tokens"])
        assert rows is None or k == rows.shape[0], (s["step"], k, rows.shape)
    return out


def run_in_process(engine, steps: list, max_tokens: int | None = None) -> dict:
    """Drive the engine's step function as bin/trace_run does."""
    from pico_engine.cache import PAGE
    n = max_tokens or max_tokens_of(steps)
    engine.cache = engine.stepper = None
    engine._graphs.clear()
    engine._want_tokens = engine._want_context = None
    engine.ensure_cache(n, min(n, engine.model.plan.max_positions), max_seqs=max(1, n // PAGE))
    assert engine.cache.n_pages == n // PAGE
    stepper, cache = engine.stepper, engine.cache
    slot_of, results = {}, {}
    for s in steps:
        for e in s["entries"]:
            if e["id"] not in slot_of:
                slot_of[e["id"]] = cache.open()
        logits = stepper.step([slot_of[e["id"]] for e in s["entries"]], [e["tokens"] for e in s["entries"]],
                              [e["want"] for e in s["entries"]])
        results[s["step"]] = logits.cpu().numpy()
        for r in s["end"]:
            cache.close(slot_of.pop(r))
        cache.check()
    assert not slot_of and not cache.lengths and all(g.pages.free_count == g.pages.n for g in cache.groups)
    return collect(steps, lambda i: results[i])


def run_binary(model_dir: str, dtype: str, steps: list, out_dir: str, vocab: int, max_tokens: int | None = None,
               env: dict | None = None) -> dict:
    """The same through ``bin/trace_run``, one line at a time, waiting for each ``done``."""
    n = max_tokens or max_tokens_of(steps)
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                             "--out", out_dir, "--max-tokens", str(n)], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                            text=True, env=env)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"trace_run answered {line!r} to step {s['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    return collect(steps, lambda i: np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, vocab))


def plain_logits(cfg: dict, weights: dict, requests: dict) -> dict:
    import plain_qwen2 as plain
    out = {}
    for rid, toks in requests.items():
        logits = plain.forward(cfg, weights, toks).cpu().numpy()
        for p in range(len(toks)):
            out[(rid, p)] = logits[p]
    return out


def compare(got: dict, want: dict, dtype: str, what: str) -> None:
    """Every wanted (request, position) is there and close to the plain logits; the first
    wrong place is reported by request and position."""
    from conftest import close_enough
    assert set(got) == set(want), (what, sorted(set(want) - set(got))[:5], sorted(set(got) - set(want))[:5])
    for key in sorted(want, key=lambda k: (str(k[0]), k[1])):
        ok, msg = close_enough(torch.from_numpy(np.asarray(got[key])), torch.from_numpy(np.asarray(want[key])), dtype)
        assert ok, f"{what}: request {key[0]!r} position {key[1]}: {msg}"
