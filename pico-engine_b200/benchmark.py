"""Measuring decode and prefill throughput, with the work of each step counted in bytes and
floating-point operations so that a number can be set against the machine's peaks.

The protocol is pico-engine's evidence protocol (src/pico_engine/evidence.py:35-56, 138-163):
warm-ups, then repetitions summarised by median, 10th and 90th percentile; its benchmark times
one prefill and a decode loop (src/pico_engine/benchmark.py:18-44).  Here the device is timed
with CUDA events on the launching stream, and the end-to-end figure goes through
``Engine.generate`` with host tokens in and out.

    python -m pico_engine.benchmark MODEL --batch 1,8,64 --context 4096 --prefill 2048 --n-tokens 128
"""
from __future__ import annotations

import argparse
import json
import time
from typing import Dict, List, Sequence

import torch


# ---------------------------------------------------------------------------- statistics

def percentile(values: Sequence[float], q: float) -> float:
    """Linear interpolation between order statistics (pico-engine src/pico_engine/evidence.py:35-44)."""
    if not values:
        raise ValueError("no values")
    v = sorted(values)
    if len(v) == 1:
        return float(v[0])
    x = (len(v) - 1) * q / 100.0
    lo = int(x)
    hi = min(lo + 1, len(v) - 1)
    return float(v[lo] + (v[hi] - v[lo]) * (x - lo))


def summary(values: Sequence[float]) -> Dict[str, float]:
    """median / p10 / p90 / min / max (pico-engine src/pico_engine/evidence.py:47-56)."""
    return {"median": percentile(values, 50), "p10": percentile(values, 10), "p90": percentile(values, 90),
            "min": float(min(values)), "max": float(max(values)), "n": len(values)}


# ---------------------------------------------------------------------------- work accounting

def kv_bytes_per_token(engine) -> int:
    """Bytes of keys and values one cached token holds over all layers."""
    total = 0
    itemsize = torch.empty(0, dtype=engine.dtype).element_size()
    for need in engine.model.cache_needs():
        if need is not None and need.kv is not None:
            total += 2 * need.kv.n_kv_heads * need.kv.head_dim * itemsize
    return total


def decode_step_bytes(engine, batch: int, mean_context: float) -> float:
    """What a decode step has to read: every weight it uses once, and the cache of the live sequences."""
    return engine.model.step_weight_bytes() + batch * mean_context * kv_bytes_per_token(engine)


def prefill_flops(engine, tokens: int) -> float:
    """Multiply-adds of one sequence of ``tokens`` from an empty cache, times two: all matrices
    for every token, the head for the last, causal attention for every layer."""
    model = engine.model
    flops = 0.0
    for entry in model.plan.schedule:
        layer = model.layers[entry.layer]
        for part in (layer.mixer, layer.feed_forward):
            if part is not None:
                flops += sum(2.0 * tokens * t.numel() for t in part.weights() if t.dim() == 2)
        spec = layer.mixer.spec if layer.mixer is not None else None
        if hasattr(spec, "n_heads"):
            w = spec.window
            seen = sum(min(p + 1, w) if w else p + 1 for p in range(tokens))
            flops += 4.0 * spec.n_heads * spec.head_dim * seen
    return flops + 2.0 * model.head.numel()


# ---------------------------------------------------------------------------- setting sequences up

def open_sequences(engine, batch: int, length: int, seed: int = 0) -> List[int]:
    """``batch`` sequences of ``length`` random tokens in the cache (filled one sequence at a time)."""
    g = torch.Generator().manual_seed(seed)
    slots = []
    for _ in range(batch):
        s = engine.cache.open()
        ids = torch.randint(0, engine.model.plan.vocab_size, (length,), generator=g).tolist()
        for at in range(0, length, 4096):
            engine.stepper.step([s], [ids[at:at + 4096]], [[]])
        slots.append(s)
    return slots


def close_sequences(engine, slots) -> None:
    for s in slots:
        engine.cache.close(s)


# ---------------------------------------------------------------------------- measurements

@torch.inference_mode()
def decode_device(engine, batch: int, context: int, steps: int, warmup: int, use_graph: bool = True, seed: int = 0) -> dict:
    """Device time of ``steps`` decode steps of ``batch`` sequences whose length reaches ``context`` at
    the last step.  Each step is the whole step: embedding to the chosen token."""
    from .engine.graph import GraphedDecode
    from .ops import library
    from .sampling import Sampler, SamplingParams
    start = context - steps - warmup
    if start < 1:
        raise ValueError(f"context {context} has no room for {steps} + {warmup} steps")
    engine.ensure_cache(batch * ((context + 63) // 64) * 64, context, max_seqs=max(batch, engine.max_batch))
    slots = open_sequences(engine, batch, start, seed)
    sampler = Sampler(SamplingParams(temperature=0.0))
    g = torch.Generator().manual_seed(seed + 1)
    tokens = torch.randint(0, engine.model.plan.vocab_size, (steps + warmup, batch), generator=g).tolist()
    reqs, zeros = list(range(batch)), [0] * batch
    dec = None
    try:
        if use_graph:
            dec = GraphedDecode(engine.stepper, sampler, batch)
            run = lambda i: dec.run(slots, tokens[i], reqs, zeros)
        else:
            run = lambda i: sampler.choose(engine.stepper.step(slots, [[t] for t in tokens[i]]), None, None)
        before = library.LAUNCHES[0]
        run(0)                                                       # with a graph: warm-up runs and the capture
        first = library.LAUNCHES[0] - before
        per_step = first // 4 if dec is not None and dec.graph is not None else first   # 3 warm-up runs + 1 capture
        for i in range(1, warmup):
            run(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch.cuda.nvtx.range_push("pico_decode")
        for i in range(warmup, warmup + steps):
            run(i)
        torch.cuda.nvtx.range_pop()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
    finally:
        close_sequences(engine, slots)
    mean_ctx = context - (steps - 1) / 2.0
    nbytes = decode_step_bytes(engine, batch, mean_ctx)
    return {"batch": batch, "context": context, "steps": steps, "ms_per_step": ms, "tokens_per_s": batch * 1000.0 / ms,
            "bytes_per_step": nbytes, "gbytes_per_s": nbytes / ms / 1e6, "launches_per_step": per_step,
            "graph": bool(dec is not None and dec.graph is not None)}


@torch.inference_mode()
def prefill_device(engine, tokens: int, repetitions: int = 5, warmup: int = 3, seed: int = 0) -> dict:
    """Device time of one step that runs a prompt of ``tokens`` tokens and returns its last logits."""
    engine.ensure_cache(((tokens + 63) // 64) * 64, tokens)
    ids = torch.randint(0, engine.model.plan.vocab_size, (tokens,), generator=torch.Generator().manual_seed(seed)).tolist()
    times = []
    for i in range(warmup + repetitions):
        s = engine.cache.open()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch.cuda.nvtx.range_push("pico_prefill")
        engine.stepper.step([s], [ids])
        torch.cuda.nvtx.range_pop()
        e1.record()
        torch.cuda.synchronize()
        engine.cache.close(s)
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    ms = percentile(times, 50)
    flops = prefill_flops(engine, tokens)
    return {"tokens": tokens, "ms": ms, "tokens_per_s": tokens * 1000.0 / ms, "flops": flops,
            "tflops_per_s": flops / ms / 1e9, "times_ms": summary(times)}


def decode_end_to_end(engine, batch: int, context: int, steps: int, use_graph: bool = True, seed: int = 0) -> dict:
    """Decode throughput through ``Engine.generate``: prompts and results are host token lists;
    every step copies its inputs from pinned host memory and reads its chosen tokens back."""
    start = context - steps
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, engine.model.plan.vocab_size, (start,), generator=g).tolist() for _ in range(batch)]
    engine.max_batch = max(engine.max_batch, batch)
    # an untimed call first: the first generation of a process captures its graph and loads its kernels
    engine.generate([p[:64] for p in prompts], max_tokens=4, temperature=0.0, use_graph=use_graph, stop_token_ids=())
    out = engine.generate(prompts, max_tokens=steps + 1, temperature=0.0, use_graph=use_graph, stop_token_ids=())
    t = engine.last_timing
    assert all(len(o) == steps + 1 for o in out) and t["decode_steps"] == steps
    return {"batch": batch, "context": context, "steps": steps, "tokens_per_s": batch * steps / t["decode_s"],
            "ms_per_step": 1000.0 * t["decode_s"] / steps, "prefill_s": t["prefill_s"],
            "h2d_bytes_per_step": t["h2d_bytes"] // max(t["decode_steps"], 1), "d2h_bytes_per_step": 4 * batch}


# ---------------------------------------------------------------------------- command line

def main(argv=None) -> None:
    p = argparse.ArgumentParser(description="Decode and prefill throughput of a model folder on one B200")
    p.add_argument("model", nargs="?", help="folder with config.json and model.safetensors")
    p.add_argument("--random", metavar="SHAPE", help="instead of a folder: random weights of a named shape, e.g. qwen2.5-0.5b")
    p.add_argument("--seed", type=int, default=2, help="seed of the random weights")
    p.add_argument("--layers", type=int, help="with --random: fewer layers than the shape has")
    p.add_argument("--batch", default="1,8,64", help="decode batch sizes")
    p.add_argument("--context", type=int, default=4096, help="sequence length reached at the last timed step")
    p.add_argument("--prefill", type=int, default=2048, help="prompt length of the prefill measurement")
    p.add_argument("--n-tokens", type=int, default=128, help="timed decode steps")
    p.add_argument("--warmups", type=int, default=2)
    p.add_argument("--repetitions", type=int, default=3)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--no-graph", action="store_true", help="decode without CUDA graphs")
    p.add_argument("--output", help="write the JSON record here")
    args = p.parse_args(argv)
    from .engine.engine import Engine
    if (args.model is None) == (args.random is None):
        p.error("give a model folder or --random SHAPE")
    if args.random:
        from .config import config_from_dict
        from .config.shapes import shape
        d = shape(args.random)
        if args.layers:
            d["num_hidden_layers"] = args.layers
        eng = Engine.from_config(config_from_dict(d), seed=args.seed, draw_on="cuda", dtype=args.dtype)
    else:
        eng = Engine(args.model, dtype=args.dtype)
    batches = [int(x) for x in args.batch.split(",") if x]
    if batches:
        eng.ensure_cache(max(batches) * ((args.context + 63) // 64) * 64, args.context, max_seqs=max(batches))
    record = {"model": args.model or args.random, "dtype": args.dtype, "graph": not args.no_graph, "decode": {}, "time": time.time()}
    if args.prefill > 0:
        pre = prefill_device(eng, args.prefill, repetitions=args.repetitions, warmup=args.warmups)
        record["prefill"] = pre
        print(f"prefill {pre['tokens']} tokens: {pre['ms']:.3f} ms  {pre['tokens_per_s']:.0f} tok/s  {pre['tflops_per_s']:.1f} TFLOP/s")
    for b in batches:
        runs = [decode_device(eng, b, args.context, args.n_tokens, args.warmups, not args.no_graph, seed=r)
                for r in range(args.repetitions)]
        s = summary([r["tokens_per_s"] for r in runs])
        record["decode"][str(b)] = {"tokens_per_s": s, "last": runs[-1]}
        print(f"decode batch {b}: median {s['median']:.0f} tok/s (p10 {s['p10']:.0f}, p90 {s['p90']:.0f}), "
              f"{runs[-1]['gbytes_per_s']:.0f} GB/s of weights and cache, {runs[-1]['launches_per_step']} launches a step")
    if args.output:
        with open(args.output, "w") as f:
            json.dump(record, f, indent=1)


if __name__ == "__main__":
    main()
