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
import threading
import time
from typing import Dict, List, Optional, Sequence

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


class ClockSampler:
    """Reads SM clocks and throttle reasons through NVML while the timed region runs (reading only)."""

    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int = 0, period_s: float = 0.02):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period_s, self._stop, self._thread, self._h, self._nvml = period_s, threading.Event(), None, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:                                   # noqa: BLE001 - no NVML: the record says so
            self._nvml = None

    def _read(self):
        n = self._nvml
        try:
            self.samples.append(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM))
            bits = n.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons") \
                else n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
            for bit, name in self.REASONS.items():
                if bits & bit and name != "gpu_idle":
                    self.reasons.add(name)
        except Exception:                                   # noqa: BLE001
            pass

    def __enter__(self):
        if self._nvml is not None:
            def loop():
                while not self._stop.is_set():
                    self._read()
                    self._stop.wait(self.period_s)
            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def record(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable: NVML gave no sample"]}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


# ---------------------------------------------------------------------------- work accounting

def kv_bytes_per_token(engine) -> int:
    """Bytes of keys and values one cached token holds over all layers."""
    total = 0
    itemsize = torch.empty(0, dtype=engine.dtype).element_size()
    for need in engine.model.cache_needs():
        if need is not None and need.kv is not None:
            v_heads, v_dim = need.kv.value_shape
            total += (need.kv.n_kv_heads * need.kv.head_dim + v_heads * v_dim) * itemsize
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
def prefill_device(engine, tokens: int, repetitions: int = 5, warmup: int = 3, seed: int = 0, use_graph: bool = True) -> dict:
    """Device time of one step that runs a prompt of ``tokens`` tokens and returns its last logits: the step as
    ``Engine.generate`` runs it (with ``use_graph`` a prompt step of sizes that have come before is a captured graph)."""
    engine.ensure_cache(((tokens + 63) // 64) * 64, tokens)
    ids = torch.randint(0, engine.model.plan.vocab_size, (tokens,), generator=torch.Generator().manual_seed(seed)).tolist()
    times = []
    for i in range(warmup + repetitions):
        s = engine.cache.open()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if i == warmup + repetitions - 1:                 # one step, the last, is marked for a profiler's launch list
            torch.cuda.nvtx.range_push("pico_prefill")
        engine.stepper.step([s], [ids], use_graph=use_graph)
        if i == warmup + repetitions - 1:
            torch.cuda.nvtx.range_pop()
        e1.record()
        torch.cuda.synchronize()
        engine.cache.close(s)
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    ms = percentile(times, 50)
    flops = prefill_flops(engine, tokens)
    return {"tokens": tokens, "ms": ms, "tokens_per_s": tokens * 1000.0 / ms, "flops": flops,
            "tflops_per_s": flops / ms / 1e9, "times_ms": summary(times), "graph": use_graph}


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


@torch.inference_mode()
def generate_protocol(engine, n_requests: int, shortest: int, longest: int, steps: int, warmups: int = 1,
                      repetitions: int = 3, seed: int = 0, use_graph: bool = True) -> dict:
    """``n_requests`` prompts with lengths uniform in [shortest, longest] (seeded), ``steps`` decode steps, all through
    ``Engine.generate`` with host token lists in and out: every repetition's prefill and decode times are kept, and
    summarised by median, 10th and 90th percentile (pico-engine's protocol, src/pico_engine/evidence.py:138-163,
    294-325, which writes every sample and the environment to its receipt)."""
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(shortest, longest + 1, (n_requests,), generator=g).tolist()
    vocab = engine.model.plan.vocab_size
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
    engine.max_batch = max(engine.max_batch, n_requests)
    samples = []
    with ClockSampler(period_s=0.05) as clocks:
        for rep in range(warmups + repetitions):
            t0 = time.perf_counter()
            out = engine.generate(prompts, max_tokens=steps + 1, temperature=0.0, use_graph=use_graph, stop_token_ids=())
            wall = time.perf_counter() - t0
            t = engine.last_timing
            assert all(len(o) == steps + 1 for o in out)
            if rep >= warmups:
                samples.append({"wall_s": wall, "prefill_s": t["prefill_s"], "decode_s": t["decode_s"],
                                "decode_steps": t["decode_steps"],
                                "prefill_tokens_per_s": sum(lengths) / t["prefill_s"],
                                "decode_tokens_per_s": n_requests * t["decode_steps"] / t["decode_s"]})
    mean_ctx = sum(lengths) / n_requests + steps / 2.0
    step_bytes = decode_step_bytes(engine, n_requests, mean_ctx)
    decode = summary([s["decode_tokens_per_s"] for s in samples])
    return {"requests": n_requests, "prompt_lengths": lengths, "prompt_tokens": sum(lengths), "decode_steps": steps,
            "graph": use_graph, "samples": samples, "decode_tokens_per_s": decode,
            "prefill_tokens_per_s": summary([s["prefill_tokens_per_s"] for s in samples]),
            "decode_bytes_per_step": step_bytes,
            "decode_gbytes_per_s": step_bytes * decode["median"] / n_requests / 1e9,
            "clocks": clocks.record(), "weights_bytes": engine.model.step_weight_bytes(),
            "cache_bytes": engine.cache.bytes() if engine.cache is not None else 0}


@torch.inference_mode()
def last_logits(engine, prompts: Sequence[Sequence[int]], batch: int = 8) -> torch.Tensor:
    """float32 logits [len(prompts), vocab] at each prompt's last position (prompts run ``batch`` at a time), on the host."""
    rows = []
    need = max(sum(sorted(((len(p) + 63) // 64 * 64 for p in prompts), reverse=True)[:batch]), 64)
    engine.ensure_cache(need, max(len(p) for p in prompts), max_seqs=batch)
    for at in range(0, len(prompts), batch):
        group = prompts[at:at + batch]
        slots = [engine.cache.open() for _ in group]
        rows.append(engine.stepper.step(slots, group).cpu())
        for s in slots:
            engine.cache.close(s)
    return torch.cat(rows)


def agreement(config, seed: int, prompts: Sequence[Sequence[int]]) -> dict:
    """The bfloat16 engine against the float32 engine on the same weights (drawn once in bfloat16, so that the two
    differ in arithmetic only): the largest difference of the last-position logits relative to their size, and
    how often the most likely token is the same."""
    import gc
    from .engine.engine import Engine
    out = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_config(config, seed=seed, draw_on="cuda", dtype=dtype)
        out[dtype] = last_logits(eng, prompts)
        del eng
        gc.collect(); torch.cuda.empty_cache()
    a, b = out["float32"], out["bfloat16"]
    scale = float(a.abs().max())
    return {"prompts": len(prompts), "logit_scale": scale, "max_difference_of_scale": float((a - b).abs().max()) / scale,
            "same_most_likely_token": float((a.argmax(-1) == b.argmax(-1)).float().mean())}


@torch.inference_mode()
def product_times(engine, rows: int) -> dict:
    """Device time of the first layer's four matrix products at ``rows`` rows, each as this library's tcgen05 kernel
    with its fused epilogue and as the library product followed by this library's separate kernel: the measurement
    by which ``ops.linear`` chooses (a captured graph of six calls, best of three replays), in microseconds."""
    import sys
    from .ops import kernels
    L = sys.modules[__package__ + ".ops.linear"]
    layer = engine.model.layers[0]
    att, ffn = layer.mixer, layer.feed_forward
    dev, dt = engine.device, torch.bfloat16
    out = {}
    if engine.dtype != dt or att is None or ffn is None or not hasattr(att, "w_qkv") or not hasattr(ffn, "w_gate_up"):
        return out
    s = att.spec
    h = torch.randn(rows, s.hidden, device=dev).to(dt)
    a = torch.randn(rows, att.w_o.shape[1], device=dev).to(dt)
    act = torch.randn(rows, ffn.w_down.shape[1], device=dev).to(dt)
    x = torch.zeros(rows, s.hidden, device=dev)
    pos = torch.zeros(rows, dtype=torch.int32, device=dev)
    engine.model.prepare(max(rows, 64))
    cos, sin = getattr(att.position, "cos", None), getattr(att.position, "sin", None)
    t = L._device_time
    out["gate_up_swiglu"] = {"tcgen05": t(lambda: kernels.gemm_tcgen05(h, ffn.w_gate_up, swiglu=True)),
                             "library": t(lambda: kernels.swiglu(torch.mm(h, ffn.w_gate_up.t())))}
    if s.head_dim in kernels.GEMM_ROPE_HEAD_DIMS:
        def library_qkv():
            y = torch.addmm(att.b_qkv, h, att.w_qkv.t()) if att.b_qkv is not None else torch.mm(h, att.w_qkv.t())
            kernels.rope_store(y, s.n_heads, s.n_kv_heads, s.head_dim, cos, sin, pos, pos, None, None, None, 0)
        out["qkv_rope"] = {"tcgen05": t(lambda: kernels.gemm_qkv_rope_store(h, att.w_qkv, att.b_qkv, s.n_heads, s.n_kv_heads,
                                                                              s.head_dim, cos, sin, pos, pos, None, None, None, 0)),
                           "library": t(library_qkv)}
    out["o_proj_residual"] = {"tcgen05": t(lambda: kernels.gemm_tcgen05(a, att.w_o, accumulate_into=x)),
                              "library": t(lambda: kernels.residual_add(x, torch.mm(a, att.w_o.t())))}
    out["down_residual"] = {"tcgen05": t(lambda: kernels.gemm_tcgen05(act, ffn.w_down, accumulate_into=x)),
                            "library": t(lambda: kernels.residual_add(x, torch.mm(act, ffn.w_down.t())))}
    if rows <= kernels.SPLITK_MAX_ROWS:
        # the two kernels for 17 to 64 rows that nothing chooses by itself: K cut over a cluster on tcgen05
        # (csrc/gemm_splitk.cu), and the mma.sync kernel with the norm in its prologue (csrc/linear_batch.cu; its
        # counterpart on the library's side has the norm as a kernel of its own)
        norm1, norm2 = layer.mixer_norm, layer.feed_forward_norm
        xs = torch.randn(rows, s.hidden, device=dev)
        out["gate_up_swiglu"]["splitk"] = t(lambda: kernels.gemm_tcgen05(h, ffn.w_gate_up, swiglu=True, orientation="splitk"))
        out["qkv_rope"] = out.get("qkv_rope", {})
        out["qkv_rope"]["splitk"] = t(lambda: kernels.gemm_qkv_rope_store(h, att.w_qkv, att.b_qkv, s.n_heads, s.n_kv_heads, s.head_dim,
                                                                            cos, sin, pos, pos, None, None, None, 0, orientation="splitk"))
        out["o_proj_residual"]["splitk"] = t(lambda: kernels.gemm_tcgen05(a, att.w_o, accumulate_into=x, orientation="splitk"))
        out["down_residual"]["splitk"] = t(lambda: kernels.gemm_tcgen05(act, ffn.w_down, accumulate_into=x, orientation="splitk"))
        if rows > kernels.FUSED_MAX_ROWS and hasattr(norm1, "eps") and hasattr(norm2, "eps"):
            out["gate_up_swiglu"]["batch_with_norm"] = t(lambda: kernels.norm_gate_up_swiglu(xs, norm2.weight, norm2.eps, ffn.w_gate_up))
            out["gate_up_swiglu"]["library_with_norm"] = t(lambda: kernels.swiglu(torch.mm(
                kernels.rmsnorm(xs, norm2.weight, norm2.eps, dt), ffn.w_gate_up.t())))
            out["qkv_rope"]["batch_with_norm"] = t(lambda: kernels.norm_qkv_rope_store(
                xs, norm1.weight, norm1.eps, att.w_qkv, att.b_qkv, s.n_heads, s.n_kv_heads, s.head_dim, cos, sin, pos, pos, None, None, None, 0))
            out["o_proj_residual"]["batch"] = t(lambda: kernels.linear_fused(a, att.w_o, accumulate_into=x))
            out["down_residual"]["batch"] = t(lambda: kernels.linear_fused(act, ffn.w_down, accumulate_into=x))
    kernels.check_status(dev)
    return out


def environment() -> dict:
    """What the numbers were measured on (pico-engine's receipts carry the same, src/pico_engine/evidence.py:294-325)."""
    import platform
    p = torch.cuda.get_device_properties(0) if torch.cuda.is_available() else None
    return {"gpu": p.name if p else None, "sms": p.multi_processor_count if p else None,
            "memory_gb": round(p.total_memory / 2 ** 30, 1) if p else None, "torch": torch.__version__,
            "cuda": torch.version.cuda, "python": platform.python_version(), "time": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}


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
    p.add_argument("--save-choices", metavar="FILE", help="write which implementation each matrix product got (ops.linear.Choice); "
                   "PICO_ENGINE_GEMM_CHOICES=FILE makes a later run start from them")
    p.add_argument("--products", default="", metavar="ROWS[,ROWS...]", help="also: the first layer's matrix products at these "
                   "row counts, as this library's fused tcgen05 kernel and as the library product plus the separate pass")
    p.add_argument("--requests", type=int, default=0, help="also: generation of this many requests with unequal prompts "
                   "through Engine.generate (--prompt-lengths, --n-tokens decode steps)")
    p.add_argument("--prompt-lengths", default="64,2048", metavar="SHORTEST,LONGEST", help="prompt lengths are uniform in this range")
    p.add_argument("--agreement", action="store_true", help="with --random and --requests: compare the last-position logits of "
                   "the bfloat16 engine with the float32 engine's on the same weights")
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
    record = {"model": args.model or args.random, "dtype": args.dtype, "graph": not args.no_graph, "decode": {},
              "environment": environment()}
    if args.random and args.layers:
        record["layers"] = args.layers
    if args.prefill > 0:
        pre = prefill_device(eng, args.prefill, repetitions=args.repetitions, warmup=max(args.warmups, 2), use_graph=not args.no_graph)
        record["prefill"] = pre
        print(f"prefill {pre['tokens']} tokens: {pre['ms']:.3f} ms  {pre['tokens_per_s']:.0f} tok/s  {pre['tflops_per_s']:.1f} TFLOP/s")
    for b in batches:
        runs = [decode_device(eng, b, args.context, args.n_tokens, args.warmups, not args.no_graph, seed=r)
                for r in range(args.repetitions)]
        s = summary([r["tokens_per_s"] for r in runs])
        record["decode"][str(b)] = {"tokens_per_s": s, "last": runs[-1]}
        print(f"decode batch {b}: median {s['median']:.0f} tok/s (p10 {s['p10']:.0f}, p90 {s['p90']:.0f}), "
              f"{runs[-1]['gbytes_per_s']:.0f} GB/s of weights and cache, {runs[-1]['launches_per_step']} launches a step")
    for rows in [int(x) for x in args.products.split(",") if x]:
        times = product_times(eng, rows)
        record.setdefault("products", {})[str(rows)] = times
        for name, t in times.items():
            print(f"{rows} rows {name}: " + ", ".join(f"{k} {v:.1f} us" for k, v in t.items()))
    if args.requests > 0:
        lo, hi = (int(x) for x in args.prompt_lengths.split(","))
        gen = generate_protocol(eng, args.requests, lo, hi, args.n_tokens, args.warmups, args.repetitions, use_graph=not args.no_graph)
        record["generate"] = gen
        d, f = gen["decode_tokens_per_s"], gen["prefill_tokens_per_s"]
        print(f"generate {args.requests} requests of {lo}..{hi} prompt tokens, {args.n_tokens} steps: decode median {d['median']:.0f} tok/s "
              f"(p10 {d['p10']:.0f}, p90 {d['p90']:.0f}), {gen['decode_gbytes_per_s']:.0f} GB/s of weights and cache; prefill median "
              f"{f['median']:.0f} tok/s")
        if args.agreement:
            if not args.random:
                p.error("--agreement needs --random (the float32 engine is drawn from the same seed)")
            g = torch.Generator().manual_seed(0)
            lengths = gen["prompt_lengths"]
            prompts = [torch.randint(0, eng.model.plan.vocab_size, (n,), generator=g).tolist() for n in lengths]
            config, seed = eng.config, args.seed
            del eng
            import gc
            gc.collect(); torch.cuda.empty_cache()
            record["agreement"] = agreement(config, seed, prompts)
            a = record["agreement"]
            print(f"bfloat16 against float32: logits differ by {a['max_difference_of_scale']:.3g} of their size, "
                  f"same most likely token in {a['same_most_likely_token']:.2f} of {a['prompts']} prompts")
    import sys
    choice = sys.modules[__package__ + ".ops.linear"].Choice
    record["product_choices"] = {"|".join(str(x) for x in k): {"taken": v, "tcgen05_us": choice.timings.get(k, (None, None))[0],
                                                               "library_us": choice.timings.get(k, (None, None))[1]}
                                 for k, v in choice.table.items()}
    if args.save_choices:
        choice.save(args.save_choices)
    if args.output:
        with open(args.output, "w") as f:
            json.dump(record, f, indent=1)


if __name__ == "__main__":
    main()
