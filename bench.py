"""The benchmark the build driver runs: decode tokens per second of the Qwen2.5-0.5B shape
(random weights, bfloat16) at batch 8 and context 4096 on one B200, with the 2,048-token
prefill, decode at batch 1 and 64, the end-to-end figure through ``Engine.generate`` and the
roofline fractions on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A "step" is one decode step of the whole batch.  This library runs on one GPU: for
``--gpus N`` with N > 1 it says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED, BATCH, CONTEXT, PREFILL_TOKENS = 2, 8, 4096, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            if d.get("hbm_gbs") and d.get("bf16_tflops"):
                return d, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def reference_arm(steps: int, warmup: int, layers) -> int:
    """pico-engine itself from baseline/_ref (see baseline/reference_arm.py), in a process of its own with a time
    limit; whatever goes wrong there becomes the ``unavailable`` line."""
    import subprocess
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "--steps", str(steps), "--warmup", str(warmup)]
    if layers:
        cmd += ["--layers", str(layers)]
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
        lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
        if proc.returncode == 0 and lines:
            print(lines[-1])
            return 0
        why = (proc.stderr.strip().splitlines() or ["no output"])[-1][:300]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference run ended with code {proc.returncode}: {why}"}))
    except subprocess.TimeoutExpired:
        print(json.dumps({"impl": "reference", "unavailable": "the reference run did not finish within 1500 s"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (recorded in config)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args.steps, max(args.warmup, 3), args.layers)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)

    import torch
    from pico_engine import benchmark as B
    from pico_engine.config import config_from_dict
    from pico_engine.engine.engine import Engine

    from pico_engine.config.shapes import shape
    cfg_dict = shape("qwen2.5-0.5b")                       # BASELINE.json configs[2]
    layers_full = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    cfg = config_from_dict(cfg_dict)
    eng = Engine.from_config(cfg, seed=SEED, draw_on="cuda", dtype="bfloat16", device="cuda:0", max_batch=64)
    eng.ensure_cache(64 * CONTEXT, CONTEXT, max_seqs=64)
    pk, pk_kind = peaks()

    with B.ClockSampler() as clocks:
        main_run = B.decode_device(eng, BATCH, CONTEXT, args.steps, warmup)
    side_steps = min(args.steps, 128)
    b1 = B.decode_device(eng, 1, CONTEXT, side_steps, warmup)
    b64 = B.decode_device(eng, 64, CONTEXT, side_steps, warmup)
    pre = B.prefill_device(eng, PREFILL_TOKENS)
    e2e = B.decode_end_to_end(eng, BATCH, CONTEXT, min(args.steps, 256))

    record = {
        "metric": "decode tokens/s, batch 8, context 4096 (Qwen2.5-0.5B shape)", "value": main_run["tokens_per_s"],
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": main_run["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "Qwen2.5-0.5B shape, random weights seed 2", "global_batch": BATCH, "seq_len": CONTEXT,
                   "parallelism": "none", "layers": cfg.num_hidden_layers, "layers_of_configuration": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied_head": cfg.tie_word_embeddings, "prefill_tokens": PREFILL_TOKENS, "cuda_graph": main_run["graph"],
                   "l2": "each step reads 0.99 GB of weights, more than the 126 MB L2",
                   "context_during_timing": f"{CONTEXT - args.steps + 1}..{CONTEXT}", "peaks": pk_kind},
        "e2e": {"value": e2e["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e2e["d2h_bytes_per_step"], "ms_per_step": e2e["ms_per_step"],
                "clock": "host clock around Engine.generate's decode steps: token lists in and out, each step's "
                         "description copied from pinned memory, each step's tokens read back; the loop launches "
                         "a step before it has read the one in flight, so host work hides behind the device"},
        "gpu_launches": main_run["launches_per_step"] * args.steps,
        "prefill": {"value": pre["tokens_per_s"], "tokens": pre["tokens"], "ms": pre["ms"],
                    "frac": pre["tflops_per_s"] / pk["bf16_tflops"]},
        "roofline": {"bound": "hbm", "achieved": main_run["gbytes_per_s"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": main_run["gbytes_per_s"] / pk["hbm_gbs"]},
        "points": {"decode_b1": b1["tokens_per_s"], "decode_b64": b64["tokens_per_s"],
                   "decode_b1_hbm_frac": b1["gbytes_per_s"] / pk["hbm_gbs"],
                   "decode_b64_hbm_frac": b64["gbytes_per_s"] / pk["hbm_gbs"]},
        "clocks": clocks.record(),
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
