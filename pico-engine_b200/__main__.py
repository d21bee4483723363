"""Command line: load a model folder and generate token ids.

Options are pico-engine's (src/pico_engine/__main__.py:23-39) with their names, defaults and
meanings: ``--prompt``, ``--max-tokens 64``, ``--temperature 0.7`` (0 is greedy), ``--top-p 0.9``,
``--top-k 0``, ``--no-graph``.  There is no tokenizer in this library, so ``--prompt`` takes token
ids ("5,17,3"; repeat the option for a batch) and the output is token ids; ``--seed`` and
``--dtype`` are additions.  ``--n-gpu-layers`` (offload of another architecture) is not taken.
"""
from __future__ import annotations

import argparse
import json
import time
from pathlib import Path


def parse_ids(text: str) -> list[int]:
    text = text.strip()
    if text.startswith("["):
        return [int(t) for t in json.loads(text)]
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv=None) -> None:
    p = argparse.ArgumentParser(
        prog="pico_engine", description="Generate token ids with a dense Qwen2 model folder on one B200",
        epilog='example: python -m pico_engine models/tiny --prompt "5,17,3" --max-tokens 11 --temperature 0')
    p.add_argument("model", type=Path, help="folder with config.json and model.safetensors")
    p.add_argument("--prompt", action="append", help='token ids of a prompt, e.g. "5,17,3"; repeat for a batch')
    p.add_argument("--prompt-file", type=Path, help="JSON file holding a list of prompts (lists of token ids)")
    p.add_argument("--max-tokens", type=int, default=64)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--seed", type=int, default=0, help="names the stream of random draws")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--no-graph", action="store_true", help="disable CUDA-graph decode and launch every kernel")
    args = p.parse_args(argv)

    if not (args.model / "config.json").is_file():
        p.error(f"model folder has no config.json: {args.model}")
    if args.max_tokens < 0:
        p.error("--max-tokens must be non-negative")
    prompts = [parse_ids(t) for t in (args.prompt or [])]
    if args.prompt_file:
        prompts += [list(map(int, q)) for q in json.loads(args.prompt_file.read_text())]
    if not prompts:
        p.error("give --prompt or --prompt-file")
    import torch
    if not torch.cuda.is_available():
        p.error("a CUDA device is required: this library has no CPU implementation")

    from .engine.engine import Engine
    t0 = time.perf_counter()
    eng = Engine(args.model, dtype=args.dtype)
    load_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    outs = eng.generate(prompts, args.max_tokens, args.temperature, args.top_k, args.top_p,
                        use_graph=not args.no_graph, seed=args.seed)
    gen_s = time.perf_counter() - t0
    n = sum(len(o) for o in outs)
    print(f"\n[engine] loaded in {load_s:.1f}s; generated {n} tokens in {gen_s:.2f}s ({n / max(gen_s, 1e-9):.1f} tok/s)")
    print("=" * 60)
    for prompt, out in zip(prompts, outs):
        print(json.dumps({"prompt": prompt, "output": out}), flush=True)


if __name__ == "__main__":
    main()
