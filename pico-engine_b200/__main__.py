"""Command line: load a model folder and generate token ids.

Options are pico-engine's (src/pico_engine/__main__.py:23-39) with their names, defaults and
meanings: ``--prompt``, ``--max-tokens 64``, ``--temperature 0.7`` (0 is greedy), ``--top-p 0.9``,
``--top-k 0``, ``--no-graph``.  There is no tokenizer in this library, so ``--prompt`` takes token
ids ("5,17,3"; repeat the option for a batch) and the output is token ids; ``--seed``,
``--dtype`` and ``--stop-token-ids`` are additions.  Without a model folder, ``--random-config NAME``
draws the weights of a named shape from ``--seed`` and ``--random-prompt LEN[,LEN...]`` draws
prompts, so that random weights become tokens in one line.  ``--n-gpu-layers`` (offload of
another architecture) is not taken.
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


def random_prompts(lengths, vocab: int, seed: int) -> list[list[int]]:
    """Prompts of the given lengths, token ids uniform in [0, vocab), the same for the same seed."""
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def main(argv=None) -> None:
    p = argparse.ArgumentParser(
        prog="pico_engine", description="Generate token ids with a dense Qwen2 model folder on one B200",
        epilog='example: python -m pico_engine models/tiny --prompt "5,17,3" --max-tokens 11 --temperature 0')
    p.add_argument("model", type=Path, nargs="?", help="folder with config.json and model.safetensors")
    p.add_argument("--random-config", metavar="NAME", help="instead of a folder: random weights (from --seed) of a named "
                   "shape: tiny-a, tiny-b, qwen2.5-0.5b, qwen2.5-7b, qwen2.5-14b")
    p.add_argument("--layers", type=int, help="with --random-config: fewer layers than the shape has")
    p.add_argument("--prompt", action="append", help='token ids of a prompt, e.g. "5,17,3"; repeat for a batch')
    p.add_argument("--prompt-file", type=Path, help="JSON file holding a list of prompts (lists of token ids)")
    p.add_argument("--random-prompt", metavar="LEN[,LEN...]", help="prompts of these lengths with token ids drawn from --seed")
    p.add_argument("--stop-token-ids", metavar="ID[,ID...]", help="tokens that end a sequence (and are not returned); "
                   "default: the configuration's eos ids; \"\" for none")
    p.add_argument("--max-tokens", type=int, default=64)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--seed", type=int, default=0, help="names the stream of random draws")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--no-graph", action="store_true", help="disable CUDA-graph decode and launch every kernel")
    args = p.parse_args(argv)

    if (args.model is None) == (args.random_config is None):
        p.error("give a model folder or --random-config NAME")
    config = None
    if args.random_config:
        from .config import config_from_dict
        from .config.shapes import shape
        try:
            d = shape(args.random_config)
        except KeyError as e:
            p.error(str(e.args[0]))
        if args.layers is not None:
            if args.layers < 1:
                p.error("--layers must be at least 1")
            d["num_hidden_layers"] = args.layers
            d["max_window_layers"] = min(d.get("max_window_layers", args.layers), args.layers)
        config = config_from_dict(d)
    elif args.layers is not None:
        p.error("--layers goes with --random-config")
    elif not (args.model / "config.json").is_file():
        p.error(f"model folder has no config.json: {args.model}")
    if args.max_tokens < 0:
        p.error("--max-tokens must be non-negative")
    prompts = [parse_ids(t) for t in (args.prompt or [])]
    if args.prompt_file:
        prompts += [list(map(int, q)) for q in json.loads(args.prompt_file.read_text())]
    if args.random_prompt:
        lengths = parse_ids(args.random_prompt)
        if not lengths or min(lengths) < 1:
            p.error("--random-prompt takes positive lengths")
        if config is None:
            from .config.registry import read_config
            vocab = read_config(str(args.model)).plan().vocab_size
        else:
            vocab = config.plan().vocab_size
        prompts += random_prompts(lengths, vocab, args.seed)
    if not prompts:
        p.error("give --prompt, --prompt-file or --random-prompt")
    stop = None if args.stop_token_ids is None else parse_ids(args.stop_token_ids)
    import torch
    if not torch.cuda.is_available():
        p.error("a CUDA device is required: this library has no CPU implementation")

    from .engine.engine import Engine
    t0 = time.perf_counter()
    if config is not None:
        eng = Engine.from_config(config, seed=args.seed, dtype=args.dtype)
    else:
        eng = Engine(args.model, dtype=args.dtype)
    load_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    outs = eng.generate(prompts, args.max_tokens, args.temperature, args.top_k, args.top_p,
                        use_graph=not args.no_graph, seed=args.seed, stop_token_ids=stop)
    gen_s = time.perf_counter() - t0
    n = sum(len(o) for o in outs)
    print(f"\n[engine] loaded in {load_s:.1f}s; generated {n} tokens in {gen_s:.2f}s ({n / max(gen_s, 1e-9):.1f} tok/s)")
    print("=" * 60)
    for prompt, out in zip(prompts, outs):
        print(json.dumps({"prompt": prompt, "output": out}), flush=True)


if __name__ == "__main__":
    main()
