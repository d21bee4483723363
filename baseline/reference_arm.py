"""The reference arm of bench.py: Labeeb2339/pico-engine itself, unmodified, from ``baseline/_ref``.

pico-engine loads GGUF files only, so a GGUF file of the Qwen2.5-0.5B shape is written first
(float16 tensors drawn at random with the benchmark's distributions, a byte-level vocabulary
of the right size, no merges, no eos token): that is input data, not a change to the engine.
The prompt is text whose every character becomes one token.  pico-engine runs one sequence at
a time, so "batch 8" is eight requests one after another.  Timing follows its own benchmark
(src/pico_engine/benchmark.py:18-44: cache, decode graph, one prefill, greedy decode loop
through ``_decode_step``) with one loaded engine for all requests, because that function
loads the file anew on every call.

Prints one JSON line (``"impl": "reference"``), or the ``unavailable`` line with the reason.
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

SHAPE = dict(layers=24, hidden=896, heads=14, kv_heads=2, head_dim=64, intermediate=4864, vocab=151936,
             rope_theta=1000000.0, eps=1e-6)
BATCH, CONTEXT = 8, 4096


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


# ---------------------------------------------------------------------------- a GGUF file of random weights

def _s(text: str) -> bytes:
    b = text.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, vtype: int, payload: bytes) -> bytes:
    return _s(key) + struct.pack("<I", vtype) + payload


def write_gguf(path: str, layers: int, seed: int = 2) -> None:
    import numpy as np
    sys.path.insert(0, REF)
    from pico_engine.tokenizer import _BYTE_ENCODER
    H, I, V = SHAPE["hidden"], SHAPE["intermediate"], SHAPE["vocab"]
    nq, nkv = SHAPE["heads"] * SHAPE["head_dim"], SHAPE["kv_heads"] * SHAPE["head_dim"]
    U32, F32, STR, ARR = 4, 6, 8, 9
    tokens = [_BYTE_ENCODER[b] for b in range(256)] + [f"§t{i}" for i in range(V - 256)]
    meta = [
        _kv("general.architecture", STR, _s("qwen2")), _kv("general.alignment", U32, struct.pack("<I", 32)),
        _kv("qwen2.block_count", U32, struct.pack("<I", layers)), _kv("qwen2.embedding_length", U32, struct.pack("<I", H)),
        _kv("qwen2.attention.head_count", U32, struct.pack("<I", SHAPE["heads"])),
        _kv("qwen2.attention.head_count_kv", U32, struct.pack("<I", SHAPE["kv_heads"])),
        _kv("qwen2.attention.layer_norm_rms_epsilon", F32, struct.pack("<f", SHAPE["eps"])),
        _kv("qwen2.rope.freq_base", F32, struct.pack("<f", SHAPE["rope_theta"])),
        _kv("qwen2.feed_forward_length", U32, struct.pack("<I", I)),
        _kv("qwen2.context_length", U32, struct.pack("<I", CONTEXT + 64)),
        _kv("tokenizer.ggml.model", STR, _s("gpt2")),
        _kv("tokenizer.ggml.tokens", ARR, struct.pack("<IQ", STR, len(tokens)) + b"".join(_s(t) for t in tokens)),
        _kv("tokenizer.ggml.merges", ARR, struct.pack("<IQ", STR, 0)),
    ]
    # (name, shape as [rows, cols] or [n], float32?)
    tensors = [("token_embd.weight", (V, H), False), ("output_norm.weight", (H,), True), ("output.weight", (V, H), False)]
    for i in range(layers):
        p = f"blk.{i}."
        tensors += [(p + "attn_norm.weight", (H,), True), (p + "ffn_norm.weight", (H,), True),
                    (p + "attn_q.weight", (nq, H), False), (p + "attn_q.bias", (nq,), True),
                    (p + "attn_k.weight", (nkv, H), False), (p + "attn_k.bias", (nkv,), True),
                    (p + "attn_v.weight", (nkv, H), False), (p + "attn_v.bias", (nkv,), True),
                    (p + "attn_output.weight", (H, nq), False), (p + "ffn_gate.weight", (I, H), False),
                    (p + "ffn_up.weight", (I, H), False), (p + "ffn_down.weight", (H, I), False)]
    infos, offset = [], 0
    for name, shape, f32 in tensors:
        n = 1
        for d in shape:
            n *= d
        dims = tuple(reversed(shape))                       # GGUF lists the fastest dimension first
        infos.append(_s(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims) +
                     struct.pack("<IQ", 0 if f32 else 1, offset))
        offset += (n * (4 if f32 else 2) + 31) // 32 * 32
    rng = np.random.default_rng(seed)
    with open(path, "wb") as f:
        f.write(struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(meta)))
        for m in meta:
            f.write(m)
        for info in infos:
            f.write(info)
        f.write(b"\0" * (-f.tell() % 32))
        embedding = None
        for name, shape, f32 in tensors:
            if name == "output.weight":                      # the tied head: the embedding table again
                arr = embedding
            elif name.endswith("norm.weight"):
                arr = (1.0 + 0.02 * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
            else:
                arr = (0.02 * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32 if f32 else np.float16)
            if name == "token_embd.weight":
                embedding = arr
            raw = arr.tobytes()
            f.write(raw)
            f.write(b"\0" * (-len(raw) % 32))


# ---------------------------------------------------------------------------- the measurement

def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=SHAPE["layers"])
    ap.add_argument("--requests", type=int, default=BATCH)
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(REF, "pico_engine")):
        return unavailable("baseline/_ref holds no install of pico-engine (pip install --no-index --no-deps --target baseline/_ref)")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        sys.path.insert(0, REF)
        from pico_engine.engine import Engine                # the unmodified reference
    except Exception as e:                                   # noqa: BLE001
        return unavailable(f"pico-engine does not import here: {type(e).__name__}: {e}")

    warmup = max(args.warmup, 3)
    prompt_len = CONTEXT - args.steps - warmup
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "random-qwen2.5-0.5b-f16.gguf")
        try:
            write_gguf(path, args.layers)
            eng = Engine(path)
        except Exception as e:                               # noqa: BLE001
            return unavailable(f"pico-engine could not load the generated GGUF: {type(e).__name__}: {e}")
    try:
        letters = "abcdefghijklmnopqrstuvwxyz"
        decode_s, decoded, prefill_s = 0.0, 0, 0.0
        for r in range(args.requests):
            prompt = "".join(letters[(r * 7 + i * i) % 26] for i in range(prompt_len))   # one token a character
            ids = eng.tok.encode(prompt)
            assert len(ids) == prompt_len, (len(ids), prompt_len)
            cache = eng._empty_cache(len(ids) + warmup + args.steps)      # src/pico_engine/benchmark.py:21-23
            graph = eng._build_decode_graph(cache)
            tokens = torch.tensor(ids, device=eng.device)
            positions = torch.arange(len(ids), device=eng.device)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            logits = eng.model.forward(tokens, positions, cache)          # benchmark.py:28-31
            torch.cuda.synchronize()
            prefill_s += time.perf_counter() - t0
            generated = []
            for i in range(warmup + args.steps):                          # benchmark.py:33-43, greedy
                if i == warmup:
                    torch.cuda.synchronize()
                    t0 = time.perf_counter()
                nxt = int(logits.argmax())
                pos = len(ids) + len(generated)
                generated.append(nxt)
                logits = eng._decode_step(nxt, pos, cache, graph)
            torch.cuda.synchronize()
            decode_s += time.perf_counter() - t0
            decoded += args.steps
    except Exception as e:                                   # noqa: BLE001
        return unavailable(f"pico-engine failed while generating: {type(e).__name__}: {e}")

    value = decoded / decode_s
    print(json.dumps({
        "impl": "reference", "metric": "decode tokens/s, batch 8, context 4096 (Qwen2.5-0.5B shape)", "value": value,
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": 1000.0 * decode_s / decoded * args.requests, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32 decode, fp16 prefill (the reference's own precisions), f16 GGUF weights",
        "data": "synthetic",
        "config": {"model": "Qwen2.5-0.5B shape, random weights", "global_batch": args.requests, "seq_len": CONTEXT,
                   "parallelism": "none", "layers": args.layers, "layers_of_configuration": SHAPE["layers"],
                   "batching": "one request after another: pico-engine runs a single sequence",
                   "timing": "host clock around its own decode loop with CUDA graph, as in its benchmark.py",
                   "prefill_tokens_per_s": args.requests * prompt_len / prefill_s},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 16, "d2h_bytes_per_step": 8}}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
