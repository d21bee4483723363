"""The random-weights mode: tensors drawn from a configuration and a seed, and the writer of
a model folder (config.json, model.safetensors) that the ordinary loader then reads.

pico-engine has no such mode (it only loads published GGUF files); the distributions are
linear weights, embeddings and biases N(0, 0.02), norm weights 1 + N(0, 0.02).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Tuple

import torch

from .loader import ParamSpec
from .safetensors_io import write_safetensors

STD = 0.02


def _seed_of(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec: ParamSpec, seed: int, store_dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """One tensor; its values depend on (seed, name) only, not on the order of creation."""
    g = torch.Generator(device=device)
    g.manual_seed(_seed_of(seed, name))
    t = torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32) * STD
    if spec.init == "one_plus_normal":
        t = t + 1.0
    elif spec.init != "normal":
        raise ValueError(f"tensor {name!r}: unknown init {spec.init!r}")
    return t.to(store_dtype)


def random_tensors(expected: Dict[str, ParamSpec], seed: int, store_dtype: torch.dtype = torch.bfloat16,
                   device="cpu", float32_names=()) -> Iterator[Tuple[str, torch.Tensor]]:
    """``(name, tensor)`` for every expected tensor.  Names in ``float32_names`` are stored
    in float32 whatever ``store_dtype`` is."""
    for name, spec in expected.items():
        dt = torch.float32 if name in float32_names else store_dtype
        yield name, random_tensor(name, spec, seed, dt, device)


def write_random_model(config, seed: int, folder: str, store_dtype: torch.dtype = torch.bfloat16,
                       float32_names=(), device="cpu") -> None:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` for ``config``."""
    from ..config.registry import architecture
    arch = architecture(config.ARCHITECTURE)
    model = arch.build_model(config, store_dtype, "meta")
    os.makedirs(folder, exist_ok=True)
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[store_dtype]
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(model.expected_tensors(), seed, store_dtype, device, float32_names),
                      metadata={"format": "pt", "seed": seed})
