"""Weights by tensor name: checking a checkpoint against what the model's parts expect,
converting dtypes, and handing each part its tensors.

pico-engine dequantizes every tensor to float32 and lets a missing name surface as a
``KeyError`` deep in the model (src/pico_engine/engine.py:80-98, model.py:86); here the
whole comparison is made first and reported in one error.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Callable, Dict, Tuple

import torch

from .safetensors_io import Checkpoint


class WeightError(ValueError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and ``wrong_shape``
    hold the details that the message lists."""

    def __init__(self, missing, unexpected, wrong_shape, where: str):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"weights in {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: stored {list(have)}, model needs {list(want)}" for n, have, want in self.wrong_shape))
        super().__init__("\n".join(lines))


class UnusedWeightsWarning(UserWarning):
    """The checkpoint holds tensors that the model does not use; they are named and left unread."""


@dataclass(frozen=True)
class ParamSpec:
    """What a part expects of one tensor.  ``init`` names the distribution of the
    random-weights mode: "normal" is N(0, 0.02), "one_plus_normal" is 1 + N(0, 0.02)."""
    shape: Tuple[int, ...]
    init: str = "normal"


def check(expected: Dict[str, ParamSpec], stored: Dict[str, Tuple[int, ...]], ignorable=(), where="the checkpoint"):
    """A checkpoint that lacks a tensor or holds one in another shape is refused with one
    :class:`WeightError` that names every missing, unexpected and mis-shaped tensor.  A checkpoint that
    is complete but carries tensors nobody asks for (older conversions store ``rotary_emb.inv_freq``;
    pico-engine looks tensors up by name and never notices extras, src/pico_engine/model.py:86-97) loads
    with one :class:`UnusedWeightsWarning` that lists them."""
    missing = sorted(n for n in expected if n not in stored)
    unexpected = sorted(n for n in stored if n not in expected and n not in ignorable)
    wrong = sorted((n, tuple(stored[n]), tuple(expected[n].shape)) for n in expected
                   if n in stored and tuple(stored[n]) != tuple(expected[n].shape))
    if missing or wrong:
        raise WeightError(missing, unexpected, wrong, where)
    if unexpected:
        warnings.warn(f"weights in {where}: {len(unexpected)} tensor(s) are not used by the model and are left "
                      f"unread: " + ", ".join(unexpected), UnusedWeightsWarning, stacklevel=3)


def convert(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The dtype a stored tensor is kept in.

    float32 engine: every floating tensor becomes float32.  bfloat16 engine: 16-bit floats are
    kept as bfloat16, a tensor stored in 32 bits (or 64) stays float32.  Integer tables
    become int32.
    """
    if t.dtype == torch.bool:
        raise ValueError("boolean tensors are not weights")
    if not t.dtype.is_floating_point:
        return t.to(torch.int32)
    if dtype == torch.float32:
        return t.to(torch.float32)
    if dtype == torch.bfloat16:
        return t.to(torch.bfloat16) if t.element_size() <= 2 else t.to(torch.float32)
    raise ValueError(f"engine dtype must be float32 or bfloat16, not {dtype}")


def load_into(model, source: Callable[[str], torch.Tensor], stored_shapes: Dict[str, Tuple[int, ...]],
              where: str) -> None:
    """Check ``stored_shapes`` against the model, then let the model take its tensors from
    ``source(name)``, converted and moved to the model's device."""
    check(model.expected_tensors(), stored_shapes, model.plan.ignorable_tensors, where)
    dtype, device = model.dtype, model.device

    def get(name: str) -> torch.Tensor:
        return convert(source(name), dtype).to(device).contiguous()
    model.take_tensors(get)


def load_folder(model, folder: str) -> None:
    ckpt = Checkpoint(folder)
    load_into(model, ckpt.read, {n: e.shape for n, e in ckpt.entries.items()}, repr(folder))
