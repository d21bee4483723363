"""Shared fixtures: the two tiny configurations, model folders in temporary places, and the
comparison rules.  Tests marked ``gpu`` need a CUDA device; everything else runs on the CPU."""
from __future__ import annotations

import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 160, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 128, "tie_word_embeddings": True, "use_sliding_window": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "intermediate_size": 352, "vocab_size": 512, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "max_position_embeddings": 256, "tie_word_embeddings": False, "use_sliding_window": True,
    "sliding_window": 32, "max_window_layers": 1, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
# A third one at head size 64, where prompts take the tcgen05 attention kernel: a window on the upper layer that is
# no multiple of a page, a vocabulary and widths that are no powers of two.
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 64,
    "intermediate_size": 200, "vocab_size": 328, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "max_position_embeddings": 512, "tie_word_embeddings": False, "use_sliding_window": True,
    "sliding_window": 70, "max_window_layers": 1, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}


def tensor_shapes(cfg: dict) -> dict:
    """Names and shapes of a dense Qwen2 checkpoint, written out here independently of the library."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or H // nh
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not cfg.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (V, H)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shapes.update({
            p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
            p + "self_attn.q_proj.weight": (nh * hd, H), p + "self_attn.q_proj.bias": (nh * hd,),
            p + "self_attn.k_proj.weight": (nkv * hd, H), p + "self_attn.k_proj.bias": (nkv * hd,),
            p + "self_attn.v_proj.weight": (nkv * hd, H), p + "self_attn.v_proj.bias": (nkv * hd,),
            p + "self_attn.o_proj.weight": (H, nh * hd),
            p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H), p + "mlp.down_proj.weight": (H, I)})
    return shapes


def make_weights(cfg: dict, seed: int, std: float = 0.02, sharp: bool = False) -> dict:
    """Random weights, rounded to bfloat16 values (kept in float32 here).  ``sharp`` gives
    matrices the scale 1/sqrt(inputs), so that activations keep their size from layer to layer,
    attention scores spread over several units and logits over a few: weights of 0.02 would
    hide a key read from the wrong place behind a nearly uniform softmax."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm.weight"):
            t = 1.0 + torch.randn(shape, generator=g) * 0.02
        elif len(shape) == 1:
            t = torch.randn(shape, generator=g) * (0.3 if sharp else std)
        else:
            s = shape[1] ** -0.5 if sharp else std
            t = torch.randn(shape, generator=g) * s
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def write_model(folder, cfg: dict, weights: dict, store: torch.dtype = torch.bfloat16, float32_names=()) -> str:
    """A model folder written with the safetensors package, not with the library's own writer."""
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({n: (t.to(torch.float32) if n in float32_names else t.to(store)).contiguous() for n, t in weights.items()},
              os.path.join(folder, "model.safetensors"))
    return str(folder)


def close_enough(got: torch.Tensor, want: torch.Tensor, dtype: str) -> tuple[bool, str]:
    """The comparison rule of the engine tests.  The error is measured against the size of the
    logits: float32 runs must agree to 2e-5 of it, bfloat16 runs to 4e-2."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    scale = max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    tol = {"float32": 2e-5, "bfloat16": 4e-2}[dtype] * scale
    if os.environ.get("PICO_TEST_STATS"):                  # a developer's record of how close runs come
        with open(os.environ["PICO_TEST_STATS"], "a") as f:
            f.write(f"{dtype} {err / scale:.3e} {scale:.3f}\n")
    return err <= tol, f"max error {err:.3e} (allowed {tol:.3e}, logits up to {scale:.3f})"


@pytest.fixture(params=["A", "B"])
def tiny(request):
    return request.param, dict(TINY[request.param])
