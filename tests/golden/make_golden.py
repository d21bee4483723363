"""Makes ``reference_logits.npz``: logits of Labeeb2339/pico-engine's own dense forward
(src/pico_engine/model.py, class Transformer) on the CPU for tiny random models, against which
``tests/test_plain.py`` checks the plain implementation.

    python tests/golden/make_golden.py /path/to/pico-engine

The project's model code is imported unchanged under another module name.  Its four Triton
entry points cannot launch without a GPU, so they are replaced by the project's own CPU
formulas: ``Transformer._rmsnorm_cpu`` and ``_rope_cpu`` (model.py:291-300), ``g*sigmoid(g)*u``
(kernels.py:73) and the softmax attention of model.py:342-344 with key/value heads repeated
for the group as its own kernel test does (tests/test_kernels.py:80-84).  Prompts go through
its fused attention on the CPU (model.py:201-209), single tokens through the patched
``decode_attn`` (model.py:211).  It has no sliding window and no tied head: tiny-B runs with
``use_sliding_window`` off, and tiny-A's embedding table is passed as ``output.weight`` too.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from conftest import TINY_A, TINY_B, make_weights  # noqa: E402

GGUF_NAME = {
    "input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
    "self_attn.q_proj.weight": "attn_q.weight", "self_attn.q_proj.bias": "attn_q.bias",
    "self_attn.k_proj.weight": "attn_k.weight", "self_attn.k_proj.bias": "attn_k.bias",
    "self_attn.v_proj.weight": "attn_v.weight", "self_attn.v_proj.bias": "attn_v.bias",
    "self_attn.o_proj.weight": "attn_output.weight", "mlp.gate_proj.weight": "ffn_gate.weight",
    "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight"}


def load_reference(root: str):
    pkg_dir = os.path.join(root, "src", "pico_engine")
    spec = importlib.util.spec_from_file_location("ref_pico_engine", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    pkg = importlib.util.module_from_spec(spec)
    sys.modules["ref_pico_engine"] = pkg
    spec.loader.exec_module(pkg)
    model = importlib.import_module("ref_pico_engine.model")
    T = model.Transformer
    model.rmsnorm = lambda x, w, eps: T._rmsnorm_cpu(x, w, eps)
    model.rope = lambda x, cos, sin: T._rope_cpu(x, cos[:, None, :], sin[:, None, :])
    model.silu_mul = lambda gu, ffn: gu[:, :ffn] * torch.sigmoid(gu[:, :ffn]) * gu[:, ffn:]

    def decode_attn(q, k, v, S=None, stride=None, scale=None):
        n_head, hd = q.shape
        S = int(S)
        group = n_head // k.shape[0]
        kk = k[:, :S].repeat_interleave(group, dim=0)
        vv = v[:, :S].repeat_interleave(group, dim=0)
        scores = torch.einsum("hd,hsd->hs", q, kk) * (hd ** -0.5)
        return torch.einsum("hs,hsd->hd", torch.softmax(scores, dim=-1), vv)
    model.decode_attn = decode_attn
    return model


def to_gguf_names(cfg: dict, w: dict) -> dict:
    out = {"token_embd.weight": w["model.embed_tokens.weight"], "output_norm.weight": w["model.norm.weight"],
           "output.weight": w.get("lm_head.weight", w["model.embed_tokens.weight"])}
    for i in range(cfg["num_hidden_layers"]):
        for hf, gg in GGUF_NAME.items():
            out[f"blk.{i}.{gg}"] = w[f"model.layers.{i}.{hf}"]
    return out


def run(model, cfg: dict, seed: int, tokens, prefills, decode_from: int) -> dict:
    w = make_weights(cfg, seed, sharp=True)
    mc = model.ModelConfig(vocab_size=cfg["vocab_size"], n_layers=cfg["num_hidden_layers"], hidden=cfg["hidden_size"],
                           n_head=cfg["num_attention_heads"], n_kv_head=cfg["num_key_value_heads"],
                           head_dim=cfg["head_dim"], ffn_dim=cfg["intermediate_size"], rope_base=cfg["rope_theta"],
                           eps=cfg["rms_norm_eps"], context_len=cfg["max_position_embeddings"])
    tr = model.Transformer(mc, to_gguf_names(cfg, w), torch.device("cpu"))
    ids = torch.tensor(tokens)
    n = len(tokens)

    def cache():
        return [(torch.zeros(mc.n_kv_head, n, mc.head_dim), torch.zeros(mc.n_kv_head, n, mc.head_dim))
                for _ in range(mc.n_layers)]
    out = {}
    for L in prefills:                                     # whole prompts of several lengths: the last row each
        out[f"prefill_{L}"] = tr.forward(ids[:L], torch.arange(L), cache()).numpy()
    c = cache()
    tr.forward(ids[:decode_from], torch.arange(decode_from), c)
    for p in range(decode_from, n):                        # then token by token from the cache
        out[f"decode_{p}"] = tr.forward(ids[p:p + 1], torch.tensor([p]), c).numpy()
    return out


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py PATH_TO_PICO_ENGINE_CHECKOUT")
    root = sys.argv[1]
    model = load_reference(root)
    g = torch.Generator().manual_seed(1234)
    result = {}
    for name, cfg, seed in (("A", TINY_A, 0), ("B", {**TINY_B, "use_sliding_window": False}, 1)):
        tokens = torch.randint(0, cfg["vocab_size"], (45,), generator=g).tolist()
        result[f"{name}_tokens"] = np.asarray(tokens, dtype=np.int64)
        for k, v in run(model, cfg, seed, tokens, prefills=(1, 5, 13, 45), decode_from=5).items():
            result[f"{name}_{k}"] = v.astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "reference_logits.npz"), **result)
    print("wrote", len(result), "arrays")


if __name__ == "__main__":
    with torch.inference_mode():
        main()
