"""Plain, slow implementation of the dense Qwen2 decoder, used as the oracle by the tests.

Whole sequences, no cache, float32 (or float64) torch on whatever device the inputs
live on, one function per part.  It shares no code with the product package: it reads
``config.json`` keys from a plain ``dict`` and weights from a plain ``dict`` keyed by the
checkpoint's tensor names.

Every function cites the lines of Labeeb2339/pico-engine it restates
(paths relative to that project).  The sliding window and tied embeddings do not exist
in that project's dense path; their rules are stated here and are the authority for the
tests (``tests/golden/`` holds the comparison of the rest with the project's own code).
"""
from __future__ import annotations

import torch


# ----------------------------------------------------------------------------- parts

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w``, the weight multiplying directly.

    src/pico_engine/kernels.py:19-23 (Triton), src/pico_engine/model.py:291-294 (CPU twin).
    """
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin of ``p * theta^(-2j/head_dim)``, ``j = 0..head_dim/2-1``; shape (L, head_dim/2).

    src/pico_engine/model.py:75-79.
    """
    j = torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device)
    inv_freq = 1.0 / (theta ** (j / head_dim))
    angles = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return angles.cos(), angles.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing: element j with j + head_dim/2.  x: (L, heads, head_dim).

    src/pico_engine/kernels.py:42-47, src/pico_engine/model.py:296-300.
    """
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)


def visible(n: int, window: int | None, device=None) -> torch.Tensor:
    """mask[p, j] = query p may see key j.

    Causal: ``j <= p`` (src/pico_engine/model.py:206; decode keeps keys ``< pos + 1``,
    src/pico_engine/kernels.py:111,117).  With a window (not in that project):
    additionally ``p - j < window``.
    """
    p = torch.arange(n, device=device)[:, None]
    j = torch.arange(n, device=device)[None, :]
    mask = j <= p
    if window is not None:
        mask = mask & (p - j < window)
    return mask


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None) -> torch.Tensor:
    """Grouped-query softmax attention of one sequence.  q: (L, nh, hd); k, v: (L, nkv, hd).

    Scores ``q.k * hd^-0.5`` (src/pico_engine/kernels.py:116,149-150; model.py:342), query
    head h reads kv head ``h // (nh/nkv)`` (kernels.py:99), softmax over visible keys
    (kernels.py:118-125; model.py:343-344).  Returns (L, nh*hd), heads concatenated
    (model.py:213).
    """
    L, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    mask = visible(L, window, q.device)
    out = torch.empty(L, nh, hd, dtype=q.dtype, device=q.device)
    for h in range(nh):
        kh = k[:, h // group, :]
        vh = v[:, h // group, :]
        scores = (q[:, h, :] @ kh.T) * (hd ** -0.5)
        scores = scores.masked_fill(~mask, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h, :] = probs @ vh
    return out.reshape(L, nh * hd)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``gate * sigmoid(gate) * up``.  src/pico_engine/kernels.py:71-73."""
    return gate * torch.sigmoid(gate) * up


# ----------------------------------------------------------------------------- config

def head_dim_of(cfg: dict) -> int:
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


def layer_window(cfg: dict, layer: int) -> int | None:
    """The window of a layer: layers ``>= max_window_layers`` when ``use_sliding_window``."""
    if not cfg.get("use_sliding_window", False):
        return None
    if layer >= int(cfg.get("max_window_layers", cfg["num_hidden_layers"])):
        return int(cfg["sliding_window"])
    return None


# ----------------------------------------------------------------------------- the model

def decoder_layer(cfg: dict, w: dict, i: int, x: torch.Tensor, cos, sin) -> torch.Tensor:
    """One pre-norm block.  src/pico_engine/model.py:167-237."""
    nh = int(cfg["num_attention_heads"])
    nkv = int(cfg["num_key_value_heads"])
    hd = head_dim_of(cfg)
    eps = float(cfg["rms_norm_eps"])
    p = f"model.layers.{i}."
    L = x.shape[0]

    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)                      # model.py:175
    q = h @ w[p + "self_attn.q_proj.weight"].T + w[p + "self_attn.q_proj.bias"]  # model.py:177 (fused there)
    k = h @ w[p + "self_attn.k_proj.weight"].T + w[p + "self_attn.k_proj.bias"]
    v = h @ w[p + "self_attn.v_proj.weight"].T + w[p + "self_attn.v_proj.bias"]
    q = apply_rope(q.view(L, nh, hd), cos, sin)                                # model.py:179-182
    k = apply_rope(k.view(L, nkv, hd), cos, sin)
    v = v.view(L, nkv, hd)                                                     # model.py:183
    a = attention(q, k, v, layer_window(cfg, i))                               # model.py:201-211
    x = x + a @ w[p + "self_attn.o_proj.weight"].T                             # model.py:213

    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)             # model.py:222
    g = h @ w[p + "mlp.gate_proj.weight"].T                                    # model.py:223
    u = h @ w[p + "mlp.up_proj.weight"].T
    x = x + swiglu(g, u) @ w[p + "mlp.down_proj.weight"].T                     # model.py:224,235
    return x


def forward(cfg: dict, weights: dict, token_ids, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Logits at every position of one sequence, (L, vocab).  src/pico_engine/model.py:146-165.

    The project returns the last row only (model.py:164); all rows are the same formula.
    A tied head reuses the embedding table (the project's dense path has no tied head).
    """
    w = {k: v.to(dtype) for k, v in weights.items()}
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=next(iter(w.values())).device)
    L = ids.shape[0]
    x = w["model.embed_tokens.weight"][ids]                                    # model.py:152
    cos, sin = rope_angles(torch.arange(L, device=ids.device), head_dim_of(cfg), float(cfg["rope_theta"]))
    for i in range(int(cfg["num_hidden_layers"])):                             # model.py:157-158
        x = decoder_layer(cfg, w, i, x, cos, sin)
    x = rms_norm(x, w["model.norm.weight"], float(cfg["rms_norm_eps"]))        # model.py:159
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ head.T                                                          # model.py:164


# ----------------------------------------------------------------------------- sampling

def uniform_for(seed: int, request: int, step: int) -> float:
    """The uniform in [0, 1) that a draw uses: a 64-bit mix of (seed, request, step).

    The project draws from torch's global generator (src/pico_engine/sampler.py:25); a
    seeded library has to name its stream, and this is it (splitmix64 finaliser).
    """
    m = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """src/pico_engine/sampler.py:8-27, with the multinomial draw replaced by the
    inverse CDF in index order at the given uniform ``u``."""
    logits = logits.to(torch.float32).clone()
    if temperature <= 0:                                                       # sampler.py:26-27
        return int(torch.argmax(logits))
    logits = logits / temperature                                              # sampler.py:13
    if top_k > 0:                                                              # sampler.py:14-16
        kth = torch.topk(logits, min(top_k, logits.numel())).values[-1]
        logits[logits < kth] = float("-inf")
    if top_p < 1.0:                                                            # sampler.py:17-23
        sorted_logits, sorted_idx = torch.sort(logits, descending=True, stable=True)
        cum = torch.cumsum(torch.softmax(sorted_logits, dim=-1), dim=-1)
        remove = cum > top_p
        remove[1:] = remove[:-1].clone()
        remove[0] = False
        logits[sorted_idx[remove]] = float("-inf")
    probs = torch.softmax(logits, dim=-1)                                      # sampler.py:24
    cdf = torch.cumsum(probs.to(torch.float64), dim=-1)
    idx = int(torch.searchsorted(cdf, torch.tensor(u * float(cdf[-1]), dtype=torch.float64), right=True))
    return min(idx, logits.numel() - 1)


def generate(cfg: dict, weights: dict, prompt, max_tokens: int, temperature: float = 0.0,
             top_k: int = 0, top_p: float = 1.0, seed: int = 0, request: int = 0,
             stop: tuple[int, ...] = (), dtype: torch.dtype = torch.float32) -> list[int]:
    """The generation loop of src/pico_engine/engine.py:328-337 for one request, recomputing
    the whole sequence each step: sample, stop before appending a stop token, append."""
    ids = list(prompt)
    out: list[int] = []
    for step in range(max_tokens):
        logits = forward(cfg, weights, ids + out, dtype)[-1]
        nxt = sample(logits, temperature, top_k, top_p, uniform_for(seed, request, step))
        if nxt in stop:                                                        # engine.py:331-332
            break
        out.append(nxt)                                                        # engine.py:334
    return out


def param_count(cfg: dict) -> int:
    H, I, V = int(cfg["hidden_size"]), int(cfg["intermediate_size"]), int(cfg["vocab_size"])
    nh, nkv, hd = int(cfg["num_attention_heads"]), int(cfg["num_key_value_heads"]), head_dim_of(cfg)
    per_layer = (nh + 2 * nkv) * hd * (H + 1) + H * nh * hd + 3 * H * I + 2 * H
    total = int(cfg["num_hidden_layers"]) * per_layer + V * H + H
    if not cfg.get("tie_word_embeddings", False):
        total += V * H
    return total

