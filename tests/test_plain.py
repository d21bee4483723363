"""The plain implementation against pico-engine's own forward (committed outputs of
tests/golden/make_golden.py) and against small cases worked out by hand (CPU)."""
import math
import os

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from conftest import TINY_A, TINY_B, make_weights

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_logits.npz")


@pytest.mark.parametrize("name,cfg,seed", [("A", TINY_A, 0), ("B", {**TINY_B, "use_sliding_window": False}, 1)])
def test_equals_pico_engines_own_forward(name, cfg, seed):
    gold = np.load(GOLDEN)
    tokens = gold[f"{name}_tokens"].tolist()
    w = make_weights(cfg, seed, sharp=True)
    logits = plain.forward(cfg, w, tokens)
    scale = float(logits.abs().max())
    assert scale > 1.0                                     # the weights are sharp enough to tell positions apart
    checked = 0
    for key in gold.files:
        kind, _, num = key[len(name) + 1:].partition("_")
        if not key.startswith(name + "_") or kind not in ("prefill", "decode"):
            continue
        row = int(num) - 1 if kind == "prefill" else int(num)
        err = float((logits[row] - torch.from_numpy(gold[key])).abs().max())
        assert err < 2e-5 * scale, (key, err)
        checked += 1
    assert checked == 44


def test_window_rule_by_hand():
    m = plain.visible(6, 3)
    assert m.int().tolist() == [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0],
                                [0, 1, 1, 1, 0, 0], [0, 0, 1, 1, 1, 0], [0, 0, 0, 1, 1, 1]]
    assert plain.visible(4, None).int().tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [1, 1, 1, 1]]
    assert [plain.layer_window(TINY_B, i) for i in range(3)] == [None, 32, 32]
    assert plain.layer_window(TINY_A, 1) is None


def test_windowed_attention_against_loops_written_out():
    """plain.attention with a window against the definition spelled out token by token (query p sees key j iff
    0 <= p - j < window; query head h reads key/value head h // group): no mask helper, no batched product."""
    L, nh, nkv, hd, window = 11, 4, 2, 6, 4
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(L, n, hd, generator=g, dtype=torch.float64) for n in (nh, nkv, nkv))
    want = torch.zeros(L, nh, hd, dtype=torch.float64)
    for p in range(L):
        for h in range(nh):
            kvh = h // (nh // nkv)
            keys = [j for j in range(L) if 0 <= p - j < window]
            assert keys == list(range(max(0, p - window + 1), p + 1))
            scores = [sum(float(q[p, h, d]) * float(k[j, kvh, d]) for d in range(hd)) / math.sqrt(hd) for j in keys]
            top = max(scores)
            e = [math.exp(x - top) for x in scores]
            for j, wgt in zip(keys, e):
                want[p, h] += wgt / sum(e) * v[j, kvh]
    got = plain.attention(q.float(), k.float(), v.float(), window).view(L, nh, hd)
    assert torch.allclose(got.double(), want, atol=1e-5)
    assert not torch.allclose(plain.attention(q.float(), k.float(), v.float(), None).view(L, nh, hd).double(), want, atol=1e-2)


def test_window_changes_only_positions_beyond_it():
    w = make_weights(TINY_B, 1, sharp=True)
    ids = torch.randint(0, 512, (50,), generator=torch.Generator().manual_seed(3)).tolist()
    with_w = plain.forward(TINY_B, w, ids)
    without = plain.forward({**TINY_B, "use_sliding_window": False}, w, ids)
    assert torch.allclose(with_w[:32], without[:32], atol=1e-6)
    assert float((with_w[40:] - without[40:]).abs().max()) > 1e-3


def test_rope_and_norm_by_hand():
    cos, sin = plain.rope_angles(torch.tensor([0, 3]), 4, 100.0)
    assert torch.allclose(cos[0], torch.ones(2)) and torch.allclose(sin[0], torch.zeros(2))
    assert math.isclose(float(cos[1, 1]), math.cos(3 * 100.0 ** -0.5), rel_tol=1e-6)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]]).repeat(2, 1, 1)
    y = plain.apply_rope(x, cos, sin)
    a = 3.0
    assert torch.allclose(y[0], x[0])
    assert math.isclose(float(y[1, 0, 0]), 1 * math.cos(a) - 3 * math.sin(a), rel_tol=1e-5)
    assert math.isclose(float(y[1, 0, 2]), 1 * math.sin(a) + 3 * math.cos(a), rel_tol=1e-5)
    n = plain.rms_norm(torch.tensor([[3.0, 4.0]]), torch.tensor([2.0, 0.5]), 0.0)
    assert torch.allclose(n, torch.tensor([[3.0 * 2, 4.0 * 0.5]]) / math.sqrt(12.5))


def test_attention_groups_and_far_key():
    # one key far back gets a large score: the output must be its value, for every head of its group
    L, nh, nkv, hd = 40, 4, 2, 8
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(L, nh, hd, generator=g), torch.randn(L, nkv, hd, generator=g), torch.randn(L, nkv, hd, generator=g)
    k[3, 1] = 20.0 * q[39, 2] / q[39, 2].norm()
    out = plain.attention(q, k, v, None).view(L, nh, hd)
    assert torch.allclose(out[39, 2], v[3, 1], atol=1e-3) and not torch.allclose(out[39, 1], v[3, 0], atol=1e-1)
    assert torch.allclose(out[0, 3], v[0, 1], atol=1e-6)               # the first token sees itself only
    out_w = plain.attention(q, k, v, 8).view(L, nh, hd)
    assert not torch.allclose(out_w[39, 2], v[3, 1], atol=1e-1)         # outside a window of 8


def test_sampler_rules():
    logits = torch.tensor([1.0, 3.0, 3.0, 0.0, 2.0])
    assert plain.sample(logits, 0.0, 0, 1.0, 0.5) == 1                      # greedy: first maximum
    assert plain.sample(logits, 1.0, 1, 1.0, 0.99) in (1, 2)                # top-k keeps ties
    assert plain.sample(logits, 1.0, 2, 1.0, 0.99) == 2
    p = torch.softmax(logits, -1)
    top_p = float(p[1] + p[2]) - 1e-4                                       # the crossing token stays
    assert plain.sample(logits, 1.0, 0, top_p, 0.9999) == 2
    assert plain.sample(logits, 1.0, 0, float(p[1] + p[2] + p[4]) - 1e-4, 0.9999) == 4
    assert plain.sample(logits, 1.0, 0, 1e-6, 0.9999) == 1                  # the first token always stays
    # inverse CDF in index order
    cdf = torch.cumsum(p, 0)
    assert plain.sample(logits, 1.0, 0, 1.0, float(cdf[0]) * 0.5) == 0
    assert plain.sample(logits, 1.0, 0, 1.0, float(cdf[2]) + 1e-4) == 3
    us = [plain.uniform_for(1, r, s) for r in range(3) for s in range(50)]
    assert all(0 <= u < 1 for u in us) and len(set(us)) == len(us) and abs(sum(us) / len(us) - 0.5) < 0.1
    assert plain.uniform_for(1, 0, 0) != plain.uniform_for(2, 0, 0)


def test_generate_stops_before_the_stop_token():
    w = make_weights(TINY_A, 0, sharp=True)
    full = plain.generate(TINY_A, w, [1, 2, 3], 6)
    assert len(full) == 6
    cut = plain.generate(TINY_A, w, [1, 2, 3], 6, stop=(full[2],))
    assert cut == full[:full.index(full[2])]
    assert plain.param_count(TINY_A) == sum(t.numel() for t in w.values())
