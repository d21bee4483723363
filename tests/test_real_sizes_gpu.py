"""The engine at the layer sizes of real Qwen2.5 models (fewer layers, random weights) against the
plain implementation, which here runs on the GPU in float32 (its matrix products are the
library's float32 ones: no reduced-precision mode is enabled).  Every way of cutting: whole
prompts, the last tokens one by one, a batch of unequal lengths whose shorter requests end earlier."""
import gc

import pytest
import torch

import replay

pytestmark = pytest.mark.gpu

SHAPES = [("qwen2.5-0.5b", 2, 3), ("qwen2.5-7b", 1, 4), ("qwen2.5-14b", 1, 5)]      # (shape, layers kept, seed)
LENGTHS = [70, 33, 5, 129]


def _setup(name, layers, seed):
    from pico_engine.config import config_from_dict
    from pico_engine.config.registry import architecture
    from pico_engine.config.shapes import shape
    from pico_engine.weights import random_tensor
    d = shape(name)
    d["num_hidden_layers"] = layers
    cfg = config_from_dict(d)
    expected = architecture(cfg.ARCHITECTURE).build_model(cfg, torch.bfloat16, "meta").expected_tensors()
    weights = {n: random_tensor(n, spec, seed, torch.bfloat16, "cuda").float() for n, spec in expected.items()}
    g = torch.Generator().manual_seed(seed)
    reqs = {f"r{i}": torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for i, n in enumerate(LENGTHS)}
    want = replay.plain_logits(d, weights, reqs)
    del weights
    gc.collect(); torch.cuda.empty_cache()
    return cfg, reqs, want


@pytest.mark.parametrize("name,layers,seed", SHAPES, ids=[s[0] for s in SHAPES])
def test_real_layer_sizes_every_way_of_cutting(name, layers, seed):
    from pico_engine.engine.engine import Engine
    cfg, reqs, want = _setup(name, layers, seed)
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_config(cfg, seed=seed, draw_on="cuda", dtype=dtype)
        replay.compare(replay.run_in_process(eng, replay.whole(reqs)), want, dtype, f"{name} whole")
        replay.compare(replay.run_in_process(eng, replay.tail(reqs, 8)), want, dtype, f"{name} tail")
        replay.compare(replay.run_in_process(eng, replay.batched(reqs, 3, 0.4)), want, dtype, f"{name} batched")
        del eng
        gc.collect(); torch.cuda.empty_cache()


@pytest.mark.parametrize("name,layers,seed", SHAPES[:2], ids=[s[0] for s in SHAPES[:2]])
def test_real_layer_sizes_generation_with_graphs(name, layers, seed):
    """Greedy generation in bfloat16 through the entry point at head sizes 64 and 128, with the decode graphs and one
    step ahead of the host (what the benchmark times): the same tokens as without graphs, each a (near) maximum of the
    plain float32 logits for the engine's own prefix; and 24 requests at once, whose steps take the products for
    more than 16 rows."""
    import plain_qwen2 as plain
    from pico_engine.config import config_from_dict
    from pico_engine.config.registry import architecture
    from pico_engine.config.shapes import shape
    from pico_engine.engine.engine import Engine
    from pico_engine.weights import random_tensor
    d = shape(name)
    d["num_hidden_layers"] = layers
    cfg = config_from_dict(d)
    expected = architecture(cfg.ARCHITECTURE).build_model(cfg, torch.bfloat16, "meta").expected_tensors()
    weights = {n: random_tensor(n, spec, seed, torch.bfloat16, "cuda").float() for n, spec in expected.items()}
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (70, 33, 5, 129)]
    eng = Engine.from_config(cfg, seed=seed, draw_on="cuda", dtype="bfloat16")
    graphed = eng.generate(prompts, max_tokens=[10, 6, 12, 3], temperature=0.0, use_graph=True, stop_token_ids=())
    eager = eng.generate(prompts, max_tokens=[10, 6, 12, 3], temperature=0.0, use_graph=False, stop_token_ids=())
    assert graphed == eager
    many = [torch.randint(0, cfg.vocab_size, (3 + i % 5,), generator=g).tolist() for i in range(24)]
    crowd = eng.generate(many, max_tokens=[2 + i % 4 for i in range(24)], temperature=0.0, use_graph=True, stop_token_ids=())
    for p, out in list(zip(prompts, graphed)) + list(zip(many, crowd))[::5]:
        logits = plain.forward(d, weights, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[tok]) <= 4e-2 * max(1.0, float(row.abs().max())), (i, tok)
    del eng, weights
    gc.collect(); torch.cuda.empty_cache()
