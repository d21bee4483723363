"""The engine against the plain implementation: every way of cutting the same requests into
steps, in float32 and in bfloat16, on both tiny configurations."""

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import replay
from conftest import TINY, close_enough, make_weights, write_model

pytestmark = pytest.mark.gpu

SEEDS = {"A": 0, "B": 1, "C": 2}


def random_requests(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{(config, dtype): (engine, cfg, weights)}; the folders live in a temporary place."""
    from pico_engine.engine.engine import Engine
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name, cfg in TINY.items():
        weights = make_weights(cfg, SEEDS[name], sharp=True)
        folder = write_model(root / name, cfg, weights)
        for dtype in ("float32", "bfloat16"):
            out[(name, dtype)] = (Engine(folder, dtype=dtype), dict(cfg), weights)
    return out


LENGTHS = {"A": [5, 9, 13, 40, 66, 100, 33, 1], "B": [1, 17, 40, 64, 65, 130, 200, 35],
           "C": [129, 3, 300, 128, 71, 257, 64, 190]}
CASES = [(n, d) for n in ("A", "B", "C") for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_requests(models, name, dtype):
    eng, cfg, w = models[(name, dtype)]
    reqs = random_requests(cfg, LENGTHS[name], 10)
    replay.compare(replay.run_in_process(eng, replay.whole(reqs)), replay.plain_logits(cfg, w, reqs), dtype, "whole")


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_tokens_one_by_one(models, name, dtype):
    eng, cfg, w = models[(name, dtype)]
    reqs = random_requests(cfg, LENGTHS[name], 11)
    replay.compare(replay.run_in_process(eng, replay.tail(reqs, 32)), replay.plain_logits(cfg, w, reqs), dtype, "tail")


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("batch_size,fraction", [(3, 0.5), (4, 0.2), (8, 0.9)])
def test_unequal_batches_one_after_another(models, name, dtype, batch_size, fraction):
    """Shorter requests end earlier; the next batch takes the slots and pages just given back
    (the cache is sized for one batch only)."""
    eng, cfg, w = models[(name, dtype)]
    reqs = random_requests(cfg, LENGTHS[name] + LENGTHS[name][::-1], 12 + batch_size)
    steps = replay.batched(reqs, batch_size, fraction)
    assert replay.max_tokens_of(steps) < sum((len(t) + 63) // 64 * 64 for t in reqs.values())
    replay.compare(replay.run_in_process(eng, steps), replay.plain_logits(cfg, w, reqs), dtype, "batched")


def many_short_requests(cfg, name, n, seed):
    """``n`` requests of 2 to 40 tokens, a few of them longer than the window where there is one."""
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(2, 41, (n,), generator=g).tolist()
    for i, extra in zip(range(3, n, 11), ({"A": 0, "B": 45, "C": 110}[name],) * n):
        lengths[i] += extra
    return random_requests(cfg, lengths, seed + 1)


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("batch_size", [24, 64])
def test_one_token_steps_of_many_rows(models, name, dtype, batch_size):
    """Batches of 24 and 64 requests: their one-token steps have 17 to 64 rows, which take other
    matrix products than the steps of a few rows; requests end one by one, so every row count from
    the batch size down is run, and the second batch reuses the first one's slots."""
    eng, cfg, w = models[(name, dtype)]
    reqs = many_short_requests(cfg, name, batch_size + 9, 30 + batch_size)
    steps = replay.batched(reqs, batch_size, 0.5)
    assert max(len(s["entries"]) for s in steps[1:]) == batch_size
    replay.compare(replay.run_in_process(eng, steps), replay.plain_logits(cfg, w, reqs), dtype, f"batched by {batch_size}")


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("batch_size", [24, 64])
def test_one_token_steps_of_many_rows_with_their_fused_products(models, name, batch_size):
    """The same with the fused products for 17 to 64 rows switched on (csrc/linear_batch.cu, off unless asked for):
    prompt steps of up to 64 tokens take them too."""
    from pico_engine.ops import kernels
    eng, cfg, w = models[(name, "bfloat16")]
    reqs = many_short_requests(cfg, name, batch_size + 9, 30 + batch_size)
    steps = replay.batched(reqs, batch_size, 0.5)
    was = kernels.set_batch_fused(True)
    try:
        got = replay.run_in_process(eng, steps)
        kernels.check_status("cuda")
    finally:
        kernels.set_batch_fused(was)
    replay.compare(got, replay.plain_logits(cfg, w, reqs), "bfloat16", f"batched by {batch_size}, fused")


PIECE_LENGTHS = {"A": [100, 7, 64, 33, 128], "B": [200, 9, 130, 64, 256], "C": [300, 20, 150, 257, 129]}


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompts_in_pieces(models, name, dtype):
    """A prompt brought in two or three steps: the later pieces start inside the sequence and bring several
    tokens.  On B and C (windows of 32 and 70) the first piece of the long requests is longer than a
    page plus the window, so the windowed group has given pages back before the next piece arrives
    and that piece attends over a page table with holes."""
    eng, cfg, w = models[(name, dtype)]
    reqs = random_requests(cfg, PIECE_LENGTHS[name], 40)
    steps = replay.pieces(reqs)
    assert any(len(e["tokens"]) > 1 for s in steps[1:] for e in s["entries"])
    replay.compare(replay.run_in_process(eng, steps), replay.plain_logits(cfg, w, reqs), dtype, "pieces")
    if name != "A":                                      # the holes are really there
        eng.ensure_cache(1024, cfg["max_position_embeddings"], max_seqs=4)
        slot = eng.cache.open()
        eng.stepper.step([slot], [reqs["r0"][:len(reqs["r0"]) // 2]], [[]])
        windowed = [g for g in eng.cache.groups if g.need.window is not None]
        assert windowed and windowed[0].table[slot][0] == -1
        eng.cache.close(slot)


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_steps(models, name, dtype):
    """One step carries a fresh prompt, a piece of another and single tokens of others."""
    eng, cfg, w = models[(name, dtype)]
    reqs = random_requests(cfg, PIECE_LENGTHS[name][::-1] + [12, 3], 41)
    steps = replay.mixed(reqs)
    kinds = [sorted({"one" if len(e["tokens"]) == 1 else "many" for e in s["entries"]}) for s in steps]
    assert ["many", "one"] in kinds
    replay.compare(replay.run_in_process(eng, steps), replay.plain_logits(cfg, w, reqs), dtype, "mixed")


@pytest.mark.parametrize("name,dtype", CASES)
def test_cutting_does_not_change_float32_results_beyond_rounding(models, name, dtype):
    eng, cfg, w = models[(name, dtype)]
    reqs = random_requests(cfg, LENGTHS[name], 13)
    a = replay.run_in_process(eng, replay.whole(reqs))
    b = replay.run_in_process(eng, replay.tail(reqs, 32))
    c = replay.run_in_process(eng, replay.batched(reqs, 3, 0.5))
    for key in a:
        for other in (b, c):
            ok, msg = close_enough(torch.from_numpy(other[key]), torch.from_numpy(a[key]), dtype)
            assert ok, (key, msg)
            if dtype == "float32":
                assert float(np.abs(other[key] - a[key]).max()) <= 2e-5 * max(1.0, float(np.abs(a[key]).max())), key


@pytest.mark.parametrize("name,dtype", CASES)
def test_long_decoding_and_first_tokens(models, name, dtype):
    """Three prompt tokens, then token by token up to the longest sequence the model allows:
    crosses cache pages and, for tiny-B, leaves the window's pages behind."""
    eng, cfg, w = models[(name, dtype)]
    n = cfg["max_position_embeddings"]
    reqs = random_requests(cfg, [n, 2, 3], 14)
    steps = replay.tail(reqs, n - 3)
    got = replay.run_in_process(eng, steps)
    replay.compare(got, replay.plain_logits(cfg, w, reqs), dtype, "long decode")
    if name == "B":                                     # in steady state the window group held about a window
        eng.ensure_cache(512, 256, max_seqs=8)
        s = eng.cache.open()
        eng.stepper.step([s], [reqs["r0"][:100]])
        for t in reqs["r0"][100:240]:
            eng.stepper.step([s], [[t]])
        held = [sum(p >= 0 for p in g.table[s]) for g in eng.cache.groups]
        assert held == [4, 1] or held == [4, 2], held
        eng.cache.close(s)


def test_padding_and_neighbours_change_nothing(models):
    """A request's float32 logits with and without neighbours in the batch."""
    eng, cfg, w = models[("B", "float32")]
    reqs = random_requests(cfg, [50, 7, 120], 15)
    alone = replay.run_in_process(eng, replay.whole({"r0": reqs["r0"]}))
    together = replay.run_in_process(eng, [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}
                                                                    for r, t in reqs.items()], "end": list(reqs)}])
    for p in range(50):
        assert np.array_equal(alone[("r0", p)], together[("r0", p)]), p


def test_step_refuses_what_it_cannot_run(models):
    from pico_engine.cache import CacheFull
    from pico_engine.engine.step import StepError
    eng, cfg, w = models[("A", "float32")]
    eng.cache = eng.stepper = None
    eng.ensure_cache(128, 128, max_seqs=2)
    s = eng.cache.open()
    for bad, err in ((([s], [[]]), StepError), (([s], [[999]]), StepError), (([s, s], [[1], [2]]), StepError),
                     (([s], [[1, 2]], [[5]]), StepError), (([s], [list(range(129))]), StepError)):
        with pytest.raises(err):
            eng.stepper.step(*bad)
    t = eng.cache.open()
    eng.stepper.step([s], [[1] * 100])
    with pytest.raises(CacheFull):
        eng.stepper.step([t], [[1] * 100])
    eng.cache.close(s); eng.cache.close(t)


# ---------------------------------------------------------------------------- generation through the entry point

@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("use_graph", [False, True])
def test_greedy_generation_float32(models, name, use_graph):
    eng, cfg, w = models[(name, "float32")]
    lengths = [5, 9, 13] if name == "A" else [1, 17, 40, 64]
    prompts = list(random_requests(cfg, lengths, 16).values())
    got = eng.generate(prompts, max_tokens=8 if name == "A" else 16, temperature=0.0, use_graph=use_graph)
    want = [plain.generate(cfg, w, p, 8 if name == "A" else 16) for p in prompts]
    assert got == want
    assert eng.generate(prompts[0], max_tokens=4, temperature=0) == want[0][:4]      # one prompt in, one list out
    assert not eng.cache.lengths


@pytest.mark.parametrize("name", ["A", "B"])
def test_seeded_sampling_float32(models, name):
    eng, cfg, w = models[(name, "float32")]
    prompts = list(random_requests(cfg, [1, 17, 40, 64], 17).values())
    kw = dict(temperature=0.8, top_k=0, top_p=1.0, seed=5)
    got = eng.generate(prompts, max_tokens=16, **kw)
    want = [plain.generate(cfg, w, p, 16, request=i, **kw) for i, p in enumerate(prompts)]
    assert got == want
    again = eng.generate(prompts[::-1], max_tokens=16, **kw)
    assert again != got[::-1]                                     # a request's stream is named by its place in the call
    assert eng.generate(prompts, max_tokens=16, **kw) == got
    narrowed = eng.generate(prompts, max_tokens=16, temperature=0.8, top_k=3, top_p=0.7, seed=5, use_graph=False)
    assert narrowed == [plain.generate(cfg, w, p, 16, temperature=0.8, top_k=3, top_p=0.7, seed=5, request=i)
                        for i, p in enumerate(prompts)]


@pytest.mark.parametrize("name", ["A", "B"])
def test_stop_tokens_and_many_batches(models, name):
    eng, cfg, w = models[(name, "float32")]
    prompts = list(random_requests(cfg, [3, 30, 8, 21, 2, 14, 9], 18).values())
    free = [plain.generate(cfg, w, p, 12) for p in prompts]
    stop = (free[1][4], free[3][0])
    eng.max_batch, old = 3, eng.max_batch
    try:
        got = eng.generate(prompts, max_tokens=12, temperature=0.0, stop_token_ids=stop)
    finally:
        eng.max_batch = old
    want = [plain.generate(cfg, w, p, 12, stop=stop) for p in prompts]
    assert got == want and len(got[1]) <= 4 and got[3] == []
    assert not eng.cache.lengths and eng.cache.slots.free_count == eng.cache.max_seqs


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("use_graph", [False, True])
def test_greedy_generation_bfloat16(models, name, use_graph):
    """Each chosen token must be a (near) maximum of the plain logits for the engine's own
    prefix: bfloat16 rounding may swap candidates whose plain logits are within the tolerance."""
    eng, cfg, w = models[(name, "bfloat16")]
    prompts = list(random_requests(cfg, [5, 9, 13, 40], 19).values())
    got = eng.generate(prompts, max_tokens=12, temperature=0.0, use_graph=use_graph)
    exact = 0
    for p, out in zip(prompts, got):
        assert len(out) == 12
        logits = plain.forward(cfg, w, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[tok]) <= 4e-2 * max(1.0, float(row.abs().max())), (i, tok)
            exact += int(row.argmax()) == tok
    assert exact >= 40


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_decoding_one_step_ahead_changes_no_token(models, name):
    """With graphs the loop launches a step before it has read the one in flight; without, it does
    not.  Budgets that differ, stop tokens that fall early, late and on the last token, sampling."""
    eng, cfg, w = models[(name, "float32")]
    prompts = list(random_requests(cfg, [3, 30, 8, 21, 2, 14], 23).values())
    budgets = [1, 20, 7, 20, 2, 13]
    kw = dict(temperature=0.9, top_k=0, top_p=1.0, seed=11)
    free = eng.generate(prompts, max_tokens=budgets, use_graph=False, stop_token_ids=(), **kw)
    stop = (free[1][9], free[3][19], free[5][0])
    ahead = eng.generate(prompts, max_tokens=budgets, use_graph=True, stop_token_ids=stop, **kw)
    plainly = eng.generate(prompts, max_tokens=budgets, use_graph=False, stop_token_ids=stop, **kw)
    assert ahead == plainly
    assert ahead == [plain.generate(cfg, w, p, m, stop=stop, request=i, **kw) for i, (p, m) in enumerate(zip(prompts, budgets))]
    assert len(ahead[1]) <= 9 and ahead[5] == [] and len(ahead[0]) <= 1
    assert not eng.cache.lengths and eng.cache.slots.free_count == eng.cache.max_seqs


@pytest.mark.parametrize("name", ["B", "C"])
def test_graph_and_eager_decode_agree(models, name):
    eng, cfg, w = models[(name, "bfloat16")]
    prompts = list(random_requests(cfg, [20, 70, 3], 20).values())
    a = eng.generate(prompts, max_tokens=70, temperature=0.7, top_p=0.9, seed=3, use_graph=True)
    b = eng.generate(prompts, max_tokens=70, temperature=0.7, top_p=0.9, seed=3, use_graph=False)
    assert a == b


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "float32"), ("C", "bfloat16")])
def test_many_requests_share_a_few_graphs(models, name, dtype):
    """64 requests whose budgets differ end one by one, so the decode steps have every row count from 64 down:
    they run in the graphs of a few row buckets (idle rows fill a bucket), with the tokens of eager decoding.
    Other temperatures and seeds are numbers that a graph reads at run time: they capture nothing new."""
    eng, cfg, w = models[(name, dtype)]
    g = torch.Generator().manual_seed(31)
    lengths = torch.randint(2, 13, (64,), generator=g).tolist()
    prompts = list(random_requests(cfg, lengths, 32).values())
    budgets = [1 + (5 * i) % 23 for i in range(64)]
    eng._graphs.clear()
    graphed = eng.generate(prompts, max_tokens=budgets, temperature=0.0, use_graph=True, stop_token_ids=())
    assert 3 <= len(eng._graphs) <= 7, sorted(eng._graphs)
    eager = eng.generate(prompts, max_tokens=budgets, temperature=0.0, use_graph=False, stop_token_ids=())
    assert [len(o) for o in graphed] == budgets
    if dtype == "float32":
        assert graphed == eager
        for i in (0, 17, 63):
            assert graphed[i] == plain.generate(cfg, w, prompts[i], budgets[i])
    else:                                               # bfloat16: rows of a bucket of 64 and of 16 take different kernels
        for p, out in zip(prompts, graphed):
            logits = plain.forward(cfg, w, p + out)
            for i, tok in enumerate(out):
                row = logits[len(p) + i - 1]
                assert float(row.max() - row[tok]) <= 4e-2 * max(1.0, float(row.abs().max())), (i, tok)
    kw = dict(max_tokens=6, top_k=0, top_p=1.0, stop_token_ids=())
    first = eng.generate(prompts[:8], temperature=0.8, seed=1, use_graph=True, **kw)
    held = len(eng._graphs)
    second = eng.generate(prompts[:8], temperature=0.5, seed=2, use_graph=True, **kw)
    third = eng.generate(prompts[:8], temperature=0.8, seed=1, use_graph=True, **kw)
    assert len(eng._graphs) == held and third == first and second != first
    if dtype == "float32":
        assert second == eng.generate(prompts[:8], temperature=0.5, seed=2, use_graph=False, **kw)
        assert second == [plain.generate(cfg, w, p, 6, temperature=0.5, seed=2, request=i) for i, p in enumerate(prompts[:8])]


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompt_steps_as_captured_graphs(models, name, dtype):
    """With graphs, a step that brings prompts runs as a captured graph of padded sizes from the second time its sizes
    come up: rows and tokens are filled up with idle rows.  Logits and tokens are those of the step launched kernel by
    kernel; other prompts of the same sizes, and prompts that continue (pieces), go through the same graph."""
    eng, cfg, w = models[(name, dtype)]
    reqs = random_requests(cfg, [33, 5, 70, 1, 100], 50)
    want = replay.plain_logits(cfg, w, reqs)
    eng.cache = eng.stepper = None
    eng.ensure_cache(1024, cfg["max_position_embeddings"], max_seqs=8)
    st, cache = eng.stepper, eng.cache

    def run(tokens_of, use_graph):
        slots = [cache.open() for _ in tokens_of]
        first = st.step(slots, [t[:len(t) // 2 + 1] for t in tokens_of], use_graph=use_graph).cpu()      # a first piece of every prompt
        for s_ in slots:
            cache.close(s_)
        return first
    prompts = list(reqs.values())
    eager = run(prompts, False)
    assert not st._prompt_graphs
    a = run(prompts, True)                                    # the sizes come up for the first time: padded, kernel by kernel
    assert next(iter(st._prompt_graphs.values())).graph is None
    b = run(prompts, True)                                    # captured and replayed
    c = run(prompts, True)                                    # replayed
    assert len(st._prompt_graphs) == 1 and next(iter(st._prompt_graphs)) == (10, 128)
    assert next(iter(st._prompt_graphs.values())).graph is not None
    assert torch.equal(a, b) and torch.equal(b, c)            # the same kernels at the same sizes, captured or not
    for got in (a, b, c):
        assert got.shape == eager.shape
        for i, (rid, toks) in enumerate(reqs.items()):
            ok, msg = close_enough(got[i], torch.from_numpy(want[(rid, len(toks) // 2)]), dtype)
            assert ok, (rid, msg)
    if dtype == "float32":
        assert torch.equal(b, eager) and torch.equal(c, eager)
    # other prompts of other lengths, the same sizes after padding: the same graph, no new capture
    others = list(random_requests(cfg, [40, 9, 60, 7, 12], 51).values())
    held = next(iter(st._prompt_graphs.values()))
    again = run(others, True)
    assert len(st._prompt_graphs) == 1 and next(iter(st._prompt_graphs.values())) is held
    ref = run(others, False)
    ok, msg = close_enough(again, ref, dtype)
    assert ok, msg
    cache.check()
    assert not cache.lengths
    # through the entry point: three calls with the same prompts give the same tokens, with and without graphs
    outs = [eng.generate(prompts, max_tokens=5, temperature=0.0, use_graph=g) for g in (True, True, True, False)]
    assert outs[0] == outs[1] == outs[2]
    if dtype == "float32":
        assert outs[2] == outs[3] == [plain.generate(cfg, w, p, 5) for p in prompts]


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("budget", [64, 33])
def test_generation_with_prompts_in_portions(models, name, dtype, budget):
    """A batch whose prompts have more tokens than a step may take is prefilled in several steps: with 64 tokens a step
    the cuts fall on page edges and leave the first prompt (66 or 130 tokens) a tail of two; with 33 they fall inside pages and, for
    B, one token past its window of 32.  The tokens are those of prompts taken whole."""
    eng, cfg, w = models[(name, dtype)]
    prompts = list(random_requests(cfg, [66 if name == "A" else 130, 64, 7, 100, 65], 60 + budget).values())
    whole = eng.generate(prompts, max_tokens=6, temperature=0.0, use_graph=False)
    eng.prefill_tokens_per_step, old = budget, eng.prefill_tokens_per_step
    try:
        cut = eng.generate(prompts, max_tokens=6, temperature=0.0, use_graph=False)
        cut_graphed = eng.generate(prompts, max_tokens=6, temperature=0.0, use_graph=True)
    finally:
        eng.prefill_tokens_per_step = old
    assert not eng.cache.lengths
    if dtype == "float32":
        assert cut == whole == cut_graphed == [plain.generate(cfg, w, p, 6) for p in prompts]
    else:
        for p, out in zip(prompts, cut):
            logits = plain.forward(cfg, w, p + out)
            for i, tok in enumerate(out):
                row = logits[len(p) + i - 1]
                assert float(row.max() - row[tok]) <= 4e-2 * max(1.0, float(row.abs().max())), (i, tok)


def test_weights_stored_in_float32_stay_so(tmp_path):
    """A checkpoint whose norms and one projection are stored in 32 bits, run by the bfloat16 engine."""
    from pico_engine.engine.engine import Engine
    cfg = dict(TINY["A"])
    w = make_weights(cfg, 3, sharp=True)
    f32 = {n for n in w if "norm" in n} | {"model.layers.1.mlp.down_proj.weight"}
    eng = Engine(write_model(tmp_path / "m", cfg, w, float32_names=f32), dtype="bfloat16")
    assert eng.model.layers[1].feed_forward.w_down.dtype == torch.float32
    reqs = random_requests(cfg, [40, 9], 21)
    replay.compare(replay.run_in_process(eng, replay.tail(reqs, 8)), replay.plain_logits(cfg, w, reqs), "bfloat16", "mixed")


def test_random_weights_mode_end_to_end(tmp_path):
    """The library's own writer, its loader, and generation; compared with the plain implementation
    reading the same folder through the safetensors package."""
    from safetensors.torch import load_file
    from pico_engine.config import config_from_dict
    from pico_engine.engine.engine import Engine
    from pico_engine.weights import write_random_model
    cfg = dict(TINY["B"])
    write_random_model(config_from_dict(cfg), 1, str(tmp_path / "r"))
    w = {k: v.float() for k, v in load_file(str(tmp_path / "r" / "model.safetensors")).items()}
    eng = Engine(str(tmp_path / "r"), dtype="float32")
    reqs = random_requests(cfg, [1, 17, 40, 64], 22)
    replay.compare(replay.run_in_process(eng, replay.batched(reqs, 4, 1.0)), replay.plain_logits(cfg, w, reqs), "float32", "random")
    direct = Engine.from_config(config_from_dict(cfg), seed=1, dtype="float32")
    assert torch.equal(direct.model.head.cpu(), w["lm_head.weight"])
