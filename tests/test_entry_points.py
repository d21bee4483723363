"""Command line parsing, the benchmark's statistics and bench.py's contract for more than one GPU (CPU)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_percentile_and_summary():
    """The statistics of pico-engine's evidence protocol (tests/test_evidence.py there: interpolation, keys, empty input)."""
    from pico_engine.benchmark import percentile, summary
    assert percentile([1, 2, 3, 4], 50) == 2.5 and percentile([10], 90) == 10.0
    assert percentile([4, 1, 3, 2], 0) == 1.0 and percentile([4, 1, 3, 2], 100) == 4.0
    assert abs(percentile(list(range(11)), 10) - 1.0) < 1e-12
    s = summary([3.0, 1.0, 2.0])
    assert s["median"] == 2.0 and s["min"] == 1.0 and s["max"] == 3.0 and s["n"] == 3 and s["p10"] < s["p90"]
    with pytest.raises(ValueError):
        percentile([], 50)


def test_prompt_ids_parsing():
    from pico_engine.__main__ import parse_ids
    assert parse_ids("5,17,3") == [5, 17, 3] and parse_ids(" 5 17  3 ") == [5, 17, 3] and parse_ids("[1, 2]") == [1, 2]
    with pytest.raises(ValueError):
        parse_ids("5,x")


def test_command_line_refuses_bad_arguments(tmp_path):
    def run(*args):
        return subprocess.run([sys.executable, "-m", "pico_engine", *args], cwd=ROOT, capture_output=True, text=True)
    r = run(str(tmp_path), "--prompt", "1,2")
    assert r.returncode != 0 and "config.json" in r.stderr
    (tmp_path / "config.json").write_text("{}")
    r = run(str(tmp_path), "--prompt", "1,2", "--max-tokens", "-1")
    assert r.returncode != 0 and "non-negative" in r.stderr
    r = run(str(tmp_path))
    assert r.returncode != 0 and "--prompt" in r.stderr
    r = run("--help")
    assert r.returncode == 0 and all(o in r.stdout for o in ("--max-tokens", "--temperature", "--top-p", "--top-k", "--no-graph"))


def test_bench_says_so_for_more_than_one_gpu():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True)
    assert r.returncode == 2 and len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_sampling_params_follow_the_reference_defaults():
    from pico_engine.sampling import SamplingParams
    p = SamplingParams()
    assert (p.temperature, p.top_k, p.top_p) == (0.7, 0, 0.9) and not p.greedy and SamplingParams(temperature=0).greedy
    for bad in (dict(top_k=-1), dict(top_p=0.0), dict(top_p=1.5)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


def test_named_shapes_are_valid_configurations():
    from pico_engine.config import config_from_dict
    from pico_engine.config.shapes import SHAPES, shape
    for name in SHAPES:
        cfg = config_from_dict(shape(name))
        assert cfg.plan().layers and cfg.num_attention_heads % cfg.num_key_value_heads == 0
    b = json.load(open(os.path.join(ROOT, "BASELINE.json")))["configs"][2]
    c = config_from_dict(shape("qwen2.5-0.5b"))
    for word in ("24 layers", "hidden 896", "14 heads", "2 KV heads", "head_dim 64", "intermediate 4864", "vocab 151936"):
        assert word in b
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size, c.vocab_size, c.tie_word_embeddings) == (24, 896, 14, 2, 64, 4864, 151936, True)
    with pytest.raises(KeyError):
        shape("qwen9")


def test_kernel_library_refuses_to_run_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from pico_engine.ops.library import KernelError, require_cuda
    with pytest.raises(KernelError, match="CUDA"):
        require_cuda("cpu")
    with pytest.raises(KernelError, match="no CUDA device"):
        require_cuda("cuda")


def test_command_line_refuses_bad_random_arguments(tmp_path):
    def run(*args):
        return subprocess.run([sys.executable, "-m", "pico_engine", *args], cwd=ROOT, capture_output=True, text=True)
    r = run("--random-config", "qwen9", "--prompt", "1")
    assert r.returncode != 0 and "unknown shape" in r.stderr
    r = run(str(tmp_path), "--random-config", "tiny-a", "--prompt", "1")
    assert r.returncode != 0 and "model folder or --random-config" in r.stderr
    r = run("--random-config", "tiny-a", "--random-prompt", "0")
    assert r.returncode != 0 and "positive lengths" in r.stderr
    r = run("--random-config", "tiny-a", "--layers", "0", "--prompt", "1")
    assert r.returncode != 0 and "--layers" in r.stderr


def test_random_prompts_are_seeded():
    from pico_engine.__main__ import random_prompts
    a, b = random_prompts([5, 9], 256, 3), random_prompts([5, 9], 256, 3)
    assert a == b and [len(p) for p in a] == [5, 9] and all(0 <= t < 256 for p in a for t in p)
    assert random_prompts([5, 9], 256, 4) != a


# ---------------------------------------------------------------------------- the command lines on a GPU

def _outputs(stdout: str):
    return [json.loads(line) for line in stdout.splitlines() if line.startswith("{")]


@pytest.mark.gpu
def test_command_line_generates_the_plain_tokens(tmp_path):
    """``python -m pico_engine FOLDER --prompt ... --prompt ... --temperature 0`` prints the token ids that
    the plain implementation chooses (float32, so that the comparison is exact), stops at a stop token, and
    the same model drawn at random from its name gives tokens too."""
    import plain_qwen2 as plain
    from conftest import TINY_B, make_weights, write_model
    cfg = dict(TINY_B)
    w = make_weights(cfg, 1, sharp=True)
    folder = write_model(tmp_path / "m", cfg, w)
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6], [27, 18, 28]]
    base = [sys.executable, "-m", "pico_engine", folder, "--prompt", "3,1,4,1,5,9,2,6", "--prompt", "27 18 28",
            "--max-tokens", "7", "--temperature", "0", "--dtype", "float32"]
    r = subprocess.run(base, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    outs = _outputs(r.stdout)
    want = [plain.generate(cfg, w, p, 7) for p in prompts]
    assert [o["prompt"] for o in outs] == prompts and [o["output"] for o in outs] == want
    assert "[engine] loaded in" in r.stdout and "tok/s" in r.stdout
    stop = want[0][3]
    r = subprocess.run(base + ["--stop-token-ids", str(stop), "--no-graph"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [o["output"] for o in _outputs(r.stdout)] == [plain.generate(cfg, w, p, 7, stop=(stop,)) for p in prompts]
    r = subprocess.run([sys.executable, "-m", "pico_engine", "--random-config", "tiny-a", "--random-prompt", "5,9,13",
                        "--max-tokens", "8", "--temperature", "0.8", "--seed", "4"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    outs = _outputs(r.stdout)
    assert [len(o["prompt"]) for o in outs] == [5, 9, 13] and all(len(o["output"]) == 8 for o in outs)


@pytest.mark.gpu
def test_benchmark_command_line_writes_its_record(tmp_path):
    out = tmp_path / "record.json"
    r = subprocess.run([sys.executable, "-m", "pico_engine.benchmark", "--random", "tiny-a", "--batch", "1,3", "--context", "96",
                        "--prefill", "64", "--n-tokens", "8", "--warmups", "1", "--repetitions", "2", "--output", str(out)],
                       cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    rec = json.loads(out.read_text())
    assert rec["prefill"]["tokens"] == 64 and rec["prefill"]["ms"] > 0
    for b in ("1", "3"):
        s = rec["decode"][b]["tokens_per_s"]
        assert s["n"] == 2 and 0 < s["p10"] <= s["median"] <= s["p90"]
    assert "decode batch 3" in r.stdout
