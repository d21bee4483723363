"""bin/trace_run as a user runs it: a model folder, steps on standard input, logits on disk."""
import os
import subprocess
import sys

import pytest
import torch

import replay
from conftest import TINY, make_weights, write_model

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_in_three_cuts(tmp_path, name, dtype):
    cfg = dict(TINY[name])
    w = make_weights(cfg, 30, sharp=True)
    folder = write_model(tmp_path / "model", cfg, w)
    g = torch.Generator().manual_seed(31)
    lengths = [40, 7, 70, 33, 100] if name == "A" else [1, 90, 64, 140, 35]
    reqs = {f"q{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
    want = replay.plain_logits(cfg, w, reqs)
    for cut, steps in (("whole", replay.whole(reqs)), ("tail", replay.tail(reqs, 32)), ("batched", replay.batched(reqs, 3, 0.6))):
        got = replay.run_binary(folder, dtype, steps, str(tmp_path / f"out_{cut}"), cfg["vocab_size"])
        replay.compare(got, want, dtype, f"{name} {dtype} {cut}")


def test_steps_without_wanted_logits_write_no_file(tmp_path):
    cfg = dict(TINY["A"])
    folder = write_model(tmp_path / "model", cfg, make_weights(cfg, 0))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}], "end": ["a"]},
             {"step": 2, "entries": [], "end": []}]
    got = replay.run_binary(folder, "float32", steps, str(tmp_path / "out"), cfg["vocab_size"], max_tokens=64)
    assert sorted(os.listdir(tmp_path / "out")) == ["1.f32"] and list(got) == [("a", 3)]


def test_a_bad_model_folder_fails_with_the_reason(tmp_path):
    cfg = dict(TINY["A"])
    w = make_weights(cfg, 0)
    del w["model.norm.weight"]
    folder = write_model(tmp_path / "model", cfg, w)
    proc = subprocess.run([sys.executable, os.path.join(replay.ROOT, "bin", "trace_run"), "--model", folder, "--dtype",
                           "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"], input="", capture_output=True, text=True)
    assert proc.returncode != 0 and "missing (1): model.norm.weight" in proc.stderr
