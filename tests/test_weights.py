"""The safetensors container, the checked loader and the random-weights mode (CPU)."""
import json

import pytest
import torch

from conftest import TINY_A, TINY_B, make_weights, tensor_shapes, write_model
from pico_engine.config import config_from_dict
from pico_engine.parts import DecoderModel
from pico_engine.weights import (Checkpoint, ParamSpec, SafetensorsError, WeightError, check, convert, load_folder,
                                 random_tensor, write_random_model, write_safetensors)


def test_expected_tensors_are_the_checkpoint_names():
    for d in (TINY_A, TINY_B):
        model = DecoderModel(config_from_dict(d).plan(), torch.bfloat16, "meta")
        assert {n: tuple(s.shape) for n, s in model.expected_tensors().items()} == tensor_shapes(d)


def test_container_round_trip_matches_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
               "c": torch.randn(4), "d": torch.randn(2, 2).to(torch.float16)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors.items(), {"note": "x"})
    theirs = load_file(path)
    ours = Checkpoint(str(tmp_path))
    assert set(ours.entries) == set(tensors)
    for n, t in tensors.items():
        assert torch.equal(theirs[n], t) and torch.equal(ours.read(n), t) and ours.read(n).dtype == t.dtype
    # and the other way: a file of the package is read by ours
    write_model(tmp_path / "m", TINY_A, make_weights(TINY_A, 0))
    ck = Checkpoint(str(tmp_path / "m"))
    assert ck.entries["model.embed_tokens.weight"].dtype == "BF16" and ck.read("model.norm.weight").shape == (64,)


def test_broken_containers_are_refused(tmp_path):
    (tmp_path / "model.safetensors").write_bytes(b"\x05\x00")
    with pytest.raises(SafetensorsError, match="too short"):
        Checkpoint(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        Checkpoint(str(tmp_path))
    head = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    (tmp_path / "model.safetensors").write_bytes(len(head).to_bytes(8, "little") + head + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="does not match"):
        Checkpoint(str(tmp_path))
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        Checkpoint(str(tmp_path / "empty"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    w = make_weights(TINY_B, 1)
    del w["model.layers.1.mlp.up_proj.weight"], w["model.layers.2.self_attn.k_proj.bias"]
    w["model.layers.0.extra.weight"] = torch.zeros(3)
    w["model.norm.weight"] = torch.zeros(95)
    w["lm_head.weight"] = torch.zeros(96, 512)
    folder = write_model(tmp_path / "m", TINY_B, w)
    model = DecoderModel(config_from_dict(TINY_B).plan(), torch.float32, "cpu")
    with pytest.raises(WeightError) as e:
        load_folder(model, folder)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.layers.2.self_attn.k_proj.bias"]
    assert err.unexpected == ["model.layers.0.extra.weight"]
    assert [(n, have, want) for n, have, want in err.wrong_shape] == [
        ("lm_head.weight", (96, 512), (512, 96)), ("model.norm.weight", (95,), (96,))]
    text = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (2)", "stored [95], model needs [96]", "up_proj"):
        assert word in text


def test_tensors_nobody_asks_for_are_a_warning_that_names_them(tmp_path):
    """A complete checkpoint with extra tensors (older conversions store rotary_emb.inv_freq) loads."""
    from pico_engine.weights import UnusedWeightsWarning
    w = make_weights(TINY_A, 0)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    w["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    model = DecoderModel(config_from_dict(TINY_A).plan(), torch.float32, "cpu")
    with pytest.warns(UnusedWeightsWarning, match=r"2 tensor\(s\).*layers\.0\.self_attn\.rotary_emb\.inv_freq, model\.layers\.1"):
        load_folder(model, write_model(tmp_path / "m", TINY_A, w))
    assert torch.equal(model.embedding, w["model.embed_tokens.weight"])


def test_tied_model_may_carry_a_head_it_does_not_use(tmp_path):
    w = make_weights(TINY_A, 0)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    model = DecoderModel(config_from_dict(TINY_A).plan(), torch.float32, "cpu")
    load_folder(model, write_model(tmp_path / "m", TINY_A, w))
    assert model.head is model.embedding


def test_dtype_rules():
    bf, f16, f32, f64 = (torch.ones(2).to(d) for d in (torch.bfloat16, torch.float16, torch.float32, torch.float64))
    i64 = torch.arange(3)
    assert convert(bf, torch.bfloat16).dtype == torch.bfloat16 and convert(f16, torch.bfloat16).dtype == torch.bfloat16
    assert convert(f32, torch.bfloat16).dtype == torch.float32      # a tensor stored in 32 bits stays so
    assert convert(f64, torch.bfloat16).dtype == torch.float32
    assert all(convert(t, torch.float32).dtype == torch.float32 for t in (bf, f16, f32, f64))
    assert convert(i64, torch.bfloat16).dtype == torch.int32 and convert(i64, torch.float32).dtype == torch.int32


def test_loader_keeps_stored_float32_and_fuses_projections(tmp_path):
    w = make_weights(TINY_A, 0)
    folder = write_model(tmp_path / "m", TINY_A, w, float32_names={"model.norm.weight", "model.layers.0.input_layernorm.weight"})
    model = DecoderModel(config_from_dict(TINY_A).plan(), torch.bfloat16, "cpu")
    load_folder(model, folder)
    assert model.final_norm.weight.dtype == torch.float32 and model.layers[0].mixer_norm.weight.dtype == torch.float32
    assert model.layers[1].mixer_norm.weight.dtype == torch.bfloat16 and model.embedding.dtype == torch.bfloat16
    att = model.layers[0].mixer
    want = torch.cat([w[f"model.layers.0.self_attn.{n}_proj.weight"] for n in "qkv"]).to(torch.bfloat16)
    assert torch.equal(att.w_qkv, want) and att.b_qkv.shape == (4 * 16 + 2 * 2 * 16,)
    assert model.layers[0].feed_forward.w_gate_up.shape == (320, 64)


def test_random_mode_writes_a_folder_the_loader_reads(tmp_path):
    cfg = config_from_dict(TINY_B)
    write_random_model(cfg, 7, str(tmp_path / "r"), float32_names={"model.norm.weight"})
    assert json.load(open(tmp_path / "r" / "config.json"))["architectures"] == ["Qwen2ForCausalLM"]
    ck = Checkpoint(str(tmp_path / "r"))
    assert {n: e.shape for n, e in ck.entries.items()} == tensor_shapes(TINY_B)
    assert ck.entries["model.norm.weight"].dtype == "F32" and ck.entries["lm_head.weight"].dtype == "BF16"
    model = DecoderModel(cfg.plan(), torch.bfloat16, "cpu")
    load_folder(model, str(tmp_path / "r"))
    # same seed, same values, whatever the order of creation; another seed, other values
    spec = ParamSpec((512, 96))
    again = random_tensor("lm_head.weight", spec, 7, torch.bfloat16)
    assert torch.equal(model.head, again) and not torch.equal(again, random_tensor("lm_head.weight", spec, 8, torch.bfloat16))
    norm = ck.read("model.layers.0.input_layernorm.weight").float()
    assert abs(float(norm.mean()) - 1.0) < 0.02 and 0.005 < float(ck.read("lm_head.weight").float().std()) < 0.04


def test_check_accepts_a_fitting_checkpoint():
    check({"a": ParamSpec((2, 3))}, {"a": (2, 3), "b": (1,)}, ignorable=("b",))
