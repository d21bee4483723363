"""Each part alone against its plain formula, and a model put together in other ways than
Qwen2's own plan (a layer named twice, a layer that reads another layer's cache)."""
from dataclasses import replace
from types import SimpleNamespace

import pytest
import torch

import plain_qwen2 as plain
from conftest import TINY_B, make_weights

pytestmark = pytest.mark.gpu


def step_context(mixers, lens, starts, dtype, hd_tokens=512):
    """A context for one step over a fresh cache in which every row already holds ``starts[b]`` tokens."""
    from pico_engine.cache import Cache
    from pico_engine.engine.step import Stepper
    cache = Cache([m.cache_needs() for m in mixers], hd_tokens, 8, dtype, "cuda")
    stub = SimpleNamespace(plan=SimpleNamespace(vocab_size=1 << 20), dtype=dtype)
    stepper = Stepper(stub, cache, 512)
    slots = [cache.open() for _ in lens]
    for s, st in zip(slots, starts):
        if st:
            cache.reserve(s, st); cache.advance(s, st)
    lay, host, st = stepper.describe(slots, lens, None, None)
    return stepper.context(lay, stepper.upload(host), lens, st, slots), cache, slots


def test_norm_part():
    from pico_engine.config import RMSNormSpec
    from pico_engine.parts import NORMS, build_part
    w = 1 + torch.randn(96) * 0.1
    part = build_part(NORMS, "norm", RMSNormSpec(96, 1e-5, "n.weight"), torch.bfloat16, "cuda")
    assert list(part.expected_tensors()) == ["n.weight"] and part.expected_tensors()["n.weight"].shape == (96,)
    part.take_tensors(lambda name: w.cuda())
    x = torch.randn(5, 96) * 4
    assert torch.allclose(part.forward(x.cuda(), torch.float32).cpu(), plain.rms_norm(x, w, 1e-5), atol=1e-5)
    assert part.forward(x.cuda(), torch.bfloat16).dtype == torch.bfloat16


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_with_and_without_position_encoding(dtype):
    from pico_engine.config import GQAAttentionSpec, NoPositionSpec, RotaryHalfSpec
    from pico_engine.parts import MIXERS, build_part
    H, nh, nkv, hd = 80, 5, 1, 16
    g = torch.Generator().manual_seed(0)
    tensors = {f"a.{n}_proj.weight": (torch.randn(o, H, generator=g) * H ** -0.5).bfloat16().float()
               for n, o in (("q", nh * hd), ("k", nkv * hd), ("v", nkv * hd))}
    tensors["a.o_proj.weight"] = (torch.randn(H, nh * hd, generator=g) * 0.1).bfloat16().float()
    tensors.update({f"a.{n}_proj.bias": (torch.randn(o, generator=g) * 0.2).bfloat16().float()
                    for n, o in (("q", nh * hd), ("k", nkv * hd), ("v", nkv * hd))})
    lens = [70, 9]
    h = (torch.randn(sum(lens), H, generator=g)).bfloat16().float()
    for position in (RotaryHalfSpec(hd, 5e4), NoPositionSpec()):
        spec = GQAAttentionSpec(hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd, qkv_bias=True, window=None,
                                scale=0.4, position=position, prefix="a.")
        part = build_part(MIXERS, "mixer", spec, dtype, "cuda")
        assert set(part.expected_tensors()) == set(tensors)
        part.take_tensors(lambda n: tensors[n].to(dtype).cuda())
        part.prepare(128)
        ctx, cache, slots = step_context([part], lens, [0, 0], dtype)
        got = part.apply(h.to(dtype).cuda(), ctx, 0, 0, True).float().cpu()
        at = 0
        for n in lens:
            x = h[at:at + n]
            q = (x @ tensors["a.q_proj.weight"].T + tensors["a.q_proj.bias"]).view(n, nh, hd)
            k = (x @ tensors["a.k_proj.weight"].T + tensors["a.k_proj.bias"]).view(n, nkv, hd)
            v = (x @ tensors["a.v_proj.weight"].T + tensors["a.v_proj.bias"]).view(n, nkv, hd)
            if isinstance(position, RotaryHalfSpec):
                cos, sin = plain.rope_angles(torch.arange(n), hd, 5e4)
                q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
            a = plain.attention(q * (0.4 / hd ** -0.5), k, v, None)          # the spec's scale, not head_dim^-0.5
            want = a @ tensors["a.o_proj.weight"].T
            tol = 1e-4 if dtype == torch.float32 else 5e-2
            assert torch.allclose(got[at:at + n], want, atol=tol, rtol=tol), float((got[at:at + n] - want).abs().max())
            at += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from pico_engine.config import SwiGLUSpec
    from pico_engine.parts import FEED_FORWARDS, build_part
    g = torch.Generator().manual_seed(1)
    H, I = 48, 200
    t = {"f.gate_proj.weight": torch.randn(I, H, generator=g) * 0.2, "f.up_proj.weight": torch.randn(I, H, generator=g) * 0.2,
         "f.down_proj.weight": torch.randn(H, I, generator=g) * 0.1}
    t = {k: v.bfloat16().float() for k, v in t.items()}
    part = build_part(FEED_FORWARDS, "feed-forward", SwiGLUSpec(H, I, "f."), dtype, "cuda")
    part.take_tensors(lambda n: t[n].to(dtype).cuda())
    h = torch.randn(7, H, generator=g).bfloat16().float()
    want = plain.swiglu(h @ t["f.gate_proj.weight"].T, h @ t["f.up_proj.weight"].T) @ t["f.down_proj.weight"].T
    got = part.apply(h.to(dtype).cuda(), SimpleNamespace(dtype=dtype)).float().cpu()
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol)


def test_layer_block_equals_the_plain_layer():
    from pico_engine.config import config_from_dict
    from pico_engine.parts import Layer
    cfg = dict(TINY_B)
    w = make_weights(cfg, 1, sharp=True)
    plan = config_from_dict(cfg).plan()
    layer = Layer(plan.layers[1], torch.float32, "cuda")                      # a windowed layer
    for part in layer.parts():
        part.take_tensors(lambda n: w[n].cuda())
        part.prepare(256)
    n = 90
    x = torch.randn(n, 96, generator=torch.Generator().manual_seed(2))
    ctx, cache, slots = step_context([layer.mixer], [n], [0], torch.float32)
    xd = x.clone().cuda()
    layer.run(xd, ctx, 0, 0, True)
    cos, sin = plain.rope_angles(torch.arange(n), 32, 1e6)
    want = plain.decoder_layer(cfg, w, 1, x, cos, sin)
    assert torch.allclose(xd.cpu(), want, atol=1e-4, rtol=1e-4)


def test_unknown_part_and_arrangement_are_refused():
    from pico_engine.config import ConfigError, PartSpec, config_from_dict
    from pico_engine.parts import MIXERS, Layer, build_part
    with pytest.raises(ConfigError, match="no mixer is registered"):
        build_part(MIXERS, "mixer", PartSpec(), torch.float32, "cuda")
    spec = replace(config_from_dict(TINY_B).plan().layers[0], arrangement="sandwich")
    with pytest.raises(ConfigError, match="sandwich"):
        Layer(spec, torch.float32, "cuda")


def plain_scheduled(cfg, w, ids, schedule):
    """The plain forward with the order of layer executions as data: ``(layer, cache_of)``; an
    execution with ``cache_of`` attends with its own queries to that earlier execution's keys and values."""
    nh, nkv, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    L = len(ids)
    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    cos, sin = plain.rope_angles(torch.arange(L), hd, cfg["rope_theta"])
    kept = {}
    for e, (i, cache_of) in enumerate(schedule):
        p = f"model.layers.{i}."
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], eps)
        q = plain.apply_rope((h @ w[p + "self_attn.q_proj.weight"].T + w[p + "self_attn.q_proj.bias"]).view(L, nh, hd), cos, sin)
        if cache_of is None:
            k = plain.apply_rope((h @ w[p + "self_attn.k_proj.weight"].T + w[p + "self_attn.k_proj.bias"]).view(L, nkv, hd), cos, sin)
            v = (h @ w[p + "self_attn.v_proj.weight"].T + w[p + "self_attn.v_proj.bias"]).view(L, nkv, hd)
            kept[e] = (k, v)
        else:
            k, v = kept[cache_of]
        x = x + plain.attention(q, k, v, plain.layer_window(cfg, i)) @ w[p + "self_attn.o_proj.weight"].T
        h = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + plain.swiglu(h @ w[p + "mlp.gate_proj.weight"].T, h @ w[p + "mlp.up_proj.weight"].T) @ w[p + "mlp.down_proj.weight"].T
    return plain.rms_norm(x, w["model.norm.weight"], eps) @ w["lm_head.weight"].T


def test_the_order_of_layers_is_data():
    """Layer 0 runs twice (two caches of its own) and the last execution reads the cache of the second."""
    from pico_engine.cache import Cache
    from pico_engine.config import ScheduleEntry, config_from_dict
    from pico_engine.engine.step import Stepper
    from pico_engine.parts import DecoderModel
    cfg = dict(TINY_B)
    w = make_weights(cfg, 4, sharp=True)
    order = [(0, None), (1, None), (0, None), (2, 1)]
    plan = replace(config_from_dict(cfg).plan(), schedule=tuple(ScheduleEntry(l, c) for l, c in order))
    model = DecoderModel(plan, torch.float32, "cuda")
    model.take_tensors(lambda n: w[n].cuda())
    model.prepare(256)
    needs = model.cache_needs()
    assert needs[3] is None and needs[0] == needs[2]
    cache = Cache(needs, 256, 4, torch.float32, "cuda")
    assert [g.entries for g in cache.groups] == [[0, 2], [1]]
    stepper = Stepper(model, cache, 256)
    ids = torch.randint(0, 512, (80,), generator=torch.Generator().manual_seed(5)).tolist()
    s = cache.open()
    first = stepper.step([s], [ids[:50]], [list(range(50))]).cpu()
    rest = torch.cat([stepper.step([s], [[t]]).cpu() for t in ids[50:]])
    want = plain_scheduled(cfg, w, ids, order)
    assert torch.allclose(torch.cat([first, rest]), want, atol=1e-4 * float(want.abs().max()))
    plain_order = plain_scheduled(cfg, w, ids, [(0, None), (1, None), (2, None)])
    assert torch.allclose(plain_order, plain.forward(cfg, w, ids), atol=1e-5)          # the helper is the plain model
    assert not torch.allclose(want, plain_order, atol=1e-2)
