"""A toy mixer with per-sequence state of its own, a toy routed feed-forward and a toy position
encoding, all defined here, are registered, built and stepped without touching the library's files."""
from dataclasses import dataclass

import pytest
import torch

pytestmark = pytest.mark.gpu


def define_toy():
    from pico_engine.cache import CacheNeeds
    from pico_engine.config import (LayerSpec, ModelPlan, PartSpec, RMSNormSpec, ScheduleEntry, SwiGLUSpec, GQAAttentionSpec,
                                    register_architecture)
    from pico_engine.parts import FeedForward, Mixer, Position, register_feed_forward, register_mixer, register_position
    from pico_engine.ops import kernels
    from pico_engine.weights import ParamSpec

    @dataclass(frozen=True)
    class DecaySpec(PartSpec):
        """y_t = W s_t with s_t = decay * s_{t-1} + h_t: a state of ``hidden`` numbers per sequence."""
        hidden: int
        decay: float
        weight: str

    @register_mixer(DecaySpec)
    class DecayMixer(Mixer):
        def expected_tensors(self):
            return {self.spec.weight: ParamSpec((self.spec.hidden, self.spec.hidden))}

        def take_tensors(self, get):
            self.w = get(self.spec.weight)

        def cache_needs(self):
            return CacheNeeds(kv=None, state_elems=self.spec.hidden)

        def apply(self, h, ctx, entry, cache_entry, owns_cache):
            state = ctx.state(cache_entry)
            out = torch.empty(h.shape, dtype=torch.float32, device=h.device)
            at = 0
            for slot, n in zip(ctx.slot_ids, ctx.lens):
                s = state[slot].clone()
                for t in range(at, at + n):
                    s = self.spec.decay * s + h[t].float()
                    out[t] = s
                state[slot] = s
                at += n
            return (out @ self.w.float().T).to(ctx.dtype)

    @dataclass(frozen=True)
    class Top1Spec(PartSpec):
        """Two experts (plain matrices); each token goes to the one with the larger router logit."""
        hidden: int
        prefix: str

    @register_feed_forward(Top1Spec)
    class Top1FeedForward(FeedForward):
        def expected_tensors(self):
            H = self.spec.hidden
            return {self.spec.prefix + "router": ParamSpec((2, H)), self.spec.prefix + "experts": ParamSpec((2 * H, H))}

        def take_tensors(self, get):
            self.router, self.experts = get(self.spec.prefix + "router"), get(self.spec.prefix + "experts")

        def apply(self, h, ctx):
            H = self.spec.hidden
            choice = (h.float() @ self.router.float().T).argmax(dim=-1)              # router logits in 32-bit
            both = (h.float() @ self.experts.float().T).view(-1, 2, H)
            return both[torch.arange(h.shape[0]), choice].to(ctx.dtype)

    @dataclass(frozen=True)
    class SignFlipSpec(PartSpec):
        """Odd positions negate queries and keys: a position encoding that is no rotation."""

    @register_position(SignFlipSpec)
    class SignFlip(Position):
        def rotate_and_store(self, qkv, n_q, n_kv, head_dim, ctx, kv):
            sign = (1 - 2 * (ctx.tok_pos % 2)).to(qkv.dtype)[:, None]
            qkv[:, :(n_q + n_kv) * head_dim] *= sign
            if kv is not None:                                                         # the library's store-only kernel
                kernels.rope_store(qkv, n_q, n_kv, head_dim, None, None, ctx.tok_pos, ctx.tok_row, kv.k, kv.v, kv.table, kv.stride)

    @dataclass(frozen=True)
    class ToyConfig:
        ARCHITECTURE = "ToyForTests"
        vocab_size: int = 50
        hidden: int = 32

        def plan(self):
            H = self.hidden
            norm = lambda n: RMSNormSpec(H, 1e-5, n)
            attn = GQAAttentionSpec(hidden=H, n_heads=2, n_kv_heads=1, head_dim=16, qkv_bias=False, window=None,
                                    scale=0.25, position=SignFlipSpec(), prefix="l1.attn.")
            layers = (LayerSpec(DecaySpec(H, 0.9, "l0.mix"), norm("l0.n1"), Top1Spec(H, "l0.ffn."), norm("l0.n2")),
                      LayerSpec(attn, norm("l1.n1"), SwiGLUSpec(H, 40, "l1.mlp."), norm("l1.n2")))
            return ModelPlan("ToyForTests", self.vocab_size, H, "emb", layers, (ScheduleEntry(0), ScheduleEntry(1)),
                             norm("final"), None, 512)

    register_architecture("ToyForTests", ToyConfig)
    return ToyConfig


def plain_toy(w, ids, H=32):
    """The toy model written out whole, with no cache and no state carried."""
    import plain_qwen2 as plain
    L = len(ids)
    x = w["emb"][torch.tensor(ids)]
    h = plain.rms_norm(x, w["l0.n1"], 1e-5)
    s, rows = torch.zeros(H), []
    for t in range(L):
        s = 0.9 * s + h[t]
        rows.append(s)
    x = x + torch.stack(rows) @ w["l0.mix"].T
    h = plain.rms_norm(x, w["l0.n2"], 1e-5)
    choice = (h @ w["l0.ffn.router"].T).argmax(-1)
    x = x + (h @ w["l0.ffn.experts"].T).view(L, 2, H)[torch.arange(L), choice]
    h = plain.rms_norm(x, w["l1.n1"], 1e-5)
    sign = (1 - 2 * (torch.arange(L) % 2)).float()[:, None, None]
    q = (h @ w["l1.attn.q_proj.weight"].T).view(L, 2, 16) * sign
    k = (h @ w["l1.attn.k_proj.weight"].T).view(L, 1, 16) * sign
    v = (h @ w["l1.attn.v_proj.weight"].T).view(L, 1, 16)
    x = x + plain.attention(q, k, v, None) @ w["l1.attn.o_proj.weight"].T
    h = plain.rms_norm(x, w["l1.n2"], 1e-5)
    x = x + plain.swiglu(h @ w["l1.mlp.gate_proj.weight"].T, h @ w["l1.mlp.up_proj.weight"].T) @ w["l1.mlp.down_proj.weight"].T
    return plain.rms_norm(x, w["final"], 1e-5) @ w["emb"].T


def test_toy_parts_are_registered_built_and_stepped():
    from pico_engine.cache import Cache
    from pico_engine.config import architecture
    from pico_engine.engine.step import Stepper
    from pico_engine.weights import load_into, random_tensor
    Toy = define_toy()
    model = architecture("ToyForTests").build_model(Toy(), torch.float32, "cuda")
    expected = model.expected_tensors()
    w = {n: random_tensor(n, s, 3, torch.float32) * (8.0 if s.init == "normal" else 1.0) for n, s in expected.items()}
    load_into(model, lambda n: w[n], {n: s.shape for n, s in expected.items()}, "toy weights")
    model.prepare(512)
    needs = model.cache_needs()
    assert needs[0].kv is None and needs[0].state_elems == 32 and needs[1].kv is not None
    cache = Cache(needs, 512, 3, torch.float32, "cuda")
    stepper = Stepper(model, cache, 512)
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, 50, (n,), generator=g).tolist() for n in (70, 9, 33)]
    want = [plain_toy(w, s) for s in seqs]
    # a batch of unequal prompts in one step, then one token each
    slots = [cache.open() for _ in seqs]
    heads = [40, 4, 33]
    got = [[] for _ in seqs]
    first = stepper.step(slots, [s[:h] for s, h in zip(seqs, heads)], [list(range(h)) for h in heads]).cpu()
    at = 0
    for i, h in enumerate(heads):
        got[i].append(first[at:at + h]); at += h
    pos = list(heads)
    while any(p < len(s) for p, s in zip(pos, seqs)):
        live = [i for i in range(3) if pos[i] < len(seqs[i])]
        out = stepper.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live]).cpu()
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1]); pos[i] += 1
    for i in range(3):
        assert torch.allclose(torch.cat(got[i]), want[i], atol=2e-4 * float(want[i].abs().max())), i
    # the state of a slot that is used again starts from zero
    for s in slots:
        cache.close(s)
    again = cache.open()
    assert again == slots[0] and float(cache.state_of(0)[again].abs().sum()) == 0.0
    out = stepper.step([again], [seqs[1]], [list(range(9))]).cpu()
    assert torch.allclose(out, want[1], atol=2e-4 * float(want[1].abs().max()))
    cache.close(again)
