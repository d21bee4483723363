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


# ---------------------------------------------------------------------------- state inside a captured decode step

def define_graph_toy():
    """A second toy architecture: layer 0 is a mixer-only block (no feed-forward, no second norm) whose mixer
    keeps per-sequence state and finds its rows through the context's device arrays alone, so that it can be
    captured in the decode graph; layer 1 is attention with a gated feed-forward."""
    from pico_engine.cache import CacheNeeds
    from pico_engine.config import (LayerSpec, ModelPlan, PartSpec, RMSNormSpec, ScheduleEntry, SwiGLUSpec, GQAAttentionSpec,
                                    NoPositionSpec, register_architecture)
    from pico_engine.parts import Mixer, register_mixer
    from pico_engine.weights import ParamSpec

    @dataclass(frozen=True)
    class DeviceDecaySpec(PartSpec):
        hidden: int
        decay: float
        weight: str

    @register_mixer(DeviceDecaySpec)
    class DeviceDecayMixer(Mixer):
        """s_t = decay * s_{t-1} + h_t per sequence, y_t = W s_t, for any mix of rows: only device arrays are read
        (``tok_row``, ``row_first``, ``slots``), as a kernel would, so the same code runs eagerly and in a graph."""

        def expected_tensors(self):
            return {self.spec.weight: ParamSpec((self.spec.hidden, self.spec.hidden))}

        def take_tensors(self, get):
            self.w = get(self.spec.weight)

        def cache_needs(self):
            return CacheNeeds(kv=None, state_elems=self.spec.hidden)

        def apply(self, h, ctx, entry, cache_entry, owns_cache):
            state, d = ctx.state(cache_entry), self.spec.decay
            T = h.shape[0]
            row = ctx.tok_row.long()
            t = torch.arange(T, device=h.device)
            local = t - ctx.row_first.long()[row]                                   # index of a token within its row
            same = (row[:, None] == row[None, :]) & (t[:, None] >= t[None, :])
            power = (t[:, None] - t[None, :]).clamp(min=0).float()
            weights = torch.where(same, torch.pow(d, power), 0.0)
            start = state.index_select(0, ctx.slots.long())                         # [B, hidden]
            s = weights @ h.float() + torch.pow(d, (local + 1).float())[:, None] * start[row]
            last = ctx.row_first.long()[1:] - 1                                     # each row's last token
            state.index_copy_(0, ctx.slots.long(), s.index_select(0, last))
            return (s @ self.w.float().T).to(ctx.dtype)

    @dataclass(frozen=True)
    class GraphToyConfig:
        ARCHITECTURE = "GraphToyForTests"
        vocab_size: int = 50
        hidden: int = 32

        def plan(self):
            H = self.hidden
            norm = lambda n: RMSNormSpec(H, 1e-5, n)
            attn = GQAAttentionSpec(hidden=H, n_heads=2, n_kv_heads=1, head_dim=16, qkv_bias=False, window=None,
                                    scale=0.25, position=NoPositionSpec(), prefix="l1.attn.")
            layers = (LayerSpec(DeviceDecaySpec(H, 0.9, "l0.mix"), norm("l0.n1")),             # a mixer-only block
                      LayerSpec(attn, norm("l1.n1"), SwiGLUSpec(H, 40, "l1.mlp."), norm("l1.n2")))
            return ModelPlan("GraphToyForTests", self.vocab_size, H, "emb", layers, (ScheduleEntry(0), ScheduleEntry(1)),
                             norm("final"), None, 512)

    register_architecture("GraphToyForTests", GraphToyConfig)
    return GraphToyConfig


def plain_graph_toy(w, ids, H=32):
    import plain_qwen2 as plain
    L = len(ids)
    x = w["emb"][torch.tensor(ids)]
    h = plain.rms_norm(x, w["l0.n1"], 1e-5)
    s, rows = torch.zeros(H), []
    for t in range(L):
        s = 0.9 * s + h[t]
        rows.append(s)
    x = x + torch.stack(rows) @ w["l0.mix"].T                                      # no feed-forward in this block
    h = plain.rms_norm(x, w["l1.n1"], 1e-5)
    q = (h @ w["l1.attn.q_proj.weight"].T).view(L, 2, 16)
    k = (h @ w["l1.attn.k_proj.weight"].T).view(L, 1, 16)
    v = (h @ w["l1.attn.v_proj.weight"].T).view(L, 1, 16)
    x = x + plain.attention(q, k, v, None) @ w["l1.attn.o_proj.weight"].T
    h = plain.rms_norm(x, w["l1.n2"], 1e-5)
    x = x + plain.swiglu(h @ w["l1.mlp.gate_proj.weight"].T, h @ w["l1.mlp.up_proj.weight"].T) @ w["l1.mlp.down_proj.weight"].T
    return plain.rms_norm(x, w["final"], 1e-5) @ w["emb"].T


def test_state_survives_graph_capture_in_a_mixer_only_block():
    """Greedy generation through the entry point with CUDA graphs: capturing a decode step runs it several times
    on trial, which must not advance a mixer's state; the graphs are those of row buckets, so some rows are idle."""
    from pico_engine.engine.engine import Engine
    from pico_engine.weights import random_tensor
    Toy = define_graph_toy()
    eng = Engine.from_config(Toy(), seed=5, dtype="float32")
    assert eng.model.layers[0].feed_forward is None and len(eng.model.layers[0].parts()) == 2
    expected = eng.model.expected_tensors()
    w = {n: random_tensor(n, s, 5, torch.bfloat16).float() for n, s in expected.items()}
    sharp = {n: t * (8.0 if expected[n].init == "normal" else 1.0) for n, t in w.items()}
    eng.model.take_tensors(lambda n: sharp[n].to("cuda"))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 50, (n,), generator=g).tolist() for n in (7, 20, 3)]
    budgets = [9, 4, 12]

    def plain_generate(p, n):
        out = []
        for _ in range(n):
            out.append(int(plain_graph_toy(sharp, p + out)[-1].argmax()))
        return out
    want = [plain_generate(p, n) for p, n in zip(prompts, budgets)]
    eager = eng.generate(prompts, max_tokens=budgets, temperature=0.0, use_graph=False, stop_token_ids=())
    graphed = eng.generate(prompts, max_tokens=budgets, temperature=0.0, use_graph=True, stop_token_ids=())
    assert eager == want and graphed == want
    assert sorted(k[0] for k in eng._graphs) == [1, 2, 4]        # 3 rows ran in the graph of 4, one of them idle
