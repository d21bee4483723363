"""Each CUDA kernel alone against the plain float32 formulas, at sizes other than the engine's."""
import math
import os
import random

import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

DT = {"f32": torch.float32, "bf16": torch.bfloat16}


@pytest.fixture(scope="module")
def K():
    from pico_engine.ops import kernels
    return kernels


def dev(t):
    return t.to("cuda")


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def bf(t):
    """Values rounded to bfloat16, kept in float32."""
    return t.to(torch.bfloat16).to(torch.float32)


# ---------------------------------------------------------------------------- small kernels

@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_embed(K, dtype):
    table = bf(rnd(1000, 200))
    ids = torch.tensor([0, 999, 5, 5, 321], dtype=torch.int32)
    out = K.embed(dev(table.to(DT[dtype])), dev(ids))
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), table[ids.long()])


@pytest.mark.parametrize("H", [100, 896, 3584])
@pytest.mark.parametrize("wdtype,odtype", [("f32", "f32"), ("bf16", "bf16"), ("f32", "bf16")])
def test_rmsnorm(K, H, wdtype, odtype):
    x, w = rnd(7, H, seed=1, scale=3.0), bf(1 + rnd(H, seed=2) * 0.1)
    want = plain.rms_norm(x, w, 1e-5)
    got = K.rmsnorm(dev(x), dev(w.to(DT[wdtype])), 1e-5, DT[odtype])
    tol = 1e-5 if odtype == "f32" else 2e-2
    assert got.dtype == DT[odtype] and torch.allclose(got.float().cpu(), want, atol=tol, rtol=tol)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    got = K.rmsnorm(dev(x), dev(w.to(DT[wdtype])), 1e-5, DT[odtype], dev(rows))
    assert torch.allclose(got.float().cpu(), want[rows.long()], atol=tol, rtol=tol)


@pytest.mark.parametrize("H", [100, 896, 2052, 5120])
@pytest.mark.parametrize("ydtype", ["f32", "bf16"])
def test_add_rmsnorm(K, H, ydtype):
    """The residual sum and the norm in one pass: x is updated in place, the norm is of the sum.
    2052 and 5120 columns leave a thread more groups than it keeps in registers."""
    x, y, w = rnd(9, H, seed=1, scale=3.0), bf(rnd(9, H, seed=4)), bf(1 + rnd(H, seed=2) * 0.1)
    xd = dev(x.clone())
    got = K.add_rmsnorm(xd, dev(y.to(DT[ydtype])), dev(w.to(torch.bfloat16)), 1e-6, torch.bfloat16)
    assert torch.allclose(xd.cpu(), x + y, atol=1e-6)
    assert torch.allclose(got.float().cpu(), plain.rms_norm(x + y, w, 1e-6), atol=2e-2, rtol=2e-2)
    # the same numbers as the two kernels one after the other
    xs = K.residual_add(dev(x.clone()), dev(y.to(DT[ydtype])))
    assert torch.equal(got, K.rmsnorm(xs, dev(w.to(torch.bfloat16)), 1e-6, torch.bfloat16))


@pytest.mark.parametrize("H", [100, 896, 1024, 1028])
@pytest.mark.parametrize("rows", [2601, 4100])
def test_rmsnorm_of_many_rows(K, H, rows):
    """More rows than the device holds blocks at once; from 4,096 rows on a warp takes a row."""
    x, y, w = rnd(rows, H, seed=1, scale=3.0), bf(rnd(rows, H, seed=4)), bf(1 + rnd(H, seed=2) * 0.1)
    for odtype, tol in (("f32", 1e-5), ("bf16", 2e-2)):
        got = K.rmsnorm(dev(x), dev(w), 1e-6, DT[odtype])
        assert torch.allclose(got.float().cpu(), plain.rms_norm(x, w, 1e-6), atol=tol, rtol=tol)
    xd = dev(x.clone())
    got = K.add_rmsnorm(xd, dev(y.to(torch.bfloat16)), dev(w.to(torch.bfloat16)), 1e-6, torch.bfloat16)
    assert torch.allclose(xd.cpu(), x + y, atol=1e-6)
    assert torch.allclose(got.float().cpu(), plain.rms_norm(x + y, w, 1e-6), atol=2e-2, rtol=2e-2)


def test_rmsnorm_eps_matters(K):
    x, w = torch.full((1, 64), 1e-3), torch.ones(64)
    for eps in (1e-6, 1e-2):
        got = K.rmsnorm(dev(x), dev(w), eps, torch.float32).cpu()
        assert torch.allclose(got, plain.rms_norm(x, w, eps), rtol=1e-5)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("T,I", [(5, 352), (3, 4864), (700, 1000)])
def test_swiglu(K, dtype, T, I):
    gu = bf(rnd(T, 2 * I, seed=3, scale=2.0))
    want = plain.swiglu(gu[:, :I], gu[:, I:])
    got = K.swiglu(dev(gu.to(DT[dtype])))
    assert torch.allclose(got.float().cpu(), want, atol=1e-5 if dtype == "f32" else 3e-2, rtol=1e-5 if dtype == "f32" else 1e-2)


def test_residual_and_bias_add(K):
    x, y, b = rnd(6, 50, seed=1), bf(rnd(6, 50, seed=2)), rnd(50, seed=3)
    got = K.residual_add(dev(x.clone()), dev(y.to(torch.bfloat16)))
    assert torch.allclose(got.cpu(), x + y, atol=1e-6)
    got = K.bias_add(dev(y.clone()), dev(b))
    assert torch.allclose(got.cpu(), y + b, atol=1e-6)


# ---------------------------------------------------------------------------- paged cache helpers

PAGE = 64


class Paged:
    """Keys and values of a few sequences scattered over shuffled pages of a pool."""

    def __init__(self, lens, nkv, hd, dtype, seed=0, extra_pages=3):
        g = torch.Generator().manual_seed(seed)
        self.lens, self.nkv, self.hd = lens, nkv, hd
        self.k = [bf(torch.randn(n, nkv, hd, generator=g)) for n in lens]
        self.v = [bf(torch.randn(n, nkv, hd, generator=g)) for n in lens]
        n_pages = sum((n + PAGE - 1) // PAGE for n in lens) + extra_pages
        order = list(range(n_pages))
        random.Random(seed).shuffle(order)
        width = max((n + PAGE - 1) // PAGE for n in lens) + 1
        self.table = torch.full((len(lens), width), -1, dtype=torch.int32)
        self.k_pool = torch.full((n_pages, nkv, PAGE, hd), 7.0)      # finite rubbish where nothing was written
        self.v_pool = torch.full((n_pages, nkv, PAGE, hd), -7.0)
        for b, n in enumerate(lens):
            for pi in range((n + PAGE - 1) // PAGE):
                self.table[b, pi] = order.pop()
        self.dtype = dtype
        self.write()

    def write(self):
        for b, n in enumerate(self.lens):
            for pos in range(n):
                pg = int(self.table[b, pos // PAGE])
                self.k_pool[pg, :, pos % PAGE] = self.k[b][pos]
                self.v_pool[pg, :, pos % PAGE] = self.v[b][pos]

    def cuda(self):
        return dev(self.k_pool.to(self.dtype)), dev(self.v_pool.to(self.dtype)), dev(self.table)


def attention_error(got, want, what=""):
    """The largest error of a bfloat16 attention result against the float64 reference on the same
    bfloat16-rounded inputs, relative to 1 + |reference|.  What a correct kernel leaves: the rounding of the
    output (2^-9 of its value) and of the probabilities that enter P.V on the tensor cores (2^-9 each, averaged
    over the keys).  A key left out or counted twice among a few hundred moves an output by a few 1e-3 at least."""
    got, want = got.double().cpu().reshape(-1), want.double().cpu().reshape(-1)
    err = float(((got - want).abs() / (1.0 + want.abs())).max())
    if os.environ.get("PICO_TEST_STATS"):
        with open(os.environ["PICO_TEST_STATS"], "a") as f:
            f.write(f"attention {what} {err:.3e}\n")
    return err


# bfloat16 attention against float64 on the same bfloat16-rounded inputs.  Worst cases measured on a B200 over the
# cases of this file: float32-arithmetic kernel 1.9e-3, decode 2.0e-3 (long sequences 1.6e-3), prefill kernels 4.0e-3
# (their probabilities are rounded to bfloat16 for runs of up to 128 queries, whose outputs are smaller and so
# relatively coarser); the bounds leave a factor of 1.5 to 2 over that.  (They were 2e-2 absolute and relative.)
ATTENTION_BOUND = 4e-3
PREFILL_ATTENTION_BOUND = 6e-3


def reference_attention(q_rows, paged, tok_row, tok_pos, nh, window):
    """q_rows [T, nh, hd]; token t attends keys of sequence tok_row[t] up to tok_pos[t]."""
    out = []
    for t, (b, p) in enumerate(zip(tok_row, tok_pos)):
        L = p + 1
        q = torch.zeros(L, nh, paged.hd)
        q[p] = q_rows[t]
        out.append(plain.attention(q, paged.k[b][:L], paged.v[b][:L], window)[p])
    return torch.stack(out)


def attention_case(nh, nkv, hd, lens, window, seed):
    """Queries for the last token of every sequence plus a few inner ones."""
    tok_row, tok_pos = [], []
    rng = random.Random(seed)
    for b, n in enumerate(lens):
        for p in sorted({n - 1, 0, rng.randrange(n), max(0, n - 2)}):
            tok_row.append(b); tok_pos.append(p)
    q = bf(rnd(len(tok_row), nh, hd, seed=seed + 1))
    return q, tok_row, tok_pos


CASES = [  # nh, nkv, hd, lens, window
    (4, 2, 16, [5, 70, 129], None),
    (3, 1, 32, [64, 1, 200], 32),
    (14, 2, 64, [300, 65], None),
    (6, 6, 48, [100], 17),
    (5, 1, 128, [130, 40], 64),
    (20, 1, 80, [90], None),
]


@pytest.mark.parametrize("nh,nkv,hd,lens,window", CASES)
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_attention_generic(K, nh, nkv, hd, lens, window, dtype):
    paged = Paged(lens, nkv, hd, DT[dtype], seed=hd)
    q, tok_row, tok_pos = attention_case(nh, nkv, hd, lens, window, seed=nh)
    kp, vp, table = paged.cuda()
    got = K.attention_generic(dev(q.reshape(len(tok_row), -1).to(DT[dtype])), nh * hd, nh, nkv, hd, kp, vp, table,
                              table.shape[1], dev(torch.tensor(tok_pos, dtype=torch.int32)),
                              dev(torch.tensor(tok_row, dtype=torch.int32)), window, hd ** -0.5)
    want = reference_attention(q, paged, tok_row, tok_pos, nh, window)
    if dtype == "f32":
        assert torch.allclose(got.cpu(), want, atol=2e-5, rtol=2e-5), float((got.cpu() - want).abs().max())
    else:                                                   # float32 arithmetic, the result rounded to bfloat16
        err = attention_error(got, one_query_attention(q, paged, tok_row, tok_pos, nh, window), "generic")
        assert err < ATTENTION_BOUND, err


@pytest.mark.parametrize("nh,nkv,hd,lens,window", CASES)
@pytest.mark.parametrize("max_context", [None, 4096])
def test_attention_decode(K, nh, nkv, hd, lens, window, max_context):
    paged = Paged(lens, nkv, hd, torch.bfloat16, seed=hd + 1)
    q, tok_row, tok_pos = attention_case(nh, nkv, hd, lens, window, seed=nh + 7)
    kp, vp, table = paged.cuda()
    # queries sit inside a wider row, as they do in the fused q/k/v buffer
    stride = (nh + 2 * nkv) * hd
    buf = torch.zeros(len(tok_row), stride)
    buf[:, :nh * hd] = q.reshape(len(tok_row), -1)
    got = K.attention_decode(dev(buf.to(torch.bfloat16)), stride, nh, nkv, hd, kp, vp, table, table.shape[1],
                             dev(torch.tensor(tok_pos, dtype=torch.int32)), dev(torch.tensor(tok_row, dtype=torch.int32)),
                             window, hd ** -0.5, max_context or max(lens))
    assert torch.allclose(reference_attention(q, paged, tok_row, tok_pos, nh, window).double().reshape(len(tok_row), -1),
                          one_query_attention(q, paged, tok_row, tok_pos, nh, window).reshape(len(tok_row), -1), atol=1e-5)
    err = attention_error(got, one_query_attention(q, paged, tok_row, tok_pos, nh, window), "decode")
    assert err < ATTENTION_BOUND, err
    # started only when everything before it has ended (for callers that rewrite other cache rows): the same numbers
    late = K.attention_decode(dev(buf.to(torch.bfloat16)), stride, nh, nkv, hd, kp, vp, table, table.shape[1],
                              dev(torch.tensor(tok_pos, dtype=torch.int32)), dev(torch.tensor(tok_row, dtype=torch.int32)),
                              window, hd ** -0.5, max_context or max(lens), early_pages=False)
    assert torch.equal(late, got)


def one_query_attention(q_rows, paged, tok_row, tok_pos, nh, window):
    """The rows of ``reference_attention`` computed one query at a time (long sequences)."""
    out = []
    G = nh // paged.nkv
    for t, (b, p) in enumerate(zip(tok_row, tok_pos)):
        lo = 0 if not window else max(0, p - window + 1)
        k = paged.k[b][lo:p + 1].repeat_interleave(G, dim=1)          # [L, nh, hd]
        v = paged.v[b][lo:p + 1].repeat_interleave(G, dim=1)
        s = torch.einsum("hd,lhd->hl", q_rows[t].double(), k.double()) * paged.hd ** -0.5
        out.append(torch.einsum("hl,lhd->hd", torch.softmax(s, dim=-1), v.double()))
    return torch.stack(out)


LONG_CASES = [                        # (nh, nkv, hd, lens, window): what each is there for
    (4, 2, 64, [3000, 700], None),    # eight page ranges a sequence, merged across the cluster
    (16, 8, 128, [1100] * 20, None),  # one CTA a sequence and kv head: its ring of pages wraps several times
    (4, 1, 32, [2500], 1000),         # a window that starts in the middle of a page, many pages back
    (8, 4, 256, [1500] * 10, None),   # three ranges a sequence, a ring of two pages
    (7, 1, 64, [4096, 4033, 65], None),
]


@pytest.mark.parametrize("nh,nkv,hd,lens,window", LONG_CASES)
def test_attention_decode_long(K, nh, nkv, hd, lens, window):
    paged = Paged(lens, nkv, hd, torch.bfloat16, seed=hd + 3)
    q, tok_row, tok_pos = attention_case(nh, nkv, hd, lens, window, seed=nh + 9)
    small = [i for i, p in enumerate(tok_pos) if p < 80]              # the two references agree where both are cheap
    if small:
        a = reference_attention(q[small], paged, [tok_row[i] for i in small], [tok_pos[i] for i in small], nh, window)
        b = one_query_attention(q[small], paged, [tok_row[i] for i in small], [tok_pos[i] for i in small], nh, window)
        assert torch.allclose(a.reshape(b.shape).double(), b, atol=1e-5)
    kp, vp, table = paged.cuda()
    for repeat in range(2):                                            # the second launch finds the barriers' memory used
        got = K.attention_decode(dev(q.reshape(len(tok_row), -1).to(torch.bfloat16)), nh * hd, nh, nkv, hd, kp, vp, table,
                                 table.shape[1], dev(torch.tensor(tok_pos, dtype=torch.int32)),
                                 dev(torch.tensor(tok_row, dtype=torch.int32)), window, hd ** -0.5, max(lens))
        K.check_status("cuda")
        want = one_query_attention(q, paged, tok_row, tok_pos, nh, window).reshape(len(tok_row), -1)
        err = ((got.double().cpu() - want).abs() / (1.0 + want.abs())).max(dim=1).values
        attention_error(got, want, "decode_long")
        assert float(err.max()) < ATTENTION_BOUND, (float(err.max()), tok_row[int(err.argmax())], tok_pos[int(err.argmax())])


@pytest.mark.parametrize("nh,nkv,hd,lens,window", CASES)
@pytest.mark.parametrize("cached", [0, 37])
def test_attention_prefill(K, nh, nkv, hd, lens, window, cached):
    """Every token of every sequence from position ``cached`` on, in one launch."""
    paged = Paged(lens, nkv, hd, torch.bfloat16, seed=hd + 2)
    starts = [min(cached, n - 1) for n in lens]
    step_lens = [n - s for n, s in zip(lens, starts)]
    tok_row = [b for b, n in enumerate(step_lens) for _ in range(n)]
    tok_pos = [s + i for s, n in zip(starts, step_lens) for i in range(n)]
    q = bf(rnd(len(tok_row), nh, hd, seed=5))
    kp, vp, table = paged.cuda()
    tiles = K.prefill_tiles(step_lens, starts, "cuda")
    got = K.attention_prefill(dev(q.reshape(len(tok_row), -1).to(torch.bfloat16)), nh * hd, nh, nkv, hd, kp, vp, table,
                              table.shape[1], tiles, len(tok_row), window, hd ** -0.5)
    want = one_query_attention(q, paged, tok_row, tok_pos, nh, window).reshape(len(tok_row), -1)
    err = ((got.double().cpu() - want).abs() / (1.0 + want.abs())).max(dim=1).values
    attention_error(got, want, "prefill")
    assert float(err.max()) < PREFILL_ATTENTION_BOUND, (float(err.max()), int(err.argmax()), tok_row[int(err.argmax())], tok_pos[int(err.argmax())])


TCGEN05_CASES = [  # nh, nkv, hd, lens, window
    (14, 2, 64, [300, 65], None),
    (5, 1, 128, [130, 40], 64),
    (3, 3, 64, [1, 128, 129, 7], None),       # runs of exactly one tile, one token more, and of a single token
    (4, 2, 64, [700], 100),                   # a window that leaves whole pages behind inside a run's range
    (2, 1, 128, [1000, 333], None),           # the ring of pages wraps many times
    (6, 2, 128, [400], 129),
]


@pytest.mark.parametrize("nh,nkv,hd,lens,window", TCGEN05_CASES)
@pytest.mark.parametrize("cached", [0, 37])
def test_attention_prefill_tcgen05(K, nh, nkv, hd, lens, window, cached):
    """The tcgen05 kernel (runs of 128 tokens, S and O in tensor memory), with q as a strided view
    of a wider matrix, as the engine hands it over."""
    paged = Paged(lens, nkv, hd, torch.bfloat16, seed=hd + 4)
    starts = [min(cached, n - 1) for n in lens]
    step_lens = [n - s for n, s in zip(lens, starts)]
    tok_row = [b for b, n in enumerate(step_lens) for _ in range(n)]
    tok_pos = [s + i for s, n in zip(starts, step_lens) for i in range(n)]
    q = bf(rnd(len(tok_row), nh, hd, seed=6))
    kp, vp, table = paged.cuda()
    wide = torch.zeros(len(tok_row), (nh + 2 * nkv) * hd, dtype=torch.bfloat16, device="cuda")
    wide[:, :nh * hd] = dev(q.reshape(len(tok_row), -1).to(torch.bfloat16))
    tiles = K.prefill_tiles(step_lens, starts, "cuda", K.PREFILL_TILE_TCGEN05)
    got = K.attention_prefill_tcgen05(wide, wide.shape[1], nh, nkv, hd, kp, vp, table, table.shape[1], tiles,
                                      len(tok_row), window, hd ** -0.5)
    K.check_status("cuda")
    want = one_query_attention(q, paged, tok_row, tok_pos, nh, window).reshape(len(tok_row), -1)
    err = ((got.double().cpu() - want).abs() / (1.0 + want.abs())).max(dim=1).values
    attention_error(got, want, "prefill")
    assert float(err.max()) < PREFILL_ATTENTION_BOUND, (float(err.max()), int(err.argmax()), tok_row[int(err.argmax())], tok_pos[int(err.argmax())])


@pytest.mark.parametrize("kernel", ["generic_f32", "generic_bf16", "decode", "prefill", "prefill_tcgen05"])
def test_attention_finds_a_far_key_and_respects_the_windows_edge(K, kernel):
    """One key among hundreds is made to dominate.  Without a window the output must be its
    value; with a window ending just before it, it must not show; with one that just includes it, it must."""
    nh, nkv, hd, n = 4, 2, (64 if kernel == "prefill_tcgen05" else 32), 333
    dtype = torch.float32 if kernel == "generic_f32" else torch.bfloat16
    far = 70                                                  # on the second page
    for window, visible in ((None, True), (n - far, True), (n - far - 1, False)):
        paged = Paged([n], nkv, hd, dtype, seed=11)
        q = bf(rnd(1, nh, hd, seed=12))
        paged.k[0][far, 1] = bf(30.0 * q[0, 3] / q[0, 3].norm())          # head 3 reads kv head 1
        paged.write()
        kp, vp, table = paged.cuda()
        pos, row = dev(torch.tensor([n - 1], dtype=torch.int32)), dev(torch.tensor([0], dtype=torch.int32))
        qd = dev(q.reshape(1, -1).to(dtype))
        if kernel.startswith("generic"):
            got = K.attention_generic(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1], pos, row, window, 1.0)
        elif kernel == "decode":
            got = K.attention_decode(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1], pos, row, window, 1.0, 512)
        elif kernel == "prefill":
            tiles = K.prefill_tiles([1], [n - 1], "cuda")
            got = K.attention_prefill(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1], tiles, 1, window, 1.0)
        else:
            tiles = K.prefill_tiles([1], [n - 1], "cuda", K.PREFILL_TILE_TCGEN05)
            got = K.attention_prefill_tcgen05(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1], tiles, 1, window, 1.0)
            K.check_status("cuda")
        head3 = got.float().cpu().view(nh, hd)[3]
        hit = torch.allclose(head3, paged.v[0][far, 1], atol=3e-2)
        assert hit == visible, (kernel, window, head3[:4], paged.v[0][far, 1][:4])


def _attend_last(K, kernel, paged, q, n, nh, nkv, hd, window=None):
    """The last token's attention with the named kernel; q [1, nh, hd]."""
    dtype = torch.float32 if kernel == "generic_f32" else torch.bfloat16
    kp, vp, table = paged.cuda()
    pos, row = dev(torch.tensor([n - 1], dtype=torch.int32)), dev(torch.tensor([0], dtype=torch.int32))
    qd = dev(q.reshape(1, -1).to(dtype))
    if kernel.startswith("generic"):
        return K.attention_generic(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1], pos, row, window, 1.0)
    if kernel == "decode":
        got = K.attention_decode(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1], pos, row, window, 1.0, n)
    elif kernel == "prefill":
        tiles = K.prefill_tiles([1], [n - 1], "cuda")
        got = K.attention_prefill(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1], tiles, 1, window, 1.0)
    else:
        tiles = K.prefill_tiles([1], [n - 1], "cuda", K.PREFILL_TILE_TCGEN05)
        got = K.attention_prefill_tcgen05(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1], tiles, 1, window, 1.0)
    K.check_status("cuda")
    return got


@pytest.mark.parametrize("kernel", ["generic_bf16", "decode", "prefill", "prefill_tcgen05"])
@pytest.mark.parametrize("n,far", [(333, 0), (333, 63), (333, 64), (333, 127), (333, 128), (333, 255), (333, 256), (333, 332),
                                   (3000, 383), (3000, 384), (3000, 767), (3000, 768), (3000, 2943), (3000, 2944)])
def test_attention_finds_a_key_at_every_edge(K, kernel, n, far):
    """The dominating key stands at the first and the last place of a cache page, of a step of 128 keys, of a range
    of pages that one CTA of a cluster takes (a sequence of 3,000 tokens is dealt to 8 ranges of 6 pages), and at the
    query's own position: a kernel that drops or doubles an edge key gives another head's output."""
    if n > 1000 and kernel not in ("decode", "prefill_tcgen05"):
        pytest.skip("the long case is for the kernels that cut a sequence into ranges and rings")
    nh, nkv, hd = 4, 2, (64 if kernel in ("prefill_tcgen05",) or n > 1000 else 32)
    paged = Paged([n], nkv, hd, torch.bfloat16, seed=21)
    q = bf(rnd(1, nh, hd, seed=22))
    paged.k[0][far, 1] = bf(30.0 * q[0, 3] / q[0, 3].norm())              # head 3 reads kv head 1
    paged.write()
    got = _attend_last(K, kernel, paged, q, n, nh, nkv, hd).float().cpu().view(nh, hd)
    assert torch.allclose(got[3], paged.v[0][far, 1], atol=3e-2), (kernel, far, got[3][:4], paged.v[0][far, 1][:4])
    assert not torch.allclose(got[0], paged.v[0][far, 0], atol=3e-2)      # the other kv head has no such key


@pytest.mark.parametrize("kernel", ["generic_bf16", "prefill", "prefill_tcgen05"])
@pytest.mark.parametrize("j", [1, 63, 64, 100, 127, 128, 191])
def test_attention_causal_edge_inside_a_run(K, kernel, j):
    """All tokens of a sequence in one launch, every query pointing at key j, which dominates: the queries before j
    must not see it (it lies in their own run, one place ahead at the closest), the query at j and those after must."""
    nh, nkv, hd, n = 2, 1, (64 if kernel == "prefill_tcgen05" else 32), 200
    paged = Paged([n], nkv, hd, torch.bfloat16, seed=31)
    direction = bf(rnd(hd, seed=32))
    direction = direction / direction.norm()
    paged.k[0][:, 0] = bf(paged.k[0][:, 0] - (paged.k[0][:, 0] @ direction)[:, None] * direction)    # no other key points there
    paged.k[0][j, 0] = bf(30.0 * direction)
    paged.write()
    q = bf(direction.repeat(n, nh, 1))
    kp, vp, table = paged.cuda()
    tok_pos = dev(torch.arange(n, dtype=torch.int32))
    tok_row = dev(torch.zeros(n, dtype=torch.int32))
    qd = dev(q.reshape(n, -1).to(torch.bfloat16))
    if kernel == "generic_bf16":
        got = K.attention_generic(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1], tok_pos, tok_row, None, 1.0)
    elif kernel == "prefill":
        got = K.attention_prefill(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1], K.prefill_tiles([n], [0], "cuda"),
                                  n, None, 1.0)
    else:
        got = K.attention_prefill_tcgen05(qd, nh * hd, nh, nkv, hd, kp, vp, table, table.shape[1],
                                          K.prefill_tiles([n], [0], "cuda", K.PREFILL_TILE_TCGEN05), n, None, 1.0)
        K.check_status("cuda")
    got = got.float().cpu().view(n, nh, hd)
    hit = [bool(torch.allclose(got[p, 1], paged.v[0][j, 0], atol=3e-2)) for p in range(n)]
    assert hit == [p >= j for p in range(n)], (kernel, j, [p for p in range(n) if hit[p] != (p >= j)][:6])


# ---------------------------------------------------------------------------- rotary encoding and the cache write

@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("nq,nkv,hd,theta", [(4, 2, 16, 1e4), (3, 1, 32, 1e6), (14, 2, 64, 1e6)])
def test_rope_store(K, dtype, nq, nkv, hd, theta):
    lens, starts = [3, 70], [62, 5]                            # rows continue from these lengths; the first crosses a page
    tok_row = [b for b, n in enumerate(lens) for _ in range(n)]
    tok_pos = [s + i for s, n in zip(starts, lens) for i in range(n)]
    T = len(tok_row)
    qkv = bf(rnd(T, (nq + 2 * nkv) * hd, seed=4))
    cos, sin = plain.rope_angles(torch.arange(200), hd, theta)
    table = torch.tensor([[2, 0, -1], [3, 1, 4]], dtype=torch.int32)
    kp = torch.zeros(5, nkv, PAGE, hd, dtype=DT[dtype], device="cuda")
    vp = torch.zeros_like(kp)
    buf = dev(qkv.to(DT[dtype]))
    K.rope_store(buf, nq, nkv, hd, dev(cos), dev(sin), dev(torch.tensor(tok_pos, dtype=torch.int32)),
                 dev(torch.tensor(tok_row, dtype=torch.int32)), kp, vp, dev(table), 3)
    c, s = cos[torch.tensor(tok_pos)], sin[torch.tensor(tok_pos)]
    qk = plain.apply_rope(qkv[:, :(nq + nkv) * hd].view(T, nq + nkv, hd), c, s)
    v = qkv[:, (nq + nkv) * hd:].view(T, nkv, hd)
    tol = 1e-5 if dtype == "f32" else 2e-2
    got = buf.float().cpu()
    assert torch.allclose(got[:, :(nq + nkv) * hd].view(T, nq + nkv, hd), qk, atol=tol, rtol=tol)
    assert torch.equal(got[:, (nq + nkv) * hd:], qkv[:, (nq + nkv) * hd:])
    kc, vc = kp.float().cpu(), vp.float().cpu()
    for t, (b, p) in enumerate(zip(tok_row, tok_pos)):
        pg = int(table[b, p // PAGE])
        assert torch.allclose(kc[pg, :, p % PAGE], qk[t, nq:], atol=tol, rtol=tol), (t, b, p)
        assert torch.equal(vc[pg, :, p % PAGE], v[t])
    assert int((kc != 0).any(dim=-1).sum()) == T * nkv          # nothing else was touched
    # no tables: nothing rotates, keys still reach the cache; no pools: nothing is stored
    buf2 = dev(qkv.to(DT[dtype])); kp.zero_()
    K.rope_store(buf2, nq, nkv, hd, None, None, dev(torch.tensor(tok_pos, dtype=torch.int32)),
                 dev(torch.tensor(tok_row, dtype=torch.int32)), kp, vp, dev(table), 3)
    assert torch.equal(buf2.float().cpu(), qkv) and int((kp != 0).any(dim=-1).sum()) == T * nkv


# ---------------------------------------------------------------------------- matrix products

@pytest.mark.parametrize("M,N,K_", [(1, 70, 45), (3, 64, 64), (77, 130, 96), (5, 1000, 352), (130, 96, 160)])
@pytest.mark.parametrize("adt,wdt", [("f32", "f32"), ("bf16", "bf16"), ("bf16", "f32")])
def test_linear_simt(K, M, N, K_, adt, wdt):
    a, w, b = bf(rnd(M, K_, seed=1)), bf(rnd(N, K_, seed=2)), bf(rnd(N, seed=3))
    want = a.double() @ w.double().T
    A, W = dev(a.to(DT[adt])), dev(w.to(DT[wdt]))
    got = K.linear_simt(A, W, out_dtype=torch.float32)
    assert torch.allclose(got.cpu().double(), want, atol=1e-4, rtol=1e-5)
    got = K.linear_simt(A, W, dev(b), out_dtype=torch.bfloat16)
    assert got.dtype == torch.bfloat16 and torch.allclose(got.float().cpu().double(), want + b.double(), atol=6e-2, rtol=1e-2)
    x = rnd(M, N, seed=4)
    got = K.linear_simt(A, W, dev(b), accumulate_into=dev(x.clone()))
    assert torch.allclose(got.cpu().double(), x.double() + want + b.double(), atol=1e-4, rtol=1e-5)


def test_linear_simt_rows_do_not_depend_on_their_neighbours(K):
    a, w = rnd(70, 352, seed=1), rnd(96, 352, seed=2)
    whole = K.linear_simt(dev(a), dev(w), out_dtype=torch.float32)
    for r in (0, 13, 69):
        assert torch.equal(K.linear_simt(dev(a[r:r + 1]), dev(w), out_dtype=torch.float32)[0], whole[r])


@pytest.mark.parametrize("M", [1, 8, 13, 64])
@pytest.mark.parametrize("N,K_", [(100, 96), (896, 896), (1152, 896), (896, 4864), (9728, 896), (70, 160), (4000, 3584)])
def test_linear_mma(K, M, N, K_):
    a, w, b = bf(rnd(M, K_, seed=1)), bf(rnd(N, K_, seed=2, scale=K_ ** -0.5)), bf(rnd(N, seed=3))
    want = a.double() @ w.double().T
    A, W = dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16))
    assert K.linear_mma_takes(A, W)
    got = K.linear_mma(A, W, out_dtype=torch.float32)
    assert torch.allclose(got.cpu().double(), want, atol=1e-4, rtol=1e-4), float((got.cpu().double() - want).abs().max())
    got = K.linear_mma(A, W, dev(b), out_dtype=torch.bfloat16)
    assert torch.allclose(got.float().cpu().double(), want + b.double(), atol=4e-2, rtol=1e-2)
    x = rnd(M, N, seed=4)
    for _ in range(2):                                             # the tickets of the split ranges are left clean
        got = K.linear_mma(A, W, dev(b), accumulate_into=dev(x.clone()))
        assert torch.allclose(got.cpu().double(), x.double() + want + b.double(), atol=1e-4, rtol=1e-4)


def test_linear_mma_rows_do_not_depend_on_their_neighbours(K):
    a, w = bf(rnd(64, 4864, seed=1)), bf(rnd(896, 4864, seed=2, scale=0.02))
    W = dev(w.to(torch.bfloat16))
    whole = K.linear_mma(dev(a.to(torch.bfloat16)), W, out_dtype=torch.float32)
    for rows in ([5], [0, 63], list(range(20, 29))):
        part = K.linear_mma(dev(a[rows].to(torch.bfloat16)), W, out_dtype=torch.float32)
        assert torch.equal(part, whole[rows])


def test_linear_dispatch(K):
    from pico_engine.ops import linear
    a, w = bf(rnd(200, 96, seed=1)), bf(rnd(130, 96, seed=2))
    want = a @ w.T
    for adt, wdt, tol in (("bf16", "bf16", 5e-2), ("f32", "f32", 1e-4), ("bf16", "f32", 5e-2)):
        got = linear(dev(a.to(DT[adt])), dev(w.to(DT[wdt])), out_dtype=DT[adt])
        assert got.dtype == DT[adt] and torch.allclose(got.float().cpu(), want, atol=tol, rtol=1e-2)
        x = rnd(200, 130, seed=5)
        got = linear(dev(a.to(DT[adt])), dev(w.to(DT[wdt])), dev(w[:, 0].contiguous().to(DT[wdt])), accumulate_into=dev(x.clone()))
        assert torch.allclose(got.cpu(), x + want + w[:, 0], atol=tol, rtol=1e-2)
    got = linear(dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16)), out_dtype=torch.float32)
    assert got.dtype == torch.float32


# ---------------------------------------------------------------------------- sampling

@pytest.mark.parametrize("V", [1000, 151936])
def test_argmax(K, V):
    logits = rnd(5, V, seed=9)
    logits[2, 17] = logits[2, 900] = 50.0                           # equal maxima: the first wins
    logits[3, V - 1] = 60.0
    got = K.argmax(dev(logits)).cpu().tolist()
    assert got == logits.argmax(dim=-1).tolist() and got[2] == 17 and got[3] == V - 1


@pytest.mark.parametrize("V", [257, 5000, 151936])             # 1, 2 and 38 chunks a row
@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.8, 0, 1.0), (0.7, 0, 0.9), (1.3, 5, 1.0),
                                                     (1.0, 40, 0.5), (0.5, 1, 1.0), (2.0, 0, 0.05)])
def test_sample_equals_the_plain_sampler(K, V, temperature, top_k, top_p):
    B = 24
    logits = rnd(B, V, seed=V, scale=3.0)
    request = torch.arange(B, dtype=torch.int32) + 3
    step = torch.arange(B, dtype=torch.int32) * 2
    got = K.sample(dev(logits), temperature, top_k, top_p, 1234, dev(request), dev(step)).cpu().tolist()
    want = [plain.sample(logits[b], temperature, top_k, top_p, plain.uniform_for(1234, int(request[b]), int(step[b])))
            for b in range(B)]
    assert got == want
    again = K.sample(dev(logits), temperature, top_k, top_p, 1234, dev(request), dev(step)).cpu().tolist()
    assert again == got                                            # the kernels leave their state clean
    assert all(abs(K.draw_uniform(1234, r, s) - plain.uniform_for(1234, r, s)) == 0 for r in (0, 5) for s in (0, 9))


def test_sample_draws_do_not_depend_on_the_batch(K):
    logits = rnd(6, 777, seed=1, scale=2.0)
    req, st = torch.tensor([4, 9, 1, 0, 7, 3], dtype=torch.int32), torch.tensor([0, 5, 2, 2, 1, 8], dtype=torch.int32)
    whole = K.sample(dev(logits), 0.9, 0, 0.95, 5, dev(req), dev(st)).cpu()
    for b in (0, 3, 5):
        one = K.sample(dev(logits[b:b + 1]), 0.9, 0, 0.95, 5, dev(req[b:b + 1]), dev(st[b:b + 1])).cpu()
        assert int(one[0]) == int(whole[b])
    hist = torch.zeros(4)
    peaked = torch.tensor([[0.0, math.log(2.0), math.log(4.0), math.log(1.0)]]).repeat(4000, 1)
    draws = K.sample(dev(peaked), 1.0, 0, 1.0, 1, dev(torch.arange(4000, dtype=torch.int32)),
                     dev(torch.zeros(4000, dtype=torch.int32))).cpu()
    for i in range(4):
        hist[i] = (draws == i).sum()
    assert torch.allclose(hist / 4000, torch.tensor([1, 2, 4, 1]) / 8.0, atol=0.03)


# ---------------------------------------------------------------------------- fused decode products

@pytest.mark.parametrize("M", [1, 8, 13, 16])
@pytest.mark.parametrize("N,K_", [(100, 96), (896, 896), (896, 4864), (9728, 896), (70, 160), (5000, 3584),
                                  (40, 9000), (100, 2080),       # K cut into 8 and 3 ranges over a cluster
                                  (4744, 512)])                  # two row tiles a CTA, the last CTA has one
def test_linear_fused(K, M, N, K_):
    a, w, b = bf(rnd(M, K_, seed=1)), bf(rnd(N, K_, seed=2, scale=K_ ** -0.5)), bf(rnd(N, seed=3))
    want = a.double() @ w.double().T
    A, W = dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16))
    assert K.fused_takes(M, W, A)
    got = K.linear_fused(A, W, out_dtype=torch.float32)
    assert torch.allclose(got.cpu().double(), want, atol=1e-4, rtol=1e-4), float((got.cpu().double() - want).abs().max())
    got = K.linear_fused(A, W, dev(b), out_dtype=torch.bfloat16)
    assert torch.allclose(got.float().cpu().double(), want + b.double(), atol=4e-2, rtol=1e-2)
    x = rnd(M, N, seed=4)
    got = K.linear_fused(A, W, dev(b.to(torch.bfloat16)), accumulate_into=dev(x.clone()))
    assert torch.allclose(got.cpu().double(), x.double() + want + b.double(), atol=1e-4, rtol=1e-4)
    # the operand as the RMSNorm of float32 rows
    xs, nw = rnd(M, K_, seed=5, scale=2.0), bf(1 + rnd(K_, seed=6) * 0.1)
    h = plain.rms_norm(xs, nw, 1e-5).to(torch.bfloat16).double()
    for nw_dtype in (torch.bfloat16, torch.float32):
        got = K.linear_fused(None, W, out_dtype=torch.float32, norm_of=dev(xs), norm_weight=dev(nw.to(nw_dtype)), eps=1e-5)
        assert torch.allclose(got.cpu().double(), h @ w.double().T, atol=3e-2, rtol=1e-2)   # a bfloat16 rounding of h may flip


def test_linear_fused_rows_do_not_depend_on_their_neighbours(K):
    a, w = bf(rnd(16, 4864, seed=1)), bf(rnd(896, 4864, seed=2, scale=0.02))
    W = dev(w.to(torch.bfloat16))
    whole = K.linear_fused(dev(a.to(torch.bfloat16)), W, out_dtype=torch.float32)
    for rows in ([5], [0, 15], list(range(3, 12))):
        assert torch.equal(K.linear_fused(dev(a[rows].to(torch.bfloat16)), W, out_dtype=torch.float32), whole[rows])


@pytest.mark.parametrize("M,H,I", [(1, 64, 160), (8, 896, 4864), (16, 96, 352), (5, 3584, 1000), (13, 512, 2504),
                                   (16, 896, 4864)])           # the last three take two row tiles a CTA; 2504 / 8 is odd
def test_norm_gate_up_swiglu(K, M, H, I):
    x, nw = rnd(M, H, seed=1, scale=2.0), bf(1 + rnd(H, seed=2) * 0.1)
    w = bf(rnd(2 * I, H, seed=3, scale=H ** -0.5))
    h = plain.rms_norm(x, nw, 1e-6).to(torch.bfloat16).float()
    gu = (h @ w.T).to(torch.bfloat16).float()
    want = plain.swiglu(gu[:, :I], gu[:, I:])
    got = K.norm_gate_up_swiglu(dev(x), dev(nw.to(torch.bfloat16)), 1e-6, dev(w.to(torch.bfloat16)))
    assert got.shape == (M, I) and torch.allclose(got.float().cpu(), want, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("nq,nkv,hd,H,theta,rotate", [(4, 2, 16, 64, 1e4, True), (3, 1, 32, 96, 1e6, True),
                                                       (14, 2, 64, 896, 1e6, True), (5, 5, 48, 240, 1e4, False)])
def test_norm_qkv_rope_store(K, nq, nkv, hd, H, theta, rotate):
    lens, starts = [1] * 7, [62, 5, 63, 64, 0, 130, 17]           # seven sequences, one token each
    M = len(lens)
    x, nw = rnd(M, H, seed=1, scale=2.0), bf(1 + rnd(H, seed=2) * 0.1)
    w, b = bf(rnd((nq + 2 * nkv) * hd, H, seed=3, scale=H ** -0.5)), bf(rnd((nq + 2 * nkv) * hd, seed=4, scale=0.3))
    cos, sin = plain.rope_angles(torch.arange(200), hd, theta)
    table = torch.arange(M * 3, dtype=torch.int32).flip(0).view(M, 3).contiguous()
    kp = torch.zeros(M * 3, nkv, PAGE, hd, dtype=torch.bfloat16, device="cuda")
    vp = torch.zeros_like(kp)
    pos, row = torch.tensor(starts, dtype=torch.int32), torch.arange(M, dtype=torch.int32)
    q = K.norm_qkv_rope_store(dev(x), dev(nw.to(torch.bfloat16)), 1e-6, dev(w.to(torch.bfloat16)), dev(b.to(torch.bfloat16)),
                              nq, nkv, hd, dev(cos) if rotate else None, dev(sin) if rotate else None, dev(pos), dev(row),
                              kp, vp, dev(table), 3)
    h = plain.rms_norm(x, nw, 1e-6).to(torch.bfloat16).float()
    qkv = (h @ w.T + b).to(torch.bfloat16).float()
    qk = qkv[:, :(nq + nkv) * hd].view(M, nq + nkv, hd)
    if rotate:
        qk = plain.apply_rope(qk, cos[pos.long()], sin[pos.long()])
    v = qkv[:, (nq + nkv) * hd:].view(M, nkv, hd)
    assert torch.allclose(q.float().cpu().view(M, nq, hd), qk[:, :nq], atol=4e-2, rtol=2e-2)
    kc, vc = kp.float().cpu(), vp.float().cpu()
    for m, p_ in enumerate(starts):
        pg = int(table[m, p_ // PAGE])
        assert torch.allclose(kc[pg, :, p_ % PAGE], qk[m, nq:], atol=4e-2, rtol=2e-2), m
        assert torch.allclose(vc[pg, :, p_ % PAGE], v[m], atol=4e-2, rtol=2e-2), m
    assert int((kc != 0).any(dim=-1).sum()) == M * nkv and int((vc != 0).any(dim=-1).sum()) == M * nkv
    # without pools nothing is stored
    kp.zero_()
    K.norm_qkv_rope_store(dev(x), dev(nw.to(torch.bfloat16)), 1e-6, dev(w.to(torch.bfloat16)), None, nq, nkv, hd,
                          None, None, dev(pos), dev(row), None, None, dev(table), 3)
    assert float(kp.abs().sum()) == 0.0


# ---------------------------------------------------------------------------- the same for 17 to 64 rows (csrc/linear_batch.cu)

@pytest.mark.parametrize("M", [17, 32, 33, 47, 64])
@pytest.mark.parametrize("N,K_", [(100, 96), (896, 896), (896, 4864), (9728, 896), (70, 168), (1000, 3584),
                                  (40, 9000), (136, 72), (264, 200),      # K ends in the middle of a 16-column step
                                  (4744, 512)])
def test_linear_batch(K, M, N, K_):
    a, w, b = bf(rnd(M, K_, seed=1)), bf(rnd(N, K_, seed=2, scale=K_ ** -0.5)), bf(rnd(N, seed=3))
    want = a.double() @ w.double().T
    A, W = dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16))
    assert K.fused_takes(M, W, A, max_rows=K.BATCH_MAX_ROWS) and not K.fused_takes(M, W, A)
    x = rnd(M, N, seed=4)
    got = K.linear_fused(A, W, accumulate_into=dev(x.clone()))
    K.check_status("cuda")
    err, at = rel_err(got, x.double() + want)
    assert err < 2e-5, (err, at)
    got = K.linear_fused(A, W, dev(b.to(torch.float32)), accumulate_into=dev(x.clone()))
    err, at = rel_err(got, x.double() + want + b.double())
    assert err < 2e-5, (err, at)
    got = K.linear_fused(A, W, dev(b.to(torch.bfloat16)), out_dtype=torch.bfloat16)
    err, at = rel_err(got.float(), want + b.double())
    assert got.shape == (M, N) and err < 5e-3, (err, at)
    # the operand as the RMSNorm of float32 rows
    xs, nw = rnd(M, K_, seed=5, scale=2.0), bf(1 + rnd(K_, seed=6) * 0.1)
    h = plain.rms_norm(xs, nw, 1e-5).to(torch.bfloat16).double()
    for nw_dtype in (torch.bfloat16, torch.float32):
        got = K.linear_fused(None, W, accumulate_into=dev(x.clone()), norm_of=dev(xs), norm_weight=dev(nw.to(nw_dtype)), eps=1e-5)
        K.check_status("cuda")
        assert torch.allclose(got.cpu().double(), x.double() + h @ w.double().T, atol=3e-2, rtol=1e-2)   # a bfloat16 rounding of h may flip


def test_linear_batch_rows_do_not_depend_on_their_neighbours(K):
    a, w = bf(rnd(64, 4864, seed=1)), bf(rnd(896, 4864, seed=2, scale=0.02))
    W = dev(w.to(torch.bfloat16))
    zero = lambda n: torch.zeros(n, 896, dtype=torch.float32, device="cuda")
    whole = K.linear_fused(dev(a.to(torch.bfloat16)), W, accumulate_into=zero(64))
    for rows in (list(range(20)), list(range(3, 64, 2)), list(range(40, 64)) + list(range(10))):
        assert torch.equal(K.linear_fused(dev(a[rows].to(torch.bfloat16)), W, accumulate_into=zero(len(rows))), whole[rows])


@pytest.mark.parametrize("M,H,I", [(17, 64, 160), (64, 896, 4864), (40, 96, 352), (33, 3584, 1000), (24, 512, 2504), (32, 200, 72)])
def test_batch_norm_gate_up_swiglu(K, M, H, I):
    x, nw = rnd(M, H, seed=1, scale=2.0), bf(1 + rnd(H, seed=2) * 0.1)
    w = bf(rnd(2 * I, H, seed=3, scale=H ** -0.5))
    h = plain.rms_norm(x, nw, 1e-6).to(torch.bfloat16).float()
    gu = (h @ w.T).to(torch.bfloat16).float()
    want = plain.swiglu(gu[:, :I], gu[:, I:])
    got = K.norm_gate_up_swiglu(dev(x), dev(nw.to(torch.bfloat16)), 1e-6, dev(w.to(torch.bfloat16)))
    K.check_status("cuda")
    assert got.shape == (M, I) and torch.allclose(got.float().cpu(), want, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("M", [17, 40, 64])
@pytest.mark.parametrize("nq,nkv,hd,H,theta,rotate", [(4, 2, 16, 64, 1e4, True), (3, 1, 32, 96, 1e6, True), (14, 2, 64, 896, 1e6, True),
                                                       (5, 5, 48, 240, 1e4, False), (7, 1, 128, 200, 1e6, True), (28, 4, 128, 3584, 1e6, True)])
def test_batch_norm_qkv_rope_store(K, M, nq, nkv, hd, H, theta, rotate):
    """Tokens of several sequences in one step, some sequences with several tokens (a short prompt step)."""
    g = torch.Generator().manual_seed(M)
    row = torch.sort(torch.randint(0, 9, (M,), generator=g)).values.to(torch.int32)
    first = torch.tensor([62, 5, 63, 64, 0, 100, 17, 30, 1], dtype=torch.int32)
    pos = torch.zeros(M, dtype=torch.int32)
    for m in range(M):                                            # consecutive positions within a sequence
        pos[m] = first[row[m]] + int((row[:m] == row[m]).sum())
    x, nw = rnd(M, H, seed=1, scale=2.0), bf(1 + rnd(H, seed=2) * 0.1)
    w, b = bf(rnd((nq + 2 * nkv) * hd, H, seed=3, scale=H ** -0.5)), bf(rnd((nq + 2 * nkv) * hd, seed=4, scale=0.3))
    cos, sin = plain.rope_angles(torch.arange(200), hd, theta)
    table = torch.arange(9 * 3, dtype=torch.int32).flip(0).view(9, 3).contiguous()
    kp = torch.zeros(9 * 3, nkv, PAGE, hd, dtype=torch.bfloat16, device="cuda")
    vp = torch.zeros_like(kp)
    q = K.norm_qkv_rope_store(dev(x), dev(nw.to(torch.bfloat16)), 1e-6, dev(w.to(torch.bfloat16)), dev(b.to(torch.float32)),
                              nq, nkv, hd, dev(cos) if rotate else None, dev(sin) if rotate else None, dev(pos), dev(row),
                              kp, vp, dev(table), 3)
    K.check_status("cuda")
    h = plain.rms_norm(x, nw, 1e-6).to(torch.bfloat16).float()
    qkv = (h @ w.T + b).to(torch.bfloat16).float()
    qk = qkv[:, :(nq + nkv) * hd].view(M, nq + nkv, hd)
    if rotate:
        qk = plain.apply_rope(qk, cos[pos.long()], sin[pos.long()])
    v = qkv[:, (nq + nkv) * hd:].view(M, nkv, hd)
    assert torch.allclose(q.float().cpu().view(M, nq, hd), qk[:, :nq], atol=4e-2, rtol=2e-2)
    kc, vc = kp.float().cpu(), vp.float().cpu()
    for m in range(M):
        p_ = int(pos[m])
        pg = int(table[int(row[m]), p_ // PAGE])
        assert torch.allclose(kc[pg, :, p_ % PAGE], qk[m, nq:], atol=4e-2, rtol=2e-2), m
        assert torch.allclose(vc[pg, :, p_ % PAGE], v[m], atol=4e-2, rtol=2e-2), m
    assert int((kc != 0).any(dim=-1).sum()) == M * nkv and int((vc != 0).any(dim=-1).sum()) == M * nkv
    kp.zero_()
    K.norm_qkv_rope_store(dev(x), dev(nw.to(torch.bfloat16)), 1e-6, dev(w.to(torch.bfloat16)), None, nq, nkv, hd,
                          None, None, dev(pos), dev(row), None, None, dev(table), 3)
    assert float(kp.abs().sum()) == 0.0


# ---------------------------------------------------------------------------- tcgen05 products for more than 16 rows

ORIENTATIONS = ["rows", "pairs", "swapped"]       # 128 rows of a CTA / 256 rows of a CTA pair / rows of the weight on the lanes


def rel_err(got, want):
    """Largest error relative to 1 + |want| (float64)."""
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs() / (1.0 + want.abs())
    return float(err.max()), divmod(int(err.argmax()), want.shape[-1])


@pytest.mark.parametrize("orientation", ORIENTATIONS)
@pytest.mark.parametrize("M,N,K_", [(17, 1152, 896), (33, 3584, 3584), (64, 896, 4864), (65, 136, 72), (128, 1152, 896),
                                    (129, 264, 200), (300, 896, 896), (513, 2048, 136), (700, 4608, 896), (2048, 896, 896)])
def test_gemm_tcgen05(K, orientation, M, N, K_):
    """Against the float64 product of the same bfloat16 operands: the stored result is held to bfloat16's
    rounding (2^-8 of the value, plus the bias's), the sum into the float32 stream to float32 accumulation."""
    if orientation == "swapped" and M > 600:
        pytest.skip("the swapped orientation is for a few hundred rows at most")
    a, w, b = bf(rnd(M, K_, seed=1)), bf(rnd(N, K_, seed=2, scale=K_ ** -0.5)), bf(rnd(N, seed=3))
    A, W = dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16))
    assert K.gemm_tcgen05_takes(A, W)
    want = a.double() @ w.double().T
    for bias_dtype in (torch.bfloat16, torch.float32):
        got = K.gemm_tcgen05(A, W, dev(b.to(bias_dtype)), orientation=orientation)
        K.check_status("cuda")
        err, at = rel_err(got.float(), want + b.double())
        assert got.shape == (M, N) and err < 5e-3, (err, at)
    x = rnd(M, N, seed=4)
    got = K.gemm_tcgen05(A, W, accumulate_into=dev(x.clone()), orientation=orientation)
    K.check_status("cuda")
    err, at = rel_err(got, x.double() + want)
    assert err < 2e-5, (err, at)


@pytest.mark.parametrize("orientation", ORIENTATIONS)
@pytest.mark.parametrize("M,H,I", [(24, 896, 4864), (64, 896, 4864), (70, 64, 160), (129, 96, 352), (200, 3584, 1000),
                                   (2048, 896, 4864)])
def test_gemm_tcgen05_swiglu(K, orientation, M, H, I):
    if orientation == "swapped" and M > 600:
        pytest.skip("the swapped orientation is for a few hundred rows at most")
    a, w = bf(rnd(M, H, seed=1)), bf(rnd(2 * I, H, seed=3, scale=H ** -0.5))
    gu = (a.double() @ w.double().T).to(torch.bfloat16).float()         # gate and up are rounded to bfloat16 first
    want = plain.swiglu(gu[:, :I], gu[:, I:])
    got = K.gemm_tcgen05(dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16)), swiglu=True, orientation=orientation)
    K.check_status("cuda")
    err, at = rel_err(got.float(), want)
    # a gate or up value that rounds the other way (float32 against float64 accumulation) moves the result by 2^-8 of it
    assert got.shape == (M, I) and err < 1.2e-2, (err, at)


@pytest.mark.parametrize("orientation", ORIENTATIONS + ["splitk"])
@pytest.mark.parametrize("nq,nkv,hd,H,theta,rotate,M", [(4, 2, 16, 64, 1e4, True, 40), (3, 1, 32, 96, 1e6, True, 70),
                                                         (14, 2, 64, 896, 1e6, True, 200), (28, 4, 128, 3584, 1e6, True, 130),
                                                         (5, 5, 64, 240, 1e4, False, 33), (14, 2, 64, 896, 1e6, True, 64),
                                                         (14, 2, 64, 896, 1e6, True, 600), (5, 1, 48, 200, 1e4, True, 50),
                                                         (28, 4, 128, 3584, 1e6, True, 47), (3, 1, 32, 96, 1e6, True, 17)])
def test_gemm_qkv_rope_store(K, orientation, nq, nkv, hd, H, theta, rotate, M):
    """The q/k/v product with bias, rotation and cache write in its epilogue: M tokens of a few sequences of
    unequal lengths that start at unequal places of their (shuffled) pages."""
    if orientation == "splitk" and M > K.SPLITK_MAX_ROWS:
        pytest.skip("K cut over a cluster is for up to 64 rows")
    if orientation != "splitk" and hd not in K.GEMM_ROPE_HEAD_DIMS:
        pytest.skip("head sizes that are no power of two: only with K cut over a cluster")
    lens, starts, left, i = [], [], M, 0
    while left > 0:
        n = min(left, [1, 37, 64, 9, 100][i % 5])
        lens.append(n); starts.append([62, 5, 63, 0, 130][i % 5]); left -= n; i += 1
    B = len(lens)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).int()
    row = torch.cat([torch.full((n,), b_) for b_, n in enumerate(lens)]).int()
    width = max((s + n + PAGE - 1) // PAGE for s, n in zip(starts, lens))
    table = torch.randperm(B * width, generator=torch.Generator().manual_seed(5)).int().view(B, width).contiguous()
    N = (nq + 2 * nkv) * hd
    a, w, b = bf(rnd(M, H, seed=1)), bf(rnd(N, H, seed=2, scale=H ** -0.5)), bf(rnd(N, seed=3, scale=0.3))
    cos, sin = plain.rope_angles(torch.arange(400), hd, theta)
    kp = torch.zeros(B * width, nkv, PAGE, hd, dtype=torch.bfloat16, device="cuda")
    vp = torch.zeros_like(kp)
    q = K.gemm_qkv_rope_store(dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16)), dev(b.to(torch.bfloat16)), nq, nkv, hd,
                              dev(cos) if rotate else None, dev(sin) if rotate else None, dev(pos), dev(row), kp, vp,
                              dev(table), width, orientation=orientation)
    K.check_status("cuda")
    qkv = (a.double() @ w.double().T + b.double()).to(torch.bfloat16).float()      # rounded before the rotation
    qk = qkv[:, :(nq + nkv) * hd].view(M, nq + nkv, hd)
    if rotate:
        qk = plain.apply_rope(qk, cos[pos.long()], sin[pos.long()])
    v = qkv[:, (nq + nkv) * hd:].view(M, nkv, hd)
    err, at = rel_err(q.float().view(M, nq * hd), qk[:, :nq].reshape(M, nq * hd))
    assert err < 1.2e-2, ("q", err, at)
    kw, vw = torch.zeros(B * width, nkv, PAGE, hd), torch.zeros(B * width, nkv, PAGE, hd)
    for m in range(M):
        pg = int(table[int(row[m]), int(pos[m]) // PAGE])
        kw[pg, :, int(pos[m]) % PAGE] = qk[m, nq:]
        vw[pg, :, int(pos[m]) % PAGE] = v[m]
    err, at = rel_err(kp.float().view(-1, hd), kw.view(-1, hd))            # every other place of the pool stays zero
    assert err < 1.2e-2, ("k", err, at)
    err, at = rel_err(vp.float().view(-1, hd), vw.view(-1, hd))
    assert err < 1.2e-2, ("v", err, at)
    # without pools nothing is stored and the queries are the same
    kp.zero_()
    q2 = K.gemm_qkv_rope_store(dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16)), dev(b.to(torch.bfloat16)), nq, nkv, hd,
                               dev(cos) if rotate else None, dev(sin) if rotate else None, dev(pos), dev(row), None, None,
                               None, 0, orientation=orientation)
    assert torch.equal(q, q2) and float(kp.abs().sum()) == 0.0


@pytest.mark.parametrize("M", [17, 32, 33, 64])
@pytest.mark.parametrize("N,K_", [(1152, 896), (896, 896), (896, 4864), (136, 72), (264, 200), (3584, 3584), (100, 64), (4608, 128)])
def test_gemm_splitk(K, M, N, K_):
    """The product for 17 to 64 rows with K cut over a cluster (csrc/gemm_splitk.cu): widths that are no multiple of the
    128-row tile or of the 64-column block, one to eight ranges."""
    a, w, b = bf(rnd(M, K_, seed=1)), bf(rnd(N, K_, seed=2, scale=K_ ** -0.5)), bf(rnd(N, seed=3))
    A, W = dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16))
    want = a.double() @ w.double().T
    for bias_dtype in (torch.bfloat16, torch.float32):
        got = K.gemm_tcgen05(A, W, dev(b.to(bias_dtype)), orientation="splitk")
        K.check_status("cuda")
        err, at = rel_err(got.float(), want + b.double())
        assert got.shape == (M, N) and err < 5e-3, (err, at)
    x = rnd(M, N, seed=4)
    got = K.gemm_tcgen05(A, W, accumulate_into=dev(x.clone()), orientation="splitk")
    K.check_status("cuda")
    err, at = rel_err(got, x.double() + want)
    assert err < 2e-5, (err, at)
    again = K.gemm_tcgen05(A, W, accumulate_into=dev(x.clone()), orientation="splitk")
    assert torch.equal(got, again)                                  # the ranges are added in a fixed order
    part = K.gemm_tcgen05(A[:20].contiguous(), W, accumulate_into=dev(x[:20].clone()), orientation="splitk")
    assert torch.equal(part, got[:20])                              # a row does not depend on its neighbours


@pytest.mark.parametrize("M,H,I", [(24, 896, 4864), (64, 896, 4864), (40, 64, 160), (33, 96, 352), (17, 3584, 1000)])
def test_gemm_splitk_swiglu(K, M, H, I):
    a, w = bf(rnd(M, H, seed=1)), bf(rnd(2 * I, H, seed=3, scale=H ** -0.5))
    gu = (a.double() @ w.double().T).to(torch.bfloat16).float()
    want = plain.swiglu(gu[:, :I], gu[:, I:])
    got = K.gemm_tcgen05(dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16)), swiglu=True, orientation="splitk")
    K.check_status("cuda")
    err, at = rel_err(got.float(), want)
    assert got.shape == (M, I) and err < 1.2e-2, (err, at)


def test_gemm_tcgen05_refuses_what_it_does_not_take(K):
    from pico_engine.ops.library import KernelError
    a, w = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda"), torch.zeros(144, 64, dtype=torch.bfloat16, device="cuda")
    pos = torch.zeros(64, dtype=torch.int32, device="cuda")
    with pytest.raises(KernelError, match="head size 48"):
        K.gemm_qkv_rope_store(a, w, None, 1, 1, 48, None, None, pos, pos, None, None, None, 0)
    with pytest.raises(KernelError):
        K.gemm_tcgen05(a[:, :60].contiguous(), w[:, :60].contiguous())        # K must be a multiple of 8


def test_product_choice_is_made_once_and_both_ways_agree(K):
    """ops.linear times this library's fused kernel against the library product plus the separate pass, once per
    shape; whichever it takes, the result is the same within bfloat16's rounding."""
    import sys
    import pico_engine.ops                                   # noqa: F401  (the package's attribute `linear` is the function)
    L = sys.modules["pico_engine.ops.linear"]
    a, w = bf(rnd(300, 896, seed=1)), bf(rnd(2 * 1000, 896, seed=2, scale=896 ** -0.5))
    A, W = dev(a.to(torch.bfloat16)), dev(w.to(torch.bfloat16))
    key = ("swiglu", 512, 2000, 896)
    L.Choice.table.pop(key, None)
    first = L.gate_up_swiglu(A, W)
    assert L.Choice.table[key] in ("tcgen05", "library") and (L._FORCED != "auto" or key in L.Choice.timings)
    taken = L.Choice.table[key]
    L.Choice.table[key] = "library" if taken == "tcgen05" else "tcgen05"
    other = L.gate_up_swiglu(A, W)
    L.Choice.table[key] = taken
    err, at = rel_err(first.float(), other.float())
    assert err < 1.2e-2, (err, at)
    assert torch.equal(L.gate_up_swiglu(A, W), first)
