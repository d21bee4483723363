"""One Python function per CUDA kernel: argument checks, then the launch on torch's current
stream.  Tensors are passed as raw device pointers; outputs are allocated by the caller or
here with torch's allocator.  There is no other implementation behind these functions.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .library import DTYPE_CODE, KernelError, check, core, extras, stream_ptr

PAGE = 64     # tokens per cache page; PE_PAGE in csrc/common.cuh


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    # the passing case first and cheaply: these checks run a few hundred times a step
    if (t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype)
            and (shape is None or t.shape == shape or tuple(t.shape) == tuple(shape))):
        return
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, not {t.dtype}")
    raise KernelError(f"{name} must have shape {tuple(shape)}, not {tuple(t.shape)}")


def _code(t: torch.Tensor, name: str) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{name} must be float32 or bfloat16, not {t.dtype}") from None


def embed(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows ``ids`` (int32, [T]) of ``table`` [V, H] as float32 [T, H]."""
    V, H = table.shape
    T = ids.shape[0]
    _need(table, "table"); _need(ids, "ids", torch.int32, (T,))
    if out is None:
        out = torch.empty(T, H, dtype=torch.float32, device=table.device)
    _need(out, "out", torch.float32, (T, H))
    check(core().pe_embed(table.data_ptr(), _code(table, "table"), ids.data_ptr(), out.data_ptr(), T, H, V,
                          stream_ptr()), "embed")
    return out


def select_tokens(ids: torch.Tensor, prev: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """``ids[j] = prev[src[j]]`` where ``src[j] >= 0`` (all int32, on the device): the ids of rows whose
    token the step before chose and the host has not read yet."""
    n = ids.shape[0]
    _need(ids, "ids", torch.int32, (n,)); _need(prev, "prev", torch.int32); _need(src, "src", torch.int32, (n,))
    check(core().pe_select_tokens(ids.data_ptr(), prev.data_ptr(), src.data_ptr(), n, stream_ptr()), "select_tokens")
    return ids


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows_index: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of float32 rows [T, H]; with ``rows_index`` (int32 [R]) only of those rows."""
    T, H = x.shape
    _need(x, "x", torch.float32); _need(weight, "weight", None, (H,))
    rows = T if rows_index is None else rows_index.shape[0]
    if rows_index is not None:
        _need(rows_index, "rows_index", torch.int32)
    if out is None:
        out = torch.empty(rows, H, dtype=out_dtype, device=x.device)
    _need(out, "out", out_dtype, (rows, H))
    check(core().pe_rmsnorm(x.data_ptr(), _ptr(rows_index), weight.data_ptr(), _code(weight, "weight"), float(eps),
                            out.data_ptr(), _code(out, "out"), rows, H, stream_ptr()), "rmsnorm")
    return out


def add_rmsnorm(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x += y (float32 rows [T, H], in place), then RMSNorm of every row: the residual sum and the
    norm that follows it in one pass over the stream."""
    T, H = x.shape
    _need(x, "x", torch.float32); _need(y, "y", None, (T, H)); _need(weight, "weight", None, (H,))
    if out is None:
        out = torch.empty(T, H, dtype=out_dtype, device=x.device)
    _need(out, "out", out_dtype, (T, H))
    check(core().pe_add_rmsnorm(x.data_ptr(), y.data_ptr(), _code(y, "y"), weight.data_ptr(), _code(weight, "weight"),
                                float(eps), out.data_ptr(), _code(out, "out"), T, H, stream_ptr()), "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(gate) * up of [T, 2I] (gate first) as [T, I]."""
    T, I2 = gate_up.shape
    _need(gate_up, "gate_up")
    if I2 % 2:
        raise KernelError("gate_up needs an even number of columns")
    if out is None:
        out = torch.empty(T, I2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    _need(out, "out", gate_up.dtype, (T, I2 // 2))
    check(core().pe_swiglu(gate_up.data_ptr(), out.data_ptr(), _code(gate_up, "gate_up"), T, I2 // 2, stream_ptr()),
          "swiglu")
    return out


def residual_add(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """x += y in float32; x is the float32 residual stream."""
    _need(x, "x", torch.float32); _need(y, "y", None, x.shape)
    check(core().pe_residual_add(x.data_ptr(), y.data_ptr(), _code(y, "y"), x.numel(), stream_ptr()), "residual_add")
    return x


def bias_add(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    M, N = y.shape
    _need(y, "y"); _need(bias, "bias", None, (N,))
    check(core().pe_bias_add(y.data_ptr(), _code(y, "y"), bias.data_ptr(), _code(bias, "bias"), M, N, stream_ptr()),
          "bias_add")
    return y


def rope_store(qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int, cos: Optional[torch.Tensor],
               sin: Optional[torch.Tensor], tok_pos: torch.Tensor, tok_row: torch.Tensor,
               k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], block_table: Optional[torch.Tensor],
               table_stride: int) -> None:
    """Rotate the query and key heads of ``qkv`` [T, (n_q + 2 n_kv) * head_dim] in place and
    write keys and values to the cache pages of their sequences (skipped when ``k_pool`` is None)."""
    T = qkv.shape[0]
    _need(qkv, "qkv", None, (T, (n_q + 2 * n_kv) * head_dim))
    _need(tok_pos, "tok_pos", torch.int32); _need(tok_row, "tok_row", torch.int32)
    if cos is not None:
        _need(cos, "cos", torch.float32); _need(sin, "sin", torch.float32, cos.shape)
        if cos.shape[1] != head_dim // 2:
            raise KernelError("cos/sin tables need head_dim/2 columns")
    store = k_pool is not None
    if store:
        _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype, k_pool.shape)
        _need(block_table, "block_table", torch.int32)
        if tuple(k_pool.shape[1:]) != (n_kv, PAGE, head_dim):
            raise KernelError(f"cache pool must be [pages, {n_kv}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    check(core().pe_rope_store(qkv.data_ptr(), _code(qkv, "qkv"), T, n_q, n_kv, head_dim, _ptr(cos), _ptr(sin),
                               tok_pos.data_ptr(), tok_row.data_ptr(), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                               table_stride, 1 if store else 0, stream_ptr()), "rope_store")


_EPILOGUE_STORE = {torch.float32: 0, torch.bfloat16: 1}


def linear_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, accumulate_into: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T (+ bias) with float32 multiply-adds.  Either stored as
    ``out_dtype`` or added into the float32 tensor ``accumulate_into`` [M, N]."""
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a"); _need(w, "w", None, (N, K))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    if accumulate_into is not None:
        _need(accumulate_into, "accumulate_into", torch.float32, (M, N))
        out, epilogue = accumulate_into, 2
    else:
        if out is None:
            out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
        _need(out, "out", None, (M, N))
        epilogue = _EPILOGUE_STORE[out.dtype]
    check(core().pe_linear_simt(a.data_ptr(), _code(a, "a"), w.data_ptr(), _code(w, "w"), _ptr(bias),
                                0 if bias is None else _code(bias, "bias"), out.data_ptr(), epilogue, M, N, K,
                                stream_ptr()), "linear_simt")
    return out


def attention_generic(q: torch.Tensor, q_stride: int, n_heads: int, n_kv_heads: int, head_dim: int,
                      k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int,
                      tok_pos: torch.Tensor, tok_row: torch.Tensor, window: Optional[int], scale: float,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of T tokens over the cache.  ``q`` holds the query heads of token t at
    ``t * q_stride + h * head_dim``; the result is [T, n_heads * head_dim] in q's dtype."""
    T = tok_pos.shape[0]
    _need(q, "q"); _need(k_pool, "k_pool", q.dtype); _need(v_pool, "v_pool", q.dtype, k_pool.shape)
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pool must be [pages, {n_kv_heads}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    _need(block_table, "block_table", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32, (T,)); _need(tok_row, "tok_row", torch.int32, (T,))
    if out is None:
        out = torch.empty(T, n_heads * head_dim, dtype=q.dtype, device=q.device)
    _need(out, "out", q.dtype, (T, n_heads * head_dim))
    check(core().pe_attention_generic(q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                      _code(q, "q"), block_table.data_ptr(), table_stride, tok_pos.data_ptr(),
                                      tok_row.data_ptr(), T, n_heads, n_kv_heads, head_dim, window or 0, float(scale),
                                      stream_ptr()), "attention_generic")
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    B, V = logits.shape
    _need(logits, "logits", torch.float32)
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, (B,))
    from .workspace import scratch
    lib = core()
    ws = scratch("argmax.partial", lib.pe_argmax_scratch_bytes(B, V), logits.device)
    check(lib.pe_argmax(logits.data_ptr(), out.data_ptr(), B, V, ws.data_ptr(), stream_ptr()), "argmax", 2)
    return out


def sample_settings_words(temperature: float, top_k: int, top_p: float, seed: int):
    """The six int32 words of the sampler's settings as the kernels read them from device memory."""
    import struct
    return list(struct.unpack("<6i", struct.pack("<fifiQ", float(temperature), int(top_k), float(top_p), 0,
                                                 int(seed) & ((1 << 64) - 1))))


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, request: torch.Tensor,
           step: torch.Tensor, out: Optional[torch.Tensor] = None, settings: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One draw per row of float32 logits [B, V]; row b uses the uniform of (seed, request[b], step[b]).
    ``settings`` (int32 [6] on the device, ``sample_settings_words``): where given, the kernels read
    temperature, top_k, top_p and the seed from there at run time (a captured launch then follows settings
    that change); the arguments still decide which passes run, i.e. whether there is a cut by rank and by mass."""
    B, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(request, "request", torch.int32, (B,)); _need(step, "step", torch.int32, (B,))
    if not temperature > 0:
        raise KernelError("sample needs a positive temperature; use argmax for greedy choice")
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, (B,))
    from .workspace import scratch
    lib = core()
    ws = scratch("sample.state", lib.pe_sample_scratch_bytes(B, V), logits.device, zeroed=True)
    cut_k, cut_p = 0 < top_k < V, top_p < 1.0
    if settings is not None:
        _need(settings, "settings", torch.int32, (6,))
        if settings.data_ptr() % 8:
            raise KernelError("settings must start on an 8-byte boundary")
    check(lib.pe_sample(logits.data_ptr(), out.data_ptr(), B, V, float(temperature), int(top_k), float(top_p),
                        int(seed) & ((1 << 64) - 1), request.data_ptr(), step.data_ptr(), ws.data_ptr(), _ptr(settings),
                        stream_ptr()),
          "sample", 2 + 3 * cut_k + 3 * cut_p)
    return out


def draw_uniform(seed: int, request: int, step: int) -> float:
    """The uniform the sampling kernel uses for (seed, request, step), computed on the host."""
    m = (1 << 64) - 1
    return float(core().pe_draw_uniform(seed & m, request & m, step & m))


# ---------------------------------------------------------------------------- tensor-core kernels (bfloat16)

def linear_mma_takes(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes these operands (else another one is used)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] <= 64 and a.shape[1] % 8 == 0
            and a.is_contiguous() and w.is_contiguous() and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def linear_mma(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
               out_dtype: Optional[torch.dtype] = None, accumulate_into: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M <= 64, K] . w [N, K]^T (+ bias), bfloat16 operands, float32 accumulation on the
    tensor cores; stored as ``out_dtype`` or added into float32 ``accumulate_into``."""
    from .workspace import scratch
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a", torch.bfloat16); _need(w, "w", torch.bfloat16, (N, K))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    if accumulate_into is not None:
        _need(accumulate_into, "accumulate_into", torch.float32, (M, N))
        out, epilogue = accumulate_into, 2
    else:
        if out is None:
            out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
        _need(out, "out", None, (M, N))
        epilogue = _EPILOGUE_STORE[out.dtype]
    lib = extras()
    partial = tickets = None
    if lib.pe_linear_mma_splits(N, K) > 1:
        partial = scratch("linear_mma.partial", lib.pe_linear_mma_scratch_bytes(64, N, K), a.device).data_ptr()
        tickets = scratch("linear_mma.tickets", 4 * ((N + 15) // 16), a.device, zeroed=True).data_ptr()
    check(lib.pe_linear_mma(a.data_ptr(), w.data_ptr(), _ptr(bias), 0 if bias is None else _code(bias, "bias"),
                            out.data_ptr(), epilogue, M, N, K, partial, tickets, stream_ptr()), "linear_mma")
    return out


def attention_decode(q: torch.Tensor, q_stride: int, n_heads: int, n_kv_heads: int, head_dim: int,
                     k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int,
                     tok_pos: torch.Tensor, tok_row: torch.Tensor, window: Optional[int], scale: float,
                     max_context: int, out: Optional[torch.Tensor] = None, early_pages: bool = True) -> torch.Tensor:
    """Attention of T single tokens (bfloat16) over the cache; ``max_context`` bounds every
    token's position + 1 and fixes the launch shape.  With ``early_pages`` the kernel copies cache pages
    while the two kernels before it on the stream may still run: they must have written keys and values
    at each token's own position only (the library's own parts do).  A part that rewrites other cache
    rows shortly before attending passes False: the kernel then starts when everything before it has ended."""
    from .library import for_head_dim
    T = tok_pos.shape[0]
    _need(q, "q", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pool must be [pages, {n_kv_heads}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    _need(block_table, "block_table", torch.int32)
    _need(tok_pos, "tok_pos", torch.int32, (T,)); _need(tok_row, "tok_row", torch.int32, (T,))
    if out is None:
        out = torch.empty(T, n_heads * head_dim, dtype=torch.bfloat16, device=q.device)
    _need(out, "out", torch.bfloat16, (T, n_heads * head_dim))
    lib = for_head_dim(head_dim)
    check(lib.pe_attention_decode(q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                  block_table.data_ptr(), table_stride, tok_pos.data_ptr(), tok_row.data_ptr(), T,
                                  n_heads, n_kv_heads, head_dim, window or 0, float(scale), int(max_context),
                                  1 if early_pages else 0, status_ptr(q.device), stream_ptr()), "attention_decode")
    return out


PREFILL_TILE = 64             # AP_QTILE of csrc/attention_prefill.cu
PREFILL_TILE_TCGEN05 = 128    # AT_QTILE of csrc/attention_prefill_tcgen05.cu
TCGEN05_HEAD_DIMS = (64, 128)


def prefill_tile_rows(lens, starts, tile: int = PREFILL_TILE):
    """[(batch row, first packed token, tokens, position of the first token), ...]: the packed tokens of a
    step cut into runs of at most ``tile`` tokens of one sequence, the runs that see the most keys first
    (they take longest, so they are scheduled first)."""
    rows = []
    tok = 0
    for b, (n, st) in enumerate(zip(lens, starts)):
        for off in range(0, n, tile):
            rows.append((b, tok + off, min(tile, n - off), st + off))
        tok += n
    rows.sort(key=lambda r: -(r[3] + r[2]))
    return rows


def prefill_tiles(lens, starts, device, tile: int = PREFILL_TILE) -> torch.Tensor:
    """``prefill_tile_rows`` as int32 [tiles, 4] on ``device``."""
    return torch.tensor(prefill_tile_rows(lens, starts, tile), dtype=torch.int32).to(device, non_blocking=True)


def _prefill_args(q, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table, tiles, n_tokens, out):
    _need(q, "q", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    if tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pool must be [pages, {n_kv_heads}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    _need(block_table, "block_table", torch.int32); _need(tiles, "tiles", torch.int32)
    if out is None:
        out = torch.empty(n_tokens, n_heads * head_dim, dtype=torch.bfloat16, device=q.device)
    _need(out, "out", torch.bfloat16, (n_tokens, n_heads * head_dim))
    return out


def attention_prefill(q: torch.Tensor, q_stride: int, n_heads: int, n_kv_heads: int, head_dim: int,
                      k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int,
                      tiles: torch.Tensor, n_tokens: int, window: Optional[int], scale: float,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention (bfloat16) of the token runs ``tiles`` (of at most 64 tokens) over the cache:
    the mma.sync kernel, which takes every head size."""
    from .library import for_head_dim
    out = _prefill_args(q, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table, tiles, n_tokens, out)
    check(for_head_dim(head_dim).pe_attention_prefill(
        q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(),
        table_stride, tiles.data_ptr(), None, None, tiles.shape[0], n_heads, n_kv_heads, head_dim, window or 0,
        float(scale), stream_ptr()), "attention_prefill")
    return out


def attention_prefill_tcgen05_takes(head_dim: int, scale: float) -> bool:
    return head_dim in TCGEN05_HEAD_DIMS and scale > 0


def attention_prefill_tcgen05(q: torch.Tensor, q_stride: int, n_heads: int, n_kv_heads: int, head_dim: int,
                              k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int,
                              tiles: torch.Tensor, n_tokens: int, window: Optional[int], scale: float,
                              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same on the tcgen05 tensor cores, for head sizes 64 and 128 and runs ``tiles`` of at most
    128 tokens.  ``q`` is a view of ``n_tokens`` rows, ``q_stride`` elements apart."""
    from .library import for_head_dim
    out = _prefill_args(q, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table, tiles, n_tokens, out)
    check(for_head_dim(head_dim).pe_attention_prefill_tcgen05(
        q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0], block_table.data_ptr(),
        table_stride, tiles.data_ptr(), tiles.shape[0], n_tokens, n_heads, n_kv_heads, head_dim, window or 0,
        float(scale), status_ptr(q.device), stream_ptr()), "attention_prefill_tcgen05")
    return out


def attention(q: torch.Tensor, q_stride: int, n_heads: int, n_kv_heads: int, head_dim: int, k_pool: torch.Tensor,
              v_pool: torch.Tensor, block_table: torch.Tensor, table_stride: int, tok_pos: torch.Tensor,
              tok_row: torch.Tensor, window: Optional[int], scale: float, ctx, own_rows_only: bool = True) -> torch.Tensor:
    """Attention of the step's tokens over the cache, with the kernel the step calls for:
    bfloat16 uses the tensor-core kernels (single tokens: decode; longer runs: prefill),
    float32 the float32 kernel.  ``own_rows_only``: the kernels launched just before wrote no cache row
    but each token's own (see ``attention_decode``); a caller that cannot promise this passes False."""
    if q.dtype == torch.bfloat16:
        if ctx.one_token_each:
            return attention_decode(q, q_stride, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table,
                                    table_stride, tok_pos, tok_row, window, scale, ctx.max_context,
                                    early_pages=own_rows_only)
        tcgen05 = attention_prefill_tcgen05_takes(head_dim, scale)
        name = "prefill_tiles_128" if tcgen05 else "prefill_tiles"
        tiles = ctx.scratch.get(name)
        if tiles is None:
            tiles = ctx.scratch[name] = prefill_tiles(ctx.lens, ctx.starts, q.device,
                                                      PREFILL_TILE_TCGEN05 if tcgen05 else PREFILL_TILE)
        run = attention_prefill_tcgen05 if tcgen05 else attention_prefill
        return run(q, q_stride, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table, table_stride, tiles,
                   tok_pos.shape[0], window, scale)
    return attention_generic(q, q_stride, n_heads, n_kv_heads, head_dim, k_pool, v_pool, block_table, table_stride,
                             tok_pos, tok_row, window, scale)


# ---------------------------------------------------------------------------- fused decode products (bfloat16, up to 16 rows)

FUSED_MAX_ROWS = 16


_status_words = {}


def status_word(device) -> torch.Tensor:
    """The int32 word in which a kernel records that a bounded wait of its own ran out (0: none did)."""
    word = _status_words.get(device)
    if word is None:
        from .workspace import scratch
        word = _status_words[device] = scratch("status", 4, torch.device(device), zeroed=True)[:4].view(torch.int32)
        _status_ptrs[device] = word.data_ptr()
    return word


_status_ptrs = {}


def status_ptr(device) -> int:
    """The address of ``status_word(device)``."""
    ptr = _status_ptrs.get(device)
    if ptr is None:
        ptr = status_word(device).data_ptr()
    return ptr


def check_status(device) -> None:
    """Raise if a kernel gave up waiting for its own copies since the last check.  Synchronises."""
    word = status_word(device)
    code = int(word.item())
    if code:
        word.zero_()
        raise KernelError(f"a kernel gave up a bounded wait (status {code}); its results are incomplete")


# A weight this large streams faster through the library's product even for a few rows: measured on a B200 at
# 8 rows, 37888 x 3584 (271 MB): 46 us (5.9 TB/s) against 61 us; 3584 x 18944 (136 MB): 28 us against 33 us;
# 151936 x 896 (272 MB, into float32): 52 us against 72 us.  The fused kernel's CTAs restart their pipeline
# for every tile; smaller weights are faster there, with what precedes and follows the product fused in.
FUSED_MAX_WEIGHT_BYTES = int(os.environ.get("PICO_ENGINE_FUSED_MAX_MB", "100")) << 20


def fused_takes(rows: int, w: torch.Tensor, *others: torch.Tensor, max_rows: int = FUSED_MAX_ROWS) -> bool:
    """Whether the fused decode kernels take a product with ``rows`` rows and weight ``w``."""
    return (rows <= max_rows and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.is_contiguous()
            and w.data_ptr() % 16 == 0 and all(t.is_contiguous() and t.data_ptr() % 16 == 0 for t in others)
            and w.numel() * 2 <= FUSED_MAX_WEIGHT_BYTES)


# The same fused products for 17 to 64 rows are another kernel (csrc/linear_batch.cu: 64 rows of the weight a CTA
# instead of 16, operands through shared memory by TMA); the three functions below take either number of rows.
# It is not what a decode step of that many rows runs unless PICO_ENGINE_BATCH_FUSED=1: measured on a B200 at the
# Qwen2.5-0.5B widths and 64 rows, in captured graphs, norm + q/k/v + rotation take 10.9 us in it against 7.5 us as
# three kernels around the library's product, the output projection 6.5 against 5.3, norm + gate/up + SwiGLU 25.6
# against 9.1, the down projection 9.7 against 10.1; at the 7B widths it streams weights at 1.2 to 2.1 TB/s where
# the library reaches 4 to 5.  Two things bound it: mma.sync runs at about a quarter of the tcgen05 rate (1,000
# cycles for a chunk of 128 columns), and every CTA converts the float32 rows of the residual stream itself, which
# for gate/up (152 CTAs x 229 KB) is all the L2 delivers.
BATCH_MAX_ROWS = 64
BATCH_ENABLED = os.environ.get("PICO_ENGINE_BATCH_FUSED", "0") == "1"


def decode_fused_takes(rows: int, w: torch.Tensor, *others: torch.Tensor) -> bool:
    """Whether a decode step of ``rows`` sequences can run this product fused with its neighbours."""
    return fused_takes(rows, w, *others, max_rows=BATCH_MAX_ROWS if BATCH_ENABLED else FUSED_MAX_ROWS)


def set_batch_fused(on: bool) -> bool:
    """Let decode steps of 17 to 64 rows run the fused products of csrc/linear_batch.cu (or not); returns what was set."""
    global BATCH_ENABLED
    was, BATCH_ENABLED = BATCH_ENABLED, bool(on)
    return was


def linear_fused(a: Optional[torch.Tensor], w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, accumulate_into: Optional[torch.Tensor] = None,
                 norm_of: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                 eps: float = 0.0) -> torch.Tensor:
    """a [M <= 64, K] . w [N, K]^T (+ bias); with ``norm_of`` (float32 [M, K]) the operand is
    RMSNorm(norm_of) with ``norm_weight`` instead of ``a``.  (More than 16 rows: bfloat16 or accumulated results.)"""
    src = norm_of if norm_of is not None else a
    M, K = src.shape
    N = w.shape[0]
    _need(w, "w", torch.bfloat16, (N, K))
    if norm_of is not None:
        _need(norm_of, "norm_of", torch.float32); _need(norm_weight, "norm_weight", None, (K,))
    else:
        _need(a, "a", torch.bfloat16)
    if bias is not None:
        _need(bias, "bias", None, (N,))
    if accumulate_into is not None:
        _need(accumulate_into, "accumulate_into", torch.float32, (M, N))
        out, epilogue = accumulate_into, 2
    else:
        out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=w.device)
        epilogue = _EPILOGUE_STORE[out.dtype]
    fn, name = (core().pe_linear_fused, "linear_fused") if M <= FUSED_MAX_ROWS else (extras().pe_linear_batch, "linear_batch")
    check(fn(_ptr(a), _ptr(norm_of), _ptr(norm_weight), 0 if norm_weight is None else _code(norm_weight, "norm_weight"), float(eps),
             w.data_ptr(), _ptr(bias), 0 if bias is None else _code(bias, "bias"), out.data_ptr(),
             epilogue, M, N, K, status_ptr(w.device), stream_ptr()), name)
    return out


def norm_gate_up_swiglu(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(h Wg^T) * (h Wu^T) with h = RMSNorm(x); x float32 [M <= 64, K], w_gate_up [2I, K] (gate rows first)."""
    M, K = x.shape
    I = w_gate_up.shape[0] // 2
    _need(x, "x", torch.float32); _need(norm_weight, "norm_weight", None, (K,)); _need(w_gate_up, "w_gate_up", torch.bfloat16, (2 * I, K))
    act = torch.empty(M, I, dtype=torch.bfloat16, device=x.device)
    fn = core().pe_norm_gate_up_swiglu if M <= FUSED_MAX_ROWS else extras().pe_batch_norm_gate_up_swiglu
    check(fn(x.data_ptr(), norm_weight.data_ptr(), _code(norm_weight, "norm_weight"), float(eps),
             w_gate_up.data_ptr(), act.data_ptr(), M, I, K, status_ptr(x.device), stream_ptr()), "norm_gate_up_swiglu")
    return act


def norm_qkv_rope_store(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, w_qkv: torch.Tensor,
                        b_qkv: Optional[torch.Tensor], n_q: int, n_kv: int, head_dim: int, cos: Optional[torch.Tensor],
                        sin: Optional[torch.Tensor], tok_pos: torch.Tensor, tok_row: torch.Tensor,
                        k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                        block_table: Optional[torch.Tensor], table_stride: int) -> torch.Tensor:
    """Rotated queries [M, n_q * head_dim] of h = RMSNorm(x); rotated keys and the values go to
    the cache pages (skipped when ``k_pool`` is None)."""
    M, K = x.shape
    N = (n_q + 2 * n_kv) * head_dim
    _need(x, "x", torch.float32); _need(norm_weight, "norm_weight", None, (K,)); _need(w_qkv, "w_qkv", torch.bfloat16, (N, K))
    if b_qkv is not None:
        _need(b_qkv, "b_qkv", None, (N,))
    _need(tok_pos, "tok_pos", torch.int32, (M,)); _need(tok_row, "tok_row", torch.int32, (M,))
    if cos is not None:
        _need(cos, "cos", torch.float32); _need(sin, "sin", torch.float32, cos.shape)
    store = k_pool is not None
    if store:
        _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
        _need(block_table, "block_table", torch.int32)
        if tuple(k_pool.shape[1:]) != (n_kv, PAGE, head_dim):
            raise KernelError(f"cache pool must be [pages, {n_kv}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    q = torch.empty(M, n_q * head_dim, dtype=torch.bfloat16, device=x.device)
    tail = (q.data_ptr(), M, K, n_q, n_kv, head_dim, _ptr(cos), _ptr(sin), tok_pos.data_ptr(), tok_row.data_ptr(), _ptr(k_pool),
            _ptr(v_pool), _ptr(block_table), table_stride, 1 if store else 0, status_ptr(x.device), stream_ptr())
    head = (x.data_ptr(), norm_weight.data_ptr(), _code(norm_weight, "norm_weight"), float(eps), w_qkv.data_ptr(), _ptr(b_qkv),
            0 if b_qkv is None else _code(b_qkv, "b_qkv"))
    if M <= FUSED_MAX_ROWS:
        check(core().pe_norm_qkv_rope_store(None, *head, *tail), "norm_qkv_rope_store")
    else:
        check(extras().pe_batch_norm_qkv_rope_store(*head, *tail), "batch_norm_qkv_rope_store")
    return q


# ---------------------------------------------------------------------------- tcgen05 products for more than 16 rows (bfloat16)

ORIENTATION = {None: 0, "rows": 1, "swapped": 2, "pairs": 3}
# Orientation "splitk" (csrc/gemm_splitk.cu): rows of w on the lanes, K cut into ranges over a thread-block cluster, for up
# to 64 rows of a.  Nothing chooses it by itself: measured on a B200 at the Qwen2.5-0.5B widths and 64 rows, in captured
# graphs, it takes 8.5 / 7.2 / 11.8 / 9.5 us for q/k/v + RoPE, o + residual, gate/up + SwiGLU and down + residual where
# the library's product with the pass that follows it takes 5.9 / 5.3 / 7.7 / 10.1; at the 7B widths it streams
# gate/up at 4.6 to 5.0 TB/s (library 5.2).  One thread issues a stage's three TMA copies and another its four MMAs at
# 150 to 200 cycles an instruction, which is 700 cycles for 24 KB of operands, whatever the accumulators' number.
SPLITK_MAX_ROWS = 64


def gemm_tcgen05_takes(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and w.shape[0] % 8 == 0
            and a.is_contiguous() and w.is_contiguous() and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 accumulate_into: Optional[torch.Tensor] = None, swiglu: bool = False,
                 orientation: Optional[str] = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T on the tcgen05 tensor cores with a fused epilogue: bfloat16 result
    (+ bias); or added into the float32 tensor ``accumulate_into``; or, with ``swiglu`` and
    w = [gate rows; up rows], silu(gate) * up as bfloat16 [M, N / 2].  ``orientation``: "rows" puts
    the rows of ``a`` on the accumulator's lanes, "pairs" the same with 256 rows to a pair of CTAs
    (``cta_group::2``), "swapped" the rows of ``w`` (for up to a few hundred rows of ``a``); None
    chooses by M."""
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a", torch.bfloat16); _need(w, "w", torch.bfloat16, (N, K))
    if bias is not None:
        _need(bias, "bias", None, (N,))
    if accumulate_into is not None:
        _need(accumulate_into, "accumulate_into", torch.float32, (M, N))
        out, epilogue = accumulate_into, 1
    elif swiglu:
        out, epilogue = torch.empty(M, N // 2, dtype=torch.bfloat16, device=a.device), 2
    else:
        out, epilogue = torch.empty(M, N, dtype=torch.bfloat16, device=a.device), 0
    if orientation == "splitk":                  # rows of w on the lanes, K cut over a cluster (up to 64 rows of a)
        check(extras().pe_gemm_splitk(a.data_ptr(), w.data_ptr(), _ptr(bias), 0 if bias is None else _code(bias, "bias"),
                                    out.data_ptr(), epilogue, M, N, K, status_ptr(a.device), stream_ptr()), "gemm_splitk")
        return out
    check(core().pe_gemm_tcgen05(a.data_ptr(), w.data_ptr(), _ptr(bias), 0 if bias is None else _code(bias, "bias"),
                                 out.data_ptr(), epilogue, M, N, K, ORIENTATION[orientation], status_ptr(a.device),
                                 stream_ptr()), "gemm_tcgen05")
    return out


GEMM_ROPE_HEAD_DIMS = (16, 32, 64, 128)      # a 128-row tile of the weight holds whole heads


def gemm_qkv_rope_store(a: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor], n_q: int, n_kv: int,
                        head_dim: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], tok_pos: torch.Tensor,
                        tok_row: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                        block_table: Optional[torch.Tensor], table_stride: int,
                        orientation: Optional[str] = None) -> torch.Tensor:
    """Rotated queries [M, n_q * head_dim] of bfloat16 rows ``a`` [M, K]: the q/k/v product with bias, the
    rotation of q and k and the write of keys and values into their cache pages in one tcgen05 kernel
    (the cache write is skipped when ``k_pool`` is None)."""
    M, K = a.shape
    N = (n_q + 2 * n_kv) * head_dim
    _need(a, "a", torch.bfloat16); _need(w_qkv, "w_qkv", torch.bfloat16, (N, K))
    if head_dim not in GEMM_ROPE_HEAD_DIMS and orientation != "splitk":
        raise KernelError(f"head size {head_dim} is not taken by the fused q/k/v product: {GEMM_ROPE_HEAD_DIMS} are")
    if b_qkv is not None:
        _need(b_qkv, "b_qkv", None, (N,))
    _need(tok_pos, "tok_pos", torch.int32, (M,)); _need(tok_row, "tok_row", torch.int32, (M,))
    if cos is not None:
        _need(cos, "cos", torch.float32); _need(sin, "sin", torch.float32, cos.shape)
        if cos.shape[1] != head_dim // 2:
            raise KernelError("cos/sin tables need head_dim/2 columns")
    store = k_pool is not None
    if store:
        _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
        _need(block_table, "block_table", torch.int32)
        if tuple(k_pool.shape[1:]) != (n_kv, PAGE, head_dim):
            raise KernelError(f"cache pool must be [pages, {n_kv}, {PAGE}, {head_dim}], not {tuple(k_pool.shape)}")
    q = torch.empty(M, n_q * head_dim, dtype=torch.bfloat16, device=a.device)
    if orientation == "splitk":
        check(extras().pe_gemm_splitk_rope(a.data_ptr(), w_qkv.data_ptr(), _ptr(b_qkv), 0 if b_qkv is None else _code(b_qkv, "b_qkv"),
                                         q.data_ptr(), M, K, n_q, n_kv, head_dim, _ptr(cos), _ptr(sin), tok_pos.data_ptr(),
                                         tok_row.data_ptr(), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), table_stride,
                                         1 if store else 0, status_ptr(a.device), stream_ptr()), "gemm_splitk_rope")
        return q
    check(core().pe_gemm_tcgen05_rope(a.data_ptr(), w_qkv.data_ptr(), _ptr(b_qkv), 0 if b_qkv is None else _code(b_qkv, "b_qkv"),
                                      q.data_ptr(), M, K, n_q, n_kv, head_dim, _ptr(cos), _ptr(sin), tok_pos.data_ptr(),
                                      tok_row.data_ptr(), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), table_stride,
                                      1 if store else 0, ORIENTATION[orientation], status_ptr(a.device), stream_ptr()),
          "gemm_qkv_rope_store")
    return q
