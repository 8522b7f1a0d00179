"""Tensor-level faces of the CUDA kernels.

Each function checks device, dtype and layout, then launches on torch's current
stream. Nothing here computes with torch: a tensor that is not on a CUDA device
is an error, not a cue to fall back.
"""

from __future__ import annotations

import torch

from matricxon_b200.ops.library import KernelLibraryError, check, library

F32, BF16 = 0, 1
EPILOGUE_NONE, EPILOGUE_GELU, EPILOGUE_RESIDUAL, EPILOGUE_F32 = 0, 1, 2, 3

launch_count = 0      # kernels of this library launched so far in this process


def _launched(n: int = 1) -> None:
    global launch_count
    launch_count += n


STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a cache slot outside the pool",
               4: "a block-table entry that names no page", 8: "a device-side wait ran out"}


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelLibraryError(f"kernels take float32 or bfloat16, not {dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index: int | None = None


def _stream() -> int:
    """The current stream's handle. ``torch.cuda.current_stream()`` builds a Python object and looks the
    device up through several layers on every call (a third of a prompt step's host time when asked
    once per launch); the raw query is one C call. One device per process."""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype: torch.dtype | None = None, contiguous: bool = True):
    if not t.is_cuda:
        raise KernelLibraryError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelLibraryError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelLibraryError(f"{name} must be contiguous")


def set_chained_launch(on: bool) -> None:
    """Programmatic dependent launch for the kernels launched from here on (decode kernels only
    take part): what a graph captures stays with the graph."""
    library().mx_set_chained_launch(1 if on else 0)


def describe_status(word: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if word & bit) or "no error"


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
          scale: float = 1.0) -> None:
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    _need(out, "out", torch.float32)
    _need(status, "status", torch.int32)
    n, hidden = out.shape
    assert ids.numel() == n and table.shape[1] == hidden
    check(library().mx_embed(_ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(out), n, hidden,
                             table.shape[0], float(scale), _ptr(status), _stream()), "embed")
    _launched()


def softcap(logits: torch.Tensor, cap: float) -> None:
    """logits <- cap * tanh(logits / cap) in place (float32)."""
    _need(logits, "logits", torch.float32)
    check(library().mx_softcap(_ptr(logits), logits.numel(), float(cap), _stream()), "softcap")
    _launched()


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, eps: float,
              out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """out[r] = LayerNorm(x[rows[r]] if rows is given else x[r]); x is the float residual stream."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _need(out, "out")
    n_rows, hidden = out.shape
    assert x.shape[1] == hidden and weight.numel() == hidden
    assert rows is None or rows.numel() == n_rows
    assert rows is not None or x.shape[0] == n_rows
    check(library().mx_layernorm(_ptr(x), _ptr(rows), _ptr(weight), _ptr(bias), _ptr(out),
                                 dtype_code(out.dtype), n_rows, hidden, float(eps), _stream()),
          "layernorm")
    _launched()


def layernorm_sum(x: torch.Tensor, acc: torch.Tensor, col_bias: torch.Tensor | None, weight: torch.Tensor,
                  bias: torch.Tensor | None, eps: float, out: torch.Tensor) -> None:
    """``x += acc + col_bias`` (the residual epilogue of a product whose float accumulator is ``acc``),
    then ``out = LayerNorm(x)``, in one pass over the rows."""
    _need(x, "x", torch.float32)
    _need(acc, "acc", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(out, "out")
    assert acc.shape == x.shape and out.shape == x.shape, (x.shape, acc.shape, out.shape)
    if col_bias is not None:
        _need(col_bias, "col_bias", torch.float32)
        assert col_bias.numel() == x.shape[1]
    if bias is not None:
        _need(bias, "bias", torch.float32)
    check(library().mx_layernorm_sum(_ptr(x), _ptr(acc), _ptr(col_bias), _ptr(weight), _ptr(bias), _ptr(out),
                                     dtype_code(out.dtype), x.shape[0], x.shape[1], float(eps), _stream()),
          "layernorm_sum")
    _launched()


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                  slots: torch.Tensor | None, cache: torch.Tensor | None, n_heads: int,
                  n_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                  status: torch.Tensor, bias: torch.Tensor | None = None) -> None:
    """Rotates q (and k) of each row of ``qkv`` in float; writes k and v to the cache pages.

    ``cache`` is [pages, 2, kv heads, page_size, head_dim]; None rotates q only. ``bias`` (float32,
    one per column of ``qkv``): the bias of the product that made ``qkv``, still to be added; each
    sum is rounded to the dtype of ``qkv`` before it is used, as a separate epilogue would."""
    _need(qkv, "qkv")
    _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    _need(status, "status", torch.int32)
    n = qkv.shape[0]
    assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert inv_freq.numel() == rotary_dim // 2
    write = cache is not None
    n_pages = 0
    if write:
        _need(cache, "cache", qkv.dtype)
        _need(slots, "slots", torch.int32)
        assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim), cache.shape
        n_pages = cache.shape[0]
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == qkv.shape[1]
    check(library().mx_rope_kv_write_bias(_ptr(qkv), dtype_code(qkv.dtype), qkv.stride(0),
                                          _ptr(positions), _ptr(inv_freq), _ptr(slots), _ptr(cache), n,
                                          n_heads, n_kv_heads, head_dim, rotary_dim, page_size, n_pages,
                                          1 if write else 0, _ptr(status), _ptr(bias), _stream()),
          "rope_kv_write")
    _launched()


def epilogue(acc: torch.Tensor, bias: torch.Tensor | None, residual: torch.Tensor | None,
             out: torch.Tensor, mode: int) -> None:
    _need(acc, "acc")
    _need(out, "out")
    n_rows, n_cols = acc.shape
    check(library().mx_epilogue(_ptr(acc), dtype_code(acc.dtype), _ptr(bias), _ptr(residual),
                                _ptr(out), dtype_code(out.dtype), n_rows, n_cols, mode, _stream()),
          "epilogue")
    _launched()


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
              residual: torch.Tensor | None, out: torch.Tensor, mode: int) -> None:
    """out = epilogue(a @ w.T + bias) with float accumulation on the FP32 cores."""
    _need(a, "a", contiguous=False)
    _need(w, "w")
    _need(out, "out")
    if a.stride(1) != 1:
        raise KernelLibraryError("a must have unit stride along K")
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n), (a.shape, w.shape, out.shape)
    assert w.dtype == a.dtype
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == n
    if residual is not None:
        _need(residual, "residual", torch.float32)
        assert tuple(residual.shape) == (m, n)
    check(library().mx_gemm_simt(_ptr(a), _ptr(w), dtype_code(a.dtype), _ptr(bias), _ptr(residual),
                                 _ptr(out), dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0),
                                 out.stride(0), mode, _stream()), "gemm_simt")
    _launched()


_default_status: dict[int, torch.Tensor] = {}


def default_status(device: torch.device) -> torch.Tensor:
    """The status word kernels with bounded waits report to when the caller names none; a step
    runner registers its own with ``set_default_status`` so that one read covers everything."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _default_status:
        _default_status[index] = torch.zeros(1, dtype=torch.int32, device=device)
    return _default_status[index]


def set_default_status(status: torch.Tensor) -> None:
    _default_status[status.device.index if status.device.index is not None
                    else torch.cuda.current_device()] = status


def tcgen05_gemm_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
                 residual: torch.Tensor | None, out: torch.Tensor, mode: int,
                 status: torch.Tensor | None = None) -> None:
    """The prompt-sized product on the tcgen05 tensor cores: TMA-fed, accumulator in tensor
    memory, epilogue fused."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(out, "out")
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n), (a.shape, w.shape, out.shape)
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == n
    if residual is not None:
        _need(residual, "residual", torch.float32)
        assert tuple(residual.shape) == (m, n) and residual.stride(0) == out.stride(0)
    if status is None:
        status = default_status(a.device)
    check(library().mx_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                    dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0),
                                    out.stride(0), mode, _ptr(status), _stream()), "gemm_tcgen05")
    _launched()


def gemm_tcgen05_force_tiles(rows: int) -> None:
    """Makes ``gemm_tcgen05`` use its 128-, 256- or 512-row kernel wherever the shape allows it; 0
    gives the choice back to the shape. For tests that run all three on the same product."""
    check(library().mx_gemm_tcgen05_force_tiles(int(rows)), "gemm_tcgen05_force_tiles")


_sm_counts: dict[int, int] = {}


def sm_count(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def stream_gemm_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and 0 < a.shape[0] <= 128 and a.shape[1] % 8 == 0 and a.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_stream(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
                residual: torch.Tensor | None, out: torch.Tensor, mode: int,
                status: torch.Tensor | None = None) -> None:
    """The product for up to 128 rows (decoding, short prompt portions): the weight matrix is streamed
    from HBM once, dealt out evenly over the SMs, through TMA into tcgen05 products with the tokens
    as the narrow side; the epilogue is fused. A row's result does not depend on the other rows."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(out, "out")
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n), (a.shape, w.shape, out.shape)
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == n
    if residual is not None:
        _need(residual, "residual", torch.float32)
        assert tuple(residual.shape) == (m, n) and residual.stride(0) == out.stride(0)
    if status is None:
        status = default_status(a.device)
    check(library().mx_gemm_stream(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                   dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0),
                                   out.stride(0), mode, _ptr(status), _stream()), "gemm_stream")
    _launched()


def skinny_gemm_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[0] <= 16 and a.shape[1] % 32 == 0
            and a.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
                residual: torch.Tensor | None, out: torch.Tensor, mode: int) -> None:
    """The decode product: at most 16 rows of bfloat16 ``a`` against all of ``w``, streamed once,
    with the epilogue fused."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(out, "out")
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n), (a.shape, w.shape, out.shape)
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == n
    if residual is not None:
        _need(residual, "residual", torch.float32)
        assert tuple(residual.shape) == (m, n) and residual.stride(0) == out.stride(0)
    check(library().mx_gemm_skinny(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                                   dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0),
                                   out.stride(0), mode, _stream()), "gemm_skinny")
    _launched()


def gemm_skinny_rope(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, qkv: torch.Tensor,
                     positions: torch.Tensor, inv_freq: torch.Tensor, slots: torch.Tensor | None,
                     cache: torch.Tensor | None, n_heads: int, n_kv_heads: int, head_dim: int,
                     page_size: int, status: torch.Tensor) -> None:
    """The decode QKV product with the rotation and the cache write in its epilogue: rotated
    queries go to the query columns of ``qkv``, rotated keys and the values to ``slots`` of
    ``cache`` (both None: nothing stored). The rotation spans the whole head."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(qkv, "qkv", torch.bfloat16)
    _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    _need(status, "status", torch.int32)
    m, k = a.shape
    n = (n_heads + 2 * n_kv_heads) * head_dim
    assert tuple(w.shape) == (n, k) and tuple(qkv.shape) == (m, n), (a.shape, w.shape, qkv.shape)
    assert inv_freq.numel() == head_dim // 2 and positions.numel() >= m
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == n
    n_pages = 0
    if cache is not None:
        _need(cache, "cache", torch.bfloat16)
        _need(slots, "slots", torch.int32)
        assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim), cache.shape
        n_pages = cache.shape[0]
    check(library().mx_gemm_skinny_rope(_ptr(a), _ptr(w), _ptr(bias), _ptr(qkv), m, k, a.stride(0),
                                        w.stride(0), qkv.stride(0), _ptr(positions), _ptr(inv_freq),
                                        _ptr(slots) if cache is not None else None, _ptr(cache), n_pages,
                                        n_heads, n_kv_heads, head_dim, page_size, _ptr(status), _stream()),
          "gemm_skinny_rope")
    _launched()


def attention_scratch_bytes(n_tokens: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return int(library().mx_attention_scratch_bytes(n_tokens, n_heads, head_dim, n_splits))


def paged_attention(q: torch.Tensor, q_stride: int, cache: torch.Tensor, block_tables: torch.Tensor,
                    tok_seq: torch.Tensor, positions: torch.Tensor, n_tokens: int, n_heads: int,
                    n_kv_heads: int, head_dim: int, window: int | None, scale: float,
                    out: torch.Tensor, status: torch.Tensor, n_splits: int = 1,
                    scratch: torch.Tensor | None = None) -> None:
    """Attention of ``n_tokens`` query rows over the paged cache.

    ``q`` points at the first query head of row 0 and rows are ``q_stride`` elements apart
    (so the q part of a fused qkv buffer can be used in place). ``out`` is [tokens, heads * dim].
    """
    _need(q, "q", contiguous=False)
    _need(cache, "cache", q.dtype)
    _need(block_tables, "block_tables", torch.int32)
    _need(tok_seq, "tok_seq", torch.int32)
    _need(positions, "positions", torch.int32)
    _need(out, "out", q.dtype)
    _need(status, "status", torch.int32)
    page_size = cache.shape[3]
    assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim), cache.shape
    assert out.shape[1] == n_heads * head_dim and out.shape[0] >= n_tokens
    if n_splits > 1:
        need = attention_scratch_bytes(n_tokens, n_heads, head_dim, n_splits)
        if scratch is None or scratch.numel() * scratch.element_size() < need:
            raise KernelLibraryError(f"attention with {n_splits} splits needs {need} bytes of scratch")
        _need(scratch, "scratch", torch.float32)
    check(library().mx_paged_attention(
        _ptr(q), dtype_code(q.dtype), q_stride, _ptr(cache), cache.shape[0], page_size,
        _ptr(block_tables), block_tables.stride(0), _ptr(tok_seq), _ptr(positions), n_tokens,
        n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), _ptr(out), out.stride(0),
        n_splits, _ptr(scratch), _ptr(status), _stream()), "paged_attention")
    _launched(2 if n_splits > 1 else 1)


def attention_tile_lists(q_lens: list[int], group: int,
                         token_tiles: bool = False) -> tuple[list[int], list[int]]:
    """Row tiles of the tensor-core attention for sequences that bring ``q_lens`` tokens and
    ``group`` query heads per KV head. Sequences with at most 16 rows (decode tokens) go to the
    narrow list, one (sequence, 0) tile each. The others go to the wide list: cut into 64-row
    tiles as (sequence, first row) pairs, or, with ``token_tiles`` (the tcgen05 kernel), into
    tiles of 128 // group tokens as (sequence, first token) pairs, the latest tokens first
    because they have the most keys to walk."""
    narrow: list[int] = []
    wide: list[int] = []
    per_tile = max(1, 128 // group)
    for seq, q_len in enumerate(q_lens):
        rows = q_len * group
        if rows <= 0:
            continue
        if rows <= 16:
            narrow.extend((seq, 0))
        elif token_tiles:
            for token in range((q_len - 1) // per_tile * per_tile, -1, -per_tile):
                wide.extend((seq, token))
        else:
            for row in range(0, rows, 64):
                wide.extend((seq, row))
    return narrow, wide


def tc_attention_supported(dtype: torch.dtype, head_dim: int, page_size: int, q_stride: int,
                           group: int) -> bool:
    """Whether prompt portions can run on the tcgen05 attention kernel."""
    return (dtype == torch.bfloat16 and head_dim == 128 and page_size in (16, 32)
            and q_stride % 8 == 0 and 1 <= group <= 128)


def paged_attention_tc(q: torch.Tensor, q_stride: int, cache: torch.Tensor, block_tables: torch.Tensor,
                       cu_q: torch.Tensor, context_lens: torch.Tensor, tiles: torch.Tensor, n_tiles: int,
                       n_tokens: int, n_heads: int, n_kv_heads: int, head_dim: int, window: int | None,
                       scale: float, out: torch.Tensor, status: torch.Tensor, n_splits: int = 1,
                       scratch: torch.Tensor | None = None) -> None:
    """Attention of prompt portions on tcgen05 (bfloat16, head_dim 128, pages of 16 or 32).
    ``tiles`` is int32 [n_tiles, 2]: (sequence, first token) of tiles of 128 // group tokens
    (``attention_tile_lists(..., token_tiles=True)``); ``q`` holds the step's rows, query head h
    at column h * head_dim. ``n_splits`` > 1 shares every tile's keys out between that many blocks
    (few tiles, long contexts); ``scratch`` (float32, ``attention_scratch_bytes``) takes their parts."""
    _need(q, "q", torch.bfloat16, contiguous=False)
    _need(cache, "cache", torch.bfloat16)
    for name, tensor in (("block_tables", block_tables), ("cu_q", cu_q),
                         ("context_lens", context_lens), ("tiles", tiles), ("status", status)):
        _need(tensor, name, torch.int32)
    _need(out, "out", torch.bfloat16)
    page_size = cache.shape[3]
    assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim), cache.shape
    assert out.shape[1] == n_heads * head_dim and out.shape[0] >= n_tokens and q.shape[0] >= n_tokens
    assert tiles.numel() >= 2 * n_tiles
    if n_splits > 1:
        _need(scratch, "scratch", torch.float32)
        assert scratch.numel() * 4 >= attention_scratch_bytes(n_tokens, n_heads, head_dim, n_splits)
    check(library().mx_paged_attention_tc_split(
        _ptr(q), q_stride, _ptr(cache), cache.shape[0], page_size, _ptr(block_tables),
        block_tables.stride(0), _ptr(cu_q), _ptr(context_lens), _ptr(tiles), n_tiles, n_tokens,
        n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), _ptr(out), out.stride(0),
        int(n_splits), _ptr(scratch) if n_splits > 1 else None, _ptr(status), _stream()),
        "paged_attention_tc")
    _launched()


def paged_attention_mma(q: torch.Tensor, q_stride: int, cache: torch.Tensor,
                        block_tables: torch.Tensor, cu_q: torch.Tensor, context_lens: torch.Tensor,
                        tiles: torch.Tensor, n_tiles: int, narrow: bool, n_tokens: int, n_heads: int,
                        n_kv_heads: int, head_dim: int, window: int | None, scale: float,
                        out: torch.Tensor, status: torch.Tensor, n_splits: int = 1,
                        scratch: torch.Tensor | None = None) -> None:
    """Tensor-core attention (bfloat16, head_dim 64 or 128). ``tiles`` is int32 [n_tiles, 2]:
    (sequence, first row) of each tile of the (token, head-in-group) rows; ``narrow`` tiles
    hold at most 16 rows, the others 64 (see ``attention_tile_lists``)."""
    _need(q, "q", torch.bfloat16, contiguous=False)
    _need(cache, "cache", torch.bfloat16)
    for name, tensor in (("block_tables", block_tables), ("cu_q", cu_q),
                         ("context_lens", context_lens), ("status", status)):
        _need(tensor, name, torch.int32)
    _need(out, "out", torch.bfloat16)
    page_size = cache.shape[3]
    assert tuple(cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim), cache.shape
    assert out.shape[1] == n_heads * head_dim and out.shape[0] >= n_tokens
    if tiles is None:
        # no list: tile i is the whole of sequence i (narrow tiles only: every sequence brings at most 16 rows)
        assert narrow and n_tiles <= context_lens.numel()
    else:
        _need(tiles, "tiles", torch.int32)
        assert tiles.numel() >= 2 * n_tiles
    if n_splits > 1:
        need = attention_scratch_bytes(n_tokens, n_heads, head_dim, n_splits)
        if scratch is None or scratch.numel() * scratch.element_size() < need:
            raise KernelLibraryError(f"attention with {n_splits} splits needs {need} bytes of scratch")
        _need(scratch, "scratch", torch.float32)
    check(library().mx_paged_attention_mma(
        _ptr(q), q_stride, _ptr(cache), cache.shape[0], page_size, _ptr(block_tables),
        block_tables.stride(0), _ptr(cu_q), _ptr(context_lens), _ptr(tiles) if tiles is not None else None, n_tiles,
        1 if narrow else 0, n_tokens, n_heads, n_kv_heads, head_dim, int(window or 0), float(scale),
        _ptr(out), out.stride(0), n_splits, _ptr(scratch), _ptr(status), _stream()),
        "paged_attention_mma")
    _launched(2 if n_splits > 1 else 1)


def mma_attention_supported(dtype: torch.dtype, head_dim: int, page_size: int, q_stride: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and page_size in (8, 16, 32)
            and q_stride % 8 == 0)
