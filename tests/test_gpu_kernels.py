"""Each CUDA kernel alone against a plain float64 reference, at sizes other than the engine's."""

import math

import pytest
import torch

from plain_reference import (
    plain_apply_rope,
    plain_attention_core,
    plain_gelu_tanh,
    plain_layernorm,
    plain_rope_tables,
)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def kernels():
    from matricxon_b200.ops import kernels as k

    return k


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def tol(dtype):
    return dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("hidden", [96, 100, 3072])          # 16-byte rows (the vector kernel) and not
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype, hidden):
    k = kernels()
    table = torch.randn(1000, hidden, device=DEV).to(dtype)
    ids = torch.tensor([0, 999, 17, 17, 500], dtype=torch.int32, device=DEV)
    out = torch.empty(5, hidden, device=DEV)
    st = status()
    k.embed(ids, table, out, st)
    assert torch.equal(out, table[ids.long()].float()) and st.item() == 0
    k.embed(ids, table, out, st, scale=3.0)
    assert torch.equal(out, table[ids.long()].float() * 3.0) and st.item() == 0
    bad = torch.tensor([3, 1000, -1], dtype=torch.int32, device=DEV)
    out = torch.full((3, hidden), float("nan"), device=DEV)
    k.embed(bad, table, out, st)
    assert st.item() == 1 and torch.all(out[1:] == 0) and torch.equal(out[0], table[3].float())


def test_softcap():
    k = kernels()
    logits = torch.randn(7, 1003, device=DEV) * 40
    expected = 30.0 * torch.tanh(logits.double() / 30.0)
    k.softcap(logits, 30.0)
    assert torch.allclose(logits.double(), expected, atol=1e-4)


# ------------------------------------------------------------------ LayerNorm
@pytest.mark.parametrize("hidden", [16, 100, 3072, 6144])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layernorm(hidden, dtype):
    k = kernels()
    torch.manual_seed(hidden)
    x = (torch.randn(37, hidden, device=DEV) * 3 + 5)        # a mean far from zero
    w = 1 + 0.1 * torch.randn(hidden, device=DEV)
    b = 0.1 * torch.randn(hidden, device=DEV)
    out = torch.empty(37, hidden, dtype=dtype, device=DEV)
    k.layernorm(x, w, b, 1e-6, out)
    ref = plain_layernorm(x.double().cpu(), w.double().cpu(), b.double().cpu(), 1e-6)
    assert torch.allclose(out.double().cpu(), ref, **tol(dtype))
    # without bias, and on gathered rows
    rows = torch.tensor([36, 0, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(3, hidden, dtype=dtype, device=DEV)
    k.layernorm(x, w, None, 1e-5, out, rows)
    ref = plain_layernorm(x.double().cpu()[[36, 0, 5]], w.double().cpu(), None, 1e-5)
    assert torch.allclose(out.double().cpu(), ref, **tol(dtype))


@pytest.mark.parametrize("hidden,rows", [(64, 37), (3072, 64), (3072, 300), (1002, 33), (96, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("with_bias", [True, False])
def test_layernorm_that_adds_up_the_residual_sum_first(hidden, rows, dtype, with_bias):
    """``x += acc + col_bias; out = LayerNorm(x)`` in one launch against the epilogue kernel followed by the
    norm: the same x and the same out, bit for bit (1002 columns take the general kernels)."""
    k = kernels()
    torch.manual_seed(hidden + rows)
    x = torch.randn(rows, hidden, device=DEV) * 3 + 5
    acc = torch.randn(rows, hidden, device=DEV)
    col_bias = torch.randn(hidden, device=DEV) if with_bias else None
    w = 1 + 0.1 * torch.randn(hidden, device=DEV)
    b = 0.1 * torch.randn(hidden, device=DEV)
    x_two = x.clone()
    k.epilogue(acc, col_bias, x_two, x_two, k.EPILOGUE_RESIDUAL)
    out_two = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    k.layernorm(x_two, w, b, 1e-5, out_two)
    x_one = x.clone()
    out_one = torch.full((rows, hidden), float("nan"), dtype=dtype, device=DEV)
    k.layernorm_sum(x_one, acc, col_bias, w, b, 1e-5, out_one)
    assert torch.equal(x_one, x_two)
    assert torch.equal(out_one, out_two)
    total = x.double().cpu() + acc.double().cpu() + (col_bias.double().cpu() if with_bias else 0)
    assert torch.allclose(x_one.double().cpu(), total, atol=1e-5, rtol=1e-6)
    ref = plain_layernorm(total, w.double().cpu(), b.double().cpu(), 1e-5)
    assert torch.allclose(out_one.double().cpu(), ref, **tol(dtype))


# ------------------------------------------------------------------ FP32-core GEMM
@pytest.mark.parametrize("m,n,k_dim", [(1, 1000, 96), (7, 130, 352), (65, 64, 17), (200, 3584, 300)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_simt_all_epilogues(m, n, k_dim, dtype):
    k = kernels()
    torch.manual_seed(m * n)
    a = torch.randn(m, k_dim, device=DEV).to(dtype)
    w = (torch.randn(n, k_dim, device=DEV) / math.sqrt(k_dim)).to(dtype)
    bias = torch.randn(n, device=DEV)
    residual = torch.randn(m, n, device=DEV)
    acc = a.double().cpu() @ w.double().cpu().T + bias.double().cpu()
    out = torch.empty(m, n, dtype=dtype, device=DEV)
    k.gemm_simt(a, w, bias, None, out, k.EPILOGUE_NONE)
    assert torch.allclose(out.double().cpu(), acc, **tol(dtype))
    k.gemm_simt(a, w, bias, None, out, k.EPILOGUE_GELU)
    assert torch.allclose(out.double().cpu(), plain_gelu_tanh(acc), **tol(dtype))
    out32 = residual.clone()
    k.gemm_simt(a, w, bias, out32, out32, k.EPILOGUE_RESIDUAL)          # in place
    assert torch.allclose(out32.double().cpu(), acc + residual.double().cpu(), atol=2e-5, rtol=1e-5)
    k.gemm_simt(a, w, None, None, out32, k.EPILOGUE_F32)
    assert torch.allclose(out32.double().cpu(), acc - bias.double().cpu(), atol=2e-5, rtol=1e-5)


def test_gemm_simt_row_result_does_not_depend_on_the_batch():
    k = kernels()
    a = torch.randn(70, 300, device=DEV)
    w = torch.randn(130, 300, device=DEV)
    whole = torch.empty(70, 130, device=DEV)
    k.gemm_simt(a, w, None, None, whole, k.EPILOGUE_F32)
    one = torch.empty(1, 130, device=DEV)
    k.gemm_simt(a[33:34], w, None, None, one, k.EPILOGUE_F32)
    assert torch.equal(one[0], whole[33])


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
# (3584, 3072) and (160, 1088) take the kernel with more loads in flight (few blocks, a long K); the second
# leaves its warps with five and four pieces of K
@pytest.mark.parametrize("n,k_dim", [(3584, 3072), (160, 1088), (1000, 96), (50, 352), (17, 32)])
def test_skinny_gemm_all_epilogues(m, n, k_dim):
    """The decode product against float64, all epilogues, rows and columns that fill no tile."""
    k = kernels()
    torch.manual_seed(m * n + k_dim)
    a = torch.randn(m, k_dim, device=DEV).bfloat16()
    w = (torch.randn(n, k_dim, device=DEV) / math.sqrt(k_dim)).bfloat16()
    bias = torch.randn(n, device=DEV)
    residual = torch.randn(m, n, device=DEV)
    assert k.skinny_gemm_supported(a, w)
    acc = a.double().cpu() @ w.double().cpu().T + bias.double().cpu()
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.gemm_skinny(a, w, bias, None, out, k.EPILOGUE_NONE)
    assert torch.allclose(out.double().cpu(), acc, **tol(torch.bfloat16))
    k.gemm_skinny(a, w, bias, None, out, k.EPILOGUE_GELU)
    assert torch.allclose(out.double().cpu(), plain_gelu_tanh(acc), **tol(torch.bfloat16))
    out32 = residual.clone()
    k.gemm_skinny(a, w, bias, out32, out32, k.EPILOGUE_RESIDUAL)
    assert torch.allclose(out32.double().cpu(), acc + residual.double().cpu(), atol=1e-4, rtol=1e-5)
    k.gemm_skinny(a, w, None, None, out32, k.EPILOGUE_F32)
    assert torch.allclose(out32.double().cpu(), acc - bias.double().cpu(), atol=1e-4, rtol=1e-5)
    # a row's result does not depend on the rest of the batch
    one = torch.empty(1, n, device=DEV)
    k.gemm_skinny(a[m - 1:m], w, None, None, one, k.EPILOGUE_F32)
    assert torch.equal(one[0], out32[m - 1])
    # rows of a wider buffer (the q part of a fused qkv row, say)
    wide = torch.randn(m, k_dim + 64, device=DEV).bfloat16()
    view = wide[:, 32:32 + k_dim]
    if k.skinny_gemm_supported(view, w):
        k.gemm_skinny(view, w, None, None, out32, k.EPILOGUE_F32)
        assert torch.allclose(out32.double().cpu(), view.double().cpu() @ w.double().cpu().T, atol=1e-4, rtol=1e-5)
    assert not k.skinny_gemm_supported(torch.zeros(17, 64, device=DEV).bfloat16(), w[:, :64].contiguous()) \
        or k_dim < 64


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
@pytest.mark.parametrize("n", [1000, 1002])                  # four columns per thread; one at a time
def test_library_product_with_epilogue(mode, n):
    from matricxon_b200.ops.linear import linear

    torch.manual_seed(mode)
    a = torch.randn(33, 96, device=DEV).bfloat16()
    w = (torch.randn(n, 96, device=DEV) / 10).bfloat16()
    bias = torch.randn(n, device=DEV)
    residual = torch.randn(33, n, device=DEV)
    acc = a.double().cpu() @ w.double().cpu().T + bias.double().cpu()
    expected = [acc, plain_gelu_tanh(acc), acc + residual.double().cpu(), acc][mode]
    out = linear(a, w, bias, mode, residual=residual.clone() if mode == 2 else None, backend="library")
    assert out.dtype == (torch.float32 if mode >= 2 else torch.bfloat16)
    assert torch.allclose(out.double().cpu(), expected, atol=3e-2, rtol=2e-2)


# ------------------------------------------------------------------ rotary + cache write
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,rot", [(4, 2, 16, 16), (3, 1, 32, 32), (6, 3, 48, 32), (24, 2, 128, 128)])
def test_rope_kv_write(dtype, heads, kv_heads, dim, rot):
    k = kernels()
    torch.manual_seed(dim)
    n, page_size, pages = 9, 4, 7
    theta = 100000.0
    qkv = torch.randn(n, (heads + 2 * kv_heads) * dim, device=DEV).to(dtype)
    original = qkv.clone()
    positions = torch.tensor([0, 1, 2, 3, 500, 4095, 16000, 7, 8], dtype=torch.int32, device=DEV)
    slots = torch.tensor([5, 6, 7, 0, 27, 13, 12, 1, 2], dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV)
    cache = torch.full((pages, 2, kv_heads, page_size, dim), float("nan"), dtype=dtype, device=DEV)
    st = status()
    k.rope_kv_write(qkv, positions, inv_freq, slots, cache, heads, kv_heads, dim, rot, page_size, st)
    assert st.item() == 0

    src = original.double().cpu()
    q = src[:, : heads * dim].view(n, heads, dim).transpose(0, 1)
    kk = src[:, heads * dim: (heads + kv_heads) * dim].view(n, kv_heads, dim).transpose(0, 1)
    vv = src[:, (heads + kv_heads) * dim:].view(n, kv_heads, dim).transpose(0, 1)
    cos, sin = plain_rope_tables(positions.cpu(), rot, theta)

    def rotate(x):
        out = x.clone()
        out[..., :rot] = plain_apply_rope(x[..., :rot], cos, sin)
        return out

    q_ref, k_ref = rotate(q), rotate(kk)
    got_q = qkv[:, : heads * dim].double().cpu().view(n, heads, dim).transpose(0, 1)
    assert torch.allclose(got_q, q_ref, **tol(dtype))
    # v part of the row is untouched, k part of the row is untouched (only the cache gets rotated k)
    assert torch.equal(qkv[:, heads * dim:], original[:, heads * dim:])
    from matricxon_b200.cache.storage import keys_view, values_view

    keys, values = keys_view(cache), values_view(cache)       # [p, h, slot, d] and [p, h, d, slot]
    for t in range(n):
        page, off = divmod(int(slots[t]), page_size)
        assert torch.allclose(keys[page, :, off].double().cpu(), k_ref[:, t], **tol(dtype))
        assert torch.equal(values[page, :, :, off].double().cpu(), vv[:, t])
    written = torch.zeros(pages * page_size, dtype=torch.bool)
    written[slots.cpu().long()] = True
    for flat in (keys.permute(0, 2, 1, 3).reshape(pages * page_size, -1),
                 values.permute(0, 3, 1, 2).reshape(pages * page_size, -1)):
        assert torch.isnan(flat[~written]).all() and not torch.isnan(flat[written]).any()


@pytest.mark.parametrize("m", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("heads,kv_heads,dim,k_dim,with_bias", [(6, 2, 64, 192, True), (3, 1, 16, 96, False),
                                                               (4, 4, 128, 256, True), (5, 1, 48, 160, True),
                                                               (24, 2, 128, 3072, True), (2, 1, 128, 1536, False)])
def test_skinny_gemm_with_rotation_equals_product_then_rope(m, heads, kv_heads, dim, k_dim, with_bias):
    """The QKV product with rotation and cache write in its epilogue against the plain product
    followed by the rotary kernel (each checked against float64 above): same queries, same cache."""
    k = kernels()
    torch.manual_seed(m * 131 + dim)
    n = (heads + 2 * kv_heads) * dim
    page_size, pages = 4, 9
    a = torch.randn(m, k_dim, device=DEV).bfloat16()
    w = (torch.randn(n, k_dim, device=DEV) / math.sqrt(k_dim)).bfloat16()
    bias = torch.randn(n, device=DEV) if with_bias else None
    positions = torch.tensor([0, 1, 2, 3, 500, 4095, 16000, 7, 8, 9, 33, 34, 35, 36, 37, 38][:m], dtype=torch.int32, device=DEV)
    slot_list = [5, 6, 7, 0, 27, 13, 12, 1, 2, -1, 20, 21, 22, 23, 30, 31][:m]
    slots = torch.tensor(slot_list, dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / (100000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))).to(DEV)
    st = status()
    # the two kernels one after the other
    qkv_ref = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    k.gemm_skinny(a, w, bias, None, qkv_ref, k.EPILOGUE_NONE)
    cache_ref = torch.full((pages, 2, kv_heads, page_size, dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.rope_kv_write(qkv_ref, positions, inv_freq, slots, cache_ref, heads, kv_heads, dim, dim, page_size, st)
    # the one kernel
    qkv = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    cache = torch.full((pages, 2, kv_heads, page_size, dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.gemm_skinny_rope(a, w, bias, qkv, positions, inv_freq, slots, cache, heads, kv_heads, dim, page_size, st)
    assert st.item() == 0
    q_cols = heads * dim
    assert torch.equal(qkv[:, :q_cols], qkv_ref[:, :q_cols])
    assert torch.isnan(qkv[:, q_cols:]).all()                        # key and value columns are not written
    assert torch.equal(torch.isnan(cache), torch.isnan(cache_ref))   # the same slots, nothing else
    assert torch.equal(torch.nan_to_num(cache), torch.nan_to_num(cache_ref))
    # without a cache only the queries are produced
    qkv2 = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.gemm_skinny_rope(a, w, bias, qkv2, positions, inv_freq, None, None, heads, kv_heads, dim, page_size, st)
    assert torch.equal(qkv2[:, :q_cols], qkv_ref[:, :q_cols])
    # a slot outside the pool is reported, not written
    bad = slots.clone()
    bad[0] = pages * page_size
    k.gemm_skinny_rope(a, w, bias, qkv2, positions, inv_freq, bad, cache, heads, kv_heads, dim, page_size, st)
    assert st.item() == 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,rot", [(4, 2, 16, 16), (6, 3, 48, 32), (3, 1, 20, 12), (24, 2, 128, 128)])
def test_rope_kv_write_adds_the_products_bias_like_an_epilogue_before_it(dtype, heads, kv_heads, dim, rot):
    """``bias=`` (the product ran without its epilogue) against the epilogue kernel followed by the
    rotation: the same rounding, so the same bits, in the queries and in the cache; with a rotary width
    below the head size (the tails need their bias too) and sizes that leave the 16-byte path."""
    k = kernels()
    torch.manual_seed(dim + rot)
    n, page_size, pages = 9, 4, 7
    cols = (heads + 2 * kv_heads) * dim
    raw = torch.randn(n, cols, device=DEV).to(dtype)
    bias = torch.randn(cols, device=DEV)
    positions = torch.tensor([0, 1, 2, 3, 500, 4095, 16000, 7, 8], dtype=torch.int32, device=DEV)
    slots = torch.tensor([5, 6, 7, 0, 27, 13, -1, 1, 2], dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV)
    st = status()
    two = torch.empty_like(raw)
    k.epilogue(raw, bias, None, two, k.EPILOGUE_NONE)
    cache_two = torch.full((pages, 2, kv_heads, page_size, dim), float("nan"), dtype=dtype, device=DEV)
    k.rope_kv_write(two, positions, inv_freq, slots, cache_two, heads, kv_heads, dim, rot, page_size, st)
    one = raw.clone()
    cache_one = torch.full((pages, 2, kv_heads, page_size, dim), float("nan"), dtype=dtype, device=DEV)
    k.rope_kv_write(one, positions, inv_freq, slots, cache_one, heads, kv_heads, dim, rot, page_size, st, bias=bias)
    assert st.item() == 0
    assert torch.equal(one[:, :heads * dim], two[:, :heads * dim])              # the queries, tails included
    assert torch.equal(torch.isnan(cache_one), torch.isnan(cache_two))
    assert torch.equal(torch.nan_to_num(cache_one), torch.nan_to_num(cache_two))
    # without a cache: queries only
    q_only = raw.clone()
    k.rope_kv_write(q_only, positions, inv_freq, None, None, heads, kv_heads, dim, rot, page_size, st, bias=bias)
    assert torch.equal(q_only[:, :heads * dim], two[:, :heads * dim])


def test_rope_bad_slot_sets_status_and_padding_slot_is_silent():
    k = kernels()
    qkv = torch.randn(3, 4 * 16, device=DEV)
    positions = torch.zeros(3, dtype=torch.int32, device=DEV)
    inv_freq = torch.ones(8, device=DEV)
    cache = torch.zeros(2, 2, 1, 4, 16, device=DEV)
    st = status()
    k.rope_kv_write(qkv, positions, inv_freq, torch.tensor([0, -1, 1], dtype=torch.int32, device=DEV),
                    cache, 2, 1, 16, 16, 4, st)
    assert st.item() == 0
    k.rope_kv_write(qkv, positions, inv_freq, torch.tensor([0, 8, 1], dtype=torch.int32, device=DEV),
                    cache, 2, 1, 16, 16, 4, st)
    assert st.item() == 2


# ------------------------------------------------------------------ paged attention
def paged_case(dtype, heads, kv_heads, dim, page_size, seq_lens, q_lens, seed, scale_up=None):
    """Random K/V for several sequences scattered over shuffled pages; the last q_len positions
    of each sequence are the queries. Returns kernel inputs and dense per-sequence tensors."""
    generator = torch.Generator().manual_seed(seed)
    n_seq = len(seq_lens)
    pages_per_seq = [(length + page_size - 1) // page_size for length in seq_lens]
    total_pages = sum(pages_per_seq) + 3
    order = torch.randperm(total_pages, generator=generator).tolist()
    width = max(pages_per_seq) + 1
    tables = torch.full((n_seq, width), -1, dtype=torch.int32)
    cache = torch.full((total_pages, 2, kv_heads, page_size, dim), float("nan"))
    dense = []
    cursor = 0
    for s, length in enumerate(seq_lens):
        ks = torch.randn(kv_heads, length, dim, generator=generator)
        vs = torch.randn(kv_heads, length, dim, generator=generator)
        qs = torch.randn(heads, q_lens[s], dim, generator=generator)
        if scale_up is not None:
            scale_up(s, qs, ks, vs)
        ks, vs, qs = ks.to(dtype).float(), vs.to(dtype).float(), qs.to(dtype).float()
        dense.append((qs, ks, vs))
        for lp in range(pages_per_seq[s]):
            page = order[cursor]
            cursor += 1
            tables[s, lp] = page
            lo, hi = lp * page_size, min(length, (lp + 1) * page_size)
            cache[page, 0, :, : hi - lo] = ks[:, lo:hi]
            # values are stored transposed: [kv head][dim][slot]
            cache[page, 1].view(kv_heads, dim, page_size)[:, :, : hi - lo] = vs[:, lo:hi].transpose(1, 2)
    q_rows, tok_seq, positions = [], [], []
    for s, (qs, _, _) in enumerate(dense):
        for i in range(q_lens[s]):
            q_rows.append(qs[:, i].reshape(-1))
            tok_seq.append(s)
            positions.append(seq_lens[s] - q_lens[s] + i)
    q = torch.stack(q_rows)
    return (q.to(dtype).to(DEV), cache.to(dtype).to(DEV), tables.to(DEV),
            torch.tensor(tok_seq, dtype=torch.int32, device=DEV),
            torch.tensor(positions, dtype=torch.int32, device=DEV), dense)


def reference_attention(dense, q_lens, seq_lens, scale, window):
    rows = []
    for (qs, ks, vs), q_len, length in zip(dense, q_lens, seq_lens):
        out = plain_attention_core(qs.double(), ks.double(), vs.double(), scale, window,
                                   offset=length - q_len)
        rows.append(out.transpose(0, 1).reshape(q_len, -1))
    return torch.cat(rows)


def run_attention(k, q, cache, tables, tok_seq, positions, heads, kv_heads, dim, window, scale, n_splits,
                  impl="simt"):
    n = q.shape[0]
    out = torch.full((n, heads * dim), float("nan"), dtype=q.dtype, device=DEV)
    st = status()
    scratch = None
    if n_splits > 1:
        need = k.attention_scratch_bytes(n, heads, dim, n_splits)
        scratch = torch.full((need // 4,), float("nan"), device=DEV)
    if impl == "simt":
        k.paged_attention(q, q.stride(0), cache, tables, tok_seq, positions, n, heads, kv_heads, dim,
                          window, scale, out, st, n_splits=n_splits, scratch=scratch)
        return out, st.item()
    # the tensor-core kernel takes per-sequence metadata and a list of 16-row tiles
    seq_ids = tok_seq.cpu().tolist()
    n_seq = max(seq_ids) + 1
    q_lens = [seq_ids.count(s) for s in range(n_seq)]
    cu_q = [0]
    for length in q_lens:
        cu_q.append(cu_q[-1] + length)
    pos = positions.cpu().tolist()
    context = [pos[cu_q[s]] for s in range(n_seq)]
    group = heads // kv_heads
    narrow, wide = k.attention_tile_lists(q_lens, group, token_tiles=(impl == "tc"))
    as_int = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for tiles, is_narrow, others in ((narrow, True, wide), (wide, False, narrow)):
        if not tiles:
            continue
        if impl == "tc" and not is_narrow:          # prompt portions on the tcgen05 kernel
            splits = n_splits if not others else 1
            k.paged_attention_tc(q, q.stride(0), cache, tables, as_int(cu_q), as_int(context), as_int(tiles),
                                 len(tiles) // 2, n, heads, kv_heads, dim, window, scale, out, st,
                                 n_splits=splits, scratch=scratch if splits > 1 else None)
            continue
        splits = n_splits if not others else 1      # splits need a launch that covers every token
        k.paged_attention_mma(q, q.stride(0), cache, tables, as_int(cu_q), as_int(context), as_int(tiles),
                              len(tiles) // 2, is_narrow, n, heads, kv_heads, dim, window, scale, out, st,
                              n_splits=splits, scratch=scratch)
    return out, st.item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,page_size", [
    (4, 2, 16, 16), (3, 1, 32, 16), (24, 2, 128, 16), (5, 5, 48, 8), (40, 2, 64, 32), (2, 1, 256, 16),
    (8, 8, 64, 16), (14, 2, 128, 64), (36, 4, 128, 16)])
@pytest.mark.parametrize("window", [None, 24, 100])
def test_paged_attention_mixed_batch(dtype, heads, kv_heads, dim, page_size, window):
    k = kernels()
    seq_lens, q_lens = [1, 37, 130, 64, 301], [1, 37, 1, 5, 2]
    scale = dim ** -0.5
    q, cache, tables, tok_seq, positions, dense = paged_case(
        dtype, heads, kv_heads, dim, page_size, seq_lens, q_lens, seed=dim + heads)
    ref = reference_attention(dense, q_lens, seq_lens, scale, window)
    for n_splits in (1, 3, 16):
        out, st = run_attention(k, q, cache, tables, tok_seq, positions, heads, kv_heads, dim,
                                window, scale, n_splits)
        assert st == 0
        assert torch.allclose(out.double().cpu(), ref, **tol(dtype)), (n_splits, (out.double().cpu() - ref).abs().max())


@pytest.mark.parametrize("heads,kv_heads,dim,page_size", [
    (24, 2, 128, 16), (4, 4, 64, 16), (14, 2, 64, 8), (7, 1, 128, 32), (32, 2, 128, 16), (6, 3, 64, 32),
    (40, 2, 64, 16), (36, 4, 128, 16)])
@pytest.mark.parametrize("window", [None, 24, 100])
def test_tensor_core_attention_mixed_batch(heads, kv_heads, dim, page_size, window):
    """The bfloat16 tensor-core kernel on decode rows, short portions and a long portion at
    once, over a cache whose unwritten slots hold NaN."""
    k = kernels()
    seq_lens, q_lens = [1, 37, 130, 64, 301, 257], [1, 37, 1, 5, 2, 257]
    scale = dim ** -0.5
    q, cache, tables, tok_seq, positions, dense = paged_case(
        torch.bfloat16, heads, kv_heads, dim, page_size, seq_lens, q_lens, seed=dim + heads)
    ref = reference_attention(dense, q_lens, seq_lens, scale, window)
    out, st = run_attention(k, q, cache, tables, tok_seq, positions, heads, kv_heads, dim,
                            window, scale, 1, impl="mma")
    assert st == 0
    worst = (out.double().cpu() - ref).abs().max(dim=1).values
    assert torch.allclose(out.double().cpu(), ref, **tol(torch.bfloat16)), (worst.argmax(), worst.max())
    # decode tokens alone and prompt portions alone, with the keys split
    for seq_lens, q_lens in (([1, 300, 33, 1000, 64], [1, 1, 1, 1, 1]), ([257, 90, 700], [257, 40, 100])):
        q, cache, tables, tok_seq, positions, dense = paged_case(
            torch.bfloat16, heads, kv_heads, dim, page_size, seq_lens, q_lens, seed=dim + heads + 1)
        ref = reference_attention(dense, q_lens, seq_lens, scale, window)
        for n_splits in (1, 3, 16):
            out, st = run_attention(k, q, cache, tables, tok_seq, positions, heads, kv_heads, dim,
                                    window, scale, n_splits, impl="mma")
            assert st == 0
            worst = (out.double().cpu() - ref).abs().max(dim=1).values
            assert torch.allclose(out.double().cpu(), ref, **tol(torch.bfloat16)), (n_splits, worst.argmax(), worst.max())


@pytest.mark.parametrize("heads,kv_heads,page_size", [(24, 2, 16), (7, 1, 32), (32, 2, 16), (6, 6, 16), (16, 1, 32),
                                                      (9, 3, 16), (36, 4, 16), (48, 4, 16)])
@pytest.mark.parametrize("window", [None, 24, 100, 300])
def test_tcgen05_attention_prompt_portions(heads, kv_heads, page_size, window):
    """The tcgen05 kernel on prompt portions (with decode rows beside them on the narrow kernel),
    over a cache whose unwritten slots hold NaN: whole prompts, portions deep in a sequence,
    lengths on both sides of the 128-key chunks and of the token tiles."""
    k = kernels()
    dim, scale = 128, 128 ** -0.5
    cases = [([1, 37, 130, 64, 301, 257], [1, 37, 1, 5, 2, 257]),
             ([257, 90, 700, 128], [257, 40, 100, 128]),
             ([1300, 129], [1300, 2])]
    for index, (seq_lens, q_lens) in enumerate(cases):
        q, cache, tables, tok_seq, positions, dense = paged_case(
            torch.bfloat16, heads, kv_heads, dim, page_size, seq_lens, q_lens, seed=heads + index)
        ref = reference_attention(dense, q_lens, seq_lens, scale, window)
        out, st = run_attention(k, q, cache, tables, tok_seq, positions, heads, kv_heads, dim,
                                window, scale, 1, impl="tc")
        assert st == 0
        got = out.double().cpu()
        assert torch.isfinite(got).all(), f"case {index}: non-finite output at rows {torch.nonzero(~torch.isfinite(got).all(dim=1)).flatten()[:8].tolist()}"
        worst = (got - ref).abs().max(dim=1).values
        assert torch.allclose(got, ref, **tol(torch.bfloat16)), (index, int(worst.argmax()), float(worst.max()))
    # keys shared out between blocks (portions only, so that the merge covers every row): more splits than
    # some tiles have chunks, a window that leaves shares empty
    for index, (seq_lens, q_lens, n_splits) in enumerate([([700, 1300], [100, 130], 3), ([2100], [40], 8),
                                                          ([300, 129], [300, 17], 5)]):
        q, cache, tables, tok_seq, positions, dense = paged_case(
            torch.bfloat16, heads, kv_heads, dim, page_size, seq_lens, q_lens, seed=50 + heads + index)
        ref = reference_attention(dense, q_lens, seq_lens, scale, window)
        out, st = run_attention(k, q, cache, tables, tok_seq, positions, heads, kv_heads, dim,
                                window, scale, n_splits, impl="tc")
        got = out.double().cpu()
        assert st == 0 and torch.isfinite(got).all(), f"split case {index}"
        worst = (got - ref).abs().max(dim=1).values
        assert torch.allclose(got, ref, **tol(torch.bfloat16)), ("split", index, int(worst.argmax()), float(worst.max()))


@pytest.mark.parametrize("edge", ["window_first_visible", "just_outside_window", "page_last_slot",
                                  "page_first_slot", "self", "far_key_full_attention", "chunk_last_key",
                                  "chunk_first_key"])
def test_tcgen05_attention_one_key_stands_out(edge):
    """As the stand-out test below, for the last query of a 40-token portion on the tcgen05 kernel."""
    k = kernels()
    heads, kv_heads, dim, page_size = 4, 2, 128, 16
    length, q_len, window = 400, 40, 96
    p = length - 1
    target = {"window_first_visible": p - window + 1, "just_outside_window": p - window,
              "page_last_slot": 367, "page_first_slot": 368, "self": p, "far_key_full_attention": 3,
              "chunk_last_key": 383, "chunk_first_key": 384}[edge]
    use_window = None if edge == "far_key_full_attention" else window

    def scale_up(s, qs, ks, vs):
        ks[:, target] = qs[0::2, -1] * 4.0          # aligned with the last query of heads 0 and 2
        qs[:, -1] *= 3.0

    scale = dim ** -0.5
    q, cache, tables, tok_seq, positions, dense = paged_case(
        torch.bfloat16, heads, kv_heads, dim, page_size, [length], [q_len], seed=11, scale_up=scale_up)
    ref = reference_attention(dense, [q_len], [length], scale, use_window)
    out, st = run_attention(k, q, cache, tables, tok_seq, positions, heads, kv_heads, dim, use_window, scale, 1,
                            impl="tc")
    assert st == 0
    assert torch.allclose(out.double().cpu(), ref, **tol(torch.bfloat16))
    qs, ks, vs = dense[0]
    head0 = ref[q_len - 1, :dim]
    if edge == "just_outside_window":
        assert (head0 - vs[0, target].double()).abs().max() > 0.3
    else:
        assert (head0 - vs[0, target].double()).abs().max() < 0.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("edge", ["window_first_visible", "just_outside_window", "page_last_slot",
                                  "page_first_slot", "self", "far_key_full_attention"])
@pytest.mark.parametrize("impl", ["simt", "mma"])
def test_paged_attention_one_key_stands_out(dtype, edge, impl):
    """One key gets a score far above the rest, so the output is (almost) that key's value if
    it is visible and unchanged by it if it is not: a wrong mask edge or page offset shows."""
    if impl == "mma" and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernel is bfloat16 only")
    k = kernels()
    heads, kv_heads, dim, page_size = 4, 2, (64 if impl == "mma" else 32), 16
    length, window = 400, 96
    p = length - 1
    target = {"window_first_visible": p - window + 1, "just_outside_window": p - window,
              "page_last_slot": 367, "page_first_slot": 368, "self": p,
              "far_key_full_attention": 3}[edge]
    use_window = None if edge == "far_key_full_attention" else window

    def scale_up(s, qs, ks, vs):
        ks[:, target] = qs[0::2, 0] * 4.0 if kv_heads == 2 else qs[0, 0] * 4.0   # aligned with the query
        qs *= 3.0

    scale = dim ** -0.5
    q, cache, tables, tok_seq, positions, dense = paged_case(
        dtype, heads, kv_heads, dim, page_size, [length], [1], seed=7, scale_up=scale_up)
    ref = reference_attention(dense, [1], [length], scale, use_window)
    for n_splits in (1, 4):
        out, st = run_attention(k, q, cache, tables, tok_seq, positions, heads, kv_heads, dim,
                                use_window, scale, n_splits, impl=impl)
        assert st == 0
        assert torch.allclose(out.double().cpu(), ref, **tol(dtype))
    qs, ks, vs = dense[0]
    head0 = ref[0, :dim]
    if edge == "just_outside_window":
        assert (head0 - vs[0, target].double()).abs().max() > 0.3
    else:
        assert (head0 - vs[0, target].double()).abs().max() < 0.05


def test_paged_attention_missing_page_sets_status():
    k = kernels()
    q, cache, tables, tok_seq, positions, _ = paged_case(torch.float32, 2, 1, 16, 16, [40], [1], seed=1)
    tables[0, 1] = -1
    _, st = run_attention(k, q, cache, tables, tok_seq, positions, 2, 1, 16, None, 0.25, 1)
    assert st == 4


def test_paged_attention_padding_rows_are_zero():
    k = kernels()
    q, cache, tables, tok_seq, positions, dense = paged_case(torch.float32, 2, 1, 16, 16, [40, 9], [1, 1], seed=2)
    tok_seq[1] = -1
    for n_splits in (1, 2):
        out, st = run_attention(k, q, cache, tables, tok_seq, positions, 2, 1, 16, None, 0.25, n_splits)
        assert st == 0 and torch.all(out[1] == 0)
        ref = reference_attention(dense[:1], [1], [40], 0.25, None)
        assert torch.allclose(out[:1].double().cpu(), ref, atol=2e-5)


def test_kernels_refuse_unsupported_sizes():
    from matricxon_b200.ops.library import KernelLibraryError

    k = kernels()
    q = torch.zeros(1, 2 * 24, device=DEV)
    cache = torch.zeros(1, 2, 1, 16, 24, device=DEV)
    tables = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    zeros = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelLibraryError, match="head_dim 24"):
        k.paged_attention(q, 48, cache, tables, zeros, zeros, 1, 2, 1, 24, None, 1.0,
                          torch.zeros(1, 48, device=DEV), status())
    with pytest.raises(KernelLibraryError, match="CUDA tensor"):
        k.layernorm(torch.zeros(2, 8), torch.ones(8), None, 1e-5, torch.zeros(2, 8))
