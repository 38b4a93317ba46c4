"""Each kernel alone against its plain PyTorch statement, at sizes other than the models'."""
import pytest
import torch

import kernel_references as ref
import plain_impl

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def status(dev):
    return torch.zeros(1, dtype=torch.int32, device=dev)


@pytest.mark.parametrize("table_dtype", DTYPES)
def test_embed(dev, table_dtype):
    from einf_b200 import ops

    table = torch.randn(301, 72, device=dev).to(table_dtype)
    tokens = torch.tensor([0, 300, 7, 7, 150], dtype=torch.int32, device=dev)
    out = torch.empty(5, 72, device=dev)
    st = status(dev)
    ops.embed(tokens, table, out, st)
    assert torch.equal(out, table[tokens.long()].float()) and int(st) == 0
    bad = torch.tensor([3, 301], dtype=torch.int32, device=dev)
    out2 = torch.ones(2, 72, device=dev)
    ops.embed(bad, table, out2, st)
    assert int(st) == ops.STATUS_BAD_TOKEN and torch.equal(out2[1], torch.zeros(72, device=dev))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [24, 200, 1000, 3584, 6002])
def test_add_rmsnorm(dev, dtype, hidden):
    from einf_b200 import ops

    torch.manual_seed(hidden)
    x = torch.randn(7, hidden, device=dev).to(dtype)
    residual = torch.randn(7, hidden, device=dev)
    weight = torch.rand(hidden, device=dev) + 0.5
    want_res, want_out = residual.clone(), torch.empty(7, hidden, device=dev, dtype=dtype)
    ref.add_rmsnorm(x, want_res, weight, 1e-5, want_out)
    out = torch.empty_like(want_out)
    ops.add_rmsnorm(x, residual, weight, 1e-5, out)
    torch.testing.assert_close(residual, want_res, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out, want_out, **tol(dtype))
    # without x, with split partial sums, and for chosen rows only
    out0, want0 = torch.empty_like(out), torch.empty_like(out)
    before = residual.clone()
    ops.add_rmsnorm(None, residual, weight, 1e-6, out0)
    ref.add_rmsnorm(None, before.clone(), weight, 1e-6, want0)
    assert torch.equal(residual, before)
    torch.testing.assert_close(out0, want0, **tol(dtype))
    parts = torch.randn(3, 7, hidden, device=dev)
    r1, r2 = residual.clone(), residual.clone()
    o1, o2 = torch.empty_like(out), torch.empty_like(out)
    ops.add_rmsnorm(parts, r1, weight, 1e-5, o1)
    ref.add_rmsnorm(parts, r2, weight, 1e-5, o2)
    torch.testing.assert_close(r1, r2, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(o1, o2, **tol(dtype))
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=dev)
    o3, o4 = torch.empty(3, hidden, device=dev, dtype=dtype), torch.empty(3, hidden, device=dev, dtype=dtype)
    r3 = residual.clone()
    ops.add_rmsnorm(x, r3, weight, 1e-5, o3, rows)
    ref.add_rmsnorm(x, residual.clone(), weight, 1e-5, o4, rows)
    assert torch.equal(r3, residual)  # rows: the residual is left alone
    torch.testing.assert_close(o3, o4, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, size, rotary", [(5, 1, 32, 32), (4, 2, 80, 80), (3, 3, 64, 32), (2, 1, 16, 0)])
def test_rope_kv_write(dev, dtype, heads, kv_heads, size, rotary):
    from einf_b200 import ops

    torch.manual_seed(size)
    tokens, page_size, pages = 9, 4, 7
    width = (heads + 2 * kv_heads) * size
    qkv = torch.randn(tokens, width, device=dev).to(dtype)
    bias = torch.randn(width, device=dev)
    positions = torch.tensor([0, 1, 2, 3, 4, 900, 901, 17, 40000], dtype=torch.int32, device=dev)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, rotary, 2).float() / max(rotary, 1)))).to(dev)
    slots = torch.tensor([4, 5, 6, 7, 24, 0, 1, -1, 13], dtype=torch.int32, device=dev)
    caches = [torch.full((pages, kv_heads, page_size, size), 7.0, device=dev, dtype=dtype) for _ in range(4)]
    q1 = torch.empty(tokens, heads, size, device=dev, dtype=dtype)
    q2 = torch.empty_like(q1)
    st = status(dev)
    ops.rope_kv_write(qkv, bias, positions, inv_freq, slots, q1, caches[0], caches[1], heads, kv_heads, size, st)
    ref.rope_kv_write(qkv, bias, positions, inv_freq, slots, q2, caches[2], caches[3], heads, kv_heads, size, st)
    assert int(st) == 0
    torch.testing.assert_close(q1, q2, **tol(dtype))
    torch.testing.assert_close(caches[0], caches[2], **tol(dtype))
    torch.testing.assert_close(caches[1], caches[3], **tol(dtype))
    # V is a copy (+ bias): what is written equals what is read, and untouched slots stay
    assert torch.equal(caches[1][2, :, 1], torch.full((kv_heads, size), 7.0, device=dev, dtype=dtype))
    # without a bias V is a plain copy of the rows: bit for bit what came in
    # (the reference asks the same of its cache write, tests/test_torch_custom_ops.py:589-590)
    plain_k = torch.full((pages, kv_heads, page_size, size), 7.0, device=dev, dtype=dtype)
    plain_v = torch.full_like(plain_k, 7.0)
    ops.rope_kv_write(qkv, None, positions, inv_freq, slots, torch.empty_like(q1), plain_k, plain_v, heads, kv_heads, size, st)
    v_rows = qkv[:, (heads + kv_heads) * size:].view(tokens, kv_heads, size)
    for token, slot in enumerate(slots.tolist()):
        if slot >= 0:
            assert torch.equal(plain_v[slot // page_size, :, slot % page_size], v_rows[token]), token
    assert int((plain_v != 7.0).any(-1).sum()) <= (tokens - 1) * kv_heads      # nothing else was written
    # an unrotated key (no rotary dims at all) is a plain copy too
    if rotary == 0:
        k_rows = qkv[:, heads * size:(heads + kv_heads) * size].view(tokens, kv_heads, size)
        for token, slot in enumerate(slots.tolist()):
            if slot >= 0:
                assert torch.equal(plain_k[slot // page_size, :, slot % page_size], k_rows[token]), token
    # the rotation agrees with the reference's rotate-half formula
    if rotary == size:
        cos, sin = plain_impl.rope_cos_sin(positions.cpu().tolist(), size, 10000.0)
        q_plain = (qkv.float().cpu() + bias.cpu())[:, : heads * size].view(tokens, heads, size)
        want = plain_impl.apply_rope(q_plain, cos, sin)
        torch.testing.assert_close(q1.float().cpu(), want, **(dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else tol(dtype)))
    # without slots only Q is produced; a slot beyond the pool sets the status word
    q3 = torch.empty_like(q1)
    ops.rope_kv_write(qkv, None, positions, inv_freq, None, q3, None, None, heads, kv_heads, size, st)
    bad = slots.clone()
    bad[0] = pages * page_size
    ops.rope_kv_write(qkv, bias, positions, inv_freq, bad, q1, caches[0], caches[1], heads, kv_heads, size, st)
    assert int(st) == ops.STATUS_BAD_PAGE


@pytest.mark.parametrize("splits", [1, 15, 16, 17, 38])
def test_consumers_add_many_partial_sums(dev, splits):
    """Norm, rotary and activation add up the partial sums of a split-K product themselves, sixteen
    loads at a time: counts around that batch size, few rows (the per-head and cluster kernels)."""
    from einf_b200 import ops

    torch.manual_seed(splits)
    rows, hidden = 5, 896
    parts = torch.randn(splits, rows, hidden, device=dev)
    residual = torch.randn(rows, hidden, device=dev)
    weight = torch.rand(hidden, device=dev) + 0.5
    r1, r2 = residual.clone(), residual.clone()
    o1 = torch.empty(rows, hidden, device=dev, dtype=torch.bfloat16)
    o2 = torch.empty_like(o1)
    ops.add_rmsnorm(parts, r1, weight, 1e-6, o1)
    ref.add_rmsnorm(parts, r2, weight, 1e-6, o2)
    torch.testing.assert_close(r1, r2, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(o1, o2, **tol(torch.bfloat16))
    heads, kv_heads, size, page_size, pages = 14, 2, 64, 16, 4
    width = (heads + 2 * kv_heads) * size
    qkv = torch.randn(splits, rows, width, device=dev)
    bias = torch.randn(width, device=dev)
    positions = torch.tensor([0, 5, 900, 17, 40000], dtype=torch.int32, device=dev)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, size, 2).float() / size))).to(dev)
    slots = torch.tensor([3, 17, 40, -1, 63], dtype=torch.int32, device=dev)
    caches = [torch.full((pages, kv_heads, page_size, size), 7.0, device=dev, dtype=torch.bfloat16) for _ in range(4)]
    q1 = torch.empty(rows, heads, size, device=dev, dtype=torch.bfloat16)
    q2 = torch.empty_like(q1)
    st = status(dev)
    ops.rope_kv_write(qkv, bias, positions, inv_freq, slots, q1, caches[0], caches[1], heads, kv_heads, size, st)
    ref.rope_kv_write(qkv, bias, positions, inv_freq, slots, q2, caches[2], caches[3], heads, kv_heads, size, st)
    assert int(st) == 0
    torch.testing.assert_close(q1, q2, **tol(torch.bfloat16))
    torch.testing.assert_close(caches[0], caches[2], **tol(torch.bfloat16))
    torch.testing.assert_close(caches[1], caches[3], **tol(torch.bfloat16))
    inter = 264
    gate_up = torch.randn(splits, rows, 2 * inter, device=dev)
    a, b = torch.empty(rows, inter, device=dev, dtype=torch.bfloat16), torch.empty(rows, inter, device=dev, dtype=torch.bfloat16)
    ops.silu_mul(gate_up, a)
    ref.silu_mul(gate_up, b)
    torch.testing.assert_close(a, b, **tol(torch.bfloat16))


@pytest.mark.parametrize("hidden", [100, 896, 1536, 3584, 4100])
@pytest.mark.parametrize("x_dtype, out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32), (torch.float32, torch.bfloat16)])
def test_add_rmsnorm_many_rows(dev, hidden, x_dtype, out_dtype):
    """Hundreds of rows take the one-warp-per-row kernel (widths up to 4,096) or the block kernel."""
    from einf_b200 import ops

    torch.manual_seed(hidden)
    rows = 301
    x = torch.randn(rows, hidden, device=dev).to(x_dtype)
    residual = torch.randn(rows, hidden, device=dev) * 3
    weight = 1 + 0.1 * torch.randn(hidden, device=dev)
    r1, r2 = residual.clone(), residual.clone()
    out, want = torch.empty(rows, hidden, device=dev, dtype=out_dtype), torch.empty(rows, hidden, device=dev, dtype=out_dtype)
    ops.add_rmsnorm(x, r1, weight, 1e-6, out)
    ref.add_rmsnorm(x, r2, weight, 1e-6, want)
    torch.testing.assert_close(r1, r2, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out, want, **(tol(out_dtype) if out_dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)))
    # without x the residual stays; with a row list only those rows are normalised
    out0, want0 = torch.empty_like(out), torch.empty_like(out)
    ops.add_rmsnorm(None, r1, weight, 1e-5, out0)
    ref.add_rmsnorm(None, r2, weight, 1e-5, want0)
    torch.testing.assert_close(out0, want0, **(tol(out_dtype) if out_dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)))
    picked = torch.randperm(rows, device=dev)[:200].to(torch.int32)
    o3, o4 = torch.empty(200, hidden, device=dev, dtype=out_dtype), torch.empty(200, hidden, device=dev, dtype=out_dtype)
    before = r1.clone()
    ops.add_rmsnorm(x, r1, weight, 1e-5, o3, picked)
    ref.add_rmsnorm(x, r2.clone(), weight, 1e-5, o4, picked)
    assert torch.equal(r1, before)
    torch.testing.assert_close(o3, o4, **(tol(out_dtype) if out_dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)))


@pytest.mark.parametrize("rows, intermediate", [(3, 4864), (300, 200), (257, 2056)])
def test_silu_mul_vector_kernel(dev, rows, intermediate):
    """bfloat16 rows whose width is a multiple of 8; large gates of both signs (the exponential
    overflows for very negative ones: the result must be zero, not NaN)."""
    from einf_b200 import ops

    torch.manual_seed(rows)
    gate_up = (torch.randn(rows, 2 * intermediate, device=dev) * 4).to(torch.bfloat16)
    gate_up[0, :8] = torch.tensor([-200.0, -90.0, -30.0, 0.0, 30.0, 90.0, 200.0, -1e30], device=dev).to(torch.bfloat16)
    out = torch.full((rows, intermediate), float("nan"), device=dev, dtype=torch.bfloat16)
    want = torch.empty_like(out)
    ops.silu_mul(gate_up, out)
    ref.silu_mul(gate_up, want)
    assert torch.isfinite(out.float()).all()
    torch.testing.assert_close(out, want, **tol(torch.bfloat16))


def test_report_writes_pinned_host_memory(dev):
    from einf_b200 import ops

    tokens = torch.arange(100, 170, dtype=torch.int32, device=dev)
    st = torch.tensor([5], dtype=torch.int32, device=dev)
    for count in (0, 1, 8, 70):
        host = torch.full((80,), -1, dtype=torch.int32).pin_memory()
        ops.report(tokens, count, st, host)
        torch.cuda.synchronize()
        assert host[:count].tolist() == list(range(100, 100 + count))
        assert int(host[count]) == 5 and int(host[count + 1]) == -1
    with pytest.raises(ValueError):
        ops.report(tokens, 3, st, torch.zeros(8, dtype=torch.int32))          # not pinned


def test_advance_decode(dev):
    from einf_b200 import ops

    page, width, requests, live = 4, 6, 5, 3
    token_ids = torch.tensor([7, 8, 9, 0, 0], dtype=torch.int32, device=dev)
    positions = torch.tensor([3, 10, 0, 0, 0], dtype=torch.int32, device=dev)
    context_lens = positions + 1
    sampled = torch.tensor([70, 80, 90], dtype=torch.int32, device=dev)
    tables = [torch.randint(0, 50, (requests, width), dtype=torch.int32, device=dev) for _ in range(2)]
    slots = [torch.tensor([11, 22, 33, -1, -1], dtype=torch.int32, device=dev),
             torch.tensor([5, -1, 6, -1, -1], dtype=torch.int32, device=dev)]
    want = [t.clone() for t in (token_ids, positions, context_lens, *slots)]
    ref.advance_decode(want[0], want[1], want[2], sampled.cpu().to(dev), want[3:], tables, page)
    ops.advance_decode(token_ids, positions, context_lens, sampled, slots, tables, page)
    for got, expected in zip((token_ids, positions, context_lens, *slots), want):
        assert torch.equal(got, expected)
    assert positions.tolist() == [4, 11, 1, 0, 0] and token_ids.tolist() == [70, 80, 90, 0, 0]
    assert slots[0][0] == tables[0][0, 1] * page + 0 and slots[1][1] == -1 and slots[0][3] == -1


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dev, dtype):
    from einf_b200 import ops

    gate_up = (torch.randn(11, 2 * 77, device=dev) * 3).to(dtype)
    out, want = torch.empty(11, 77, device=dev, dtype=dtype), torch.empty(11, 77, device=dev, dtype=dtype)
    ops.silu_mul(gate_up, out)
    ref.silu_mul(gate_up, want)
    torch.testing.assert_close(out, want, **tol(dtype))


@pytest.mark.parametrize("m, n, k", [(1, 5, 3), (7, 130, 67), (64, 64, 64), (65, 127, 200), (300, 33, 1000)])
@pytest.mark.parametrize("a_dtype, w_dtype, out_dtype", [
    (torch.float32, torch.float32, torch.float32),
    (torch.bfloat16, torch.float32, torch.bfloat16),
    (torch.float32, torch.bfloat16, torch.float32),
    (torch.bfloat16, torch.bfloat16, torch.float32),
])
def test_gemm_simt(dev, m, n, k, a_dtype, w_dtype, out_dtype):
    from einf_b200 import ops

    torch.manual_seed(m * n + k)
    a = torch.randn(m, k, device=dev).to(a_dtype)
    w = torch.randn(n, k, device=dev).to(w_dtype)
    bias = torch.randn(n, device=dev)
    out = torch.empty(m, n, device=dev, dtype=out_dtype)
    ops.gemm_simt(a, w, bias, out)
    want = a.double() @ w.double().T + bias.double()
    scale = float(want.abs().max())
    if out_dtype == torch.float32:
        torch.testing.assert_close(out.double(), want, rtol=1e-5, atol=2e-6 * max(scale, 1.0) * (k ** 0.5))
    else:
        torch.testing.assert_close(out.double(), want, rtol=1e-2, atol=1e-2 * scale)
    # rows of A may be a strided view
    wide = torch.randn(m, k + 8, device=dev).to(a_dtype)
    view = wide[:, 3:3 + k] if (3 * wide.element_size()) % 4 == 0 or True else wide[:, :k]
    out2 = torch.empty(m, n, device=dev, dtype=out_dtype)
    ops.gemm_simt(view, w, None, out2)
    want2 = view.double() @ w.double().T
    torch.testing.assert_close(out2.double(), want2, rtol=1e-2 if out_dtype != torch.float32 else 1e-5,
                               atol=(1e-2 if out_dtype != torch.float32 else 2e-6 * (k ** 0.5)) * max(float(want2.abs().max()), 1.0))


@pytest.mark.parametrize("tokens, n, k, splits", [
    (8, 128, 64, 1), (1, 128, 896, 1), (8, 1152, 896, 14), (16, 331, 80, 2), (5, 100, 72, 2), (17, 1000, 264, 3),
    (64, 896, 4864, 19), (100, 300, 136, 1), (256, 512, 1024, 1), (300, 640, 512, 4), (700, 1152, 896, 1),
])
def test_gemm_tcgen05(dev, tokens, n, k, splits):
    from einf_b200 import ops

    torch.manual_seed(tokens + n + k)
    x = torch.randn(tokens, k, device=dev).bfloat16()
    w = torch.randn(n, k, device=dev).bfloat16()
    bias = torch.randn(n, device=dev)
    want = x.double() @ w.double().T
    scale = float(want.abs().max())
    st = status(dev)
    splits = ops.gemm_tcgen05_splits(k, splits)
    if splits > 1:
        out = torch.full((splits, tokens, n), float("nan"), device=dev)
        ops.gemm_tcgen05(x, w, bias, out, st, splits)
        torch.testing.assert_close(out.double().sum(0), want + bias.double(), rtol=1e-5, atol=1e-5 * scale)
    else:
        for out_dtype, tolerance in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
            out = torch.full((tokens, n), float("nan"), device=dev, dtype=out_dtype)
            ops.gemm_tcgen05(x, w, None, out, st)
            torch.testing.assert_close(out.double(), want, rtol=tolerance, atol=tolerance * scale)
            ops.gemm_tcgen05(x, w, bias, out, st)
            torch.testing.assert_close(out.double(), want + bias.double(), rtol=tolerance, atol=tolerance * scale)
    # rows of x may be a strided view whose stride keeps them 16-byte aligned
    wide = torch.randn(tokens, k + 16, device=dev).bfloat16()
    view = wide[:, 8:8 + k]
    out = torch.empty((tokens, n), device=dev)
    ops.gemm_tcgen05(view, w, None, out, st)
    torch.testing.assert_close(out.double(), view.double() @ w.double().T, rtol=1e-5, atol=1e-5 * scale)
    assert int(st) == 0
    with pytest.raises(ops.UnsupportedSize):
        ops.gemm_tcgen05(torch.zeros(4, 12, device=dev).bfloat16(), torch.zeros(8, 12, device=dev).bfloat16(), None,
                         torch.zeros(4, 8, device=dev), st)


@pytest.mark.parametrize("rows, hidden, splits", [(5, 896, 14), (8, 896, 16), (8, 1536, 12), (33, 200, 2), (64, 1000, 7), (12, 128, 16)])
def test_add_rmsnorm_with_partial_sums_fetched_by_tma(dev, rows, hidden, splits):
    """With the step's status word at hand, a handful of rows of split-K partial sums take the kernel
    that brings a row's partial sums into shared memory by TMA; same results as the plain statement,
    also with a row gather (the final norm) and for the last box of a row that is no multiple of 256."""
    from einf_b200 import ops

    torch.manual_seed(rows + hidden + splits)
    x = torch.randn(splits, rows, hidden, device=dev)
    weight = torch.randn(hidden, device=dev)
    for out_dtype in (torch.bfloat16, torch.float32):
        res1, res2 = torch.randn(rows, hidden, device=dev), None
        res2 = res1.clone()
        out1 = torch.full((rows, hidden), float("nan"), device=dev, dtype=out_dtype)
        out2 = torch.empty_like(out1)
        st = status(dev)
        ops.add_rmsnorm(x, res1, weight, 1e-5, out1, None, st)
        ref.add_rmsnorm(x, res2, weight, 1e-5, out2)
        assert int(st) == 0
        torch.testing.assert_close(res1, res2, rtol=1e-6, atol=1e-5)
        torch.testing.assert_close(out1, out2, **(dict(rtol=1e-5, atol=1e-5) if out_dtype == torch.float32 else tol(out_dtype)))
        # gathered rows: the residual stays, the output has one row per index
        pick = torch.tensor([rows - 1, 0, 2, 2, rows // 2], dtype=torch.int32, device=dev)
        before = res1.clone()
        g1 = torch.full((5, hidden), float("nan"), device=dev, dtype=out_dtype)
        g2 = torch.empty_like(g1)
        ops.add_rmsnorm(x, res1, weight, 1e-5, g1, pick, st)
        ref.add_rmsnorm(x, res2, weight, 1e-5, g2, pick)
        assert torch.equal(res1, before) and int(st) == 0
        torch.testing.assert_close(g1, g2, **(dict(rtol=1e-5, atol=1e-5) if out_dtype == torch.float32 else tol(out_dtype)))


def test_consumers_add_up_partial_sums(dev):
    """The rotary and activation kernels take the float partial sums of a split-K product."""
    from einf_b200 import ops

    torch.manual_seed(3)
    heads, kv_heads, size, tokens = 3, 1, 32, 5
    width = (heads + 2 * kv_heads) * size
    parts = torch.randn(4, tokens, width, device=dev)
    dense = parts.sum(0).bfloat16()
    positions = torch.arange(7, 7 + tokens, dtype=torch.int32, device=dev)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, size, 2).float() / size))).to(dev)
    slots = torch.arange(tokens, dtype=torch.int32, device=dev)
    st = status(dev)
    results = []
    for source in (parts, dense):
        cache = [torch.zeros(2, kv_heads, 4, size, device=dev, dtype=torch.bfloat16) for _ in range(2)]
        q = torch.empty(tokens, heads, size, device=dev, dtype=torch.bfloat16)
        ops.rope_kv_write(source, None, positions, inv_freq, slots, q, cache[0], cache[1], heads, kv_heads, size, st)
        results.append((q, *cache))
    for a, b in zip(*results):
        torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-2)
    gate_up = torch.randn(3, tokens, 2 * 40, device=dev)
    a, b = torch.empty(tokens, 40, device=dev, dtype=torch.bfloat16), torch.empty(tokens, 40, device=dev, dtype=torch.bfloat16)
    ops.silu_mul(gate_up, a)
    ref.silu_mul(gate_up.sum(0), b)
    torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("m, n, k", [(1, 40, 24), (8, 331, 80), (77, 160, 96), (200, 1000, 264)])
def test_linear_bfloat16(dev, m, n, k):
    from einf_b200 import ops

    a = torch.randn(m, k, device=dev).bfloat16()
    w = torch.randn(n, k, device=dev).bfloat16()
    bias = torch.randn(n, device=dev)
    want = a.double() @ w.double().T
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.empty(m, n, device=dev, dtype=out_dtype)
        ops.linear(a, w, None, out)
        torch.testing.assert_close(out.double(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()))
        ops.linear(a, w, bias, out)
        torch.testing.assert_close(out.double(), want + bias.double(), rtol=1e-2, atol=1e-2 * float(want.abs().max()))


def _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window, seed=0, layout="shuffled"):
    """requests: list of (start, q_len).  Builds caches over shuffled pages; ``layout`` "runs" gives
    every request pages that follow one another in the pool, "broken runs" the same with a few
    neighbours swapped."""
    from einf_b200 import ops

    generator = torch.Generator().manual_seed(seed)
    contexts = [s + q for s, q in requests]
    pages_each = [-(-c // page_size) for c in contexts]
    num_pages = sum(pages_each) + 3
    order = torch.randperm(num_pages, generator=generator).tolist()
    if layout != "shuffled":
        order = list(range(1, num_pages)) + [0]
        if layout == "broken runs":
            for at in range(5, num_pages - 2, 11):
                order[at], order[at + 1] = order[at + 1], order[at]
    width = max(pages_each) + 2
    table = torch.full((len(requests), width), -1, dtype=torch.int32)
    k_cache = torch.randn((num_pages, kv_heads, page_size, size), generator=generator).to(dtype)
    v_cache = torch.randn((num_pages, kv_heads, page_size, size), generator=generator).to(dtype)
    cursor = 0
    for r, count in enumerate(pages_each):
        table[r, :count] = torch.tensor(order[cursor:cursor + count], dtype=torch.int32)
        cursor += count
    seq, pos = [], []
    for r, (start, q_len) in enumerate(requests):
        seq += [r] * q_len
        pos += list(range(start, start + q_len))
    tokens = len(seq)
    q = torch.randn((tokens, heads, size), generator=generator).to(dtype)
    args = [t.to(dev) for t in (q, k_cache, v_cache, table,
                                 torch.tensor(seq, dtype=torch.int32), torch.tensor(pos, dtype=torch.int32))]
    return args, size ** -0.5, window


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, size, page_size", [
    (4, 2, 16, 4), (3, 1, 32, 8), (14, 2, 64, 16), (6, 2, 48, 16), (8, 8, 128, 16), (7, 1, 256, 3),
])
@pytest.mark.parametrize("window", [None, 5])
def test_paged_attention_generic(dev, dtype, heads, kv_heads, size, page_size, window):
    from einf_b200 import ops

    # context 1; an exact page edge; a partial last page; a portion with start > 0; decode tokens
    requests = [(0, 1), (0, 2 * page_size), (3, 6), (15, 6), (page_size * 4 - 1, 1), (70, 1), (0, 37)]
    (q, k, v, table, seq, pos), scale, window = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window)
    out, want = torch.empty_like(q), torch.empty_like(q)
    st = status(dev)
    ops.paged_attention_generic(q, k, v, table, seq, pos, out, scale, window, st)
    ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st)
    assert int(st) == 0
    torch.testing.assert_close(out, want, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else tol(dtype)))


@pytest.mark.parametrize("heads, kv_heads, size, page_size", [
    (4, 2, 16, 4), (3, 1, 32, 8), (14, 2, 64, 16), (6, 2, 48, 16), (8, 8, 128, 16), (34, 2, 64, 5), (7, 1, 80, 16),
    (4, 1, 64, 8), (2, 2, 128, 64), (3, 1, 64, 128), (34, 2, 64, 32), (28, 4, 128, 16),
])
@pytest.mark.parametrize("window", [None, 5, 70])
def test_tensor_core_attention(dev, heads, kv_heads, size, page_size, window):
    """Decode (every split count) and prefill kernels against the plain statement."""
    from einf_b200 import ops

    dtype = torch.bfloat16
    # decode: one token per request at many context lengths, page edges included
    lengths = [1, 2, page_size, page_size + 1, 63, 64, 65, 128, 200, 513, 1500]
    requests = [(n - 1, 1) for n in lengths]
    (q, k, v, table, seq, pos), scale, window = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window)
    want = torch.empty_like(q)
    st = status(dev)
    ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st)
    for splits in (1, 2, 3, 8, 32):
        workspace = ops.DecodeWorkspace(len(lengths), heads, kv_heads, size, splits, dev)
        out = torch.full_like(q, float("nan"))
        ops.paged_decode_attention(q, k, v, table, seq, pos, out, scale, window, workspace, splits, st)
        torch.testing.assert_close(out, want, **tol(dtype))
        assert int(workspace.counters.abs().sum()) == 0      # the counters are left at zero
        ops.paged_decode_attention(q, k, v, table, seq, pos, out, scale, window, workspace, splits, st)
        torch.testing.assert_close(out, want, **tol(dtype))  # and a second launch works on them
    for cluster in (1, 2, 4, 8):
        out = torch.full_like(q, float("nan"))
        ops.paged_decode_attention_cluster(q, k, v, table, seq, pos, out, scale, window, cluster, st)
        torch.testing.assert_close(out, want, **tol(dtype))
    decode_kernels = [ops.paged_decode_attention_cluster]
    if ops.has_tcgen05_attention(size, page_size):
        decode_kernels.append(ops.paged_decode_attention_tcgen05)
        for cluster in (1, 2, 3, 4, 5, 6, 7, 8):
            out = torch.full_like(q, float("nan"))
            ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, window, cluster, st)
            assert int(st) == 0
            torch.testing.assert_close(out, want, **tol(dtype))
    # with a token list only the listed tokens are touched (the others belong to another kernel)
    chosen = torch.tensor([9, 0, 4], dtype=torch.int32, device=dev)
    untouched = [i for i in range(len(lengths)) if i not in (9, 0, 4)]
    for kernel in decode_kernels:
        out = torch.full_like(q, float("nan"))
        kernel(q, k, v, table, seq, pos, out, scale, window, 4, st, chosen)
        torch.testing.assert_close(out[chosen.long()], want[chosen.long()], **tol(dtype))
        assert torch.isnan(out[untouched].float()).all()
    assert int(st) == 0
    # prefill: portions with start 0 and > 0, one-row tiles, a portion longer than two tiles
    requests = [(0, 1), (0, 2 * page_size), (3, 6), (15, 70), (page_size * 4 - 1, 1), (70, 1), (0, 150), (100, 64), (37, 300)]
    (q, k, v, table, seq, pos), scale, window = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window, seed=1)
    tiles, cursor = [], 0
    for r, (start, q_len) in enumerate(requests):
        for first in range(0, q_len, ops.Q_TILE):
            tiles.append((r, cursor + first, min(ops.Q_TILE, q_len - first), start + first))
        cursor += q_len
    q_tiles = torch.tensor(tiles, dtype=torch.int32, device=dev)
    want = torch.empty_like(q)
    ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st)
    kernels = [(False, 0)]
    if ops.has_tcgen05_attention(size, page_size):
        kernels += [(True, cluster) for cluster in (0, 1, 2, 3, 5, 8)]   # CTAs that share a row tile's keys
    for use_tcgen05, cluster in kernels:
        out = torch.full_like(q, float("nan"))
        ops.paged_prefill_attention(q, k, v, table, q_tiles, out, scale, window, st, use_tcgen05=use_tcgen05,
                                    prefill_cluster=cluster)
        assert int(st) == 0
        torch.testing.assert_close(out, want, **tol(dtype))


def test_tensor_core_attention_far_key_and_window_edge(dev):
    from einf_b200 import ops

    dtype = torch.bfloat16
    for far in (0, 3, 63, 64, 130, 257, 511, 599):
        requests = [(600, 1), (0, 700)]
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, 4, 2, 32, 16, requests, None, seed=far)
        q.mul_(0.05)
        page, offset = int(table[0, far // 16]), far % 16
        k[page, :, offset, :] = 0
        k[page, :, offset, 0] = 40.0
        q[0, :, 0] = 2.0 / scale
        st = status(dev)
        out = torch.empty_like(q)
        workspace = ops.DecodeWorkspace(701, 4, 2, 32, 8, dev)
        ops.paged_decode_attention(q, k, v, table, seq, pos, out, scale, None, workspace, 8, st)
        torch.testing.assert_close(out[0, 0].float(), v[page, 0, offset].float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(out[0, 3].float(), v[page, 1, offset].float(), rtol=2e-2, atol=2e-2)
    window = 9
    for kernel in ("decode", "prefill"):
        for inside in (True, False):
            (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, 2, 1, 16, 4, [(40, 1)], window, seed=3)
            q.mul_(0.05)
            key = 40 - window + 1 if inside else 40 - window
            page, offset = int(table[0, key // 4]), key % 4
            k[page, :, offset, :] = 0
            k[page, :, offset, 0] = 30.0
            q[0, :, 0] = 12.0
            out = torch.empty_like(q)
            st = status(dev)
            if kernel == "decode":
                ops.paged_decode_attention(q, k, v, table, seq, pos, out, scale, window, ops.DecodeWorkspace(1, 2, 1, 16, 2, dev), 2, st)
            else:
                tiles = torch.tensor([[0, 0, 1, 40]], dtype=torch.int32, device=dev)
                ops.paged_prefill_attention(q, k, v, table, tiles, out, scale, window, st)
            heard = torch.allclose(out[0, 0].float(), v[page, 0, offset].float(), rtol=2e-2, atol=2e-2)
            assert heard == inside, (kernel, inside)
    with pytest.raises(ops.UnsupportedSize):
        big = torch.empty(1, 2, 256, device=dev, dtype=dtype)
        cache = torch.empty(1, 1, 4, 256, device=dev, dtype=dtype)
        ops.paged_prefill_attention(big, cache, cache, table, tiles, big.clone(), 1.0, None, st)


@pytest.mark.parametrize("first_case", [0, 20, 40, 60])
def test_tcgen05_prefill_random_shapes(dev, first_case):
    """Seeded random launches of the tcgen05 prefill kernel: head sizes 64 and 128, every page size
    it takes, one to four requests whose portions start anywhere in contexts of up to 4,500 tokens,
    with and without a window, pages shuffled, in runs or in broken runs, keys scaled so that rows
    are peaked and references move, every cluster size; against the generic kernel."""
    import random

    from einf_b200 import ops

    for case in range(first_case, first_case + 20):
        rng = random.Random(case)
        size, page_size = rng.choice([64, 128]), rng.choice([8, 16, 32, 64, 128])
        kv_heads, group = rng.choice([1, 2, 4]), rng.choice([1, 2, 3, 6, 7, 8])
        window = rng.choice([None, None, 5, 130, 700, 2000])
        requests = []
        for _ in range(rng.randint(1, 4)):
            start = rng.choice([0, 0, rng.randrange(1, 200), rng.randrange(200, 3000)])
            requests.append((start, rng.choice([2, rng.randrange(2, 140), rng.randrange(100, 700), rng.randrange(2, 1500)])))
        layout = rng.choice(["shuffled", "runs", "broken runs"])
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, torch.bfloat16, kv_heads * group, kv_heads, size, page_size,
                                                               requests, window, seed=case, layout=layout)
        k.mul_(rng.choice([1.0, 1.0, 3.0, 8.0]))
        tiles, cursor = [], 0
        for r, (start, q_len) in enumerate(requests):
            for first in range(0, q_len, ops.Q_TILE):
                tiles.append((r, cursor + first, min(ops.Q_TILE, q_len - first), start + first))
            cursor += q_len
        q_tiles = torch.tensor(tiles, dtype=torch.int32, device=dev)
        st = status(dev)
        want = torch.empty_like(q)
        ops.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st)
        out = torch.full_like(q, float("nan"))
        ops.paged_prefill_attention(q, k, v, table, q_tiles, out, scale, window, st, use_tcgen05=True,
                                    prefill_cluster=rng.randrange(0, 9), cached_before=max(s for s, _ in requests))
        assert int(st) == 0, case
        torch.testing.assert_close(out, want, **tol(torch.bfloat16), msg=lambda m: f"case {case}: {m}")


@pytest.mark.parametrize("heads, kv_heads, size, page_size", [(14, 2, 64, 16), (8, 2, 128, 16)])
def test_tcgen05_prefill_long_prompts(dev, heads, kv_heads, size, page_size):
    """Thousands of keys per row (dozens of key tiles per CTA: every ring and every barrier goes
    round many times), whole and as a late portion, alone and as clusters, with and without a
    window, against the generic kernel (32-bit arithmetic on the same bfloat16 cache), which the
    plain statement covers at small sizes.  One key far back carries most of a late row's weight."""
    from einf_b200 import ops

    dtype = torch.bfloat16
    requests = [(0, 5000), (6100, 200)]
    for window in (None, 1500):
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window,
                                                               seed=5, layout="broken runs")
        far = 333
        page, offset = int(table[1, far // page_size]), far % page_size
        k[page, :, offset, :] = 0
        k[page, :, offset, 0] = 30.0
        q[5000:, :, 0] = 1.0 / scale
        tiles, cursor = [], 0
        for r, (start, q_len) in enumerate(requests):
            for first in range(0, q_len, ops.Q_TILE):
                tiles.append((r, cursor + first, min(ops.Q_TILE, q_len - first), start + first))
            cursor += q_len
        q_tiles = torch.tensor(tiles, dtype=torch.int32, device=dev)
        st = status(dev)
        want = torch.empty_like(q)
        ops.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st)
        for cluster in (1, 3, 8):
            out = torch.full_like(q, float("nan"))
            ops.paged_prefill_attention(q, k, v, table, q_tiles, out, scale, window, st, use_tcgen05=True,
                                        prefill_cluster=cluster)
            assert int(st) == 0
            torch.testing.assert_close(out, want, **tol(dtype))
        if window is None:   # the far key lies inside every late row's reach: they hear it above all else
            torch.testing.assert_close(out[5100, 0].float(), v[page, 0, offset].float(), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("heads, kv_heads, size, page_size", [(14, 2, 64, 16), (8, 2, 128, 16), (4, 1, 64, 8)])
def test_tcgen05_attention_after_a_kernel_that_left_nans_in_shared_memory(dev, heads, kv_heads, size, page_size):
    """A tile with fewer than 128 keys leaves rows of its V stage that no TMA fills; whatever an
    earlier kernel left there meets probabilities of zero, and zero times a NaN is a NaN.  So first
    a launch whose values are all NaN fills every SM's stages with them, then short requests of
    every length run on the same SMs: prefill and decode, each against the plain statement."""
    from einf_b200 import ops

    dtype = torch.bfloat16
    st = status(dev)

    def poison():
        requests = [(0, 2048)]
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, None, seed=1)
        v.fill_(float("nan"))
        tiles = torch.tensor([(0, first, 128, first) for first in range(0, 2048, ops.Q_TILE)], dtype=torch.int32, device=dev)
        out = torch.empty_like(q)
        ops.paged_prefill_attention(q, k, v, table, tiles, out, scale, None, st, use_tcgen05=True)
        many = [(2047, 1)] * 40
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, many, None, seed=2)
        v.fill_(float("nan"))
        out = torch.empty_like(q)
        ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, None, 4, st)
        assert torch.isnan(out).all()

    for length in (1, 5, page_size, page_size + 3, 40, 100, 127, 129, 200, 300):
        poison()
        requests = [(0, length)]
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, None, seed=length)
        tiles = torch.tensor([(0, first, min(ops.Q_TILE, length - first), first) for first in range(0, length, ops.Q_TILE)],
                             dtype=torch.int32, device=dev)
        want, out = torch.empty_like(q), torch.full_like(q, float("nan"))
        ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, None, st)
        ops.paged_prefill_attention(q, k, v, table, tiles, out, scale, None, st, use_tcgen05=True)
        torch.testing.assert_close(out, want, **tol(dtype))
        poison()
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, [(length - 1, 1)] * 3, None, seed=length)
        want, out = torch.empty_like(q), torch.full_like(q, float("nan"))
        ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, None, st)
        for cluster in (1, 2):
            ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, None, cluster, st)
            torch.testing.assert_close(out, want, **tol(dtype))
    assert int(st) == 0


@pytest.mark.parametrize("size, page_size", [(64, 16), (128, 32)])
@pytest.mark.parametrize("growth", [-20.0, 3.0, 6.0, 11.0, 25.0, 90.0])
def test_tcgen05_prefill_when_the_maximum_moves(dev, size, page_size, growth):
    """The prefill kernel scales P and O by a reference that stays where a row's first tile put
    it until a tile's sum of probabilities says that the scores have left it far behind (2^40);
    then the reference moves to that tile's maximum, O and the sums are rescaled and the tile is
    done again.  Random scores never get there, so here the score of key j is made to grow by
    ``growth`` (exponent of two) per 128 keys, on top of a little noise: every row's weight then
    sits on its last few keys (or, falling, on its first), and each of the two warpgroups, which
    take every other tile, sees its scores rise by twice that from one tile to its next: not at
    all, slowly (the reference serves for several tiles), and by more than the limit every tile.
    One far key that outweighs everything is added for the rows behind it, in a tile that is not
    a row's first."""
    from einf_b200 import ops

    dtype = torch.bfloat16
    heads, kv_heads = 6, 2
    requests = [(0, 1100), (900, 300)]
    (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, None,
                                                           seed=int(abs(growth)), layout="runs")
    q.mul_(0.2)
    k.mul_(0.2)
    # dim 0 carries the ramp: q[.., 0] = a, k_j[.., 0] = b * j with a * b * scale * log2(e) * 128 = growth
    a = 4.0
    b = growth / (a * scale * 1.4426950408889634 * 128.0)
    q[:, :, 0] = a
    for r, (start, q_len) in enumerate(requests):
        for j in range(start + q_len):
            k[int(table[r, j // page_size]), :, j % page_size, 0] = b * j
    # key 700 of request 0: far above the ramp for every row that sees it
    far = 700
    k[int(table[0, far // page_size]), :, far % page_size, 0] = abs(b) * 1100 + 60.0 / (a * scale)
    tiles, cursor = [], 0
    for r, (start, q_len) in enumerate(requests):
        for first in range(0, q_len, ops.Q_TILE):
            tiles.append((r, cursor + first, min(ops.Q_TILE, q_len - first), start + first))
        cursor += q_len
    q_tiles = torch.tensor(tiles, dtype=torch.int32, device=dev)
    want = torch.empty_like(q)
    st = status(dev)
    ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, None, st)
    assert torch.isfinite(want.float()).all()
    for cluster in (1, 2, 3):
        out = torch.full_like(q, float("nan"))
        ops.paged_prefill_attention(q, k, v, table, q_tiles, out, scale, None, st, use_tcgen05=True, prefill_cluster=cluster)
        assert int(st) == 0
        torch.testing.assert_close(out, want, **tol(dtype))
    # rows behind the far key hear it alone
    row = 800
    page, offset = int(table[0, far // page_size]), far % page_size
    torch.testing.assert_close(out[row, 0].float(), v[page, 0, offset].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("size, page_size", [(64, 16), (128, 32)])
def test_tcgen05_decode_far_key_and_window_edge(dev, size, page_size):
    """The tcgen05 decode kernel at every cluster size: one key far back (first and last key of a
    tile, of a page, of a CTA's share) carries the whole weight; a key just inside the window is
    heard and the one just outside is not."""
    from einf_b200 import ops

    dtype = torch.bfloat16
    context = 1100
    for far in (0, 1, page_size - 1, page_size, 127, 128, 129, 255, 256, 511, 512, 640, 1023, 1024, 1098, 1099):
        requests = [(context - 1, 1), (30, 1)]
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, 6, 2, size, page_size, requests, None, seed=far)
        q.mul_(0.05)
        page, offset = int(table[0, far // page_size]), far % page_size
        k[page, :, offset, :] = 0
        k[page, :, offset, 0] = 40.0
        q[0, :, 0] = 2.0 / scale
        for cluster in (1, 2, 4, 8):
            st = status(dev)
            out = torch.full_like(q, float("nan"))
            ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, None, cluster, st)
            assert int(st) == 0
            torch.testing.assert_close(out[0, 0].float(), v[page, 0, offset].float(), rtol=2e-2, atol=2e-2)
            torch.testing.assert_close(out[0, 5].float(), v[page, 1, offset].float(), rtol=2e-2, atol=2e-2)
    for window in (9, 128, 300):
        for inside in (True, False):
            (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, 2, 1, size, page_size, [(700, 1)], window, seed=3)
            q.mul_(0.05)
            key = 700 - window + 1 if inside else 700 - window
            page, offset = int(table[0, key // page_size]), key % page_size
            k[page, :, offset, :] = 0
            k[page, :, offset, 0] = 30.0
            q[0, :, 0] = 12.0
            for cluster in (1, 4):
                out = torch.empty_like(q)
                st = status(dev)
                ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, window, cluster, st)
                heard = torch.allclose(out[0, 0].float(), v[page, 0, offset].float(), rtol=2e-2, atol=2e-2)
                assert heard == inside, (window, inside, cluster)


@pytest.mark.parametrize("layout", ["runs", "broken runs"])
@pytest.mark.parametrize("heads, kv_heads, size, page_size", [(14, 2, 64, 16), (12, 2, 128, 16), (4, 1, 64, 8), (3, 1, 128, 64), (28, 4, 128, 16)])
def test_tcgen05_decode_over_runs_of_consecutive_pages(dev, layout, heads, kv_heads, size, page_size):
    """Pages that follow one another in the pool are fetched as one box per 128 keys; a tile whose
    pages do not (a swapped pair, the end of a context, a window's start) falls back to one box a
    page, tile by tile.  Same results as the plain statement either way, at every cluster size."""
    from einf_b200 import ops

    dtype = torch.bfloat16
    lengths = [1, 127, 128, 129, 256, 700, 1500, 2049]
    requests = [(n - 1, 1) for n in lengths]
    for window in (None, 300):
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window,
                                                               seed=7, layout=layout)
        want = torch.empty_like(q)
        st = status(dev)
        ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st)
        for cluster in (1, 2, 3, 4, 6, 7, 8):
            out = torch.full_like(q, float("nan"))
            ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, window, cluster, st)
            assert int(st) == 0
            torch.testing.assert_close(out, want, **tol(dtype))


@pytest.mark.parametrize("layout", ["runs", "broken runs"])
@pytest.mark.parametrize("heads, kv_heads, size, page_size", [(14, 2, 64, 16), (12, 2, 128, 16), (4, 1, 64, 8), (3, 1, 128, 64), (28, 4, 128, 16)])
def test_tcgen05_prefill_over_runs_of_consecutive_pages(dev, layout, heads, kv_heads, size, page_size):
    """The prefill kernel takes the same two ways to its keys: portions that begin at 0 and later,
    ends inside a tile and inside a page, with and without a window, at several cluster sizes."""
    from einf_b200 import ops

    dtype = torch.bfloat16
    requests = [(0, 300), (700, 129), (1500, 2), (127, 1), (0, 128), (1000, 257)]
    for window in (None, 300):
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window,
                                                               seed=11, layout=layout)
        tiles, cursor = [], 0
        for r, (start, q_len) in enumerate(requests):
            for first in range(0, q_len, ops.Q_TILE):
                tiles.append((r, cursor + first, min(ops.Q_TILE, q_len - first), start + first))
            cursor += q_len
        q_tiles = torch.tensor(tiles, dtype=torch.int32, device=dev)
        want = torch.empty_like(q)
        st = status(dev)
        ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st)
        for cluster in (1, 2, 8):
            out = torch.full_like(q, float("nan"))
            ops.paged_prefill_attention(q, k, v, table, q_tiles, out, scale, window, st, use_tcgen05=True,
                                        prefill_cluster=cluster)
            assert int(st) == 0
            torch.testing.assert_close(out, want, **tol(dtype))
        # the cluster that the wrapper picks itself from the longest cached prefix, as the engine calls it
        for cached_before in (None, 0, 300, 1500, 100000):
            out = torch.full_like(q, float("nan"))
            ops.paged_prefill_attention(q, k, v, table, q_tiles, out, scale, window, st, cached_before=cached_before)
            assert int(st) == 0
            torch.testing.assert_close(out, want, **tol(dtype))


def test_prefill_cluster_choice_fits_the_device(dev):
    """The cluster picked for a prompt portion never makes a grid that the device cannot hold at
    once, never exceeds what the cached prefix gives every CTA a key tile of, and is 1 for a
    portion at the start of its prompt."""
    from einf_b200 import ops

    for head_size in (64, 128):
        rooms = {c: ops.tcgen05_prefill_cluster_room(head_size, c) for c in range(1, 9)}
        assert rooms[1] >= 100 and all(rooms[c] >= 1 for c in rooms), rooms
        for ctas in (1, 7, 14, 28, 48, 56, 112, 150, 400):
            assert ops.prefill_cluster_size(ctas, head_size, 0) == 1
            assert ops.prefill_cluster_size(ctas, head_size, None) == 1
            for cached_before in (100, 256, 700, 5000):
                cluster = ops.prefill_cluster_size(ctas, head_size, cached_before)
                assert 1 <= cluster <= ops.prefill_prefix_bucket(cached_before)
                assert cluster == 1 or ctas <= rooms[cluster]
        assert ops.prefill_cluster_size(1, head_size, 5000) == 8


@pytest.mark.parametrize("heads, kv_heads, size, page_size", [(14, 2, 64, 16), (28, 4, 128, 16), (12, 2, 128, 16), (4, 2, 32, 16), (8, 8, 64, 5)])
def test_the_planned_decode_kernel_is_right_at_every_batch(dev, heads, kv_heads, size, page_size):
    """What ``decode_plan`` picks for a batch (which kernel, which cluster size; the choice asks the
    occupancy calculator of this device) is what the engine launches: run exactly that, at batches
    from one token to a few hundred, against the plain statement."""
    from einf_b200 import ops

    dtype = torch.bfloat16
    for tokens in (1, 3, 8, 33, 64, 300):
        lengths = [1 + (37 * i * i + 11 * tokens) % 700 for i in range(tokens)]
        requests = [(n - 1, 1) for n in lengths]
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, None,
                                                               seed=tokens, layout="runs" if tokens % 2 else "shuffled")
        kernel, cluster, splits = ops.decode_plan(tokens, heads, kv_heads, size, page_size)
        assert kernel == ("tcgen05" if ops.has_tcgen05_attention(size, page_size) else "mma")
        assert 1 <= cluster <= (16 if kernel == "tcgen05" else 8) and splits == 1   # contexts up to 4,096: one cluster a token
        want, out, st = torch.empty_like(q), torch.full_like(q, float("nan")), status(dev)
        ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, None, st)
        ops.paged_decode_attention_auto(q, k, v, table, seq, pos, out, scale, None, st)
        assert int(st) == 0
        torch.testing.assert_close(out, want, **tol(dtype))


@pytest.mark.parametrize("heads, kv_heads, size, page_size", [(14, 2, 64, 16), (28, 4, 128, 16), (5, 1, 64, 8), (20, 1, 128, 32)])
def test_tcgen05_decode_with_several_clusters_per_token(dev, heads, kv_heads, size, page_size):
    """A token's keys over several clusters that meet in global memory (what a few requests with
    long contexts get): every shape of (cluster size, clusters per token) that the device holds,
    clusters above eight included, contexts from one key (most CTAs have none) to thousands, with
    and without a window and a token list, against the plain statement; each launch twice, since
    the second finds the arrival counters as the first left them."""
    from einf_b200 import ops

    dtype = torch.bfloat16
    lengths = [1, 17, 129, 700, 3000, 5555]
    requests = [(n - 1, 1) for n in lengths]
    head_blocks = (heads // kv_heads + 15) // 16
    ran = 0
    for window in (None, 900):
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window,
                                                               seed=21, layout="runs" if window else "shuffled")
        want = torch.empty_like(q)
        st = status(dev)
        ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st)
        chosen = torch.tensor([5, 0, 3], dtype=torch.int32, device=dev)
        for cluster, splits in ((9, 1), (16, 1), (1, 2), (4, 2), (16, 2), (5, 3), (2, 4), (16, 4), (3, 8), (1, 8)):
            for token_list in (None, chosen):
                tokens = len(lengths) if token_list is None else len(chosen)
                if tokens * kv_heads * head_blocks * splits > ops.tcgen05_decode_cluster_room(size, cluster):
                    continue
                for _ in range(2):
                    out = torch.full_like(q, float("nan"))
                    ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, window, cluster, st, token_list, splits)
                    assert int(st) == 0
                    rows = slice(None) if token_list is None else chosen.long()
                    torch.testing.assert_close(out[rows], want[rows], **tol(dtype))
                ran += 1
    assert ran >= 12, "the device held too few of the shapes for this to be a test"
    with pytest.raises(ops.UnsupportedSize):
        ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, None, 4, st, None, 9)
    with pytest.raises(ops.UnsupportedSize):
        ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, None, 17, st)


@pytest.mark.parametrize("seed", range(6))
def test_tcgen05_decode_random_shapes(dev, seed):
    """Seeded random launches of the tcgen05 decode kernel: head counts and groups (up to two head
    blocks), both head sizes, page sizes, any cluster size up to 16 and any number of clusters per
    token, windows, token lists, contexts from one key to thousands, against the plain statement."""
    import random

    from einf_b200 import ops

    rng = random.Random(4000 + seed)
    dtype = torch.bfloat16
    for _ in range(10):
        size = rng.choice([64, 128])
        page_size = rng.choice([8, 16, 32, 64, 128])
        kv_heads = rng.choice([1, 2, 3, 4])
        heads = kv_heads * rng.choice([1, 2, 5, 7, 8, 16, 20])
        tokens = rng.choice([1, 2, 3, 5, 9])
        lengths = [rng.choice([1, rng.randint(1, 200), rng.randint(1, 1500), rng.randint(1, 6000)]) for _ in range(tokens)]
        window = rng.choice([None, None, rng.randint(1, 50), rng.randint(100, 2000)])
        cluster = rng.randint(1, 16)
        splits = rng.choice([1, 1, 2, 3, 4, 5, 8])
        head_blocks = (heads // kv_heads + 15) // 16
        if tokens * kv_heads * head_blocks * splits > ops.DECODE_SPLIT_SHARES:
            splits = 1
        requests = [(n - 1, 1) for n in lengths]
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window,
                                                               seed=rng.randrange(1 << 30), layout=rng.choice(["shuffled", "runs", "broken runs"]))
        chosen = None
        if tokens > 1 and rng.random() < 0.3:
            chosen = torch.tensor(sorted(rng.sample(range(tokens), rng.randint(1, tokens - 1))), dtype=torch.int32, device=dev)
        want, out, st = torch.empty_like(q), torch.full_like(q, float("nan")), status(dev)
        ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st)
        ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, window, cluster, st, chosen, splits)
        assert int(st) == 0
        rows = slice(None) if chosen is None else chosen.long()
        torch.testing.assert_close(out[rows], want[rows], **tol(dtype),
                                   msg=lambda m: f"{m}\n{(heads, kv_heads, size, page_size, lengths, window, cluster, splits)}")


@pytest.mark.parametrize("size", [64, 128])
def test_tcgen05_decode_finds_one_far_key_in_any_cluster_of_a_token(dev, size):
    """One key carries the whole weight: in the first, a middle and the last cluster's share of a
    long context, on the first and the last key of a share.  A share that is lost, or weighted
    against the wrong maximum when the shares are added up, shows."""
    from einf_b200 import ops

    dtype, page_size, context = torch.bfloat16, 16, 6000
    for cluster, splits in ((4, 2), (2, 4), (16, 2), (1, 8)):
        if 2 * splits > ops.tcgen05_decode_cluster_room(size, cluster):
            continue
        share = -(-(-(-context // (cluster * splits))) // 128) * 128        # keys per CTA, whole tiles
        for far in (0, share - 1, share, share * cluster - 1, share * cluster, share * cluster * (splits - 1), context - 1):
            far = min(far, context - 1)
            (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, 6, 2, size, page_size, [(context - 1, 1)], None, seed=far)
            q.mul_(0.05)
            page, offset = int(table[0, far // page_size]), far % page_size
            k[page, :, offset, :] = 0
            k[page, :, offset, 0] = 40.0
            q[0, :, 0] = 2.0 / scale
            st = status(dev)
            out = torch.full_like(q, float("nan"))
            ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, None, cluster, st, None, splits)
            assert int(st) == 0
            torch.testing.assert_close(out[0, 0].float(), v[page, 0, offset].float(), rtol=2e-2, atol=2e-2)
            torch.testing.assert_close(out[0, 5].float(), v[page, 1, offset].float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("heads, kv_heads, size", [(14, 2, 64), (28, 4, 128)])
def test_the_planned_decode_kernel_at_long_contexts(dev, heads, kv_heads, size):
    """What ``decode_plan`` picks when it is told the longest context: every shape fits the device
    and the scratch space at any batch and context; a few requests with long contexts get several
    clusters per token, many requests or short contexts get one; and the planned launch is right."""
    from einf_b200 import ops

    dtype, page_size = torch.bfloat16, 16
    for tokens in (1, 2, 3, 8, 16, 64, 256):
        for context in (None, 100, 4096, 4097, 20000, 32768, 131072):
            kernel, cluster, splits = ops.decode_plan(tokens, heads, kv_heads, size, page_size, context)
            pairs = tokens * kv_heads
            assert kernel == "tcgen05" and 1 <= cluster <= 16 and 1 <= splits <= ops.DECODE_MAX_SPLITS
            assert cluster == 1 or pairs * splits <= ops.tcgen05_decode_cluster_room(size, cluster)
            assert pairs * splits <= ops.DECODE_SPLIT_SHARES or splits == 1
            if context is None or context <= 4096 or tokens >= 64:
                assert splits == 1
    _, cluster, splits = ops.decode_plan(1, heads, kv_heads, size, page_size, 32768)
    assert cluster > 8 or splits > 1             # one long request: more CTAs than a cluster of eight
    assert ops.decode_plan(1, 14, 2, 64, page_size, 32768)[2] > 1
    assert ops.decode_plan(1, 14, 2, 64, page_size, 4096)[1:] == (16, 1)
    for lengths in ([20000], [9000, 4100, 13]):
        requests = [(n - 1, 1) for n in lengths]
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, None, seed=5)
        want, out, st = torch.empty_like(q), torch.full_like(q, float("nan")), status(dev)
        ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, None, st)
        ops.paged_decode_attention_auto(q, k, v, table, seq, pos, out, scale, None, st, max_context=max(lengths))
        assert int(st) == 0
        torch.testing.assert_close(out, want, **tol(dtype))


def test_attention_finds_one_far_key(dev):
    """Among hundreds of keys one, far back and on another page, matches the query: the
    output must be its value.  Random scores would hide a key that is skipped."""
    from einf_b200 import ops

    for dtype in DTYPES:
        for far in (0, 3, 130, 257, 511):
            requests = [(600, 1), (0, 700)]
            (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, 4, 2, 32, 16, requests, None, seed=far)
            q.mul_(0.05)
            page, offset = int(table[0, far // 16]), far % 16
            k[page, :, offset, :] = 0
            k[page, :, offset, 0] = 40.0
            q[0, :, 0] = 40.0 / scale / 40.0 * 2.0   # score 80 for that key alone
            out = torch.empty_like(q)
            st = status(dev)
            ops.paged_attention_generic(q, k, v, table, seq, pos, out, scale, None, st)
            torch.testing.assert_close(out[0, 0].float(), v[page, 0, offset].float(), rtol=2e-2, atol=2e-2)
            torch.testing.assert_close(out[0, 3].float(), v[page, 1, offset].float(), rtol=2e-2, atol=2e-2)


def test_attention_window_edge(dev):
    """A loud key just outside the window must not be heard; just inside it must."""
    from einf_b200 import ops

    window = 9
    for dtype in DTYPES:
        for inside in (True, False):
            requests = [(40, 1)]
            (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, 2, 1, 16, 4, requests, window, seed=3)
            q.mul_(0.05)
            key = 40 - window + 1 if inside else 40 - window
            page, offset = int(table[0, key // 4]), key % 4
            k[page, :, offset, :] = 0
            k[page, :, offset, 0] = 30.0
            q[0, :, 0] = 12.0
            out = torch.empty_like(q)
            st = status(dev)
            ops.paged_attention_generic(q, k, v, table, seq, pos, out, scale, window, st)
            heard = torch.allclose(out[0, 0].float(), v[page, 0, offset].float(), rtol=2e-2, atol=2e-2)
            assert heard == inside


def test_attention_reports_a_bad_page(dev):
    from einf_b200 import ops

    (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, torch.float32, 2, 1, 16, 4, [(0, 9)], None)
    table[0, 1] = 1000
    st = status(dev)
    out = torch.empty_like(q)
    ops.paged_attention_generic(q, k, v, table, seq, pos, out, scale, None, st)
    assert int(st) == ops.STATUS_BAD_PAGE and torch.isfinite(out).all()
    with pytest.raises(ops.UnsupportedSize):
        ops.paged_attention_generic(torch.empty(1, 2, 20, device=dev), torch.empty(1, 1, 4, 20, device=dev),
                                    torch.empty(1, 1, 4, 20, device=dev), table, seq, pos,
                                    torch.empty(1, 2, 20, device=dev), 1.0, None, st)


def test_kernels_refuse_the_cpu():
    from einf_b200 import ops

    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.silu_mul(torch.zeros(2, 4), torch.zeros(2, 2))


@pytest.mark.parametrize("vocab", [5, 331, 1024, 151936, 400003])   # the last: too long for the cluster kernel
def test_argmax_and_sampling(dev, vocab):
    from einf_b200 import ops

    torch.manual_seed(vocab)
    rows = 6
    logits = torch.randn(rows, vocab, device=dev) * 2
    logits[1, vocab // 2] = 50.0
    logits[2, 0] = logits[2, vocab - 1] = 60.0   # a tie: the first index wins
    tokens = torch.zeros(rows, dtype=torch.int32, device=dev)
    ops.argmax(logits, tokens)
    assert tokens.tolist() == torch.argmax(logits, -1).tolist() and int(tokens[2]) == 0
    # sampling: each draw lands where the plain inverse CDF puts it, up to rounding of the sums
    cases = [
        dict(temperature=0.0), dict(temperature=0.7), dict(temperature=1.3, top_k=min(3, vocab)),
        dict(temperature=1.0, top_p=0.6), dict(temperature=0.9, min_p=0.3),
        dict(temperature=1.1, top_k=min(50, vocab), top_p=0.8, min_p=0.05),
    ]
    def column(key, default, dtype):
        return torch.tensor([c.get(key, default) for c in cases], dtype=dtype, device=dev)
    temperature, top_k = column("temperature", 0.0, torch.float32), column("top_k", 0, torch.int32)
    top_p, min_p = column("top_p", 1.0, torch.float32), column("min_p", 0.0, torch.float32)
    for index in range(40):
        seed = torch.full((rows,), 1234, dtype=torch.int64, device=dev)
        sample_index = torch.full((rows,), index, dtype=torch.int64, device=dev)
        ops.sample(logits, tokens, temperature, top_k, top_p, min_p, seed, sample_index)
        got = tokens.tolist()
        assert got[0] == int(torch.argmax(logits[0]))
        u = ref.keyed_uniform(1234, index)
        for r in range(1, rows):
            c = cases[r]
            weights = ref.kept_weights(logits[r].cpu(), c["temperature"], c.get("top_k", 0), c.get("top_p", 1.0), c.get("min_p", 0.0)).double()
            assert weights[got[r]] > 0, (r, "drew a token the filters drop")
            cumulative = weights.cumsum(0) / weights.sum()
            low = float(cumulative[got[r]] - weights[got[r]] / weights.sum())
            high = float(cumulative[got[r]])
            assert low - 1e-4 <= u <= high + 1e-4, (r, index, u, low, high)


def test_sampling_filters_on_a_peaked_row_and_twice_the_same(dev):
    """Rows as a model makes them (a few tokens far above a bulk that lies 10 to 25 below the
    maximum, ties among the best, a k that ends inside a tie, a top-p that ends on the first
    token), each drawn many times: the token is always one the filters keep, the same call gives
    the same tokens again, and over many draws every kept token of a small kept set turns up."""
    from einf_b200 import ops

    torch.manual_seed(7)
    vocab = 151936
    cases = [
        dict(temperature=0.7, top_k=5), dict(temperature=1.0, top_p=0.5), dict(temperature=1.0, top_k=3, top_p=0.99),
        dict(temperature=0.9, top_p=0.9, min_p=0.02), dict(temperature=1.0, top_k=4), dict(temperature=1.2, top_p=0.3),
    ]
    rows = len(cases)
    logits = torch.randn(rows, vocab, device=dev) * 2 - 15.0
    for r in range(rows):
        best = torch.randperm(vocab, device=dev)[:12]
        logits[r, best] = torch.linspace(6.0, 3.0, 12, device=dev)
    logits[4, 100] = logits[4, 200] = logits[4, 300] = logits[4, 400] = logits[4, 500] = 9.0   # five tied, k = 4: all five stay
    logits[5, 77] = 20.0                                                                      # one token holds more than top_p
    def column(key, default, dtype):
        return torch.tensor([c.get(key, default) for c in cases], dtype=dtype, device=dev)
    temperature, top_k = column("temperature", 0.0, torch.float32), column("top_k", 0, torch.int32)
    top_p, min_p = column("top_p", 1.0, torch.float32), column("min_p", 0.0, torch.float32)
    kept = [ref.kept_weights(logits[r].cpu(), c["temperature"], c.get("top_k", 0), c.get("top_p", 1.0), c.get("min_p", 0.0)) > 0
            for r, c in enumerate(cases)]
    assert int(kept[4].sum()) == 5 and int(kept[5].sum()) == 1 and kept[5][77]
    seen = [set() for _ in cases]
    tokens, again = torch.zeros(rows, dtype=torch.int32, device=dev), torch.zeros(rows, dtype=torch.int32, device=dev)
    seed = torch.full((rows,), 99, dtype=torch.int64, device=dev)
    for index in range(300):
        sample_index = torch.full((rows,), index, dtype=torch.int64, device=dev)
        ops.sample(logits, tokens, temperature, top_k, top_p, min_p, seed, sample_index)
        ops.sample(logits, again, temperature, top_k, top_p, min_p, seed, sample_index)
        assert tokens.tolist() == again.tolist()
        for r, token in enumerate(tokens.tolist()):
            assert kept[r][token], (r, index, token)
            seen[r].add(token)
    for r in (0, 2, 4, 5):   # small kept sets: 300 draws find every member
        assert seen[r] == set(torch.nonzero(kept[r]).flatten().tolist()), r


@pytest.mark.parametrize("first_case", [0, 30])
def test_sampling_random_rows_and_filters(dev, first_case):
    """Seeded random rows and filters: vocabularies from 1 to 151,936 (fewer tokens than the
    cluster has CTAs, no multiple of eight, the benchmark's), flat, wide, peaked, tied and far
    negative logits, k of 1, of the whole vocabulary and beyond, top-p down to one in a million,
    min-p up to 1; every draw is a token the filters keep and lands where the inverse cumulative
    distribution of the kept weights puts it."""
    import random

    from einf_b200 import ops

    for case in range(first_case, first_case + 30):
        rng = random.Random(case)
        vocab = rng.choice([1, 2, 5, 7, 8, 9, 31, 100, 257, 1000, 4099, 32000, 50257, 151936])
        rows = rng.choice([1, 2, 3, 8])
        torch.manual_seed(case)
        style = rng.choice(["flat", "wide", "peaked", "ties", "far below zero"])
        logits = torch.randn(rows, vocab) * {"flat": 0.1, "wide": 5.0, "peaked": 2.0, "ties": 1.0, "far below zero": 3.0}[style]
        if style == "peaked":
            logits[:, rng.randrange(vocab)] += 25.0
        if style == "ties":
            logits = torch.round(logits * 2) / 2
        if style == "far below zero":
            logits -= 200.0
        logits = logits.to(dev)
        temperatures = [rng.choice([0.0, 0.3, 0.8, 1.0, 1.7]) for _ in range(rows)]
        top_ks = [rng.choice([0, 0, 1, 2, 5, 50, vocab, vocab + 3]) for _ in range(rows)]
        top_ps = [rng.choice([1.0, 1.0, 0.999, 0.9, 0.5, 0.05, 1e-6]) for _ in range(rows)]
        min_ps = [rng.choice([0.0, 0.0, 0.01, 0.3, 1.0]) for _ in range(rows)]
        columns = (torch.tensor(temperatures, device=dev), torch.tensor(top_ks, dtype=torch.int32, device=dev),
                   torch.tensor(top_ps, device=dev), torch.tensor(min_ps, device=dev))
        weights = [None if t == 0.0 else ref.kept_weights(logits[r].cpu(), t, top_ks[r], top_ps[r], min_ps[r]).double()
                   for r, t in enumerate(temperatures)]
        tokens = torch.zeros(rows, dtype=torch.int32, device=dev)
        for index in range(4):
            ops.sample(logits, tokens, *columns, torch.full((rows,), case, dtype=torch.int64, device=dev),
                       torch.full((rows,), index, dtype=torch.int64, device=dev))
            u = ref.keyed_uniform(case, index)
            for r, token in enumerate(tokens.tolist()):
                if weights[r] is None:
                    assert token == int(torch.argmax(logits[r])), (case, r)
                    continue
                assert 0 <= token < vocab and weights[r][token] > 0, (case, r, index, token)
                cumulative = weights[r].cumsum(0) / weights[r].sum()
                low = float(cumulative[token] - weights[r][token] / weights[r].sum())
                assert low - 1e-4 <= u <= float(cumulative[token]) + 1e-4, (case, r, index, u)


def test_sampling_frequencies(dev):
    from einf_b200 import ops

    logits = torch.tensor([[0.1, 2.0, 1.0, -1.0, 0.5]], device=dev).repeat(4000, 1)
    tokens = torch.zeros(4000, dtype=torch.int32, device=dev)
    ones = torch.ones(4000, device=dev)
    ops.sample(logits, tokens, ones * 0.8, torch.zeros(4000, dtype=torch.int32, device=dev), ones, ones * 0,
               torch.full((4000,), 5, dtype=torch.int64, device=dev), torch.arange(4000, dtype=torch.int64, device=dev))
    counts = torch.bincount(tokens.long().cpu(), minlength=5).float() / 4000
    want = torch.softmax(logits[0].cpu() / 0.8, -1)
    assert (counts - want).abs().max() < 0.03
