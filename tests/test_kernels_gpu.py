"""Each CUDA kernel alone against its plain reference, at sizes other than the
tiny models': head sizes in steps of 16, odd head counts and groups, widths and
vocabularies that are no power of two."""

from __future__ import annotations

import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def kernels():
    import vllm_from_scratch_b200.kernels as k
    return k


def close(actual, expected, dtype, scale=1.0, what=""):
    bound = (2e-5 if dtype == torch.float32 else 1.6e-2) * scale
    diff = float((actual.float() - expected.float()).abs().max())
    assert diff <= bound, f"{what}: max |diff| {diff:.3e} > {bound:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,hidden", [(1, 64), (7, 1000), (33, 2048), (5, 5120), (3, 8192 + 24),
                                           # many rows, as a portion of a prompt brings
                                           (300, 2048), (777, 1000), (260, 8192 + 24), (2050, 160)])
def test_add_rmsnorm(dtype, tokens, hidden):
    k = kernels()
    g = torch.Generator(device="cuda").manual_seed(tokens * hidden)
    x = torch.randn(tokens, hidden, device="cuda", generator=g).to(dtype)
    residual = torch.randn(tokens, hidden, device="cuda", generator=g) * 3
    weight = 1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)
    for with_x in (True, False):
        res_a, res_b = residual.clone(), residual.clone()
        out_a = torch.empty(tokens, hidden, device="cuda", dtype=dtype)
        out_b = torch.empty_like(out_a)
        k.add_rmsnorm(x if with_x else None, res_a, weight, 1e-5, out_a)
        plain_ops.add_rmsnorm(x if with_x else None, res_b, weight, 1e-5, out_b)
        close(out_a, out_b, dtype, scale=4, what="normed")
        assert torch.allclose(res_a, res_b, atol=1e-6), "residual sum"
    rows = torch.tensor([tokens - 1, 0], dtype=torch.int32, device="cuda")
    res_a = residual.clone()
    out_a = torch.empty(2, hidden, device="cuda", dtype=dtype)
    out_b = torch.empty_like(out_a)
    k.add_rmsnorm(x, res_a, weight, 1e-6, out_a, rows)
    plain_ops.add_rmsnorm(x, residual.clone(), weight, 1e-6, out_b, rows)
    close(out_a, out_b, dtype, scale=4, what="gathered rows")
    assert torch.equal(res_a, residual), "gathered norm must not touch the residual"


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_bad_id(dtype):
    k = kernels()
    table = torch.randn(503, 96, device="cuda").to(dtype)
    ids = torch.tensor([0, 502, 17, 17, 250], dtype=torch.int32, device="cuda")
    out = torch.empty(5, 96, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    k.embedding(table, ids, out, flag)
    assert torch.equal(out, table[ids.long()].float()) and int(flag) == 0
    ids[3] = 503
    k.embedding(table, ids, out, flag)
    assert int(flag) == 4 and float(out[3].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,inter", [(1, 160), (9, 6144), (130, 1111)])
def test_silu_mul(dtype, tokens, inter):
    k = kernels()
    gate_up = (torch.randn(tokens, 2 * inter, device="cuda") * 3).to(dtype)
    out_a = torch.empty(tokens, inter, device="cuda", dtype=dtype)
    out_b = torch.empty_like(out_a)
    k.silu_mul(gate_up, out_a)
    plain_ops.silu_mul(gate_up, out_b)
    close(out_a, out_b, dtype, scale=10, what="silu_mul")


@pytest.mark.parametrize("m,n,k_", [(1, 503, 96), (5, 64, 64), (70, 257, 130), (129, 1000, 2048), (2, 4099, 77)])
def test_gemm_f32_is_true_float32(m, n, k_):
    k = kernels()
    g = torch.Generator(device="cuda").manual_seed(m + n + k_)
    x = torch.randn(m, k_, device="cuda", generator=g)
    w = torch.randn(n, k_, device="cuda", generator=g)
    out = torch.empty(m, n, device="cuda")
    k.gemm(x, w, out)
    exact = (x.double() @ w.double().T)
    # float32 accumulation error grows like sqrt(K) * 2^-24 * |x||w|; TF32 would be ~1e-3.
    assert float((out.double() - exact).abs().max()) < 2e-6 * (k_ ** 0.5) * 4
    # a row's result does not depend on the rows beside it
    alone = torch.empty(1, n, device="cuda")
    k.gemm(x[m - 1:m].contiguous(), w, alone)
    assert torch.equal(alone[0], out[m - 1])


@pytest.mark.parametrize("m,n,k_", [(1, 512, 128), (8, 503, 96), (70, 264, 136), (300, 1024, 2048)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16(m, n, k_, out_dtype):
    k = kernels()
    g = torch.Generator(device="cuda").manual_seed(m + n + k_)
    x = torch.randn(m, k_, device="cuda", generator=g).bfloat16()
    w = torch.randn(n, k_, device="cuda", generator=g).bfloat16()
    out = torch.empty(m, n, device="cuda", dtype=out_dtype)
    k.gemm(x, w, out)
    exact = x.double() @ w.double().T
    scale = float(exact.abs().max())
    bound = scale * (2 ** -8 if out_dtype == torch.bfloat16 else 1e-5)
    assert float((out.double() - exact).abs().max()) <= bound


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot,page", [(4, 2, 16, 16, 16), (6, 2, 32, 32, 8), (5, 5, 48, 48, 16),
                                               (16, 8, 128, 128, 16), (3, 1, 80, 32, 4), (8, 2, 256, 256, 32)])
def test_head_norm_rope_cache(dtype, nq, nkv, d, rot, page):
    k = kernels()
    tokens, pages = 37, 12
    g = torch.Generator(device="cuda").manual_seed(nq * d)
    qkv = torch.randn(tokens, (nq + 2 * nkv) * d, device="cuda", generator=g).to(dtype)
    positions = torch.randint(0, 5000, (tokens,), device="cuda", generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * page, device="cuda", generator=g)[:tokens].to(torch.int32)
    slots[5] = -1
    qw = 1 + 0.1 * torch.randn(d, device="cuda", generator=g)
    kw = 1 + 0.1 * torch.randn(d, device="cuda", generator=g)
    inv_freq = 1.0 / (1e4 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot)).cuda()
    for use_norm in (True, False):
        outs = []
        for op in (k.head_norm_rope_cache, plain_ops.head_norm_rope_cache):
            q_out = torch.zeros(tokens, nq * d, device="cuda", dtype=dtype)
            kp = torch.zeros(pages, nkv, page, d, device="cuda", dtype=dtype)
            vp = torch.zeros_like(kp)
            op(qkv, positions, slots, qw if use_norm else None, kw if use_norm else None, inv_freq, rot,
               1e-6, q_out, kp, vp, nq, nkv, d, page)
            outs.append((q_out, kp, vp))
        scale = 1.0 if use_norm else 4.0
        close(outs[0][0], outs[1][0], dtype, scale=4 * scale, what="queries")
        close(outs[0][1], outs[1][1], dtype, scale=4 * scale, what="key pages")
        assert torch.equal(outs[0][2], outs[1][2]), "values are copied as they are"
    # no cache given: only queries are produced
    q_out = torch.zeros(tokens, nq * d, device="cuda", dtype=dtype)
    k.head_norm_rope_cache(qkv, positions, slots, qw, kw, inv_freq, rot, 1e-6, q_out, None, None, nq, nkv, d, page)
    assert float(q_out.abs().max()) > 0


def _attention_case(dtype, nq, nkv, d, page, q_lens, seq_lens, window, seed=0, standout=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    requests = len(q_lens)
    tokens = sum(q_lens)
    pages_per = [-(-s // page) for s in seq_lens]
    total_pages = sum(pages_per) + 3
    order = torch.randperm(total_pages, device="cuda", generator=g).tolist()
    table = torch.full((requests, max(pages_per)), -1, dtype=torch.int32, device="cuda")
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
        at += n
    kp = torch.randn(total_pages, nkv, page, d, device="cuda", generator=g).to(dtype)
    vp = torch.randn(total_pages, nkv, page, d, device="cuda", generator=g).to(dtype)
    q = torch.randn(tokens, nq * d, device="cuda", generator=g).to(dtype)
    if standout:
        # One far key gets a large score for every query of request 0: the result
        # must be dominated by that key's value.
        far = 3
        page_id, offset = int(table[0, far // page]), far % page
        kp[page_id, :, offset, :] = 0
        kp[page_id, :, offset, 0] = 30.0
        q.view(tokens, nq, d)[:q_lens[0], :, 0] = 6.0
    import itertools
    query_start = torch.tensor([0] + list(itertools.accumulate(q_lens)), dtype=torch.int32, device="cuda")
    seq = torch.tensor(seq_lens, dtype=torch.int32, device="cuda")
    return q, kp, vp, query_start, seq, table


ATTENTION_SHAPES = [
    # nq, nkv, d, page, q_lens, seq_lens, window
    (4, 2, 16, 16, [5, 1, 17], [5, 40, 33], None),
    (6, 2, 32, 8, [1, 1, 1, 1], [1, 7, 64, 130], None),
    (5, 5, 48, 16, [40, 2], [100, 77], 24),
    (16, 8, 128, 16, [1, 64, 3], [700, 64, 290], None),
    (8, 1, 64, 32, [33], [300], 50),
    (3, 3, 80, 4, [20, 1], [20, 90], None),
    (2, 1, 256, 16, [18, 1], [50, 200], None),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATTENTION_SHAPES)
def test_paged_attention(dtype, shape):
    k = kernels()
    nq, nkv, d, page, q_lens, seq_lens, window = shape
    for standout in (False, True):
        q, kp, vp, start, seq, table = _attention_case(dtype, nq, nkv, d, page, q_lens, seq_lens, window,
                                                       seed=nq * d + page, standout=standout)
        out_a = torch.zeros_like(q)
        out_b = torch.zeros_like(q)
        args = (start, seq, table, nq, nkv, d, page, d ** -0.5, window, max(q_lens), max(seq_lens))
        k.paged_attention(q, kp, vp, out_a, *args)
        plain_ops.paged_attention(q, kp, vp, out_b, *args)
        close(out_a, out_b, dtype, scale=4, what=f"attention standout={standout}")


@pytest.mark.parametrize("d", [32, 128])
@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge_and_released_pages(dtype, d):
    """A key exactly at the window's edge is read, the one before it is not, and a
    page that was given back (-1 in the table) is never touched.  (Head size 128 in
    bfloat16 goes through the decode kernel that copies whole pages.)"""
    k = kernels()
    nq, nkv, page, window = 2, 1, 8, 10
    q, kp, vp, start, seq, table = _attention_case(dtype, nq, nkv, d, page, [1], [41], window, seed=9)
    # query at position 40 reads keys 31..40; make key 31 (edge, inside) and key 30 (outside) stand out
    q.view(1, nq, d)[:] = 0
    q.view(1, nq, d)[:, :, 0] = 8.0
    for pos, value in ((31, 12.0), (30, 20.0)):
        kp[int(table[0, pos // page]), :, pos % page, :] = 0
        kp[int(table[0, pos // page]), :, pos % page, 0] = value
    released = table.clone()
    released[0, :3] = -1                       # positions 0..23 lie before every window
    outs = []
    for tab in (table, released):
        out = torch.zeros_like(q)
        k.paged_attention(q, kp, vp, out, start, seq, tab, nq, nkv, d, page, d ** -0.5, window, 1, 41)
        outs.append(out)
    expected = torch.zeros_like(q)
    plain_ops.paged_attention(q, kp, vp, expected, start, seq, table, nq, nkv, d, page, d ** -0.5, window, 1, 41)
    close(outs[0], expected, dtype, scale=4, what="window edge")
    assert torch.equal(outs[0], outs[1]), "released pages must not matter"
    edge_value = vp[int(table[0, 31 // page]), 0, 31 % page].float()
    assert float((outs[0].view(nq, d)[0].float() - edge_value).abs().max()) < 0.05, "edge key must dominate"


TENSOR_CORE_SHAPES = [
    # nq, nkv, d, page, q_lens, seq_lens, window      (decode: every q_len is 1)
    (16, 8, 128, 16, [1, 1, 1], [700, 64, 2900], None),
    (16, 8, 128, 16, [1], [5000], None),
    (32, 8, 128, 16, [1, 1], [1, 333], None),
    (64, 8, 128, 32, [1, 1, 1, 1, 1], [17, 300, 1000, 64, 65], None),
    (4, 4, 64, 8, [1, 1], [100, 3000], 700),
    (4, 1, 256, 16, [1, 1], [50, 600], None),
    (16, 8, 128, 128, [1, 1], [300, 1000], None),
    (8, 4, 128, 64, [1, 1, 1], [64, 65, 700], 100),
    (16, 8, 128, 16, [200, 1, 64, 3], [200, 500, 300, 131], None),
    (8, 2, 64, 16, [130, 70], [130, 1000], None),
    (6, 3, 128, 16, [300], [1500], 256),
    (2, 1, 256, 8, [65, 1], [65, 90], None),
    # pages whose size is no power of two: the decode kernel with per-thread copies and the general one
    (16, 8, 128, 24, [1, 1, 1], [700, 23, 2900], None),
    (8, 2, 64, 48, [1, 1], [49, 1500], 300),
    (8, 4, 128, 48, [130, 1, 70], [130, 500, 1000], None),
    (4, 2, 64, 24, [200, 3], [333, 75], 100),
]


@pytest.mark.parametrize("shape", TENSOR_CORE_SHAPES)
def test_tensor_core_attention(shape):
    """The bfloat16 tensor-core kernels (decode with split keys, and the general one)
    against the plain reference, with and without a key that must dominate."""
    k = kernels()
    from vllm_from_scratch_b200.kernels import attention_bf16
    nq, nkv, d, page, q_lens, seq_lens, window = shape
    for standout in (False, True):
        q, kp, vp, start, seq, table = _attention_case(torch.bfloat16, nq, nkv, d, page, q_lens, seq_lens,
                                                       window, seed=nq + d + page, standout=standout)
        out_a = torch.zeros_like(q)
        out_b = torch.zeros_like(q)
        args = (start, seq, table, nq, nkv, d, page, d ** -0.5, window, max(q_lens), max(seq_lens))
        assert attention_bf16.paged_attention_bf16(q, kp, vp, out_a, *args), "shape must take the fast path"
        plain_ops.paged_attention(q, kp, vp, out_b, *args)
        close(out_a, out_b, torch.bfloat16, scale=2, what=f"tensor-core attention standout={standout}")


def test_decode_attention_same_for_any_split():
    """The number of splits is a launch detail: planning for a longer context
    (more splits) must give the same result beyond rounding."""
    from vllm_from_scratch_b200.kernels import attention_bf16
    nq, nkv, d, page = 16, 8, 128, 16
    q, kp, vp, start, seq, table = _attention_case(torch.bfloat16, nq, nkv, d, page, [1, 1], [900, 77], None, seed=4)
    outs = []
    for planned in (900, 40000):
        out = torch.zeros_like(q)
        assert attention_bf16.paged_attention_bf16(q, kp, vp, out, start, seq, table, nq, nkv, d, page,
                                                   d ** -0.5, None, 1, planned)
        outs.append(out.float())
    assert float((outs[0] - outs[1]).abs().max()) < 8e-3


@pytest.mark.parametrize("m,n,k_", [(1, 512, 128), (8, 4096, 2048), (3, 2048, 6144), (16, 503, 96), (9, 264, 160),
                                    (16, 12288, 2048), (5, 151936, 256), (3, 1003, 256), (7, 5, 12288), (8, 77, 384),
                                    (12, 2048, 2048), (9, 1003, 6144)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_few_rows_gemm(m, n, k_, out_dtype):
    """The weight-streaming kernel (M <= 16): exact float64 reference, and a token's
    result must not depend on the other tokens of the launch."""
    from vllm_from_scratch_b200.kernels import gemm_bf16
    g = torch.Generator(device="cuda").manual_seed(m + n + k_)
    x = torch.randn(m, k_, device="cuda", generator=g).bfloat16()
    w = torch.randn(n, k_, device="cuda", generator=g).bfloat16()
    out = torch.full((m, n), 7.0, device="cuda", dtype=out_dtype)
    gemm_bf16._skinny(x, w, out, 0)
    exact = x.double() @ w.double().T
    scale = float(exact.abs().max())
    bound = scale * (2 ** -8 if out_dtype == torch.bfloat16 else 1e-5)
    assert float((out.double() - exact).abs().max()) <= bound
    # (up to 8 rows and from 9 rows on are different kernels: compare within each)
    fewer = 1 if m <= 8 else 9
    alone = torch.empty(fewer, n, device="cuda", dtype=out_dtype)
    gemm_bf16._skinny(x[m - fewer:m].clone(), w, alone, 0)
    assert torch.equal(alone[-1], out[m - 1])


@pytest.mark.parametrize("m,inter,k_", [(1, 160, 96), (8, 6144, 2048), (16, 1111, 64), (40, 256, 128), (5, 1003, 256),
                                        (2, 8, 6144), (12, 1003, 256), (16, 6144, 2048)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_silu_gemm(m, inter, k_, dtype):
    k = kernels()
    g = torch.Generator(device="cuda").manual_seed(m + inter)
    x = torch.randn(m, k_, device="cuda", generator=g).to(dtype)
    w = (torch.randn(2 * inter, k_, device="cuda", generator=g) * 0.1).to(dtype)
    out_a = torch.empty(m, inter, device="cuda", dtype=dtype)
    out_b = torch.empty_like(out_a)
    k.gated_silu_gemm(x, w, out_a)
    plain_ops.gated_silu_gemm(x, w, out_b)
    bound = float(out_b.float().abs().max()) * (2 ** -7 if dtype == torch.bfloat16 else 1e-5)
    assert float((out_a.float() - out_b.float()).abs().max()) <= bound
    if dtype == torch.bfloat16 and m <= 16 and k_ % 32 == 0:
        # the fused few-rows kernel itself, whatever the dispatch above chose
        from vllm_from_scratch_b200.kernels import gemm_bf16
        fused = torch.empty_like(out_a)
        gemm_bf16._skinny(x, w, fused, inter)
        assert float((fused.float() - out_b.float()).abs().max()) <= bound


# token rows, residual width, width of the rows that go into the first product, width of the gated product
SPLIT_NORM_SHAPES = [(1, 128, 256, 24), (8, 2048, 2048, 6144), (5, 1152, 384, 1000), (12, 2048, 6144, 264),
                     (16, 5120, 128, 512), (9, 384, 1024, 8), (3, 6144, 128, 64)]


@pytest.mark.parametrize("shape", SPLIT_NORM_SHAPES)
def test_rmsnorm_split_over_two_products(shape):
    """A product that adds into the residual and hands on half-normalised rows, then a gated and a
    plain product that apply the root: each against its plain version, the pair against the
    unsplit sequence (product, add + RMSNorm, product), and a token's results must not depend on
    the other tokens of the launch."""
    k = kernels()
    m, hidden, first_k, inter = shape
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    rand = lambda *dims, scale=1.0: torch.randn(*dims, device="cuda", generator=g) * scale
    x = rand(m, first_k).bfloat16()
    w_first = rand(hidden, first_k, scale=first_k ** -0.5).bfloat16()
    w_gate_up = rand(2 * inter, hidden, scale=hidden ** -0.5).bfloat16()
    w_plain = rand(inter, hidden, scale=hidden ** -0.5).bfloat16()
    weight = 1 + 0.1 * rand(hidden)
    residual = rand(m, hidden, scale=3.0)
    residual[m - 1, 7] = 300.0                       # one large element: the sums of squares must carry it
    eps = 1e-5
    for w in (w_first, w_plain):
        assert k.split_norm_ok(m, w, fold=True) and k.split_norm_ok(m, w, fold=False)
    assert k.split_norm_ok(m, w_gate_up, fold=False, gated=True)

    def run(ops, rows):
        res = residual[:rows].clone()
        half = torch.full((rows, hidden), 7.0, device="cuda", dtype=torch.bfloat16)
        squares = torch.full((rows, hidden // 8), 7.0, device="cuda")
        ops.gemm(x[:rows].contiguous(), w_first, half, fold=(res, weight, squares))
        act = torch.full((rows, inter), 7.0, device="cuda", dtype=torch.bfloat16)
        ops.gated_silu_gemm(half, w_gate_up, act, scale=(squares, eps))
        out = torch.full((rows, inter), 7.0, device="cuda", dtype=torch.bfloat16)
        ops.gemm(half, w_plain, out, scale=(squares, eps))
        return res, half, squares, act, out

    got, want = run(k, m), run(plain_ops, m)
    # The residual carries the first product rounded to bfloat16: sums taken in another order may
    # round it the other way, one unit in its last place.
    rounding = float((x.float() @ w_first.float().T).abs().max()) * 2 ** -7
    for name, a, b in zip(("residual", "half-normalised rows", "sums of squares", "gated product", "product"), got, want):
        bound = float(b.float().abs().max()) * 2 ** -7 if name != "residual" else rounding
        diff = float((a.float() - b.float()).abs().max())
        assert diff <= bound, f"{name}: max |diff| {diff:.3e} > {bound:.3e}"
    # the same through a norm of its own
    res = residual.clone()
    first = torch.empty(m, hidden, device="cuda", dtype=torch.bfloat16)
    plain_ops.gemm(x, w_first, first)
    normed = torch.empty_like(first)
    plain_ops.add_rmsnorm(first, res, weight, eps, normed)
    act, out = torch.empty_like(got[3]), torch.empty_like(got[4])
    plain_ops.gated_silu_gemm(normed, w_gate_up, act)
    plain_ops.gemm(normed, w_plain, out)
    assert float((got[0] - res).abs().max()) <= rounding
    for name, a, b in (("gated product", got[3], act), ("product", got[4], out)):
        bound = float(b.float().abs().max()) * 2 ** -6
        assert float((a.float() - b.float()).abs().max()) <= bound, name
    fewer = 1 if m <= 8 else 9                       # up to 8 rows and from 9 rows on are different kernels
    if m > fewer:
        alone = run(k, fewer)
        for a, b in zip(alone, got):
            assert torch.equal(a[fewer - 1], b[fewer - 1])


def test_split_norm_refusals():
    k = kernels()
    bf = lambda *dims: torch.zeros(*dims, device="cuda", dtype=torch.bfloat16)
    assert not k.split_norm_ok(17, bf(256, 256), fold=False)          # too many token rows
    assert not k.split_norm_ok(4, bf(256, 192), fold=False)           # K is no multiple of 128
    assert not k.split_norm_ok(4, bf(260, 256), fold=True)            # no whole blocks of eight columns
    assert not k.split_norm_ok(4, torch.zeros(256, 256, device="cuda"), fold=False)      # float32
    with pytest.raises(k.KernelError):
        k.gemm(bf(4, 192), bf(256, 192), bf(4, 256), scale=(torch.ones(4, 24, device="cuda"), 1e-6))


# token rows, intermediate width, K: tiles of 2 x 96 and 2 x 128 rows, one block of token rows and many,
# a last block that is partly empty, the benchmark's prompt through the dispatch
TENSOR_MEMORY_GATED_SHAPES = [(1, 96, 64), (130, 384, 320), (300, 192, 128), (128, 6144, 2048), (2048, 6144, 2048),
                              (2304, 1280, 4096), (2048, 480, 192)]


@pytest.mark.parametrize("shape", TENSOR_MEMORY_GATED_SHAPES)
def test_tensor_memory_gated_product(shape):
    """The feed-forward's first product with its activation on the 5th-generation tensor cores,
    against the plain version; where the engine's dispatch uses it (whole blocks of 128 token
    rows from 2048 on) also through ``kernels.gated_silu_gemm``."""
    from vllm_from_scratch_b200.kernels import gemm_bf16
    k = kernels()
    m, inter, width = shape
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    x = torch.randn(m, width, device="cuda", generator=g).bfloat16()
    w = (torch.randn(2 * inter, width, device="cuda", generator=g) * width ** -0.5).bfloat16()
    want = torch.empty(m, inter, device="cuda", dtype=torch.bfloat16)
    plain_ops.gated_silu_gemm(x, w, want)
    bound = float(want.float().abs().max()) * 2 ** -7
    got = torch.full_like(want, 7.0)
    gemm_bf16.tc_gated_gemm(x, w, got)
    assert float((got.float() - want.float()).abs().max()) <= bound
    if gemm_bf16.tc_gated_ok(m, inter, width, x, w, got):
        through = torch.full_like(want, 7.0)
        k.gated_silu_gemm(x, w, through)
        assert torch.equal(through, got)
    assert k.device_error() is None


SPLIT_BATCH_SHAPES = [
    # nq, nkv, d, page, q_lens (single tokens first), seq_lens, window
    (8, 2, 64, 16, [1, 1, 1, 40, 70], [300, 64, 1, 40, 170], None),
    (4, 2, 128, 16, [1, 1, 200, 65], [500, 129, 200, 300], None),
    (4, 4, 128, 8, [1, 130], [77, 130], 64),
    (16, 8, 128, 16, [1] * 9 + [300, 2, 256], [2100, 64, 65, 1, 700, 33, 1000, 128, 4000, 300, 50, 900], None),
]


@pytest.mark.parametrize("shape", SPLIT_BATCH_SHAPES)
def test_mixed_batch_in_two_launches(shape):
    """A step whose first requests bring one token and whose others bring portions: the single
    tokens go to the decode kernel, the portions (which begin at a row other than 0) to theirs."""
    k = kernels()
    from vllm_from_scratch_b200.kernels import attention_bf16
    nq, nkv, d, page, q_lens, seq_lens, window = shape
    singles = sum(1 for n in q_lens if n == 1)
    q, kp, vp, start, seq, table = _attention_case(torch.bfloat16, nq, nkv, d, page, q_lens, seq_lens, window,
                                                   seed=nq + d)
    out_a = torch.full_like(q, 7.0)
    out_b = torch.zeros_like(q)
    before = k.launch_count
    k.paged_attention(q, kp, vp, out_a, start, seq, table, nq, nkv, d, page, d ** -0.5, window, max(q_lens),
                      max(seq_lens), singles)
    assert k.launch_count == before + 2
    assert attention_bf16.attention_error_code() == 0
    plain_ops.paged_attention(q, kp, vp, out_b, start, seq, table, nq, nkv, d, page, d ** -0.5, window, max(q_lens),
                              max(seq_lens))
    close(out_a, out_b, torch.bfloat16, scale=2, what="mixed batch in two launches")


FUSED_DECODE_SHAPES = [
    # nq, nkv, page, seq_lens, window, head norms
    (16, 8, 16, [1, 63, 64, 65, 129, 1000, 2100, 17], None, True),
    (4, 4, 8, [2, 300, 128, 513], None, True),
    (16, 1, 64, [700, 64, 1, 1025], None, False),
    (6, 2, 16, [40, 600, 257, 1024], 256, True),
    (8, 2, 128, [128, 129, 3000], None, True),
]


@pytest.mark.parametrize("shape", FUSED_DECODE_SHAPES)
def test_fused_decode_attention(shape):
    """Head norms, rotation, the store of the new key and value and the attention of a decode step
    in one kernel give what the two kernels give one after the other: the same output, the same
    pages, bit for bit (the arithmetic is the same), and nothing stored for a negative slot."""
    k = kernels()
    from vllm_from_scratch_b200.kernels import attention_bf16
    nq, nkv, page, seq_lens, window, normed = shape
    d = 128
    requests = len(seq_lens)
    _, kp, vp, _, seq, table = _attention_case(torch.bfloat16, nq, nkv, d, page, [1] * requests, seq_lens, window,
                                               seed=nq + page)
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(requests, (nq + 2 * nkv) * d, device="cuda", generator=g).bfloat16()
    positions = (seq - 1).to(torch.int32)
    page_of = table[torch.arange(requests, device="cuda"), ((seq - 1) // page).long()]
    slots = (page_of * page + (seq - 1) % page).to(torch.int32)
    slots[-1] = -1                                       # the last request stores nothing
    q_w = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)) if normed else None
    k_w = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)) if normed else None
    inv_freq = (1e4 ** (-torch.arange(0, d, 2, device="cuda").float() / d)).contiguous()
    start = torch.arange(requests + 1, dtype=torch.int32, device="cuda")
    # one after the other
    kp_a, vp_a = kp.clone(), vp.clone()
    q = torch.empty(requests, nq * d, device="cuda", dtype=torch.bfloat16)
    k.head_norm_rope_cache(qkv, positions, slots, q_w, k_w, inv_freq, d, 1e-6, q, kp_a, vp_a, nq, nkv, d, page)
    out_a = torch.zeros_like(q)
    k.paged_attention(q, kp_a, vp_a, out_a, start, seq, table, nq, nkv, d, page, d ** -0.5, window, 1, max(seq_lens))
    # in one
    kp_b, vp_b = kp.clone(), vp.clone()
    out_b = torch.zeros_like(q)
    assert k.fused_decode_attention(qkv, positions, slots, q_w, k_w, inv_freq, d, 1e-6, kp_b, vp_b, out_b, seq, table,
                                    nq, nkv, d, page, d ** -0.5, window, max(seq_lens))
    assert attention_bf16.attention_error_code() == 0
    assert torch.equal(kp_a, kp_b) and torch.equal(vp_a, vp_b)
    assert not torch.equal(kp_a, kp)                     # something was stored
    stored = slots[:-1].long()
    assert torch.equal(kp_b.view(-1, nkv, page, d)[stored // page, :, stored % page],
                       kp_a.view(-1, nkv, page, d)[stored // page, :, stored % page])
    # The request that stores nothing reads what its slot held before in the first path and its
    # own new key in the second: compare the others exactly, and all of them with the plain
    # reference given the pages after the store.
    assert torch.equal(out_a[:-1], out_b[:-1])
    kp_c, vp_c = kp_a.clone(), vp_a.clone()
    q_c = torch.empty_like(q)
    all_slots = (page_of * page + (seq - 1) % page).to(torch.int32)
    k.head_norm_rope_cache(qkv, positions, all_slots, q_w, k_w, inv_freq, d, 1e-6, q_c, kp_c, vp_c, nq, nkv, d, page)
    expected = torch.zeros_like(q)
    plain_ops.paged_attention(q_c, kp_c, vp_c, expected, start, seq, table, nq, nkv, d, page, d ** -0.5, window, 1,
                              max(seq_lens))
    close(out_b, expected, torch.bfloat16, scale=2, what="fused decode attention")


TENSOR_MEMORY_ATTENTION_SHAPES = [
    # nq, nkv, d, page, q_lens, seq_lens, window
    (2, 1, 128, 16, [128], [128], None),
    (16, 8, 128, 16, [300], [300], None),
    (4, 2, 128, 16, [200, 1, 64, 3], [200, 500, 300, 131], None),
    (8, 2, 128, 32, [130, 70], [130, 1000], None),
    (6, 3, 128, 8, [333], [1500], 256),
    (4, 4, 128, 128, [257, 64], [257, 640], None),
    (2, 2, 128, 16, [1, 2, 63, 65, 129], [1, 2, 63, 65, 129], None),
    (2, 1, 128, 16, [384, 100], [2500, 1100], 700),
    (16, 8, 128, 16, [512], [8192], None),
    (1, 1, 128, 16, [64, 300], [3000, 300], None),
    # a whole prompt: the row blocks far from its beginning are divided, the first ones are not
    (16, 8, 128, 16, [2048], [2048], None),
    (8, 4, 128, 16, [1000, 700], [1000, 2000], None),
    (4, 2, 128, 32, [1300], [1300], 500),
]


@pytest.mark.parametrize("divide_keys", [True, False])
@pytest.mark.parametrize("shape", TENSOR_MEMORY_ATTENTION_SHAPES)
def test_tensor_memory_attention(shape, divide_keys, monkeypatch):
    """The tcgen05 kernel for portions of prompts against the plain reference, with and without
    the division of a row block's keys over several blocks (which launches of few row blocks
    over many keys get, as all of these do whose requests are 512 keys long and more)."""
    from vllm_from_scratch_b200.kernels import attention_bf16
    monkeypatch.setattr(attention_bf16, "USE_TC_KEY_SPLIT", divide_keys)
    nq, nkv, d, page, q_lens, seq_lens, window = shape
    for standout in (False, True):
        q, kp, vp, start, seq, table = _attention_case(torch.bfloat16, nq, nkv, d, page, q_lens, seq_lens,
                                                       window, seed=nq + page, standout=standout)
        out_a = torch.zeros_like(q)
        out_b = torch.zeros_like(q)
        args = (start, seq, table, nq, nkv, d, page, d ** -0.5, window, max(q_lens), max(seq_lens))
        assert attention_bf16.paged_attention_bf16(q, kp, vp, out_a, *args)
        assert attention_bf16.attention_error_code() == 0
        plain_ops.paged_attention(q, kp, vp, out_b, *args)
        close(out_a, out_b, torch.bfloat16, scale=2, what=f"tensor-memory attention standout={standout}")


def test_tensor_map_cache_keeps_copies_valid():
    """The cache of tensor maps empties itself when it is full; a launcher that has taken one map
    and then asks for another must not be left with a dangling one.  Host-only: more maps than
    the cache holds are encoded over one buffer, nothing is launched."""
    from vllm_from_scratch_b200.kernels import attention_bf16
    assert attention_bf16.tensor_map_cache_self_check(5000) == 0
    assert attention_bf16.tensor_map_cache_self_check(9000) == 0


def test_sm_count_comes_from_the_device():
    from vllm_from_scratch_b200.kernels import attention_bf16
    assert attention_bf16.sm_count() == torch.cuda.get_device_properties(0).multi_processor_count


def test_status_words_are_collected_without_a_wait():
    """The words a step carries to the host beside its sampled ids: the token-id flag of the
    embedding kernel and the error words of the libraries that are loaded."""
    k = kernels()
    table = torch.randn(50, 32, device="cuda")
    out = torch.empty(3, 32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    words = torch.full((k.STATUS_WORDS,), -1, dtype=torch.int32, device="cuda")
    k.embedding(table, torch.tensor([1, 2, 3], dtype=torch.int32, device="cuda"), out, flag)
    k.collect_status(flag, words)
    assert words.tolist() == [0, 0, 0] and k.status_problem(words.tolist()) is None
    k.embedding(table, torch.tensor([1, 50, 3], dtype=torch.int32, device="cuda"), out, flag)
    k.collect_status(flag, words)
    assert words.tolist() == [2, 0, 0]
    assert "batch row 1" in k.status_problem(words.tolist(), 50)
    k.collect_status(None, words)
    assert words.tolist() == [0, 0, 0]
