"""The decode-attention entry point that allocates nothing.

Some users of the library cannot allocate device memory where they call it: all
of the device was given to another allocator at start-up, or they are a plug-in
that gets raw pointers and a stream and must leave the host's allocator alone.
For them ``b200_decode_attention_bf16_static`` keeps the scratch of the split-key
decode attention in a fixed array inside the library.  This test calls it through
its exported C symbol and compares it with the plain reference of the operation and
with the ordinary entry point of the same kernel (``b200_decode_attention_bf16``,
whose scratch the caller allocates, called with the same number of splits): two
calls in a row (the shared array keeps the first call's contents when the second
starts), then a size beyond the stated maximum, which must be refused.

The file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""

from __future__ import annotations

import ctypes
import itertools

import pytest
import torch

pytestmark = pytest.mark.gpu

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _case(nq, nkv, d, page, seq_lens, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    requests = len(seq_lens)
    pages_per = [-(-s // page) for s in seq_lens]
    total = sum(pages_per) + 2
    order = torch.randperm(total, device="cuda", generator=g).tolist()
    table = torch.full((requests, max(pages_per)), -1, dtype=torch.int32, device="cuda")
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
        at += n
    kp = torch.randn(total, nkv, page, d, device="cuda", generator=g).bfloat16()
    vp = torch.randn(total, nkv, page, d, device="cuda", generator=g).bfloat16()
    q = torch.randn(requests, nq * d, device="cuda", generator=g).bfloat16()
    start = torch.tensor([0] + list(itertools.accumulate([1] * requests)), dtype=torch.int32, device="cuda")
    seq = torch.tensor(seq_lens, dtype=torch.int32, device="cuda")
    return q, kp, vp, start, seq, table


def _static(lib, q, kp, vp, out, seq, table, nq, nkv, d, page, scale, window, splits):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.b200_decode_attention_bf16_static(
        _P(q.data_ptr()), _P(kp.data_ptr()), _P(vp.data_ptr()), _P(out.data_ptr()), _P(seq.data_ptr()),
        _P(table.data_ptr()), _I(seq.shape[0]), _I(table.shape[1]), _I(nq), _I(nkv), _I(d), _I(page),
        _F(scale), _I(window), _I(splits), stream)


def _allocating(lib, q, kp, vp, out, seq, table, nq, nkv, d, page, scale, window, splits):
    """The ordinary entry point of the same kernel; the caller brings the scratch."""
    rows = seq.shape[0] * nq * splits
    partial_o = torch.empty(rows, d, dtype=torch.float32, device="cuda")
    partial_ml = torch.empty(rows, 2, dtype=torch.float32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = lib.b200_decode_attention_bf16(
        _P(q.data_ptr()), _P(kp.data_ptr()), _P(vp.data_ptr()), _P(out.data_ptr()), _P(partial_o.data_ptr()),
        _P(partial_ml.data_ptr()), _P(seq.data_ptr()), _P(table.data_ptr()), _I(seq.shape[0]), _I(table.shape[1]),
        _I(nq), _I(nkv), _I(d), _I(page), _F(scale), _I(window), _I(splits), stream)
    torch.cuda.synchronize()            # the scratch must outlive the kernels
    return status


def test_static_scratch_entry_point_matches_the_allocating_one():
    import plain_ops
    from vllm_from_scratch_b200.csrc.build import load_library
    from vllm_from_scratch_b200.kernels import attention_bf16
    lib = load_library("decode_attention_static")
    lib.b200_decode_attention_bf16_static.restype = ctypes.c_int
    ordinary = load_library("attention_bf16")
    cases = [
        # nq, nkv, d, page, seq_lens, window, context the splits are planned for
        (16, 8, 128, 16, [900, 77, 2500], 0, 4096),
        (8, 2, 64, 8, [1300, 5], 600, 2048),
    ]
    for index, (nq, nkv, d, page, seq_lens, window, planned) in enumerate(cases):
        q, kp, vp, start, seq, table = _case(nq, nkv, d, page, seq_lens, seed=40 + index)
        scale = d ** -0.5
        plain = torch.zeros_like(q)
        plain_ops.paged_attention(q, kp, vp, plain, start, seq, table, nq, nkv, d, page, scale, window or None,
                                  1, max(seq_lens))
        splits = attention_bf16.decode_splits(len(seq_lens), nkv, planned)
        assert splits > 1, "the case must use the scratch memory"
        same_kernel = torch.zeros_like(q)
        status = _allocating(ordinary, q, kp, vp, same_kernel, seq, table, nq, nkv, d, page, scale, window, splits)
        assert status == 0, ordinary.b200_last_error().decode()
        out = torch.zeros_like(q)
        status = _static(lib, q, kp, vp, out, seq, table, nq, nkv, d, page, scale, window, splits)
        assert status == 0, lib.b200_last_error().decode()
        torch.cuda.synchronize()
        # against the plain reference: the tolerance of the attention kernels' own tests
        diff = float((out.float() - plain.float()).abs().max())
        assert diff <= 1.6e-2 * 2, f"call {index}: max |diff| to the plain reference {diff:.3e}"
        # against the same kernel with scratch from the caller, same splits: the same arithmetic
        assert torch.equal(out, same_kernel), f"call {index}: differs from the allocating entry point"
        assert float(out.float().abs().max()) > 0

    # beyond the stated maximum: refused with a message, nothing launched
    q, kp, vp, start, seq, table = _case(16, 8, 128, 16, [64] * 9, seed=50)
    out = torch.zeros_like(q)
    status = _static(lib, q, kp, vp, out, seq, table, 16, 8, 128, 16, 128 ** -0.5, 0, 64)   # 9 * 16 * 64 rows
    assert status != 0
    assert "B200_STATIC_MAX_PARTIAL_ROWS" in lib.b200_last_error().decode()
    assert float(out.float().abs().max()) == 0.0
