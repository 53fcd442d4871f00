"""Which few-rows products go to the engine's own kernels: the size rule alone (no GPU)."""

from vllm_from_scratch_b200.kernels.gemm_bf16 import own_limit_bytes


def takes(m, rows, k, gated=False):
    size = (2 if gated else 1) * rows * k * 2
    return size <= own_limit_bytes(m, rows, gated)


def test_the_benchmarks_widths_keep_their_kernels_up_to_sixteen_rows():
    for m in (1, 4, 8, 12, 16):
        assert takes(m, 4096, 2048) and takes(m, 2048, 2048) and takes(m, 2048, 6144)      # q/k/v, output, down
        assert takes(m, 6144, 2048, gated=True)
        assert not takes(m, 151936, 2048)                                                   # over the vocabulary


def test_larger_matrices_leave_with_more_rows():
    # widths of Qwen3-4B: q/k/v 6144 x 2560, output 2560 x 4096, down 2560 x 9728, gate and up 2 x 9728 x 2560
    assert takes(4, 6144, 2560) and not takes(8, 6144, 2560)
    assert takes(8, 2560, 4096) and takes(16, 2560, 4096)
    assert takes(4, 2560, 9728) and not takes(8, 2560, 9728)
    assert not takes(1, 9728, 2560, gated=True)
    # widths of Qwen3-8B: the output product 4096 x 4096 up to 8 rows, nothing else
    assert takes(8, 4096, 4096) and not takes(16, 4096, 4096)
    assert not takes(1, 6144, 4096) and not takes(1, 4096, 12288)
    # never more with more rows
    for rows, k in ((4096, 2048), (2560, 9728), (6144, 2560), (4096, 4096)):
        limits = [own_limit_bytes(m, rows, False) for m in range(1, 17)]
        assert limits == sorted(limits, reverse=True)
