"""Tensor-core attention kernels of the bfloat16 run mode.

``paged_attention_bf16`` returns True when it ran a kernel and False when the
shape is one these kernels refuse (head sizes other than 64, 128, 256, or more
than 16 query heads per key/value head); the caller then uses the
float32-arithmetic kernel, which takes every shape.
"""

from __future__ import annotations

import ctypes

import torch

from ..csrc.build import load_library

TC_MIN_QUERY_LEN = 64      # shorter portions go to the 64-row mma.sync kernel
# Which kernel serves a shape that more than one takes.  Each default is the faster one; a test
# sets a switch to False to drive the kernel behind it through the same call.
USE_TMA_DECODE = True      # decode attention fed by tensor copies (pages of 8, 16, 32, ... keys)
USE_FUSED_DECODE = True    # head norms, rotation and the store of the new key and value in the decode kernel
USE_TC_ATTENTION = True    # tcgen05 / tensor-memory kernel for portions of TC_MIN_QUERY_LEN tokens and more
USE_TC_KEY_SPLIT = True    # ... with the keys of a row block divided over several blocks where few blocks would run
_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


_sm_count: dict[int, int] = {}


def sm_count() -> int:
    """Number of SMs of the current device, asked of the device once."""
    device = torch.cuda.current_device()
    count = _sm_count.get(device)
    if count is None:
        count = int(load_library("attention_bf16").b200_sm_count())
        if count <= 0:
            raise RuntimeError("could not read the number of SMs of the current device")
        _sm_count[device] = count
    return count


def tensor_map_cache_self_check(count: int = 5000) -> int:
    """Host-only check of the tensor-map cache: more maps than it holds are encoded over one
    buffer (nothing is launched) and the first ones compared with fresh copies.  0 = sound."""
    buffer = torch.empty(count * 16 + 64 * 64 * 2 + 256, dtype=torch.uint8, device="cuda")
    lib = load_library("attention_bf16")
    return int(lib.b200_tensor_map_cache_self_check(_P(buffer.data_ptr()), ctypes.c_longlong(buffer.numel()),
                                                    _I(count)))


def decode_splits(num_requests: int, num_kv_heads: int, max_seq_len: int) -> int:
    """Over how many blocks the keys of one (request, key/value head) are split.
    Three blocks fit on an SM at a time.  Few pairs: the split is chosen so that the blocks fill
    whole rounds of the GPU (a last round with few blocks would leave it idle), with at least 512
    keys per block at the planned length (256 for one or two requests).  Pairs that fill half of
    the GPU by themselves stream at the memory's rate without any split: there the split only has
    to keep the last round from being a few lone blocks, and every split more costs its set-up and
    the merge, which a count of rounds does not see."""
    pairs = max(1, num_requests * num_kv_heads)
    slots = 3 * sm_count()
    most = max(1, min(16, max_seq_len // 512))
    if 2 * pairs >= slots:
        # Time in steps of a lone block's tile of 64 keys: a round of blocks that fills the GPU is
        # bound by the memory and takes three such steps a tile, a round of few blocks one; a block
        # costs seven steps beside its tiles, the merge four (measured at 32, 64 and 128 requests of
        # 2100 keys: no split 51 us against 56 with five at 32; three to five 95 to 98 against 113
        # without at 64).
        tiles_whole = -(-max_seq_len // 64)
        best, best_cost = 1, None
        for splits in range(1, most + 1):
            tiles = -(-tiles_whole // splits)
            blocks = pairs * splits
            full, last = divmod(blocks, slots)
            cost = full * tiles * 3.0 + (tiles * max(3.0 * last / slots, 1.0) if last else 0.0) + 7.0
            cost += 4.0 if splits > 1 else 0.0
            if best_cost is None or cost < best_cost:
                best, best_cost = splits, cost
        return best
    best, best_fill = 1, 0.0
    # One or two requests cannot fill half of the GPU with 512 keys a block: they get 256
    # (a step at batch 1 takes 1.21 against 1.29 ms, at batch 2 1.27 against 1.31; from batch 4
    # on the finer split loses to its own merge and set-up).
    min_keys = 256 if pairs * max(1, max_seq_len // 512) < slots // 2 else 512
    for splits in range(1, max(1, min(16, max_seq_len // min_keys)) + 1):
        blocks = pairs * splits
        fill = blocks / (-(-blocks // slots) * slots) - 0.002 * splits     # a split more costs a little
        if fill > best_fill:
            best, best_fill = splits, fill
    return best


def _decode(lib, q, k_pages, v_pages, out, seq_lens, block_table, num_q_heads, num_kv_heads, head_dim,
            page_size, scale, window, max_seq_len) -> int:
    """One token per request (row r of q belongs to request r)."""
    from . import _stream
    requests = seq_lens.shape[0]
    splits = decode_splits(requests, num_kv_heads, max_seq_len)
    partial_o = partial_ml = None
    if splits > 1:
        partial_o = torch.empty((requests * num_q_heads * splits, head_dim), dtype=torch.float32, device=q.device)
        partial_ml = torch.empty((requests * num_q_heads * splits, 2), dtype=torch.float32, device=q.device)
    common = (_P(q.data_ptr()), _P(k_pages.data_ptr()), _P(v_pages.data_ptr()), _P(out.data_ptr()),
              _P(partial_o.data_ptr() if splits > 1 else 0), _P(partial_ml.data_ptr() if splits > 1 else 0),
              _P(seq_lens.data_ptr()), _P(block_table.data_ptr()), _I(requests), _I(block_table.shape[1]),
              _I(num_q_heads), _I(num_kv_heads), _I(head_dim), _I(page_size))
    tail = (_F(scale), _I(window or 0), _I(splits), _stream())
    if (USE_TMA_DECODE
            and lib.b200_decode_attention_tma_supports(num_q_heads, num_kv_heads, head_dim, page_size)):
        # keys and values by tensor copies straight from the pages
        return lib.b200_decode_attention_tma_bf16(*common, _I(k_pages.shape[0]), *tail)
    return lib.b200_decode_attention_bf16(*common, *tail)


def _portions(lib, q, k_pages, v_pages, out, query_start, seq_lens, block_table, num_q_heads, num_kv_heads,
              head_dim, page_size, scale, window, max_query_len, max_seq_len, token_offset) -> int:
    """Portions of prompts (any number of tokens per request).  ``q`` and ``out`` are the whole
    batch's, ``query_start`` holds rows of them; the requests given begin at ``token_offset``."""
    from . import _stream
    requests = seq_lens.shape[0]
    tokens = q.shape[0]
    if (max_query_len >= TC_MIN_QUERY_LEN and USE_TC_ATTENTION
            and lib.b200_prefill_attention_tc_supports(num_q_heads, num_kv_heads, head_dim, page_size)):
        # long portions of prompts: the tcgen05 / tensor-memory kernel; few row blocks over many
        # keys are divided over several blocks each, with partial results that a second kernel merges
        splits = 1
        if USE_TC_KEY_SPLIT:
            splits = lib.b200_prefill_attention_tc_splits(_I(tokens - token_offset), _I(requests), _I(num_q_heads),
                                                          _I(max_seq_len))
        partial_o = partial_ml = None
        if splits > 1:
            partial_o = torch.empty((tokens * num_q_heads * splits, head_dim), dtype=torch.float32, device=q.device)
            partial_ml = torch.empty((tokens * num_q_heads * splits, 2), dtype=torch.float32, device=q.device)
        return lib.b200_prefill_attention_tc_bf16(
            _P(q.data_ptr()), _P(k_pages.data_ptr()), _P(v_pages.data_ptr()), _P(out.data_ptr()),
            _P(query_start.data_ptr()), _P(seq_lens.data_ptr()), _P(block_table.data_ptr()), _I(requests),
            _I(tokens), _I(block_table.shape[1]), _I(num_q_heads), _I(num_kv_heads), _I(head_dim),
            _I(page_size), _I(k_pages.shape[0]), _F(scale), _I(window or 0), _I(token_offset), _I(splits),
            _P(partial_o.data_ptr() if splits > 1 else 0), _P(partial_ml.data_ptr() if splits > 1 else 0), _stream())
    return lib.b200_prefill_attention_bf16(
        _P(q.data_ptr()), _P(k_pages.data_ptr()), _P(v_pages.data_ptr()), _P(out.data_ptr()),
        _P(query_start.data_ptr()), _P(seq_lens.data_ptr()), _P(block_table.data_ptr()), _I(requests),
        _I(tokens), _I(block_table.shape[1]), _I(num_q_heads), _I(num_kv_heads), _I(head_dim),
        _I(page_size), _F(scale), _I(window or 0), _I(token_offset), _stream())


def paged_attention_bf16(q, k_pages, v_pages, out, query_start, seq_lens, block_table, num_q_heads,
                         num_kv_heads, head_dim, page_size, scale, window, max_query_len,
                         max_seq_len, num_decode: int = 0, decode_done: bool = False) -> bool:
    """``num_decode``: the first that many requests bring one token each and the others
    portions (0: one kind only); the two kinds then go to their own kernels.
    ``decode_done``: the single tokens have been attended to already (by the fused kernel)."""
    lib = load_library("attention_bf16")
    if not lib.b200_attention_bf16_supports(num_q_heads, num_kv_heads, head_dim):
        return False
    from . import KernelError, count_launch
    requests = seq_lens.shape[0]
    tokens = q.shape[0]
    shape = (num_q_heads, num_kv_heads, head_dim, page_size, scale, window)
    if max_query_len == 1 and tokens == requests:
        status = _decode(lib, q, k_pages, v_pages, out, seq_lens, block_table, *shape, max_seq_len)
    elif 0 < num_decode < requests:
        n = num_decode
        status = 0
        if not decode_done:
            status = _decode(lib, q[:n], k_pages, v_pages, out[:n], seq_lens[:n], block_table[:n], *shape,
                             max_seq_len)
            count_launch()
        if status == 0:
            status = _portions(lib, q, k_pages, v_pages, out, query_start[n:], seq_lens[n:], block_table[n:],
                               *shape, max_query_len, max_seq_len, n)
    elif decode_done:
        raise KernelError("paged_attention: decode_done without a split of the batch")
    else:
        status = _portions(lib, q, k_pages, v_pages, out, query_start, seq_lens, block_table, *shape,
                           max_query_len, max_seq_len, 0)
    if status != 0:
        raise KernelError(lib.b200_last_error().decode())
    count_launch()
    return True


def fused_decode_attention_bf16(qkv, positions, slots, q_weight, k_weight, inv_freq, rotary_dim, eps, k_pages,
                                v_pages, out, seq_lens, block_table, num_q_heads, num_kv_heads, head_dim,
                                page_size, scale, window, max_seq_len) -> bool:
    """A decode step's attention straight from the packed projection: head norms, rotation,
    the store of the new key and value, and the attention over the pages in one kernel (and
    the merge of the splits).  False if the shape is not one that kernel takes (or
    ``USE_FUSED_DECODE`` is off): the caller then runs the two kernels one after the other."""
    if not (USE_FUSED_DECODE and USE_TMA_DECODE):
        return False
    lib = load_library("attention_bf16")
    if not lib.b200_decode_attention_fused_supports(num_q_heads, num_kv_heads, head_dim, rotary_dim, page_size):
        return False
    from . import KernelError, _stream, count_launch
    requests = seq_lens.shape[0]
    splits = decode_splits(requests, num_kv_heads, max_seq_len)
    partial_o = partial_ml = None
    if splits > 1:
        partial_o = torch.empty((requests * num_q_heads * splits, head_dim), dtype=torch.float32, device=qkv.device)
        partial_ml = torch.empty((requests * num_q_heads * splits, 2), dtype=torch.float32, device=qkv.device)
    status = lib.b200_decode_attention_fused_bf16(
        _P(qkv.data_ptr()), _P(positions.data_ptr()), _P(slots.data_ptr()),
        _P(q_weight.data_ptr() if q_weight is not None else 0), _P(k_weight.data_ptr() if k_weight is not None else 0),
        _P(inv_freq.data_ptr()), _F(eps), _P(k_pages.data_ptr()), _P(v_pages.data_ptr()), _P(out.data_ptr()),
        _P(partial_o.data_ptr() if splits > 1 else 0), _P(partial_ml.data_ptr() if splits > 1 else 0),
        _P(seq_lens.data_ptr()), _P(block_table.data_ptr()), _I(requests), _I(block_table.shape[1]),
        _I(num_q_heads), _I(num_kv_heads), _I(head_dim), _I(page_size), _I(k_pages.shape[0]), _F(scale),
        _I(window or 0), _I(splits), _stream())
    if status != 0:
        raise KernelError(lib.b200_last_error().decode())
    count_launch()
    return True


def attention_error_code() -> int:
    """0, or the code left by an attention kernel whose bounded wait ran out (synchronises)."""
    return int(load_library("attention_bf16").b200_attention_error())
