"""Plain tensor-code versions of the engine's kernels, one per kernel and with the
kernel's signature.  They serve two purposes in the tests: the reference each CUDA
kernel is compared with on the GPU, and (patched over ``kernels``) a way to run
the engine's host-side logic on a machine without a GPU.  They are not part of
the engine and the engine never imports them.

All arithmetic is float32 (float64 where the input is float64); results are
rounded once to the output's dtype.
"""

from __future__ import annotations

import torch


def embedding(table, ids, residual, error_flag):
    residual.copy_(table[ids.long()].to(torch.float32))


def add_rmsnorm(x, residual, weight, eps, out, rows=None):
    total = residual if x is None else residual + x.to(torch.float32)
    if rows is None:
        if x is not None:
            residual.copy_(total)
    else:
        total = total[rows.long()]
    variance = total.pow(2).mean(dim=-1, keepdim=True)
    out.copy_((total * torch.rsqrt(variance + eps) * weight).to(out.dtype))


def silu_mul(gate_up, out):
    inter = out.shape[1]
    gate, up = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    out.copy_((gate * torch.sigmoid(gate) * up).to(out.dtype))


def _root(scale, width):
    """The factor a product applies whose rows are half-normalised: rsqrt(sum of the pieces / width + eps)."""
    squares, eps = scale
    return torch.rsqrt(squares.float().sum(dim=-1, keepdim=True) / width + eps)


def gemm(x, w, out, scale=None, fold=None):
    product = x.float() @ w.float().T
    if scale is not None:
        product = product * _root(scale, x.shape[1])
    if fold is None:
        out.copy_(product.to(out.dtype))
        return
    # residual += rounded product; out = residual * weight; sums of squares over blocks of eight columns
    residual, weight, squares_out = fold
    residual += product.to(out.dtype).float()
    out.copy_((residual * weight).to(out.dtype))
    squares_out.copy_(residual.pow(2).reshape(residual.shape[0], -1, 8).sum(dim=-1))


def gated_silu_gemm(x, w_gate_up, out, scale=None):
    inter = out.shape[1]
    gate_up = x.float() @ w_gate_up.float().T
    if scale is not None:
        gate_up = gate_up * _root(scale, x.shape[1])
    gate, up = gate_up[:, :inter], gate_up[:, inter:]
    out.copy_((gate * torch.sigmoid(gate) * up).to(out.dtype))


def head_norm_rope_cache(qkv, positions, slots, q_weight, k_weight, inv_freq, rotary_dim, eps, q_out,
                         k_pages, v_pages, num_q_heads, num_kv_heads, head_dim, page_size):
    tokens = qkv.shape[0]
    nq, nkv, d = num_q_heads, num_kv_heads, head_dim
    wide = qkv.float()
    q = wide[:, :nq * d].reshape(tokens, nq, d)
    k = wide[:, nq * d:(nq + nkv) * d].reshape(tokens, nkv, d)
    v = wide[:, (nq + nkv) * d:].reshape(tokens, nkv, d)

    def norm(t, weight):
        if weight is None:
            return t
        return t * torch.rsqrt(t.pow(2).mean(dim=-1, keepdim=True) + eps) * weight

    def rotate(t):
        if not rotary_dim:
            return t
        half = rotary_dim // 2
        angles = positions.float()[:, None] * inv_freq[None, :]
        c, s = angles.cos()[:, None, :], angles.sin()[:, None, :]
        x1, x2, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
        return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), dim=-1)

    q, k = rotate(norm(q, q_weight)), rotate(norm(k, k_weight))
    q_out.copy_(q.reshape(tokens, nq * d).to(q_out.dtype))
    if k_pages is None:
        return
    keep = slots >= 0
    page = (slots[keep] // page_size).long()
    offset = (slots[keep] % page_size).long()
    k_pages[page, :, offset, :] = k[keep].to(k_pages.dtype)
    v_pages[page, :, offset, :] = v[keep].to(v_pages.dtype)


def paged_attention(q, k_pages, v_pages, out, query_start, seq_lens, block_table, num_q_heads,
                    num_kv_heads, head_dim, page_size, scale, window, max_query_len, max_seq_len, num_decode=0,
                    decode_done=False):
    assert not decode_done, "the plain version runs every request itself"
    nq, nkv, d = num_q_heads, num_kv_heads, head_dim
    group = nq // nkv
    starts = query_start.tolist()
    for request, seq_len in enumerate(seq_lens.tolist()):
        begin, end = starts[request], starts[request + 1]
        q_len = end - begin
        if q_len == 0:
            continue
        past = seq_len - q_len
        key_pos = torch.arange(seq_len, device=q.device)
        pages = block_table[request, (key_pos // page_size).long()].long()
        live = pages >= 0
        safe = pages.clamp(min=0)
        keys = k_pages[safe, :, (key_pos % page_size).long(), :].float()       # [S, nkv, d]
        values = v_pages[safe, :, (key_pos % page_size).long(), :].float()
        keys = keys.repeat_interleave(group, dim=1)
        values = values.repeat_interleave(group, dim=1)
        queries = q[begin:end].float().reshape(q_len, nq, d)
        scores = torch.einsum("ihd,jhd->hij", queries, keys) * scale
        q_pos = past + torch.arange(q_len, device=q.device)[:, None]
        visible = (key_pos[None, :] <= q_pos) & live[None, :]
        if window:
            visible = visible & (key_pos[None, :] > q_pos - window)
        scores = scores.masked_fill(~visible[None], float("-inf"))
        probs = torch.softmax(scores, dim=-1).nan_to_num(0.0)
        result = torch.einsum("hij,jhd->ihd", probs, values).reshape(q_len, nq * d)
        out[begin:end] = result.to(out.dtype)


def fused_decode_attention(*args, **kwargs):
    """There is no plain version of the kernel that does both: the caller runs the two steps."""
    return False


ALL = ("embedding", "add_rmsnorm", "silu_mul", "gemm", "gated_silu_gemm", "head_norm_rope_cache", "paged_attention",
       "fused_decode_attention")


def patch(monkeypatch) -> None:
    """Put the plain versions in place of the CUDA kernels (CPU-only tests)."""
    import vllm_from_scratch_b200.kernels as kernels
    for name in ALL:
        monkeypatch.setattr(kernels, name, globals()[name])


def sample(logits, temperature, top_k, top_p, min_p, seeds, draw_index, tokens, greedy_eps, kinds=3):
    """Greedy rows only: enough to drive the engine on the CPU."""
    assert kinds & 1, "greedy rows are rows without a filter"
    if bool((temperature >= greedy_eps).any()):
        raise NotImplementedError("the plain stand-in samples greedily only")
    tokens.copy_(logits.argmax(dim=-1).to(tokens.dtype))


def mask_tokens(logits, rows, tokens):
    logits[rows.long(), tokens.long()] = float("-inf")


ALL = ALL + ("sample", "mask_tokens")
