"""The step function: one batch of (request, its next tokens) through the model.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.
Only the tokens given are run; everything earlier comes from the cache.  The
result is the float32 logits at the wanted places and nothing else.

The reference's counterpart is ``GPUModelRunner.execute_model`` (minivllm/worker/
gpu_model_runner.py:1582-1678) with its input packing ``_prepare_inputs``
(:865-941): positions = computed + offset, ``query_start_loc``, ``seq_lens``,
``slot = block_table[pos // bs] * bs + pos % bs`` (minivllm/worker/
block_table.py:93-116), logits only at selected rows (:1647-1653).  Here the
packing is one int32 buffer filled on the host and copied to the device in one
transfer; the pages are booked by the caller (scheduler or replay program)
through the cache manager before the step.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import RELEASED, CacheManager, CacheStorage
from ..parts.base import GroupContext, StepContext
from ..parts.model import DecoderModel


@dataclass
class StepEntry:
    """One request's share of a step: its next ``tokens``, the first of which sits
    at position ``start`` of the request, and the places among these tokens
    (``want``, indices into ``tokens``) whose logits are asked for."""

    request_id: str
    tokens: list[int]
    start: int
    want: list[int] = field(default_factory=list)


class StepFunction:
    def __init__(self, model: DecoderModel, storage: CacheStorage, manager: CacheManager) -> None:
        self.model, self.storage, self.manager = model, storage, manager
        self.device = model.device
        self.page_size = storage.page_size
        self.last_context: StepContext | None = None     # kept for the packed-inputs trace

    # ------------------------------------------------------------------ packing
    def pack(self, entries: list[StepEntry]) -> tuple[StepContext, torch.Tensor, torch.Tensor, int]:
        """Build the device-side description of the batch.  Returns the context,
        the token ids, the wanted rows and their number."""
        page_size = self.page_size
        num_requests = len(entries)
        lengths = [len(entry.tokens) for entry in entries]
        num_tokens = sum(lengths)
        query_start = np.zeros(num_requests + 1, dtype=np.int32)
        np.cumsum(lengths, out=query_start[1:])
        seq_lens = np.array([entry.start + n for entry, n in zip(entries, lengths)], dtype=np.int32)
        slots = np.array([self.manager.slot(entry.request_id) for entry in entries], dtype=np.int32)
        token_ids = np.concatenate([np.asarray(entry.tokens, dtype=np.int32) for entry in entries])
        positions = np.concatenate([np.arange(entry.start, entry.start + n, dtype=np.int32)
                                    for entry, n in zip(entries, lengths)])
        token_request = np.repeat(np.arange(num_requests, dtype=np.int32), lengths)
        want_rows: list[int] = []
        for row, entry in enumerate(entries):
            for place in entry.want:
                if not 0 <= place < lengths[row]:
                    raise ValueError(f"request {entry.request_id!r}: wanted place {place} is outside "
                                     f"its {lengths[row]} tokens of this step")
                want_rows.append(int(query_start[row]) + place)
        want = np.asarray(want_rows, dtype=np.int32)

        pieces = [token_ids, positions, token_request, query_start, seq_lens, slots, want]
        group_shapes = []
        for group in range(len(self.storage.groups)):
            tables = [self.manager.block_table(entry.request_id, group) for entry in entries]
            needed = [-(-int(total) // page_size) for total in seq_lens]
            for entry, table, pages in zip(entries, tables, needed):
                if len(table) < pages:
                    raise ValueError(
                        f"request {entry.request_id!r} holds {len(table)} pages in group {group} but "
                        f"this step reaches position {pages * page_size - 1}: allocate before the step")
            width = max(needed)
            block_table = np.full((num_requests, width), RELEASED, dtype=np.int32)
            for row, (table, pages) in enumerate(zip(tables, needed)):
                block_table[row, :pages] = table[:pages]
            page_of_token = block_table[token_request, positions // page_size]
            if num_tokens and int(page_of_token.min()) < 0:
                bad = int(np.argmin(page_of_token))
                raise ValueError(f"token row {bad} would be written to a page that was given back")
            slot_mapping = (page_of_token * page_size + positions % page_size).astype(np.int32)
            pieces += [slot_mapping, block_table.reshape(-1)]
            group_shapes.append(width)

        sizes = [piece.size for piece in pieces]
        host = torch.empty(sum(sizes), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        np.concatenate(pieces, out=host.numpy())
        packed = host.to(self.device, non_blocking=True)
        parts = list(torch.split(packed, sizes))
        ids_d, pos_d, req_d, start_d, lens_d, slots_d, want_d = parts[:7]
        ctx = StepContext(
            num_tokens=num_tokens, num_requests=num_requests, positions=pos_d, query_start=start_d,
            seq_lens=lens_d, state_slots=slots_d, token_request=req_d,
            max_query_len=max(lengths), max_seq_len=int(seq_lens.max()),
            host_query_start=query_start.tolist(), host_seq_lens=seq_lens.tolist(),
            host_state_slots=slots.tolist())
        for group, width in enumerate(group_shapes):
            slot_d, table_d = parts[7 + 2 * group], parts[8 + 2 * group]
            ctx.groups[group] = GroupContext(page_size, table_d.view(num_requests, width), slot_d, width)
        return ctx, ids_d, want_d, len(want_rows)

    # ---------------------------------------------------------------------- run
    def run(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """Run the batch; returns float32 logits ``[wanted, vocab]`` in the order
        of the entries and of their ``want`` lists, or None if nothing is wanted."""
        entries = [entry for entry in entries if entry.tokens]
        if not entries:
            return None
        for entry in entries:
            if entry.start < 0:
                raise ValueError(f"request {entry.request_id!r}: negative start position")
        self.storage.zero_slots(self.manager.take_fresh_slots())
        ctx, token_ids, want_rows, num_wanted = self.pack(entries)
        self.last_context = ctx
        x, residual = self.model.forward(token_ids, ctx, self.storage.views)
        if num_wanted == 0:
            return None
        return self.model.logits(x, residual, want_rows)
