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

from .. import kernels
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
        self._validated_shapes: set[tuple[int, int, int]] = set()

    # ------------------------------------------------------------------ packing
    def pack_host(self, entries: list[StepEntry], pad_requests: int | None = None,
                  table_width: int | None = None, pad_tokens: int = 1, pad_wanted: int = 0
                  ) -> tuple[torch.Tensor, dict]:
        """Describe the batch in one pinned int32 buffer.  For shapes fixed in advance:
        ``pad_requests`` adds requests of ``pad_tokens`` tokens (one or none) that read and
        write nothing, ``pad_wanted`` repeats the first token's row up to that many wanted
        rows, ``table_width`` fixes the width of the block tables.

        Requests that bring one token are put ahead of those that bring a portion of a
        prompt (the order among each kind stays), so that a mixer may give the first
        ``num_decode`` rows to its kernel for single tokens and the rest to the one for
        portions; the wanted rows keep the order of ``entries`` and of their ``want``."""
        page_size = self.page_size
        real = len(entries)
        order = ([i for i, entry in enumerate(entries) if len(entry.tokens) == 1]
                 + [i for i, entry in enumerate(entries) if len(entry.tokens) != 1])
        num_decode = sum(1 for entry in entries if len(entry.tokens) == 1)
        row_of = {index: row for row, index in enumerate(order)}
        given, entries = entries, [entries[i] for i in order]
        num_requests = max(real, pad_requests or 0)
        padding = num_requests - real
        lengths = [len(entry.tokens) for entry in entries] + [pad_tokens] * padding
        num_tokens = sum(lengths)
        query_start = np.zeros(num_requests + 1, dtype=np.int32)
        np.cumsum(lengths, out=query_start[1:])
        seq_lens = np.array([entry.start + len(entry.tokens) for entry in entries] + [0] * padding,
                            dtype=np.int32)
        # Padded requests use the spare state slot past the last real one.
        slots = np.array([self.manager.slot(entry.request_id) for entry in entries]
                         + [self.storage.max_requests] * padding, dtype=np.int32)
        zeros = np.zeros(padding * pad_tokens, dtype=np.int32)
        token_ids = np.concatenate([np.asarray(entry.tokens, dtype=np.int32) for entry in entries] + [zeros])
        positions = np.concatenate([np.arange(entry.start, entry.start + len(entry.tokens), dtype=np.int32)
                                    for entry in entries] + [zeros])
        token_request = np.repeat(np.arange(num_requests, dtype=np.int32), lengths)
        want_rows: list[int] = []
        for index, entry in enumerate(given):
            row = row_of[index]
            for place in entry.want:
                if not 0 <= place < lengths[row]:
                    raise ValueError(f"request {entry.request_id!r}: wanted place {place} is outside "
                                     f"its {lengths[row]} tokens of this step")
                want_rows.append(int(query_start[row]) + place)
        want_rows += [0] * max(0, pad_wanted - len(want_rows))
        want = np.asarray(want_rows, dtype=np.int32)

        pieces = [token_ids, positions, token_request, query_start, seq_lens, slots, want]
        widths = []
        real_tokens = int(query_start[real])
        for group in range(len(self.storage.groups)):
            tables = [self.manager.block_table(entry.request_id, group) for entry in entries]
            needed = [-(-int(total) // page_size) for total in seq_lens[:real]]
            for entry, table, pages in zip(entries, tables, needed):
                if len(table) < pages:
                    raise ValueError(
                        f"request {entry.request_id!r} holds {len(table)} pages in group {group} but "
                        f"this step reaches position {pages * page_size - 1}: allocate before the step")
            width = max(needed) if table_width is None else table_width
            if width < max(needed):
                raise ValueError(f"block table width {width} is too small for {max(needed)} pages")
            block_table = np.full((num_requests, width), RELEASED, dtype=np.int32)
            for row, (table, pages) in enumerate(zip(tables, needed)):
                block_table[row, :pages] = table[:pages]
            slot_mapping = np.full(num_tokens, -1, dtype=np.int32)
            page_of_token = block_table[token_request[:real_tokens], positions[:real_tokens] // page_size]
            if real_tokens and int(page_of_token.min()) < 0:
                bad = int(np.argmin(page_of_token))
                raise ValueError(f"token row {bad} would be written to a page that was given back")
            slot_mapping[:real_tokens] = page_of_token * page_size + positions[:real_tokens] % page_size
            pieces += [slot_mapping, block_table.reshape(-1)]
            widths.append(width)

        sizes = [piece.size for piece in pieces]
        host = torch.empty(sum(sizes), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        np.concatenate(pieces, out=host.numpy())
        meta = {
            "sizes": sizes, "widths": widths, "num_tokens": num_tokens, "num_requests": num_requests,
            "num_wanted": len(want_rows), "max_query_len": max(lengths),
            "max_seq_len": int(seq_lens.max()), "query_start": query_start.tolist(),
            "seq_lens": seq_lens.tolist(), "slots": slots.tolist(),
            # single-token requests ahead of portions; 0 when the step has only one kind
            "num_decode": num_decode if 0 < num_decode < real else 0,
        }
        return host, meta

    def context_from(self, packed: torch.Tensor, meta: dict
                     ) -> tuple[StepContext, torch.Tensor, torch.Tensor]:
        """Views into the device copy of a packed buffer: context, token ids, wanted rows."""
        parts = list(torch.split(packed, meta["sizes"]))
        ids_d, pos_d, req_d, start_d, lens_d, slots_d, want_d = parts[:7]
        ctx = StepContext(
            num_tokens=meta["num_tokens"], num_requests=meta["num_requests"], positions=pos_d,
            query_start=start_d, seq_lens=lens_d, state_slots=slots_d, token_request=req_d,
            max_query_len=meta["max_query_len"], max_seq_len=meta["max_seq_len"],
            host_query_start=meta["query_start"], host_seq_lens=meta["seq_lens"],
            host_state_slots=meta["slots"], num_decode=meta.get("num_decode", 0))
        for group, width in enumerate(meta["widths"]):
            slot_d, table_d = parts[7 + 2 * group], parts[8 + 2 * group]
            ctx.groups[group] = GroupContext(self.page_size, table_d.view(meta["num_requests"], width),
                                             slot_d, width)
        return ctx, ids_d, want_d

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
        host, meta = self.pack_host(entries)
        ctx, token_ids, want_rows = self.context_from(host.to(self.device, non_blocking=True), meta)
        self.last_context = ctx
        # Operand checks run the first time a batch shape is seen; later steps of that
        # shape go through the same code with the same sizes.
        shape = (meta["num_tokens"], meta["num_requests"], meta["num_wanted"])
        first_time = shape not in self._validated_shapes
        with kernels.validation(first_time):
            x, residual = self.model.forward(token_ids, ctx, self.storage.views)
            logits = None if meta["num_wanted"] == 0 else self.model.logits(x, residual, want_rows)
        self._validated_shapes.add(shape)
        return logits
