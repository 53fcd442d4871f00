"""From a step's logits to one token per request.

Order of operations as in the reference's sampler (minivllm/sample/sampler.py:
73-120, 243-288): float32 logits -> penalties -> stop tokens masked while a
request is below ``min_tokens`` -> greedy rows take the argmax (never divided by
the temperature), the other rows are scaled by their temperature, filtered by
min-p, top-k and top-p and drawn.  The draw is keyed by the request's seed and by
how many tokens it has generated, so a request's tokens do not depend on what
else is in the batch or on the order of calls (the scheme of minivllm/worker/gpu/
sample/gumbel.py:94-131).
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .. import kernels
from .params import GREEDY_EPS, SamplingParams


class _Seen:
    """The distinct tokens that a request has seen, sorted, and how often each was generated:
    what the penalties need, kept up from step to step instead of being counted again."""

    __slots__ = ("tokens", "counts", "outputs")

    def __init__(self, prompt: Sequence[int]) -> None:
        self.tokens = np.unique(np.asarray(prompt, dtype=np.int32))
        self.counts = np.zeros(self.tokens.shape[0], dtype=np.int32)
        self.outputs = 0                        # output tokens counted so far

    def extend(self, output: Sequence[int]) -> None:
        fresh = output[self.outputs:]
        self.outputs = len(output)
        if len(fresh) > 32:                     # a whole history at once
            values, counts = np.unique(np.asarray(fresh, dtype=np.int32), return_counts=True)
            tokens = np.union1d(self.tokens, values)
            merged = np.zeros(tokens.shape[0], dtype=np.int32)
            merged[np.searchsorted(tokens, self.tokens)] = self.counts
            merged[np.searchsorted(tokens, values)] += counts.astype(np.int32)
            self.tokens, self.counts = tokens, merged
            return
        for token in fresh:
            at = int(np.searchsorted(self.tokens, token))
            if at < self.tokens.shape[0] and self.tokens[at] == token:
                self.counts[at] += 1
            else:
                self.tokens = np.insert(self.tokens, at, token)
                self.counts = np.insert(self.counts, at, 1)


class Sampler:
    def __init__(self, vocab_size: int, device: torch.device | str) -> None:
        self.vocab_size = vocab_size
        self.device = torch.device(device)
        self._seen: dict[str, _Seen] = {}       # by the key a caller names a request with

    def forget(self, key: str) -> None:
        """The request of this key is over (its key may name another request later)."""
        self._seen.pop(key, None)

    def _to_device(self, array: np.ndarray) -> torch.Tensor:
        return torch.from_numpy(array).to(self.device, non_blocking=True)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               prompts: Sequence[Sequence[int]], outputs: Sequence[Sequence[int]],
               keys: Sequence[str] | None = None) -> list[int]:
        """``logits`` is ``[rows, vocab]`` float32 on the device (changed in place by
        penalties and masks); the other arguments have one entry per row.  ``keys``: a name
        per request, the same from step to step; what a request has seen is then kept up under
        its name instead of being counted anew every step (``forget`` it when the request ends)."""
        tokens = self.sample_device(logits, params, seeds, prompts, outputs, keys=keys)
        return tokens.tolist()

    def sample_device(self, logits, params, seeds, prompts, outputs, ahead: int = 0,
                      extra: int = 0, keys: Sequence[str] | None = None,
                      last: tuple[torch.Tensor, Sequence[int]] | None = None) -> torch.Tensor:
        """The sampled ids as an int32 tensor on the device, without waiting for them.
        ``ahead``: how many output tokens of every row (none or one) are still on their way to
        the host and so missing from ``outputs``; they count for the draw index and for
        ``min_tokens``, and rows with penalties need them: ``last`` is then the device tensor that
        holds them and, per row, the place of the row's token in it.  ``extra``: that
        many more int32 words are allocated behind the ids for the caller to fill (the
        step's status words, so that one copy brings both to the host)."""
        rows = logits.shape[0]
        if rows != len(params):
            raise ValueError(f"{rows} rows of logits for {len(params)} requests")
        width = self.logprob_width(params)
        raw = logits
        if width and (any(p.has_penalties for p in params)
                      or any(len(o) + ahead < p.min_tokens for p, o in zip(params, outputs))):
            raw = logits.clone()                # log-probabilities are those of the logits as the model gave them
        if ahead not in (0, 1):
            raise ValueError("at most one token of a row may be on its way")
        if ahead and last is None and any(p.has_penalties for p in params):
            raise ValueError("penalties need every earlier token: name the tensor that holds the one on its way")
        self._penalties(logits, params, prompts, outputs, keys, last if ahead else None)
        self._min_tokens(logits, params, outputs, ahead)
        # The six per-row arrays travel as one buffer: 64-bit words first, so that every view is aligned.
        words = np.empty(rows * 8, dtype=np.int32)
        wide = words[:rows * 4].view(np.int64)
        wide[:rows] = [s & 0x7FFFFFFFFFFFFFFF for s in seeds]
        wide[rows:] = [len(o) + ahead for o in outputs]
        temperature, top_p, min_p = (words[rows * (4 + i):rows * (5 + i)].view(np.float32) for i in (0, 2, 3))
        top_k = words[rows * 5:rows * 6]
        temperature[:] = [p.temperature for p in params]
        top_k[:] = [p.top_k if p.top_k > 0 else 0 for p in params]
        top_p[:] = [p.top_p for p in params]
        min_p[:] = [p.min_p for p in params]
        tokens = torch.empty(rows + extra + self.logprob_words(rows, width), dtype=torch.int32, device=logits.device)
        filtered = (temperature >= GREEDY_EPS) & ((top_k > 0) | ~(top_p >= 1.0) | ~(min_p <= 0.0))
        kinds = (1 if not filtered.all() else 0) | (2 if filtered.any() else 0)
        on_device = self._to_device(words)
        wide_d = on_device[:rows * 4].view(torch.int64)
        part = lambda i: on_device[rows * (4 + i):rows * (5 + i)]
        kernels.sample(logits, part(0).view(torch.float32), part(1), part(2).view(torch.float32), part(3).view(torch.float32),
                       wide_d[:rows], wide_d[rows:], tokens[:rows], GREEDY_EPS, kinds)
        if width:
            wanted = self._to_device(np.array([-1 if p.logprobs is None else p.logprobs for p in params], dtype=np.int32))
            ids, values, place = self.logprob_views(tokens[rows + extra:], rows, width)
            kernels.logprobs(raw, tokens[:rows], wanted, ids, values.view(torch.float32), place)
        return tokens

    # Log-probabilities ride behind the ids (and the caller's extra words) in the same tensor, so that
    # one copy brings everything to the host: [rows x width] token ids, [rows x width] float32
    # values as their bits, [rows] places.
    @staticmethod
    def logprob_width(params: Sequence[SamplingParams]) -> int:
        """Columns per row: the sampled token and the longest list; 0 if no row wants any."""
        wanted = [p.logprobs for p in params if p.logprobs is not None]
        return 1 + max(wanted) if wanted else 0

    @staticmethod
    def logprob_words(rows: int, width: int) -> int:
        return rows * (2 * width + 1) if width else 0

    @staticmethod
    def logprob_views(words, rows: int, width: int):
        """(ids, values as int32 bits, places) of ``words``, the tail of a sampled tensor or of
        its host copy (a tensor or a numpy array)."""
        ids = words[:rows * width].reshape(rows, width)
        values = words[rows * width:2 * rows * width].reshape(rows, width)
        return ids, values, words[2 * rows * width:2 * rows * width + rows]

    def _penalties(self, logits, params, prompts, outputs, keys=None, last=None) -> None:
        if not any(p.has_penalties for p in params):
            return
        offsets, seen, counts = [0], [], []
        for row, (p, prompt, output) in enumerate(zip(params, prompts, outputs)):
            if p.has_penalties:
                history = self._seen.get(keys[row]) if keys is not None else None
                if history is None or history.outputs > len(output):
                    history = _Seen(prompt)
                    if keys is not None:
                        self._seen[keys[row]] = history
                history.extend(output)
                seen.append(history.tokens)
                counts.append(history.counts)
            offsets.append(offsets[-1] + (seen[-1].shape[0] if p.has_penalties else 0))
        if offsets[-1] == 0 and last is None:
            return
        seen = np.concatenate(seen) if seen else np.zeros(0, dtype=np.int32)
        counts = np.concatenate(counts) if counts else np.zeros(0, dtype=np.int32)
        last_tokens = last_rows = None
        if last is not None:
            last_tokens = last[0]
            last_rows = self._to_device(np.asarray(last[1], dtype=np.int32))
        kernels.apply_penalties(
            logits, self._to_device(np.array(offsets, dtype=np.int32)),
            self._to_device(seen.astype(np.int32, copy=False)), self._to_device(counts.astype(np.int32, copy=False)),
            self._to_device(np.array([p.repetition_penalty for p in params], dtype=np.float32)),
            self._to_device(np.array([p.frequency_penalty for p in params], dtype=np.float32)),
            self._to_device(np.array([p.presence_penalty for p in params], dtype=np.float32)),
            last_tokens, last_rows)

    def _min_tokens(self, logits, params, outputs, ahead: int = 0) -> None:
        rows, tokens = [], []
        for row, (p, output) in enumerate(zip(params, outputs)):
            if len(output) + ahead < p.min_tokens:
                for token in sorted(p.all_stop_token_ids):
                    rows.append(row)
                    tokens.append(token)
        if rows:
            kernels.mask_tokens(logits, self._to_device(np.array(rows, dtype=np.int32)),
                                self._to_device(np.array(tokens, dtype=np.int32)))
