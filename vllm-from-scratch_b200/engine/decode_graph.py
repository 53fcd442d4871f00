"""CUDA-graph replay of decode steps.

A step in which every request brings exactly one token has a shape that depends
only on the number of requests.  For each batch size from a short list the whole
step (every kernel of the model and the output product) is captured once into a
CUDA graph over fixed input buffers; later steps of that size copy their packed
inputs into the buffers and replay the graph: one launch instead of hundreds.
Batches between two sizes are padded with requests that read and write nothing
(slot -1, length 0), the scheme of the reference's full graphs for uniform decode
batches (minivllm/worker/gpu_model_runner.py:1108-1165, 1215-1276, 1415-1477).
Block tables are captured at their full width (``max_model_len`` positions) and
kernel launch shapes are chosen for that length, so a replay is valid for any
context length.

Steps that also bring portions of prompts repeat their shapes too (a prompt cut
under a token budget fills the budget step after step): ``MixedGraphs`` keeps a
graph per (tokens, requests rounded up to a power of two, wanted rows likewise,
kind of longest portion) once a shape has come twice, and runs other shapes through
the ordinary step function.  The requests added by the rounding have no tokens, the
wanted rows added repeat row 0 and are dropped from the result.  Everything that
differs between steps of one shape (which tokens belong to which request, positions,
lengths, pages) is data in the packed buffer.
"""

from __future__ import annotations

import torch

from .runner import ModelRunner
from .step import StepEntry

CAPTURE_SIZES = (1, 2, 4, 8, 16, 32, 64, 128, 256)


class _Captured:
    def __init__(self, graph, packed, meta, logits, keep_alive) -> None:
        self.graph, self.packed, self.meta, self.logits = graph, packed, meta, logits
        # The graph holds raw addresses only: every tensor its kernels read must
        # outlive it.
        self.keep_alive = keep_alive


class DecodeGraphs:
    def __init__(self, runner: ModelRunner, max_num_seqs: int, max_model_len: int) -> None:
        self.runner = runner
        self.step_function = runner.step_function
        self.sizes = [size for size in CAPTURE_SIZES if size < max_num_seqs] + [max_num_seqs]
        self.table_width = -(-max_model_len // runner.storage.page_size)
        self.max_model_len = max_model_len
        self._graphs: dict[int, _Captured] = {}
        self._pool = None
        self.replays = 0
        self.last_h2d_bytes = 0

    def accepts(self, entries: list[StepEntry]) -> bool:
        return (0 < len(entries) <= self.sizes[-1] and all(len(e.tokens) == 1 for e in entries)
                and all(e.start + 1 <= self.max_model_len for e in entries))

    def _bucket(self, count: int) -> int:
        return next(size for size in self.sizes if size >= count)

    def _capture(self, size: int, host: torch.Tensor, meta: dict) -> _Captured:
        device = self.runner.device
        packed = torch.empty(host.numel(), dtype=torch.int32, device=device)
        packed.copy_(host, non_blocking=True)
        # Launch shapes must hold for every later replay: plan for the longest context.
        meta = {**meta, "max_seq_len": self.max_model_len}
        ctx, token_ids, _ = self.step_function.context_from(packed, meta)
        rows = torch.arange(size, dtype=torch.int32, device=device)
        model, views = self.runner.model, self.runner.storage.views

        def body() -> torch.Tensor:
            x, residual = model.forward(token_ids, ctx, views)
            return model.logits(x, residual, rows)

        # Warm-up: kernels compiled and loaded before the capture.  It runs this very batch, and
        # the replay after the capture runs it again: keys and values land in the same slots
        # both times, but state of fixed size per request would be advanced twice, so it is
        # put back as it was.
        states = self.runner.storage.states
        saved = {index: state.clone() for index, state in states.items()}
        stream = torch.cuda.Stream(device=device)
        stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(stream):
            body()
            for index, state in states.items():
                state.copy_(saved[index])
        torch.cuda.current_stream(device).wait_stream(stream)
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, pool=self._pool):
            logits = body()
        if self._pool is None:
            self._pool = graph.pool()
        return _Captured(graph, packed, meta, logits, (rows, ctx, token_ids))

    def run(self, entries: list[StepEntry],
            device_tokens: tuple[torch.Tensor, list[int]] | None = None) -> torch.Tensor | None:
        """The same result as ``StepFunction.run`` for a batch of single tokens.
        ``device_tokens = (ids, rows)``: entry i's token is ``ids[rows[i]]``, an int32
        tensor on the device (the ids an earlier step sampled, which the host may not
        have yet); the entries' own token values are then ignored."""
        size = self._bucket(len(entries))
        self.runner.storage.zero_slots(self.runner.manager.take_fresh_slots())
        # Every row's logits are computed; only the wanted ones are handed back.
        wanted = [row for row, entry in enumerate(entries) if entry.want]
        plain = [StepEntry(e.request_id, e.tokens, e.start, []) for e in entries]
        host, meta = self.step_function.pack_host(plain, pad_requests=size, table_width=self.table_width)
        captured = self._graphs.get(size)
        if captured is None:
            captured = self._graphs[size] = self._capture(size, host, meta)
        captured.packed.copy_(host, non_blocking=True)
        self.last_h2d_bytes = host.numel() * host.element_size()
        if device_tokens is not None:
            ids, rows = device_tokens
            count = len(entries)
            token_ids = captured.keep_alive[2]
            if rows == list(range(count)):
                token_ids[:count].copy_(ids[:count])
            else:
                index = torch.tensor(rows, dtype=torch.int64).to(ids.device, non_blocking=True)
                token_ids[:count].copy_(ids.index_select(0, index))
                self.last_h2d_bytes += 8 * count
        captured.graph.replay()
        self.replays += 1
        if not wanted:
            return None
        if len(wanted) == len(entries):
            return captured.logits[:len(entries)]
        return captured.logits[torch.tensor(wanted, device=captured.logits.device)]


class MixedGraphs:
    """Graph replay for steps of any composition whose shape has been seen before."""

    def __init__(self, runner: ModelRunner, max_model_len: int, max_graphs: int = 24) -> None:
        self.runner = runner
        self.step_function = runner.step_function
        self.table_width = -(-max_model_len // runner.storage.page_size)
        self.max_model_len = max_model_len
        self.max_graphs = max_graphs
        self._seen: dict[tuple, int] = {}
        self._graphs: dict[tuple, _Captured] = {}
        self._pool = None
        self.replays = 0
        self.last_h2d_bytes = 0

    @staticmethod
    def _portion_kind(longest: int) -> int:
        """What the kernels' dispatch distinguishes about the longest portion."""
        from ..kernels.attention_bf16 import TC_MIN_QUERY_LEN
        return 0 if longest == 1 else (2 if longest >= TC_MIN_QUERY_LEN else 1)

    def run(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """The same result as ``StepFunction.run``."""
        entries = [entry for entry in entries if entry.tokens]
        if not entries or any(e.start + len(e.tokens) > self.max_model_len for e in entries):
            return self.step_function.run(entries)
        tokens = sum(len(e.tokens) for e in entries)
        wanted = sum(len(e.want) for e in entries)
        requests_up = 1 << (len(entries) - 1).bit_length()
        wanted_up = 0 if wanted == 0 else max(requests_up, 1 << (wanted - 1).bit_length())
        singles = sum(1 for e in entries if len(e.tokens) == 1)      # the mixers' kernels split the batch there
        key = (tokens, requests_up, wanted_up, self._portion_kind(max(len(e.tokens) for e in entries)),
               singles if singles < len(entries) else 0)
        captured = self._graphs.get(key)
        if captured is None:
            self._seen[key] = self._seen.get(key, 0) + 1
            if self._seen[key] < 2 or len(self._graphs) >= self.max_graphs:
                return self.step_function.run(entries)
        self.runner.storage.zero_slots(self.runner.manager.take_fresh_slots())
        host, meta = self.step_function.pack_host(entries, pad_requests=requests_up, table_width=self.table_width,
                                                  pad_tokens=0, pad_wanted=wanted_up)
        if captured is None:
            captured = self._graphs[key] = self._capture(host, meta)
        captured.packed.copy_(host, non_blocking=True)
        self.last_h2d_bytes = host.numel() * host.element_size()
        captured.graph.replay()
        self.replays += 1
        return None if wanted == 0 else captured.logits[:wanted]

    def _capture(self, host: torch.Tensor, meta: dict) -> _Captured:
        device = self.runner.device
        packed = torch.empty(host.numel(), dtype=torch.int32, device=device)
        packed.copy_(host, non_blocking=True)
        meta = {**meta, "max_seq_len": self.max_model_len}
        ctx, token_ids, want_rows = self.step_function.context_from(packed, meta)
        model, views = self.runner.model, self.runner.storage.views

        def body() -> torch.Tensor | None:
            x, residual = model.forward(token_ids, ctx, views)
            return None if meta["num_wanted"] == 0 else model.logits(x, residual, want_rows)

        # A warm-up run of this very body: the step that came before went through the ordinary
        # step function with its own request count, table width and longest context, so the
        # padded shape planned for max_model_len may pick other kernels or splits (a key
        # split, the merge kernel), whose first launch (module load, attribute set-up) must
        # not fall inside the capture.  The body writes the same keys and values to the same
        # slots as the capture and the replay after it, so running it once more changes nothing.
        stream = torch.cuda.Stream(device=device)
        stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(stream):
            body()
        torch.cuda.current_stream(device).wait_stream(stream)
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, pool=self._pool):
            logits = body()
        if self._pool is None:
            self._pool = graph.pool()
        return _Captured(graph, packed, meta, logits, (ctx, token_ids, want_rows))
