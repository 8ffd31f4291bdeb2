"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step's entries may be portions of prompts of any length beside single decoded tokens.  They
are flattened into one batch (no padding), every index a kernel will use is checked on the
host (miniserve/engine/flat_batch.py:490-569 does the same for its decode rows), the index
arrays travel to the device in one copy, the model runs once over all tokens, and the logits
come back only for the positions that were asked for.  MiniServe runs a step as one forward
per prompt portion plus one for the decode rows (miniserve/engine/executor.py:239-255) and
computes logits for every position of a portion; this engine does neither.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from .. import kernels
from ..cache.manager import RELEASED, CacheManager, StepReservation
from ..parts.context import StepContext


@dataclass
class StepEntry:
    """A request's next tokens and the indices among them whose logits are wanted."""

    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


class DecodeGraph:
    """One captured decode step for exactly ``rows`` rows, with fixed device buffers.

    Mechanics of miniserve/engine/graph.py:645-823: the index arrays live in one static buffer
    that a replay overwrites with a single copy; rows beyond the live ones are padding that reads
    and writes only the pool's scratch page; positions feed the rotation inside the graph, so
    nothing about a position is baked in; the pools never move.  Unlike there, every batch size
    up to the largest bucket replays a graph (the next bucket up, padded).
    """

    def __init__(self, step_function: "StepFunction", rows: int) -> None:
        sf = step_function
        self.rows = rows
        manager, storage = sf.manager, sf.storage
        ps = self.page_size = manager.page_size
        self.width = (sf.max_model_len + ps - 1) // ps
        n_groups = len(manager.paged_needs)
        # layout: tokens, positions, request_of_token, query_start, context_lens, state_slots, logit_rows,
        #         draw_index, then per group (block_tables, slots)
        sizes = [rows, rows, rows, rows + 1, rows, rows, rows, rows] + [rows * self.width, rows] * n_groups
        self.offsets = [0]
        for size in sizes:
            self.offsets.append(self.offsets[-1] + size)
        self.host = torch.empty(self.offsets[-1], dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()             # same memory, cheaper to fill from Python lists
        self.live_rows = -1
        self.copied: Optional[torch.cuda.Event] = None     # recorded after the last copy of the host mirror
        # per row: (the request's cache record, pages of its committed table that the mirror shows, per group)
        self.row_owner: list = [None] * rows
        self.has_windows = any(need.window is not None for need in manager.paged_needs)
        self.meta = torch.zeros(self.offsets[-1], dtype=torch.int32, device=sf.device)
        self.n_groups = n_groups
        self.scratch = storage.scratch_page
        self.scratch_slot = storage.scratch_slot
        self._fill_padding(0)
        self.meta.copy_(self.host)
        views = [self.meta[self.offsets[i]:self.offsets[i + 1]] for i in range(len(sizes))]
        group_views = [(views[8 + 2 * g].view(rows, self.width), views[9 + 2 * g]) for g in range(n_groups)]
        self.ctx_args = dict(
            n_tokens=rows, n_requests=rows, token_ids=views[0], positions=views[1], request_of_token=views[2],
            query_start=views[3], context_lens=views[4], state_slots=views[5], logit_rows=views[6],
            max_query_len=1, max_context_len=sf.max_model_len, dtype=sf.model.dtype, device=sf.device,
            group_views=group_views)
        self.draw_index = views[7]
        self.tokens_out = torch.zeros(rows, dtype=torch.int32, device=sf.device)
        self.logits: Optional[torch.Tensor] = None
        self.graph = torch.cuda.CUDAGraph()
        self.kernel_launches = 0

        def body() -> torch.Tensor:
            ctx = StepContext(**self.ctx_args)
            logits = sf.model.forward(ctx, storage)
            kernels.sample(logits, storage.sampling_records, ctx.state_slots, self.draw_index, self.tokens_out)
            return logits

        side = torch.cuda.Stream(device=sf.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            body()                       # warm-up outside the capture (lazy library set-up happens here)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        before = kernels.launch_count
        with torch.cuda.graph(self.graph, pool=sf.graph_pool):
            self.logits = body()
        self.kernel_launches = kernels.launch_count - before

    def _fill_padding(self, first_row: int) -> None:
        """Rows from ``first_row`` on become padding: token 0 at position 0 on the scratch page, in the scratch slot."""
        import numpy

        o, rows, host = self.offsets, self.rows, self.host_np
        ps = self.page_size
        host[o[0] + first_row:o[1]] = 0
        host[o[1] + first_row:o[2]] = 0
        host[o[2]:o[3]] = numpy.arange(rows, dtype=numpy.int32)
        host[o[3]:o[4]] = numpy.arange(rows + 1, dtype=numpy.int32)
        host[o[4] + first_row:o[5]] = 1
        host[o[5] + first_row:o[6]] = self.scratch_slot
        host[o[6]:o[7]] = numpy.arange(rows, dtype=numpy.int32)
        host[o[7] + first_row:o[8]] = 0
        for g in range(self.n_groups):
            tables = host[o[8 + 2 * g]:o[9 + 2 * g]].reshape(rows, self.width)
            tables[first_row:] = self.scratch
            host[o[9 + 2 * g] + first_row:o[10 + 2 * g]] = self.scratch * ps


class StepFunction:
    def __init__(self, model, storage, manager: CacheManager, max_model_len: int, use_graphs: bool = False) -> None:
        self.model, self.storage, self.manager = model, storage, manager
        self.max_model_len = max_model_len
        self.device = model.device
        self.vocab_size = model.spec.vocab_size
        self.use_graphs = use_graphs
        self.graphs: dict[int, DecodeGraph] = {}
        self.graph_pool = None
        self.graph_replays = 0
        self.eager_steps = 0
        self.last_tokens: Optional[torch.Tensor] = None   # tokens sampled inside the last replayed graph
        self.last_graph: Optional[DecodeGraph] = None

    # ------------------------------------------------------------------ batch building
    def build_context(self, entries: Sequence[StepEntry], reservation: StepReservation) -> StepContext:
        import numpy

        manager, ps = self.manager, self.manager.page_size
        if len(entries) != len(reservation.items):
            raise ValueError("the reservation was made for other entries")
        int32 = numpy.int32
        token_parts, position_parts, request_parts, slot_parts = [], [], [], None
        query_start = [0]
        context_lens: list[int] = []
        state_slots: list[int] = []
        logit_rows: list[int] = []
        n_groups = len(manager.paged_needs)
        slot_parts = [[] for _ in range(n_groups)]
        width = 1
        n = 0
        for row, (entry, item) in enumerate(zip(entries, reservation.items)):
            count = len(entry.tokens)
            if entry.request_id != item.request_id or count != item.end - item.start:
                raise ValueError(f"entry {row} does not match its reservation")
            if item.end > self.max_model_len:
                raise ValueError(f"request {entry.request_id!r} would reach {item.end} tokens; the limit is {self.max_model_len}")
            ids = numpy.asarray(entry.tokens, dtype=numpy.int64)      # (no copy if the caller holds its tokens as such an array)
            if count and (int(ids.min()) < 0 or int(ids.max()) >= self.vocab_size):
                raise ValueError(f"a token id of request {entry.request_id!r} lies outside the vocabulary of {self.vocab_size}")
            for index in entry.want:
                if not 0 <= index < count:
                    raise ValueError(f"wanted index {index} outside the {count} tokens of the entry")
                logit_rows.append(n + index)
            token_parts.append(ids.astype(int32))
            position_parts.append(numpy.arange(item.start, item.end, dtype=int32))
            request_parts.append(numpy.full(count, row, dtype=int32))
            n += count
            query_start.append(n)
            context_lens.append(item.end)
            state_slots.append(manager.requests[entry.request_id].slot)
            for group in range(n_groups):
                slot_parts[group].append(numpy.asarray(item.slots[group], dtype=int32))
                width = max(width, len(item.tables[group]))

        scratch = self.storage.scratch_page
        limit = self.storage.num_pages
        r = len(entries)
        tables = []
        slots = []
        for group in range(n_groups):
            table = numpy.full((r, width), scratch, dtype=int32)
            for row, item in enumerate(reservation.items):
                pages = numpy.asarray(item.tables[group], dtype=int32)
                pages = numpy.where(pages == RELEASED, scratch, pages)
                if pages.size and (int(pages.min()) < 0 or int(pages.max()) > limit):
                    raise ValueError(f"a page of request {item.request_id!r} lies outside the pool of {limit}")
                table[row, :pages.size] = pages
            tables.append(table.reshape(-1))
            group_slots = numpy.concatenate(slot_parts[group]) if slot_parts[group] else numpy.zeros(0, dtype=int32)
            if group_slots.size and (int(group_slots.min()) < 0 or int(group_slots.max()) >= limit * ps):
                raise ValueError("a slot lies outside the pool")
            slots.append(group_slots)

        empty = numpy.zeros(0, dtype=int32)
        pieces = [numpy.concatenate(token_parts) if token_parts else empty,
                  numpy.concatenate(position_parts) if position_parts else empty,
                  numpy.concatenate(request_parts) if request_parts else empty,
                  numpy.asarray(query_start, dtype=int32), numpy.asarray(context_lens, dtype=int32),
                  numpy.asarray(state_slots, dtype=int32), numpy.asarray(logit_rows, dtype=int32)]
        for group in range(n_groups):
            pieces += [tables[group], slots[group]]
        total = sum(p.size for p in pieces)
        staging = torch.empty(max(total, 1), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        staging_np = staging.numpy()
        offset = 0
        spans = []
        for piece in pieces:
            staging_np[offset:offset + piece.size] = piece
            spans.append((offset, piece.size))
            offset += piece.size
        on_device = staging.to(self.device, non_blocking=True)
        views = [on_device[start:start + length] for start, length in spans]
        group_views = []
        for group in range(n_groups):
            group_views.append((views[7 + 2 * group].view(r, width), views[8 + 2 * group]))
        return StepContext(
            n_tokens=n, n_requests=r, token_ids=views[0], positions=views[1], request_of_token=views[2],
            query_start=views[3], context_lens=views[4], state_slots=views[5], logit_rows=views[6],
            max_query_len=max((len(e.tokens) for e in entries), default=0),
            max_context_len=max(context_lens, default=0), dtype=self.model.dtype, device=self.device,
            host_query_start=query_start, host_context_lens=context_lens, host_state_slots=state_slots,
            group_views=group_views)

    # ------------------------------------------------------------------ running
    def replays(self, entries: Sequence[StepEntry]) -> bool:
        """Whether these entries run as a captured graph: single tokens, all of whose logits are wanted."""
        return bool(self.use_graphs and entries and len(entries) <= DECODE_BUCKETS[-1]
                    and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries))

    def run(self, entries: Sequence[StepEntry], reservation: StepReservation,
            draw_index: Optional[Sequence[int]] = None, feed_back: bool = False) -> torch.Tensor:
        """float32 logits ``[number of wanted positions, vocab]`` on the device, in entry order.

        A step of single tokens whose logits are all wanted replays a captured graph when graphs
        are on; the graph also samples, and ``last_tokens`` then holds one token per entry
        (``draw_index``: each request's draw count, for its random stream).  ``feed_back``: the
        entries are the rows of the last replay, in its order, and each row's token is the one that
        replay sampled for it; it is taken on the device, and the entries' own token ids are ignored.
        """
        self.last_tokens = None
        if self.replays(entries):
            return self._replay(entries, reservation, draw_index, feed_back)
        if feed_back:
            raise ValueError("only a replayed step can take its tokens from the step before")
        ctx = self.build_context(entries, reservation)
        self.eager_steps += 1
        return self.model.forward(ctx, self.storage)

    def graph_for(self, n: int) -> "DecodeGraph":
        """The captured decode step of the smallest bucket that holds ``n`` rows (captured on first use)."""
        rows = next(b for b in DECODE_BUCKETS if b >= n)
        graph = self.graphs.get(rows)
        if graph is None:
            if self.graph_pool is None:
                self.graph_pool = torch.cuda.graph_pool_handle()
            graph = self.graphs[rows] = DecodeGraph(self, rows)
        return graph

    def capture_decode_graphs(self, max_rows: int) -> None:
        """Captures every bucket up to ``max_rows`` now, so that no step pays for a capture later
        (MiniServe captures its batched graphs at start-up too: miniserve/engine/graph.py:689-729)."""
        if not self.use_graphs:
            return
        for bucket in DECODE_BUCKETS:
            self.graph_for(min(bucket, max_rows))
            if bucket >= max_rows:
                break

    def _replay(self, entries, reservation, draw_index, feed_back: bool = False) -> torch.Tensor:
        n = len(entries)
        graph = self.graph_for(n)
        if feed_back and (graph is not self.last_graph or graph.live_rows != n):
            raise ValueError("the step before was not a replay of the same rows")
        if graph.copied is not None:
            graph.copied.synchronize()       # the host mirror is free once the last copy of it has run
        manager, ps = self.manager, self.manager.page_size
        limit, scratch = self.storage.num_pages, self.storage.scratch_page
        o, host = graph.offsets, graph.host_np
        if graph.live_rows != n:
            graph._fill_padding(n)
            for row in range(n, graph.rows):
                graph.row_owner[row] = None
            graph.live_rows = n
        tokens, positions, lens, slots_state = [], [], [], []
        for row, (entry, item) in enumerate(zip(entries, reservation.items)):
            token = int(entry.tokens[0])
            if entry.request_id != item.request_id or item.end - item.start != 1:
                raise ValueError(f"entry {row} does not match its reservation")
            if not 0 <= token < self.vocab_size:
                raise ValueError(f"token id {token} outside the vocabulary of {self.vocab_size}")
            if item.end > self.max_model_len:
                raise ValueError(f"request {entry.request_id!r} would reach {item.end} tokens; the limit is {self.max_model_len}")
            tokens.append(token)
            positions.append(item.start)
            lens.append(item.end)
            record = manager.requests[entry.request_id]
            slots_state.append(record.slot)
            owner = graph.row_owner[row]
            if feed_back and (owner is None or owner[0] is not record):
                raise ValueError(f"row {row} of the step before belonged to another request")
            # The row keeps what it shows only for the very same admission (a request id can come back after a
            # release, with other pages), and only as far as the pages were committed when they were written:
            # a page reserved for a step that was aborted may be another one next time.
            same = owner is not None and owner[0] is record and not graph.has_windows
            for g in range(graph.n_groups):
                table = item.tables[g]
                if len(table) > graph.width:
                    raise ValueError("a block table is wider than the model's longest context")
                # committed pages that this row already shows stay; the others are checked and written
                first = owner[1][g] if same and owner[1][g] <= len(table) else 0
                fresh = table[first:]
                if any(p != RELEASED and not 0 <= p < limit for p in fresh):
                    raise ValueError("a page lies outside the pool")
                base = o[8 + 2 * g] + row * graph.width
                if fresh:
                    host[base + first:base + len(table)] = [scratch if p == RELEASED else p for p in fresh]
                if first == 0:
                    host[base + len(table):base + graph.width] = scratch
                slot = int(item.slots[g][0])
                if not 0 <= slot < limit * ps:
                    raise ValueError(f"slot {slot} outside the pool")
                host[o[9 + 2 * g] + row] = slot
            graph.row_owner[row] = (record, [len(item.tables[g]) - len(item.new_pages[g]) for g in range(graph.n_groups)])
        host[o[0]:o[0] + n] = tokens
        host[o[1]:o[1] + n] = positions
        host[o[4]:o[4] + n] = lens
        host[o[5]:o[5] + n] = slots_state
        host[o[7]:o[7] + n] = 0 if draw_index is None else list(draw_index)
        graph.meta.copy_(graph.host, non_blocking=True)
        if graph.copied is None:
            graph.copied = torch.cuda.Event()
        graph.copied.record()
        if feed_back:
            graph.meta[o[0]:o[0] + n].copy_(graph.tokens_out[:n])
        self.last_graph = graph
        graph.graph.replay()
        self.graph_replays += 1
        self.last_tokens = graph.tokens_out[:n]
        return graph.logits[:n]
