"""The step function: one flattened batch of (request, its next tokens) through the model.

The reference never mixes: a forward is either one request's prompt piece with its own
cache (app/runtime/chat_engine.py:162-176) or B single decode tokens over a padded batch
cache (app/runtime/batch_decode.py:70-87, app/runtime/batch_cache.py:22-49). Here every
entry of a step contributes any number of next tokens (a portion of a prompt, cut
anywhere, or one decoded token); all of them run as one batch from the paged cache, and
float32 logits come back for exactly the wanted positions.

Per step the host builds, in one pinned buffer copied once to the device:
  token_ids[N], positions[N], tok_seq[N] (which entry a token belongs to), cu_q[S+1],
  context_lens[S] (tokens cached before the step), state_slots[S], logit_rows[n_out],
  and per cache group: slots[N] (where each token's k/v go) and block_tables[S, width].
The cache manager reserves pages before the launch and commits lengths after it, the
two-phase write of the reference's cache (app/runtime/kv_cache.py:53-72).
"""

from __future__ import annotations

import gc
import os
import time
from dataclasses import dataclass, field

import numpy as np
import torch

from matricxon_b200.cache.manager import CacheManager, OutOfPages
from matricxon_b200.cache.storage import CacheStorage
from matricxon_b200.ops import kernels


class StepError(RuntimeError):
    """A step whose inputs were malformed or whose kernels reported a bad index.

    ``request_ids`` names the requests at fault when the host could tell (a malformed entry is
    found before anything is reserved or launched, so the other requests of the step are
    untouched and can run in the next one); it is empty when a kernel reported the fault, and
    the step is then void for every request in it."""

    def __init__(self, message: str, request_ids: list[str] | None = None) -> None:
        super().__init__(message)
        self.request_ids = list(request_ids or ())


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and which of them want logits."""

    request_id: str
    tokens: list[int]
    want: list[int] = field(default_factory=list)    # indices into ``tokens``


@dataclass
class GroupStep:
    slots: torch.Tensor           # int32 [N]
    block_tables: torch.Tensor    # int32 [S, width]


@dataclass
class HostStep:
    """The same step on the host, for mixers that walk sequences in Python."""

    q_lens: list[int]
    context_lens: list[int]
    state_slots: list[int]
    fresh: list[bool]             # the request has nothing committed yet (state starts at zero)


class StepContext:
    """Device-side description of the tokens of one step, handed to every part."""

    def __init__(self, runner: "StepRunner") -> None:
        self._runner = runner
        self.n_tokens = 0
        self.n_seqs = 0
        self.max_kv_len = 0
        self.token_ids: torch.Tensor = None
        self.positions: torch.Tensor = None
        self.tok_seq: torch.Tensor = None
        self.cu_q: torch.Tensor = None
        self.context_lens: torch.Tensor = None
        self.state_slots: torch.Tensor = None
        self.logit_rows: torch.Tensor = None
        self.groups: list[GroupStep] = []
        self.status: torch.Tensor = runner.status
        self.host: HostStep = None
        self.capturing = False        # inside a CUDA-graph capture: buffers must belong to the graph
        self.padded = False           # a fixed-size decode batch: every sequence has one row or none
        self.memo: dict = {}          # what parts derive from the step once and share (tile lists, ...)
        # ops.linear.PendingSum: a block lets its parts leave a residual sum to the next norm (sums_may_pend);
        # the model lets a block hand such a sum on to the next block (pending_sum_wanted)
        self.sums_may_pend = False
        self.pending_sum_wanted = False

    def hidden(self, hidden_size: int) -> torch.Tensor:
        if self.capturing:
            return torch.empty((self.n_tokens, hidden_size), dtype=torch.float32,
                               device=self.token_ids.device)
        return self._runner.hidden_buffer(self.n_tokens, hidden_size)

    @property
    def device(self) -> torch.device:
        return self.token_ids.device if self.token_ids is not None else self._runner.device

    @property
    def sm_count(self) -> int:
        return self._runner.sm_count

    def scratch(self, nbytes: int) -> torch.Tensor:
        """Float32 scratch memory of at least ``nbytes`` for one kernel launch of this step. Every
        call of a step may get the same memory (launches of a step run in stream order and none
        keeps its scratch beyond its own merge), except inside a capture, where each caller gets
        memory that belongs to the graph."""
        if self.capturing:
            return torch.empty((nbytes + 3) // 4, dtype=torch.float32, device=self.device)
        return self._runner.scratch_buffer(nbytes)


class StepRunner:
    def __init__(self, model, cache: CacheManager, storage: CacheStorage,
                 max_step_tokens: int = 8192, max_step_seqs: int = 256,
                 max_model_len: int | None = None, use_graphs: bool = True,
                 max_graph_batch: int = 64, max_shape_graphs: int = 24,
                 shape_graph_max_tokens: int = 1024) -> None:
        self.model = model
        self.cache = cache
        self.storage = storage
        self.device = model.runtime.device
        self.max_step_tokens = max_step_tokens
        self.max_step_seqs = max_step_seqs
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        kernels.set_default_status(self.status)     # kernels with bounded waits report here too
        self._hidden: torch.Tensor | None = None
        self._scratch: torch.Tensor | None = None
        self._ints_host: torch.Tensor | None = None
        self._ints_dev: torch.Tensor | None = None
        self._upload_done: torch.cuda.Event | None = None
        self.steps_run = 0
        self.tokens_run = 0
        limit = max_model_len or model.spec.max_position_embeddings
        self.graph_table_width = (limit + cache.page_size - 1) // cache.page_size
        self.use_graphs = use_graphs and getattr(model, "capturable", False)
        self.max_graph_batch = max_graph_batch
        self._graphs: dict[int, tuple] = {}
        # steps that are not pure decoding are captured too, one graph per exact shape (how many
        # tokens each entry brings and where it wants logits), from the second time a shape is seen:
        # a prompt cut into equal portions, or the same mix of portions and decoded tokens step
        # after step, then costs the host one metadata copy and one replay instead of some three
        # hundred launches. Shapes seen once (the ragged end of a prompt) run eagerly.
        self.max_shape_graphs = max_shape_graphs
        # A graph saves the host's launch time (about 5 us a kernel), which only matters for steps that the
        # device finishes about as fast; a capture costs the step twice over. Larger steps run eagerly
        # (32 requests of 7B sizes: 14 captures of 2,048-token steps, 27 ms each, were replayed once).
        self.shape_graph_max_tokens = shape_graph_max_tokens
        self._shape_graphs: dict[tuple, tuple] = {}        # shape -> record, oldest use first
        self._shape_pool = None
        self._shape_seen: dict[tuple, int] = {}
        self.host_seconds = 0.0           # time the host spent inside ``run`` so far ...
        self.wait_seconds = 0.0           # ... of which waiting for the device to be done with a metadata buffer
        self._status_host: torch.Tensor | None = None
        self.chained_launch_rows = int(os.environ.get("MATRICXON_CHAINED_ROWS", "1024"))
        self._graph_host_arrays: dict[int, tuple] = {}       # bucket -> (pinned tensor, its numpy view)
        self._arange = np.arange(max_graph_batch + 2, dtype=np.int32)
        self._graph_pool = None
        # token ids are checked against the vocabulary on the host before a step is built; a caller
        # that vouches for its ids may switch the scan off (the embedding kernel still refuses a bad
        # id: it writes zeros and sets a status bit, which voids the step for all its requests)
        self.check_ids_on_host = True
        self.last_upload_bytes = 0        # host-to-device bytes of the latest step's metadata
        self.launches_per_step = 0        # this library's kernel launches in the latest step
        model.bind_cache(storage.groups, storage.states)

    # ------------------------------------------------------------------ buffers
    def hidden_buffer(self, n_tokens: int, hidden_size: int) -> torch.Tensor:
        if self._hidden is None or self._hidden.shape[0] < n_tokens or self._hidden.shape[1] != hidden_size:
            rows = max(n_tokens, 64)
            self._hidden = torch.empty((rows, hidden_size), dtype=torch.float32, device=self.device)
        return self._hidden[:n_tokens]

    def scratch_buffer(self, nbytes: int) -> torch.Tensor:
        count = (nbytes + 3) // 4
        if self._scratch is None or self._scratch.numel() < count:
            self._scratch = torch.empty(max(count, 1 << 18), dtype=torch.float32, device=self.device)
        return self._scratch

    def _int_buffers(self, count: int) -> tuple[torch.Tensor, torch.Tensor]:
        if self._ints_host is None or self._ints_host.numel() < count:
            size = max(count, 1 << 14)
            self._ints_host = torch.empty(size, dtype=torch.int32, pin_memory=True)
            self._ints_dev = torch.empty(size, dtype=torch.int32, device=self.device)
        return self._ints_host, self._ints_dev

    # ------------------------------------------------------------------ building a step
    def _validate(self, entries: list[StepEntry]) -> None:
        """Everything the host can check, before a page is reserved or a kernel launched. One
        error lists every fault and names the requests at fault."""
        if not entries:
            raise StepError("a step needs at least one entry")
        faults: list[str] = []
        at_fault: list[str] = []
        seen = set()
        total = 0
        vocab = self.model.spec.vocab_size
        for entry in entries:
            problems = []
            if entry.request_id in seen:
                problems.append("appears twice in one step")
            seen.add(entry.request_id)
            if not self.cache.has_request(entry.request_id):
                problems.append("is not live in the cache")
            if not entry.tokens:
                problems.append("brings no tokens")
            elif self.check_ids_on_host and not (0 <= min(entry.tokens) and max(entry.tokens) < vocab):
                bad = next(t for t in entry.tokens if not 0 <= t < vocab)
                problems.append(f"brings token id {bad}, outside the vocabulary of {vocab}")
            for index in entry.want:
                if not 0 <= index < len(entry.tokens):
                    problems.append(f"wants logits at {index}, but brings {len(entry.tokens)} tokens")
                    break
            total += len(entry.tokens)
            if problems:
                faults.append(f"request {entry.request_id!r} " + " and ".join(problems))
                if entry.request_id not in at_fault:
                    at_fault.append(entry.request_id)
        if faults:
            raise StepError("; ".join(faults), at_fault)
        if total > self.max_step_tokens:
            raise StepError(f"step of {total} tokens exceeds max_step_tokens={self.max_step_tokens}")
        if len(entries) > self.max_step_seqs:
            raise StepError(f"step of {len(entries)} requests exceeds max_step_seqs={self.max_step_seqs}")

    def build(self, entries: list[StepEntry], pad_to: int | None = None,
              table_widths: list[int] | None = None, buffers=None) -> StepContext:
        """Reserves pages for every entry and lays the step's metadata out on the device.
        Raises OutOfPages (with every reservation of this step undone) if the pool is short.

        ``pad_to`` (single-token entries only) pads the batch to a fixed number of rows with
        padding rows (``tok_seq = -1``, ``slot = -1``) and ``table_widths`` fixes the block
        tables' widths, so that the layout depends on nothing but those numbers: what a
        captured CUDA graph needs. ``buffers`` is a (pinned host, device, event) triple to use
        instead of the runner's growing ones."""
        self._validate(entries)
        cache = self.cache
        reserved: list[str] = []
        try:
            for entry in entries:
                cache.reserve(entry.request_id, len(entry.tokens))
                reserved.append(entry.request_id)
        except Exception:
            for request_id in reserved:
                cache.cancel_reservation(request_id)
            raise

        page_size = cache.page_size
        n_groups = len(cache.rules)
        n_seq_real = len(entries)
        n_tok_real = sum(len(e.tokens) for e in entries)
        n_seq = pad_to if pad_to is not None else n_seq_real
        n_tok = pad_to if pad_to is not None else n_tok_real
        records = [cache.record(e.request_id) for e in entries]
        if table_widths is None:
            table_widths = [max(1, max(len(r.tables[g]) for r in records)) for g in range(n_groups)]
        n_out = n_tok if pad_to is not None else sum(len(e.want) for e in entries)

        lengths = [n_tok, n_tok, n_tok, n_seq + 1, n_seq, n_seq, n_out]
        for g in range(n_groups):
            lengths.extend((n_tok, n_seq * table_widths[g]))
        offsets = []
        total = 0
        for length in lengths:
            offsets.append(total)
            total += (length + 3) & ~3              # keep every array 16-byte aligned
        flat = np.zeros(max(total, 4), dtype=np.int32)

        def part(i: int) -> np.ndarray:
            return flat[offsets[i]:offsets[i] + lengths[i]]

        token_ids, positions, tok_seq, cu_q = part(0), part(1), part(2), part(3)
        context_lens, state_slots, logit_rows = part(4), part(5), part(6)
        tok_seq[:] = -1
        context_list: list[int] = []
        slot_list: list[int] = []
        fresh: list[bool] = []
        max_kv = 0
        base = 0
        out_row = 0
        for s, (entry, record) in enumerate(zip(entries, records)):
            start = record.length
            n = len(entry.tokens)
            token_ids[base:base + n] = entry.tokens
            positions[base:base + n] = np.arange(start, start + n, dtype=np.int32)
            tok_seq[base:base + n] = s
            cu_q[s + 1] = base + n
            context_lens[s] = start
            state_slots[s] = record.state_slot
            context_list.append(start)
            slot_list.append(record.state_slot)
            fresh.append(record.fresh_state and start == 0)
            if pad_to is None:
                for index in entry.want:
                    logit_rows[out_row] = base + index
                    out_row += 1
            for g in range(n_groups):
                table = record.tables[g]
                width = table_widths[g]
                if len(table) > width:
                    raise StepError(f"request {entry.request_id!r} holds {len(table)} pages, "
                                    f"the fixed table width is {width}")
                part(8 + 2 * g)[s * width:(s + 1) * width] = cache.table_row(entry.request_id, g, width)
                slots_g = part(7 + 2 * g)
                if n == 1:
                    page = table[start // page_size]
                    if page < 0:
                        raise StepError(f"position {start} of {entry.request_id!r} has no page")
                    slots_g[base] = page * page_size + start % page_size
                else:
                    slots_g[base:base + n] = cache.slot_ids(entry.request_id, g, start, n)
            max_kv = max(max_kv, start + n)
            base += n
        if pad_to is not None:
            cu_q[n_seq_real + 1:] = base
            logit_rows[:] = np.arange(n_tok, dtype=np.int32)
            for g in range(n_groups):
                part(7 + 2 * g)[n_tok_real:] = -1
                part(8 + 2 * g)[n_seq_real * table_widths[g]:] = -1

        if buffers is None:
            host, dev = self._int_buffers(max(total, 4))
            if self._upload_done is None:
                self._upload_done = torch.cuda.Event()
            done = self._upload_done
        else:
            host, dev, done = buffers
        waited = time.perf_counter()
        done.synchronize()                           # the pinned buffer may still be in flight
        self.wait_seconds += time.perf_counter() - waited
        host[:total].copy_(torch.from_numpy(flat[:total]))
        dev[:total].copy_(host[:total], non_blocking=True)
        done.record()
        self.last_upload_bytes = total * 4

        def view(i: int) -> torch.Tensor:
            return dev[offsets[i]:offsets[i] + lengths[i]]

        ctx = StepContext(self)
        ctx.n_tokens, ctx.n_seqs, ctx.max_kv_len = n_tok, n_seq, max_kv
        ctx.padded = pad_to is not None
        ctx.token_ids, ctx.positions, ctx.tok_seq = view(0), view(1), view(2)
        ctx.cu_q, ctx.context_lens, ctx.state_slots, ctx.logit_rows = view(3), view(4), view(5), view(6)
        ctx.groups = [GroupStep(slots=view(7 + 2 * g),
                                block_tables=view(8 + 2 * g).view(n_seq, table_widths[g]))
                      for g in range(n_groups)]
        ctx.host = HostStep(q_lens=[len(e.tokens) for e in entries], context_lens=context_list,
                            state_slots=slot_list, fresh=fresh)
        for slot, is_fresh in zip(slot_list, fresh):
            if is_fresh:
                self.storage.zero_state(slot)
        return ctx

    # ------------------------------------------------------------------ running a step
    def _forward(self, ctx: StepContext, decode_rows: bool = False) -> torch.Tensor | None:
        """``decode_rows``: every row is one new token of its own sequence and wants logits."""
        hidden = self.model.forward(ctx)
        if ctx.logit_rows.numel() == 0:
            return None
        return self.model.logits(hidden, ctx.logit_rows)

    def _graph_bucket(self, entries: list[StepEntry]) -> int | None:
        """The captured batch size a pure decode step can replay, or None for an eager step."""
        if not self.use_graphs:
            return None
        if len(entries) > self.max_graph_batch:
            return None
        if any(len(e.tokens) != 1 or e.want != [0] for e in entries):
            return None
        page_size = self.cache.page_size
        stateful = bool(self.model.cache_plan.state_bytes_per_request)
        for entry in entries:
            if not self.cache.has_request(entry.request_id):
                return None
            record = self.cache.record(entry.request_id)
            if record.length // page_size >= self.graph_table_width:
                return None                      # longer than the captured block tables
            if record.fresh_state and stateful:
                return None                      # its state slot is zeroed on the eager path first
        bucket = 1
        while bucket < len(entries):
            bucket *= 2
        return bucket

    def _graph_buffers(self, n_tokens: int, n_seqs: int, widths: list[int]):
        """A pinned and a device buffer of a graph's own for the step's metadata, and the event
        that says when the latest copy between them is done."""
        layout_ints = 16 * max(n_tokens, n_seqs) + 64 + sum((n_tokens + 4) + n_seqs * (w + 4) for w in widths)
        buffers = (torch.empty(layout_ints, dtype=torch.int32, pin_memory=True),
                   torch.zeros(layout_ints, dtype=torch.int32, device=self.device),
                   torch.cuda.Event())
        buffers[2].record()
        return buffers

    def _capture(self, ctx: StepContext, decode_rows: bool, chained: bool, pool_name: str = "_graph_pool"):
        """Runs the step of ``ctx`` once eagerly (which also builds what parts keep per step) and
        captures it as a CUDA graph. Returns (graph, the graph's own logits, launches per step)."""
        ctx.max_kv_len = self.graph_table_width * self.cache.page_size
        launches_before = kernels.launch_count
        # steps of very few rows gain from kernels that start while their predecessor drains
        kernels.set_chained_launch(chained)
        try:
            self._forward(ctx, decode_rows=decode_rows)             # warm-up, outside the capture
            launches = kernels.launch_count - launches_before
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            ctx.capturing = True
            # no garbage collection inside the capture: a collected object may free pinned memory or
            # destroy a stream-ordered resource, which invalidates a capture in progress
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=getattr(self, pool_name)):
                    static_logits = self._forward(ctx, decode_rows=decode_rows)
            finally:
                if gc_was_on:
                    gc.enable()
            ctx.capturing = False
        finally:
            kernels.set_chained_launch(False)
        if getattr(self, pool_name) is None:
            setattr(self, pool_name, graph.pool())
        return graph, static_logits, launches

    def _run_graph(self, entries: list[StepEntry], bucket: int, token_feed: torch.Tensor | None = None) -> torch.Tensor:
        record = self._graphs.get(bucket)
        if token_feed is not None and record is None:
            raise StepError("a step fed from the device needs the graph of its batch size to exist already")
        widths = [self.graph_table_width] * len(self.cache.rules)
        if record is None:
            buffers = self._graph_buffers(bucket, bucket, widths)
            ctx = self.build(entries, pad_to=bucket, table_widths=widths, buffers=buffers)
            graph, static_logits, launches = self._capture(ctx, True, bucket <= self.chained_launch_rows)
            self.launches_per_step = launches
            # the captured kernels hold raw pointers into everything the context owns (the tile
            # list among them), so the context lives as long as the graph
            self._graphs[bucket] = (graph, static_logits, buffers, self.launches_per_step, ctx)
            graph.replay()
            return static_logits[:len(entries)]
        graph, static_logits, buffers, launches, _ctx = record
        self._refill_decode(entries, bucket, widths, buffers)
        if token_feed is not None:
            # the rows' token ids are still on the device (the step before has not been read yet): they
            # go over the placeholders that the metadata copy just wrote (ids are the buffer's first array)
            buffers[1][:len(entries)].copy_(token_feed[:len(entries)], non_blocking=True)
        graph.replay()
        self.launches_per_step = launches
        return static_logits[:len(entries)]

    def _shape_key(self, entries: list[StepEntry]) -> tuple | None:
        """The exact shape of a step that may run as a graph of its own, or None."""
        if not self.use_graphs or self.max_shape_graphs <= 0:
            return None
        if sum(len(entry.tokens) for entry in entries) > self.shape_graph_max_tokens:
            return None
        page_size = self.cache.page_size
        stateful = bool(self.model.cache_plan.state_bytes_per_request)
        for entry in entries:
            if not self.cache.has_request(entry.request_id):
                return None
            record = self.cache.record(entry.request_id)
            if (record.length + len(entry.tokens) - 1) // page_size >= self.graph_table_width:
                return None                      # longer than the captured block tables
            if record.fresh_state and stateful:
                return None
        return tuple((len(entry.tokens), tuple(entry.want)) for entry in entries)

    def _run_shape_graph(self, entries: list[StepEntry], key: tuple) -> torch.Tensor | None:
        """A step of a shape seen before: captured at its second appearance, replayed from then on."""
        record = self._shape_graphs.pop(key, None)
        widths = [self.graph_table_width] * len(self.cache.rules)
        if record is None:
            seen = self._shape_seen.get(key, 0) + 1
            self._shape_seen[key] = seen
            if len(self._shape_seen) > 4096:
                self._shape_seen.clear()
            if seen < 2:
                return self._run_eager(entries)
            n_tokens = sum(len(entry.tokens) for entry in entries)
            buffers = self._graph_buffers(n_tokens, len(entries), widths)
            ctx = self.build(entries, table_widths=widths, buffers=buffers)
            # a memory pool apart from the decode graphs': their small buffers then stay close together
            # instead of being scattered through the blocks that prompt-sized steps leave behind
            graph, static_logits, launches = self._capture(ctx, False, False, "_shape_pool")
            record = (graph, static_logits, buffers, launches, ctx)
            while len(self._shape_graphs) >= self.max_shape_graphs:
                self._shape_graphs.pop(next(iter(self._shape_graphs)))      # the least recently used
        else:
            self.build(entries, table_widths=widths, buffers=record[2])
        self._shape_graphs[key] = record
        record[0].replay()
        self.launches_per_step = record[3]
        return record[1]

    def _run_eager(self, entries: list[StepEntry]) -> torch.Tensor | None:
        ctx = self.build(entries)
        launches_before = kernels.launch_count
        logits = self._forward(ctx)
        self.launches_per_step = kernels.launch_count - launches_before
        return logits

    def _refill_decode(self, entries: list[StepEntry], bucket: int, widths: list[int], buffers) -> None:
        """The metadata of a captured decode step, written straight into the graph's pinned buffer
        and copied once: what ``build(entries, pad_to=bucket, ...)`` lays out, without the
        intermediate arrays and the context object a replay does not need."""
        self._validate(entries)
        cache = self.cache
        reserved: list[str] = []
        try:
            for entry in entries:
                cache.reserve(entry.request_id, 1)
                reserved.append(entry.request_id)
        except Exception:
            for request_id in reserved:
                cache.cancel_reservation(request_id)
            raise
        host, dev, done = buffers
        n, page_size, n_groups = len(entries), cache.page_size, len(cache.rules)
        lengths = [bucket, bucket, bucket, bucket + 1, bucket, bucket, bucket]
        for g in range(n_groups):
            lengths.extend((bucket, bucket * widths[g]))
        offsets, total = [], 0
        for length in lengths:
            offsets.append(total)
            total += (length + 3) & ~3
        arrays = self._graph_host_arrays.get(bucket)
        if arrays is None or arrays[0] is not host:
            arrays = (host, host.numpy())
            self._graph_host_arrays[bucket] = arrays
        flat = arrays[1]
        records = [cache.requests[entry.request_id] for entry in entries]
        lens = [record.length for record in records]
        waited = time.perf_counter()
        done.synchronize()                           # the pinned buffer may still be in flight
        self.wait_seconds += time.perf_counter() - waited
        try:
            def part(i: int) -> np.ndarray:
                return flat[offsets[i]:offsets[i] + lengths[i]]

            token_ids, positions, tok_seq, cu_q = part(0), part(1), part(2), part(3)
            token_ids[:n] = [entry.tokens[0] for entry in entries]
            token_ids[n:] = 0
            positions[:n] = lens
            positions[n:] = 0
            tok_seq[:n] = self._arange[:n]
            tok_seq[n:] = -1
            cu_q[:n + 1] = self._arange[:n + 1]
            cu_q[n + 1:] = n
            context_lens, state_slots, logit_rows = part(4), part(5), part(6)
            context_lens[:n] = lens
            context_lens[n:] = 0
            state_slots[:n] = [record.state_slot for record in records]
            state_slots[n:] = 0
            logit_rows[:] = self._arange[:bucket]
            for g in range(n_groups):
                width = widths[g]
                slots_g, tables_g = part(7 + 2 * g), part(8 + 2 * g).reshape(bucket, width)
                for s, (entry, record, start) in enumerate(zip(entries, records, lens)):
                    table = record.tables[g]
                    if len(table) > width:
                        raise StepError(f"request {entry.request_id!r} holds {len(table)} pages, "
                                        f"the fixed table width is {width}")
                    page = table[start // page_size]
                    if page < 0:
                        raise StepError(f"position {start} of {entry.request_id!r} has no page")
                    slots_g[s] = page * page_size + start % page_size
                    tables_g[s] = cache.table_row(entry.request_id, g, width)
                slots_g[n:] = -1
                tables_g[n:] = -1
        except Exception:
            for request_id in reserved:
                cache.cancel_reservation(request_id)
            raise
        dev[:total].copy_(host[:total], non_blocking=True)
        done.record()
        self.last_upload_bytes = total * 4

    def can_feed_from_device(self, entries: list[StepEntry]) -> bool:
        """Whether ``run(entries, token_feed=...)`` is possible: a pure decode step whose graph exists."""
        bucket = self._graph_bucket(entries)
        return bucket is not None and bucket in self._graphs

    def run(self, entries: list[StepEntry], token_feed: torch.Tensor | None = None) -> torch.Tensor | None:
        """Runs the entries as one batch and commits them. Returns float32 logits
        [wanted, vocab] in the order of the entries and of each ``want``, or None.

        ``token_feed`` (int32 on the device, one id per entry, in entry order) replaces the
        entries' single tokens: for a decode step launched before the ids that the step before
        it chose have reached the host. Only steps that replay an existing graph take it.

        A step of single decode tokens replays a CUDA graph captured for its batch size
        (rounded up to a power of two with padding rows); any other step replays a graph of its
        exact shape from the second time that shape is seen. The logits a replay returns live in
        the graph's memory and are overwritten by the next step of that shape."""
        started = time.perf_counter()
        bucket = self._graph_bucket(entries)
        try:
            if token_feed is not None and bucket is None:
                raise StepError("only a captured decode step can take its token ids from the device")
            if bucket is not None:
                logits = self._run_graph(entries, bucket, token_feed)
            else:
                key = self._shape_key(entries)
                logits = self._run_shape_graph(entries, key) if key is not None else self._run_eager(entries)
        except OutOfPages:
            raise
        except Exception:
            for entry in entries:
                if self.cache.has_request(entry.request_id):
                    self.cache.cancel_reservation(entry.request_id)
            raise
        for entry in entries:
            self.cache.commit(entry.request_id, len(entry.tokens))
        self.steps_run += 1
        self.tokens_run += len(entries) if bucket is not None else sum(len(e.tokens) for e in entries)
        self.host_seconds += time.perf_counter() - started
        return logits

    def enqueue_status_read(self) -> None:
        """Queues a copy of the status word to pinned host memory on the current stream; after the
        next synchronisation of that stream ``check_status(synchronised=True)`` reads it for free."""
        if self._status_host is None:
            self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self._status_host.copy_(self.status, non_blocking=True)

    def check_status(self, synchronised: bool = False) -> None:
        """Raises if a kernel met a bad index during the steps since the last check. Reads the
        device status word (a synchronisation), or, with ``synchronised``, the copy that
        ``enqueue_status_read`` queued before the caller's last synchronisation."""
        if synchronised and self._status_host is not None:
            word = int(self._status_host[0])
        else:
            word = int(self.status.item())
        if word != 0:
            self.status.zero_()
            raise StepError(f"a kernel reported: {kernels.describe_status(word)}")
