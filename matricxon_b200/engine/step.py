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

from dataclasses import dataclass, field

import torch

from matricxon_b200.cache.manager import CacheManager
from matricxon_b200.cache.storage import CacheStorage
from matricxon_b200.ops import kernels


class StepError(RuntimeError):
    """A step whose inputs were malformed or whose kernels reported a bad index."""


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

    def hidden(self, hidden_size: int) -> torch.Tensor:
        return self._runner.hidden_buffer(self.n_tokens, hidden_size)

    def attention_splits(self, n_heads: int, n_kv_heads: int, head_dim: int,
                         window: int | None) -> tuple[int, torch.Tensor | None]:
        """How many key splits the attention launch should use, and its scratch memory.

        Few query tokens (decoding) leave most SMs idle unless the keys are split; many
        tokens fill the GPU by themselves."""
        group = n_heads // n_kv_heads
        blocks = self.n_tokens * n_kv_heads * ((group + 15) // 16)
        span = self.max_kv_len if window is None else min(self.max_kv_len, window)
        chunks = span // 32 + 2
        target = self._runner.sm_count * 4
        n_splits = max(1, min(target // max(blocks, 1), chunks // 2, 64))
        if n_splits == 1:
            return 1, None
        need = kernels.attention_scratch_bytes(self.n_tokens, n_heads, head_dim, n_splits)
        return n_splits, self._runner.scratch_buffer(need)


class StepRunner:
    def __init__(self, model, cache: CacheManager, storage: CacheStorage,
                 max_step_tokens: int = 8192, max_step_seqs: int = 256) -> None:
        self.model = model
        self.cache = cache
        self.storage = storage
        self.device = model.runtime.device
        self.max_step_tokens = max_step_tokens
        self.max_step_seqs = max_step_seqs
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._hidden: torch.Tensor | None = None
        self._scratch: torch.Tensor | None = None
        self._ints_host: torch.Tensor | None = None
        self._ints_dev: torch.Tensor | None = None
        self._upload_done: torch.cuda.Event | None = None
        self.steps_run = 0
        self.tokens_run = 0
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
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        total = 0
        for entry in entries:
            if entry.request_id in seen:
                raise StepError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            if not entry.tokens:
                raise StepError(f"request {entry.request_id!r} brings no tokens")
            for index in entry.want:
                if not 0 <= index < len(entry.tokens):
                    raise StepError(f"request {entry.request_id!r} wants logits at {index}, "
                                    f"but brings {len(entry.tokens)} tokens")
            total += len(entry.tokens)
        if total > self.max_step_tokens:
            raise StepError(f"step of {total} tokens exceeds max_step_tokens={self.max_step_tokens}")
        if len(entries) > self.max_step_seqs:
            raise StepError(f"step of {len(entries)} requests exceeds max_step_seqs={self.max_step_seqs}")

    def build(self, entries: list[StepEntry]) -> StepContext:
        """Reserves pages for every entry and lays the step's metadata out on the device.
        Raises OutOfPages (with every reservation of this step undone) if the pool is short."""
        self._validate(entries)
        cache = self.cache
        reserved: list[str] = []
        try:
            for entry in entries:
                if not cache.has_request(entry.request_id):
                    raise StepError(f"request {entry.request_id!r} is not live in the cache")
                cache.reserve(entry.request_id, len(entry.tokens))
                reserved.append(entry.request_id)
        except Exception:
            for request_id in reserved:
                cache.cancel_reservation(request_id)
            raise

        page_size = cache.page_size
        n_groups = len(cache.rules)
        token_ids: list[int] = []
        positions: list[int] = []
        tok_seq: list[int] = []
        cu_q = [0]
        context_lens: list[int] = []
        state_slots: list[int] = []
        logit_rows: list[int] = []
        fresh: list[bool] = []
        slots: list[list[int]] = [[] for _ in range(n_groups)]
        max_kv = 0
        for s, entry in enumerate(entries):
            record = cache.record(entry.request_id)
            start = record.length
            n = len(entry.tokens)
            base = len(token_ids)
            token_ids.extend(entry.tokens)
            positions.extend(range(start, start + n))
            tok_seq.extend([s] * n)
            cu_q.append(base + n)
            context_lens.append(start)
            state_slots.append(record.state_slot)
            fresh.append(record.fresh_state and start == 0)
            logit_rows.extend(base + index for index in entry.want)
            for g in range(n_groups):
                slots[g].extend(cache.slot_ids(entry.request_id, g, start, n))
            max_kv = max(max_kv, start + n)
        n_tok, n_seq = len(token_ids), len(entries)
        widths = []
        tables: list[list[int]] = []
        for g in range(n_groups):
            width = max(1, max(len(cache.record(e.request_id).tables[g]) for e in entries))
            widths.append(width)
            flat: list[int] = []
            for entry in entries:
                table = cache.record(entry.request_id).tables[g]
                flat.extend(table)
                flat.extend([-1] * (width - len(table)))
            tables.append(flat)
        del page_size

        pieces = [token_ids, positions, tok_seq, cu_q, context_lens, state_slots, logit_rows]
        for g in range(n_groups):
            pieces.extend((slots[g], tables[g]))
        offsets = []
        total = 0
        for piece in pieces:
            offsets.append(total)
            total += (len(piece) + 3) & ~3          # keep every array 16-byte aligned
        host, dev = self._int_buffers(max(total, 4))
        flat_all = torch.zeros(total, dtype=torch.int32)
        for piece, offset in zip(pieces, offsets):
            if piece:
                flat_all[offset:offset + len(piece)] = torch.tensor(piece, dtype=torch.int32)
        if self._upload_done is not None:
            self._upload_done.synchronize()      # the pinned buffer may still be in flight
        host[:total].copy_(flat_all)
        dev[:total].copy_(host[:total], non_blocking=True)
        self.last_upload_bytes = total * 4
        if self._upload_done is None:
            self._upload_done = torch.cuda.Event()
        self._upload_done.record()

        def view(i: int) -> torch.Tensor:
            return dev[offsets[i]:offsets[i] + len(pieces[i])]

        ctx = StepContext(self)
        ctx.n_tokens, ctx.n_seqs, ctx.max_kv_len = n_tok, n_seq, max_kv
        ctx.token_ids, ctx.positions, ctx.tok_seq = view(0), view(1), view(2)
        ctx.cu_q, ctx.context_lens, ctx.state_slots, ctx.logit_rows = view(3), view(4), view(5), view(6)
        ctx.groups = [GroupStep(slots=view(7 + 2 * g),
                                block_tables=view(8 + 2 * g).view(n_seq, widths[g]))
                      for g in range(n_groups)]
        ctx.host = HostStep(q_lens=[len(e.tokens) for e in entries], context_lens=context_lens,
                            state_slots=state_slots, fresh=fresh)
        for slot, is_fresh in zip(state_slots, fresh):
            if is_fresh:
                self.storage.zero_state(slot)
        return ctx

    # ------------------------------------------------------------------ running a step
    def run(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """Runs the entries as one batch and commits them. Returns float32 logits
        [wanted, vocab] in the order of the entries and of each ``want``, or None."""
        ctx = self.build(entries)
        launches_before = kernels.launch_count
        try:
            hidden = self.model.forward(ctx)
            logits = None
            if ctx.logit_rows.numel() > 0:
                logits = self.model.logits(hidden, ctx.logit_rows)
        except Exception:
            for entry in entries:
                self.cache.cancel_reservation(entry.request_id)
            raise
        for entry in entries:
            self.cache.commit(entry.request_id, len(entry.tokens))
        self.steps_run += 1
        self.tokens_run += ctx.n_tokens
        self.launches_per_step = kernels.launch_count - launches_before
        return logits

    def check_status(self) -> None:
        """Reads the device status word (a synchronisation) and raises if a kernel met a
        bad index during the steps since the last check."""
        word = int(self.status.item())
        if word != 0:
            self.status.zero_()
            raise StepError(f"a kernel reported: {kernels.describe_status(word)}")
