"""Helpers that drive ``bin/trace_run`` as a user would: a child process fed JSON lines."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
TRACE_RUN = ROOT / "bin" / "trace_run"


class TraceSession:
    """One running ``bin/trace_run``. ``step`` sends a step, waits for ``done``, and returns
    the logits file's contents (or None)."""

    def __init__(self, model_dir, dtype: str, max_tokens: int, out_dir, vocab: int,
                 extra_args: tuple[str, ...] = (), capture_stderr: bool = False) -> None:
        self.out_dir = Path(out_dir)
        self.vocab = vocab
        self.next_step = 0
        self.last_report: dict = {}
        env = dict(os.environ)
        self.proc = subprocess.Popen(
            [sys.executable, str(TRACE_RUN), "--model", str(model_dir), "--dtype", dtype,
             "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra_args],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE if capture_stderr else None,
            text=True, env=env)

    def step(self, entries: list[dict], end: list[str] = ()) -> np.ndarray | None:
        number = self.next_step
        self.next_step += 1
        self.proc.stdin.write(json.dumps({"step": number, "entries": entries, "end": list(end)}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {number}":
            self.proc.kill()
            raise RuntimeError(f"trace_run answered {line!r} to step {number} "
                               f"(exit code {self.proc.poll()})")
        with open(self.out_dir / f"{number}.json") as handle:
            self.last_report = json.load(handle)
        path = self.out_dir / f"{number}.f32"
        wanted = sum(len(e.get("want", [])) for e in entries)
        if wanted == 0:
            assert not path.exists()
            return None
        data = np.fromfile(path, dtype="<f4")
        assert data.size == wanted * self.vocab, (data.size, wanted, self.vocab)
        return data.reshape(wanted, self.vocab)

    def close(self) -> int:
        self.proc.stdin.close()
        code = self.proc.wait(timeout=120)
        self.proc.stdout.close()
        return code


class Collector:
    """Logits by (request, absolute position), filled from step outputs."""

    def __init__(self) -> None:
        self.logits: dict[tuple[str, int], np.ndarray] = {}
        self.progress: dict[str, int] = {}

    def run(self, session: TraceSession, portions: list[tuple[str, list[int]]], end=(),
            want_all: bool = True) -> None:
        """``portions``: (request, its next tokens) for one step; every position is wanted."""
        entries = []
        keys = []
        for request, tokens in portions:
            start = self.progress.get(request, 0)
            want = list(range(len(tokens))) if want_all else []
            entries.append({"id": request, "tokens": tokens, "want": want})
            keys.extend((request, start + i) for i in want)
            self.progress[request] = start + len(tokens)
        out = session.step(entries, end)
        # the program's own account of its rows: (request, absolute position), in order
        assert [tuple(row) for row in session.last_report["rows"]] == keys
        if keys:
            for key, row in zip(keys, out):
                assert key not in self.logits
                self.logits[key] = row

    def of(self, request: str, length: int) -> np.ndarray:
        return np.stack([self.logits[(request, i)] for i in range(length)])
