"""Trace replay through ``bin/trace_run`` against the plain implementation: every way of
cutting and batching the same requests, in float32 and in bfloat16, for both tiny
configurations, with a pool small enough that pages are used again."""

import numpy as np
import pytest
import torch

from plain_reference import plain_forward, plain_load_model
from tiny_configs import TINY, random_ids, write_tiny_model
from trace_utils import Collector, TraceSession

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 40, 64, 100], "B": [1, 3, 23, 24, 25, 100, 70]}
CHUNKS = [7, 2, 5, 3, 11, 2, 4, 13, 2, 9]


def tolerance(dtype, reference):
    if dtype == "float32":
        return 2e-5
    return 0.03 * float(np.abs(reference).max())


@pytest.fixture(scope="module", params=[("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    name, dtype = request.param
    folder = tmp_path_factory.mktemp(f"model_{name}_{dtype}")
    # bfloat16 runs read bfloat16 files, so the plain implementation sees the very same weights
    write_tiny_model(folder, name, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    cfg, weights = plain_load_model(folder)
    prompts = {f"r{i}": random_ids(n, cfg["vocab"], seed=10 * i + len(name))
               for i, n in enumerate(LENGTHS[name])}
    reference = {rid: plain_forward(cfg, weights, ids).numpy() for rid, ids in prompts.items()}
    out_dir = tmp_path_factory.mktemp(f"out_{name}_{dtype}")
    # room for the four longest requests at once, each rounded up to 64 tokens
    longest = sorted((len(p) for p in prompts.values()), reverse=True)[:4]
    max_tokens = sum((n + 63) // 64 * 64 for n in longest)
    session = TraceSession(folder, dtype, max_tokens, out_dir, cfg["vocab"])
    yield dict(name=name, dtype=dtype, cfg=cfg, prompts=prompts, reference=reference, session=session)
    assert session.close() == 0


def check(setup, collector, request_ids=None):
    for rid in request_ids or setup["prompts"]:
        ref = setup["reference"][rid]
        got = collector.of(rid, len(setup["prompts"][rid]))
        worst = np.abs(got - ref).max(axis=1)
        limit = tolerance(setup["dtype"], ref)
        first_bad = np.nonzero(worst > limit)[0]
        assert first_bad.size == 0, (f"{rid}: first wrong position {first_bad[0]} of {len(ref)}, "
                                     f"error {worst[first_bad[0]]:.3e} > {limit:.1e}")


def test_whole(setup):
    collector = Collector()
    for rid, ids in setup["prompts"].items():
        collector.run(setup["session"], [(rid, ids)], end=[rid])
    check(setup, collector)


def test_first_tokens(setup):
    """The first positions alone: a one-token request and the start of a longer one."""
    collector = Collector()
    rid = max(setup["prompts"], key=lambda r: len(setup["prompts"][r]))
    ids = setup["prompts"][rid]
    collector.run(setup["session"], [("first", ids[:1])])
    collector.run(setup["session"], [("first", ids[1:2])], end=["first"])
    ref = setup["reference"][rid][:2]
    got = collector.of("first", 2)
    assert np.abs(got - ref).max() <= tolerance(setup["dtype"], ref)


def test_tail_decoded_one_by_one(setup):
    collector = Collector()
    for rid, ids in setup["prompts"].items():
        head = max(len(ids) - 32, 0)
        if head:
            collector.run(setup["session"], [(rid, ids[:head])])
        for i in range(head, len(ids)):
            collector.run(setup["session"], [(rid, ids[i:i + 1])],
                          end=[rid] if i == len(ids) - 1 else [])
    check(setup, collector)


def test_portions_of_changing_size(setup):
    collector = Collector()
    for rid, ids in setup["prompts"].items():
        start, turn = 0, 0
        while start < len(ids):
            size = min(CHUNKS[turn % len(CHUNKS)], len(ids) - start)
            turn += 1
            last = start + size == len(ids)
            collector.run(setup["session"], [(rid, ids[start:start + size])], end=[rid] if last else [])
            start += size
    check(setup, collector)


def test_mixed_batches_with_page_reuse(setup):
    """Up to four live requests; prompt portions of some beside single decoded tokens of
    others; requests end and new ones take their pages."""
    prompts = setup["prompts"]
    order = sorted(prompts, key=lambda r: -len(prompts[r]))
    waiting = list(order) + [f"{rid}#again" for rid in order[:3]]     # a second round reuses pages
    tokens = {**prompts, **{f"{rid}#again": prompts[rid] for rid in order[:3]}}
    live: dict[str, int] = {}
    collector = Collector()
    turn = 0
    owners: dict[tuple[int, int], set] = {}     # (group, physical page) -> requests that held it
    reused_before = None
    while waiting or live:
        while waiting and len(live) < 4:
            live[waiting.pop(0)] = 0
        portions, ended = [], []
        for slot, (rid, done) in enumerate(list(live.items())):
            ids = tokens[rid]
            remaining = len(ids) - done
            if (turn + slot) % 5 == 4 and len(live) > 1:
                continue                                   # this request sits the step out
            prefill_part = max(len(ids) - 12, 1)           # the last tokens go one by one
            if done < prefill_part:
                size = min(CHUNKS[(turn + slot) % len(CHUNKS)], prefill_part - done)
            else:
                size = 1
            size = min(size, remaining)
            portions.append((rid, ids[done:done + size]))
            live[rid] = done + size
            if live[rid] == len(ids):
                ended.append(rid)
        turn += 1
        if portions:
            collector.run(setup["session"], portions, end=ended)
            report = setup["session"].last_report["pages"]
            if reused_before is None:
                reused_before = report["reused"]
            held = 0
            for rid, state in report["requests"].items():
                assert state["length"] == live[rid]
                for group, table in enumerate(state["pages"]):
                    for page in table:
                        if page >= 0:
                            owners.setdefault((group, page), set()).add(rid)
                            held += 1
            # no page lost: what is free and what the live requests hold is the pool
            assert sum(report["free"]) + held == sum(report["total"])
        for rid in ended:
            del live[rid]
    shared = [page for page, who in owners.items() if len(who) > 1]
    assert shared, "no physical page served two requests: the pool was not small enough"
    assert setup["session"].last_report["pages"]["reused"] > reused_before
    for rid, ids in tokens.items():
        base = rid.split("#")[0]
        ref = setup["reference"][base]
        got = collector.of(rid, len(ids))
        worst = np.abs(got - ref).max(axis=1)
        limit = tolerance(setup["dtype"], ref)
        first_bad = np.nonzero(worst > limit)[0]
        assert first_bad.size == 0, (f"{rid}: first wrong position {first_bad[0]}, "
                                     f"error {worst[first_bad[0]]:.3e} > {limit:.1e}")


def test_long_decoding(setup):
    """A short prompt, then every further token one by one, far past the window."""
    rid = max(setup["prompts"], key=lambda r: len(setup["prompts"][r]))
    ids = setup["prompts"][rid]
    collector = Collector()
    collector.run(setup["session"], [("long", ids[:3])])
    for i in range(3, len(ids)):
        collector.run(setup["session"], [("long", ids[i:i + 1])], end=["long"] if i == len(ids) - 1 else [])
    ref = setup["reference"][rid]
    got = collector.of("long", len(ids))
    assert np.abs(got - ref).max() <= tolerance(setup["dtype"], ref)


def test_steps_without_wanted_logits_write_no_file(setup):
    session = setup["session"]
    rid = max(setup["prompts"], key=lambda r: len(setup["prompts"][r]))
    ids = setup["prompts"][rid][:4]
    assert session.step([{"id": "quiet", "tokens": ids[:2], "want": []}]) is None
    out = session.step([{"id": "quiet", "tokens": ids[2:4], "want": [1]}], end=["quiet"])
    ref = setup["reference"][rid][3]
    assert out.shape == (1, setup["cfg"]["vocab"])
    assert np.abs(out[0] - ref).max() <= tolerance(setup["dtype"], ref)


def test_a_line_that_is_no_step_ends_the_run_with_a_message(tmp_path):
    """Host-side faults of a trace: the program says which line and why, and exits with 2;
    nothing reaches the GPU."""
    import json
    import subprocess
    import sys

    from trace_utils import TRACE_RUN

    folder = tmp_path / "model"
    write_tiny_model(folder, "A", torch.float32)
    vocab = TINY["A"][0]["vocab_size"]
    good = {"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": []}
    cases = {
        "not json": ("{this is not json", "not JSON"),
        "no tokens": (json.dumps({"step": 1, "entries": [{"id": "a", "tokens": []}]}), "non-empty list"),
        "bad id": (json.dumps({"step": 1, "entries": [{"id": "a", "tokens": [vocab + 3], "want": [0]}]}),
                   "outside the vocabulary"),
        "twice": (json.dumps({"step": 1, "entries": [{"id": "a", "tokens": [1]}, {"id": "a", "tokens": [2]}]}),
                  "appears twice"),
        "want": (json.dumps({"step": 1, "entries": [{"id": "a", "tokens": [1, 2], "want": [2]}]}),
                 "wants logits at 2"),
        "unknown end": (json.dumps({"step": 1, "entries": [], "end": ["nobody"]}), "not live"),
    }
    for label, (line, expected) in cases.items():
        out = tmp_path / f"out_{label.replace(' ', '_')}"
        done = subprocess.run(
            [sys.executable, str(TRACE_RUN), "--model", str(folder), "--dtype", "float32", "--out", str(out),
             "--max-tokens", "128"], input=json.dumps(good) + "\n" + line + "\n",
            capture_output=True, text=True, timeout=300)
        assert done.returncode == 2, (label, done.returncode, done.stderr[-500:])
        assert "input line 2" in done.stderr and expected in done.stderr, (label, done.stderr[-500:])
        assert done.stdout.split() == ["done", "0"], (label, done.stdout)
        assert (out / "0.f32").exists() and not (out / "1.f32").exists()
