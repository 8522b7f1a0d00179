"""Steps that are not pure decoding replay a CUDA graph of their exact shape from the second time
the shape is seen: the first run is eager, the second captures, the rest replay. The logits must
not care which of the three a step was, nor whose requests, contents and pages it carries."""

import numpy as np
import pytest
import torch

from plain_reference import plain_config, plain_forward
from tiny_configs import TINY, random_ids, tiny_config, tiny_tensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make(dtype, **core_options):
    from matricxon_b200.engine.core import EngineCore, model_from_tensors

    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = tiny_tensors("B", store)
    model = model_from_tensors(tiny_config("B"), tensors, dtype=dtype, device=DEV)
    core = EngineCore(model, max_cache_tokens=1024, max_requests=8, poison_cache=True, **core_options)
    return core, plain_config(TINY["B"][0]), {k: v.float() for k, v in tensors.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_repeated_mixed_shape_is_captured_and_replayed(dtype):
    from matricxon_b200.engine.step import StepEntry

    core, cfg, weights = make(dtype)
    runner, cache = core.runner, core.cache
    vocab = cfg["vocab"]
    sequences = {"d1": random_ids(40, vocab, 1), "d2": random_ids(55, vocab, 2), "p": random_ids(83, vocab, 3)}
    reference = {rid: plain_forward(cfg, weights, ids, dtype=torch.float32).numpy() for rid, ids in sequences.items()}
    for rid in sequences:
        cache.add_request(rid)
    runner.run([StepEntry("d1", sequences["d1"][:20]), StepEntry("d2", sequences["d2"][:30])])
    done = {"d1": 20, "d2": 30, "p": 0}
    got = {rid: {} for rid in sequences}
    modes = []
    for turn in range(8):                       # the same shape eight times: 1 + 1 + 10 tokens
        entries = [StepEntry("d1", sequences["d1"][done["d1"]:done["d1"] + 1], [0]),
                   StepEntry("d2", sequences["d2"][done["d2"]:done["d2"] + 1], [0]),
                   StepEntry("p", sequences["p"][done["p"]:done["p"] + 10], [9, 0])]
        graphs_before = len(runner._shape_graphs)
        logits = runner.run(entries).clone()
        modes.append(len(runner._shape_graphs) - graphs_before)
        got["d1"][done["d1"]] = logits[0]
        got["d2"][done["d2"]] = logits[1]
        got["p"][done["p"] + 9] = logits[2]
        got["p"][done["p"]] = logits[3]
        done["d1"] += 1
        done["d2"] += 1
        done["p"] += 10
    runner.check_status()
    assert modes == [0, 1, 0, 0, 0, 0, 0, 0]            # eager, captured, then replayed
    assert len(runner._shape_graphs) == 1 and not runner._graphs
    for rid, rows in got.items():
        for position, row in rows.items():
            ref = reference[rid][position]
            limit = 2e-5 if dtype == "float32" else 0.03 * float(np.abs(reference[rid]).max())
            assert np.abs(row.cpu().numpy() - ref).max() <= limit, (rid, position)
    # other requests, other pages, the same shape: the graph serves them too
    for rid in sequences:
        cache.free_request(rid)
    fresh = {"x": random_ids(30, vocab, 4), "y": random_ids(30, vocab, 5), "z": random_ids(30, vocab, 6)}
    for rid in fresh:
        cache.add_request(rid)
    runner.run([StepEntry("x", fresh["x"][:12]), StepEntry("y", fresh["y"][:7])])
    logits = runner.run([StepEntry("x", fresh["x"][12:13], [0]), StepEntry("y", fresh["y"][7:8], [0]),
                         StepEntry("z", fresh["z"][:10], [9, 0])]).clone()
    runner.check_status()
    assert len(runner._shape_graphs) == 1
    for row, (rid, position) in zip(logits, (("x", 12), ("y", 7), ("z", 9), ("z", 0))):
        ref = plain_forward(cfg, weights, fresh[rid], dtype=torch.float32).numpy()
        limit = 2e-5 if dtype == "float32" else 0.03 * float(np.abs(ref).max())
        assert np.abs(row.cpu().numpy() - ref[position]).max() <= limit, (rid, position)


def test_graphs_of_shapes_are_bounded_and_the_oldest_goes():
    from matricxon_b200.engine.step import StepEntry

    core, cfg, weights = make("float32")
    runner, cache = core.runner, core.cache
    runner.max_shape_graphs = 2
    ids = random_ids(400, cfg["vocab"], 7)
    reference = plain_forward(cfg, weights, ids[:200], dtype=torch.float32).numpy()
    for size in (5, 6, 7, 5):                     # three shapes, two slots; 5 comes back after it went
        cache.add_request("r")
        done = 0
        for _ in range(4):
            logits = runner.run([StepEntry("r", ids[done:done + size], [size - 1])])
            assert np.abs(logits[0].cpu().numpy() - reference[done + size - 1]).max() <= 2e-5
            done += size
        cache.free_request("r")
        assert len(runner._shape_graphs) <= 2
    runner.check_status()
    assert [key[0][0] for key in runner._shape_graphs] == [7, 5]
