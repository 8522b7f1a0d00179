#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, StarCoder2-3B layer sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line. A "step" is one decode step of a batch of 8 requests at the context
length of the benchmark configuration (random bf16 weights, random token ids). ``value`` is
decoded tokens per second timed on the device with CUDA events around K steps; ``e2e`` is the
same through the Python entry point (``ChatEngine.step``: host token ids in, sampled ids back
on the host each step). ``prefill`` is one 2,048-token prompt in one step; ``roofline``
relates the decode step's necessary bytes (every weight once plus the live cache) to its
time; ``points`` adds decoding at batch 1 and 64. Between timed iterations the working set
(6 GB of weights) is larger than L2, so nothing is flushed explicitly.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

STARCODER2_3B = {
    "model_type": "starcoder2", "architectures": ["Starcoder2ForCausalLM"],
    "num_hidden_layers": 30, "hidden_size": 3072, "num_attention_heads": 24,
    "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 49152,
    "rope_theta": 999999.4420358813, "sliding_window": 4096, "max_position_embeddings": 16384,
    "norm_epsilon": 1e-5, "use_bias": True, "tie_word_embeddings": True,
    "hidden_act": "gelu_pytorch_tanh",
}
CONTEXT = 4096           # tokens per request in the benchmark configuration
PREFILL_TOKENS = 2048
PAGE_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                raw = json.load(handle)
            peaks = dict(FALLBACK_PEAKS)
            for key in peaks:
                if isinstance(raw.get(key), (int, float)):
                    peaks[key] = float(raw[key])
            return peaks, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self) -> None:
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.rows.append(parts)

    def mark(self) -> int:
        return len(self.rows)

    def stop(self) -> None:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, begin: int = 0, end: int | None = None) -> dict:
        rows = self.rows[begin:end] or self.rows
        clocks = sorted(int(r[0]) for r in rows if r[0].isdigit())
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no nvidia-smi samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [name for i, name in enumerate(names) if any(r[2 + i].lower() == "active" for r in rows)]
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": int(rows[0][1]) if rows[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(clocks)}


def reference_arm(args) -> int:
    """The reference arm: nesmind/matricxon's own stock code (``baseline/reference_arm.py`` says
    which calls) on the same configuration, with the same steps, warm-up and context. pip cannot
    install the reference (no package metadata), so a plain copy under ``baseline/_ref`` is put on
    the path; without it, or if its GPU path fails, the line says ``unavailable`` and why."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as arm

    if args.warmup < 3:
        args.warmup = 3
    clocks = ClockSampler()
    try:
        arm.import_reference()
        clocks.start()
        context = min(args.context, CONTEXT - args.steps - args.warmup - 8)
        record = arm.run(args, STARCODER2_3B, context, PREFILL_TOKENS, CONTEXT, clocks)
    except arm.ReferenceUnavailable as error:
        print(json.dumps({"impl": "reference", "unavailable": str(error)}))
        return 0
    except Exception as error:                      # the reference's own code failed at these sizes
        text = f"{type(error).__name__}: {error}".replace("\n", " ")[:300]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference's GPU path failed: {text}"}))
        return 0
    finally:
        clocks.stop()
    print(json.dumps(record))
    return 0


def build_engine(config_dict: dict, n_layers: int, max_active: int, cache_tokens: int,
                 max_batched_tokens: int, use_graphs: bool = True):
    import torch

    from matricxon_b200 import ChatEngine
    from matricxon_b200.config.registry import config_from_dict
    from matricxon_b200.engine.core import build_model
    from matricxon_b200.weights.random_init import RandomInit, RandomSource, weight_specs_for

    raw = dict(config_dict)
    raw["num_hidden_layers"] = n_layers
    config = config_from_dict(raw)
    source = RandomSource(weight_specs_for(config), seed=0,
                          init=RandomInit(weight_std=0.02, bias_std=0.02), device="cuda:0",
                          store_dtype=torch.bfloat16)
    model = build_model(config, source, "bfloat16", "cuda:0", PAGE_SIZE)
    engine = ChatEngine(model, max_cache_tokens=cache_tokens, max_active=max_active,
                        max_batched_tokens=max_batched_tokens, prefill_chunk=PREFILL_TOKENS,
                        max_model_len=CONTEXT, use_graphs=use_graphs)
    return config, model, engine


def fill_cache(engine, batch: int, context: int, vocab: int):
    """Gives ``batch`` requests ``context`` cached tokens each by running real prefill steps."""
    import torch

    from matricxon_b200.engine.step import StepEntry

    generator = torch.Generator().manual_seed(1)
    ids = []
    for b in range(batch):
        rid = f"bench-{b}"
        engine.core.cache.add_request(rid)
        ids.append(rid)
        done = 0
        while done < context:
            n = min(PREFILL_TOKENS, context - done)
            tokens = torch.randint(0, vocab, (n,), generator=generator).tolist()
            engine.core.runner.run([StepEntry(rid, tokens, [])])
            done += n
    engine.core.runner.check_status()
    return ids


def percentile(values, q: float) -> float:
    ordered = sorted(values)
    if not ordered:
        return float("nan")
    return ordered[min(len(ordered) - 1, int(round(q * (len(ordered) - 1))))]


def time_decode(engine, ids, vocab, steps, warmup, detail: dict | None = None):
    """K decode steps of the whole batch, timed on the device: one CUDA event before every step
    and one after the last, so that the K steps are timed exactly and each step's own time is
    known too. Every step appends one token per request, so the context grows by K."""
    import torch

    from matricxon_b200.engine.step import StepEntry

    generator = torch.Generator().manual_seed(2)
    runner = engine.core.runner

    def one_step():
        tokens = torch.randint(0, vocab, (len(ids),), generator=generator).tolist()
        return runner.run([StepEntry(rid, [tok], [0]) for rid, tok in zip(ids, tokens)])
    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    host_before = runner.host_seconds - runner.wait_seconds
    for i in range(steps):
        marks[i].record()
        one_step()
    marks[steps].record()
    torch.cuda.synchronize()
    runner.check_status()
    per_step = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
    if detail is not None:
        detail["step_ms_p50"] = round(percentile(per_step, 0.5), 4)
        detail["step_ms_p99"] = round(percentile(per_step, 0.99), 4)
        # the host's own work per step (building and uploading the metadata, replaying the graph), without
        # the time it sat waiting for the device to release the step's metadata buffer
        detail["host_ms_per_step"] = round((runner.host_seconds - runner.wait_seconds - host_before) / steps * 1e3, 4)
    return marks[0].elapsed_time(marks[steps]) / steps


def decode_bytes(config, n_layers, batch, context, model) -> float:
    """Bytes one decode step must read: every weight once, and the cache of the live requests."""
    h, i, v = config.hidden_size, config.intermediate_size, config.vocab_size
    q, kv = config.num_attention_heads * config.head_dim, config.num_key_value_heads * config.head_dim
    per_layer = (h * (q + 2 * kv) + q * h + 2 * h * i) * 2 + ((q + 2 * kv) + h + i + h + 4 * h) * 4
    head = v * h * 2
    window = config.sliding_window or context
    cache = batch * min(context, window) * n_layers * 2 * kv * 2
    return n_layers * per_layer + head + cache


def prefill_flops(config, n_layers, tokens) -> float:
    h, i, v = config.hidden_size, config.intermediate_size, config.vocab_size
    q, kv = config.num_attention_heads * config.head_dim, config.num_key_value_heads * config.head_dim
    gemm = 2.0 * tokens * (h * (q + 2 * kv) + q * h + 2 * h * i)
    attention = 2.0 * 2.0 * q * tokens * (tokens + 1) / 2.0          # causal QK^T and PV
    return n_layers * (gemm + attention) + 2.0 * v * h               # one row of logits


STARCODER2_7B = dict(STARCODER2_3B, num_hidden_layers=32, hidden_size=4608, num_attention_heads=36,
                     num_key_value_heads=4, intermediate_size=18432, rope_theta=1000000.0,
                     tie_word_embeddings=False)
STARCODER2_15B = dict(STARCODER2_3B, num_hidden_layers=40, hidden_size=6144, num_attention_heads=48,
                      num_key_value_heads=4, intermediate_size=24576, rope_theta=100000.0,
                      tie_word_embeddings=False)


def run_workload(tag: str, config_dict: dict, prompt_lens: list[int], decode_steps: int, chunk: int,
                 temperature: float, max_len: int, peaks: dict, bias_std: float = 0.0) -> dict:
    """A whole workload through the public entry point: every request is added at once, the scheduler
    cuts the prompts into portions of ``chunk`` tokens beside the decoding requests, and every request
    generates ``decode_steps`` tokens. Reports generated tokens a second (end to end, host ids in and
    out), prompt tokens a second while prompts were running, step latencies, the most pages held at
    once, preemptions, and for the steps in which everybody decoded the bytes they had to read over
    their time, as a fraction of the copy peak."""
    import torch

    from matricxon_b200 import ChatEngine, SamplingConfig
    from matricxon_b200.config.registry import config_from_dict
    from matricxon_b200.engine.core import build_model
    from matricxon_b200.weights.random_init import RandomInit, RandomSource, weight_specs_for

    config = config_from_dict(dict(config_dict))
    source = RandomSource(weight_specs_for(config), seed=0, init=RandomInit(weight_std=0.02, bias_std=bias_std),
                          device="cuda:0", store_dtype=torch.bfloat16)
    model = build_model(config, source, "bfloat16", "cuda:0", PAGE_SIZE)
    window = config.sliding_window or max_len
    # room for every request at its longest: pages of a window (plus the portion being written) or of the whole
    per_request = min(max_len, window + chunk + 2 * PAGE_SIZE)
    cache_tokens = len(prompt_lens) * per_request
    engine = ChatEngine(model, max_cache_tokens=cache_tokens, max_active=len(prompt_lens),
                        max_batched_tokens=max(chunk + len(prompt_lens), 2048), prefill_chunk=chunk,
                        max_model_len=max_len)
    generator = torch.Generator().manual_seed(11)
    sampling = SamplingConfig(temperature=temperature, top_k=0, top_p=1.0, repeat_penalty=1.0,
                              num_predict=decode_steps, num_ctx=max_len, seed=5)
    for n in prompt_lens:
        engine.add_request(torch.randint(0, config.vocab_size, (n,), generator=generator).tolist(), sampling)
    pool = engine.core.cache.pools[0]
    step_ms, decode_ms, prompt_ms = [], [], 0.0
    generated = 0
    high_water = 0
    torch.cuda.synchronize()
    started = time.perf_counter()
    while engine.has_unfinished():
        prompts_running = any(s.remaining > 1 for s in engine.scheduler.running) or bool(engine.scheduler.waiting)
        t0 = time.perf_counter()
        produced = engine.step()
        dt = (time.perf_counter() - t0) * 1e3
        step_ms.append(dt)
        generated += sum(1 for _, token, _ in produced if token is not None)
        high_water = max(high_water, pool.num_pages - pool.free_count)
        if prompts_running:
            prompt_ms += dt
        elif len(produced) == len(prompt_lens):
            decode_ms.append(dt)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    engine.core.runner.check_status()
    # bytes a step of pure decoding has to read: every weight once, and each request's visible cache
    n_layers = config.num_hidden_layers
    mean_ctx = sum(min(n + decode_steps / 2, window) for n in prompt_lens)
    kv = config.num_key_value_heads * config.head_dim
    necessary = decode_bytes(config, n_layers, 0, 0, model) + mean_ctx * n_layers * 2 * kv * 2
    p50 = percentile(decode_ms, 0.5)
    out = {
        f"{tag}_tok_s": round(generated / seconds, 1),
        f"{tag}_prompt_tok_s": round(sum(prompt_lens) / (prompt_ms * 1e-3), 1) if prompt_ms else None,
        f"{tag}_step_ms_p50": round(percentile(step_ms, 0.5), 3),
        f"{tag}_step_ms_p99": round(percentile(step_ms, 0.99), 3),
        f"{tag}_decode_step_ms_p50": round(p50, 3) if decode_ms else None,
        f"{tag}_decode_hbm_frac": round(necessary / (p50 * 1e-3) / 1e9 / peaks["hbm_gbs"], 4) if decode_ms else None,
        f"{tag}_pages_high_water": high_water, f"{tag}_pages_total": pool.num_pages,
        f"{tag}_preemptions": engine.scheduler.num_preemptions, f"{tag}_steps": len(step_ms),
    }
    del engine, model, source
    torch.cuda.empty_cache()
    return out


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--layers", type=int, default=STARCODER2_3B["num_hidden_layers"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=CONTEXT - 1024,
                        help="cached tokens per request when decode timing starts")
    parser.add_argument("--skip-points", action="store_true")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--skip-workloads", action="store_true",
                        help="leave out the 7B and 15B workloads through the scheduler")
    parser.add_argument("--no-graphs", action="store_true",
                        help="launch every kernel of a decode step by itself (for profilers)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from matricxon_b200 import SamplingConfig

    if not torch.cuda.is_available():
        print("bench.py: no CUDA device")
        return 1
    peaks, peak_source = load_peaks()
    n_layers = args.layers
    clocks = ClockSampler()
    clocks.start()

    # ---- the headline: decode at batch 8
    batch = args.batch
    cache_tokens = 64 * CONTEXT
    config, model, engine = build_engine(STARCODER2_3B, n_layers, 64, cache_tokens, 8192,
                                         use_graphs=not args.no_graphs)
    vocab = config.vocab_size
    context = min(args.context, CONTEXT - args.steps - args.warmup - 1)
    ids = fill_cache(engine, batch, context, vocab)
    mark_a = clocks.mark()
    decode_detail: dict = {}
    ms_step = time_decode(engine, ids, vocab, args.steps, args.warmup, decode_detail)
    mark_b = clocks.mark()
    pages_in_use = engine.core.cache.pools[0].num_pages - engine.core.cache.free_pages()[0]
    mean_context = context + args.warmup + args.steps / 2
    necessary = decode_bytes(config, n_layers, batch, mean_context, model)
    achieved_gbs = necessary / (ms_step * 1e-3) / 1e9
    launches = None
    for rid in ids:
        engine.core.cache.free_request(rid)

    # ---- other batch sizes
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            ids_b = fill_cache(engine, b, context, vocab)
            ms = time_decode(engine, ids_b, vocab, max(8, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(b / (ms * 1e-3), 1)
            points[f"decode_b{b}_hbm_frac"] = round(
                decode_bytes(config, n_layers, b, mean_context, model) / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
            for rid in ids_b:
                engine.core.cache.free_request(rid)

    # ---- prefill of 2,048 tokens in one step
    from matricxon_b200.engine.step import StepEntry

    generator = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=generator).tolist()
    prefill_ms = []
    for rep in range(0 if args.skip_prefill else 5):
        engine.core.cache.add_request("prefill")
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        engine.core.runner.run([StepEntry("prefill", prompt, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.core.cache.free_request("prefill")
        if rep >= 2:
            prefill_ms.append(begin.elapsed_time(end))
    # the same prompt in portions of 256 tokens, one step each (the scheduler's default portion)
    portion_ms = []
    portion_host = 0.0
    for rep in range(0 if (args.skip_prefill or args.skip_points) else 4):
        engine.core.cache.add_request("portions")
        torch.cuda.synchronize()
        host_before = engine.core.runner.host_seconds - engine.core.runner.wait_seconds
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for start in range(0, PREFILL_TOKENS, 256):
            last = start + 256 >= PREFILL_TOKENS
            engine.core.runner.run([StepEntry("portions", prompt[start:start + 256], [255] if last else [])])
        end.record()
        torch.cuda.synchronize()
        engine.core.cache.free_request("portions")
        portion_ms.append(begin.elapsed_time(end))
        portion_host = (engine.core.runner.host_seconds - engine.core.runner.wait_seconds - host_before) / (PREFILL_TOKENS // 256)
    if portion_ms:
        points["prefill_2048_in_256_token_steps"] = round(PREFILL_TOKENS / (min(portion_ms) * 1e-3), 1)
        points["prefill_256_token_step_ms"] = round(min(portion_ms) / (PREFILL_TOKENS // 256), 3)
        points["prefill_256_token_step_host_ms"] = round(portion_host * 1e3, 3)
    pf_ms = sorted(prefill_ms)[len(prefill_ms) // 2] if prefill_ms else float("nan")
    pf_flops = prefill_flops(config, n_layers, PREFILL_TOKENS)
    pf_frac = pf_flops / (pf_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)

    # ---- end to end through the entry point: host ids in, sampled ids out, every step
    # every request decodes through the whole timed region: K steps of the full batch, then cancel
    sampling = SamplingConfig(temperature=0.0, num_predict=args.steps + args.warmup + 64, num_ctx=CONTEXT)
    e2e_context = min(context, CONTEXT - (args.steps + args.warmup + 64) - 8)
    prompts = [torch.randint(0, vocab, (e2e_context,), generator=generator).tolist() for _ in range(batch)]
    rids = [] if args.skip_e2e else [engine.add_request(p, sampling) for p in prompts]
    produced = {rid: 0 for rid in rids}
    while rids and min(produced.values()) < args.warmup:        # prefill + warm-up decode steps
        for rid, _, _ in engine.step():
            produced[rid] += 1
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    tokens_out = 0
    e2e_steps = 0
    for _ in range(args.steps if rids else 0):
        tokens_out += len(engine.step())
        e2e_steps += 1
    torch.cuda.synchronize()
    e2e_seconds = time.perf_counter() - t0
    for rid in rids:
        engine.cancel(rid)
        engine.result(rid)
    e2e_value = tokens_out / e2e_seconds if e2e_seconds > 0 else 0.0
    h2d_bytes = engine.core.runner.last_upload_bytes + engine.sampler.last_upload_bytes
    d2h_bytes = batch * 4 + 4

    launches = engine.core.runner.launches_per_step
    pool_pages = engine.core.cache.pools[0].num_pages
    # ---- the two larger configurations, whole workloads through the scheduler (shortened where the
    # full one would take minutes: the names say how)
    if not (args.skip_points or args.skip_workloads):
        del engine, model
        gc.collect()
        torch.cuda.empty_cache()
        lengths = torch.randint(128, 6001, (32,), generator=torch.Generator().manual_seed(7)).tolist()
        points.update(run_workload("w7b_32req_chunk512_256steps", STARCODER2_7B, lengths, 256, 512, 0.0, 16384, peaks))
        points.update(run_workload("w15b_8x12288_128steps", STARCODER2_15B, [12288] * 8, 128, 512, 1.0, 16384, peaks))
        engine = None
    clocks.stop()
    value = batch / (ms_step * 1e-3)
    record = {
        "metric": "decode tok/s @ batch 8 (StarCoder2-3B bf16, one B200)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids",
        "impl": "ours",
        "config": {
            "model": "StarCoder2-3B layer sizes", "layers": n_layers, "layers_in_model": 30,
            "hidden": config.hidden_size, "heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
            "intermediate": config.intermediate_size, "vocab": config.vocab_size,
            "window": config.sliding_window, "tied": config.tie_word_embeddings,
            "bias": config.use_bias, "global_batch": batch, "seq_len": CONTEXT,
            "decode_context": int(mean_context), "page_size": PAGE_SIZE,
            "cache_pool_tokens": cache_tokens, "parallelism": "single GPU",
            "l2": "working set (weights) exceeds L2; no flush", "peaks": peak_source,
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "steps": e2e_steps,
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
        "gpu_launches": launches * args.steps if launches else None,
        "prefill": {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pf_ms, 3), "frac": round(pf_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved_gbs / peaks["hbm_gbs"], 4)},
        "latency": {"step_ms_p50": decode_detail.get("step_ms_p50"), "step_ms_p99": decode_detail.get("step_ms_p99"),
                    "host_ms_per_step": decode_detail.get("host_ms_per_step"), "pages_high_water": pages_in_use,
                    "pages_total": pool_pages, "preemptions": 0},
        "points": points,
        "clocks": clocks.summary(mark_a, mark_b),
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
